"""Drop-in for efficiency/kernel/flash_latent_per_head_decoding_stage2.py."""
import torch

from .. import ops


@torch.no_grad()
def flash_decode_stage2(mid_out, mid_out_logexpsum, B_Seqlen, O, block_seq, rank_chunk=64):
    """Merge split partials (stage2.py:52).  `rank_chunk` is unused, as in the reference."""
    ops.decode_stage2(mid_out, mid_out_logexpsum, B_Seqlen, O, block_seq)
