"""Drop-in for efficiency/kernel/flash_latent_per_head_decoding_rope_stage1.py."""
import torch

from .. import ops


@torch.no_grad()
def flash_latent_per_head_decode_rope_stage1(q, latent_k, latent_v, wk, Req_to_tokens, B_req_idx, B_Seqlen,
                                             max_len_in_batch, mid_out, mid_out_logsumexp, block_seq):
    """Stage 1 for f16 latents with the reference's argument list (stage1.py:169)."""
    ops.latent_decode_stage1(q, latent_k, None, latent_v, None, wk, None, Req_to_tokens, B_req_idx, B_Seqlen,
                             max_len_in_batch, mid_out, mid_out_logsumexp, block_seq)
