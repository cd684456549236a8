"""Drop-in for efficiency/kernel/flash_int8_latent_per_head_decoding_rope_stage1.py."""
import torch

from .. import ops


@torch.no_grad()
def flash_int8_latent_per_head_decode_rope_stage1(q, latent_k, latent_k_scale, latent_v, latent_v_scale, wk,
                                                  wk_scale, Req_to_tokens, B_req_idx, B_Seqlen, max_len_in_batch,
                                                  mid_out, mid_out_logsumexp, block_seq):
    """Stage 1 with the reference's argument list (stage1.py:221).  Unlike the reference,
    `block_seq` IS the split size used (the reference ignores it and autotunes, which
    breaks its own stage 2 when the tuner picks another value)."""
    ops.latent_decode_stage1(q, latent_k, latent_k_scale, latent_v, latent_v_scale, wk,
                             None if wk_scale is None else wk_scale.reshape(-1), Req_to_tokens, B_req_idx,
                             B_Seqlen, max_len_in_batch, mid_out, mid_out_logsumexp, block_seq)
