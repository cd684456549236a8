"""Drop-in for the reference's efficiency/kernel/flash_decoding.py: same function names,
positional arguments, defaults and return values; the work is done by the sm_100a CUDA
library instead of Triton kernels."""
from __future__ import annotations

import torch

from .. import ops


def token_decode_attention_flash_int8_latent_per_head_decoding_rope(
    q,
    infer_state,
    q_head_num,
    head_dim,
    cache_latent_k,
    cache_latent_k_scale,
    cache_latent_v,
    cache_latent_v_scale,
    wk,
    wk_scale,
    out=None,
    alloc_tensor_func=torch.empty,
    block_seq: int = 256,
    *,
    wv=None,
    pos_offset=None,
    theta: float = 10000.0,
    rope_layout: str = "half",
    workspace=None,
    split_len: int = 0,
    kernel: str = "auto",
    stream=None,
):
    """int8 latents + per-token-per-head f16 scales (flash_decoding.py:3-55).

    `wk` is [Rk, Hkv*D], either int8 with `wk_scale` [1, Hkv*D] f16 (the reference
    signature) or f16 with `wk_scale=None`.  Returns O_lat [B, Hq, Rv] in q's dtype, or
    O [B, Hq, D] when the keyword `wv` ([Rv, Hkv*D] f16) is given.  `block_seq` is
    accepted for signature compatibility; like in the reference (stage1.py:221, unused
    there) it does not set the split size — `split_len` does, 0 meaning the library's
    plan."""
    q3 = q.view(infer_state.batch_size, q_head_num, head_dim)
    return ops.latent_decode(
        q3, infer_state, cache_latent_k, cache_latent_k_scale, cache_latent_v, cache_latent_v_scale, wk,
        None if wk_scale is None else wk_scale.reshape(-1), wv=wv, out=out, workspace=workspace,
        alloc_tensor_func=alloc_tensor_func, pos_offset=pos_offset, theta=theta, rope_layout=rope_layout,
        split_len=split_len, kernel=kernel, stream=stream)


def token_decode_attention_flash_latent_per_head_decoding_rope(
    q, infer_state, q_head_num, head_dim, cache_latent_k, cache_latent_v, wk, out=None,
    alloc_tensor_func=torch.empty, *, wv=None, pos_offset=None, theta: float = 10000.0,
    rope_layout: str = "half", workspace=None, split_len: int = 0, kernel: str = "auto", stream=None,
):
    """f16 latents, f16 wk, no scales (flash_decoding.py:57-95)."""
    q3 = q.view(infer_state.batch_size, q_head_num, head_dim)
    return ops.latent_decode(
        q3, infer_state, cache_latent_k, None, cache_latent_v, None, wk, None, wv=wv, out=out,
        workspace=workspace, alloc_tensor_func=alloc_tensor_func, pos_offset=pos_offset, theta=theta,
        rope_layout=rope_layout, split_len=split_len, kernel=kernel, stream=stream)


def token_decode_attention_flash_decoding(
    q, infer_state, q_head_num, head_dim, cache_k, cache_v, out=None, alloc_tensor_func=torch.empty, *,
    workspace=None, split_len: int = 0, stream=None,
):
    """Dense f16 flash-decoding on full K/V caches [T, Hkv, D] (flash_decoding.py:98-131):
    the reference's own "Flash Decoding" baseline, here as a CUDA kernel of the same
    split-KV structure."""
    q3 = q.view(infer_state.batch_size, q_head_num, head_dim)
    return ops.dense_decode(q3, infer_state, cache_k, cache_v, out=out, alloc_tensor_func=alloc_tensor_func,
                            workspace=workspace, split_len=split_len, stream=stream)
