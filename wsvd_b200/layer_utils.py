"""One-decoder-layer wrappers around the decode-attention op, with the function names and
argument lists of the reference's efficiency/layer_utils.py so that its timing and
functional scripts can import them unchanged.

Order of operations (layer_utils.py:307-358): RMSNorm (unit weight, eps 1e-5, fp32 inside)
-> x@Wdq, x@Wdk, x@Wdv -> per-head latent_q @ Wuq -> decode attention in latent space ->
@Wuvout -> residual on the *normed* input -> RMSNorm -> SwiGLU FFN -> residual on the normed
tensor.  The GEMMs are plain torch matmuls (cuBLAS); the attention is the CUDA op of this
package.  As in the reference, the new token's latent_k/latent_v are computed but not
appended to the cache (layer_utils.py:320-321).
"""
from __future__ import annotations

import math

import torch

from .infer_state import InferState
from .kernel.flash_decoding import (
    token_decode_attention_flash_int8_latent_per_head_decoding_rope,
    token_decode_attention_flash_latent_per_head_decoding_rope,
)


def _rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    xf = x.float()
    xn = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xn.to(weight.dtype) * weight).to(x.dtype)


def input_layernorm(x, weight, eps: float = 1e-5):
    return _rms_norm(x, weight, eps)


def post_attention_layernorm(x, weight, eps: float = 1e-5):
    return _rms_norm(x, weight, eps)


def _layer(head_dim, q_head_num, x, attn, Wdq, Wdk, Wdv, Wuq, Wuvout, Wup, Wgate, Wdown):
    B, one, model_dim = x.shape
    unit = torch.ones(model_dim, device=x.device, dtype=x.dtype)
    xn = input_layernorm(x, unit)
    latent_q = xn @ Wdq
    _latent_k = xn @ Wdk  # computed and dropped, as in the reference
    _latent_v = xn @ Wdv
    # the reference reinterprets Wuq [R, Hq*D] as [Hq, R, D] with a plain view (layer_utils.py:324)
    q = (latent_q.view(B, one, q_head_num, -1).transpose(1, 2) @ Wuq.view(q_head_num, -1, head_dim)).transpose(1, 2)
    o_lat = attn(q.reshape(B * one, q_head_num, head_dim)).view(B, one, -1)
    out = (o_lat @ Wuvout.view(-1, head_dim * q_head_num)).reshape(B, one, model_dim)
    res = post_attention_layernorm(xn + out, unit)
    ffn = ((res @ Wup) * torch.nn.functional.silu(res @ Wgate)) @ Wdown
    return res + ffn


def run_flash_int8_latent_per_head_decoding_rope_layer(
    seq_len, head_dim, q_head_num, input, cache_latent_k, cache_latent_k_scale, cache_latent_v,
    cache_latent_v_scale, Wdq, Wdk, Wdv, Wuq, Wuk, Wuk_scale, Wuvout, Wup, Wgate, Wdown, infer_state,
):
    """int8-latent layer (layer_utils.py:307)."""
    def attn(q):
        return token_decode_attention_flash_int8_latent_per_head_decoding_rope(
            q, infer_state, q_head_num, head_dim, cache_latent_k, cache_latent_k_scale, cache_latent_v,
            cache_latent_v_scale, Wuk, Wuk_scale)

    return _layer(head_dim, q_head_num, input, attn, Wdq, Wdk, Wdv, Wuq, Wuvout, Wup, Wgate, Wdown)


def run_flash_latent_per_head_decoding_rope_layer(
    seq_len, head_dim, q_head_num, input, cache_latent_k, cache_latent_v, Wdq, Wdk, Wdv, Wuq, Wuk, Wuvout, Wup,
    Wgate, Wdown, infer_state,
):
    """f16-latent layer (layer_utils.py:257)."""
    def attn(q):
        return token_decode_attention_flash_latent_per_head_decoding_rope(
            q, infer_state, q_head_num, head_dim, cache_latent_k, cache_latent_v, Wuk)

    return _layer(head_dim, q_head_num, input, attn, Wdq, Wdk, Wdv, Wuq, Wuvout, Wup, Wgate, Wdown)


def create_test_data_layer(batch_size=2, q_head_num=40, head_dim=128, seq_len=2048, rank_ratio=0.9,
                           kv_head_num=40, intermediate_dim=128 * 40 * 3, device="cuda", seed=None):
    """Synthetic layer inputs with the shapes and initialisation of layer_utils.py:38-95
    (randn activations/caches, xavier-uniform weights, FFN up/gate scaled by 1/sqrt(2)),
    returned in the reference's order."""
    gen = None
    if seed is not None:
        gen = torch.Generator(device=device).manual_seed(seed)
    dt = torch.float16
    R = int(rank_ratio * head_dim)
    model_dim = q_head_num * head_dim

    def randn(*shape):
        return torch.randn(*shape, device=device, dtype=torch.float32, generator=gen).to(dt)

    def xavier(rows, cols, gain=1.0):
        bound = gain * math.sqrt(6.0 / (rows + cols))
        w = torch.rand(rows, cols, device=device, dtype=torch.float32, generator=gen) * 2 - 1
        return (w * bound).to(dt)

    x = randn(batch_size, 1, model_dim)
    cache_latent_k = randn(batch_size, seq_len, kv_head_num * R)
    cache_latent_v = randn(batch_size, seq_len, kv_head_num * R)
    Wdq, Wdk, Wdv = xavier(model_dim, q_head_num * R), xavier(model_dim, kv_head_num * R), xavier(model_dim, kv_head_num * R)
    Wuq, Wuk, Wuv = xavier(R, q_head_num * head_dim), xavier(R, kv_head_num * head_dim), xavier(R, kv_head_num * head_dim)
    Wq, Wk, Wv = (xavier(model_dim, q_head_num * head_dim), xavier(model_dim, kv_head_num * head_dim),
                  xavier(model_dim, kv_head_num * head_dim))
    cache_k = randn(batch_size, seq_len, kv_head_num * head_dim)
    cache_v = randn(batch_size, seq_len, kv_head_num * head_dim)
    Wout = xavier(model_dim, model_dim)
    Wup = xavier(model_dim, intermediate_dim, 1 / math.sqrt(2))
    Wgate = xavier(model_dim, intermediate_dim, 1 / math.sqrt(2))
    Wdown = xavier(intermediate_dim, model_dim)
    infer_state = InferState(batch_size, seq_len, [seq_len] * batch_size, device=device)
    return (x, cache_latent_k, cache_latent_v, Wdq, Wdk, Wdv, Wuq, Wuk, Wuv, Wq, Wk, Wv, cache_k, cache_v, Wout, Wup,
            Wgate, Wdown, infer_state)
