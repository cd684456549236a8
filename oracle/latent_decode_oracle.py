"""CPU oracle for WSVD's per-head low-rank latent flash-decoding attention.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain torch on the CPU, the
algorithm of the reference's Triton kernels so that the CUDA path can be checked
against it.  Nothing in the product package imports it; only the tests, the smoke
check and the benchmark's CPU-baseline / reference arm do.

Parity pin: the functions below are checked (tests/test_oracle_vs_reference.py)
against golden vectors produced by the reference's own code — its torch restatement
`reference_online_rope_attention_projected_only`
(efficiency/test_functional_layer.py:176-226) and its Triton kernels run through
Triton's CPU interpreter (generator: tests/golden/make_golden.py).  The reference
holds no golden vectors of its own for this path and never checks the int8 kernel's
output, so the pin is "reference code executed on the CPU on seeded inputs".

Reference layout (efficiency/kernel/flash_int8_latent_per_head_decoding_rope_stage1.py):
  q                [B, Hq, D]        f16     (already rotated by the caller, :83-84)
  latent_k/v       [T, Hkv, Rk|Rv]   int8 or f16, T = number of token slots
  k_scale/v_scale  [T, Hkv]          f16     (int8 path only, :135-136)
  wk               [Rk, Hkv*D]       f16, or int8 with wk_scale [1, Hkv*D] (:96-108)
  req_to_token     [n_req, max_len]  int32   page table (:119-123)
  b_req_idx, b_seq_len [B]           int32
Output O_lat [B, Hq, Rv] (latent space, :206-216); with wv [Rv, Hkv*D] also
O = O_lat . wv (the fold of efficiency/test_timing_layer.py:259-262 left unfused).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

__all__ = [
    "rope_inv_freq",
    "unpack_wk",
    "quantize_per_token",
    "latent_decode_oracle",
    "latent_decode_stage1_oracle",
    "combine_oracle",
    "latent_decode_kernel_order_oracle",
    "dense_decode_oracle",
    "layer_oracle",
]


def rope_inv_freq(head_dim: int, theta: float = 10000.0, dtype=torch.float32) -> torch.Tensor:
    """inv_freq[i] = theta^(-2i/D), i in [0, D/2).

    The kernel divides the position by theta^(2i/D)
    (flash_int8_latent_per_head_decoding_rope_stage1.py:8-14); the product form is the
    one HF's rotary embedding and test_functional_layer.py:39-40 use.
    """
    idx = torch.arange(0, head_dim, 2, dtype=dtype)
    return 1.0 / (torch.tensor(theta, dtype=dtype) ** (idx / head_dim))


def unpack_wk(wk: torch.Tensor, wk_scale: Optional[torch.Tensor], n_kv_heads: int, head_dim: int,
              dtype=torch.float32) -> torch.Tensor:
    """wk [R, Hkv*D] (+ per-column scale [1, Hkv*D]) -> U [Hkv, D, R] in `dtype`.

    Column h*D+d of wk belongs to KV head h, dim d (stage1.py:94-108).
    """
    r = wk.shape[0]
    w = wk.to(dtype)
    if wk_scale is not None:
        w = w * wk_scale.reshape(1, -1).to(dtype)
    return w.reshape(r, n_kv_heads, head_dim).permute(1, 2, 0).contiguous()


F16_TINY, F16_MAX = 2.0 ** -24, 65504.0  # smallest positive (subnormal) and largest finite f16


def quantize_per_token(x: torch.Tensor, bits: int = 8) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric per-(token, head) int8 quantisation over the last dim.

    Follows fake_quant/quant_utils.py:30-33,179-184: scale = amax/maxq (1 where the
    row is all zero), q = clamp(round(x/scale), -(maxq+1), maxq).  The scale is
    stored as f16 and the rounding is done against the stored value so that
    dequantisation reproduces exactly what a kernel reading the f16 scale sees.
    """
    maxq = 2 ** (bits - 1) - 1
    xf = x.float()
    amax = xf.abs().amax(dim=-1)
    scale = amax / maxq
    scale = torch.where(amax == 0, torch.ones_like(scale), scale)
    # the cache stores the scale as f16: keep it a usable divisor when amax/maxq leaves the
    # f16 range (the reference keeps the scale in the input dtype, quant_utils.py:175-184)
    scale_h = scale.clamp(min=F16_TINY, max=F16_MAX).to(torch.float16)
    # an f16 scale that rounded down could push round(x/scale) to maxq+1; the clamp
    # keeps it in range exactly as the reference's clamp does
    q = torch.clamp(torch.round(xf / scale_h.float().unsqueeze(-1)), -(maxq + 1), maxq)
    return q.to(torch.int8), scale_h



def quant_append_oracle(x_k, x_v, b_seq_len, b_req_idx, req_to_token, latent_k, k_scale, latent_v, v_scale):
    """Append one token per sequence to the latent cache (in place, CPU tensors).

    x_k [B, Hkv, Rk], x_v [B, Hkv, Rv] are quantised with `quantize_per_token`
    (fake_quant/quant_utils.py:30-33,175-184) and stored at token slot
    req_to_token[b_req_idx[b], b_seq_len[b]].  The reference drops the new latents
    (efficiency/layer_utils.py:319-321); this states what a cache producer with its
    quantiser has to write.  Sequences whose position has no page-table column are skipped.
    """
    qk, sk = quantize_per_token(x_k)
    qv, sv = quantize_per_token(x_v)
    for b in range(x_k.shape[0]):
        pos = int(b_seq_len[b])
        if pos < 0 or pos >= req_to_token.shape[1]:
            continue
        slot = int(req_to_token[int(b_req_idx[b]), pos])
        latent_k[slot] = qk[b]
        k_scale[slot] = sk[b]
        latent_v[slot] = qv[b]
        v_scale[slot] = sv[b]


def _rope_half(k: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Half-split (NeoX/HF) pairing (i, i+D/2), the kernel's convention
    (stage1.py:65-66,165-166).  k: [S, H, D]; pos: [S]."""
    h2 = k.shape[-1] // 2
    ang = pos.to(inv_freq.dtype)[:, None] * inv_freq[None, :]  # a single fp32 multiply
    cos = torch.cos(ang)[:, None, :].to(k.dtype)
    sin = torch.sin(ang)[:, None, :].to(k.dtype)
    k0, k1 = k[..., :h2], k[..., h2:]
    return torch.cat([k0 * cos - k1 * sin, k1 * cos + k0 * sin], dim=-1)


def _rope_interleaved(k: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Interleaved pairing (2i, 2i+1) of test_functional_layer.py:25-44 (the
    reference test's own convention; it differs from its kernel's)."""
    ang = pos.to(inv_freq.dtype)[:, None] * inv_freq[None, :]
    cos = torch.cos(ang)[:, None, :].to(k.dtype)
    sin = torch.sin(ang)[:, None, :].to(k.dtype)
    ke, ko = k[..., 0::2], k[..., 1::2]
    out = torch.empty_like(k)
    out[..., 0::2] = ke * cos - ko * sin
    out[..., 1::2] = ko * cos + ke * sin
    return out


def _gather_dequant(latent, scale, tok, dtype):
    x = latent[tok].to(dtype)  # [S, Hkv, R]
    if scale is not None:
        x = x * scale[tok].to(dtype).unsqueeze(-1)
    return x


def latent_decode_oracle(
    q: torch.Tensor,
    b_seq_len: torch.Tensor,
    b_req_idx: torch.Tensor,
    req_to_token: torch.Tensor,
    latent_k: torch.Tensor,
    k_scale: Optional[torch.Tensor],
    latent_v: torch.Tensor,
    v_scale: Optional[torch.Tensor],
    wk: torch.Tensor,
    wk_scale: Optional[torch.Tensor] = None,
    wv: Optional[torch.Tensor] = None,
    theta: float = 10000.0,
    rope_layout: str = "half",
    dtype=torch.float32,
    pos_offset: Optional[torch.Tensor] = None,
):
    """fp32 (or fp64) oracle of the whole op: gather by page table -> dequantise ->
    reconstruct K against U_k -> RoPE on K at the logical position -> scaled softmax
    over the sequence -> P . latent V -> optional . U_v^T.

    Structure follows efficiency/test_functional_layer.py:146-163; RoPE pairing and
    positions follow the kernel (stage1.py:155-166).  A sequence of length 0 yields
    zeros (the reference divides by zero there, stage2.py:47).

    Returns (O_lat [B,Hq,Rv], O [B,Hq,D] or None), both in `dtype`.
    """
    B, Hq, D = q.shape
    Hkv = latent_k.shape[1]
    Rv = latent_v.shape[-1]
    g = Hq // Hkv
    U = unpack_wk(wk, wk_scale, Hkv, D, dtype)  # [Hkv, D, Rk]
    Uv = None if wv is None else unpack_wk(wv, None, Hkv, D, dtype)  # [Hkv, D, Rv]
    inv_freq = rope_inv_freq(D, theta, dtype)
    rope = {"half": _rope_half, "interleaved": _rope_interleaved}[rope_layout]
    c = 1.0 / math.sqrt(D)
    o_lat = torch.zeros(B, Hq, Rv, dtype=dtype)
    for b in range(B):
        n = int(b_seq_len[b])
        if n == 0:
            continue
        tok = req_to_token[int(b_req_idx[b]), :n].long()
        k_lat = _gather_dequant(latent_k, k_scale, tok, dtype)  # [n, Hkv, Rk]
        v_lat = _gather_dequant(latent_v, v_scale, tok, dtype)  # [n, Hkv, Rv]
        k_full = torch.einsum("shr,hdr->shd", k_lat, U)
        pos = torch.arange(n, dtype=dtype)
        if pos_offset is not None:
            pos = pos + pos_offset[b].to(dtype)
        k_rot = rope(k_full, pos, inv_freq)
        k_rot = k_rot.repeat_interleave(g, dim=1)  # [n, Hq, D]
        v_exp = v_lat.repeat_interleave(g, dim=1)
        score = torch.einsum("hd,shd->hs", q[b].to(dtype), k_rot) * c
        prob = torch.softmax(score, dim=-1)
        o_lat[b] = torch.einsum("hs,shr->hr", prob, v_exp)
    o = None
    if Uv is not None:
        o = torch.einsum("bhr,hdr->bhd", o_lat, Uv.repeat_interleave(g, dim=0))
    return o_lat, o


def latent_decode_stage1_oracle(
    q, b_seq_len, b_req_idx, req_to_token, latent_k, k_scale, latent_v, v_scale, wk,
    wk_scale=None, block_seq: int = 256, theta: float = 10000.0, dtype=torch.float32,
):
    """Split-KV stage 1: per (b, h, split) a *normalised* partial acc/sum and
    lse = max + log(sum); empty splits are left untouched (NaN here)
    (stage1.py:69-76,211-216).  Returns mid_o [B,Hq,n_split,Rv], lse [B,Hq,n_split]."""
    B, Hq, D = q.shape
    Hkv = latent_k.shape[1]
    Rv = latent_v.shape[-1]
    g = Hq // Hkv
    max_len = int(b_seq_len.max()) if B else 0
    n_split = (max_len + block_seq - 1) // block_seq
    U = unpack_wk(wk, wk_scale, Hkv, D, dtype)
    inv_freq = rope_inv_freq(D, theta, dtype)
    c = 1.0 / math.sqrt(D)
    mid = torch.full((B, Hq, n_split, Rv), float("nan"), dtype=dtype)
    lse = torch.full((B, Hq, n_split), float("nan"), dtype=dtype)
    for b in range(B):
        n = int(b_seq_len[b])
        for s in range(n_split):
            lo, hi = s * block_seq, min(n, (s + 1) * block_seq)
            if hi <= lo:
                continue
            tok = req_to_token[int(b_req_idx[b]), lo:hi].long()
            k_lat = _gather_dequant(latent_k, k_scale, tok, dtype)
            v_lat = _gather_dequant(latent_v, v_scale, tok, dtype)
            k_full = torch.einsum("shr,hdr->shd", k_lat, U)
            k_rot = _rope_half(k_full, torch.arange(lo, hi, dtype=dtype), inv_freq)
            k_rot = k_rot.repeat_interleave(g, dim=1)
            v_exp = v_lat.repeat_interleave(g, dim=1)
            score = torch.einsum("hd,shd->hs", q[b].to(dtype), k_rot) * c
            m = score.max(dim=-1).values
            e = torch.exp(score - m[:, None])
            ssum = e.sum(dim=-1)
            mid[b, :, s] = torch.einsum("hs,shr->hr", e, v_exp) / ssum[:, None]
            lse[b, :, s] = m + torch.log(ssum)
    return mid, lse


def combine_oracle(mid_o: torch.Tensor, lse: torch.Tensor, b_seq_len: torch.Tensor, block_seq: int = 256):
    """Split-KV stage 2: O = sum_i e^{lse_i - m} mid_i / sum_i e^{lse_i - m} over the
    first ceil(len/block_seq) splits (flash_latent_per_head_decoding_stage2.py:25,35-47)."""
    B, Hq, _, Rv = mid_o.shape
    out = torch.zeros(B, Hq, Rv, dtype=mid_o.dtype)
    for b in range(B):
        ns = (int(b_seq_len[b]) + block_seq - 1) // block_seq
        if ns == 0:
            continue
        l = lse[b, :, :ns]
        m = l.max(dim=-1, keepdim=True).values
        w = torch.exp(l - m)
        out[b] = (w.unsqueeze(-1) * mid_o[b, :, :ns]).sum(dim=1) / w.sum(dim=-1, keepdim=True)
    return out


def latent_decode_kernel_order_oracle(
    q, b_seq_len, b_req_idx, req_to_token, latent_k, k_scale, latent_v, v_scale, wk,
    wk_scale=None, block_seq: int = 256, block_n: int = 64, theta: float = 10000.0,
):
    """The reference kernel's own rounding order, for diagnosing differences:
    integer (or f16->f32) dot, cast to f16 *before* scaling, f16 cos/sin, f16
    rotation, f16 products summed in f16, fp32 online softmax per tile of block_n
    tokens, f16 dequantised V, fp32 accumulate, normalised partial + lse, fp32
    stage-2 merge, cast to q's dtype (stage1.py:117-216; stage2.py:35-47).
    Exact cos/sin are used where the kernel uses the fast-math intrinsics."""
    B, Hq, D = q.shape
    Hkv = latent_k.shape[1]
    Rv = latent_v.shape[-1]
    g = Hq // Hkv
    h2 = D // 2
    f16 = torch.float16
    is_int = latent_k.dtype == torch.int8
    max_len = int(b_seq_len.max()) if B else 0
    n_split = (max_len + block_seq - 1) // block_seq
    w = wk.reshape(wk.shape[0], Hkv, D)
    ws = None if wk_scale is None else wk_scale.reshape(Hkv, D).to(f16)
    c = 1.0 / math.sqrt(D)
    pair = torch.arange(0, h2, dtype=torch.float32) * 2
    freq = torch.tensor(theta, dtype=torch.float32) ** (pair / D)
    mid = torch.zeros(B, Hq, n_split, Rv, dtype=torch.float32)
    lse = torch.zeros(B, Hq, n_split, dtype=torch.float32)
    for b in range(B):
        n = int(b_seq_len[b])
        for h in range(Hq):
            hk = h // g
            q0, q1 = q[b, h, :h2].to(f16), q[b, h, h2:].to(f16)
            for s in range(n_split):
                lo, hi = s * block_seq, min(n, (s + 1) * block_seq)
                if hi <= lo:
                    continue
                mx = torch.tensor(float("-inf"))
                se = torch.tensor(0.0)
                acc = torch.zeros(Rv, dtype=torch.float32)
                for t0 in range(lo, hi, block_n):
                    t1 = min(hi, t0 + block_n)
                    tok = req_to_token[int(b_req_idx[b]), t0:t1].long()
                    lk = latent_k[tok, hk]
                    if is_int:
                        kk = (lk.to(torch.int64) @ w[:, hk].to(torch.int64)).to(torch.float32).to(f16)
                        sk = k_scale[tok, hk].to(f16)[:, None]
                        kk0 = kk[:, :h2] * sk * ws[hk, :h2][None]
                        kk1 = kk[:, h2:] * sk * ws[hk, h2:][None]
                    else:
                        kk = (lk.float() @ w[:, hk].float()).to(f16)
                        kk0, kk1 = kk[:, :h2], kk[:, h2:]
                    ang = torch.arange(t0, t1, dtype=torch.float32)[:, None] / freq[None]
                    cs, sn = torch.cos(ang).to(f16), torch.sin(ang).to(f16)
                    r0 = kk0 * cs - kk1 * sn
                    r1 = kk1 * cs + kk0 * sn
                    att = ((q0[None] * r0).sum(dim=1) + (q1[None] * r1).sum(dim=1)).float() * c
                    lv = latent_v[tok, hk]
                    if is_int:
                        lv = lv.to(f16) * v_scale[tok, hk].to(f16)[:, None]
                    new_mx = torch.maximum(att.max(), mx)
                    e = torch.exp(att - new_mx)
                    sc = torch.exp(mx - new_mx)
                    acc = acc * sc + (e[:, None] * lv.float()).sum(dim=0)
                    se = se * sc + e.sum()
                    mx = new_mx
                mid[b, h, s] = acc / se
                lse[b, h, s] = mx + torch.log(se)
    return combine_oracle(mid, lse, b_seq_len, block_seq).to(q.dtype)


def dense_decode_oracle(q, b_seq_len, b_req_idx, req_to_token, cache_k, cache_v, dtype=torch.float32):
    """Dense flash-decoding baseline: softmax(q.K^T/sqrt(D)).V on K/V caches
    [T, Hkv, D] read through the page table, no RoPE (K is stored rotated)
    (efficiency/kernel/flash_decoding_stage1.py:44-62, flash_decoding.py:98-131)."""
    B, Hq, D = q.shape
    Hkv = cache_k.shape[1]
    g = Hq // Hkv
    c = 1.0 / math.sqrt(D)
    out = torch.zeros(B, Hq, D, dtype=dtype)
    for b in range(B):
        n = int(b_seq_len[b])
        if n == 0:
            continue
        tok = req_to_token[int(b_req_idx[b]), :n].long()
        k = cache_k[tok].to(dtype).repeat_interleave(g, dim=1)
        v = cache_v[tok].to(dtype).repeat_interleave(g, dim=1)
        score = torch.einsum("hd,shd->hs", q[b].to(dtype), k) * c
        out[b] = torch.einsum("hs,shd->hd", torch.softmax(score, dim=-1), v)
    return out


def _rms_norm(x: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """RMSNorm with unit weight, fp32 inside (efficiency/layer_utils.py:11-28)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)).to(x.dtype)


def layer_oracle(head_dim, q_head_num, x, attn_fn, Wdq, Wuq, Wuvout, Wup, Wgate, Wdown):
    """One decoder layer around the op, in the order of
    efficiency/layer_utils.py:307-358: RMSNorm -> x@Wdq -> per-head @Wuq -> op ->
    @Wuvout -> residual on the *normed* input -> RMSNorm -> SwiGLU FFN -> residual
    on the normed tensor.  `attn_fn(q[B,Hq,D]) -> O_lat[B,Hq,Rv]`."""
    B, one, model_dim = x.shape
    xn = _rms_norm(x)
    lq = (xn @ Wdq).view(B, one, q_head_num, -1)
    # the reference reinterprets Wuq [R, Hq*D] as [Hq, R, D] with a plain view (layer_utils.py:324)
    q = (lq.transpose(1, 2) @ Wuq.view(q_head_num, -1, head_dim)).transpose(1, 2)
    q = q.reshape(B * one, q_head_num, head_dim)
    o_lat = attn_fn(q).to(x.dtype).view(B, one, -1)
    out = (o_lat @ Wuvout.view(-1, head_dim * q_head_num)).reshape(B, one, model_dim)
    res = _rms_norm(xn + out)
    ffn = ((res @ Wup) * torch.nn.functional.silu(res @ Wgate)) @ Wdown
    return res + ffn
