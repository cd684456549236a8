"""Tensor -> C-ABI marshalling for the latent decode-attention op.

The functions here take torch CUDA tensors, check the preconditions the reference
wrappers assert (efficiency/kernel/flash_int8_latent_per_head_decoding_rope_stage1.py:
231-243) and call libwsvd_b200.so on the current CUDA stream.  No CPU path exists.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Optional, Tuple

import torch

from . import _lib
from ._lib import LatentDecodeParams, check

I8, F16 = 0, 1
ROPE = {"half": 0, "interleaved": 1}
KERNEL = {"auto": 0, "generic": 1, "tc": 2, "mma": 3}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _need(cond: bool, msg: str, exc=ValueError):
    if not cond:
        raise exc(msg)


def _cuda_tensor(name, t, dtypes, ndim, inner_contiguous=True):
    _need(isinstance(t, torch.Tensor), f"{name} must be a torch.Tensor", TypeError)
    _need(t.is_cuda, f"{name} must be a CUDA tensor (no CPU path exists)")
    _need(t.dtype in dtypes, f"{name} has dtype {t.dtype}, expected one of {dtypes}", TypeError)
    _need(t.dim() == ndim, f"{name} must have {ndim} dims, got {tuple(t.shape)}")
    _need(not inner_contiguous or t.numel() == 0 or t.stride(-1) == 1,
          f"{name}: innermost dimension must be contiguous")


_TABLES = {}
_RETIRED_TABLES = []  # superseded tables stay allocated: cached argument blocks and captured graphs may point at them
_CALLS = {}


def _sig(t):
    return None if t is None else (t.data_ptr(), t.shape, t.stride(), t.dtype)


def rope_table(device, positions: int, head_dim: int = 128, theta: float = 10000.0, stream=None):
    """cos/sin position table for the tensor-core kernel, built once per
    (device, theta, head_dim) and grown geometrically with the longest context seen.

    Returns (buffer, rows, event).  The table is built on `stream` (default: the current
    stream); `event` is recorded right after the build so that a launch on another stream
    can order itself behind it.  A table that is replaced by a larger one is never freed:
    argument blocks handed out earlier, and CUDA graphs captured with them, keep pointing
    at memory that still holds a valid (shorter) table."""
    dev = torch.device(device)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), float(theta), int(head_dim))
    have = _TABLES.get(key)
    if have is not None and have[1] >= positions:
        return have
    rows = 4096
    while rows < positions:
        rows *= 2
    nbytes = int(_lib.lib().wsvd_rope_table_bytes(rows, head_dim))
    buf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        s = torch.cuda.current_stream() if stream is None else stream
        check(_lib.lib().wsvd_rope_table_init(_ptr(buf), nbytes, rows, head_dim, float(theta),
                                              ctypes.c_void_p(s.cuda_stream)), "wsvd_rope_table_init")
        ev = torch.cuda.Event()
        ev.record(s)
    if have is not None:
        _RETIRED_TABLES.append(have)
    _TABLES[key] = [buf, rows, ev, s.cuda_stream, False]
    return _TABLES[key]


def _order_after_table(entry, stream) -> None:
    """Make `stream` wait for the table's build when it was enqueued on another stream and
    has not finished yet.  Once the build is known to have finished nothing is done (and no
    event is queried, which a stream capture would not allow)."""
    if entry[4]:
        return
    _buf, _rows, ev, built_on, _done = entry
    s = torch.cuda.current_stream() if stream is None else stream
    if torch.cuda.is_current_stream_capturing():
        if s.cuda_stream != built_on:
            s.wait_event(ev)  # becomes a dependency of the captured graph on the build
        return
    if ev.query():
        entry[4] = True
    elif s.cuda_stream != built_on:
        s.wait_event(ev)


def kernel_status() -> int:
    """Status word of the tensor-core kernel (0 = no bounded wait timed out).  Synchronises."""
    v = ctypes.c_uint32()
    check(_lib.lib().wsvd_kernel_status(ctypes.byref(v)), "wsvd_kernel_status")
    return v.value


def build_params(
    q, b_seq_len, b_req_idx, req_to_token, max_len, latent_k, k_scale, latent_v, v_scale, wk, wk_scale=None,
    wv=None, out=None, pos_offset=None, theta=10000.0, sm_scale=0.0, rope_layout="half", split_len=0,
    kernel="auto", stream=None, max_position=None,
) -> Tuple[LatentDecodeParams, list]:
    """Validate tensors and fill a WsvdLatentDecodeParams.  Returns the struct and the
    list of tensors it points into (keep them alive until the launch is enqueued).

    `max_position`: with `pos_offset`, an upper bound of pos_offset[b] + len_b (the position
    table must reach it); when absent it is read from `pos_offset` with a device
    synchronisation."""
    _cuda_tensor("q", q, (torch.float16,), 3)
    B, Hq, D = q.shape
    _cuda_tensor("cache_latent_k", latent_k, (torch.int8, torch.float16), 3)
    _cuda_tensor("cache_latent_v", latent_v, (torch.int8, torch.float16), 3)
    _need(latent_k.dtype == latent_v.dtype, "latent K and V must share a dtype", TypeError)
    is_i8 = latent_k.dtype == torch.int8
    Hkv, Rk = latent_k.shape[1], latent_k.shape[2]
    Rv = latent_v.shape[2]
    _need(latent_v.shape[1] == Hkv, "latent K and V disagree on the number of KV heads")
    _need(Hq % Hkv == 0, f"q heads ({Hq}) must be a multiple of KV heads ({Hkv})")
    _need(D in (16, 32, 64, 128), f"head_dim {D} not in {{16, 32, 64, 128}}")
    _need(1 <= Rk <= 128 and 1 <= Rv <= 128, "per-head rank must be in [1, 128]")
    _cuda_tensor("wk", wk, (torch.int8, torch.float16), 2)
    _need(wk.shape[1] == D * Hkv, f"wk.shape[1] ({wk.shape[1]}) != head_dim * kv_heads ({D * Hkv})")
    _need(wk.shape[0] == Rk, f"wk.shape[0] ({wk.shape[0]}) != rank_k ({Rk})")
    if is_i8:
        _need(k_scale is not None and v_scale is not None, "int8 latents need k_scale and v_scale", TypeError)
        _cuda_tensor("cache_latent_k_scale", k_scale, (torch.float16,), 2, inner_contiguous=False)
        _cuda_tensor("cache_latent_v_scale", v_scale, (torch.float16,), 2, inner_contiguous=False)
        _need(k_scale.shape[0] == latent_k.shape[0] and k_scale.shape[1] == Hkv, "k_scale must be [T, Hkv]")
        _need(v_scale.shape[0] == latent_v.shape[0] and v_scale.shape[1] == Hkv, "v_scale must be [T, Hkv]")
    else:
        _need(k_scale is None and v_scale is None, "f16 latents take no scales", TypeError)
    if wk.dtype == torch.int8:
        _need(wk_scale is not None, "int8 wk needs wk_scale", TypeError)
        _need(wk_scale.is_cuda and wk_scale.dtype == torch.float16, "wk_scale must be a CUDA f16 tensor", TypeError)
        _need(wk_scale.numel() == D * Hkv and wk_scale.is_contiguous(),
              f"wk_scale must hold head_dim * kv_heads = {D * Hkv} contiguous values")
    else:
        _need(wk_scale is None, "f16 wk takes no wk_scale", TypeError)
    if wv is not None:
        _cuda_tensor("wv", wv, (torch.float16,), 2)
        _need(tuple(wv.shape) == (Rv, D * Hkv), f"wv must be [rank_v, head_dim*kv_heads] = {(Rv, D * Hkv)}")
    for name, t in (("b_seq_len", b_seq_len), ("b_req_idx", b_req_idx)):
        _cuda_tensor(name, t, (torch.int32,), 1)
        _need(t.shape[0] == B, f"{name} must have batch ({B}) entries")
    _cuda_tensor("req_to_token_indexs", req_to_token, (torch.int32,), 2)
    _need(0 <= max_len <= req_to_token.shape[1], "max_len_in_batch exceeds the page-table width")
    if pos_offset is not None:
        _cuda_tensor("pos_offset", pos_offset, (torch.int32,), 1)
        _need(pos_offset.shape[0] == B, "pos_offset must have batch entries")
    out_w = D if wv is not None else Rv
    if out is not None:
        _cuda_tensor("out", out, (torch.float16,), 3)
        _need(tuple(out.shape) == (B, Hq, out_w), f"out must be {(B, Hq, out_w)}, got {tuple(out.shape)}")
    _need(rope_layout in ROPE, f"rope_layout must be one of {list(ROPE)}")
    _need(kernel in KERNEL, f"kernel must be one of {list(KERNEL)}")

    p = LatentDecodeParams()
    p.q, p.q_stride_b, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    p.latent_k, p.k_stride_t, p.k_stride_h = latent_k.data_ptr(), latent_k.stride(0), latent_k.stride(1)
    p.latent_v, p.v_stride_t, p.v_stride_h = latent_v.data_ptr(), latent_v.stride(0), latent_v.stride(1)
    if is_i8:
        p.k_scale, p.ks_stride_t, p.ks_stride_h = k_scale.data_ptr(), k_scale.stride(0), k_scale.stride(1)
        p.v_scale, p.vs_stride_t, p.vs_stride_h = v_scale.data_ptr(), v_scale.stride(0), v_scale.stride(1)
    p.wk, p.wk_stride_r = wk.data_ptr(), wk.stride(0)
    p.wk_scale = None if wk_scale is None else wk_scale.data_ptr()
    if wv is not None:
        p.wv, p.wv_stride_r = wv.data_ptr(), wv.stride(0)
    p.req_to_token, p.rtt_stride = req_to_token.data_ptr(), req_to_token.stride(0)
    p.b_req_idx, p.b_seq_len = b_req_idx.data_ptr(), b_seq_len.data_ptr()
    p.pos_offset = None if pos_offset is None else pos_offset.data_ptr()
    if out is not None:
        p.out, p.out_stride_b, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    p.batch, p.n_q_heads, p.n_kv_heads, p.head_dim, p.rank_k, p.rank_v = B, Hq, Hkv, D, Rk, Rv
    p.max_len = int(max_len)
    p.latent_dtype = I8 if is_i8 else F16
    p.wk_dtype = I8 if wk.dtype == torch.int8 else F16
    p.rope_layout = ROPE[rope_layout]
    p.split_len = int(split_len)
    p.kernel = KERNEL[kernel]
    p.theta, p.sm_scale = float(theta), float(sm_scale)
    p.n_token_slots = min(latent_k.shape[0], latent_v.shape[0])
    if D == 128 and kernel != "generic":
        reach = int(max_len)
        if pos_offset is not None:
            reach = int(max_position) if max_position is not None else reach + max(0, int(pos_offset.max().item()))
        table, rows = rope_table(q.device, reach, D, theta, stream=stream)[:2]
        p.rope_table, p.rope_table_rows = table.data_ptr(), rows
    keep = [q, latent_k, latent_v, k_scale, v_scale, wk, wk_scale, wv, req_to_token, b_req_idx, b_seq_len,
            pos_offset, out]
    return p, keep


def plan(p: LatentDecodeParams) -> Tuple[int, int]:
    sl, ns = ctypes.c_int32(), ctypes.c_int32()
    check(_lib.lib().wsvd_latent_decode_plan(ctypes.byref(p), ctypes.byref(sl), ctypes.byref(ns)), "plan")
    return sl.value, ns.value


def workspace_bytes(p: LatentDecodeParams) -> int:
    return int(_lib.lib().wsvd_latent_decode_workspace_bytes(ctypes.byref(p)))


def _stream(stream) -> ctypes.c_void_p:
    s = torch.cuda.current_stream() if stream is None else stream
    return ctypes.c_void_p(s.cuda_stream)


def _cached_params(tag, q3, infer_state, latent_k, k_scale, latent_v, v_scale, wk, wk_scale, wv, pos_offset, theta,
                   rope_layout, split_len, kernel, stream):
    """A private copy of the validated argument block for this set of buffers and options.

    A decode loop calls with the same buffers every step, so the validated block is kept
    per (address, shape, stride) signature.  What can change underneath a cached block is
    refreshed on every hit: the position table (it is replaced by a larger one when a
    longer context arrives).  The caller gets a copy, so that filling in `out` does not
    touch the cached block and calls from several threads do not share mutable state."""
    rtt = infer_state.req_manager.req_to_token_indexs
    max_len = int(infer_state.max_len_in_batch)
    key = (tag, _sig(q3), _sig(infer_state.b_seq_len), _sig(infer_state.b_req_idx), _sig(rtt), max_len,
           _sig(latent_k), _sig(k_scale), _sig(latent_v), _sig(v_scale), _sig(wk), _sig(wk_scale), _sig(wv),
           _sig(pos_offset), float(theta), rope_layout, int(split_len), kernel)
    # position offsets may change inside the same buffer and decide how far the position table must
    # reach, so such calls are validated (and the reach read back from the device) every time
    hit = _CALLS.get(key) if pos_offset is None else None
    if hit is None:
        p, _keep = build_params(
            q3, infer_state.b_seq_len, infer_state.b_req_idx, rtt, max_len, latent_k, k_scale, latent_v, v_scale,
            wk, wk_scale, wv=wv, out=None, pos_offset=pos_offset, theta=theta, rope_layout=rope_layout,
            split_len=split_len, kernel=kernel, stream=stream)
        hit = (p, workspace_bytes(p))
        if pos_offset is None:
            if len(_CALLS) >= 64:
                _CALLS.clear()
            _CALLS[key] = hit
    cached, need = hit
    p = LatentDecodeParams.from_buffer_copy(cached)
    if cached.rope_table:
        entry = rope_table(q3.device, max(max_len, cached.rope_table_rows if pos_offset is not None else 0),
                           p.head_dim, theta, stream=stream)
        p.rope_table, p.rope_table_rows = entry[0].data_ptr(), entry[1]
        _order_after_table(entry, stream)
    return p, need


@torch.no_grad()
def latent_decode(
    q, infer_state, latent_k, k_scale, latent_v, v_scale, wk, wk_scale=None, *, wv=None, out=None,
    workspace: Optional[torch.Tensor] = None, alloc_tensor_func: Callable = torch.empty, pos_offset=None,
    theta=10000.0, rope_layout="half", split_len=0, kernel="auto", stream=None,
) -> torch.Tensor:
    """Fused latent decode attention.  Returns O_lat [B,Hq,Rv] (f16), or O [B,Hq,D] when
    `wv` ([Rv, Hkv*D] f16) is given.  `workspace` is an optional CUDA byte/float buffer of
    at least workspace_bytes(); when absent it is taken from `alloc_tensor_func`."""
    B = int(infer_state.batch_size)
    q3 = q.view(B, q.shape[-2], q.shape[-1]) if q.dim() != 3 else q
    p, need = _cached_params("decode", q3, infer_state, latent_k, k_scale, latent_v, v_scale, wk, wk_scale, wv,
                             pos_offset, theta, rope_layout, split_len, kernel, stream)
    out_w = p.head_dim if wv is not None else p.rank_v
    if out is None:
        out = alloc_tensor_func((B, p.n_q_heads, out_w), dtype=q.dtype, device=q.device)
    else:
        _cuda_tensor("out", out, (torch.float16,), 3)
        _need(tuple(out.shape) == (B, p.n_q_heads, out_w), f"out must be {(B, p.n_q_heads, out_w)}")
    p.out, p.out_stride_b, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    if workspace is None:
        workspace = alloc_tensor_func(((need + 3) // 4,), dtype=torch.float32, device=q.device)
    else:
        _need(workspace.is_cuda and workspace.is_contiguous(), "workspace must be a contiguous CUDA tensor")
    have = workspace.numel() * workspace.element_size()
    with torch.cuda.device(q.device):
        check(_lib.lib().wsvd_latent_decode(ctypes.byref(p), _ptr(workspace), have, _stream(stream)),
              "wsvd_latent_decode")
    return out


@torch.no_grad()
def latent_decode_gather(q, infer_state, latent_k, k_scale, latent_v, v_scale, wk, wk_scale, peers, *, wv=None,
                         workspace: Optional[torch.Tensor] = None, theta=10000.0, rope_layout="half", split_len=0,
                         kernel="auto", stream=None) -> None:
    """This rank's head shard of the op with the head all-gather fused into the merge
    kernel: rows go straight into every rank's gathered buffer (`peers`, a filled
    `_lib.PeerSet`, see `wsvd_b200.dist.PeerGather`).  Arguments as `latent_decode`, with the
    LOCAL heads."""
    B = int(infer_state.batch_size)
    q3 = q.view(B, q.shape[-2], q.shape[-1]) if q.dim() != 3 else q
    p, need = _cached_params("gather", q3, infer_state, latent_k, k_scale, latent_v, v_scale, wk, wk_scale, wv,
                             None, theta, rope_layout, split_len, kernel, stream)
    if workspace is None:
        workspace = torch.empty(((need + 3) // 4,), dtype=torch.float32, device=q.device)
    have = workspace.numel() * workspace.element_size()
    with torch.cuda.device(q.device):
        check(_lib.lib().wsvd_latent_decode_gather(ctypes.byref(p), ctypes.byref(peers), _ptr(workspace), have,
                                                   _stream(stream)), "wsvd_latent_decode_gather")


@torch.no_grad()
def latent_decode_stage1(q, latent_k, k_scale, latent_v, v_scale, wk, wk_scale, req_to_token, b_req_idx, b_seq_len,
                         max_len, mid_out, mid_out_lse, block_seq, *, theta=10000.0, rope_layout="half",
                         kernel="auto", stream=None):
    """Split-KV stage 1 into caller-owned partial buffers mid_out [B,Hq,n_splits,Rv] f32
    and mid_out_lse [B,Hq,n_splits] f32."""
    p, keep = build_params(q, b_seq_len, b_req_idx, req_to_token, int(max_len), latent_k, k_scale, latent_v, v_scale,
                           wk, wk_scale, theta=theta, rope_layout=rope_layout, split_len=int(block_seq),
                           kernel=kernel)
    _need(mid_out.is_cuda and mid_out.dtype == torch.float32 and mid_out.is_contiguous(), "mid_out: contiguous CUDA f32")
    _need(mid_out_lse.is_cuda and mid_out_lse.dtype == torch.float32 and mid_out_lse.is_contiguous(),
          "mid_out_logsumexp: contiguous CUDA f32")
    B, Hq, ns, Rv = mid_out.shape
    _need((B, Hq, Rv) == (p.batch, p.n_q_heads, p.rank_v), "mid_out must be [B, Hq, n_splits, rank_v]")
    _need(tuple(mid_out_lse.shape) == (B, Hq, ns), "mid_out_logsumexp must be [B, Hq, n_splits]")
    with torch.cuda.device(q.device):
        check(_lib.lib().wsvd_latent_decode_stage1(ctypes.byref(p), _ptr(mid_out), _ptr(mid_out_lse), ns,
                                                   _stream(stream)), "wsvd_latent_decode_stage1")


@torch.no_grad()
def decode_stage2(mid_out, mid_out_lse, b_seq_len, out, block_seq, *, wv=None, n_kv_heads=None, stream=None):
    """Split-KV stage 2: merge partials by log-sum-exp weights into `out` (f16)."""
    for name, t in (("mid_out", mid_out), ("mid_out_logexpsum", mid_out_lse)):
        _need(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous(), f"{name}: contiguous CUDA f32")
    B, Hq, ns, W = mid_out.shape
    _need(tuple(mid_out_lse.shape) == (B, Hq, ns), "mid_out_logexpsum must be [B, Hq, n_splits]")
    _cuda_tensor("B_Seqlen", b_seq_len, (torch.int32,), 1)
    _cuda_tensor("O", out, (torch.float16,), 3)
    head_dim, hkv, wv_stride = 0, 1, 0
    if wv is not None:
        _cuda_tensor("wv", wv, (torch.float16,), 2)
        hkv = int(n_kv_heads or Hq)
        head_dim = wv.shape[1] // hkv
        wv_stride = wv.stride(0)
        _need(tuple(out.shape) == (B, Hq, head_dim), "out must be [B, Hq, head_dim] when wv is given")
    else:
        _need(tuple(out.shape) == (B, Hq, W), "out must be [B, Hq, width]")
    with torch.cuda.device(out.device):
        check(_lib.lib().wsvd_decode_stage2(
            _ptr(mid_out), _ptr(mid_out_lse), _ptr(b_seq_len), _ptr(out), out.stride(0), out.stride(1),
            B, Hq, ns, W, int(block_seq), _ptr(wv), wv_stride, hkv, head_dim, _stream(stream)), "wsvd_decode_stage2")


@torch.no_grad()
def dense_decode(q, infer_state, cache_k, cache_v, out=None, alloc_tensor_func: Callable = torch.empty,
                 workspace=None, split_len=0, stream=None):
    """Dense f16 flash-decoding baseline: q [B,Hq,D], caches [T,Hkv,D] f16 -> [B,Hq,D] f16."""
    from ._lib import DenseDecodeParams

    _cuda_tensor("q", q, (torch.float16,), 3)
    B, Hq, D = q.shape
    _cuda_tensor("cache_k", cache_k, (torch.float16,), 3)
    _cuda_tensor("cache_v", cache_v, (torch.float16,), 3)
    Hkv = cache_k.shape[1]
    _need(cache_k.shape[2] == D and cache_v.shape[2] == D, "q and K/V disagree on head_dim")
    _need(cache_v.shape[1] == Hkv and Hq % Hkv == 0, "bad head counts")
    _need(D in (16, 32, 64, 128), f"head_dim {D} not in {{16, 32, 64, 128}}")
    rtt = infer_state.req_manager.req_to_token_indexs
    _cuda_tensor("b_seq_len", infer_state.b_seq_len, (torch.int32,), 1)
    _cuda_tensor("b_req_idx", infer_state.b_req_idx, (torch.int32,), 1)
    _cuda_tensor("req_to_token_indexs", rtt, (torch.int32,), 2)
    if out is None:
        out = alloc_tensor_func((B, Hq, D), dtype=q.dtype, device=q.device)
    _cuda_tensor("out", out, (torch.float16,), 3)
    p = DenseDecodeParams()
    p.q, p.q_stride_b, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    p.k, p.k_stride_t, p.k_stride_h = cache_k.data_ptr(), cache_k.stride(0), cache_k.stride(1)
    p.v, p.v_stride_t, p.v_stride_h = cache_v.data_ptr(), cache_v.stride(0), cache_v.stride(1)
    p.req_to_token, p.rtt_stride = rtt.data_ptr(), rtt.stride(0)
    p.b_req_idx, p.b_seq_len = infer_state.b_req_idx.data_ptr(), infer_state.b_seq_len.data_ptr()
    p.out, p.out_stride_b, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    p.batch, p.n_q_heads, p.n_kv_heads, p.head_dim = B, Hq, Hkv, D
    p.max_len, p.split_len = int(infer_state.max_len_in_batch), int(split_len)
    need = int(_lib.lib().wsvd_dense_decode_workspace_bytes(ctypes.byref(p)))
    if workspace is None:
        workspace = alloc_tensor_func(((need + 3) // 4,), dtype=torch.float32, device=q.device)
    have = workspace.numel() * workspace.element_size()
    with torch.cuda.device(q.device):
        check(_lib.lib().wsvd_dense_decode_f16(ctypes.byref(p), _ptr(workspace), have, _stream(stream)),
              "wsvd_dense_decode_f16")
    return out


def latent_quant_append(x_k, x_v, infer_state, cache_latent_k, cache_latent_k_scale, cache_latent_v,
                        cache_latent_v_scale, stream=None):
    """Quantise the new token's latents and store them in the cache (in place).

    x_k [B, Hkv, Rk], x_v [B, Hkv, Rv] (f16 or f32) are written, as int8 with one f16 scale
    per (sequence, head), to token slot ``req_to_token_indexs[b_req_idx[b], b_seq_len[b]]``:
    ``infer_state.b_seq_len`` holds the lengths before the append, the caller increments it
    afterwards.  Quantiser: fake_quant/quant_utils.py:30-33,175-184 against the stored f16
    scale.  The reference has no counterpart (efficiency/layer_utils.py:319-321 drops the
    new latents)."""
    from ._lib import QuantAppendParams

    _cuda_tensor("x_k", x_k, (torch.float16, torch.float32), 3)
    _cuda_tensor("x_v", x_v, (torch.float16, torch.float32), 3)
    _need(x_k.dtype == x_v.dtype, "x_k and x_v must share a dtype", TypeError)
    B, Hkv, Rk = x_k.shape
    Rv = x_v.shape[2]
    _need(x_v.shape[:2] == (B, Hkv), "x_k and x_v disagree on batch or heads")
    _cuda_tensor("cache_latent_k", cache_latent_k, (torch.int8,), 3)
    _cuda_tensor("cache_latent_v", cache_latent_v, (torch.int8,), 3)
    _cuda_tensor("cache_latent_k_scale", cache_latent_k_scale, (torch.float16,), 2, inner_contiguous=False)
    _cuda_tensor("cache_latent_v_scale", cache_latent_v_scale, (torch.float16,), 2, inner_contiguous=False)
    _need(cache_latent_k.shape[1:] == (Hkv, Rk) and cache_latent_v.shape[1:] == (Hkv, Rv),
          "cache shapes must be [T, Hkv, Rk] and [T, Hkv, Rv]")
    _need(0 < Rk <= 128 and 0 < Rv <= 128, "ranks must be in 1..128")
    rtt = infer_state.req_manager.req_to_token_indexs
    _cuda_tensor("b_seq_len", infer_state.b_seq_len, (torch.int32,), 1)
    _cuda_tensor("b_req_idx", infer_state.b_req_idx, (torch.int32,), 1)
    _cuda_tensor("req_to_token_indexs", rtt, (torch.int32,), 2)
    _need(infer_state.b_seq_len.numel() == B and infer_state.b_req_idx.numel() == B, "batch metadata must have B entries")
    p = QuantAppendParams()
    p.x_k, p.xk_stride_b, p.xk_stride_h = x_k.data_ptr(), x_k.stride(0), x_k.stride(1)
    p.x_v, p.xv_stride_b, p.xv_stride_h = x_v.data_ptr(), x_v.stride(0), x_v.stride(1)
    p.latent_k, p.k_stride_t, p.k_stride_h = cache_latent_k.data_ptr(), cache_latent_k.stride(0), cache_latent_k.stride(1)
    p.latent_v, p.v_stride_t, p.v_stride_h = cache_latent_v.data_ptr(), cache_latent_v.stride(0), cache_latent_v.stride(1)
    p.k_scale, p.ks_stride_t, p.ks_stride_h = (cache_latent_k_scale.data_ptr(), cache_latent_k_scale.stride(0),
                                               cache_latent_k_scale.stride(1))
    p.v_scale, p.vs_stride_t, p.vs_stride_h = (cache_latent_v_scale.data_ptr(), cache_latent_v_scale.stride(0),
                                               cache_latent_v_scale.stride(1))
    p.req_to_token, p.rtt_stride = rtt.data_ptr(), rtt.stride(0)
    p.b_req_idx, p.b_seq_len = infer_state.b_req_idx.data_ptr(), infer_state.b_seq_len.data_ptr()
    p.batch, p.n_kv_heads, p.rank_k, p.rank_v = B, Hkv, Rk, Rv
    p.max_len = rtt.shape[1]
    p.x_dtype = 1 if x_k.dtype == torch.float16 else 2
    with torch.cuda.device(x_k.device):
        check(_lib.lib().wsvd_latent_quant_append_i8(ctypes.byref(p), _stream(stream)), "wsvd_latent_quant_append_i8")


# ---- element-wise pieces of the decode step (one kernel each)

def rms_norm(x: torch.Tensor, eps: float = 1e-5, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """x [rows, cols] f16 -> x * rsqrt(mean(x^2) + eps), f16 (no weight vector)."""
    _cuda_tensor("x", x, (torch.float16,), 2)
    _need(x.is_contiguous(), "x must be contiguous")
    if out is None:
        out = torch.empty_like(x)
    check(_lib.lib().wsvd_rms_norm_f16(_ptr(x), _ptr(out), x.shape[0], x.shape[1], float(eps), _stream(stream)),
          "wsvd_rms_norm_f16")
    return out


def add_rms_norm(x: torch.Tensor, delta: torch.Tensor, eps: float = 1e-5, stream=None):
    """(x + delta, RMSNorm(x + delta)) for x, delta [rows, cols] f16: the residual update and the
    next block's normalisation as one kernel."""
    _cuda_tensor("x", x, (torch.float16,), 2)
    _cuda_tensor("delta", delta, (torch.float16,), 2)
    _need(x.is_contiguous() and delta.is_contiguous() and x.shape == delta.shape, "x and delta: same contiguous shape")
    x_out, y = torch.empty_like(x), torch.empty_like(x)
    check(_lib.lib().wsvd_add_rms_norm_f16(_ptr(x), _ptr(delta), _ptr(x_out), _ptr(y), x.shape[0], x.shape[1],
                                           float(eps), _stream(stream)), "wsvd_add_rms_norm_f16")
    return x_out, y


def rope_half_(q: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, stream=None) -> torch.Tensor:
    """Half-split rotary embedding of q [B, H, D] f16 in place at positions pos [B] int32;
    inv_freq [D/2] f32 on the device.  q may be a column slice of a wider matrix (any stride between
    sequences; the heads of a sequence are contiguous)."""
    _cuda_tensor("q", q, (torch.float16,), 3)
    _cuda_tensor("pos", pos, (torch.int32,), 1)
    _cuda_tensor("inv_freq", inv_freq, (torch.float32,), 1)
    _need(q.stride(1) == q.shape[2] and pos.numel() == q.shape[0] and inv_freq.numel() * 2 == q.shape[2],
          "q must be [B, H, D] with contiguous heads, B positions and D/2 frequencies")
    check(_lib.lib().wsvd_rope_half_f16(_ptr(q), q.stride(0), _ptr(pos), _ptr(inv_freq), q.shape[0], q.shape[1],
                                        q.shape[2], _stream(stream)), "wsvd_rope_half_f16")
    return q


def silu_mul(up: torch.Tensor, gate: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """up * silu(gate), f16 [rows, cols]; up and gate may be column slices of one wider matrix."""
    _cuda_tensor("up", up, (torch.float16,), 2)
    _cuda_tensor("gate", gate, (torch.float16,), 2)
    _need(up.shape == gate.shape, "up and gate must have the same shape")
    if out is None:
        out = torch.empty(up.shape, dtype=up.dtype, device=up.device)
    _need(out.is_contiguous() and out.shape == up.shape, "out must be contiguous and shaped like up")
    check(_lib.lib().wsvd_silu_mul_f16(_ptr(up), up.stride(0), _ptr(gate), gate.stride(0), _ptr(out), up.shape[0],
                                       up.shape[1], _stream(stream)), "wsvd_silu_mul_f16")
    return out
