"""The C-ABI library on a machine without a GPU: it loads, exports every symbol that
include/wsvd_b200.h declares, and rejects bad arguments with status codes before any
CUDA call is made."""
import ctypes
import os
import re

import pytest

from wsvd_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "wsvd_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wsvd_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.lib()
    names = _declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SYMBOLS, f"{name} has no ctypes prototype"


def test_abi_version_and_status_strings():
    lib = _lib.lib()
    assert lib.wsvd_abi_version() == 1
    for code in range(0, 9):
        assert lib.wsvd_status_string(code)
    assert lib.wsvd_status_string(0) == b"ok"
    assert b"unknown" in lib.wsvd_status_string(99)


def _params(**kw):
    p = _lib.LatentDecodeParams()
    fake = 0x1000  # never dereferenced on the host: validation only looks at NULL-ness
    for f in ("q", "latent_k", "latent_v", "k_scale", "v_scale", "wk", "req_to_token", "b_req_idx", "b_seq_len", "out"):
        setattr(p, f, fake)
    p.batch, p.n_q_heads, p.n_kv_heads, p.head_dim, p.rank_k, p.rank_v = 2, 8, 8, 128, 64, 64
    p.max_len, p.latent_dtype, p.wk_dtype, p.theta = 1000, 0, 1, 10000.0
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("field,value,status", [
    ("q", None, 1), ("latent_k", None, 1), ("b_seq_len", None, 1), ("out", None, 1),
    ("head_dim", 96, 2), ("n_kv_heads", 3, 2), ("rank_k", 0, 2), ("rank_v", 129, 2), ("batch", -1, 2),
    ("latent_dtype", 7, 3), ("k_scale", None, 3), ("rope_layout", 5, 3), ("kernel", 9, 3),
    ("batch", 70000, 8), ("theta", 0.0, 2),
])
def test_validation_status_codes(field, value, status):
    lib = _lib.lib()
    p = _params(**{field: value})
    ws = ctypes.c_void_p(0x2000)
    assert lib.wsvd_latent_decode(ctypes.byref(p), ws, 1 << 30, None) == status


@pytest.mark.parametrize("batch", [0, 2])
@pytest.mark.parametrize("field,value,status", [("q", None, 1), ("head_dim", 96, 2), ("latent_dtype", 7, 3)])
def test_static_entry_validates_like_the_workspace_entry(batch, field, value, status):
    """An invalid argument block is rejected by wsvd_latent_decode_static with the same code as
    by wsvd_latent_decode, also when the batch is empty (and before any CUDA call)."""
    lib = _lib.lib()
    p = _params(batch=batch, **{field: value})
    assert lib.wsvd_latent_decode(ctypes.byref(p), ctypes.c_void_p(0x2000), 1 << 30, None) == status
    assert lib.wsvd_latent_decode_static(ctypes.byref(p), None) == status


def test_static_entry_accepts_a_valid_empty_batch():
    lib = _lib.lib()
    p = _params(batch=0)
    assert lib.wsvd_latent_decode_static(ctypes.byref(p), None) == 0


def test_int8_wk_needs_scale_and_workspace_checks():
    lib = _lib.lib()
    p = _params(wk_dtype=0)
    assert lib.wsvd_latent_decode(ctypes.byref(p), ctypes.c_void_p(0x2000), 1 << 30, None) == 3
    p = _params()
    need = lib.wsvd_latent_decode_workspace_bytes(ctypes.byref(p))
    assert need > 0
    assert lib.wsvd_latent_decode(ctypes.byref(p), None, need, None) == 1
    assert lib.wsvd_latent_decode(ctypes.byref(p), ctypes.c_void_p(0x2000), need - 1, None) == 5
    assert lib.wsvd_latent_decode(ctypes.byref(p), ctypes.c_void_p(0x2001), need, None) == 4
    assert lib.wsvd_latent_decode(None, ctypes.c_void_p(0x2000), need, None) == 1


def test_split_plan_is_consistent_with_workspace_size():
    lib = _lib.lib()
    for max_len, split in [(1, 0), (127, 0), (8192, 0), (32768, 0), (5000, 256), (5000, 1024)]:
        for kernel in (0, 1):
            p = _params(max_len=max_len, split_len=split, kernel=kernel)
            sl, ns = ctypes.c_int32(), ctypes.c_int32()
            assert lib.wsvd_latent_decode_plan(ctypes.byref(p), ctypes.byref(sl), ctypes.byref(ns)) == 0
            assert sl.value > 0 and ns.value * sl.value >= max_len and (ns.value - 1) * sl.value < max(max_len, 1)
            if split:
                assert sl.value == split
            need = lib.wsvd_latent_decode_workspace_bytes(ctypes.byref(p))
            assert need >= p.batch * p.n_q_heads * ns.value * (p.rank_v + 1) * 4


def test_warp_mma_kernel_plan_and_workspace():
    """f16 latents, rank 62, head_dim 64: shapes of the warp-MMA kernel.  Its plan cuts the context into
    fixed splits of 256..4096 tokens, and the workspace holds the partials plus a position table of
    [2][rows][head_dim / 2] f16 when the caller passes none."""
    lib = _lib.lib()
    for head_dim, rk, rv, dtype in [(128, 64, 64, 1), (128, 62, 62, 0), (64, 40, 24, 1), (128, 128, 96, 1)]:
        for kernel in (0, 3):
            p = _params(head_dim=head_dim, rank_k=rk, rank_v=rv, latent_dtype=dtype, kernel=kernel, max_len=8192,
                        k_scale=0x1000 if dtype == 0 else None, v_scale=0x1000 if dtype == 0 else None,
                        k_stride_t=rk, k_stride_h=8192 * rk, v_stride_t=rv, v_stride_h=8192 * rv)
            sl, ns = ctypes.c_int32(), ctypes.c_int32()
            assert lib.wsvd_latent_decode_plan(ctypes.byref(p), ctypes.byref(sl), ctypes.byref(ns)) == 0
            assert 256 <= sl.value <= 4096 and sl.value % 128 == 0 and ns.value * sl.value >= 8192
            need = lib.wsvd_latent_decode_workspace_bytes(ctypes.byref(p))
            partials = p.batch * p.n_q_heads * ns.value * (rv + 1) * 4
            assert need >= partials + 8192 * head_dim * 2
    # an odd rank is not a shape of this kernel: no table in the workspace, the generic kernel's plan
    p = _params(rank_k=63, latent_dtype=1, k_scale=None, v_scale=None, max_len=8192)
    sl, ns = ctypes.c_int32(), ctypes.c_int32()
    assert lib.wsvd_latent_decode_plan(ctypes.byref(p), ctypes.byref(sl), ctypes.byref(ns)) == 0
    need = lib.wsvd_latent_decode_workspace_bytes(ctypes.byref(p))
    assert need < p.batch * p.n_q_heads * ns.value * (p.rank_v + 1) * 4 + 4096


def test_empty_batch_is_a_no_op():
    lib = _lib.lib()
    p = _params(batch=0)
    assert lib.wsvd_latent_decode(ctypes.byref(p), None, 0, None) == 0


def test_rope_table_size_and_argument_checks():
    lib = _lib.lib()
    assert lib.wsvd_rope_table_bytes(8192, 128) == 8192 * 256
    assert lib.wsvd_rope_table_bytes(1, 128) == 128 * 256
    assert lib.wsvd_rope_table_bytes(8192, 64) == 0
    assert lib.wsvd_rope_table_init(None, 0, 128, 128, 1e4, None) == 1
    assert lib.wsvd_rope_table_init(ctypes.c_void_p(0x1000), 10, 128, 128, 1e4, None) == 5
    assert lib.wsvd_rope_table_init(ctypes.c_void_p(0x1000), 1 << 20, 128, 64, 1e4, None) == 7


def test_stage2_argument_checks():
    lib = _lib.lib()
    f = ctypes.c_void_p(0x1000)
    assert lib.wsvd_decode_stage2(None, f, f, f, 64, 64, 1, 1, 1, 64, 256, None, 0, 1, 0, None) == 1
    assert lib.wsvd_decode_stage2(f, f, f, f, 64, 64, 1, 1, 1, 200, 256, None, 0, 1, 0, None) == 2
    assert lib.wsvd_decode_stage2(f, f, f, f, 64, 64, 0, 1, 1, 64, 256, None, 0, 1, 0, None) == 0


def _append_params(**kw):
    p = _lib.QuantAppendParams()
    fake = 0x1000
    for f in ("x_k", "x_v", "latent_k", "latent_v", "k_scale", "v_scale", "req_to_token", "b_req_idx", "b_seq_len"):
        setattr(p, f, fake)
    p.batch, p.n_kv_heads, p.rank_k, p.rank_v, p.max_len, p.x_dtype = 2, 4, 64, 48, 100, 1
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("field,value,status", [
    ("x_k", None, 1), ("v_scale", None, 1), ("b_seq_len", None, 1),
    ("rank_k", 129, 2), ("rank_v", 0, 2), ("n_kv_heads", 0, 2), ("batch", -1, 2),
    ("x_dtype", 0, 3), ("x_dtype", 9, 3),
])
def test_quant_append_validation(field, value, status):
    p = _append_params(**{field: value})
    assert _lib.lib().wsvd_latent_quant_append_i8(ctypes.byref(p), None) == status


def test_quant_append_empty_batch_is_a_no_op():
    assert _lib.lib().wsvd_latent_quant_append_i8(ctypes.byref(_append_params(batch=0, x_k=None)), None) == 0


def _peer_set(**kw):
    ps = _lib.PeerSet()
    for i in range(2):
        ps.out[i], ps.flags[i] = 0x3000, 0x4000
    ps.counter = 0x5000
    ps.n_peers, ps.rank, ps.head_offset, ps.epoch = 2, 0, 0, 1
    ps.out_stride_b, ps.out_stride_h = 16 * 128, 128
    for k, v in kw.items():
        setattr(ps, k, v)
    return ps


@pytest.mark.parametrize("field,value,status", [
    ("n_peers", 0, 2), ("n_peers", 9, 2), ("rank", 2, 2), ("rank", -1, 2), ("epoch", 0, 2), ("head_offset", -4, 2),
    ("timeout_ms", -1, 2), ("counter", None, 1),
])
def test_gather_peer_set_validation(field, value, status):
    lib = _lib.lib()
    ps = _peer_set(**{field: value})
    assert lib.wsvd_latent_decode_gather(ctypes.byref(_params()), ctypes.byref(ps), ctypes.c_void_p(0x2000), 1 << 30,
                                         None) == status


def test_gather_needs_every_peer_pointer():
    lib = _lib.lib()
    ps = _peer_set()
    ps.flags[1] = None
    assert lib.wsvd_latent_decode_gather(ctypes.byref(_params()), ctypes.byref(ps), ctypes.c_void_p(0x2000), 1 << 30,
                                         None) == 1
    assert lib.wsvd_latent_decode_gather(ctypes.byref(_params()), None, ctypes.c_void_p(0x2000), 1 << 30, None) == 1


def test_gather_rejects_an_empty_batch():
    """A rank that launched nothing would leave its peers waiting at the group barrier."""
    lib = _lib.lib()
    p = _params()
    p.batch = 0
    assert lib.wsvd_latent_decode_gather(ctypes.byref(p), ctypes.byref(_peer_set()), ctypes.c_void_p(0x2000), 1 << 30,
                                         None) == 2


def test_python_ops_refuse_cpu_tensors():
    """There is no CPU path: the ops raise before anything is launched."""
    import torch

    from wsvd_b200 import ops
    from wsvd_b200.infer_state import InferState

    st = InferState(1, 4, [4], device="cpu")
    x = torch.zeros(1, 2, 8)
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.latent_quant_append(x, x, st, torch.zeros(4, 2, 8, dtype=torch.int8), torch.zeros(4, 2, dtype=torch.float16),
                                torch.zeros(4, 2, 8, dtype=torch.int8), torch.zeros(4, 2, dtype=torch.float16))
    q = torch.zeros(1, 2, 128, dtype=torch.float16)
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.dense_decode(q, st, torch.zeros(4, 2, 128, dtype=torch.float16), torch.zeros(4, 2, 128, dtype=torch.float16))
