"""wsvd_latent_decode_static, the entry point for hosts that cannot give the library a
workspace (no device allocation possible around the call), against the regular entry point.

Collected last on purpose: if it fails, a run that stops at the first failure has already
run every other test."""
import ctypes

import pytest
import torch

from wsvd_b200 import _lib, inputs, ops

pytestmark = pytest.mark.gpu

STATIC_BYTES = 8 << 20


def _params(case, out, **kw):
    s = case.infer_state
    p, keep = ops.build_params(case.q, s.b_seq_len, s.b_req_idx, s.req_manager.req_to_token_indexs,
                               s.max_len_in_batch, case.latent_k, case.k_scale, case.latent_v, case.v_scale,
                               case.wk, None, wv=case.wv, out=out, **kw)
    return p, keep


@pytest.mark.parametrize("kernel", ["auto", "generic"])
def test_static_scratch_entry_matches_workspace_entry_twice(kernel):
    lib = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (lens, seed) in enumerate([([1500, 700, 0, 2049], 31), ([333, 2048, 64, 1], 32)]):
        case = inputs.make_case(len(lens), 8, 128, 64, 48, lens, 2049, seed=seed).to("cuda")
        want = torch.empty(len(lens), 8, 128, dtype=torch.float16, device="cuda")
        got = torch.full_like(want, float("nan"))
        p_ref, keep_ref = _params(case, want, kernel=kernel)
        ws = torch.empty(ops.workspace_bytes(p_ref), dtype=torch.uint8, device="cuda")
        _lib.check(lib.wsvd_latent_decode(ctypes.byref(p_ref), ctypes.c_void_p(ws.data_ptr()), ws.numel(), stream),
                   "wsvd_latent_decode")
        p_new, keep_new = _params(case, got, kernel=kernel)
        _lib.check(lib.wsvd_latent_decode_static(ctypes.byref(p_new), stream), "wsvd_latent_decode_static")
        torch.cuda.synchronize()
        assert ops.kernel_status() == 0
        assert torch.isfinite(got).all(), f"call {call}"
        err = (got.float() - want.float()).abs()
        # same kernels, same split plan: the tolerance of the parity tests is far from reached
        assert (err <= 2e-3 + 1e-2 * want.float().abs()).all(), f"call {call}: max abs {err.max().item()}"
        assert torch.equal(got, want), f"call {call}: expected bitwise-equal results"


def test_static_scratch_entry_rejects_oversized_requests():
    lib = _lib.lib()
    lens = [16]
    case = inputs.make_case(1, 4, 128, 64, 64, lens, 16, seed=5).to("cuda")
    out = torch.empty(1, 4, 128, dtype=torch.float16, device="cuda")
    p, keep = _params(case, out)
    # pretend the batch is far larger than the scratch can serve: rejected before any launch
    p.batch, p.max_len = 60000, 32768
    assert lib.wsvd_latent_decode_workspace_bytes(ctypes.byref(p)) > STATIC_BYTES
    assert lib.wsvd_latent_decode_static(ctypes.byref(p), None) == 8  # WSVD_ERR_TOO_LARGE
    assert lib.wsvd_latent_decode_static(None, None) == 1
