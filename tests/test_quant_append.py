"""The decode-step cache producer: quantise the new token's latents and append them.

CPU part: the oracle's quantiser against a golden vector made with the reference's own
`sym_quant` (fake_quant/quant_utils.py:30-33; generator: tests/golden/make_golden.py).
GPU part: the CUDA kernel through the C ABI against the oracle, bit for bit.
"""
import os

import numpy as np
import pytest
import torch

from oracle.latent_decode_oracle import quant_append_oracle, quantize_per_token

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "quant_ref_sym_int8.npz")


def test_oracle_quantiser_matches_reference_golden():
    d = np.load(GOLDEN)
    q, s = quantize_per_token(torch.from_numpy(d["x"]))
    assert q.dtype == torch.int8 and s.dtype == torch.float16
    assert np.array_equal(q.numpy(), d["q"])
    assert np.array_equal(s.numpy(), d["scale"])


def test_oracle_append_writes_only_the_new_slots():
    g = torch.Generator().manual_seed(3)
    B, H, Rk, Rv, max_len = 3, 2, 8, 4, 6
    T = B * max_len
    table = torch.randperm(T, generator=g).to(torch.int32).view(B, max_len)
    lens = torch.tensor([0, 5, 6], dtype=torch.int32)  # the last one has no free column
    lk = torch.full((T, H, Rk), -99, dtype=torch.int8)
    lv = torch.full((T, H, Rv), -99, dtype=torch.int8)
    ks = torch.full((T, H), 7.0, dtype=torch.float16)
    vs = torch.full((T, H), 7.0, dtype=torch.float16)
    xk, xv = torch.randn(B, H, Rk, generator=g), torch.randn(B, H, Rv, generator=g)
    quant_append_oracle(xk, xv, lens, torch.arange(B, dtype=torch.int32), table, lk, ks, lv, vs)
    written = {int(table[0, 0]), int(table[1, 5])}
    for t in range(T):
        if t in written:
            assert (lk[t] != -99).any() and (ks[t] != 7.0).all()
        else:
            assert (lk[t] == -99).all() and (lv[t] == -99).all() and (ks[t] == 7.0).all()
    qk, sk = quantize_per_token(xk)
    assert torch.equal(lk[int(table[1, 5])], qk[1]) and torch.equal(ks[int(table[1, 5])], sk[1])


def test_oracle_scale_stays_a_finite_nonzero_f16():
    g = torch.Generator().manual_seed(9)
    x = torch.stack([torch.randn(16, generator=g) * 2e-6, torch.randn(16, generator=g) * 3e7, torch.zeros(16)])
    q, s = quantize_per_token(x)
    assert torch.isfinite(s.float()).all() and (s.float() > 0).all()
    assert s[2] == 1.0 and (q[2] == 0).all()
    assert q[0].abs().max() > 0 and q[1].abs().max() == 127 or q[1].min() == -128


class _Req:
    def __init__(self, t):
        self.req_to_token_indexs = t


class _State:
    def __init__(self, lens, idx, table):
        self.b_seq_len, self.b_req_idx, self.req_manager = lens, idx, _Req(table)
        self.batch_size = lens.numel()
        self.max_len_in_batch = int(lens.max()) if lens.numel() else 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("B,H,Rk,Rv", [(5, 3, 64, 64), (64, 40, 64, 48), (2, 1, 128, 16), (3, 4, 33, 7)])
def test_append_matches_oracle_bit_exact(dtype, B, H, Rk, Rv):
    from wsvd_b200 import ops

    g = torch.Generator().manual_seed(B * 131 + Rk)
    max_len = 9
    T = B * max_len + 3
    table = torch.randperm(T, generator=g)[: B * max_len].to(torch.int32).view(B, max_len)
    idx = torch.randperm(B, generator=g).to(torch.int32)
    lens = torch.randint(0, max_len, (B,), generator=g, dtype=torch.int32)
    xk = (torch.randn(B, H, Rk, generator=g) * torch.rand(B, H, 1, generator=g) * 4).to(dtype)
    xv = (torch.randn(B, H, Rv, generator=g) * 0.3).to(dtype)
    xk[0, 0] = 0  # all-zero row -> scale 1
    # rows whose amax/127 leaves the f16 range: the stored scale is clamped, never 0 or inf
    xk[1, 0] = (torch.randn(Rk, generator=g) * 2e-6).to(dtype)
    if dtype == torch.float32:
        xv[1, 0] = torch.randn(Rv, generator=g) * 3e7
    lk = torch.randint(-128, 128, (T, H, Rk), generator=g, dtype=torch.int8)
    lv = torch.randint(-128, 128, (T, H, Rv), generator=g, dtype=torch.int8)
    ks = torch.rand(T, H, generator=g).to(torch.float16)
    vs = torch.rand(T, H, generator=g).to(torch.float16)
    ref = [t.clone() for t in (lk, ks, lv, vs)]
    quant_append_oracle(xk, xv, lens, idx, table, *ref)

    dev = "cuda"
    got = [t.to(dev) for t in (lk, ks, lv, vs)]
    st = _State(lens.to(dev), idx.to(dev), table.to(dev))
    ops.latent_quant_append(xk.to(dev), xv.to(dev), st, got[0], got[1], got[2], got[3])
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    for name, r, o in zip(("latent_k", "k_scale", "latent_v", "v_scale"), ref, got):
        assert torch.equal(r, o.cpu()), name


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["generic", "tc"])
def test_append_then_decode_sees_the_new_token(kernel):
    """Append a token with the kernel, extend the lengths, and decode: the result must match
    the oracle run on a cache the oracle appended to."""
    from tests.helpers import assert_close, oracle_for
    from wsvd_b200 import inputs, ops
    from wsvd_b200.kernel.flash_decoding import (
        token_decode_attention_flash_int8_latent_per_head_decoding_rope as op_i8,
    )

    case = inputs.make_case(3, 8, 128, 64, 64, [17, 128, 299], 300, seed=11)
    c = case.to("cuda")
    g = torch.Generator().manual_seed(5)
    xk = torch.randn(3, 8, 64, generator=g).to(torch.float16)
    xv = torch.randn(3, 8, 64, generator=g).to(torch.float16)
    s = case.infer_state
    quant_append_oracle(xk, xv, s.b_seq_len, s.b_req_idx, s.req_manager.req_to_token_indexs,
                        case.latent_k, case.k_scale, case.latent_v, case.v_scale)
    ops.latent_quant_append(xk.cuda(), xv.cuda(), c.infer_state, c.latent_k, c.k_scale, c.latent_v, c.v_scale)
    for st in (s, c.infer_state):
        st.b_seq_len += 1
        st.max_len_in_batch = int(st.b_seq_len.max())
    d = c.infer_state
    out = op_i8(c.q, d, c.q.shape[1], c.q.shape[2], c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None,
                kernel=kernel)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert_close(out, oracle_for(case), "decode after append")
