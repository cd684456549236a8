"""CUDA op (through the C ABI) against the CPU oracle on identical seeded inputs."""
import pytest
import torch

from tests.helpers import assert_close, oracle_for
from wsvd_b200 import inputs, ops
from wsvd_b200.kernel.flash_decoding import (
    token_decode_attention_flash_int8_latent_per_head_decoding_rope as op_i8,
    token_decode_attention_flash_latent_per_head_decoding_rope as op_f16,
)

pytestmark = pytest.mark.gpu

KERNELS = ["generic", "tc", "mma"]


def run_i8(case, kernel, wv=False, **kw):
    c = case.to("cuda")
    s = c.infer_state
    out = op_i8(c.q, s, c.q.shape[1], c.q.shape[2], c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None,
                wv=c.wv if wv else None, kernel=kernel, **kw)
    torch.cuda.synchronize()
    if kernel != "generic":
        assert ops.kernel_status() == 0, "a bounded wait in the tensor-core kernel timed out"
    return out


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("n", [1, 15, 16, 17, 127, 128, 129, 255, 256, 257, 511, 512, 513, 1000, 2048, 4096 + 7])
def test_lengths_single_sequence(kernel, n):
    case = inputs.make_case(1, 2, 128, 64, 64, [n], max(n, 1), seed=n)
    got = run_i8(case, kernel)
    assert_close(got, oracle_for(case), f"len={n}")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("rk,rv", [(64, 64), (64, 48), (32, 32), (128, 128), (48, 64), (16, 16)])
def test_ranks(kernel, rk, rv):
    case = inputs.make_case(2, 3, 128, rk, rv, [700, 333], 700, seed=rk * 131 + rv)
    if kernel == "tc" and (rk > 64 or rv > 64):
        pytest.skip("tensor-core kernel covers ranks that are multiples of 16 up to 64")
    assert_close(run_i8(case, kernel), oracle_for(case), f"rank {rk}/{rv}")
    assert_close(run_i8(case, kernel, wv=True), oracle_for(case, wv=True), f"rank {rk}/{rv} with U_v")


@pytest.mark.parametrize("kernel", KERNELS)
def test_ragged_batch_with_empty_sequence_and_poisoned_padding(kernel):
    lens = [0, 1, 300, 1025, 64, 2047]
    case = inputs.make_case(len(lens), 4, 128, 64, 64, lens, 2048, seed=7, poison=True)
    got = run_i8(case, kernel)
    want = oracle_for(case)
    assert_close(got, want, "ragged")
    assert (got[0] == 0).all(), "a sequence of length 0 must give zeros"


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("split_len", [128, 256, 512, 1024])
def test_split_lengths(kernel, split_len):
    case = inputs.make_case(2, 2, 128, 64, 64, [1500, 777], 1500, seed=split_len)
    assert_close(run_i8(case, kernel, split_len=split_len), oracle_for(case), f"split_len={split_len}")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("shuffle", [None, 5])
def test_token_major_layout_and_shuffled_page_table(kernel, shuffle):
    base = inputs.make_case(3, 4, 128, 64, 64, [513, 90, 700], 704, seed=11)
    case = inputs.token_major_copy(base, shuffle_seed=shuffle)
    assert_close(run_i8(case, kernel), oracle_for(base), f"token-major shuffle={shuffle}")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("page_size", [128, 64, 256])
def test_paged_cache_with_shuffled_pages(kernel, page_size):
    """Pages of consecutive token slots in shuffled order: tiles that lie inside one page are fetched
    with tensor copies, tiles that straddle pages (page size 64, ragged starts) by the gather."""
    base = inputs.make_case(3, 8, 128, 64, 48, [1025, 300, 1792], 1792, seed=13)
    case = inputs.token_major_copy(base, shuffle_seed=9, page_size=page_size)
    assert_close(run_i8(case, kernel), oracle_for(base), f"paged page_size={page_size}")
    assert_close(run_i8(case, kernel, split_len=256), oracle_for(base), f"paged page_size={page_size}, split 256")


@pytest.mark.parametrize("kernel", KERNELS)
def test_determinism_bitwise(kernel):
    case = inputs.make_case(2, 4, 128, 64, 64, [900, 2000], 2000, seed=3).to("cuda")
    s = case.infer_state
    a = op_i8(case.q, s, 4, 128, case.latent_k, case.k_scale, case.latent_v, case.v_scale, case.wk, None, kernel=kernel)
    b = op_i8(case.q, s, 4, 128, case.latent_k, case.k_scale, case.latent_v, case.v_scale, case.wk, None, kernel=kernel)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.parametrize("kernel", KERNELS)
def test_long_positions_against_fp64(kernel):
    """Positions up to 32k: fp32 angle rounding stays inside the tolerance of the fp64 truth."""
    n = 32768
    case = inputs.make_case(1, 1, 128, 64, 64, [n], n, seed=99)
    got = run_i8(case, kernel, wv=True)
    assert_close(got, oracle_for(case, wv=True, dtype=torch.float64), "32k vs fp64")


@pytest.mark.parametrize("kernel", ["generic", "mma"])
@pytest.mark.parametrize("d,rk,rv", [(16, 16, 16), (32, 16, 32), (64, 32, 48)])
def test_small_head_dims(kernel, d, rk, rv):
    case = inputs.make_case(2, 2, d, rk, rv, [100, 37], 100, seed=d)
    assert_close(run_i8(case, kernel), oracle_for(case), f"D={d}")


@pytest.mark.parametrize("kernel", KERNELS)
def test_f16_latents(kernel):
    case = inputs.make_case(2, 2, 128, 64, 64, [400, 129], 400, seed=21, latent_dtype=torch.float16)
    if kernel == "tc":
        pytest.skip("tensor-core kernel takes int8 latents")
    c = case.to("cuda")
    got = op_f16(c.q, c.infer_state, 2, 128, c.latent_k, c.latent_v, c.wk, kernel=kernel)
    torch.cuda.synchronize()
    assert_close(got, oracle_for(case), "f16 latents")


def _gold(name):
    import os

    import numpy as np

    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name))
    return {k: torch.from_numpy(z[k]) for k in z.files}


@pytest.mark.parametrize("kernel", KERNELS)
def test_reference_triton_int8_golden_gqa_int8_wk(kernel):
    """Inputs and output of the reference's int8 Triton kernel (GQA, int8 wk + wk_scale,
    shuffled page table).  The reference rounds to f16 inside, hence the wider tolerance."""
    from wsvd_b200.infer_state import InferState

    g = _gold("triton_i8_gqa_ragged_paged.npz")
    B, Hq, D = g["q"].shape
    st = InferState(B, g["req_to_token"].shape[1], g["b_seq_len"].tolist(), device="cuda",
                    req_to_token=g["req_to_token"], b_req_idx=g["b_req_idx"])
    got = op_i8(g["q"].cuda(), st, Hq, D, g["cache_latent_k"].cuda(), g["cache_latent_k_scale"].cuda(),
                g["cache_latent_v"].cuda(), g["cache_latent_v_scale"].cuda(), g["wk"].cuda(), g["wk_scale"].cuda(),
                kernel=kernel)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert_close(got, g["out"].float(), "vs reference Triton int8 kernel", atol=4e-3, rtol=1e-2)


def test_reference_triton_f16_golden():
    from wsvd_b200.infer_state import InferState

    g = _gold("triton_f16_ragged_paged.npz")
    B, H, D = g["q"].shape
    st = InferState(B, g["req_to_token"].shape[1], g["b_seq_len"].tolist(), device="cuda",
                    req_to_token=g["req_to_token"], b_req_idx=g["b_req_idx"])
    got = op_f16(g["q"].cuda(), st, H, D, g["cache_latent_k"].cuda(), g["cache_latent_v"].cuda(), g["wk"].cuda())
    torch.cuda.synchronize()
    assert_close(got, g["out"].float(), "vs reference Triton f16 kernel", atol=4e-3, rtol=1e-2)


@pytest.mark.parametrize("kernel", KERNELS)
def test_interleaved_rope_layout(kernel):
    case = inputs.make_case(2, 4, 128, 64, 64, [515, 130], 515, seed=77)
    got = run_i8(case, kernel, rope_layout="interleaved")
    assert_close(got, oracle_for(case, rope_layout="interleaved"), "interleaved pairing")


def test_stage_level_wrappers_match_the_op():
    """Reference-named stage 1 / stage 2 wrappers with caller-owned partial buffers."""
    from wsvd_b200.kernel.flash_int8_latent_per_head_decoding_rope_stage1 import (
        flash_int8_latent_per_head_decode_rope_stage1)
    from wsvd_b200.kernel.flash_latent_per_head_decoding_stage2 import flash_decode_stage2

    case = inputs.make_case(3, 4, 128, 64, 48, [700, 90, 1300], 1300, seed=8)
    c = case.to("cuda")
    s = c.infer_state
    block_seq = 256
    ns = (1300 + block_seq - 1) // block_seq
    mid = torch.zeros(3, 4, ns, 48, dtype=torch.float32, device="cuda")
    lse = torch.zeros(3, 4, ns, dtype=torch.float32, device="cuda")
    out = torch.empty(3, 4, 48, dtype=torch.float16, device="cuda")
    flash_int8_latent_per_head_decode_rope_stage1(c.q, c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None,
                                                  s.req_manager.req_to_token_indexs, s.b_req_idx, s.b_seq_len,
                                                  s.max_len_in_batch, mid, lse, block_seq)
    flash_decode_stage2(mid, lse, s.b_seq_len, out, block_seq)
    torch.cuda.synchronize()
    assert_close(out, oracle_for(case), "stage wrappers")
    from oracle import latent_decode_oracle as orc
    want_mid, want_lse = orc.latent_decode_stage1_oracle(*case.oracle_args(), block_seq=block_seq)
    ok = ~torch.isnan(want_lse)
    assert (mid.cpu()[ok] - want_mid[ok]).abs().max() < 2e-3
    assert (lse.cpu()[ok] - want_lse[ok]).abs().max() < 2e-3
