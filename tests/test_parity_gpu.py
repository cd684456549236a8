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

KERNELS = ["generic", "tc"]


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
    if kernel == "tc" and not (rk == 64 and rv in (48, 64)):
        pytest.skip("tensor-core kernel covers rank_k 64, rank_v 48/64")
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


@pytest.mark.parametrize("kernel", ["generic"])
@pytest.mark.parametrize("d,rk,rv", [(16, 16, 16), (32, 16, 32), (64, 32, 48)])
def test_small_head_dims_generic(kernel, d, rk, rv):
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
