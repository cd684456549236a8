"""The warp-MMA kernel (f16 or int8 latents, head_dim 16..128, even ranks) against the CPU oracle,
on the shapes the tcgen05 kernel does not take."""
import pytest
import torch

from tests.helpers import assert_close, oracle_for
from wsvd_b200 import inputs, ops
from wsvd_b200.kernel.flash_decoding import (
    token_decode_attention_flash_int8_latent_per_head_decoding_rope as op_i8,
    token_decode_attention_flash_latent_per_head_decoding_rope as op_f16,
)

pytestmark = pytest.mark.gpu


def _run(case, kernel="mma", **kw):
    c = case.to("cuda")
    H, D = c.q.shape[1], c.q.shape[2]
    if c.latent_k.dtype == torch.int8:
        out = op_i8(c.q, c.infer_state, H, D, c.latent_k, c.k_scale, c.latent_v, c.v_scale, c.wk, None,
                    kernel=kernel, **kw)
    else:
        out = op_f16(c.q, c.infer_state, H, D, c.latent_k, c.latent_v, c.wk, kernel=kernel, **kw)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("latent_dtype", [torch.float16, torch.int8])
@pytest.mark.parametrize("d,rk,rv", [(128, 62, 62), (128, 128, 96), (128, 64, 64), (64, 40, 24), (32, 6, 2)])
def test_ranks_and_head_dims(latent_dtype, d, rk, rv):
    """Ranks that are not multiples of 16 (the accuracy pipeline's uniform 62), above 64, tiny; five
    heads, so the last group of four is not full; an empty sequence and one of a single token."""
    lens = [400, 129, 0, 1, 1031]
    case = inputs.make_case(len(lens), 5, d, rk, rv, lens, 1031, seed=d + rk, latent_dtype=latent_dtype)
    got = _run(case)
    assert_close(got, oracle_for(case), f"D={d} rank {rk}/{rv} {latent_dtype}")
    assert (got[2] == 0).all()
    assert torch.equal(got, _run(case)), "bitwise repeatable"


@pytest.mark.parametrize("split_len", [0, 100, 256, 1000])
def test_f16_latents_split_lengths(split_len):
    """Any split length, not only multiples of the 16-token tile."""
    case = inputs.make_case(2, 4, 128, 64, 64, [1500, 777], 1500, seed=5, latent_dtype=torch.float16)
    assert_close(_run(case, split_len=split_len), oracle_for(case), f"split_len={split_len}")


def test_auto_takes_f16_latents_to_the_mma_kernel_and_agrees_with_the_generic_one():
    case = inputs.make_case(2, 8, 128, 64, 64, [2048, 900], 2048, seed=9, latent_dtype=torch.float16)
    auto, mma, gen = _run(case, "auto"), _run(case, "mma"), _run(case, "generic")
    assert torch.equal(auto, mma)
    assert_close(mma, gen.float().cpu(), "mma vs generic")


def test_f16_latents_long_context_against_fp64():
    n = 32768
    case = inputs.make_case(1, 1, 128, 64, 64, [n], n, seed=98, latent_dtype=torch.float16)
    assert_close(_run(case), oracle_for(case, dtype=torch.float64), "32k vs fp64")


def test_interleaved_pairing_small_head_dim():
    case = inputs.make_case(2, 3, 64, 32, 32, [515, 130], 515, seed=76, latent_dtype=torch.float16)
    assert_close(_run(case, rope_layout="interleaved"), oracle_for(case, rope_layout="interleaved"), "interleaved")


def test_odd_rank_is_refused_when_the_kernel_is_forced():
    case = inputs.make_case(1, 2, 128, 63, 64, [100], 100, seed=1)
    with pytest.raises(Exception):
        _run(case, "mma")
    assert_close(_run(case, "auto"), oracle_for(case), "odd rank on the generic kernel")
