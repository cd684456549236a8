"""Shared helpers for the parity tests."""
import torch

from oracle import latent_decode_oracle as orc

ATOL, RTOL = 2e-3, 1e-2  # |cuda - oracle| <= ATOL + RTOL*|oracle|, the op's stated tolerance


def oracle_for(case, wv=False, dtype=torch.float32, **kw):
    o_lat, o = orc.latent_decode_oracle(*case.oracle_args(), wv=case.wv if wv else None, dtype=dtype, **kw)
    return o if wv else o_lat


def assert_close(got, want, what="", atol=ATOL, rtol=RTOL):
    got = got.detach().float().cpu()
    want = want.float()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite values in the CUDA result"
    err = (got - want).abs()
    bound = atol + rtol * want.abs()
    worst = (err - bound).max().item()
    assert worst <= 0, f"{what}: max_abs={err.max().item():.3e} exceeds {atol}+{rtol}*|ref| by {worst:.3e}"
    return err.max().item()
