"""Dense f16 flash-decoding baseline against the oracle and the reference's Triton output."""
import os

import numpy as np
import pytest
import torch

from oracle import latent_decode_oracle as orc
from tests.helpers import assert_close
from wsvd_b200.infer_state import InferState
from wsvd_b200.kernel.flash_decoding import token_decode_attention_flash_decoding

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("d,hq,hkv", [(128, 4, 4), (128, 8, 2), (64, 4, 2), (32, 2, 2), (16, 2, 1)])
def test_dense_matches_oracle(d, hq, hkv):
    gen = torch.Generator().manual_seed(d + hq)
    lens = [0, 1, 300, 1025, 64, 2047]
    B, S = len(lens), 2048
    q = torch.randn(B, hq, d, generator=gen).half()
    k = torch.randn(B * S, hkv, d, generator=gen).half()
    v = torch.randn(B * S, hkv, d, generator=gen).half()
    table = torch.randperm(B * S, generator=gen).to(torch.int32).view(B, S)
    st = InferState(B, S, lens, device="cpu", req_to_token=table)
    want = orc.dense_decode_oracle(q, st.b_seq_len, st.b_req_idx, table, k, v)
    stg = InferState(B, S, lens, device="cuda", req_to_token=table)
    got = token_decode_attention_flash_decoding(q.cuda(), stg, hq, d, k.cuda(), v.cuda())
    torch.cuda.synchronize()
    assert_close(got, want, f"dense D={d}")
    assert (got[0] == 0).all()


def test_dense_matches_reference_triton_golden():
    z = np.load(os.path.join(GOLD, "triton_dense_gqa_ragged_paged.npz"))
    g = {k: torch.from_numpy(z[k]) for k in z.files}
    B, Hq, D = g["q"].shape
    st = InferState(B, g["req_to_token"].shape[1], g["b_seq_len"].tolist(), device="cuda",
                    req_to_token=g["req_to_token"], b_req_idx=g["b_req_idx"])
    got = token_decode_attention_flash_decoding(g["q"].cuda(), st, Hq, D, g["cache_k"].cuda(), g["cache_v"].cuda())
    torch.cuda.synchronize()
    assert_close(got, g["out"].float(), "dense vs reference Triton kernel", atol=2e-3, rtol=1e-2)
