"""The synthetic-input generators (the stand-in for the reference's create_test_data_layer,
efficiency/layer_utils.py:38-95, with the distributions the benchmark states): shapes, the
strided views over head-major storage, the page table, poison in the padding, and that the
token-major re-layout holds the same data — checked through the oracle."""
import torch

from oracle.latent_decode_oracle import latent_decode_oracle, quantize_per_token
from wsvd_b200 import inputs


def test_workload_specs_and_algorithmic_bytes():
    c2 = inputs.WORKLOADS["c2_13b_b16_s8192"]
    lens = inputs.seq_lens_for(c2)
    assert lens == [8192] * 16
    assert inputs.algorithmic_bytes(lens, c2.heads, c2.rank_k, c2.rank_v) == 16 * 40 * 8192 * 132 == 692060160
    c4 = inputs.WORKLOADS["c4_13b_b64_ragged32k"]
    l4 = inputs.seq_lens_for(c4)
    assert len(l4) == 64 and min(l4) >= 1024 and max(l4) <= 32768 and l4 == inputs.seq_lens_for(c4)  # seeded
    assert inputs.algorithmic_bytes(l4, 40, 64, 48) == sum(l4) * 40 * 116
    assert inputs.algorithmic_bytes([10], 2, 64, 64, latent_bytes=2) == 10 * 2 * 256  # f16 latents: no scales


def test_case_views_alias_head_major_storage_and_padding_is_poisoned():
    case = inputs.make_case(2, 3, 128, 64, 48, [5, 9], 12, seed=4)
    st = case.storage
    assert st["latent_k"].shape == (2, 3, 12, 64) and st["latent_v"].shape == (2, 3, 12, 48)
    table = case.infer_state.req_manager.req_to_token_indexs
    assert table.dtype == torch.int32 and table.shape == (2, 12)
    for b, h, s in [(0, 0, 0), (1, 2, 8), (1, 0, 3), (0, 2, 4)]:
        slot = int(table[b, s])
        assert torch.equal(case.latent_k[slot, h], st["latent_k"][b, h, s])
        assert torch.equal(case.latent_v[slot, h], st["latent_v"][b, h, s])
        assert case.k_scale[slot, h] == st["k_scale"][b, h, s]
    # what lies beyond a sequence's length must never be read: int8 -128 and NaN scales
    assert (st["latent_k"][0, :, 5:] == -128).all() and torch.isnan(st["k_scale"][0, :, 5:]).all()
    assert (st["latent_v"][1, :, 9:] == -128).all() and torch.isnan(st["v_scale"][1, :, 9:]).all()
    # orthonormal columns per head: w[r, h*D + d] = U[h, d, r]
    u = case.wk.float().view(64, 3, 128).permute(1, 2, 0)
    eye = torch.einsum("hdr,hds->hrs", u, u)
    assert (eye - torch.eye(64)).abs().max() < 5e-3


def test_generator_quantiser_is_the_oracle_quantiser():
    x = torch.randn(7, 5, 64, generator=torch.Generator().manual_seed(8)) * 2.5
    x[3, 1] = 0
    q, s = inputs._quantize(x)
    q2, s2 = quantize_per_token(x)
    assert torch.equal(q, q2) and torch.equal(s, s2)


def test_token_major_relayout_gives_the_same_attention():
    case = inputs.make_case(2, 2, 128, 64, 64, [40, 17], 48, seed=6)
    want, _ = latent_decode_oracle(*case.oracle_args())
    for seed in (None, 3):
        tm = inputs.token_major_copy(case, shuffle_seed=seed)
        assert tm.latent_k.is_contiguous() and tm.latent_k.shape == (2 * 48, 2, 64)
        got, _ = latent_decode_oracle(*tm.oracle_args())
        assert torch.equal(got, want)
