"""The CPU oracle against golden vectors produced by the reference's own code
(generator: tests/golden/make_golden.py)."""
import os

import numpy as np
import torch

from oracle import latent_decode_oracle as orc

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    z = np.load(os.path.join(GOLD, name))
    return {k: torch.from_numpy(z[k]) if z[k].ndim else z[k].item() for k in z.files}


def _report(a, b):
    d = (a.double() - b.double()).abs()
    return d.max().item(), (d / b.double().abs().clamp_min(1e-2)).max().item()


def test_torch_reference_interleaved_rope_gqa_ragged_paged():
    """reference_online_rope_attention_projected_only
    (efficiency/test_functional_layer.py:176-226) vs the oracle composed the same
    way: RMSNorm -> Wdq -> Wuq view -> op (interleaved pairing) -> Wuvout."""
    g = _load("torch_ref_gqa_ragged_paged.npz")
    D, Hq, Hkv = g["head_dim"], g["q_head_num"], g["kv_head_num"]
    x = g["x"]
    B = x.shape[0]
    xn = orc._rms_norm(x)
    lq = (xn @ g["Wdq"]).view(B, 1, Hq, -1)[:, 0]
    q = torch.einsum("bhr,hrd->bhd", lq, g["Wuq"].view(Hq, -1, D))
    o_lat, _ = orc.latent_decode_oracle(
        q, g["b_seq_len"], g["b_req_idx"], g["req_to_token"], g["cache_latent_k"], None,
        g["cache_latent_v"], None, g["Wuk"], rope_layout="interleaved", dtype=torch.float64)
    out = (o_lat.view(B, 1, -1) @ g["Wuvout"].double().view(-1, Hq * D)).view(B, 1, Hq * D)
    max_abs, _ = _report(out, g["out"])
    assert max_abs < 2e-5, max_abs
    # the kernel's half-split pairing is a different function of the same inputs
    o_half, _ = orc.latent_decode_oracle(
        q, g["b_seq_len"], g["b_req_idx"], g["req_to_token"], g["cache_latent_k"], None,
        g["cache_latent_v"], None, g["Wuk"], rope_layout="half", dtype=torch.float64)
    assert (o_half - o_lat).abs().max() > 1e-2


def test_triton_f16_latent_kernel_half_rope():
    """token_decode_attention_flash_latent_per_head_decoding_rope
    (efficiency/kernel/flash_decoding.py:57-95) run in Triton's interpreter."""
    g = _load("triton_f16_ragged_paged.npz")
    args = (g["q"], g["b_seq_len"], g["b_req_idx"], g["req_to_token"], g["cache_latent_k"], None,
            g["cache_latent_v"], None, g["wk"])
    o32, _ = orc.latent_decode_oracle(*args)
    max_abs, _ = _report(o32, g["out"].float())
    # the reference rounds K, cos, sin and the q.K products to f16
    assert max_abs < 4e-3, max_abs
    ok = orc.latent_decode_kernel_order_oracle(*args, block_seq=256, block_n=32)
    max_abs_k, _ = _report(ok.float(), g["out"].float())
    assert max_abs_k < 1.5e-3, max_abs_k
    # split-KV form of the oracle merges to the same result
    mid, lse = orc.latent_decode_stage1_oracle(*args, block_seq=256)
    o_split = orc.combine_oracle(mid, lse, g["b_seq_len"], 256)
    assert (o_split - o32).abs().max() < 1e-5


def test_triton_i8_latent_kernel_gqa():
    """token_decode_attention_flash_int8_latent_per_head_decoding_rope
    (efficiency/kernel/flash_decoding.py:3-55) run in Triton's interpreter."""
    g = _load("triton_i8_gqa_ragged_paged.npz")
    args = (g["q"], g["b_seq_len"], g["b_req_idx"], g["req_to_token"], g["cache_latent_k"],
            g["cache_latent_k_scale"], g["cache_latent_v"], g["cache_latent_v_scale"], g["wk"], g["wk_scale"])
    o32, _ = orc.latent_decode_oracle(*args)
    max_abs, _ = _report(o32, g["out"].float())
    assert max_abs < 4e-3, max_abs
    ok = orc.latent_decode_kernel_order_oracle(*args, block_seq=256, block_n=32)
    max_abs_k, _ = _report(ok.float(), g["out"].float())
    assert max_abs_k < 1.5e-3, max_abs_k


def test_triton_dense_flash_decoding():
    """token_decode_attention_flash_decoding (efficiency/kernel/flash_decoding.py:98-131)."""
    g = _load("triton_dense_gqa_ragged_paged.npz")
    o = orc.dense_decode_oracle(g["q"], g["b_seq_len"], g["b_req_idx"], g["req_to_token"],
                                g["cache_k"], g["cache_v"])
    max_abs, _ = _report(o, g["out"].float())
    assert max_abs < 1e-3, max_abs


def test_quantize_per_token_convention():
    """scale = amax/127 stored as f16, round-to-nearest, clamp
    (fake_quant/quant_utils.py:30-33,179-184)."""
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(5, 3, 64, generator=gen)
    x[0, 0] = 0
    qv, s = orc.quantize_per_token(x)
    assert qv.dtype == torch.int8 and s.dtype == torch.float16
    assert s[0, 0] == 1 and (qv[0, 0] == 0).all()
    assert qv.float().abs().max() <= 128 and qv.float().abs().amax(dim=-1).flatten()[1:].min() >= 126
    err = (qv.float() * s.float().unsqueeze(-1) - x).abs()
    assert (err <= 0.5 * s.float().unsqueeze(-1) + 1e-6).all()
