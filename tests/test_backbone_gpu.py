"""The decode step of the low-rank-KV backbone (down-projection, quantise-and-append, latent
decode attention, o-projection, FFN) against a CPU restatement built from the oracle."""
import pytest
import torch

from oracle.latent_decode_oracle import latent_decode_oracle, quant_append_oracle

pytestmark = pytest.mark.gpu


def _cpu_step(model, x):
    """fp32 on the CPU with the model's own weights and (cloned) caches."""
    from wsvd_b200.backbone import _rms_norm, rope_half

    sp, B, Hl = model.spec, model.batch, model.local_heads
    x = x.float().cpu()
    lens = model.before.b_seq_len.cpu()
    idx = model.before.b_req_idx.cpu()
    table = model.before.req_manager.req_to_token_indexs.cpu()
    for L in model.layers:
        W = {k: getattr(L, k).float().cpu() for k in ("Wq", "A_k", "A_v", "Wo", "Wup", "Wgate", "Wdown")}
        xn = _rms_norm(x)
        q = rope_half((xn @ W["Wq"]).view(B, Hl, sp.head_dim), lens, sp.theta)
        xk = (xn @ W["A_k"]).view(B, Hl, sp.rank_k)
        xv = (xn @ W["A_v"]).view(B, Hl, sp.rank_v)
        lk, ks, lv, vs = (t.cpu().clone() for t in (L.k_store, L.ks_store, L.v_store, L.vs_store))
        S = lk.shape[2]
        T = (B - 1) * Hl * S + S
        lk_v = lk.as_strided((T, Hl, sp.rank_k), (sp.rank_k, S * sp.rank_k, 1))
        lv_v = lv.as_strided((T, Hl, sp.rank_v), (sp.rank_v, S * sp.rank_v, 1))
        ks_v, vs_v = ks.as_strided((T, Hl), (1, S)), vs.as_strided((T, Hl), (1, S))
        quant_append_oracle(xk, xv, lens, idx, table, lk_v, ks_v, lv_v, vs_v)
        _, o = latent_decode_oracle(q.to(torch.float16), lens + 1, idx, table, lk_v, ks_v, lv_v, vs_v, L.wk.cpu(),
                                    wv=L.wv.cpu(), theta=sp.theta)
        x = x + o.reshape(B, -1).float() @ W["Wo"]
        h = _rms_norm(x)
        x = x + ((h @ W["Wup"]) * torch.nn.functional.silu(h @ W["Wgate"])) @ W["Wdown"]
    return x


def test_two_layer_step_matches_cpu_restatement():
    from wsvd_b200 import ops
    from wsvd_b200.backbone import BackboneSpec, LatentDecoder

    spec = BackboneSpec(layers=2, hidden=512, heads=4, head_dim=128, ffn=1024, rank_k=64, rank_v=64)
    model = LatentDecoder(spec, batch=3, context=300, capacity=310, device="cuda", seed=1)
    x = (torch.randn(3, 512, generator=torch.Generator().manual_seed(2)) * 0.5).to(torch.float16).cuda()
    want = _cpu_step(model, x)  # before the GPU step touches the caches
    got = model.step(x)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    err = (got.float().cpu() - want).abs().max().item()
    scale = want.abs().max().item()
    # f16 GEMMs against fp32 ones, and a latent that rounds the other way now and then
    assert err <= 3e-2 * scale, (err, scale)
    # the token landed where the next step will look for it
    model.advance()
    got2 = model.step(got)
    torch.cuda.synchronize()
    assert torch.isfinite(got2).all() and ops.kernel_status() == 0
    assert int(model.after.b_seq_len[0]) == 302


def test_captured_step_replays_like_the_eager_one():
    from wsvd_b200 import ops
    from wsvd_b200.backbone import BackboneSpec, LatentDecoder

    spec = BackboneSpec(layers=2, hidden=512, heads=4, head_dim=128, ffn=1024, rank_k=64, rank_v=64)
    x = (torch.randn(3, 512, generator=torch.Generator().manual_seed(4)) * 0.5).to(torch.float16).cuda()
    eager = LatentDecoder(spec, batch=3, context=200, capacity=210, device="cuda", seed=9)
    eager.step(x)
    eager.advance()
    want = eager.step(x)                      # the second step
    graphed = LatentDecoder(spec, batch=3, context=200, capacity=210, device="cuda", seed=9)
    graph, y = graphed.capture(x)             # runs the first step while warming up
    graph.replay()                            # the second step
    graphed.context += 1
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert torch.equal(y, want)
    assert int(graphed.after.b_seq_len[0]) == int(eager.after.b_seq_len[0]) + 1  # eager has not advanced yet


def test_elementwise_kernels_match_the_torch_chains():
    """RMSNorm, RoPE and SiLU*up as single kernels against the chains of torch ops they replace."""
    from wsvd_b200 import ops
    from wsvd_b200.backbone import _rms_norm, rope_half

    g = torch.Generator(device="cuda").manual_seed(7)
    x = (torch.randn(5, 4096, generator=g, device="cuda") * 0.7).to(torch.float16)
    got, want = ops.rms_norm(x), _rms_norm(x)
    assert (got.float() - want.float()).abs().max().item() <= 2e-3  # one f16 ulp near 2: the row sums differ in order

    d = (torch.randn(5, 4096, generator=g, device="cuda") * 0.3).to(torch.float16)
    xs, ys = ops.add_rms_norm(x, d)
    assert torch.equal(xs, x + d)
    assert (ys.float() - _rms_norm(x + d).float()).abs().max().item() <= 2e-3

    q = (torch.randn(5, 6, 128, generator=g, device="cuda")).to(torch.float16)
    pos = torch.tensor([0, 1, 77, 4095, 31999], dtype=torch.int32, device="cuda")
    inv = 10000.0 ** (-torch.arange(0, 128, 2, device="cuda", dtype=torch.float32) / 128)
    want = rope_half(q, pos, 10000.0)
    got = ops.rope_half_(q.clone(), pos, inv)
    assert (got.float() - want.float()).abs().max().item() <= 4e-3  # f16 rounding of values up to ~4

    up = (torch.randn(3, 11008, generator=g, device="cuda") * 2).to(torch.float16)
    gate = (torch.randn(3, 11008, generator=g, device="cuda") * 2).to(torch.float16)
    want = up * torch.nn.functional.silu(gate)
    got = ops.silu_mul(up, gate)
    assert (got.float() - want.float()).abs().max().item() <= 8e-3  # one f16 ulp at the largest products (~8..16)
    torch.cuda.synchronize()


def test_step_with_torch_elementwise_chains_agrees():
    """The fused element-wise kernels change nothing beyond f16 rounding."""
    from wsvd_b200.backbone import BackboneSpec, LatentDecoder

    spec = BackboneSpec(layers=2, hidden=512, heads=4, head_dim=128, ffn=1024, rank_k=64, rank_v=64)
    x = (torch.randn(3, 512, generator=torch.Generator().manual_seed(2)) * 0.5).to(torch.float16).cuda()
    a = LatentDecoder(spec, batch=3, context=300, capacity=310, device="cuda", seed=1).step(x)
    b = LatentDecoder(spec, batch=3, context=300, capacity=310, device="cuda", seed=1, fused_elementwise=False).step(x)
    torch.cuda.synchronize()
    assert (a.float() - b.float()).abs().max().item() <= 2e-2 * b.float().abs().max().item()
