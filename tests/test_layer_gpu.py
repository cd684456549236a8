"""The reference-named layer wrappers against the layer oracle (structure of
efficiency/test_functional_layer.py:347-399, with the kernel's RoPE pairing)."""
import pytest
import torch

from oracle import latent_decode_oracle as orc
from wsvd_b200 import layer_utils as lu

pytestmark = pytest.mark.gpu


def _setup(B=2, H=8, D=128, S=300, R=64, F=512):
    (x, ck, cv, Wdq, Wdk, Wdv, Wuq, Wuk, Wuv, _Wq, _Wk, _Wv, _k, _v, Wout, Wup, Wgate, Wdown, st) = \
        lu.create_test_data_layer(B, H, D, S, R / D, H, F, device="cuda", seed=5)
    Wuvout = (Wuv.view(R, H, D).permute(1, 0, 2).float() @ Wout.view(H, D, H * D).float()).half()  # [H, R, H*D]
    ck = ck.view(B * S, H, R)
    cv = cv.view(B * S, H, R)
    return x, ck, cv, Wdq, Wdk, Wdv, Wuq, Wuk, Wuvout, Wup, Wgate, Wdown, st, (B, H, D, S, R)


def _oracle_layer(x, attn_args, H, D, Wdq, Wuq, Wuvout, Wup, Wgate, Wdown):
    cpu = lambda t: t.detach().cpu()

    def attn(q):
        o_lat, _ = orc.latent_decode_oracle(q, *attn_args)
        return o_lat

    return orc.layer_oracle(D, H, cpu(x).float(), attn, cpu(Wdq).float(), cpu(Wuq).float(), cpu(Wuvout).float(),
                            cpu(Wup).float(), cpu(Wgate).float(), cpu(Wdown).float())


def test_f16_latent_layer():
    x, ck, cv, Wdq, Wdk, Wdv, Wuq, Wuk, Wuvout, Wup, Wgate, Wdown, st, (B, H, D, S, R) = _setup()
    y = lu.run_flash_latent_per_head_decoding_rope_layer(S, D, H, x, ck, cv, Wdq, Wdk, Wdv, Wuq, Wuk, Wuvout, Wup,
                                                         Wgate, Wdown, st)
    torch.cuda.synchronize()
    args = (st.b_seq_len.cpu(), st.b_req_idx.cpu(), st.req_manager.req_to_token_indexs.cpu(), ck.cpu(), None,
            cv.cpu(), None, Wuk.cpu())
    want = _oracle_layer(x, args, H, D, Wdq, Wuq, Wuvout, Wup, Wgate, Wdown)
    # the reference's own layer check uses atol = rtol = 2e-2 (test_functional_layer.py:395-397)
    torch.testing.assert_close(y.float().cpu(), want, atol=2e-2, rtol=2e-2)


def test_int8_latent_layer():
    x, ck, cv, Wdq, Wdk, Wdv, Wuq, Wuk, Wuvout, Wup, Wgate, Wdown, st, (B, H, D, S, R) = _setup()
    qk, sk = orc.quantize_per_token(ck.cpu())
    qv, sv = orc.quantize_per_token(cv.cpu())
    wq, ws = orc.quantize_per_token(Wuk.cpu().t().contiguous())  # per output column
    wk_i8, wk_scale = wq.t().contiguous(), ws.view(1, -1)
    y = lu.run_flash_int8_latent_per_head_decoding_rope_layer(
        S, D, H, x, qk.cuda(), sk.cuda(), qv.cuda(), sv.cuda(), Wdq, Wdk, Wdv, Wuq, wk_i8.cuda(), wk_scale.cuda(),
        Wuvout, Wup, Wgate, Wdown, st)
    torch.cuda.synchronize()
    args = (st.b_seq_len.cpu(), st.b_req_idx.cpu(), st.req_manager.req_to_token_indexs.cpu(), qk, sk, qv, sv, wk_i8,
            wk_scale)
    want = _oracle_layer(x, args, H, D, Wdq, Wuq, Wuvout, Wup, Wgate, Wdown)
    torch.testing.assert_close(y.float().cpu(), want, atol=2e-2, rtol=2e-2)
