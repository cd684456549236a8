"""Generate the golden vectors under tests/golden/ from the reference's own code.

Run where the reference checkout is available (it is imported, never copied):

    python tests/golden/make_golden.py /path/to/WSVD

Two kinds of vectors are written (numpy .npz, small):

* torch_ref_*.npz   — `reference_online_rope_attention_projected_only`
  (efficiency/test_functional_layer.py:176-226) executed on CPU tensors.  It pins
  gather-by-page-table, K reconstruction, softmax, latent-space V and the Wuvout
  fold.  Its RoPE pairing is the interleaved one of its `_rope` (:25-44).

* triton_*.npz      — the reference op wrappers
  (efficiency/kernel/flash_decoding.py:3-95) with their Triton stage-1/stage-2
  kernels executed by Triton's CPU interpreter.  The kernel sources run unmodified.
  Three things are substituted, all outside the kernels: (1) the interpreter has no
  implementation of the libdevice calls fast_powf/fast_cosf/fast_sinf, so numpy's
  float32 pow/cos/sin stand in for them; (2) the autotune search space is pinned to
  one configuration whose BLOCK_SEQ equals the 256 the wrapper sizes its workspace
  with (other choices make stage 2 read unwritten partials); (3) workspaces are
  allocated on the CPU.  These vectors pin the kernel's half-split RoPE pairing,
  its position convention, the split-KV partial format and the stage-2 merge.

* quant_ref_sym_int8.npz — `sym_quant` (fake_quant/quant_utils.py:30-33) applied with the
  per-token scale of `ActQuantizer.find_params_per_token_groupwise`
  (fake_quant/quant_utils.py:175-184: scale = amax/maxq, 1 for an all-zero row).  It pins
  the rounding and clamp of the latent quantiser that the append kernel restates.
  `quant_utils` imports three modules that the quantiser itself never touches (`utils`,
  `hadamard_utils`, `fast_hadamard_transform`); empty stand-ins are registered for them.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


class _ReqManager:
    def __init__(self, table):
        self.req_to_token_indexs = table


class _InferState:
    """CPU stand-in for efficiency/test_utils.py:9-22 with a caller-chosen page table."""

    def __init__(self, seq_lens, req_idx, table):
        self.batch_size = len(seq_lens)
        self.max_len_in_batch = int(max(seq_lens))
        self.b_seq_len = torch.tensor(seq_lens, dtype=torch.int32)
        self.b_req_idx = torch.tensor(req_idx, dtype=torch.int32)
        self.req_manager = _ReqManager(table)


def _page_table(gen, n_req, max_len, shuffle):
    slots = n_req * max_len
    perm = torch.randperm(slots, generator=gen) if shuffle else torch.arange(slots)
    return perm.to(torch.int32).view(n_req, max_len)


def _patch_interpreter():
    """numpy float32 stand-ins for the three libdevice fast-math calls, which the
    interpreter cannot execute (stage1.py:12-14)."""
    import triton.language as tl
    import triton.runtime.interpreter as interp
    from triton.language.extra.cuda import libdevice

    def wrap(npfn):
        def call(*args):
            datas, like = [], None
            for a in args:
                if isinstance(a, tl.core.tensor):
                    datas.append(np.asarray(a.handle.data, dtype=np.float32))
                    like = a
                else:
                    datas.append(np.float32(getattr(a, "value", a)))
            out = np.asarray(npfn(*datas), dtype=np.float32)
            return tl.core.tensor(interp.TensorHandle(out, tl.float32), like.type)

        return call

    libdevice.fast_powf = wrap(np.power)
    libdevice.fast_cosf = wrap(np.cos)
    libdevice.fast_sinf = wrap(np.sin)


def _pin_autotune(kernel, block_n, block_seq):
    import triton

    kernel.configs = [triton.Config({"BLOCK_N": block_n, "BLOCK_SEQ": block_seq}, num_warps=4, num_stages=1)]


def _cpu_alloc(shape, dtype=None, device=None):
    return torch.zeros(tuple(shape), dtype=dtype)


def make_torch_ref(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "efficiency"))
    import test_functional_layer as tfl

    gen = torch.Generator().manual_seed(1234)
    B, Hq, Hkv, D, R = 2, 4, 2, 64, 32
    max_len = 96
    seq_lens = [96, 41]
    model_dim = Hq * D
    f = torch.float32
    x = torch.randn(B, 1, model_dim, generator=gen, dtype=f)
    Wdq = torch.randn(model_dim, Hq * R, generator=gen, dtype=f) / model_dim ** 0.5
    Wuq = torch.randn(R, Hq * D, generator=gen, dtype=f) / R ** 0.5 * 3.0
    Wuk = torch.randn(R, Hkv * D, generator=gen, dtype=f) / R ** 0.5
    Wuvout = torch.randn(Hq, R, model_dim, generator=gen, dtype=f) / R ** 0.5
    T = 3 * max_len
    ck = torch.randn(T, Hkv, R, generator=gen, dtype=f)
    cv = torch.randn(T, Hkv, R, generator=gen, dtype=f)
    table = _page_table(gen, 3, max_len, shuffle=True)
    st = _InferState(seq_lens, [2, 0], table)
    out = tfl.reference_online_rope_attention_projected_only(D, Hq, Hkv, x, ck, cv, Wdq, Wuq, Wuk, Wuvout, st)
    np.savez_compressed(
        os.path.join(HERE, "torch_ref_gqa_ragged_paged.npz"),
        x=x.numpy(), Wdq=Wdq.numpy(), Wuq=Wuq.numpy(), Wuk=Wuk.numpy(), Wuvout=Wuvout.numpy(),
        cache_latent_k=ck.numpy(), cache_latent_v=cv.numpy(), req_to_token=table.numpy(),
        b_seq_len=st.b_seq_len.numpy(), b_req_idx=st.b_req_idx.numpy(),
        head_dim=D, q_head_num=Hq, kv_head_num=Hkv, out=out.numpy(),
    )
    print("torch_ref_gqa_ragged_paged: out", tuple(out.shape), float(out.abs().max()))


def make_triton(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "efficiency"))
    _patch_interpreter()
    import kernel.flash_decoding as fd
    import kernel.flash_int8_latent_per_head_decoding_rope_stage1 as s1_i8
    import kernel.flash_latent_per_head_decoding_rope_stage1 as s1_f16

    _pin_autotune(s1_i8._fwd_kernel_flash_int8_latent_decode_rope_stage1, 32, 256)
    _pin_autotune(s1_f16._fwd_kernel_flash_latent_decode_rope_stage1, 32, 256)

    # ---- fp16 latents, MHA, ragged, shuffled page table, rank_k 64 / rank_v 48 ----
    gen = torch.Generator().manual_seed(4321)
    B, H, D, Rk, Rv = 2, 2, 128, 64, 48
    max_len = 320
    seq_lens = [300, 77]
    T = 3 * max_len
    h = torch.float16
    q = torch.randn(B, H, D, generator=gen).to(h)
    ck = torch.randn(T, H, Rk, generator=gen).to(h)
    cv = torch.randn(T, H, Rv, generator=gen).to(h)
    wk = (torch.randn(Rk, H * D, generator=gen) / Rk ** 0.5).to(h)
    table = _page_table(gen, 3, max_len, shuffle=True)
    st = _InferState(seq_lens, [1, 2], table)
    out = fd.token_decode_attention_flash_latent_per_head_decoding_rope(
        q, st, H, D, ck, cv, wk, alloc_tensor_func=_cpu_alloc)
    np.savez_compressed(
        os.path.join(HERE, "triton_f16_ragged_paged.npz"),
        q=q.numpy(), cache_latent_k=ck.numpy(), cache_latent_v=cv.numpy(), wk=wk.numpy(),
        req_to_token=table.numpy(), b_seq_len=st.b_seq_len.numpy(), b_req_idx=st.b_req_idx.numpy(),
        out=out.numpy(),
    )
    print("triton_f16_ragged_paged: out", tuple(out.shape), float(out.float().abs().max()))

    # ---- int8 latents + int8 wk, GQA (Hq=4, Hkv=2), ragged, shuffled page table ----
    # Magnitudes are kept small enough that the kernel's cast of the int32 dot to f16
    # before scaling (stage1.py:149-153) stays finite.
    gen = torch.Generator().manual_seed(987)
    B, Hq, Hkv, D, Rk, Rv = 2, 4, 2, 128, 64, 64
    max_len = 288
    seq_lens = [260, 31]
    T = 2 * max_len
    q = torch.randn(B, Hq, D, generator=gen).to(h)
    ck = torch.randint(-20, 21, (T, Hkv, Rk), generator=gen, dtype=torch.int32).to(torch.int8)
    cv = torch.randint(-127, 128, (T, Hkv, Rv), generator=gen, dtype=torch.int32).to(torch.int8)
    ck_s = (torch.rand(T, Hkv, generator=gen) * 0.05 + 0.01).to(h)
    cv_s = (torch.rand(T, Hkv, generator=gen) * 0.02 + 0.005).to(h)
    wk = torch.randint(-20, 21, (Rk, Hkv * D), generator=gen, dtype=torch.int32).to(torch.int8)
    wk_s = (torch.rand(1, Hkv * D, generator=gen) * 0.01 + 0.002).to(h)
    table = _page_table(gen, 2, max_len, shuffle=True)
    st = _InferState(seq_lens, [1, 0], table)
    out = fd.token_decode_attention_flash_int8_latent_per_head_decoding_rope(
        q, st, Hq, D, ck, ck_s, cv, cv_s, wk, wk_s, alloc_tensor_func=_cpu_alloc)
    assert torch.isfinite(out.float()).all()
    np.savez_compressed(
        os.path.join(HERE, "triton_i8_gqa_ragged_paged.npz"),
        q=q.numpy(), cache_latent_k=ck.numpy(), cache_latent_k_scale=ck_s.numpy(),
        cache_latent_v=cv.numpy(), cache_latent_v_scale=cv_s.numpy(), wk=wk.numpy(), wk_scale=wk_s.numpy(),
        req_to_token=table.numpy(), b_seq_len=st.b_seq_len.numpy(), b_req_idx=st.b_req_idx.numpy(),
        out=out.numpy(),
    )
    print("triton_i8_gqa_ragged_paged: out", tuple(out.shape), float(out.float().abs().max()))

    # ---- dense fp16 flash-decoding baseline ----
    gen = torch.Generator().manual_seed(55)
    B, Hq, Hkv, D = 2, 4, 2, 64
    max_len = 300
    seq_lens = [257, 300]
    T = 2 * max_len
    q = torch.randn(B, Hq, D, generator=gen).to(h)
    k = torch.randn(T, Hkv, D, generator=gen).to(h)
    v = torch.randn(T, Hkv, D, generator=gen).to(h)
    table = _page_table(gen, 2, max_len, shuffle=True)
    st = _InferState(seq_lens, [0, 1], table)
    out = fd.token_decode_attention_flash_decoding(q, st, Hq, D, k, v, alloc_tensor_func=_cpu_alloc)
    np.savez_compressed(
        os.path.join(HERE, "triton_dense_gqa_ragged_paged.npz"),
        q=q.numpy(), cache_k=k.numpy(), cache_v=v.numpy(),
        req_to_token=table.numpy(), b_seq_len=st.b_seq_len.numpy(), b_req_idx=st.b_req_idx.numpy(),
        out=out.numpy(),
    )
    print("triton_dense_gqa_ragged_paged: out", tuple(out.shape), float(out.float().abs().max()))


def make_quant(ref_root):
    import types

    for name in ("utils", "hadamard_utils", "fast_hadamard_transform"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.path.insert(0, os.path.join(ref_root, "fake_quant"))
    import quant_utils as qu

    gen = torch.Generator().manual_seed(77)
    x = torch.randn(6, 5, 64, generator=gen) * torch.rand(6, 5, 1, generator=gen) * 3.0
    x[1, 2] = 0.0                      # an all-zero row: scale 1
    x[2, 3, 7] = x[2, 3].abs().max() * -1.0001  # the extreme is negative
    x[3, 1] = torch.round(x[3, 1] * 4) / 8      # many exact .5 ties after scaling
    _, maxq = qu.get_minq_maxq(8, True)
    amax = x.abs().amax(dim=-1, keepdim=True)
    scale = amax / maxq
    scale[amax == 0] = 1
    # the cache stores the scale as f16; quantise against the stored value
    scale_h = scale.to(torch.float16)
    q, _ = qu.sym_quant(x, scale_h.float(), maxq)
    np.savez_compressed(
        os.path.join(HERE, "quant_ref_sym_int8.npz"),
        x=x.numpy(), scale=scale_h.squeeze(-1).numpy(), q=q.to(torch.int8).numpy(),
    )
    print("quant_ref_sym_int8: q range", int(q.min()), int(q.max()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the WSVD checkout>")
    root = sys.argv[1]
    make_torch_ref(root)
    make_triton(root)
    make_quant(root)
