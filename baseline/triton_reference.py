"""Times the reference's own Triton kernels on this GPU, through its unmodified op wrappers.

The files under baseline/_ref/ are verbatim copies made by baseline/fetch_ref.py (git-ignored).
Three wrappers of efficiency/kernel/flash_decoding.py are driven on one workload in the
reference's native token-major layout ([T, Hkv, R] caches, page table):

* token_decode_attention_flash_int8_latent_per_head_decoding_rope (:3-55) — TIMING ONLY: the
  kernel casts its int32 dot to f16 before scaling (stage1.py:149-153), which overflows on
  N(0,1)-scale latents, so its output is not compared;
* token_decode_attention_flash_latent_per_head_decoding_rope (:57-95) on the dequantised
  latents as f16 — timing, and a parity witness for this library's output;
* token_decode_attention_flash_decoding (:98-131), the reference's dense f16 baseline.

Stage 1 of both latent kernels is autotuned over BLOCK_SEQ in {256..2048}, but the wrappers
size the partial buffers and run the merge for 256 (flash_decoding.py:18,31-36,54): only the
configs with BLOCK_SEQ = 256 give a correct result, so the autotuner is restricted to those
(every other tuning parameter stays free).  The first call (the autotune sweep) is not timed.
"""
from __future__ import annotations

import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref", "efficiency")


def available() -> str:
    """'' when the reference copy is present, else the reason it cannot be run."""
    if not os.path.isfile(os.path.join(REF, "kernel", "flash_decoding.py")):
        return "baseline/_ref is absent (run baseline/fetch_ref.py where the WSVD checkout is mounted)"
    try:
        import triton  # noqa: F401
    except Exception as exc:  # pragma: no cover
        return f"triton cannot be imported: {exc}"
    return ""


def _usable_configs(kernel, call, block_seq=256):
    """Keep the autotune configs with the wrapper's BLOCK_SEQ that this Triton build can compile
    and run for `call` (one warm call per config).  Some configs of the reference kernels fail
    in Triton's own compiler passes on sm_100; the kernels themselves are not touched."""
    cand = [c for c in kernel.configs if c.kwargs.get("BLOCK_SEQ") == block_seq]
    good, first_error = [], None
    for c in cand:
        kernel.configs = [c]
        kernel.cache.clear()
        try:
            call()
            torch.cuda.synchronize()
            good.append(c)
        except Exception as exc:  # compile failure of this config
            if first_error is None:
                first_error = f"{type(exc).__name__}: {str(exc)[:120]}"
    kernel.cache.clear()
    kernel.configs = good if good else cand
    return len(good), len(cand), first_error


def _time(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps * 1e3  # microseconds


def run(spec, device, steps=20, warmup=3, ours=None):
    """Returns a dict of µs/layer and GB/s per reference kernel on workload `spec`.
    `ours`: optional callable(token-major case) -> this library's O_lat, compared with the
    reference f16-latent kernel's output."""
    why = available()
    if why:
        return {"unavailable": why}
    # the f16-latent kernel indexes with 32-bit offsets (flash_latent_per_head_decoding_rope_stage1.py:96)
    if spec.batch * spec.max_len * spec.heads * spec.head_dim >= 2 ** 31:
        return {"unavailable": f"{spec.name}: T*H*D exceeds 2^31 elements, which the reference's f16 kernels index "
                               "with 32-bit offsets"}
    from wsvd_b200 import inputs

    if REF not in sys.path:
        sys.path.insert(0, REF)
    import kernel.flash_decoding as fd
    import kernel.flash_int8_latent_per_head_decoding_rope_stage1 as s1_i8
    import kernel.flash_latent_per_head_decoding_rope_stage1 as s1_f16

    case = inputs.token_major_copy(inputs.make_workload(spec, device=device))
    st = case.infer_state
    B, H, D = case.q.shape
    lens = case.seq_lens
    tok_heads = sum(lens) * H
    out = {"workload": spec.name, "layout": "token-major [T, Hkv, R], identity page table",
           "autotune": "restricted to the configs with BLOCK_SEQ=256 that compile here; tuning calls untimed",
           "steps": steps}

    def leg(name, kernel, call, nbytes, extra=None):
        try:
            good, cand, err = _usable_configs(kernel, call) if kernel is not None else (1, 1, None)
            if good == 0:
                out[name] = {"unavailable": f"none of the {cand} BLOCK_SEQ=256 configs compiles with this Triton: {err}"}
                return None
            res = call()  # autotune over the usable configs
            us = _time(call, steps, warmup)
            out[name] = {"us_per_layer": us, "GB/s": nbytes / us / 1e3, "bytes_per_token_head": nbytes // tok_heads,
                         "configs_usable": f"{good} of {cand}"}
            if extra:
                out[name].update(extra)
            return res
        except Exception as exc:
            out[name] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
            return None

    # ---- int8 latents + int8 wk with a per-column scale (the reference int8 signature) ----
    wk32 = case.wk.float()
    wks = (wk32.abs().amax(dim=0, keepdim=True) / 127.0).clamp_min(1e-8)
    wk_i8 = torch.clamp(torch.round(wk32 / wks), -127, 127).to(torch.int8)
    wks = wks.to(torch.float16)
    leg("triton_int8_latent", s1_i8._fwd_kernel_flash_int8_latent_decode_rope_stage1,
        lambda: fd.token_decode_attention_flash_int8_latent_per_head_decoding_rope(
            case.q, st, H, D, case.latent_k, case.k_scale, case.latent_v, case.v_scale, wk_i8, wks),
        tok_heads * (spec.rank_k + spec.rank_v + 4),
        {"note": "timing only: f16 overflow inside the kernel on N(0,1)-scale latents"})

    # ---- f16 latents (the dequantised int8 latents) ----
    lk16 = (case.latent_k.float() * case.k_scale.float().unsqueeze(-1)).to(torch.float16)
    lv16 = (case.latent_v.float() * case.v_scale.float().unsqueeze(-1)).to(torch.float16)
    lk16[torch.isnan(lk16)] = 0  # padding slots carry NaN scales on purpose; the kernel masks them anyway
    lv16[torch.isnan(lv16)] = 0
    o_ref = leg("triton_f16_latent", s1_f16._fwd_kernel_flash_latent_decode_rope_stage1,
                lambda: fd.token_decode_attention_flash_latent_per_head_decoding_rope(case.q, st, H, D, lk16, lv16,
                                                                                      case.wk),
                tok_heads * 2 * (spec.rank_k + spec.rank_v))
    if ours is not None and o_ref is not None:
        o_new = ours(case)
        torch.cuda.synchronize()
        err = (o_new.float() - o_ref.float()).abs()
        ok = bool((err <= 4e-3 + 1e-2 * o_ref.float().abs()).all())
        out["triton_f16_latent"]["parity_witness"] = {
            "max_abs_diff_vs_this_library": float(err.max()), "within_4e-3+1e-2rel": ok,
            "note": "the reference rounds K, cos/sin and products to f16; this library keeps fp32"}
    del lk16, lv16

    # ---- dense f16 flash-decoding on full K/V (no autotune in the reference: BLOCK_N 16, one warp) ----
    T = case.latent_k.shape[0]
    kd = torch.randn(T, H, D, dtype=torch.float16, device=device)
    vd = torch.randn(T, H, D, dtype=torch.float16, device=device)
    leg("triton_dense_f16", None, lambda: fd.token_decode_attention_flash_decoding(case.q, st, H, D, kd, vd),
        tok_heads * 4 * D)
    return out
