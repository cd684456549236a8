#!/usr/bin/env python
"""Benchmark of the latent decode-attention op on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" = one pass of the op (split-KV stage 1 + merge, U_v applied) over the whole
batch of one decoder layer.  Rank 0 prints ONE JSON line.

* N = 1: workload c2 (LLaVA-1.5-13B shape: B16, 40 heads, head_dim 128, rank 64/64,
  context 8192), inputs resident in HBM and larger than L2.
* N > 1 (launched under torchrun, one rank per GPU): the workload's own heads are divided
  over the ranks (strong scaling: 40 -> 20/10/5 heads per GPU) and the step ends with the
  path's one exchange, the all-gather of the [B, H_local, 128] outputs, fused into the
  merge kernel as peer stores (--collective nccl: the library all-gather instead).
  --weak gives every rank a full-size shard of its own instead (weak scaling).
* `value` = algorithmic latent+scale bytes of all ranks / max-over-ranks device time.
* `strong`: the two workloads that are head-sharded by definition (c3, c4) measured the
  same way at this N (fewer steps); `triton_reference` (N = 1): the reference's own Triton
  kernels on this GPU when baseline/_ref is present.
* `e2e` = the same step through the public Python op with the per-step inputs (q and
  the batch metadata) copied from pinned host memory and the result copied back to the
  host inside the timed region; the latent KV cache is resident device state, as in the
  reference (its caches are CUDA tensors, efficiency/layer_utils.py:57-58).
* `roofline` is for the dominant kernel (stage 1), timed alone with CUDA events.
* `cpu_baseline` / `--impl reference`: the reference's own CPU-runnable torch path
  (restated in oracle/) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "latent decode-attn µs/layer & achieved HBM GB/s (1/2/4/8 B200), 7B/13B shapes"
DEFAULT_WORKLOAD = "c2_13b_b16_s8192"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one stage-1 launch from an ncu capture, keyed by
# workload: (bytes, sha256[:12] of the stage-1 kernel source the capture was taken with).  The
# number is reported only while the kernel source is unchanged; otherwise `traffic` is null.
NCU_TRAFFIC = {
    "c2_13b_b16_s8192": (706537728, "c35da991c13a"),
    "c4_13b_b64_ragged32k": (5306711048, "c35da991c13a"),
}
STAGE1_SOURCE = os.path.join(ROOT, "wsvd_b200", "csrc", "latent_decode_tc_sm100.cu")


def stage1_source_tag():
    """sha256[:12] of the stage-1 kernel's code: `//` comments and blank lines do not count, so that
    editing a comment does not orphan an ncu capture."""
    import hashlib
    import re

    try:
        with open(STAGE1_SOURCE, "r") as f:
            lines = [re.sub(r"\s*//.*$", "", ln.rstrip()) for ln in f]
    except OSError:
        return None
    code = "\n".join(ln for ln in lines if ln.strip())
    return hashlib.sha256(code.encode()).hexdigest()[:12]


def ncu_traffic(workload):
    hit = NCU_TRAFFIC.get(workload)
    if hit is None or hit[1] != stage1_source_tag():
        return None
    return hit[0]


C5_WORKLOAD = "c5_7b_b64_s4096_step"


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_reference_run(spec, steps, warmup, sample_batch=2):
    """The reference's CPU-runnable path (oracle restatement of
    efficiency/test_functional_layer.py:146-163 with the kernel's RoPE) on all host
    threads, on `sample_batch` sequences of the workload per step."""
    from oracle import latent_decode_oracle as orc
    from wsvd_b200 import inputs

    torch.set_num_threads(os.cpu_count() or 1)
    lens = inputs.seq_lens_for(spec)[:sample_batch]
    case = inputs.make_case(len(lens), spec.heads, spec.head_dim, spec.rank_k, spec.rank_v, lens, spec.max_len,
                            spec.seed, device="cpu", poison=False)
    nbytes = inputs.algorithmic_bytes(lens, spec.heads, spec.rank_k, spec.rank_v)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        orc.latent_decode_oracle(*case.oracle_args(), wv=case.wv)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    t = sum(times) / len(times)
    return {
        "value": nbytes / t / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
        "sample": f"{len(lens)} of {spec.batch} sequences of {spec.name} per step "
                  f"({nbytes / 1e6:.1f} MB of latents+scales), torch {torch.__version__} fp32",
        "ms_per_step_sample": t * 1e3,
        "us_per_layer_extrapolated": t * 1e6 * (spec.batch / len(lens)),
    }


def workload_config(spec, heads_per_gpu, world):
    """What identifies the workload; both arms print exactly this dict."""
    from wsvd_b200 import inputs

    nbytes = inputs.algorithmic_bytes(inputs.seq_lens_for(spec), heads_per_gpu, spec.rank_k, spec.rank_v)
    return {"workload": spec.name, "batch": spec.batch, "heads": spec.heads, "heads_per_gpu": heads_per_gpu,
            "head_dim": spec.head_dim, "rank_k": spec.rank_k, "rank_v": spec.rank_v, "context": spec.max_len,
            "parallelism": f"heads x{world}",
            "l2": (f"{nbytes / 1e6:.0f} MB of latents+scales per GPU per step, larger than the 126 MB L2"
                   if nbytes >= (300 << 20) else
                   f"{nbytes / 1e6:.0f} MB of latents+scales per GPU per step would fit the 126 MB L2: a 512 MB "
                   "buffer is written before every timed call")}


def run_reference(args, spec):
    """The reference arm: the reference's CPU-runnable path on the host cores, `--steps` timed
    steps after `--warmup` untimed ones, each step a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb = cpu_reference_run(spec, args.steps, max(args.warmup, 1), sample_batch=1)
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_step_sample"], "higher_is_better": True,
        "scaling": "weak" if args.weak else "strong", "vs_baseline": None,
        "dtype": "i8 latents, f32 math", "data": "synthetic",
        "config": workload_config(spec, spec.heads // args.gpus if not args.weak else spec.heads, args.gpus),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "us_per_layer_extrapolated": cb["us_per_layer_extrapolated"],
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_c5(args):
    """The 32-layer decode step (Llama-2-7B architecture, per-head low-rank K/V, batch 64,
    context 4096): down-projection, int8 quantise-and-append, latent decode attention,
    o-projection, FFN, for every layer; tensor-parallel by heads at N > 1.  tokens/s."""
    from wsvd_b200 import ops
    from wsvd_b200.backbone import BackboneSpec, LatentDecoder

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the op has no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 under torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist, pg, collective = None, None, "none"
    spec = BackboneSpec()
    B, context = 64, 4096
    args.warmup = max(args.warmup, 3)
    steps = min(args.steps, 20)
    n_e2e = min(steps, 10)
    capacity = context + args.warmup + steps + n_e2e + 3 + 8 + 2
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        collective = "nccl all_gather of [B,H_local,128] f16 per layer; nccl all_reduce of the FFN output"
        if args.o_proj == "row":
            collective = ("row-parallel o-projection: nccl all_reduce of [B,hidden] f16 per layer instead of a head "
                          "gather; nccl all_reduce of the FFN output")
        elif args.collective == "fused":
            from wsvd_b200.dist import PeerGather
            ok = torch.ones(1, device=dev)
            try:
                pg = PeerGather(B, spec.heads, spec.head_dim, device=dev, timeout_ms=10000,
                                device_epoch=not args.no_graph)
            except Exception as exc:
                print(f"[bench] rank {rank}: peer buffers unavailable ({exc}); using NCCL", file=sys.stderr)
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0:
                pg = None
            else:
                collective = ("head all-gather fused into the decode kernel (peer stores + flag barrier) per layer; "
                              "nccl all_reduce of the FFN output")
    model = LatentDecoder(spec, B, context, capacity, rank=rank, world=world, device=dev, seed=5, peer_gather=pg,
                          o_proj=args.o_proj, fused_elementwise=not args.torch_elementwise)
    x = (torch.randn(B, spec.hidden, device=dev, dtype=torch.float32) * 0.5).to(torch.float16)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    graph = None
    # (with the NCCL head gather the step is launched from Python: a run that captured it in a graph
    # did not finish and was not repeated)
    if not args.no_graph and (world == 1 or pg is not None or args.o_proj == "row"):
        graph, y_graph = model.capture(x)  # one CUDA graph replayed per step (advances the context by one)

    def step():
        if graph is not None:
            graph.replay()
            model.context += 1  # the graph advanced the device-side lengths
            return
        model.step(x)
        model.advance()

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = ms.item()

    x_host = x.cpu().pin_memory()
    y_host = torch.empty(B, spec.hidden, dtype=torch.float16).pin_memory()
    x_dev = torch.empty_like(x)

    def e2e_step():
        if graph is not None:
            x.copy_(x_host, non_blocking=True)  # the graph reads its input from x
            graph.replay()
            model.context += 1
            y_host.copy_(y_graph, non_blocking=True)
        else:
            x_dev.copy_(x_host, non_blocking=True)
            y = model.step(x_dev)
            model.advance()
            y_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    barrier()
    ms2 = torch.tensor([e0.elapsed_time(e1) / n_e2e], device=dev)
    if world > 1:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    ms_e2e = ms2.item()
    clocks = sampler.stop() if rank == 0 else None
    status = torch.tensor([ops.kernel_status()], device=dev)
    if world > 1:
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
    if rank == 0:
        peak, peak_kind = measured_peaks()
        step_bytes = model.attention_bytes() + model.weight_bytes()
        achieved = step_bytes / (ms_step * 1e-3) / 1e9
        print(json.dumps({
            "metric": "decode tokens/s, 32-layer Llama-2-7B-architecture step with per-head low-rank int8 K/V",
            "value": B / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 GEMMs (cuBLAS), i8 latents, f32 accumulate/softmax",
            "data": "synthetic",
            "config": {"workload": C5_WORKLOAD, "batch": B, "context": context, "layers": spec.layers,
                       "hidden": spec.hidden, "heads": spec.heads, "heads_per_gpu": spec.heads // world,
                       "ffn": spec.ffn, "rank_k": spec.rank_k, "rank_v": spec.rank_v,
                       "parallelism": f"heads x{world}", "collective": collective,
                       "o_proj": model.o_proj,
                       "elementwise": "torch chains" if args.torch_elementwise else "one kernel each",
                       "launch": "one CUDA graph per step" if graph is not None else "eager, from Python",
                       "l2": "caches and weights of one step (GBs per GPU) are larger than the 126 MB L2"},
            "roofline": {"bound": "hbm", "kernel": "whole step: latent+scale bytes of 32 layers + the rank's weights",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_step": step_bytes,
                         "attention_bytes_per_step": model.attention_bytes(), "traffic": None},
            "e2e": {"value": B / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
            # this package's kernels per layer: quantise-and-append, decode (+ residual-add+RMSNorm x2,
            # RoPE, SiLU*up), and the first layer's RMSNorm once per step
            "gpu_launches": steps * (spec.layers * 2 if args.torch_elementwise else spec.layers * 6 + 1),
            "kernel_status": int(status.item()), "clocks": clocks,
        }), flush=True)
    if world > 1:
        # The step's graph holds the captured NCCL all-reduces and the addresses of the peer buffers:
        # it has to go before the buffers are unmapped and the communicator is destroyed (tearing
        # those down under a live graph is what did not return on 8 ranks).
        if graph is not None:
            graph.reset()
            graph = None
        torch.cuda.synchronize()
        dist.barrier()
        if pg is not None:
            pg.close()
        dist.destroy_process_group()


class Measurement:
    """One workload on this rank's head shard: the step, stage 1 alone, the end-to-end call."""

    def __init__(self, args, spec, world, rank, dev, dist):
        import ctypes

        from wsvd_b200 import _lib, inputs, ops

        self.args, self.spec, self.world, self.rank, self.dev, self.dist = args, spec, world, rank, dev, dist
        self.ct, self._lib, self.ops, self.inputs = ctypes, _lib, ops, inputs
        self.strong = world > 1 and not args.weak
        if self.strong:
            if spec.heads % world:
                raise SystemExit(f"{spec.heads} heads do not divide over {world} ranks")
            per = spec.heads // world
            self.case = inputs.make_workload(spec, device=dev, heads=slice(rank * per, (rank + 1) * per))
        elif world > 1:
            shard_spec = inputs.WorkloadSpec(**{**spec.__dict__, "seed": spec.seed + 7919 * rank})
            self.case = inputs.make_workload(shard_spec, device=dev)
        else:
            self.case = inputs.make_workload(spec, device=dev)
        case = self.case
        st = case.infer_state
        self.B, self.H, self.D = case.q.shape
        self.lens = case.seq_lens
        self.bytes_rank = inputs.algorithmic_bytes(self.lens, self.H, spec.rank_k, spec.rank_v)
        self.bytes_total = self.bytes_rank * world
        self.out = torch.empty(self.B, self.H, self.D, dtype=torch.float16, device=dev)
        self.gathered = (torch.empty(world, self.B, self.H, self.D, dtype=torch.float16, device=dev)
                         if world > 1 else None)
        self.p, self._keep = ops.build_params(case.q, st.b_seq_len, st.b_req_idx, st.req_manager.req_to_token_indexs,
                                              st.max_len_in_batch, case.latent_k, case.k_scale, case.latent_v,
                                              case.v_scale, case.wk, None, wv=case.wv, out=self.out,
                                              split_len=args.split_len, kernel=args.kernel)
        self.split_len, self.n_splits = ops.plan(self.p)
        # c1..c4 are shapes the tensor-core kernel accepts: without a split length from the caller the
        # library then deals the batch's tiles out in equal shares, one persistent CTA per SM
        self.balanced = args.split_len == 0 and args.kernel in ("auto", "tc")
        self.distribution = ("equal shares of 128-position tiles, one persistent CTA per SM" if self.balanced
                             else "fixed-length splits, one CTA per (split, 4 heads, sequence)")
        self.ws = torch.empty((ops.workspace_bytes(self.p) + 3) // 4, dtype=torch.float32, device=dev)
        self.stream = torch.cuda.current_stream()
        self.lib = _lib.lib()
        # N>1: the path's one exchange, the all-gather of the heads.  "fused": the merge kernel of
        # every rank stores its rows into all ranks' gathered buffers and runs the group barrier
        # (wsvd_latent_decode_gather); "nccl": the plain library collective after the op.
        self.pg, self.collective = None, "none"
        if world > 1:
            self.collective = "nccl all_gather of [B,H_local,128] f16"
            if args.collective == "fused":
                from wsvd_b200.dist import PeerGather
                ok = torch.ones(1, device=dev)
                try:
                    self.pg = PeerGather(self.B, self.H * world, self.D, device=dev, timeout_ms=10000)
                except Exception as exc:  # no peer mapping on this box: say so and use the library collective
                    print(f"[bench] rank {rank}: peer buffers unavailable ({exc}); using NCCL", file=sys.stderr)
                    ok.zero_()
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                if ok.item() == 0:
                    self.pg = None
                else:
                    self.collective = ("fused into the decode kernel: the CTA that completes a head stores its row into every "
                                       "rank's gathered buffer (16-byte peer stores); the last CTA runs the flag barrier")
        # inputs smaller than ~2x the 126 MB L2 would be served from cache on repeated calls:
        # then every timed call is preceded by a write of a 512 MB buffer and timed on its own
        self.flush = (torch.empty(512 << 20, dtype=torch.uint8, device=dev)
                      if self.bytes_rank < (300 << 20) else None)

    # ---- the step
    def step(self):
        ct = self.ct
        if self.pg is not None:
            ps, _parity = self.pg.peer_set()
            self._lib.check(self.lib.wsvd_latent_decode_gather(
                ct.byref(self.p), ct.byref(ps), ct.c_void_p(self.ws.data_ptr()), self.ws.numel() * 4,
                ct.c_void_p(self.stream.cuda_stream)), "wsvd_latent_decode_gather")
            return
        self._lib.check(self.lib.wsvd_latent_decode(ct.byref(self.p), ct.c_void_p(self.ws.data_ptr()),
                                                    self.ws.numel() * 4, ct.c_void_p(self.stream.cuda_stream)),
                        "wsvd_latent_decode")
        if self.world > 1:
            self.dist.all_gather_into_tensor(self.gathered, self.out)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, k):
        """k calls bracketed by barrier+synchronize; device time by CUDA events, max over ranks."""
        self.barrier()
        if self.flush is None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(k):
                fn()
            e1.record()
            self.barrier()
            total = e0.elapsed_time(e1)
        else:
            evs = []
            for _ in range(k):
                self.flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                evs.append((e0, e1))
            self.barrier()
            total = sum(a.elapsed_time(b) for a, b in evs)
        ms = torch.tensor([total], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return ms.item()

    def time_step(self, steps, warmup):
        for _ in range(warmup):
            self.step()
        return self.timed(self.step, steps) / steps

    def time_graph(self, steps):
        """The same step replayed from a CUDA graph (one GPU): what a serving loop that captures
        its decode step pays; matters for the small workloads, which are bound by launch latency."""
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        keep = self.stream
        with torch.cuda.graph(g):
            self.stream = torch.cuda.current_stream()  # step() launches on the capturing stream
            self.step()
        self.stream = keep
        for _ in range(3):
            g.replay()
        return self.timed(g.replay, steps) / steps

    def time_stage1(self, steps):
        """The dominant kernel alone, for the roofline: the op without its merge kernel, with the
        same work distribution as the whole op (the launch of the small kernel that cuts the
        work into per-SM shares, where the op uses one, is inside the timed region)."""
        ct = self.ct

        def stage1():
            self._lib.check(self.lib.wsvd_latent_decode_partials(
                ct.byref(self.p), ct.c_void_p(self.ws.data_ptr()), self.ws.numel() * 4,
                ct.c_void_p(self.stream.cuda_stream)), "wsvd_latent_decode_partials")

        for _ in range(3):
            stage1()
        return self.timed(stage1, steps) / steps

    def gather_check(self):
        """Once, outside the timed region: the buffer the fused gather filled on this rank against
        an NCCL all-gather of every rank's local output.  True when they are identical on all ranks."""
        if self.world == 1 or self.pg is None:
            return None
        ct = self.ct
        ps, parity = self.pg.peer_set()
        self._lib.check(self.lib.wsvd_latent_decode_gather(
            ct.byref(self.p), ct.byref(ps), ct.c_void_p(self.ws.data_ptr()), self.ws.numel() * 4,
            ct.c_void_p(self.stream.cuda_stream)), "wsvd_latent_decode_gather")
        fused = self.pg.buffer(parity).clone()
        self._lib.check(self.lib.wsvd_latent_decode(ct.byref(self.p), ct.c_void_p(self.ws.data_ptr()),
                                                    self.ws.numel() * 4, ct.c_void_p(self.stream.cuda_stream)),
                        "wsvd_latent_decode")
        self.dist.all_gather_into_tensor(self.gathered, self.out)
        want = self.gathered.permute(1, 0, 2, 3).reshape(self.B, self.world * self.H, self.D)
        same = torch.tensor([1.0 if torch.equal(fused, want) else 0.0], device=self.dev)
        self.dist.all_reduce(same, op=self.dist.ReduceOp.MIN)
        return bool(same.item() == 1.0)

    def time_e2e(self, steps, op):
        """End to end through the public op: host buffers in, host result out, every step."""
        case, st, dev = self.case, self.case.infer_state, self.dev
        B, H, D, world, pg, args = self.B, self.H, self.D, self.world, self.pg, self.args
        # the step's inputs (q, lengths, request indices) travel as one pinned buffer and one copy, as a
        # serving loop would stage them; the device tensors are views of the device-side buffer
        nq, nl = case.q.numel() * 2, st.b_seq_len.numel() * 4
        in_host = torch.empty(nq + 2 * nl, dtype=torch.uint8).pin_memory()
        in_host[:nq].view(torch.float16).copy_(case.q.reshape(-1).cpu())
        in_host[nq:nq + nl].view(torch.int32).copy_(st.b_seq_len.cpu())
        in_host[nq + nl:].view(torch.int32).copy_(st.b_req_idx.cpu())
        in_dev = torch.empty(nq + 2 * nl, dtype=torch.uint8, device=dev)
        q_dev = in_dev[:nq].view(torch.float16).view(case.q.shape)
        len_dev, req_dev = in_dev[nq:nq + nl].view(torch.int32), in_dev[nq + nl:].view(torch.int32)
        # (with the fused gather the step's result is the gathered [B, H_total, D] buffer)
        out_host = torch.empty(B, H * (world if pg is not None else 1), D, dtype=torch.float16).pin_memory()
        from wsvd_b200.infer_state import InferState
        st2 = InferState(B, st.max_len_in_batch, self.lens, device=dev, req_to_token=st.req_manager.req_to_token_indexs)
        st2.b_seq_len, st2.b_req_idx = len_dev, req_dev

        def e2e_step():
            in_dev.copy_(in_host, non_blocking=True)
            if pg is not None:
                o = pg.decode(q_dev, st2, case.latent_k, case.k_scale, case.latent_v, case.v_scale, case.wk, None,
                              wv=case.wv, workspace=self.ws, split_len=args.split_len, kernel=args.kernel)
            else:
                o = op(q_dev, st2, H, D, case.latent_k, case.k_scale, case.latent_v, case.v_scale, case.wk, None,
                       wv=case.wv, out=self.out, workspace=self.ws, split_len=args.split_len, kernel=args.kernel)
                if world > 1:
                    self.dist.all_gather_into_tensor(self.gathered, o)
            out_host.copy_(o, non_blocking=True)
            torch.cuda.current_stream().synchronize()  # the caller consumes the host result every step

        for _ in range(3):
            e2e_step()
        ms = self.timed(e2e_step, steps) / steps
        return ms, in_host.numel(), out_host.numel() * 2

    def close(self):
        if self.pg is not None:
            self.pg.close()
            self.pg = None
        self.case = self.ws = self.flush = self.out = self.gathered = self._keep = None
        torch.cuda.empty_cache()


def main():
    # NCCL writes its version banner to stdout at NCCL_DEBUG=VERSION; stdout is for the one JSON line
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel", default="auto", choices=["auto", "generic", "tc", "mma"])
    ap.add_argument("--split-len", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--weak", action="store_true",
                    help="N>1: give every rank a full-size shard of its own (weak scaling) instead of dividing the "
                         "workload's heads over the ranks (strong scaling, the default)")
    ap.add_argument("--shard-heads", action="store_true", help="accepted for compatibility: strong scaling is the default")
    ap.add_argument("--no-graph", action="store_true", help="c5 step: launch from Python instead of one CUDA graph")
    ap.add_argument("--collective", default="fused", choices=["fused", "nccl"],
                    help="N>1: head all-gather fused into the decode kernel (peer stores), or an NCCL all_gather")
    ap.add_argument("--o-proj", default="gather", choices=["gather", "row"],
                    help="c5, N>1: heads gathered and a replicated Wo, or row-parallel Wo with an all-reduce")
    ap.add_argument("--torch-elementwise", action="store_true",
                    help="c5: RMSNorm / RoPE / SiLU*up as chains of torch ops instead of one kernel each")
    ap.add_argument("--no-dense", action="store_true", help="skip the dense f16 baseline kernel timing")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the `strong` list (c3, c4 at this N) and the reference Triton kernels")
    ap.add_argument("--triton-reference", action="store_true",
                    help="only time the reference's Triton kernels (baseline/_ref) on this GPU and print their line")
    args = ap.parse_args()

    from wsvd_b200 import inputs

    if args.workload == C5_WORKLOAD and args.impl == "ours":
        run_c5(args)
        return
    spec = inputs.WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, spec)
        return

    from wsvd_b200 import ops
    from wsvd_b200.kernel.flash_decoding import token_decode_attention_flash_int8_latent_per_head_decoding_rope as op

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the op has no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 under torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if args.triton_reference:
        print(json.dumps({"impl": "reference-triton", "n_gpus": 1, **triton_reference_leg(spec, dev, op, args)}),
              flush=True)
        return
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    args.warmup = max(args.warmup, 3)
    peak, peak_kind = measured_peaks()

    m = Measurement(args, spec, world, rank, dev, dist)
    for _ in range(args.warmup):
        m.step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step = m.timed(m.step, args.steps) / args.steps
    ms_graph = m.time_graph(args.steps) if world == 1 else None
    ms_stage1 = m.time_stage1(args.steps)
    ms_e2e, h2d, d2h = m.time_e2e(args.steps, op)
    clocks = sampler.stop() if rank == 0 else None
    gather_ok = m.gather_check()
    status = torch.tensor([ops.kernel_status()], device=dev)
    if world > 1:
        dist.all_reduce(status, op=dist.ReduceOp.MAX)

    line = None
    if rank == 0:
        achieved = m.bytes_rank / (ms_stage1 * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": m.bytes_total / (ms_step * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "us_per_layer": ms_step * 1e3,
            "us_per_layer_cuda_graph": None if ms_graph is None else ms_graph * 1e3,
            "higher_is_better": True, "scaling": "strong" if m.strong or world == 1 else "weak",
            "vs_baseline": None,
            "dtype": "i8 latents, f16 tensor-core operands, f32 accumulate/softmax", "data": "synthetic",
            "config": workload_config(spec, m.H, world),
            "plan": {"distribution": m.distribution, "split_len": m.split_len if not m.balanced else None,
                     "n_splits": m.n_splits if not m.balanced else None, "kernel": args.kernel,
                     "collective": m.collective},
            "roofline": {
                "bound": "hbm", "kernel": "latent decode stage 1", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                "us_per_launch": ms_stage1 * 1e3, "algorithmic_bytes_per_launch": m.bytes_rank,
                "traffic": ncu_traffic(spec.name),
            },
            # what the merge (and, at N>1, the fused exchange with its group barrier) adds to stage 1
            "us_merge_gather": (ms_step - ms_stage1) * 1e3,
            "gather_check": gather_ok,
            "e2e": {"value": m.bytes_total / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "us_per_layer": ms_e2e * 1e3,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            # per step: one kernel when the library balances the tiles itself (stage 1 merges, projects and,
            # at N > 1, stores the rows to the peers in its last-arriving CTAs), else stage 1 + the merge
            # kernel (+ the NCCL all-gather, which is not counted)
            "gpu_launches": args.steps * (1 if m.balanced and (world == 1 or m.pg is not None) else 2),
            "kernel_status": int(status.item()),
            "clocks": clocks,
        }
        if world == 1 and not args.no_dense:
            line["dense_f16_baseline"] = dense_baseline(m, spec, ms_step, max(5, args.steps // 2))
        if world == 1 and not args.no_extra:
            line["f16_latents"] = f16_latents_leg(m, spec, peak, max(5, args.steps // 2))
    m.close()

    # ---- the head-sharded workloads (c3, c4) at this N, fewer steps ----
    if not args.no_extra and spec.name == DEFAULT_WORKLOAD:
        strong = []
        for name in ("c3_next7b_b32_ragged4096", "c4_13b_b64_ragged32k"):
            xs = inputs.WORKLOADS[name]
            if xs.heads % world:
                continue
            k = max(5, min(20, args.steps // 2))
            mx = Measurement(args, xs, world, rank, dev, dist)
            ms_x = mx.time_step(k, 3)
            ms_x1 = mx.time_stage1(k)
            ok_x = mx.gather_check()
            if rank == 0:
                strong.append({
                    "workload": name, "heads_per_gpu": mx.H, "distribution": mx.distribution,
                    "steps": k, "us_per_layer": ms_x * 1e3, "GB/s": mx.bytes_total / (ms_x * 1e-3) / 1e9,
                    "us_stage1": ms_x1 * 1e3, "stage1_frac_per_gpu": mx.bytes_rank / (ms_x1 * 1e-3) / 1e9 / peak,
                    "gather_check": ok_x})
            mx.close()
        if rank == 0:
            line["strong"] = strong
    if rank == 0 and world == 1 and not args.no_extra:
        line["triton_reference"] = triton_reference_leg(spec, dev, op, args)
        ref_dense = line["triton_reference"].get("triton_dense_f16")
        if ref_dense:
            line["triton_reference"]["latent_speedup_vs_reference_dense"] = ref_dense["us_per_layer"] / (ms_step * 1e3)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cb = cpu_reference_run(spec, steps=3, warmup=1)
        line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        line["cpu_baseline"]["us_per_layer_extrapolated"] = cb["us_per_layer_extrapolated"]
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def dense_baseline(m, spec, ms_step, k):
    """This library's dense f16 flash-decoding kernel on the same shape (K/V [T,H,128] f16, 512 B
    per token-head)."""
    from wsvd_b200.infer_state import InferState
    from wsvd_b200.kernel.flash_decoding import token_decode_attention_flash_decoding as dense_op

    B, H, D, dev, S = m.B, m.H, m.D, m.dev, spec.max_len
    st = m.case.infer_state
    kd = torch.randn(B, H, S, D, dtype=torch.float16, device=dev)
    vd = torch.randn(B, H, S, D, dtype=torch.float16, device=dev)
    kv = kd.as_strided(((B - 1) * H * S + S, H, D), (D, S * D, 1))
    vv = vd.as_strided(((B - 1) * H * S + S, H, D), (D, S * D, 1))
    dst = InferState(B, S, m.lens, device=dev, req_to_token=st.req_manager.req_to_token_indexs)
    dout = torch.empty(B, H, D, dtype=torch.float16, device=dev)
    dws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    dense = lambda: dense_op(m.case.q, dst, H, D, kv, vv, out=dout, workspace=dws)
    for _ in range(3):
        dense()
    ms_dense = m.timed(dense, k) / k
    dense_bytes = sum(m.lens) * H * 4 * D
    return {"us_per_layer": ms_dense * 1e3, "GB/s": dense_bytes / (ms_dense * 1e-3) / 1e9,
            "bytes_per_token_head": 4 * D, "latent_speedup": ms_dense / ms_step,
            "byte_reduction": 4 * D / (spec.rank_k + spec.rank_v + 4)}


def f16_latents_leg(m, spec, peak, k):
    """The same shape with an f16 latent cache (the reference's f16 op, 2*(rank_k+rank_v) bytes per
    token-head, no scales): the warp-MMA kernel with fixed-length splits, then the merge kernel."""
    import ctypes as ct

    from wsvd_b200 import _lib, inputs, ops

    case = inputs.make_case(m.B, m.H, m.D, spec.rank_k, spec.rank_v, m.lens, spec.max_len, spec.seed + 1,
                            device=m.dev, latent_dtype=torch.float16)
    st = case.infer_state
    out = torch.empty(m.B, m.H, m.D, dtype=torch.float16, device=m.dev)
    p, _keep = ops.build_params(case.q, st.b_seq_len, st.b_req_idx, st.req_manager.req_to_token_indexs,
                                st.max_len_in_batch, case.latent_k, None, case.latent_v, None, case.wk, None,
                                wv=case.wv, out=out)
    split_len, n_splits = ops.plan(p)
    ws = torch.empty((ops.workspace_bytes(p) + 3) // 4, dtype=torch.float32, device=m.dev)
    lib, stream = _lib.lib(), torch.cuda.current_stream()

    def call(fn, name):
        _lib.check(fn(ct.byref(p), ct.c_void_p(ws.data_ptr()), ws.numel() * 4, ct.c_void_p(stream.cuda_stream)), name)

    full = lambda: call(lib.wsvd_latent_decode, "wsvd_latent_decode")
    stage1 = lambda: call(lib.wsvd_latent_decode_partials, "wsvd_latent_decode_partials")
    for _ in range(3):
        full()
        stage1()
    ms_full = m.timed(full, k) / k
    ms_s1 = m.timed(stage1, k) / k
    # the CUDA-core kernel on the same cache, for scale
    p.kernel = ops.KERNEL["generic"]
    ws_g = torch.empty((ops.workspace_bytes(p) + 3) // 4, dtype=torch.float32, device=m.dev)
    generic = lambda: _lib.check(lib.wsvd_latent_decode(ct.byref(p), ct.c_void_p(ws_g.data_ptr()), ws_g.numel() * 4,
                                                        ct.c_void_p(stream.cuda_stream)), "wsvd_latent_decode")
    generic()
    ms_generic = m.timed(generic, 3) / 3
    nbytes = sum(m.lens) * m.H * 2 * (spec.rank_k + spec.rank_v)
    return {"kernel": "warp-MMA (mma.sync m16n8k16), fixed-length splits", "split_len": split_len, "n_splits": n_splits,
            "bytes_per_token_head": 2 * (spec.rank_k + spec.rank_v), "us_per_layer": ms_full * 1e3,
            "us_stage1": ms_s1 * 1e3, "GB/s": nbytes / (ms_full * 1e-3) / 1e9,
            "stage1_frac": nbytes / (ms_s1 * 1e-3) / 1e9 / peak, "us_per_layer_generic_kernel": ms_generic * 1e3}


def triton_reference_leg(spec, dev, op, args):
    """The reference's Triton kernels on this GPU (baseline/_ref), or why they cannot run."""
    try:
        from baseline import triton_reference as tr
    except Exception as exc:
        return {"unavailable": f"baseline/triton_reference.py cannot be imported: {exc}"}

    def ours(case):
        s = case.infer_state
        return op(case.q, s, case.q.shape[1], case.q.shape[2], case.latent_k, case.k_scale, case.latent_v,
                  case.v_scale, case.wk, None, kernel=args.kernel)

    try:
        return tr.run(spec, dev, steps=max(5, min(20, args.steps)), warmup=3, ours=ours)
    except Exception as exc:  # the reference's code failed here: report it, keep this library's line
        return {"unavailable": f"the reference kernels raised {type(exc).__name__}: {exc}"[:300]}


if __name__ == "__main__":
    main()
