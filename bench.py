#!/usr/bin/env python
"""Benchmark of the latent decode-attention op on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" = one pass of the op (split-KV stage 1 + merge, U_v applied) over the whole
batch of one decoder layer.  Rank 0 prints ONE JSON line.

* N = 1: workload c2 (LLaVA-1.5-13B shape: B16, 40 heads, head_dim 128, rank 64/64,
  context 8192), inputs resident in HBM and larger than L2.
* N > 1 (launched under torchrun, one rank per GPU): every rank owns a head shard of
  that same shape (weak scaling: 40 local heads per GPU) and the step ends with the
  path's one exchange, the all-gather of the [B, H_local, 128] outputs, fused into the
  merge kernel as peer stores (--collective nccl: the library all-gather instead).
  --shard-heads divides the named workload's own heads over the ranks instead (strong scaling).
* `value` = algorithmic latent+scale bytes of all ranks / max-over-ranks device time.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one stage-1 launch, from the ncu capture
# summarised in profiles/latent_decode_stage1_tc_c2.md
NCU_TRAFFIC_BYTES = {"c2_13b_b16_s8192": 711555328}
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


def run_reference(args, spec):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 10))
    warm = max(1, min(args.warmup, 2))
    cb = cpu_reference_run(spec, steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": cb["ms_per_step_sample"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "i8 latents, f32 math", "data": "synthetic",
        "config": {"workload": spec.name, "batch": spec.batch, "heads": spec.heads, "head_dim": spec.head_dim,
                   "rank_k": spec.rank_k, "rank_v": spec.rank_v, "context": spec.max_len,
                   "l2": "CPU run; sample larger than the host caches"},
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
        if args.collective == "fused":
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
                collective = ("head all-gather fused into the merge kernel (peer stores + flag barrier) per layer; "
                              "nccl all_reduce of the FFN output")
    model = LatentDecoder(spec, B, context, capacity, rank=rank, world=world, device=dev, seed=5, peer_gather=pg)
    x = (torch.randn(B, spec.hidden, device=dev, dtype=torch.float32) * 0.5).to(torch.float16)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    graph = None
    # (with the NCCL head gather the step is launched from Python: a run that captured it in a graph
    # did not finish and was not repeated)
    if not args.no_graph and (world == 1 or pg is not None):
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
                       "launch": "one CUDA graph per step" if graph is not None else "eager, from Python",
                       "l2": "caches and weights of one step (GBs per GPU) are larger than the 126 MB L2"},
            "roofline": {"bound": "hbm", "kernel": "whole step: latent+scale bytes of 32 layers + the rank's weights",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_step": step_bytes,
                         "attention_bytes_per_step": model.attention_bytes(), "traffic": None},
            "e2e": {"value": B / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
            "gpu_launches": steps * spec.layers * 3,
            "kernel_status": int(status.item()), "clocks": clocks,
        }), flush=True)
    if world > 1:
        if graph is not None:
            # Every rank has passed the all-reduce of the status word after its last kernel.  With the
            # NCCL all-reduce captured in the step's graph, tearing the peer buffers and the process
            # group down did not return on 8 ranks; leave it to process exit.
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)
        if pg is not None:
            pg.close()
        dist.barrier()
        dist.destroy_process_group()


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
    ap.add_argument("--kernel", default="auto", choices=["auto", "generic", "tc"])
    ap.add_argument("--split-len", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shard-heads", action="store_true",
                    help="N>1: divide the workload's heads over the ranks (strong scaling) instead of giving "
                         "every rank a full-size shard (weak scaling, the default)")
    ap.add_argument("--no-graph", action="store_true", help="c5 step: launch from Python instead of one CUDA graph")
    ap.add_argument("--collective", default="fused", choices=["fused", "nccl"],
                    help="N>1: head all-gather fused into the merge kernel (peer stores), or an NCCL all_gather")
    ap.add_argument("--no-dense", action="store_true", help="skip the dense f16 baseline kernel timing")
    args = ap.parse_args()

    from wsvd_b200 import inputs

    if args.workload == C5_WORKLOAD and args.impl == "ours":
        run_c5(args)
        return
    spec = inputs.WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, spec)
        return

    import ctypes

    from wsvd_b200 import _lib, ops
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
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    args.warmup = max(args.warmup, 3)

    # ---- workload: this rank's head shard, generated on the device ----
    if args.shard_heads and world > 1:
        # strong scaling: the named workload's heads are divided over the ranks
        if spec.heads % world:
            raise SystemExit(f"{spec.heads} heads do not divide over {world} ranks")
        per = spec.heads // world
        case = inputs.make_workload(spec, device=dev, heads=slice(rank * per, (rank + 1) * per))
    else:
        shard_spec = inputs.WorkloadSpec(**{**spec.__dict__, "seed": spec.seed + 7919 * rank})
        case = inputs.make_workload(shard_spec, device=dev)
    st = case.infer_state
    B, H, D = case.q.shape
    lens = case.seq_lens
    bytes_rank = inputs.algorithmic_bytes(lens, H, spec.rank_k, spec.rank_v)
    bytes_total = bytes_rank * world
    out = torch.empty(B, H, D, dtype=torch.float16, device=dev)
    gathered = torch.empty(world, B, H, D, dtype=torch.float16, device=dev) if world > 1 else None
    p, _keep = ops.build_params(case.q, st.b_seq_len, st.b_req_idx, st.req_manager.req_to_token_indexs,
                                st.max_len_in_batch, case.latent_k, case.k_scale, case.latent_v, case.v_scale,
                                case.wk, None, wv=case.wv, out=out, split_len=args.split_len, kernel=args.kernel)
    split_len, n_splits = ops.plan(p)
    ws = torch.empty((ops.workspace_bytes(p) + 3) // 4, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream()
    lib = _lib.lib()

    # N>1: the path's one exchange, the all-gather of the heads.  "fused": the merge kernel of
    # every rank stores its rows into all ranks' gathered buffers and runs the group barrier
    # (wsvd_latent_decode_gather); "nccl": the plain library collective after the op.
    pg, collective = None, "none"
    if world > 1:
        collective = "nccl all_gather of [B,H_local,128] f16"
        if args.collective == "fused":
            from wsvd_b200.dist import PeerGather
            ok = torch.ones(1, device=dev)
            try:
                pg = PeerGather(B, H * world, D, device=dev, timeout_ms=10000)
            except Exception as exc:  # no peer mapping on this box: say so and use the library collective
                print(f"[bench] rank {rank}: peer buffers unavailable ({exc}); using NCCL", file=sys.stderr)
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0:
                pg = None
            else:
                collective = "fused into the merge kernel: peer stores of [B,H_local,128] f16 + flag barrier"

    def step():
        if pg is not None:
            ps, _parity = pg.peer_set()
            _lib.check(lib.wsvd_latent_decode_gather(ctypes.byref(p), ctypes.byref(ps), ctypes.c_void_p(ws.data_ptr()),
                                                     ws.numel() * 4, ctypes.c_void_p(stream.cuda_stream)),
                       "wsvd_latent_decode_gather")
            return
        _lib.check(lib.wsvd_latent_decode(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), ws.numel() * 4,
                                          ctypes.c_void_p(stream.cuda_stream)), "wsvd_latent_decode")
        if world > 1:
            dist.all_gather_into_tensor(gathered, out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # inputs smaller than ~2x the 126 MB L2 would be served from cache on repeated calls:
    # then every timed call is preceded by a write of a 512 MB buffer and timed on its own
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev) if bytes_rank < (300 << 20) else None

    def timed(fn, k):
        """k calls bracketed by barrier+synchronize; device time by CUDA events, max over ranks."""
        barrier()
        if flush is None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(k):
                fn()
            e1.record()
            barrier()
            total = e0.elapsed_time(e1)
        else:
            evs = []
            for _ in range(k):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                evs.append((e0, e1))
            barrier()
            total = sum(a.elapsed_time(b) for a, b in evs)
        ms = torch.tensor([total], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_total = timed(step, args.steps)
    ms_step = ms_total / args.steps

    # ---- the same step replayed from a CUDA graph (one GPU): what a serving loop that captures its
    #      decode step pays; matters for the small workloads, which are bound by launch latency ----
    ms_graph = None
    if world == 1:
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            stream = torch.cuda.current_stream()  # step() launches on `stream`
            step()
        stream = torch.cuda.current_stream()
        for _ in range(3):
            g.replay()
        ms_graph = timed(g.replay, args.steps) / args.steps

    # ---- dominant kernel alone (stage 1), for the roofline ----
    mid_o = ws[: B * H * n_splits * spec.rank_v]
    lse = ws[B * H * n_splits * spec.rank_v:]
    p1, _k1 = ops.build_params(case.q, st.b_seq_len, st.b_req_idx, st.req_manager.req_to_token_indexs,
                               st.max_len_in_batch, case.latent_k, case.k_scale, case.latent_v, case.v_scale,
                               case.wk, None, split_len=split_len, kernel=args.kernel)

    def stage1():
        _lib.check(lib.wsvd_latent_decode_stage1(ctypes.byref(p1), ctypes.c_void_p(mid_o.data_ptr()),
                                                 ctypes.c_void_p(lse.data_ptr()), n_splits,
                                                 ctypes.c_void_p(stream.cuda_stream)), "stage1")

    for _ in range(3):
        stage1()
    ms_stage1 = timed(stage1, args.steps) / args.steps

    # ---- end to end through the public op, host buffers in, host result out ----
    q_host = case.q.cpu().pin_memory()
    len_host = st.b_seq_len.cpu().pin_memory()
    req_host = st.b_req_idx.cpu().pin_memory()
    # (with the fused gather the step's result is the gathered [B, H_total, D] buffer)
    out_host = torch.empty(B, H * (world if pg is not None else 1), D, dtype=torch.float16).pin_memory()
    q_dev, len_dev, req_dev = torch.empty_like(case.q), torch.empty_like(st.b_seq_len), torch.empty_like(st.b_req_idx)
    from wsvd_b200.infer_state import InferState
    st2 = InferState(B, st.max_len_in_batch, lens, device=dev, req_to_token=st.req_manager.req_to_token_indexs)
    st2.b_seq_len, st2.b_req_idx = len_dev, req_dev

    def e2e_step():
        q_dev.copy_(q_host, non_blocking=True)
        len_dev.copy_(len_host, non_blocking=True)
        req_dev.copy_(req_host, non_blocking=True)
        if pg is not None:
            o = pg.decode(q_dev, st2, case.latent_k, case.k_scale, case.latent_v, case.v_scale, case.wk, None,
                          wv=case.wv, workspace=ws, split_len=args.split_len, kernel=args.kernel)
        else:
            o = op(q_dev, st2, H, D, case.latent_k, case.k_scale, case.latent_v, case.v_scale, case.wk, None,
                   wv=case.wv, out=out, workspace=ws, split_len=args.split_len, kernel=args.kernel)
            if world > 1:
                dist.all_gather_into_tensor(gathered, o)
        out_host.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller consumes the host result every step

    for _ in range(3):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    status = torch.tensor([ops.kernel_status()], device=dev)
    if world > 1:
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
    h2d = q_host.numel() * 2 + len_host.numel() * 4 + req_host.numel() * 4
    d2h = out_host.numel() * 2

    if rank == 0:
        peak, peak_kind = measured_peaks()
        achieved = bytes_rank / (ms_stage1 * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": bytes_total / (ms_step * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "us_per_layer": ms_step * 1e3,
            "us_per_layer_cuda_graph": None if ms_graph is None else ms_graph * 1e3,
            "higher_is_better": True, "scaling": "strong" if args.shard_heads and world > 1 else "weak",
            "vs_baseline": None,
            "dtype": "i8 latents, f16 tensor-core operands, f32 accumulate/softmax", "data": "synthetic",
            "config": {
                "workload": spec.name, "batch": spec.batch, "heads_per_gpu": H, "head_dim": D,
                "rank_k": spec.rank_k, "rank_v": spec.rank_v, "context": spec.max_len, "split_len": split_len,
                "n_splits": n_splits, "kernel": args.kernel, "parallelism": f"heads x{world}",
                "collective": collective,
                "l2": (f"inputs {bytes_rank / 1e6:.0f} MB per GPU, larger than the 126 MB L2" if flush is None else
                       f"inputs {bytes_rank / 1e6:.0f} MB per GPU fit L2: a 512 MB buffer is written before every "
                       "timed call"),
            },
            "roofline": {
                "bound": "hbm", "kernel": "latent decode stage 1", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                "us_per_launch": ms_stage1 * 1e3, "algorithmic_bytes_per_launch": bytes_rank,
                "traffic": NCU_TRAFFIC_BYTES.get(spec.name),
            },
            "e2e": {"value": bytes_total / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "us_per_layer": ms_e2e * 1e3,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": args.steps * 2,
            "kernel_status": int(status.item()),
            "clocks": clocks,
        }
        if world == 1 and not args.no_dense:
            # dense f16 flash-decoding of the same shape (K/V [T,H,128] f16, 512 B per token-head)
            from wsvd_b200.infer_state import InferState as _IS
            from wsvd_b200.kernel.flash_decoding import token_decode_attention_flash_decoding as dense_op
            S = spec.max_len
            kd = torch.randn(B, H, S, D, dtype=torch.float16, device=dev)
            vd = torch.randn(B, H, S, D, dtype=torch.float16, device=dev)
            kv = kd.as_strided(((B - 1) * H * S + S, H, D), (D, S * D, 1))
            vv = vd.as_strided(((B - 1) * H * S + S, H, D), (D, S * D, 1))
            dst = _IS(B, S, lens, device=dev, req_to_token=st.req_manager.req_to_token_indexs)
            dout = torch.empty(B, H, D, dtype=torch.float16, device=dev)
            dws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
            dense = lambda: dense_op(case.q, dst, H, D, kv, vv, out=dout, workspace=dws)
            for _ in range(3):
                dense()
            ms_dense = timed(dense, max(5, args.steps // 2)) / max(5, args.steps // 2)
            dense_bytes = sum(lens) * H * 4 * D
            line["dense_f16_baseline"] = {
                "us_per_layer": ms_dense * 1e3, "GB/s": dense_bytes / (ms_dense * 1e-3) / 1e9,
                "bytes_per_token_head": 4 * D, "latent_speedup": ms_dense / ms_step,
                "byte_reduction": 4 * D / (spec.rank_k + spec.rank_v + 4)}
            del kd, vd
        if world == 1 and not args.no_cpu_baseline:
            cb = cpu_reference_run(spec, steps=3, warmup=1)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
            line["cpu_baseline"]["us_per_layer_extrapolated"] = cb["us_per_layer_extrapolated"]
        print(json.dumps(line), flush=True)
    if world > 1:
        if pg is not None:
            pg.close()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
