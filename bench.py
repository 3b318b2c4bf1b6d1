#!/usr/bin/env python
"""Benchmark of the fused MoE route (router logit GEMM + select + pack) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the headline metric is quoted on): single-GPU
fp16 `fused_select`, T=4096 tokens, d_model=4096, E=64 experts, top_k=2,
hidden ~ N(0,1), router weight ~ N(0,1/d_model), +2.0 skew on the logits of
experts 0..7.  A step is one pass of the route over one batch: one
`moe_route_fused` call = router GEMM/select kernel + scatter kernel.

Prints ONE JSON line (rank 0).  Keys beyond the common contract:
  roofline      dominant kernel (the pack scatter), algorithmic bytes per launch / its average
                duration from CUDA events, against the measured HBM copy peak
  route_roofline the same fraction for the whole step (101,253,636 algorithmic bytes)
  select_pack_roofline the reference's own operator (logits given): select + count + scan + pack
  cpu_baseline  the reference's CPU routing path (torch port in oracle/cpu_route.py) on the
                host cores, a bounded sample of the same workload
  e2e           the same metric through the public API with HOST buffers (pinned), host<->device
                copies of every step inside the timed region, two steps in flight (HostRouter)
Timing: CUDA events on the launching stream around exactly K steps (captured in one CUDA graph),
max over ranks; inputs and outputs rotate over several buffer sets whose total size exceeds the
L2, so every step reads its tokens from HBM.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

T, D, E, K_TOP = 4096, 4096, 64, 2
SKEW_N, SKEW_B = 8, 2.0
ROUTE_BYTES = T * D * 2 + E * D * 2 + K_TOP * T * D * 2 + 2 * T * K_TOP * 4 + E * 4 + (E + 1) * 4  # 101,253,636
PACK_BYTES = T * D * 2 + T * K_TOP * 4 + K_TOP * T * D * 2  # 100,696,064
# dram__bytes_read.sum + dram__bytes_write.sum of one scatter launch at this size, from the ncu capture
# summarised in profiles/pack_scatter_bulk_T4096_d4096_E64_k2.md (the L2 still holds most of the
# 67 MB written when the kernel ends, hence less than the algorithmic bytes)
SCATTER_DRAM_TRAFFIC = 42_600_000
WORKLOAD = "fused_select T=4096 d_model=4096 E=64 top_k=2 fp16, +2.0 skew on experts 0..7"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    return ap.parse_args()


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# --------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------
class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while GPU work runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# --------------------------------------------------------------------------
# CPU arm
# --------------------------------------------------------------------------
def gen_inputs_cpu(seed: int):
    import torch

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, D, generator=g)
    w = torch.randn(E, D, generator=g) / (D ** 0.5)
    return x, w


def run_cpu_reference(steps: int, warmup: int):
    """The reference's CPU routing path (bench_router.py --device cpu --dtype fp32, fused_select ->
    naive_topk fallback) on this host's cores, same T/d/E/k/skew."""
    import torch
    from oracle import cpu_route

    # all host threads this process may use (a multi-rank launcher exports OMP_NUM_THREADS=1, which
    # would make the baseline single-threaded; only one rank runs it, so it takes the whole host)
    try:
        n_cpu = len(os.sched_getaffinity(0))
    except AttributeError:
        n_cpu = os.cpu_count() or 1
    if torch.get_num_threads() < n_cpu:
        torch.set_num_threads(n_cpu)
    x, w = gen_inputs_cpu(0)
    for _ in range(max(1, warmup)):
        cpu_route.one_iter(x, w, K_TOP, skew_experts=SKEW_N, skew_bias=SKEW_B)
    ts = [cpu_route.one_iter(x, w, K_TOP, skew_experts=SKEW_N, skew_bias=SKEW_B) for _ in range(steps)]
    route_ms = sum(t[3] for t in ts) / len(ts)
    return {"value": T / (route_ms * 1e-3), "ms": route_ms, "cores": torch.get_num_threads(),
            "breakdown_ms": {"t_logit": sum(t[0] for t in ts) / len(ts), "t_select": sum(t[1] for t in ts) / len(ts),
                             "t_pack": sum(t[2] for t in ts) / len(ts)}}


def main_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 20))  # each step is one full T=4096 pass (~70 ms): bounded
    r = run_cpu_reference(steps, min(args.warmup, 3))
    line = {
        "impl": "reference", "metric": "routed tokens/s per MoE layer", "value": r["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 3), "ms_per_step": r["ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD + " (CPU path: fp32, fused_select runs as naive_topk)"},
        "cpu_baseline": {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port",
                         "sample": f"{steps} full passes of T=4096 tokens", "breakdown_ms": r["breakdown_ms"]},
        "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def main_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    else:  # the expert-parallel layer below runs through torch.distributed even on one rank
        import socket

        sock = socket.socket()
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
        sock.close()
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1, device_id=dev)

    from moe_routers_b200 import ops  # raises if libmoe_b200.so is missing: there is no fallback

    steps, warmup = args.steps, max(3, args.warmup)
    n_sets = 5  # 5 x (33.5 MB tokens + 67 MB packed) = 503 MB > 126 MB L2
    g = torch.Generator(device="cpu").manual_seed(0)
    w_cpu = (torch.randn(E, D, generator=g) / (D ** 0.5)).half()
    w = w_cpu.to(dev)
    gens = torch.Generator(device=dev).manual_seed(1 + rank)
    xs = [torch.randn(T, D, device=dev, generator=gens).half() for _ in range(n_sets)]
    outs = [ops.route_fused(xs[i], w, K_TOP, skew_experts=SKEW_N, skew_bias=SKEW_B) for i in range(n_sets)]
    sel_outs = [ops.router_gemm_select(xs[i], w, K_TOP, skew_experts=SKEW_N, skew_bias=SKEW_B) for i in range(n_sets)]
    torch.cuda.synchronize()

    def step(i):
        ops.route_fused(xs[i % n_sets], w, K_TOP, skew_experts=SKEW_N, skew_bias=SKEW_B, out=outs[i % n_sets])

    # the reference's own operator: logits given (fp16), select + count + scan + pack
    lgs = [(xs[i] @ w.t()) for i in range(n_sets)]
    for lg in lgs:
        lg[:, :SKEW_N] += SKEW_B
    sp_outs = [ops.fused_select(lgs[i], xs[i], E, K_TOP) for i in range(n_sets)]

    def select_pack(i):
        ops.fused_select(lgs[i % n_sets], xs[i % n_sets], E, K_TOP, out=sp_outs[i % n_sets])

    def scatter_only(i):
        # the scatter kernel alone: tokens, indices and tile histograms of set 0 (the tokens are then
        # L2-resident, as they are right after the router kernel in the fused step), output rows into
        # rotating buffers so that every launch writes cold memory
        ops.pack_scatter(xs[0], E, dict(outs[0], packed=outs[i % n_sets]["packed"]))

    def select_only(i):
        ops.router_gemm_select(xs[i % n_sets], w, K_TOP, skew_experts=SKEW_N, skew_bias=SKEW_B)

    def capture(fn, n):
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            fn(0)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(n):
                    fn(i)
        torch.cuda.synchronize()
        return graph

    def timed(graph):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    g_route = capture(step, steps)
    g_select = capture(select_only, steps)
    g_selpack = capture(select_pack, steps)
    ops.route_fused(xs[0], w, K_TOP, skew_experts=SKEW_N, skew_bias=SKEW_B, out=outs[0])  # histograms of set 0
    torch.cuda.synchronize()
    g_scatter = capture(scatter_only, steps)

    # The same K steps issued round-robin on three streams (each with its own scratch buffer), so that
    # up to three independent batches are in flight: the scatter of one batch runs under the router
    # GEMM of the next.  Reported beside the headline, which stays one batch at a time.
    n_streams = 3
    pstreams = [torch.cuda.Stream() for _ in range(n_streams)]
    for ps in pstreams:
        with torch.cuda.stream(ps):
            step(0)  # creates the stream's scratch buffer outside the capture
    torch.cuda.synchronize()
    g_pipe = torch.cuda.CUDAGraph()
    with torch.cuda.stream(pstreams[0]):
        with torch.cuda.graph(g_pipe, stream=pstreams[0]):
            for ps in pstreams[1:]:
                ps.wait_stream(pstreams[0])
            for i in range(steps):
                with torch.cuda.stream(pstreams[i % n_streams]):
                    step(i)
            for ps in pstreams[1:]:
                pstreams[0].wait_stream(ps)
    torch.cuda.synchronize()
    g_route.replay()  # one untimed replay: graph upload
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    total_ms = timed(g_route)  # the timed region: exactly `steps` steps
    # keep the same load running a little longer so that the 2 ms clock sampler sees it (untimed)
    t_end = time.time() + 0.3
    while time.time() < t_end:
        g_route.replay()
    torch.cuda.synchronize()
    sampler.stop()
    select_ms = timed(g_select)
    selpack_us = timed(g_selpack) / steps * 1e3
    g_pipe.replay()
    pipe_ms = timed(g_pipe) / steps
    ops.route_fused(xs[0], w, K_TOP, skew_experts=SKEW_N, skew_bias=SKEW_B, out=outs[0])
    torch.cuda.synchronize()
    scatter_direct_us = timed(g_scatter) / steps * 1e3

    ms_per_step = total_ms / steps
    select_us = select_ms / steps * 1e3
    # Duration of the scatter kernel inside the timed region: fused step minus the router kernel.
    # (Launched alone back to back it is ~4 us slower, see `alone_back_to_back_us`: its 67 MB of stores
    # are absorbed by the L2 and written back to DRAM under the NEXT kernel; with nothing but scatters
    # in the queue the write-back has no read phase to hide under and write-only HBM bandwidth governs.)
    scatter_us = max(ms_per_step * 1e3 - select_us, 1e-3)
    value = world * T / (ms_per_step * 1e-3)
    peak, peak_kind = measured_peak_gbs()
    pack_gbs = PACK_BYTES / (scatter_us * 1e-6) / 1e9
    route_gbs = ROUTE_BYTES / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the public API with host buffers -------------------------------
    # Two slots on two streams: the download of step i overlaps the upload and kernels of step i+1
    # (separate copy engines); every step still uploads its x and the router weight and downloads all
    # seven result tensors.  `latency_ms` is one step alone (upload, kernels, download in series).
    from moe_routers_b200.host import HostRouter

    x_host = xs[0].cpu().pin_memory()
    hr = HostRouter(T, D, w_cpu, K_TOP, depth=2, skew_experts=SKEW_N, skew_bias=SKEW_B, device=dev,
                    upload_weight_each_call=True)
    e2e_steps = max(4, min(steps, 20))
    for _ in range(3):
        hr.route(x_host)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        hr.route(x_host)
    e2e_latency_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    prev = hr.submit(x_host)
    for _ in range(e2e_steps - 1):
        cur = hr.submit(x_host)
        hr.result(prev)
        prev = cur
    last = hr.result(prev)
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    assert int(last["offsets"][-1]) == T * K_TOP  # the downloaded result is a complete route
    if world > 1:
        t = torch.tensor([e2e_s, e2e_latency_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s, e2e_latency_s = (float(v) for v in t.tolist())
    h2d, d2h = hr.h2d_bytes, hr.d2h_bytes
    del hr

    # ---- the expert-parallel MoE layer on the same ranks (T=4096 tokens per rank, 64 experts split
    # over the ranks, 2-layer GELU experts 4096 -> 8192 -> 4096), skewed and unskewed -------------
    ep = {}
    try:
        import argparse as _ap

        from moe_routers_b200 import bench_ep

        del xs, sel_outs, lgs, sp_outs
        torch.cuda.empty_cache()
        for tag, (sn, sb) in {"skew": (SKEW_N, SKEW_B), "plain": (0, 0.0)}.items():
            ns = _ap.Namespace(experts=E, top_k=K_TOP, d_model=D, hidden=8192, tokens=T, all_strategies=False,
                               strategies=["fused_select"], strategy="fused_select", sinkhorn_iters=10,
                               sinkhorn_temperature=1.0, warmup=2, iters=5, skew_experts=sn, skew_bias=sb, transport="peer")
            r = bench_ep.run(ns)[0]
            ep[tag] = {k: r[k] for k in ("t_route_us", "t_comm_us", "t_comp_us", "t_combine_us", "t_layer_seq_us",
                                         "t_layer_overlap_us", "t_layer_back_to_back_us", "eta_overlap", "load_max_over_mean", "load_cv",
                                         "tokens_per_s")}
    except Exception as exc:  # the route numbers above stand on their own
        ep = {"error": f"{type(exc).__name__}: {exc}"}

    # sanity: the result of the last step agrees with the invariants of the route
    o = outs[0]
    assert int(o["offsets"][-1]) == T * K_TOP and int(o["counts"].sum()) == T * K_TOP
    assert ops.read_status() == 0

    if rank == 0:
        cpu = run_cpu_reference(3, 1) if world == 1 else None
        line = {
            "metric": "routed tokens/s per MoE layer", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "tokens_per_gpu": T, "d_model": D, "experts": E, "top_k": K_TOP,
                       "l2": f"{n_sets} rotating input/output sets, {n_sets * (T * D * 2 * 3) >> 20} MiB > 126 MB L2",
                       "launch": "K steps captured in one CUDA graph"},
            "breakdown_us": {"t_logit_select": select_us, "t_pack": ms_per_step * 1e3 - select_us,
                             "t_route": ms_per_step * 1e3},
            "roofline": {"kernel": "pack_scatter_bulk_kernel", "bound": "hbm", "achieved": pack_gbs, "peak": peak,
                         "unit": "GB/s", "frac": pack_gbs / peak, "traffic": SCATTER_DRAM_TRAFFIC, "peak_kind": peak_kind,
                         "algorithmic_bytes": PACK_BYTES,
                         "duration_us": scatter_us,
                         "how": "CUDA events, same run: K fused steps minus K router-kernel-only steps (both one graph)",
                         "alone_back_to_back_us": scatter_direct_us},
            "route_roofline": {"bound": "hbm", "achieved": route_gbs, "peak": peak, "unit": "GB/s",
                               "frac": route_gbs / peak, "algorithmic_bytes": ROUTE_BYTES},
            "pipelined": {"what": "the same K steps round-robin on 3 streams (independent batches in flight)",
                          "streams": n_streams, "value": world * T / (pipe_ms * 1e-3), "unit": "tokens/s",
                          "ms_per_step": pipe_ms, "route_roofline_frac": ROUTE_BYTES / (pipe_ms * 1e-3) / 1e9 / peak},
            "select_pack_roofline": {
                "what": "fused_select_forward(logits, x): select + count + scan + pack from given fp16 logits, 2 launches",
                "bound": "hbm", "duration_us": selpack_us, "algorithmic_bytes": PACK_BYTES + T * E * 2 + T * K_TOP * 4,
                "achieved": (PACK_BYTES + T * E * 2 + T * K_TOP * 4) / (selpack_us * 1e-6) / 1e9, "peak": peak,
                "unit": "GB/s", "frac": (PACK_BYTES + T * E * 2 + T * K_TOP * 4) / (selpack_us * 1e-6) / 1e9 / peak},
            "e2e": {"value": world * T / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s * 1e3, "pipeline_depth": 2,
                    "latency_ms": e2e_latency_s * 1e3},
            "gpu_launches": 2 * steps,
            "clocks": sampler.summary(),
            "ep_layer": ep,
        }
        if cpu is not None:
            line["cpu_baseline"] = {"value": cpu["value"], "unit": "tokens/s", "cores": cpu["cores"], "kind": "port",
                                    "sample": "3 full passes of T=4096 tokens (fp32, naive_topk path)",
                                    "breakdown_ms": cpu["breakdown_ms"]}
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        main_reference(a)
    else:
        main_ours(a)
