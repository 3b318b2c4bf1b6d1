#!/usr/bin/env python
"""Benchmark of the fused MoE route (router logit GEMM + select + pack) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the headline metric is quoted on): single-GPU
fp16 `fused_select`, T=4096 tokens, d_model=4096, E=64 experts, top_k=2,
hidden ~ N(0,1), router weight ~ N(0,1/d_model), +2.0 skew on the logits of
experts 0..7.  A step is one pass of the route over one batch: one
`moe_route_fused` call = router GEMM/select kernel + scatter kernel.

Prints ONE JSON line (rank 0).  Keys beyond the common contract:
  timing        the K-step graph is replayed R times, each replay between its own CUDA events;
                `ms_per_step` is the median replay / K, `min_ms_per_step` the fastest
  roofline      the whole step: 101,253,636 algorithmic bytes / ms_per_step against the measured
                HBM copy peak; `kernels` holds each kernel timed alone back to back, and the step
                with the overlap between the two kernels switched off
  peaks_local   copy / read-only / write-only streams measured in this run
  select_pack_roofline   the reference's own operator (logits given): select + count + scan + pack
  strategies    the other routing strategies and the expert FFN shapes of the benchmark
                configurations (single GPU), each with its own roofline figure
  cpu_baseline  the reference's CPU routing path on the host cores (its own bench_router.py
                --device cpu where staged under oracle/_ref, else the port in oracle/cpu_route.py)
  e2e           the same metric through the public API with HOST buffers (pinned), host<->device
                copies of every step inside the timed region, two steps in flight (HostRouter),
                downloading what a host caller consumes (indices, gates, counts, offsets, maps);
                `e2e_full` also downloads the packed rows
  ep_layer      the expert-parallel MoE layer on the same ranks; `ep_parity` checks its output
Timing: CUDA events on the launching stream, max over ranks; inputs and outputs rotate over several
buffer sets whose total size exceeds the L2, so every step reads its tokens from HBM.
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
HID = 8192
SKEW_N, SKEW_B = 8, 2.0
ROUTE_BYTES = T * D * 2 + E * D * 2 + K_TOP * T * D * 2 + 2 * T * K_TOP * 4 + E * 4 + (E + 1) * 4  # 101,253,636
PACK_BYTES = T * D * 2 + T * K_TOP * 4 + K_TOP * T * D * 2  # 100,696,064
ROUTER_BYTES = T * D * 2 + E * D * 2 + 2 * T * K_TOP * 4 + (T // 32) * E * 4  # 34,177,024
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/ (router kernel: exactly its reads; scatter: the L2 still holds most of the 67 MB written
# when the kernel ends, hence less than the algorithmic bytes)
ROUTER_DRAM_TRAFFIC = 34_150_000
SCATTER_DRAM_TRAFFIC = 42_900_000
WORKLOAD = "fused_select T=4096 d_model=4096 E=64 top_k=2 fp16, +2.0 skew on experts 0..7"
# the same object in both arms; `l2` says how the GPU arm keeps its inputs out of the L2 between steps
CONFIG = {"workload": WORKLOAD,
          "l2": "GPU arm: 5 rotating input/output sets, 480 MiB > 126 MB L2, no flush needed; CPU arm: not applicable"}
METRIC = "routed tokens/s per MoE layer"


_T0 = time.time()


def _progress(msg: str) -> None:
    """Section marks with the seconds since start, on stderr (the JSON line owns stdout)."""
    print(f"[bench {time.time() - _T0:7.1f}s] {msg}", file=sys.stderr, flush=True)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--repeats", type=int, default=0, help="timed replays of the K-step graph (0: enough for >= 40 ms)")
    ap.add_argument("--quick", action="store_true", help="skip the strategy / FFN sub-records and the EP leg")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            j = json.load(f)
        return float(j["hbm_gbs"]), float(j["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


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
def _host_threads() -> int:
    """All host threads this process may use (a multi-rank launcher exports OMP_NUM_THREADS=1, which
    would make the baseline single-threaded; only one rank runs it, so it takes the whole host)."""
    import torch

    try:
        n_cpu = len(os.sched_getaffinity(0))
    except AttributeError:
        n_cpu = os.cpu_count() or 1
    if torch.get_num_threads() < n_cpu:
        torch.set_num_threads(n_cpu)
    return torch.get_num_threads()


def run_cpu_reference(steps: int, warmup: int, strategy: str = "fused_select", skew: bool = True):
    """The reference's CPU routing path (bench_router.py --device cpu --dtype fp32; fused_select runs
    as naive_topk there, :498-501) on this host's cores, same T/d/E/k/skew.  Uses the reference's own
    file when it has been staged under oracle/_ref (kind "reference"), else the torch port."""
    import torch
    from oracle import cpu_route, ref_runner

    cores = _host_threads()
    sn, sb = (SKEW_N, SKEW_B) if skew else (0, 0.0)
    if ref_runner.available():
        r = ref_runner.run_cpu(tokens=T, d_model=D, experts=E, top_k=K_TOP, strategy=strategy, skew_experts=sn,
                               skew_bias=sb, warmup=max(1, warmup), iters=steps)
        return {"value": T / (r["t_route_ms"] * 1e-3), "ms": r["t_route_ms"], "cores": cores, "kind": "reference",
                "inputs": "the reference's own generator: torch.manual_seed(0), x ~ N(0,1), W ~ N(0,1)",
                "breakdown_ms": {"t_logit": r["t_logit_ms"], "t_select": r["t_select_ms"], "t_pack": r["t_pack_ms"]}}
    g = torch.Generator().manual_seed(0)
    x = torch.randn(T, D, generator=g)
    w = torch.randn(E, D, generator=g) / (D ** 0.5)
    st = "sinkhorn" if strategy == "sinkhorn" else "naive_topk"
    for _ in range(max(1, warmup)):
        cpu_route.one_iter(x, w, K_TOP, strategy=st, skew_experts=sn, skew_bias=sb)
    ts = [cpu_route.one_iter(x, w, K_TOP, strategy=st, skew_experts=sn, skew_bias=sb) for _ in range(steps)]
    route_ms = sum(t[3] for t in ts) / len(ts)
    return {"value": T / (route_ms * 1e-3), "ms": route_ms, "cores": cores, "kind": "port",
            "inputs": "seeded x ~ N(0,1), W ~ N(0,1/d)",
            "breakdown_ms": {"t_logit": sum(t[0] for t in ts) / len(ts), "t_select": sum(t[1] for t in ts) / len(ts),
                             "t_pack": sum(t[2] for t in ts) / len(ts)}}


def main_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(3, args.warmup)  # each step is one full T=4096 pass (~0.1 s of CPU)
    r = run_cpu_reference(steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": r["ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(CONFIG),
        "notes": "CPU path of the reference: fp32, the fused_select strategy runs as naive_topk (bench_router.py:498-501); "
                 + r["inputs"],
        "cpu_baseline": {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": r["kind"],
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

    from moe_routers_b200 import _lib, ops  # raises if libmoe_b200.so is missing: there is no fallback

    lib = _lib.lib
    steps, warmup = args.steps, max(3, args.warmup)
    peak, peak_tf, peak_kind = measured_peaks()
    n_sets = 5  # 5 x (33.5 MB tokens + 67 MB packed) = 503 MB > 126 MB L2
    g = torch.Generator(device="cpu").manual_seed(0)
    w_cpu = (torch.randn(E, D, generator=g) / (D ** 0.5)).half()
    w = w_cpu.to(dev)
    gens = torch.Generator(device=dev).manual_seed(1 + rank)
    xs = [torch.randn(T, D, device=dev, generator=gens).half() for _ in range(n_sets)]
    outs = [ops.route_fused(xs[i], w, K_TOP, skew_experts=SKEW_N, skew_bias=SKEW_B) for i in range(n_sets)]
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
        """K calls of fn in one CUDA graph; returns (graph, kernel launches captured)."""
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())  # inputs may still be in flight on the caller's stream
        with torch.cuda.stream(stream):
            fn(0)
            torch.cuda.synchronize()
            before = int(lib.moe_launch_count())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(n):
                    fn(i)
            launches = int(lib.moe_launch_count()) - before
        torch.cuda.synchronize()
        return graph, launches

    def timed(graph, repeats=1):
        """`repeats` replays, each between its own event pair; per-replay ms (max over ranks)."""
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(repeats)]
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        for a, b in evs:
            a.record()
            graph.replay()
            b.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = torch.tensor([a.elapsed_time(b) for a, b in evs], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return sorted(float(v) for v in ms.tolist())

    def med(v):
        return v[len(v) // 2]

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    g_route, route_launches = capture(step, steps)
    g_select, _ = capture(select_only, steps)
    g_selpack, _ = capture(select_pack, steps)
    step(0)  # histograms of set 0 for the scatter-only graphs
    torch.cuda.synchronize()
    g_scatter, _ = capture(scatter_only, steps)
    # the same graphs with plain stream order between the kernels (no programmatic dependent launch):
    # nothing of one kernel runs under another
    lib.moe_set_pdl(0)
    g_route_serial, _ = capture(step, steps)
    g_select_serial, _ = capture(select_only, steps)
    step(0)
    torch.cuda.synchronize()
    g_scatter_serial, _ = capture(scatter_only, steps)
    lib.moe_set_pdl(1)

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
    est_ms = timed(g_route)[0]
    repeats = args.repeats if args.repeats > 0 else max(50, min(2000, int(40.0 / max(est_ms, 1e-3)) + 1))

    sampler = ClockSampler(local_rank)
    sampler.start()
    route_ms = timed(g_route, repeats)  # the timed region: `repeats` replays of exactly `steps` steps
    # keep the same load running a little longer so that the 2 ms clock sampler sees it (untimed)
    t_end = time.time() + 0.3
    while time.time() < t_end:
        g_route.replay()
    torch.cuda.synchronize()
    sampler.stop()
    sub_rep = max(10, repeats // 4)
    select_us = med(timed(g_select, sub_rep)) / steps * 1e3
    selpack_us = med(timed(g_selpack, sub_rep)) / steps * 1e3
    g_pipe.replay()
    pipe_ms = med(timed(g_pipe, sub_rep)) / steps
    step(0)
    torch.cuda.synchronize()
    scatter_us = med(timed(g_scatter, sub_rep)) / steps * 1e3
    serial_step_us = med(timed(g_route_serial, sub_rep)) / steps * 1e3
    serial_select_us = med(timed(g_select_serial, sub_rep)) / steps * 1e3
    step(0)
    torch.cuda.synchronize()
    serial_scatter_us = med(timed(g_scatter_serial, sub_rep)) / steps * 1e3

    ms_per_step = med(route_ms) / steps
    min_ms_per_step = route_ms[0] / steps
    value = world * T / (ms_per_step * 1e-3)
    route_gbs = ROUTE_BYTES / (ms_per_step * 1e-3) / 1e9

    def event_us(fn, n=10, warm=3):
        """Median of n CUDA-event timings of fn() (eager launches), microseconds."""
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(n):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return sorted(ts)[len(ts) // 2]

    # ---- local peaks: plain streams on 1 GiB buffers, this GPU, this run ---------------------------
    peaks_local = {}
    try:
        n_el = 1 << 29  # 1 GiB of fp16
        a_buf = torch.empty(n_el, dtype=torch.float16, device=dev).normal_()
        b_buf = torch.empty(2 * n_el, dtype=torch.float16, device=dev)
        nb = n_el * 2
        peaks_local = {
            "unit": "GB/s", "how": "torch kernels on 1 GiB fp16 buffers, median of 10, CUDA events",
            "copy": 2 * nb / event_us(lambda: b_buf[:n_el].copy_(a_buf)) / 1e3,
            "read_only": nb / event_us(lambda: a_buf.sum()) / 1e3,
            "write_only": 2 * nb / event_us(lambda: b_buf.zero_()) / 1e3,
        }
        del a_buf, b_buf
        torch.cuda.empty_cache()
    except Exception as exc:
        peaks_local = {"error": f"{type(exc).__name__}: {exc}"}

    # ---- end to end through the public API with host buffers -------------------------------
    # Two slots on two streams: the download of step i overlaps the upload and kernels of step i+1
    # (separate copy engines); every step uploads its x and the router weight and downloads the
    # results.  `latency_ms` is one step alone (upload, kernels, download in series).
    from moe_routers_b200.host import HostRouter

    from moe_routers_b200.host import pin_near

    x_host = pin_near(xs[0].cpu(), dev)  # the caller's batch, pinned on the GPU's NUMA node

    def run_e2e(download):
        hr = HostRouter(T, D, w_cpu, K_TOP, depth=2, skew_experts=SKEW_N, skew_bias=SKEW_B, device=dev,
                        upload_weight_each_call=True, download=download)
        n = max(4, min(steps, 20))
        for _ in range(3):
            hr.route(x_host)
        t0 = time.perf_counter()
        for _ in range(n):
            hr.route(x_host)
        latency_s = (time.perf_counter() - t0) / n
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        prev = hr.submit(x_host)
        for _ in range(n - 1):
            cur = hr.submit(x_host)
            hr.result(prev)
            prev = cur
        last = hr.result(prev)
        per_step_s = (time.perf_counter() - t0) / n
        assert int(last["offsets"][-1]) == T * K_TOP  # the downloaded result is a complete route
        if world > 1:
            t = torch.tensor([per_step_s, latency_s], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            per_step_s, latency_s = (float(v) for v in t.tolist())
        rec = {"value": world * T / per_step_s, "unit": "tokens/s", "h2d_bytes_per_step": hr.h2d_bytes,
               "d2h_bytes_per_step": hr.d2h_bytes, "ms_per_step": per_step_s * 1e3, "pipeline_depth": 2,
               "latency_ms": latency_s * 1e3, "downloads": sorted(hr.slots[0]["host"].keys()),
               "per_rank_gbs": (hr.h2d_bytes + hr.d2h_bytes) / per_step_s / 1e9}
        del hr
        return rec

    _progress("route graphs timed; end-to-end leg")
    e2e = run_e2e(("idx", "gates", "counts", "offsets", "row_route", "route_row"))
    e2e_full = run_e2e(None)

    # sanity: the result of the last step agrees with the invariants of the route
    o = outs[0]
    assert int(o["offsets"][-1]) == T * K_TOP and int(o["counts"].sum()) == T * K_TOP
    assert ops.read_status() == 0

    # ---- the other strategies and the expert-FFN shapes of the benchmark configurations (1 GPU) ----
    strategies = {}
    if world == 1 and not args.quick:
        try:
            _progress("strategy and expert-FFN records")
            strategies = bench_strategies(torch, ops, dev, xs, w, capture, timed, med, event_us, peak, peak_tf)
            _progress("strategy records done")
        except Exception as exc:
            strategies = {"error": f"{type(exc).__name__}: {exc}"}

    # ---- the expert-parallel MoE layer on the same ranks (T=4096 tokens per rank, 64 experts split
    # over the ranks, 2-layer GELU experts 4096 -> 8192 -> 4096), skewed and unskewed -------------
    ep, ep_parity = {}, {}
    del xs, lgs, sp_outs
    torch.cuda.empty_cache()
    if not args.quick:
        try:
            _progress("expert-parallel parity check")
            ep_parity = check_ep_parity(torch, dist, dev, rank, world)
            _progress("expert-parallel parity check done")
        except Exception as exc:
            ep_parity = {"ok": False, "error": f"{type(exc).__name__}: {exc}"}
        try:
            import argparse as _ap

            from moe_routers_b200 import bench_ep

            keep = ("t_route_us", "t_comm_us", "t_comp_us", "t_combine_us", "t_layer_seq_us", "t_layer_overlap_us",
                    "t_layer_back_to_back_us", "eta_overlap", "eta_seq_over_overlap", "load_max_over_mean", "load_cv",
                    "tokens_per_s")
            for tag, (sn, sb) in {"skew": (SKEW_N, SKEW_B), "plain": (0, 0.0)}.items():
                ns = _ap.Namespace(experts=E, top_k=K_TOP, d_model=D, hidden=HID, tokens=T, all_strategies=True,
                                   strategies=None, strategy="fused_select", sinkhorn_iters=10, dtype="fp16",
                                   sinkhorn_temperature=1.0, warmup=3, iters=20, skew_experts=sn, skew_bias=sb,
                                   transport="peer")
                ep[tag] = {r["strategy"]: {k: r[k] for k in keep} for r in bench_ep.run(ns)}
        except Exception as exc:  # the route numbers above stand on their own
            ep["error"] = f"{type(exc).__name__}: {exc}"

    if rank == 0:
        _progress("CPU baseline")
        cpu = run_cpu_reference(3, 1) if world == 1 else None
        _progress("done")
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": dict(CONFIG),
            "setup": {"tokens_per_gpu": T, "d_model": D, "experts": E, "top_k": K_TOP,
                      "l2": f"{n_sets} rotating input/output sets, {n_sets * (T * D * 2 * 3) >> 20} MiB > 126 MB L2",
                      "launch": "K steps captured in one CUDA graph, replayed `repeats` times"},
            "timing": {"repeats": repeats, "median_ms_per_step": ms_per_step, "min_ms_per_step": min_ms_per_step,
                       "max_ms_per_step": route_ms[-1] / steps, "timed_region_ms": sum(route_ms)},
            "breakdown_us": {"t_logit_select": select_us, "t_pack": ms_per_step * 1e3 - select_us,
                             "t_route": ms_per_step * 1e3,
                             "note": "t_logit_select: the router kernel alone back to back; t_pack: the rest of the step"},
            "roofline": {"kernel": "route step = router_gemm_select_kernel + pack_scatter_bulk_kernel", "bound": "hbm",
                         "achieved": route_gbs, "peak": peak, "unit": "GB/s", "frac": route_gbs / peak,
                         "traffic": ROUTER_DRAM_TRAFFIC + SCATTER_DRAM_TRAFFIC, "peak_kind": peak_kind,
                         "algorithmic_bytes": ROUTE_BYTES, "duration_us": ms_per_step * 1e3,
                         "how": "CUDA events around graph replays of K steps, median of `timing.repeats`",
                         "serial_step_us": serial_step_us,
                         "kernels": {
                             "router_gemm_select_kernel": {
                                 "algorithmic_bytes": ROUTER_BYTES, "alone_us": select_us,
                                 "alone_serial_us": serial_select_us, "traffic": ROUTER_DRAM_TRAFFIC,
                                 "frac": ROUTER_BYTES / (serial_select_us * 1e-6) / 1e9 / peak},
                             "pack_scatter_bulk_kernel": {
                                 "algorithmic_bytes": PACK_BYTES, "alone_us": scatter_us,
                                 "alone_serial_us": serial_scatter_us, "traffic": SCATTER_DRAM_TRAFFIC,
                                 "frac": PACK_BYTES / (serial_scatter_us * 1e-6) / 1e9 / peak},
                             "note": "alone = K launches of that kernel back to back in one graph; serial = "
                                     "programmatic dependent launch off (plain stream order), so no part of a "
                                     "kernel runs under its neighbour; serial_step_us is the whole step that way"}},
            "peaks_local": peaks_local,
            "pipelined": {"what": "the same K steps round-robin on 3 streams (independent batches in flight)",
                          "streams": n_streams, "value": world * T / (pipe_ms * 1e-3), "unit": "tokens/s",
                          "ms_per_step": pipe_ms, "route_roofline_frac": ROUTE_BYTES / (pipe_ms * 1e-3) / 1e9 / peak},
            "select_pack_roofline": {
                "what": "fused_select_forward(logits, x): select + count + scan + pack from given fp16 logits, 2 launches",
                "bound": "hbm", "duration_us": selpack_us, "algorithmic_bytes": PACK_BYTES + T * E * 2 + T * K_TOP * 4,
                "achieved": (PACK_BYTES + T * E * 2 + T * K_TOP * 4) / (selpack_us * 1e-6) / 1e9, "peak": peak,
                "unit": "GB/s", "frac": (PACK_BYTES + T * E * 2 + T * K_TOP * 4) / (selpack_us * 1e-6) / 1e9 / peak},
            "strategies": strategies,
            "e2e": e2e, "e2e_full": e2e_full,
            "gpu_launches": route_launches * repeats,
            "gpu_launches_per_step": route_launches / max(steps, 1),
            "clocks": sampler.summary(),
            "ep_layer": ep, "ep_parity": ep_parity,
        }
        if cpu is not None:
            line["cpu_baseline"] = {"value": cpu["value"], "unit": "tokens/s", "cores": cpu["cores"], "kind": cpu["kind"],
                                    "sample": "3 full passes of T=4096 tokens (fp32, naive_topk path); " + cpu["inputs"],
                                    "breakdown_ms": cpu["breakdown_ms"]}
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def bench_strategies(torch, ops, dev, xs, w, capture, timed, med, event_us, peak, peak_tf):
    """Driver-visible figures for BASELINE configurations 1, 3, 4 and the expert FFN shapes: each
    record gives its time, its algorithmic work and the fraction of the roofline that bounds it."""
    from moe_routers_b200 import strategies as st

    n_sets = len(xs)
    out = {}
    k_steps = 10

    def graph_us(fn):
        g_, _ = capture(fn, k_steps)
        g_.replay()
        return med(timed(g_, 10)) / k_steps * 1e3

    # configuration 1/2 as naive_topk: logit GEMM + top-k (logits written) + pack, 3 launches
    for tag, (sn, sb) in {"skew": (SKEW_N, SKEW_B), "plain": (0, 0.0)}.items():
        us = graph_us(lambda i: st.route("naive_topk", xs[i % n_sets], w, K_TOP, skew_experts=sn, skew_bias=sb))
        byt = ROUTE_BYTES + T * E * 4 + T * K_TOP * 4 + (T // 32) * E * 4
        out[f"naive_topk_{tag}"] = {"t_route_us": us, "tokens_per_s": T / (us * 1e-6), "bound": "hbm",
                                    "algorithmic_bytes": byt, "frac": byt / (us * 1e-6) / 1e9 / peak}
        # configuration 4: Sinkhorn, 10 iterations, temperature 1
        us = graph_us(lambda i: st.route("sinkhorn", xs[i % n_sets], w, K_TOP, skew_experts=sn, skew_bias=sb,
                                         sinkhorn_iters=10, sinkhorn_temperature=1.0))
        lg = ops.router_gemm_select(xs[0], w, K_TOP, skew_experts=sn, skew_bias=sb, return_logits=True)[2]
        sk_us = graph_us(lambda i: ops.sinkhorn(lg, K_TOP, iters=10))
        out[f"sinkhorn_{tag}"] = {"t_route_us": us, "tokens_per_s": T / (us * 1e-6), "sinkhorn_kernel_us": sk_us,
                                  "bound": "sync latency (589,824 compulsory bytes)", "algorithmic_bytes": byt,
                                  "frac": byt / (us * 1e-6) / 1e9 / peak,
                                  "reference_traffic_model_bytes": (2 + 4 * 10) * 2 * T * E * 4}
    _progress("  naive_topk and sinkhorn routes timed")
    # combine
    o = ops.route_fused(xs[0], w, K_TOP)
    ys = [o["packed"]] + [o["packed"].clone() for _ in range(3)]  # 4 x 67 MB of expert outputs > L2
    us = graph_us(lambda i: ops.combine(ys[i % len(ys)], o["gates"], o["route_row"], K_TOP))
    out["combine"] = {"t_us": us, "bound": "hbm", "algorithmic_bytes": PACK_BYTES,
                      "frac": PACK_BYTES / (us * 1e-6) / 1e9 / peak, "inputs": "4 rotating expert-output buffers"}
    del ys
    # grouped expert FFN 4096 -> 8192 -> 4096 on 8192 routed rows: 8 experts x 1024 rows (tensor-bound),
    # 64 experts x 128 rows (weight-bound)
    _progress("  combine timed")
    flops = 2.0 * T * K_TOP * (D * HID + HID * D)
    rows = torch.randn(T * K_TOP, D, device=dev).half()
    for n_exp in (8, 64):
        w1 = (torch.randn(n_exp, HID, D, device=dev) / D ** 0.5).half()
        w2 = (torch.randn(n_exp, D, HID, device=dev) / HID ** 0.5).half()
        off = torch.arange(0, T * K_TOP + 1, T * K_TOP // n_exp, device=dev, dtype=torch.int32)
        hbuf = torch.empty((T * K_TOP, HID), dtype=torch.float16, device=dev)
        ybuf = torch.empty((T * K_TOP, D), dtype=torch.float16, device=dev)

        def ffn():
            ops.grouped_gemm(rows, w1, off, layout="nk", activation="gelu", out=hbuf)
            ops.grouped_gemm(hbuf, w2, off, layout="nk", out=ybuf)

        # two FFNs per CUDA graph, 8 replays timed one by one: the launches cost no host time inside
        # the timed region and the run stays short enough for burst clocks
        def ffn_graph_us():
            g_ffn, _ = capture(lambda i: ffn(), 2)
            g_ffn.replay()
            return med(timed(g_ffn, 8)) / 2 * 1e3

        us = ffn_graph_us()
        _progress(f"  grouped FFN {n_exp} experts timed")
        variants = None
        if n_exp == 8:
            # the same shape on the one-CTA kernel (two-tile units), same box, same protocol
            from moe_routers_b200._lib import lib as _l
            mode = _l.moe_set_gemm_mode(-1)
            _l.moe_set_gemm_mode(mode & ~1)
            variants = {"one_cta_kernel_us": ffn_graph_us()}
            _l.moe_set_gemm_mode(mode & ~2)
            variants["two_cta_one_issuer_us"] = ffn_graph_us()
            _l.moe_set_gemm_mode(mode)
            # context only: the library batched GEMM on the same operands, same protocol, without the
            # activation (what the peak in MEASURED_PEAKS.json was measured with)
            x3, h3 = rows.view(n_exp, -1, D), hbuf.view(n_exp, -1, HID)
            y3 = ybuf.view(n_exp, -1, D)
            w1t, w2t = w1.transpose(1, 2), w2.transpose(1, 2)

            def ffn_lib():
                torch.bmm(x3, w1t, out=h3)
                torch.bmm(h3, w2t, out=y3)

            g_lib, _ = capture(lambda i: ffn_lib(), 2)
            g_lib.replay()
            variants["library_bmm_no_activation_us"] = med(timed(g_lib, 8)) / 2 * 1e3
        wbytes = n_exp * 2 * D * HID * 2
        abytes = T * K_TOP * (D + 2 * HID + D) * 2
        t_tensor = flops / (peak_tf * 1e12) * 1e6
        t_hbm = (wbytes + abytes) / (peak * 1e9) * 1e6
        out[f"grouped_ffn_{n_exp}x{T * K_TOP // n_exp}"] = {
            "t_us": us, "tflops": flops / (us * 1e-6) / 1e12, "flop": flops, "weight_bytes": wbytes,
            "bound": "tensor" if t_tensor >= t_hbm else "hbm (expert weights)",
            "frac_of_tensor_peak": flops / (us * 1e-6) / 1e12 / peak_tf,
            "frac": max(t_tensor, t_hbm) / us, "floor_us": max(t_tensor, t_hbm), "peak_tflops": peak_tf,
            "timing": "median of 8 replays of a CUDA graph holding 2 FFNs"}
        if variants:
            out[f"grouped_ffn_{n_exp}x{T * K_TOP // n_exp}"]["variants"] = variants
        if n_exp == 8:
            # configuration 3: masked_matmul, E=8: every expert runs densely over all T tokens
            w8 = (torch.randn(8, D, device=dev) / D ** 0.5).half()

            def mm():
                r = st.route("masked_matmul", xs[0], w8, K_TOP)
                st.masked_matmul_forward(xs[0], r, w1, w2, K_TOP)

            _progress("  FFN variants timed")
            us = event_us(mm, n=5, warm=2)
            _progress("  masked_matmul timed")
            mflops = 8.0 * T * 2 * (D * HID + HID * D) + 2.0 * T * D * 8
            out["masked_matmul_E8"] = {"t_layer_us": us, "tokens_per_s": T / (us * 1e-6), "bound": "tensor", "flop": mflops,
                                       "tflops": mflops / (us * 1e-6) / 1e12,
                                       "frac": mflops / (us * 1e-6) / 1e12 / peak_tf, "peak_tflops": peak_tf}
        del w1, w2, hbuf, ybuf
        torch.cuda.empty_cache()
    # CPU figures beside the strategies the reference has a CPU path for (bench_router.py:484-505)
    for name, strat in (("naive_topk_plain", "naive_topk"), ("sinkhorn_plain", "sinkhorn")):
        _progress(f"  CPU reference, {strat}")
        c = run_cpu_reference(2, 1, strategy=strat, skew=False)
        out[name]["cpu_baseline"] = {"value": c["value"], "unit": "tokens/s", "cores": c["cores"], "kind": c["kind"],
                                     "sample": "2 full passes of T=4096 tokens", "breakdown_ms": c["breakdown_ms"]}
    return out


def check_ep_parity(torch, dist, dev, rank, world):
    """Correctness of the expert-parallel layer on THESE ranks, outside every timed region:
    (a) a small layer (T=512 per rank, d=256, h=512, E=64) on the peer and the nccl transport, with
    fused_select and sinkhorn, against the CPU oracle applied to the routing the layer chose (all
    expert weights are generated from one seed on every rank); (b) at the benchmark's full shape the
    two transports must produce the same output (the same kernels do the arithmetic)."""
    import numpy as np

    import oracle
    from moe_routers_b200.ep import EPMoELayer

    k = K_TOP
    worst, equal = 0.0, True

    def weights(e, d, h, seed):
        gw = torch.Generator(device=dev).manual_seed(seed)
        w_router = (torch.randn(e, d, device=dev, generator=gw) / d ** 0.5).half()
        w1 = (torch.randn(e, h, d, device=dev, generator=gw) / d ** 0.5).half()
        w2 = (torch.randn(e, d, h, device=dev, generator=gw) / h ** 0.5).half()
        return w_router, w1, w2

    # (a) small shape against the oracle
    t, d, h, e = 512, 256, 512, E
    el = e // world
    w_router, w1, w2 = weights(e, d, h, 7)
    gx = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(t, d, device=dev, generator=gx).half()
    experts = {"w1": w1.float().cpu().numpy(), "w2": w2.float().cpu().numpy()}
    for strategy in ("fused_select", "sinkhorn"):
        outs = {}
        for tr in ("peer", "nccl"):
            layer = EPMoELayer(w_router, w1[rank * el:(rank + 1) * el].contiguous(), w2[rank * el:(rank + 1) * el].contiguous(),
                               k, activation="gelu", strategy=strategy, skew_experts=SKEW_N, skew_bias=SKEW_B, transport=tr)
            for overlap in (True, False):
                out = layer(x, overlap=overlap)
                torch.cuda.synchronize()
                o = layer.last["route"]
                ref, _ = oracle.moe_layer(x.float().cpu().numpy(), o["idx"].cpu().numpy(), o["gates"].cpu().numpy(), experts,
                                          kind="gelu", layout="nk")
                ref = ref.astype(np.float32)
                err = float(np.abs(out.float().cpu().numpy() - ref).max() / max(float(np.abs(ref).max()), 1e-9))
                worst = max(worst, err)
                outs[(tr, overlap)] = out.clone()
            layer.close()
        equal = equal and all(torch.equal(outs[("peer", True)], v) for v in outs.values())
    # (b) full shape: transports agree bit for bit
    w_router, w1, w2 = weights(E, D, HID, 0)
    w1l, w2l = w1[rank * (E // world):(rank + 1) * (E // world)].contiguous(), w2[rank * (E // world):(rank + 1) * (E // world)].contiguous()
    del w1, w2
    torch.cuda.empty_cache()
    x = torch.randn(T, D, device=dev, generator=gx).half()
    full = {}
    for tr in ("peer", "nccl"):
        layer = EPMoELayer(w_router, w1l, w2l, k, activation="gelu", strategy="fused_select", transport=tr)
        full[tr] = layer(x).clone()
        torch.cuda.synchronize()
        layer.close()
    full_equal = bool(torch.equal(full["peer"], full["nccl"]))
    finite = bool(torch.isfinite(full["peer"]).all()) and float(full["peer"].abs().max()) > 0
    from moe_routers_b200 import ops

    status_ok = ops.read_status() == 0
    flags = torch.tensor([worst, 0.0 if (equal and full_equal and finite and status_ok) else 1.0], device=dev, dtype=torch.float64)
    dist.all_reduce(flags, op=dist.ReduceOp.MAX)
    worst_all, bad = float(flags[0]), float(flags[1]) > 0
    return {"world": world, "max_rel_err": worst_all, "tolerance": 2e-2, "transports_equal": not bad,
            "full_shape_transports_equal": full_equal, "ok": (not bad) and worst_all <= 2e-2,
            "what": "small layer (T=512/rank, d=256, h=512, E=64; peer+nccl, overlap on/off, fused_select+sinkhorn) vs "
                    "the CPU oracle on the routing the layer chose; full-size layer: peer output == nccl output"}


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        main_reference(a)
    else:
        main_ours(a)
