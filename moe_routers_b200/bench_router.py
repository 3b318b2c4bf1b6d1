"""Router microbenchmark (single GPU), mirroring the reference's `bench_router.py` breakdown
(:5-9): T_logit, T_select, T_pack, T_route per strategy, with the same flags (:392-446) and the same
printed table (:596-601).

    python -m moe_routers_b200.bench_router --all_strategies --skew_experts 8 --skew_bias 2.0

Stages are timed one by one with CUDA events and a device synchronise, like the reference
(`_cuda_time`, :47-54); because that protocol hides what fusion saves, the fused single-call
route time is printed next to it (`T_fused`).  There is no CPU path here: `--device cpu` is refused
(the reference's own CPU path is what `bench.py --impl reference` times).
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops
from .strategies import STRATEGIES, route


def _cuda_time(fn) -> float:
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    fn()
    end.record()
    torch.cuda.synchronize()
    return float(start.elapsed_time(end))


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--device", type=str, default="cuda")
    p.add_argument("--dtype", type=str, default="fp16", choices=["fp16"])
    p.add_argument("--tokens", type=int, default=4096)
    p.add_argument("--d_model", type=int, default=4096)
    p.add_argument("--experts", type=int, default=64)
    p.add_argument("--top_k", type=int, default=2)
    p.add_argument("--strategies", type=str, nargs="+", default=None)
    p.add_argument("--all_strategies", action="store_true")
    p.add_argument("--strategy", type=str, default="naive_topk", choices=STRATEGIES)
    p.add_argument("--sinkhorn_iters", type=int, default=10)
    p.add_argument("--sinkhorn_temperature", type=float, default=1.0)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--skew_experts", type=int, default=0)
    p.add_argument("--skew_bias", type=float, default=0.0)
    args = p.parse_args()
    if torch.device(args.device).type != "cuda":
        raise RuntimeError("inputs must be CUDA: this library has no CPU path")

    torch.manual_seed(0)
    dev = torch.device("cuda")
    x = torch.randn(args.tokens, args.d_model, device=dev).half()
    w = (torch.randn(args.experts, args.d_model, device=dev) / args.d_model ** 0.5).half()
    strategies = STRATEGIES if args.all_strategies else (args.strategies or [args.strategy])
    unknown = [s for s in strategies if s not in STRATEGIES]
    if unknown:
        raise ValueError(f"Unknown strategies: {unknown}. Valid: {STRATEGIES}")
    kw = dict(skew_experts=args.skew_experts, skew_bias=args.skew_bias)
    k, e = args.top_k, args.experts

    def one_iter(strategy):
        st = {}
        t_logit = _cuda_time(lambda: st.update(zip(("idx", "gates", "logits"),
                                                   ops.router_gemm_select(x, w, k, return_logits=True, **kw))))
        if strategy == "sinkhorn":
            t_select = _cuda_time(lambda: st.update(zip(("idx", "gates"), ops.sinkhorn(
                st["logits"], k, iters=args.sinkhorn_iters, temperature=args.sinkhorn_temperature))))
        else:
            t_select = _cuda_time(lambda: st.update(zip(("idx", "gates"), ops.topk_select(st["logits"], k))))
        t_pack = 0.0 if strategy == "masked_matmul" else _cuda_time(lambda: ops.pack(x, st["idx"], e))
        t_fused = _cuda_time(lambda: route(strategy, x, w, k, sinkhorn_iters=args.sinkhorn_iters,
                                           sinkhorn_temperature=args.sinkhorn_temperature, **kw))
        return t_logit, t_select, t_pack, t_logit + t_select + t_pack, t_fused

    results = {}
    for s in strategies:
        for _ in range(args.warmup):
            one_iter(s)
        rows = [one_iter(s) for _ in range(args.iters)]
        results[s] = [sum(r[i] for r in rows) / len(rows) for i in range(5)]

    print("strategies:", strategies)
    print("device:", dev, "dtype: torch.float16")
    print("T(tokens):", args.tokens, "d_model:", args.d_model, "E:", e, "k:", k)
    print("skew_experts:", args.skew_experts, "skew_bias:", args.skew_bias)
    print("")
    print("=== Router Latency Breakdown (ms, mean) ===")
    print(f"{'strategy':<14} {'T_logit':>10} {'T_select':>10} {'T_pack':>10} {'T_route':>10} {'T_fused':>10}")
    for s in strategies:
        r = results[s]
        print(f"{s:<14} {r[0]:10.3f} {r[1]:10.3f} {r[2]:10.3f} {r[3]:10.3f} {r[4]:10.3f}")
    print(json.dumps({s: dict(zip(("t_logit_ms", "t_select_ms", "t_pack_ms", "t_route_ms", "t_fused_ms"), results[s]))
                      for s in strategies}))


if __name__ == "__main__":
    main()
