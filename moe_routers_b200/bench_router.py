"""Router microbenchmark (single GPU), mirroring the reference's `bench_router.py` breakdown
(:5-9): T_logit, T_select, T_pack, T_route per strategy, with the same flags (:392-446) and the same
printed table (:596-601).

    python -m moe_routers_b200.bench_router --all_strategies --skew_experts 8 --skew_bias 2.0

`--perm_sweep` mirrors the reference's permutation sweep (:284-388): pack latency against batch
size with the DRAM-limit model, written as CSV (no plot).

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

_DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}


def _cuda_time(fn) -> float:
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    fn()
    end.record()
    torch.cuda.synchronize()
    return float(start.elapsed_time(end))


def _torch_pack(x, topk_idx):
    """The reference's sorted pack (bench_router.py:57-78) in torch ops, without the gate multiply:
    a comparison leg of the permutation sweep."""
    s_, k_ = topk_idx.shape
    token_ids = torch.arange(s_, device=x.device, dtype=torch.int64).unsqueeze(1).expand(s_, k_).reshape(-1)
    sort_idx = torch.argsort(topk_idx.reshape(-1).to(torch.int64))
    return x.index_select(0, token_ids).index_select(0, sort_idx)


def _torch_pack_mask_scan(x, topk_idx, n_experts: int):
    """The reference's deliberately naive pack (bench_router.py:81-120): replicate every token once per
    pick, then one boolean-mask pass over all routes per expert and a final concatenation.  Baseline
    leg of the permutation sweep (`t_perm_naive_ms`); torch ops, as in the reference."""
    s_, k_ = topk_idx.shape
    flat_e = topk_idx.reshape(-1).to(torch.int64)
    rows = x.repeat_interleave(k_, dim=0)
    parts = [rows[flat_e == ex] for ex in range(int(n_experts))]
    return torch.cat(parts, dim=0) if parts else rows[:0]


PERM_SWEEP_FIELDS = ["batch_size", "seq_len", "tokens", "experts", "top_k", "d_model", "dtype", "t_perm_naive_ms",
                     "t_perm_sorted_ms", "t_theory_ms", "peak_bw_gbs", "sorted_achieved_bw_gbs",
                     # beyond the reference's columns (bench_router.py:303-316):
                     "t_perm_torch_sorted_ms", "compulsory_bytes"]


def perm_model(tokens: int, top_k: int, d_model: int, elem_bytes: int, peak_bw_gbs: float, t_sorted_ms: float):
    """The reference's DRAM-limit model of a pack (bench_router.py:355-358): one pass reads and writes
    every routed row, ideal_bytes = 2 * R * d * elem with R = tokens * top_k; t_theory = ideal_bytes /
    peak; achieved = ideal_bytes / measured time.  `compulsory_bytes` is the smaller traffic a pack
    that reads each token once really needs, (1 + k) * T * d * elem.  Returns a dict of the derived
    CSV columns."""
    routes = tokens * top_k
    ideal = 2.0 * routes * d_model * elem_bytes
    if peak_bw_gbs is None or peak_bw_gbs <= 0:
        t_theory, achieved = float("nan"), float("nan")
    else:
        t_theory = ideal / (peak_bw_gbs * 1e9) * 1e3
        achieved = ideal / (t_sorted_ms * 1e-3) / 1e9 if t_sorted_ms > 0 else float("nan")
    return dict(t_theory_ms=t_theory, sorted_achieved_bw_gbs=achieved,
                compulsory_bytes=(1 + top_k) * tokens * d_model * elem_bytes)


def write_perm_csv(path: str, rows: list) -> None:
    import csv

    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=PERM_SWEEP_FIELDS)
        w.writeheader()
        w.writerows(rows)


def run_perm_sweep(args) -> None:
    """Permutation latency against batch size with the DRAM-limit model of bench_router.py:284-388:
    random uniform routes; per batch size the naive mask-scan pack (torch), the reference's sorted
    pack (torch) and this library's pack kernel, next to t_theory = 2 * R * d * elem / peak."""
    dev = torch.device("cuda")
    torch.manual_seed(0)
    bw = float(args.peak_bw_gbs) if args.peak_bw_gbs is not None else 6548.8
    dtype = _DTYPES[args.dtype]
    e, k, d = args.experts, args.top_k, args.d_model
    n = max(args.iters, 1)
    rows = []
    for bsz in args.batch_sizes:
        tokens = int(bsz) * int(args.seq_len)
        x = torch.randn(tokens, d, device=dev).to(dtype)
        idx = torch.randint(0, e, (tokens, k), device=dev, dtype=torch.int32)
        for _ in range(args.warmup):
            ops.pack(x, idx, e)
            _torch_pack(x, idx)
            _torch_pack_mask_scan(x, idx, e)
        t_ours = sum(_cuda_time(lambda: ops.pack(x, idx, e)) for _ in range(n)) / n
        t_torch = sum(_cuda_time(lambda: _torch_pack(x, idx)) for _ in range(n)) / n
        t_naive = sum(_cuda_time(lambda: _torch_pack_mask_scan(x, idx, e)) for _ in range(n)) / n
        row = dict(batch_size=int(bsz), seq_len=int(args.seq_len), tokens=tokens, experts=e, top_k=k, d_model=d,
                   dtype=str(dtype).replace("torch.", ""), t_perm_naive_ms=t_naive, t_perm_sorted_ms=t_ours,
                   t_perm_torch_sorted_ms=t_torch, peak_bw_gbs=bw)
        row.update(perm_model(tokens, k, d, x.element_size(), bw, t_ours))
        rows.append(row)
    write_perm_csv(args.csv_out, rows)
    print("perm_sweep: wrote CSV:", args.csv_out)
    for r in rows:
        print(f"B={r['batch_size']:<4d} tokens={r['tokens']:<6d} naive {r['t_perm_naive_ms'] * 1e3:9.1f} us  "
              f"torch sorted {r['t_perm_torch_sorted_ms'] * 1e3:8.1f} us  ours {r['t_perm_sorted_ms'] * 1e3:8.1f} us  "
              f"theory {r['t_theory_ms'] * 1e3:7.1f} us")


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--device", type=str, default="cuda")
    p.add_argument("--dtype", type=str, default="fp16", choices=["fp16", "bf16"])
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
    p.add_argument("--layer", action="store_true",
                   help="Also time the whole MoE layer per strategy (route + 2-layer GELU expert FFN + combine).")
    p.add_argument("--hidden", type=int, default=8192, help="expert hidden size used with --layer")
    p.add_argument("--perm_sweep", action="store_true",
                   help="Sweep batch size and measure the pack (permutation) latency against the DRAM limit.")
    p.add_argument("--batch_sizes", type=int, nargs="+", default=[1, 2, 4, 8, 16, 32, 64])
    p.add_argument("--seq_len", type=int, default=128, help="Used with --perm_sweep: tokens = batch_size * seq_len")
    p.add_argument("--csv_out", type=str, default="perm_efficiency.csv")
    p.add_argument("--peak_bw_gbs", type=float, default=None)
    args = p.parse_args()
    if torch.device(args.device).type != "cuda":
        raise RuntimeError("inputs must be CUDA: this library has no CPU path")
    if args.perm_sweep:
        run_perm_sweep(args)
        return

    torch.manual_seed(0)
    dev = torch.device("cuda")
    dtype = _DTYPES[args.dtype]
    x = torch.randn(args.tokens, args.d_model, device=dev).to(dtype)
    w = (torch.randn(args.experts, args.d_model, device=dev) / args.d_model ** 0.5).to(dtype)
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

    layer_ms = {}
    if args.layer:
        from .strategies import masked_matmul_forward, moe_forward

        h = args.hidden
        w1 = (torch.randn(e, h, args.d_model, device=dev) / args.d_model ** 0.5).to(dtype)
        w2 = (torch.randn(e, args.d_model, h, device=dev) / h ** 0.5).to(dtype)

        def layer_once(strategy):
            r = route(strategy, x, w, k, sinkhorn_iters=args.sinkhorn_iters,
                      sinkhorn_temperature=args.sinkhorn_temperature, **kw)
            if strategy == "masked_matmul":
                return masked_matmul_forward(x, r, w1, w2, k)
            return moe_forward(r, w1, w2, k)

        for s in strategies:
            if s == "masked_matmul" and e > 8:
                continue  # Strategy A is defined for small expert counts (benchmark configuration 3: E=8)
            for _ in range(args.warmup):
                layer_once(s)
            layer_ms[s] = sum(_cuda_time(lambda: layer_once(s)) for _ in range(args.iters)) / max(args.iters, 1)

    print("strategies:", strategies)
    print("device:", dev, "dtype:", dtype)
    print("T(tokens):", args.tokens, "d_model:", args.d_model, "E:", e, "k:", k)
    print("skew_experts:", args.skew_experts, "skew_bias:", args.skew_bias)
    print("")
    print("=== Router Latency Breakdown (ms, mean) ===")
    print(f"{'strategy':<14} {'T_logit':>10} {'T_select':>10} {'T_pack':>10} {'T_route':>10} {'T_fused':>10}")
    for s in strategies:
        r = results[s]
        print(f"{s:<14} {r[0]:10.3f} {r[1]:10.3f} {r[2]:10.3f} {r[3]:10.3f} {r[4]:10.3f}")
    if layer_ms:
        print("")
        print(f"=== MoE layer (route + expert FFN hidden={args.hidden} + combine), ms, mean ===")
        for s, v in layer_ms.items():
            print(f"{s:<14} {v:10.3f}")
    print(json.dumps({s: dict(zip(("t_logit_ms", "t_select_ms", "t_pack_ms", "t_route_ms", "t_fused_ms"), results[s]),
                              t_layer_ms=layer_ms.get(s)) for s in strategies}))


if __name__ == "__main__":
    main()
