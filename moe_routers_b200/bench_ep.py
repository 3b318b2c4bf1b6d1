"""Expert-parallel MoE layer benchmark (one process per GPU, NCCL).

Mirrors the reference's `bench_2gpu_pcie.py` (flags :175-206, timing :424-599, table :637-673) for
any world size that divides the expert count, with the combine all-to-all and gate-weighted sum the
reference leaves out:

    torchrun --nproc_per_node W -m moe_routers_b200.bench_ep --all_strategies --skew_experts 8 --skew_bias 2.0

Per strategy, per iteration (forward only), times in microseconds, max over ranks:
    T_route      route (logit GEMM + select + pack), one fused call; with the direct dispatch the rows
                 are copied by the dispatch itself (T_comm) and T_route is GEMM + select + pack plan
    T_comm       dispatch + combine exchanges, run alone
    T_comp       expert FFN on own rows + on received rows (with re-bucketing), run alone
    T_layer(seq) the whole layer as a serial chain: local pack, dispatch exchange, rank sync, expert FFN,
                 combine exchange, rank sync, gate-weighted sum (peer transport: separate push kernels;
                 nccl transport: every stage on one stream)
    T_layer(ovl) the whole layer with the exchanges overlapped with compute (peer transport: the pack
                 stores into the owners' inboxes and the second expert GEMM stores its rows into their
                 home slots, tile by tile; nccl transport: exchanges on a second stream)
    T_layer(b2b) the layer called `iters` times back to back, per call (no host sync in between)
    eta_overlap  (T_route + T_comm + T_comp + T_combine) / T_layer(ovl)      (bench_2gpu_pcie.py:586);
                 eta_seq_over_overlap = T_layer(seq) / T_layer(ovl) compares the two executions directly
    load max/mean and CV of the per-expert route counts over all ranks       (:446-457)
Each expert is a 2-layer GELU FFN d_model -> hidden -> d_model with N(0, 1/fan_in) weights.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _event_us(fn, stream=None) -> float:
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    fn()
    e.record()
    torch.cuda.synchronize()
    return float(s.elapsed_time(e)) * 1000.0


def run(args) -> list[dict]:
    from . import ops
    from .ep import EPMoELayer

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    e, k, d, h, t = args.experts, args.top_k, args.d_model, args.hidden, args.tokens
    if e % world != 0:
        raise ValueError("experts must be divisible by world_size")
    el = e // world
    dtype = {"fp16": torch.float16, "bf16": torch.bfloat16}[getattr(args, "dtype", "fp16")]
    g = torch.Generator(device=dev).manual_seed(0)  # router and expert weights: same seed on every rank
    w_router = (torch.randn(e, d, device=dev, generator=g) / d ** 0.5).to(dtype)
    gl = torch.Generator(device=dev).manual_seed(1000 + rank)
    w1 = (torch.randn(el, h, d, device=dev, generator=gl) / d ** 0.5).to(dtype)
    w2 = (torch.randn(el, d, h, device=dev, generator=gl) / h ** 0.5).to(dtype)
    x = torch.randn(t, d, device=dev, generator=gl).to(dtype)  # tokens differ per rank

    strategies = ["naive_topk", "fused_select", "sinkhorn"] if args.all_strategies else (args.strategies or [args.strategy])
    results = []
    for strategy in strategies:
        transport = getattr(args, "transport", "peer")
        layer = EPMoELayer(w_router, w1, w2, k, activation="gelu", strategy=strategy,
                           sinkhorn_iters=args.sinkhorn_iters, sinkhorn_temperature=args.sinkhorn_temperature,
                           skew_experts=args.skew_experts, skew_bias=args.skew_bias, transport=transport)
        layer.fuse_combine = not getattr(args, "no_fuse_combine", False)
        layer.direct_dispatch = not getattr(args, "no_direct_dispatch", False)
        dist.barrier()
        for _ in range(args.warmup):
            layer(x, overlap=True)
            layer(x, overlap=False)
        torch.cuda.synchronize()

        # ---- stage timings, each stage alone on the main stream ----
        acc = dict(route=0.0, comm=0.0, comp=0.0, combine=0.0, seq=0.0, ovl=0.0)
        for _ in range(args.iters):
            out = {}
            direct = transport == "peer" and layer.direct_dispatch
            acc["route"] += _event_us(lambda: out.update(o=layer.route_select(x) if direct else layer.route(x)))
            o = out["o"]
            if transport == "peer":
                pr = layer._peer
                layer._calls += 1
                call = layer._calls
                counts_all = layer.exchange_counts_peer(o["counts"], call)
                y_packed = pr["y_home"][:x.size(0) * k]

                fused = layer.fuse_combine
                targets = layer._row_targets(counts_all) if fused else None

                def comm():  # with the fused return, the result rows travel inside comp()
                    if direct:
                        layer.dispatch_direct(x, o, counts_all)
                    else:
                        layer._push(o["packed"], pr["inbox_ptrs"], counts_all, False, pr["offsets"])
                    layer._rank_sync(1, call)
                    if not fused:
                        layer._push(pr["yb"], pr["home_ptrs"], counts_all, True, None)
                    layer._rank_sync(2, call)

                def comp():
                    layer._ffn(pr["inbox"], pr["offsets"], None if fused else pr["yb"], out_rows=targets)
            else:
                counts_all, counts_host = layer.exchange_counts(o["counts"])
                pl = layer.plan(o, counts_all, counts_host, 1)
                y_packed = pl["y_packed"]

                def comm():
                    layer.dispatch(pl, 0)
                    layer.give_back(pl, 0)

                def comp():
                    layer.compute(pl, 0)

            dist.barrier()
            acc["comm"] += _event_us(comm)
            acc["comp"] += _event_us(comp)
            acc["combine"] += _event_us(lambda: ops.combine(y_packed, o["gates"], o["route_row"], k))
            dist.barrier()
            acc["seq"] += _event_us(lambda: layer(x, overlap=False))
            dist.barrier()
            acc["ovl"] += _event_us(lambda: layer(x, overlap=True))
        # the layer called back to back (one event pair around all calls, no host synchronisation in
        # between): the host's launch work hides behind the previous call's expert GEMMs, as it does
        # inside a multi-layer model
        batches = []
        for _ in range(3):  # median of three batches: one disturbed batch does not decide the figure
            dist.barrier()
            batches.append(_event_us(lambda: [layer(x, overlap=True) for _ in range(args.iters)]))
        acc["b2b"] = sorted(batches)[1]
        vals = torch.tensor([acc[n] / args.iters for n in ("route", "comm", "comp", "combine", "seq", "ovl", "b2b")],
                            device=dev, dtype=torch.float64)
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        t_route, t_comm, t_comp, t_combine, t_seq, t_ovl, t_b2b = [float(v) for v in vals.tolist()]

        counts_rk = layer.last["counts_all"] if "counts_all" in layer.last else layer.last["counts_dev"].cpu()
        counts = counts_rk.sum(dim=0).to(torch.float32)  # aggregated over ranks
        mean = float(counts.mean())
        results.append(dict(
            strategy=strategy, world=world, tokens_per_rank=t, d_model=d, hidden=h, experts=e, top_k=k,
            skew_experts=args.skew_experts, skew_bias=args.skew_bias,
            t_route_us=t_route, t_comm_us=t_comm, t_comp_us=t_comp, t_combine_us=t_combine,
            t_layer_seq_us=t_seq, t_layer_overlap_us=t_ovl, t_layer_back_to_back_us=t_b2b,
            eta_overlap=(t_route + t_comm + t_comp + t_combine) / max(t_ovl, 1e-6),
            eta_seq_over_overlap=t_seq / max(t_ovl, 1e-6),
            load_max_over_mean=float(counts.max() / (mean + 1e-9)),
            load_cv=float(counts.std(unbiased=False) / (mean + 1e-9)),
            transport=transport, direct_dispatch=bool(layer.direct_dispatch) if transport == "peer" else None,
            fuse_combine=bool(layer.fuse_combine) if transport == "peer" else None,
            rows_received_rank0=int(counts_rk[:, :el].sum()) if rank == 0 else None,
            tokens_per_s=world * t / (t_ovl * 1e-6), tokens_per_s_back_to_back=world * t / (t_b2b * 1e-6),
        ))
        layer.close()
    return results


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--dtype", type=str, default="fp16", choices=["fp16", "bf16"])
    p.add_argument("--tokens", type=int, default=4096, help="T (tokens per rank)")
    p.add_argument("--d_model", type=int, default=4096)
    p.add_argument("--hidden", type=int, default=8192)
    p.add_argument("--experts", type=int, default=64, help="E (global experts)")
    p.add_argument("--top_k", type=int, default=2)
    p.add_argument("--strategies", type=str, nargs="+", default=None)
    p.add_argument("--all_strategies", action="store_true")
    p.add_argument("--strategy", type=str, default="fused_select", choices=["naive_topk", "fused_select", "sinkhorn"])
    p.add_argument("--sinkhorn_iters", type=int, default=10)
    p.add_argument("--sinkhorn_temperature", type=float, default=1.0)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--skew_experts", type=int, default=0)
    p.add_argument("--skew_bias", type=float, default=0.0)
    p.add_argument("--transport", type=str, default="peer", choices=["peer", "nccl"],
                   help="peer: device-initiated stores into the owner's inbox over NVLink; nccl: grouped send/recv")
    p.add_argument("--no_fuse_combine", action="store_true",
                   help="peer transport: dense FFN result + a separate return push instead of the GEMM that returns its rows")
    p.add_argument("--no_direct_dispatch", action="store_true",
                   help="peer transport: pack locally and push, instead of the pack that stores into the owners' inboxes")
    p.add_argument("--json", type=str, default=None, help="also write the results to this file (rank 0)")
    args = p.parse_args()

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        results = run(args)
        if dist.get_rank() == 0:
            print("=== EP MoE layer (us, mean over iters, max over ranks) ===")
            print(f"{'strategy':<13}{'T_route':>9}{'T_comm':>9}{'T_comp':>10}{'T_comb':>8}{'T(seq)':>10}{'T(ovl)':>10}{'T(b2b)':>10}"
                  f"{'eta':>6}{'max/mean':>9}{'CV':>6}")
            for r in results:
                print(f"{r['strategy']:<13}{r['t_route_us']:9.1f}{r['t_comm_us']:9.1f}{r['t_comp_us']:10.1f}"
                      f"{r['t_combine_us']:8.1f}{r['t_layer_seq_us']:10.1f}{r['t_layer_overlap_us']:10.1f}"
                      f"{r['t_layer_back_to_back_us']:10.1f}"
                      f"{r['eta_overlap']:6.2f}{r['load_max_over_mean']:9.2f}{r['load_cv']:6.2f}")
            for r in results:
                print(json.dumps(r))
            if args.json:
                with open(args.json, "w") as f:
                    json.dump(results, f, indent=1)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
