"""Small single-GPU drivers sized for profiler captures (a few launches, at most ~5 GB on the device).

    python -m moe_routers_b200.profile_cases --case route   # 3 fused routes (L2 flushed between), combine, Sinkhorn
    python -m moe_routers_b200.profile_cases --case ffn     # grouped expert GEMM: 3 x (8 experts x 1024 rows), 2 x (64 x 128)

Shapes are the benchmark's: T=4096 tokens, d_model=4096, hidden=8192, E=64, top_k=2, fp16.
"""
from __future__ import annotations

import argparse

import torch


def case_route() -> None:
    from . import ops

    t, d, e, k = 4096, 4096, 64, 2
    x = torch.randn(t, d, device="cuda").half()
    w = (torch.randn(e, d, device="cuda") / 64).half()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2
    o = ops.route_fused(x, w, k, skew_experts=8, skew_bias=2.0)
    for _ in range(2):
        flush.zero_()
        ops.route_fused(x, w, k, skew_experts=8, skew_bias=2.0, out=o)
    flush.zero_()
    ops.combine(o["packed"], o["gates"], o["route_row"], k)
    ops.sinkhorn(x @ w.t(), k)


def case_ffn() -> None:
    from . import ops

    d, h = 4096, 8192
    x = torch.randn(8192, d, device="cuda").half()
    w1 = (torch.randn(8, h, d, device="cuda") / 64).half()
    off = torch.arange(0, 8193, 1024, device="cuda", dtype=torch.int32)
    for _ in range(3):  # tensor-bound: 8 experts x 1024 rows (two-CTA kernel)
        ops.grouped_gemm(x, w1, off, layout="nk", activation="gelu")
    del w1
    w1b = (torch.randn(64, h, d, device="cuda") / 64).half()
    off2 = torch.arange(0, 8193, 128, device="cuda", dtype=torch.int32)
    for _ in range(2):  # weight-bound: 64 experts x 128 rows
        ops.grouped_gemm(x, w1b, off2, layout="nk", activation="gelu")


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--case", choices=["route", "ffn"], required=True)
    args = p.parse_args()
    torch.manual_seed(0)
    {"route": case_route, "ffn": case_ffn}[args.case]()
    torch.cuda.synchronize()
    from . import ops

    assert ops.read_status() == 0
    print("ok")


if __name__ == "__main__":
    main()
