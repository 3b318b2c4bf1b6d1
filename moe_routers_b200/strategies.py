"""The four routing strategies of the reference's router benchmark (bench_router.py:434-438,
:468) as functions over the CUDA kernels: naive_topk, masked_matmul (A), fused_select (B),
sinkhorn (C).  Each returns the routing of a batch; `moe_forward` / `masked_matmul_forward` run
the expert FFNs on it (2-layer GELU FFN, weights [E, h, d] and [E, d, h])."""
from __future__ import annotations

import torch

from . import ops

STRATEGIES = ["naive_topk", "masked_matmul", "fused_select", "sinkhorn"]


def route(strategy: str, x: torch.Tensor, w_router: torch.Tensor, top_k: int, *, skew_experts: int = 0,
          skew_bias: float = 0.0, sinkhorn_iters: int = 10, sinkhorn_temperature: float = 1.0):
    """Routing of `x` under `strategy`.  Returns a dict with idx / gates and, for the strategies that
    permute (all but masked_matmul), counts / offsets / packed / row_route / route_row."""
    e = w_router.size(0)
    if strategy not in STRATEGIES:
        raise ValueError(f"Unknown strategies: {[strategy]}. Valid: {STRATEGIES}")
    if strategy == "fused_select":
        return ops.route_fused(x, w_router, top_k, skew_experts=skew_experts, skew_bias=skew_bias)
    if strategy == "naive_topk":
        # the same selection as fused_select (top-k of the logits, lowest index wins ties) with the
        # logits written out as well, as torch.topk on materialised logits would need them
        return ops.route_fused(x, w_router, top_k, skew_experts=skew_experts, skew_bias=skew_bias, return_logits=True)
    idx, gates, logits = ops.router_gemm_select(x, w_router, top_k, skew_experts=skew_experts,
                                                skew_bias=skew_bias, return_logits=True)
    if strategy == "sinkhorn":
        idx, gates = ops.sinkhorn(logits, top_k, iters=sinkhorn_iters, temperature=sinkhorn_temperature)
    out = dict(idx=idx, gates=gates, logits=logits)
    if strategy == "masked_matmul":
        return out  # Strategy A: no permutation
    counts, offsets, packed, row_route, route_row = ops.pack(x, idx, e)
    out.update(counts=counts, offsets=offsets, packed=packed, row_route=row_route, route_row=route_row)
    return out


def moe_forward(r: dict, w1: torch.Tensor, w2: torch.Tensor, top_k: int, activation: str = "gelu") -> torch.Tensor:
    """Sparse layer output from a routing with a packed buffer: grouped FFN + gate-weighted combine."""
    h = ops.grouped_gemm(r["packed"], w1, r["offsets"], layout="nk", activation=activation)
    y = ops.grouped_gemm(h, w2, r["offsets"], layout="nk")
    return ops.combine(y, r["gates"], r["route_row"], top_k)


def masked_matmul_forward(x: torch.Tensor, r: dict, w1: torch.Tensor, w2: torch.Tensor, top_k: int,
                          activation: str = "gelu") -> torch.Tensor:
    """Strategy A: every expert runs densely over ALL tokens; outputs are summed with the top-k gate
    as mask (zero for unselected experts).  No permutation; E times the FLOPs of the sparse layer.
    Limited to 8 experts (the combine kernel sums at most 8 rows per token)."""
    t, d = x.shape
    e = w1.size(0)
    if e > 8:
        raise RuntimeError("masked_matmul_forward supports at most 8 experts")
    dev = x.device
    seg = _one_segment(t, dev)
    y = torch.empty((e * t, d), dtype=x.dtype, device=dev)
    for ex in range(e):  # one dense GEMM pair per expert, no host synchronisation
        h = ops.grouped_gemm(x, w1[ex:ex + 1], seg, layout="nk", activation=activation)
        ops.grouped_gemm(h, w2[ex:ex + 1], seg, layout="nk", out=y[ex * t:(ex + 1) * t])
    # the combine kernel sums E rows per token: dense gates [T, E] (zero for unselected experts) and the
    # row of expert ex's result for token t, ex * T + t (a constant table, built once per shape)
    dense = torch.zeros((t, e), dtype=torch.float32, device=dev)
    dense.scatter_add_(1, r["idx"].long(), r["gates"])
    return ops.combine(y, dense, _dense_rows(t, e, dev), e)


_dense_rows_cache: dict = {}


def _dense_rows(t: int, e: int, dev) -> torch.Tensor:
    """int32 [t * e]: entry t * e + ex = ex * t + t_index, built once per (t, e, device)."""
    key = (t, e, dev)
    rows = _dense_rows_cache.get(key)
    if rows is None:
        rows = (torch.arange(e, device=dev, dtype=torch.int32).view(1, e) * t
                + torch.arange(t, device=dev, dtype=torch.int32).view(t, 1)).contiguous().view(-1)
        _dense_rows_cache[key] = rows
    return rows


_segment_cache: dict = {}


def _one_segment(t: int, dev) -> torch.Tensor:
    """offsets [0, t] of a single expert segment on `dev`, uploaded once per (t, device)."""
    key = (t, dev)
    seg = _segment_cache.get(key)
    if seg is None:
        seg = _segment_cache[key] = torch.tensor([0, t], dtype=torch.int32, device=dev)
    return seg


def _token_ids(t: int, dev) -> torch.Tensor:
    """int32 [t, 1] column 0..t-1 on `dev`, built once per (t, device)."""
    key = (t, dev)
    ids = _token_id_cache.get(key)
    if ids is None:
        ids = _token_id_cache[key] = torch.arange(t, device=dev, dtype=torch.int32).view(t, 1)
    return ids
