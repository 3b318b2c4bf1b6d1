"""CPU (torch) port of the reference's CPU routing path, used as the timed CPU baseline.

TEST / BENCHMARK INFRASTRUCTURE ONLY (see the package docstring).  It restates
the CPU branch of santiweide/moe-routers `bench_router.py:484-505` with its
pack `_pack_routes` (`bench_router.py:57-78`) and the routers
`TorchTopKRouter` / `SinkhornRouter` (`models/decoder_moe.py:58-62`, `:92-123`)
using the same torch operators, so that its run time on the host cores is the
reference's CPU figure for the same inputs.
"""
from __future__ import annotations

import time

import torch


def pack_routes(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor):
    """bench_router.py:57-78: gate-weighted gather, argsort by expert, three gathers."""
    s, k = topk_idx.shape
    token_ids = torch.arange(s, dtype=torch.int64).unsqueeze(1).expand(s, k).reshape(-1)
    expert_ids = topk_idx.reshape(-1).to(torch.int64)
    weights = topk_w.reshape(-1).unsqueeze(-1)
    x_route = x.index_select(0, token_ids) * weights
    sort_idx = torch.argsort(expert_ids)
    return (x_route.index_select(0, sort_idx), token_ids.index_select(0, sort_idx),
            expert_ids.index_select(0, sort_idx))


def sinkhorn_router(logits: torch.Tensor, top_k: int, iters: int = 10, eps: float = 1e-6, temperature: float = 1.0):
    """models/decoder_moe.py:92-123."""
    s, e = logits.shape
    scores = (logits / temperature).float()
    scores = scores - scores.max(dim=-1, keepdim=True).values
    q = torch.exp(scores)
    col_target = float(s) / float(max(e, 1))
    for _ in range(iters):
        q = q / (q.sum(dim=1, keepdim=True) + eps)
        q = q / (q.sum(dim=0, keepdim=True) + eps) * col_target
    q = q / (q.sum(dim=1, keepdim=True) + eps)
    vals, idx = torch.topk(q, k=top_k, dim=-1)
    w = vals / (vals.sum(dim=-1, keepdim=True) + eps)
    return idx.to(torch.int64), w.to(dtype=logits.dtype)


def one_iter(x: torch.Tensor, w: torch.Tensor, top_k: int, *, strategy: str = "naive_topk",
             skew_experts: int = 0, skew_bias: float = 0.0):
    """One timed iteration of bench_router.py:484-505.  Returns (t_logit, t_select, t_pack, t_route) in ms."""
    t0 = time.perf_counter()
    logits = x.float() @ w.float().t()
    t1 = time.perf_counter()
    if skew_experts > 0 and skew_bias != 0.0:
        logits[:, :skew_experts] += skew_bias
    if strategy == "sinkhorn":
        topk_idx, topk_w = sinkhorn_router(logits, top_k)
    else:  # naive_topk; the reference's CPU branch runs fused_select as naive_topk too (:498-501)
        vals, topk_idx = torch.topk(logits, k=top_k, dim=-1)
        topk_w = torch.softmax(vals, dim=-1)
    t2 = time.perf_counter()
    pack_routes(x, topk_idx, topk_w)
    t3 = time.perf_counter()
    return (t1 - t0) * 1e3, (t2 - t1) * 1e3, (t3 - t2) * 1e3, (t3 - t0) * 1e3
