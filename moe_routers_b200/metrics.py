"""Routing metrics of the MoE block: the twelve names the reference's `models/decoder_moe.py:22-35`
imports from `models/metrics.py`.

That file is missing from the reference tree, so the records and helpers here are written from how
`MoELayer.forward` uses them (models/decoder_moe.py:283-348): the field names and the call
signatures are the reference's, the helper bodies are the standard definitions their names state
(each docstring gives the formula).  Helpers take torch tensors on any device and reduce there; only
the final scalars cross to the host.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class PerformanceEfficiencyMetrics:
    """Filled at models/decoder_moe.py:305-311."""
    tokens: int
    total_moe_ms: float
    router_ms: float
    expert_ms: float
    token_latency_us: float


@dataclass
class RoutingBehaviorMetrics:
    """Filled at models/decoder_moe.py:312-319."""
    routing_entropy: float
    normalized_entropy: float
    mean_topk_probability: float
    top1_route_fraction: float
    route_distribution: torch.Tensor
    per_token_prob_sample: Optional[torch.Tensor]


@dataclass
class ExpertUsageMetrics:
    """Filled at models/decoder_moe.py:320-333."""
    active_experts: int
    active_expert_fraction: float
    avg_active_experts_per_token: float
    load_mean_routes: float
    load_std_routes: float
    load_cv: float
    load_max_over_mean: float
    load_min_over_mean: float
    dead_experts: int
    aux_load_balance_loss: float
    unique_tokens_per_expert_mean: Optional[float]
    unique_tokens_per_expert_std: Optional[float]


@dataclass
class MoEMetrics:
    """Filled at models/decoder_moe.py:335-341."""
    router_backend: str
    performance: PerformanceEfficiencyMetrics
    routing: RoutingBehaviorMetrics
    usage: ExpertUsageMetrics
    output: dict


def route_distribution_from_topk(topk_idx: torch.Tensor, n_experts: int) -> torch.Tensor:
    """p[e] = (routes sent to expert e) / (S * K), float32 [E]; zeros when there are no routes."""
    flat = topk_idx.reshape(-1).to(torch.int64)
    counts = torch.bincount(flat, minlength=int(n_experts)).to(torch.float32)
    return counts / float(max(flat.numel(), 1))


def routing_entropy_from_distribution(p: torch.Tensor) -> float:
    """Shannon entropy -sum_e p[e] ln p[e] in nats (0 ln 0 = 0)."""
    p = p.to(torch.float32)
    nz = p > 0
    if not bool(nz.any()):
        return 0.0
    return float(-(p[nz] * p[nz].log()).sum().item())


def normalized_entropy(p: torch.Tensor) -> float:
    """Entropy divided by its maximum ln E (1 = uniform use of the experts)."""
    e = int(p.numel())
    if e <= 1:
        return 0.0
    return routing_entropy_from_distribution(p) / math.log(e)


def mean_topk_probability_from_logits(logits: torch.Tensor, k: int) -> float:
    """Mean over tokens of the full-softmax probability mass that lands on the k selected experts."""
    if logits.numel() == 0:
        return 0.0
    probs = torch.softmax(logits.float(), dim=-1)
    return float(probs.topk(int(k), dim=-1).values.sum(dim=-1).mean().item())


def avg_unique_experts_per_token(topk_idx: torch.Tensor) -> float:
    """Mean number of distinct experts among a token's k picks (k when no pick repeats)."""
    if topk_idx.numel() == 0:
        return 0.0
    s = torch.sort(topk_idx.to(torch.int64), dim=-1).values
    distinct = 1 + (s[:, 1:] != s[:, :-1]).sum(dim=-1)
    return float(distinct.float().mean().item())


def aux_load_balance_loss(*, route_frac: torch.Tensor, importance: torch.Tensor, alpha: float = 1.0) -> float:
    """Switch-Transformer auxiliary loss alpha * E * sum_e f[e] * P[e]: f = fraction of routes per
    expert, P = mean full-softmax probability per expert; 1.0 * alpha for perfectly uniform routing."""
    e = int(route_frac.numel())
    return float(alpha * e * (route_frac.to(torch.float32) * importance.to(torch.float32)).sum().item())


def unique_tokens_per_expert(topk_idx: torch.Tensor, n_experts: int):
    """(mean, population std) over experts of the number of distinct tokens routed to each expert;
    None when there are no tokens."""
    if topk_idx.numel() == 0:
        return None
    s_, _k = topk_idx.shape
    hit = torch.zeros((s_, int(n_experts)), dtype=torch.bool, device=topk_idx.device)
    hit.scatter_(1, topk_idx.to(torch.int64), True)
    per_expert = hit.sum(dim=0).to(torch.float32)
    return float(per_expert.mean().item()), float(per_expert.std(unbiased=False).item())


def output_distribution_stats(out: torch.Tensor) -> dict:
    """Summary of the block's output values: mean, std, abs-mean, abs-max, fraction of exact zeros."""
    if out.numel() == 0:
        return dict(mean=0.0, std=0.0, abs_mean=0.0, abs_max=0.0, zero_fraction=0.0)
    o = out.float()
    return dict(mean=float(o.mean().item()), std=float(o.std(unbiased=False).item()),
                abs_mean=float(o.abs().mean().item()), abs_max=float(o.abs().max().item()),
                zero_fraction=float((o == 0).float().mean().item()))
