"""Drop-in for the reference's MoE block (models/decoder_moe.py:154-350).

Same constructor, attributes (`router`, `experts[i].w1/.w3/.w2`, `router_impl`,
`track_metrics`), `forward(x[B,T,d]) -> [B,T,d]` and `get_last_metrics()`.  The
forward body is the fused B200 path:

    route (logit GEMM + select + pack)  ->  grouped SwiGLU GEMM  ->  grouped down GEMM
    ->  gate-weighted combine

instead of `index_select` / `argsort` / a Python loop with one `.item()` sync per
expert / `index_add_`.  It runs in fp16 or bf16 on CUDA only, and it is forward-only
(inference): the kernels record nothing for autograd, so a call that would need
gradients raises.  `DecoderMoEBlock` wraps the layer as models/decoder_moe.py:353-391
does, around any attention / norm modules the caller supplies.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .metrics import (ExpertUsageMetrics, MoEMetrics, PerformanceEfficiencyMetrics, RoutingBehaviorMetrics,
                      aux_load_balance_loss, avg_unique_experts_per_token, mean_topk_probability_from_logits,
                      normalized_entropy, output_distribution_stats, routing_entropy_from_distribution,
                      unique_tokens_per_expert)
from .routers import CUDATopKRouter, RouterBase


class SwiGLU(torch.nn.Module):
    """SwiGLU MLP: silu(W1 x) * (W3 x) -> W2 (models/transformer_decoder_model.py:162-172)."""

    def __init__(self, d_model: int, hidden_dim: int):
        super().__init__()
        self.w1 = torch.nn.Linear(d_model, hidden_dim, bias=False)  # gate
        self.w3 = torch.nn.Linear(d_model, hidden_dim, bias=False)  # up
        self.w2 = torch.nn.Linear(hidden_dim, d_model, bias=False)  # down

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        flat = x.reshape(-1, x.size(-1))
        off = torch.tensor([0, flat.size(0)], dtype=torch.int32, device=flat.device)
        w13 = torch.cat([self.w1.weight, self.w3.weight], dim=0).unsqueeze(0)
        h = ops.grouped_gemm(flat, w13, off, layout="nk", activation="swiglu")
        y = ops.grouped_gemm(h, self.w2.weight.unsqueeze(0), off, layout="nk")
        return y.view(*x.shape[:-1], y.size(-1))


class MoELayer(torch.nn.Module):
    """Token-level MoE with top-k routing on the fused B200 path."""

    def __init__(self, d_model: int, expert_hidden_dim: int, n_experts: int, top_k: int = 2, *,
                 router_impl: Optional[RouterBase] = None, track_metrics: bool = False):
        super().__init__()
        if n_experts <= 0:
            raise ValueError("n_experts must be > 0")
        if top_k <= 0:
            raise ValueError("top_k must be > 0")
        if top_k > n_experts:
            raise ValueError("top_k must be <= n_experts")
        self.n_experts = n_experts
        self.top_k = top_k
        self.router = torch.nn.Linear(d_model, n_experts, bias=False)
        self.router_impl: RouterBase = router_impl if router_impl is not None else CUDATopKRouter()
        self.track_metrics = track_metrics
        self._last_metrics = None
        self.experts = torch.nn.ModuleList(
            [SwiGLU(d_model=d_model, hidden_dim=expert_hidden_dim) for _ in range(n_experts)]
        )
        self._stacked = None
        self._stacked_key = None

    def get_last_metrics(self):
        return self._last_metrics

    def _stacked_weights(self):
        """[E, 2h, d] (gate rows, then up rows) and [E, d, h], rebuilt when a parameter changes."""
        params = [p for ex in self.experts for p in (ex.w1.weight, ex.w3.weight, ex.w2.weight)]
        key = tuple((p.data_ptr(), p._version) for p in params)
        if self._stacked is None or key != self._stacked_key:
            w13 = torch.stack([torch.cat([ex.w1.weight, ex.w3.weight], dim=0) for ex in self.experts]).contiguous()
            w2 = torch.stack([ex.w2.weight for ex in self.experts]).contiguous()
            self._stacked = (w13.detach(), w2.detach())
            self._stacked_key = key
        return self._stacked

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Forward only: the kernels record nothing for autograd.  Called with gradients enabled on a
        tensor or parameters that require them, the layer refuses instead of silently returning an
        output without a grad_fn (the reference layer is trainable through index_select/index_add_)."""
        if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters())):
            raise RuntimeError("moe_routers_b200.MoELayer is forward-only: call it under torch.no_grad() "
                               "(or set requires_grad_(False) on the module and its input)")
        with torch.no_grad():
            return self._forward(x)

    def _forward(self, x: torch.Tensor) -> torch.Tensor:
        bsz, seq_len, d_model = x.shape
        if not x.is_cuda:
            raise RuntimeError("inputs must be CUDA")
        if x.dtype not in (torch.float16, torch.bfloat16) or self.router.weight.dtype != x.dtype:
            raise RuntimeError("x and the layer's weights must both be fp16 (Half) or both bf16")
        flat = x.reshape(-1, d_model)
        e, k = self.n_experts, self.top_k
        track = self.track_metrics
        if track:  # same event layout as models/decoder_moe.py:222-235, :277-281
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
        kernel_gemm = e <= 256 and k <= 8 and d_model % 8 == 0
        fused = type(self.router_impl) is CUDATopKRouter and kernel_gemm
        logits = None
        if fused:
            o = ops.route_fused(flat, self.router.weight, k, return_logits=track)
            gates, packed, offsets, route_row, counts = o["gates"], o["packed"], o["offsets"], o["route_row"], o["counts"]
            topk_idx = o["idx"]
            logits = o.get("logits") if track else None
        else:
            if kernel_gemm:
                # the logits of the tcgen05 router kernel (values already rounded to the layer's dtype)
                _i, _g, lg32 = ops.router_gemm_select(flat, self.router.weight, k, return_logits=True)
                logits = lg32.to(x.dtype)
            else:  # more than 256 experts: outside the router kernel's tile shapes
                logits = self.router(flat)
            topk_idx, topk_w = self.router_impl(logits, k)
            gates = topk_w.float()
            counts, offsets, packed, _row_route, route_row = ops.pack(flat, topk_idx.to(torch.int32), e)
        if track:
            ev[1].record()
        w13, w2 = self._stacked_weights()
        h = ops.grouped_gemm(packed, w13, offsets, layout="nk", activation="swiglu")
        y = ops.grouped_gemm(h, w2, offsets, layout="nk")
        out = ops.combine(y, gates, route_row, k)
        if track:
            ev[2].record()
            torch.cuda.synchronize()
            self._last_metrics = self._metrics(flat, logits, topk_idx, counts, out,
                                               total_ms=float(ev[0].elapsed_time(ev[2])),
                                               router_ms=float(ev[0].elapsed_time(ev[1])),
                                               expert_ms=float(ev[1].elapsed_time(ev[2])))
        return out.view(bsz, seq_len, d_model)

    def _metrics(self, flat, logits, topk_idx, counts, out, *, total_ms, router_ms, expert_ms) -> MoEMetrics:
        """The record of models/decoder_moe.py:283-348, reduced on the device from the route's own
        counts and indices.  `router_ms` covers the whole fused route (logit GEMM + select + pack are
        one operator here; the reference times the select alone), `expert_ms` the expert GEMMs and
        the combine."""
        s, k, e = int(flat.size(0)), self.top_k, self.n_experts
        topk_i64 = topk_idx.to(torch.int64)
        counts_f = counts.to(torch.float32)
        p_route = counts_f / float(max(s * k, 1))
        load_mean = float(counts_f.mean().item()) if e else 0.0
        load_std = float(counts_f.std(unbiased=False).item()) if e else 0.0
        active = int((counts_f > 0).sum().item())
        probs_full = torch.softmax(logits.float(), dim=-1)
        importance = probs_full.mean(dim=0)
        uniq = unique_tokens_per_expert(topk_i64, e)
        perf = PerformanceEfficiencyMetrics(tokens=s, total_moe_ms=total_ms, router_ms=router_ms, expert_ms=expert_ms,
                                            token_latency_us=total_ms * 1000.0 / max(s, 1))
        routing = RoutingBehaviorMetrics(
            routing_entropy=routing_entropy_from_distribution(p_route),
            normalized_entropy=normalized_entropy(p_route),
            mean_topk_probability=mean_topk_probability_from_logits(logits, k),
            top1_route_fraction=float(p_route.max().item()) if e else 0.0,
            route_distribution=p_route.detach().cpu(),
            per_token_prob_sample=probs_full[0].detach().cpu() if probs_full.numel() else None)
        usage = ExpertUsageMetrics(
            active_experts=active, active_expert_fraction=active / max(e, 1),
            avg_active_experts_per_token=avg_unique_experts_per_token(topk_i64),
            load_mean_routes=load_mean, load_std_routes=load_std, load_cv=load_std / (load_mean + 1e-9),
            load_max_over_mean=float(counts_f.max().item() / (load_mean + 1e-9)) if e else 0.0,
            load_min_over_mean=float(counts_f.min().item() / (load_mean + 1e-9)) if e else 0.0,
            dead_experts=e - active,
            aux_load_balance_loss=aux_load_balance_loss(route_frac=p_route, importance=importance, alpha=1.0),
            unique_tokens_per_expert_mean=uniq[0] if uniq is not None else None,
            unique_tokens_per_expert_std=uniq[1] if uniq is not None else None)
        return MoEMetrics(router_backend=self.router_impl.name, performance=perf, routing=routing, usage=usage,
                          output=output_distribution_stats(out))


class DecoderMoEBlock(torch.nn.Module):
    """Pre-norm decoder block with the MoE layer in the MLP position: the shape of the reference's
    block (models/decoder_moe.py:353-391), `x + attn(attn_norm(x))` then `x + moe(moe_norm(x))`.
    Attention and the norms are outside the routed path, so the caller supplies them (any modules
    mapping [B,T,d] -> [B,T,d]; the reference's own MaskedSelfAttention / RMSNorm fit as they are);
    `self.moe` is the drop-in layer above."""

    def __init__(self, d_model: int, moe_expert_hidden_dim: int, moe_n_experts: int, moe_top_k: int, *,
                 attn: torch.nn.Module, attn_norm: torch.nn.Module, moe_norm: torch.nn.Module,
                 router_impl: Optional[RouterBase] = None, track_metrics: bool = False):
        super().__init__()
        self.attn_norm = attn_norm
        self.attn = attn
        self.moe_norm = moe_norm
        self.moe = MoELayer(d_model=d_model, expert_hidden_dim=moe_expert_hidden_dim, n_experts=moe_n_experts,
                            top_k=moe_top_k, router_impl=router_impl, track_metrics=track_metrics)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.attn_norm(x))
        x = x + self.moe(self.moe_norm(x))
        return x
