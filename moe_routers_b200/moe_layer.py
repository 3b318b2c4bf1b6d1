"""Drop-in for the reference's MoE block (models/decoder_moe.py:154-350).

Same constructor, attributes (`router`, `experts[i].w1/.w3/.w2`, `router_impl`,
`track_metrics`), `forward(x[B,T,d]) -> [B,T,d]` and `get_last_metrics()`.  The
forward body is the fused B200 path:

    route (logit GEMM + select + pack)  ->  grouped SwiGLU GEMM  ->  grouped down GEMM
    ->  gate-weighted combine

instead of `index_select` / `argsort` / a Python loop with one `.item()` sync per
expert / `index_add_`.  It runs in fp16 or bf16 on CUDA only.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
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

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        bsz, seq_len, d_model = x.shape
        if not x.is_cuda:
            raise RuntimeError("inputs must be CUDA")
        if x.dtype not in (torch.float16, torch.bfloat16) or self.router.weight.dtype != x.dtype:
            raise RuntimeError("x and the layer's weights must both be fp16 (Half) or both bf16")
        flat = x.reshape(-1, d_model)
        e, k = self.n_experts, self.top_k
        fused = type(self.router_impl) is CUDATopKRouter and e <= 256 and k <= 8 and d_model % 8 == 0
        if fused:
            o = ops.route_fused(flat, self.router.weight, k)
            gates, packed, offsets, route_row, counts = o["gates"], o["packed"], o["offsets"], o["route_row"], o["counts"]
        else:
            logits = self.router(flat)
            topk_idx, topk_w = self.router_impl(logits, k)
            gates = topk_w.float()
            counts, offsets, packed, _row_route, route_row = ops.pack(flat, topk_idx.to(torch.int32), e)
        w13, w2 = self._stacked_weights()
        h = ops.grouped_gemm(packed, w13, offsets, layout="nk", activation="swiglu")
        y = ops.grouped_gemm(h, w2, offsets, layout="nk")
        out = ops.combine(y, gates, route_row, k)
        if self.track_metrics:
            c = counts.float()
            mean = float(c.mean().item())
            self._last_metrics = {
                "router_backend": self.router_impl.name,
                "tokens": int(flat.size(0)),
                "load_cv": float(c.std(unbiased=False).item() / (mean + 1e-9)),
                "load_max_over_mean": float(c.max().item() / (mean + 1e-9)),
                "active_experts": int((c > 0).sum().item()),
                "route_counts": counts.cpu(),
            }
        return out.view(bsz, seq_len, d_model)
