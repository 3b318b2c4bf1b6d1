"""Drop-in for the reference's `fused_select_cuda` extension module.

Same function names, argument meaning, return types and error texts as
kernels/fused_select.cu:203-316 (`fused_select_forward`) and as the call site
models/decoder_moe.py:150 (`forward(logits, k)`), backed by libmoe_b200.so.
Differences, all deliberate: work is enqueued on the CURRENT stream (the
reference uses the default stream), there is no host synchronisation, ties
resolve to the lowest expert index, and the order inside an expert segment of
`packed` is ascending token id instead of atomic-slot order.
"""
from __future__ import annotations

import torch

from . import ops

E = 64  # kernels/fused_select.cu:20
K = 2   # kernels/fused_select.cu:21


def forward(logits: torch.Tensor, top_k: int):
    """(idx int32 [S,k], w float32 [S,k]); k <= 8, logits fp16/bf16/fp32 on CUDA."""
    if not logits.is_cuda:
        raise RuntimeError("inputs must be CUDA")
    return ops.topk_select(logits, int(top_k))


def fused_select_forward(logits: torch.Tensor, x: torch.Tensor):
    """Fused Top2-Select + Count/Scan + Pack (E=64, k=2, x=half, logits=half/bf16).

    Returns (idx int32 [T,2], w float32 [T,2], counts int32 [64], offsets int32 [65],
    packed fp16 [2T, d_model]).
    """
    if not (logits.is_cuda and x.is_cuda):
        raise RuntimeError("inputs must be CUDA")
    if x.dtype != torch.float16:
        raise RuntimeError("x must be fp16 (Half)")
    if logits.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("logits must be fp16/bf16")
    if logits.dim() != 2 or logits.size(1) != E:
        raise RuntimeError("logits shape must be [T, 64]")
    if x.dim() != 2 or x.size(0) != logits.size(0):
        raise RuntimeError("x shape must be [T, d_model]")
    if not logits.is_contiguous():
        raise RuntimeError("logits must be contiguous")
    if not x.is_contiguous():
        raise RuntimeError("x must be contiguous")
    if x.size(1) <= 0:
        raise RuntimeError("d_model must be > 0")
    idx, w, counts, offsets, packed, _row_route, _route_row = ops.fused_select(logits, x, E, K)
    return idx, w, counts, offsets, packed


def fused_sinkhorn_forward(logits: torch.Tensor, x: torch.Tensor, sinkhorn_iters: int = 3):
    """The five outputs of kernels/fused_sinkhorn.cu:323-444 (never built in the reference):
    Sinkhorn-balanced top-2 followed by count/scan/pack."""
    if not (logits.is_cuda and x.is_cuda):
        raise RuntimeError("inputs must be CUDA")
    if logits.dim() != 2 or logits.size(1) != E:
        raise RuntimeError("logits shape must be [T, 64]")
    idx, w = ops.sinkhorn(logits, K, iters=int(sinkhorn_iters))
    counts, offsets, packed, _row_route, _route_row = ops.pack(x, idx, E)
    return idx, w, counts, offsets, packed
