"""Drop-in for the reference's `grouped_ffn_cuda` extension module
(kernels/grouped_ffn.cu:53-140): `grouped_ffn_forward(inputs, weights)`.

inputs: list of [M_i, K] fp16 CUDA tensors, weights: list of [K, N] fp16
row-major tensors; returns a list of fresh [M_i, N] fp16 tensors.  An empty list
gives an empty list.  When the inputs are consecutive views of one packed
buffer and the weights consecutive views of one [E, K, N] tensor (how
fused_select.py:54-71 builds them) nothing is copied; otherwise the pieces are
concatenated first.  Errors raise RuntimeError (the reference calls exit()).
"""
from __future__ import annotations

from typing import List

import torch

from . import ops


def _as_one(tensors: List[torch.Tensor]):
    """Return (base, True) if `tensors` are back-to-back views of one buffer, else (cat, False)."""
    first = tensors[0]
    expect = first.data_ptr()
    contiguous = True
    for t in tensors:
        if not t.is_contiguous() or t.data_ptr() != expect:
            contiguous = False
            break
        expect += t.numel() * t.element_size()
    if contiguous and expect - first.data_ptr() <= first.untyped_storage().nbytes() - (
            first.data_ptr() - first.untyped_storage().data_ptr()):
        total = sum(t.size(0) for t in tensors)
        return torch.as_strided(first, (total,) + tuple(first.shape[1:]), first.stride()), True
    return torch.cat([t.contiguous() for t in tensors], dim=0), False


def grouped_ffn_forward(inputs: List[torch.Tensor], weights: List[torch.Tensor]) -> List[torch.Tensor]:
    if len(inputs) == 0:
        return []
    if len(inputs) != len(weights):
        raise RuntimeError("grouped_ffn_forward: inputs and weights must have the same length")
    for a, w in zip(inputs, weights):
        if not (a.is_cuda and w.is_cuda):
            raise RuntimeError("inputs must be CUDA")
        if a.dtype != torch.float16 or w.dtype != torch.float16:
            raise RuntimeError("grouped_ffn_forward: inputs and weights must be fp16")
        if a.dim() != 2 or w.dim() != 2 or a.size(1) != w.size(0):
            raise RuntimeError("grouped_ffn_forward: expected [M,K] inputs and [K,N] weights")
    k_dim, n_dim = weights[0].shape
    if any(tuple(w.shape) != (k_dim, n_dim) for w in weights):
        raise RuntimeError("grouped_ffn_forward: all weights must have the same [K,N] shape")
    a_all, _ = _as_one(list(inputs))
    w_all, _ = _as_one([w.unsqueeze(0) for w in weights])
    counts = [int(a.size(0)) for a in inputs]
    offs = [0]
    for c in counts:
        offs.append(offs[-1] + c)
    offsets = torch.tensor(offs, dtype=torch.int32, device=a_all.device)
    out = ops.grouped_gemm(a_all, w_all.reshape(len(weights), k_dim, n_dim), offsets, layout="kn")
    return list(torch.split(out, counts, dim=0))
