"""Oracle (CPU, numpy) for the expert FFNs, the MoE block and expert parallelism.

TEST INFRASTRUCTURE ONLY: see the package docstring.  Citations are paths
inside santiweide/moe-routers.  GEMMs are fp32 products of the fp16 inputs,
rounded to fp16 where the reference stores fp16 (parity of the GEMM arithmetic
itself is unpinned: the reference's lives in an un-vendored CUTLASS).
"""
from __future__ import annotations

import numpy as np
from scipy.special import erf as _erf

from .routing import _np, combine, counts_offsets, pack_canonical


def _mm(a, b):
    return a.astype(np.float32) @ b.astype(np.float32)


def _weight_kn(w, layout: str):
    """Return the [K, N] view of a weight stored as "kn" ([K,N]) or "nk" ([N,K])."""
    w = _np(w)
    if layout == "kn":
        return w
    if layout == "nk":
        return w.T
    raise ValueError("layout must be 'kn' or 'nk'")


def gelu(v):
    """erf GELU, the default of torch.nn.functional.gelu."""
    v = v.astype(np.float32)
    return (0.5 * v * (1.0 + _erf(v / np.sqrt(2.0)))).astype(np.float32)


def silu(v):
    v = v.astype(np.float32)
    return (v / (1.0 + np.exp(-v))).astype(np.float32)


def gelu_ffn(x, w1, w2, *, layout: str = "nk", store=np.float16):
    """Two-layer GELU FFN d -> h -> d without bias (the expert of the
    benchmark configurations).  The hidden activation is stored in `store`
    (fp16), as a two-GEMM implementation does."""
    h = gelu(_mm(_np(x), _weight_kn(w1, layout))).astype(store)
    return _mm(h, _weight_kn(w2, layout)).astype(store)


def swiglu_ffn(x, w1, w3, w2, *, store=np.float16):
    """SwiGLU expert: models/transformer_decoder_model.py:162-172 and
    bench_2gpu_pcie.py:123-127.  Weights in nn.Linear layout ([out, in])."""
    x = _np(x)
    a = silu(_mm(x, _np(w1).T).astype(store))
    b = _mm(x, _np(w3).T).astype(store).astype(np.float32)
    h = (a.astype(store).astype(np.float32) * b).astype(store)
    return _mm(h, _np(w2).T).astype(store)


def grouped_gemm(inputs, weights, *, store=np.float16):
    """List of independent products [M_i,K] @ [K,N] -> [M_i,N], fp16 in and
    out, fp32 accumulation: kernels/grouped_ffn.cu:53-136."""
    return [_mm(_np(a), _np(b)).astype(store) for a, b in zip(inputs, weights)]


def _expert_apply(x, e, experts, kind, layout):
    if kind == "gelu":
        return gelu_ffn(x, experts["w1"][e], experts["w2"][e], layout=layout)
    if kind == "swiglu":
        return swiglu_ffn(x, experts["w1"][e], experts["w3"][e], experts["w2"][e])
    raise ValueError(kind)


def moe_layer(x, idx, gates, experts, *, kind: str = "gelu", layout: str = "nk"):
    """Sparse top-k MoE block output: models/decoder_moe.py:238-273.

    Routes are bucketed by expert, each bucket runs its expert FFN, and the
    result is gate-weighted and summed back per token.  `experts` is a dict of
    stacked weights ("w1", "w2" and, for SwiGLU, "w3"), first axis = expert.
    Returns (out fp16 [T,d], y_packed fp16 [T*k,d]) where y_packed holds the
    un-gated expert outputs in canonical packed order.
    """
    x = _np(x)
    idx = _np(idx).astype(np.int64)
    t, k = idx.shape
    n_experts = len(experts["w1"])
    packed, counts, offsets, _, route_row = pack_canonical(x, idx, n_experts)
    y = np.zeros_like(packed, dtype=np.float16)
    for e in range(n_experts):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if hi > lo:
            y[lo:hi] = _expert_apply(packed[lo:hi], e, experts, kind, layout)
    return combine(y, gates, route_row, k), y


def masked_matmul_layer(x, idx, gates, experts, *, kind: str = "gelu", layout: str = "nk"):
    """Strategy A (no permutation): every expert runs densely over all tokens
    and the outputs are summed with the top-k gate as mask (zero for
    unselected experts).  The nearest reference code is the dense-mixture
    branch models/decoder_moe.py:204-210; the top-k mask is the benchmark
    configuration's definition."""
    x = _np(x)
    idx = _np(idx).astype(np.int64)
    g = _np(gates).astype(np.float32)
    t, k = idx.shape
    n_experts = len(experts["w1"])
    dense_gate = np.zeros((t, n_experts), dtype=np.float32)
    for j in range(k):
        np.add.at(dense_gate, (np.arange(t), idx[:, j]), g[:, j])
    out = np.zeros((t, x.shape[1]), dtype=np.float32)
    for e in range(n_experts):
        out += dense_gate[:, e : e + 1] * _expert_apply(x, e, experts, kind, layout).astype(np.float32)
    return out.astype(np.float16)


# --------------------------------------------------------------------------
# Expert parallelism
# --------------------------------------------------------------------------
def ep_owner(expert_id, n_experts: int, world: int):
    """Owner rank of an expert: contiguous blocks of E/world experts
    (bench_2gpu_pcie.py:216-219, :372)."""
    if n_experts % world != 0:
        raise ValueError("experts must be divisible by world_size")
    return np.asarray(expert_id) // (n_experts // world)


def ep_send_splits(offsets, n_experts: int, world: int):
    """Rows this rank sends to every rank (its own block included): the packed
    buffer is expert-sorted, so destination r's rows are the slice
    offsets[r*E_local] : offsets[(r+1)*E_local] (bench_2gpu_pcie.py:305-322)."""
    e_local = n_experts // world
    off = _np(offsets).astype(np.int64)
    return [int(off[(r + 1) * e_local] - off[r * e_local]) for r in range(world)]


def ep_layer(x_ranks, router_fn, experts, *, n_experts: int, kind: str = "gelu", layout: str = "nk"):
    """Expert-parallel MoE layer over `len(x_ranks)` ranks.

    Each rank routes its own tokens with `router_fn(x) -> (idx, gates)`; every
    expert lives on exactly one rank, so the layer output for a rank's tokens
    equals the single-process block (models/decoder_moe.py:238-273) applied to
    those tokens with the global expert set.  Returns the per-rank outputs and
    the all-to-all row-count matrix splits[src][dst].
    """
    world = len(x_ranks)
    outs, splits = [], []
    for x in x_ranks:
        idx, gates = router_fn(x)
        out, _ = moe_layer(x, idx, gates, experts, kind=kind, layout=layout)
        outs.append(out)
        _, offsets = counts_offsets(idx, n_experts)
        splits.append(ep_send_splits(offsets, n_experts, world))
    return outs, splits
