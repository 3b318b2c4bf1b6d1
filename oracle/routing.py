"""Oracle (CPU, numpy) for router logits, selection, Sinkhorn, pack and combine.

TEST INFRASTRUCTURE ONLY: see the package docstring.  All functions take and
return numpy arrays; fp16 inputs are numpy float16.  Citations are paths inside
santiweide/moe-routers.
"""
from __future__ import annotations

import numpy as np


def _np(a):
    """Accept numpy arrays or CPU torch tensors (bf16 is widened to fp32)."""
    if isinstance(a, np.ndarray):
        return a
    try:
        import torch

        if isinstance(a, torch.Tensor):
            a = a.detach().cpu()
            if a.dtype == torch.bfloat16:
                a = a.float()
            return a.numpy()
    except ImportError:  # pragma: no cover
        pass
    return np.asarray(a)


# --------------------------------------------------------------------------
# Router logits
# --------------------------------------------------------------------------
def router_logits(x, w, *, skew_experts: int = 0, skew_bias: float = 0.0, out_dtype=None):
    """logits = x @ w.T, then `logits[:, :skew_experts] += skew_bias`.

    bench_router.py:512-516 (CUDA: product in the input dtype, i.e. fp32
    accumulation rounded to fp16, then an in-place add in that dtype) and
    bench_router.py:487-490 (CPU: fp32 product).  `out_dtype` defaults to the
    dtype of `x`; pass np.float32 for the CPU flavour.
    """
    x = _np(x)
    w = _np(w)
    out_dtype = np.dtype(out_dtype or x.dtype)
    acc = x.astype(np.float32) @ w.astype(np.float32).T
    logits = acc.astype(out_dtype)
    if skew_experts > 0 and skew_bias != 0.0:
        # in-place add in the logits dtype: one rounding to that dtype
        logits[:, :skew_experts] = (
            logits[:, :skew_experts].astype(np.float32) + np.float32(skew_bias)
        ).astype(out_dtype)
    return logits


# --------------------------------------------------------------------------
# Top-k selection
# --------------------------------------------------------------------------
def topk_select(logits, k: int):
    """Top-k experts per token and softmax over the k selected logits.

    models/decoder_moe.py:58-62 (`torch.topk` then `softmax(topk_vals)`), with
    the tie rule made explicit: among equal logits the LOWEST expert index
    wins (a stable descending sort).  Returns (idx int64 [T,k], gates float32
    [T,k], vals float32 [T,k]).  Gates are computed in fp32 from the logits
    widened to fp32; a caller comparing with an fp16 reference rounds them.
    """
    v = _np(logits).astype(np.float32)
    t, e = v.shape
    if not (0 < k <= e):
        raise ValueError("top_k must be in [1, n_experts]")
    order = np.argsort(-v, axis=1, kind="stable")[:, :k]
    vals = np.take_along_axis(v, order, axis=1)
    ex = np.exp(vals - vals[:, :1])
    gates = ex / ex.sum(axis=1, keepdims=True, dtype=np.float32)
    return order.astype(np.int64), gates.astype(np.float32), vals


def fused_select_gates(vals):
    """Gate arithmetic of the fused top-2 kernel: kernels/fused_select.cu:101-111.

    m = max(v0, v1); e_j = exp(v_j - m); inv = 1 / max(e0 + e1, 1e-9).
    """
    v = _np(vals).astype(np.float32)
    m = v.max(axis=1, keepdims=True)
    ex = np.exp(v - m)
    inv = np.float32(1.0) / np.maximum(ex.sum(axis=1, keepdims=True, dtype=np.float32), np.float32(1e-9))
    return (ex * inv).astype(np.float32)


# --------------------------------------------------------------------------
# Counts, offsets, pack
# --------------------------------------------------------------------------
def counts_offsets(idx, n_experts: int):
    """Per-expert route histogram and its exclusive prefix.

    kernels/fused_select.cu:116-143 (histogram) and :256-279 (offsets[0] = 0,
    offsets[1..E] = inclusive sum).  Returns (counts int32 [E], offsets int32
    [E+1]); offsets[E] == T*k (the invariant checked at :292).
    """
    idx = _np(idx).astype(np.int64).reshape(-1)
    counts = np.bincount(idx, minlength=n_experts).astype(np.int32)
    offsets = np.zeros(n_experts + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts, dtype=np.int64).astype(np.int32)
    return counts, offsets


def pack_canonical(x, idx, n_experts: int):
    """Expert-contiguous copy of the raw token rows, in canonical order.

    kernels/fused_select.cu:148-198 copies x[t] once per pick to
    offsets[e] + slot; bench_router.py:57-78 sorts routes by expert.  Both
    leave the order inside an expert segment unspecified (atomic slots /
    unstable argsort); the canonical order used here and by the CUDA path is
    ascending route id r = t*k + j inside each segment (a stable sort by
    expert).  Rows are copied bit for bit, with no gate applied
    (bench_2gpu_pcie.py:20-22).

    Returns (packed [T*k, d], counts, offsets, row_route int32 [T*k] giving
    the route id stored in each packed row, route_row int32 [T*k] its inverse).
    """
    x = _np(x)
    idx = _np(idx).astype(np.int64)
    t, k = idx.shape
    counts, offsets = counts_offsets(idx, n_experts)
    row_route = np.argsort(idx.reshape(-1), kind="stable").astype(np.int32)
    route_row = np.empty_like(row_route)
    route_row[row_route] = np.arange(t * k, dtype=np.int32)
    packed = x[row_route // k]
    return packed, counts, offsets, row_route, route_row


def fused_select_forward(logits, x):
    """The five outputs of `fused_select_forward(logits, x)` for E = 64, k = 2.

    kernels/fused_select.cu:203-311: idx int32 [T,2], w float32 [T,2], counts
    int32 [64], offsets int32 [65], packed fp16 [2T, d] (canonical order).
    """
    logits = _np(logits)
    idx, _, vals = topk_select(logits, 2)
    w = fused_select_gates(vals)
    packed, counts, offsets, _, _ = pack_canonical(x, idx, logits.shape[1])
    return idx.astype(np.int32), w, counts, offsets, packed


# --------------------------------------------------------------------------
# Sinkhorn
# --------------------------------------------------------------------------
def sinkhorn_assign(logits, *, iters: int = 10, epsilon: float = 1e-6, temperature: float = 1.0):
    """The balanced assignment matrix q [T,E] (float32): models/decoder_moe.py:103-119.

    scores = (logits / temperature).float(); scores -= rowmax; q = exp(scores);
    `iters` times { q /= rowsum + eps ; q = q / (colsum + eps) * (T / E) };
    then one more row normalisation.
    """
    lg = _np(logits)
    if iters <= 0 or epsilon <= 0 or temperature <= 0:
        raise ValueError("iters, epsilon and temperature must be > 0")
    # the division happens in the logits dtype, before the widening
    scores = (lg / lg.dtype.type(temperature)).astype(np.float32)
    t, e = scores.shape
    scores = scores - scores.max(axis=1, keepdims=True)
    q = np.exp(scores).astype(np.float32)
    eps = np.float32(epsilon)
    col_target = np.float32(float(t) / float(max(e, 1)))
    for _ in range(iters):
        q = q / (q.sum(axis=1, keepdims=True, dtype=np.float32) + eps)
        q = q / (q.sum(axis=0, keepdims=True, dtype=np.float32) + eps) * col_target
    q = q / (q.sum(axis=1, keepdims=True, dtype=np.float32) + eps)
    return q


def sinkhorn_route(logits, k: int, *, iters: int = 10, epsilon: float = 1e-6, temperature: float = 1.0):
    """Sinkhorn router: models/decoder_moe.py:92-123.

    top-k of q (lowest index wins ties), w = vals / (sum(vals) + eps).
    Returns (idx int64 [T,k], w float32 [T,k], q float32 [T,E]); the reference
    casts w to the logits dtype.
    """
    q = sinkhorn_assign(logits, iters=iters, epsilon=epsilon, temperature=temperature)
    t, e = q.shape
    if not (0 < k <= e):
        raise ValueError("top_k must be in [1, n_experts]")
    order = np.argsort(-q, axis=1, kind="stable")[:, :k]
    vals = np.take_along_axis(q, order, axis=1)
    w = vals / (vals.sum(axis=1, keepdims=True, dtype=np.float32) + np.float32(epsilon))
    return order.astype(np.int64), w.astype(np.float32), q


# --------------------------------------------------------------------------
# Combine and statistics
# --------------------------------------------------------------------------
def combine(y_packed, gates, route_row, k: int, out_dtype=np.float16):
    """out[t] = sum_j gates[t,j] * y_packed[route_row[t*k + j]].

    models/decoder_moe.py:270-271 (`expert(x_e) * w_e` then `index_add_`).
    Accumulated in fp32 in ascending j and rounded once to `out_dtype`.
    """
    y = _np(y_packed).astype(np.float32)
    g = _np(gates).astype(np.float32)
    rr = _np(route_row).astype(np.int64).reshape(-1, k)
    out = np.zeros((rr.shape[0], y.shape[1]), dtype=np.float32)
    for j in range(k):
        out += g[:, j : j + 1] * y[rr[:, j]]
    return out.astype(out_dtype)


def load_skew(counts):
    """(max/mean, CV) of per-expert route counts: bench_2gpu_pcie.py:446-457."""
    c = _np(counts).astype(np.float32)
    mean = float(c.mean())
    std = float(c.std())
    return float(c.max() / (mean + 1e-9)), float(std / (mean + 1e-9))
