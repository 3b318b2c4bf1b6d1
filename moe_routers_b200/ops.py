"""Torch-facing operators over the C ABI of libmoe_b200.so.

PyTorch is used for device memory and streams only: every function allocates
its outputs with torch, passes raw device pointers and the current stream to
the library and returns torch tensors.  All compute happens in the CUDA
kernels of the library; there is no CPU or eager fallback, CPU tensors are
rejected.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import check, lib

_DTYPE_CODE = {torch.float16: _lib.MOE_F16, torch.bfloat16: _lib.MOE_BF16, torch.float32: _lib.MOE_F32}

_workspaces: dict = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("inputs must be CUDA")  # same text as kernels/fused_select.cu:205


def workspace(device: torch.device, tokens: int, experts: int, top_k: int) -> torch.Tensor:
    """Per (device, stream) scratch buffer, grown on demand and initialised once."""
    need = int(lib.moe_workspace_bytes(int(tokens), int(experts), int(top_k)))
    need = max(need, 1 << 16)
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=device)
        check(lib.moe_workspace_init(ws.data_ptr(), ws.numel(), _stream()))
        _workspaces[key] = ws
    return ws


def read_status(device: Optional[torch.device] = None) -> int:
    """Synchronise the current stream and raise if a kernel recorded an error."""
    import ctypes

    device = device or torch.device("cuda", torch.cuda.current_device())
    ws = workspace(device, 1, 1, 1)
    out = ctypes.c_int(0)
    check(lib.moe_read_status(ws.data_ptr(), _stream(), ctypes.byref(out)))
    return out.value


def topk_select(logits: torch.Tensor, top_k: int):
    """(idx int32 [T,k], gates float32 [T,k]): lowest index wins ties."""
    _require_cuda(logits)
    if logits.dim() != 2:
        raise RuntimeError("logits shape must be [T, E]")
    if logits.dtype not in _DTYPE_CODE:
        raise RuntimeError("logits must be fp16/bf16/fp32")
    logits = logits.contiguous()
    t, e = logits.shape
    with torch.cuda.device(logits.device):
        idx = torch.empty((t, top_k), dtype=torch.int32, device=logits.device)
        gates = torch.empty((t, top_k), dtype=torch.float32, device=logits.device)
        check(lib.moe_topk_select(logits.data_ptr(), _DTYPE_CODE[logits.dtype], t, e, int(top_k),
                                  idx.data_ptr(), gates.data_ptr(), _stream()))
    return idx, gates


def pack(x: torch.Tensor, idx: torch.Tensor, experts: int, *, copy_rows: bool = True):
    """Expert-contiguous pack.  Returns (counts, offsets, packed, row_route, route_row)."""
    _require_cuda(x, idx)
    if x.dim() != 2 or idx.dim() != 2 or idx.size(0) != x.size(0):
        raise RuntimeError("x shape must be [T, d_model] and idx [T, k]")
    if x.element_size() not in (2, 4):
        raise RuntimeError("x must have 2- or 4-byte elements")
    x = x.contiguous()
    idx = idx.to(torch.int32).contiguous()
    t, d = x.shape
    k = idx.size(1)
    dev = x.device
    with torch.cuda.device(dev):
        counts = torch.empty(experts, dtype=torch.int32, device=dev)
        offsets = torch.empty(experts + 1, dtype=torch.int32, device=dev)
        packed = torch.empty((t * k, d), dtype=x.dtype, device=dev) if copy_rows else None
        row_route = torch.empty(t * k, dtype=torch.int32, device=dev)
        route_row = torch.empty(t * k, dtype=torch.int32, device=dev)
        ws = workspace(dev, t, experts, k)
        check(lib.moe_pack(x.data_ptr(), x.element_size(), idx.data_ptr(), t, d, int(experts), k,
                           counts.data_ptr(), offsets.data_ptr(),
                           packed.data_ptr() if packed is not None else None,
                           row_route.data_ptr(), route_row.data_ptr(), ws.data_ptr(), ws.numel(),
                           _stream()))
    return counts, offsets, packed, row_route, route_row


def pack_scatter(x: torch.Tensor, experts: int, out: dict) -> dict:
    """Re-run only the scatter half of `route_fused` into the buffers of `out` (a dict returned by
    route_fused for the same x).  The per-tile histograms of that call are read from
    `out["workspace"]`, the scratch buffer route_fused used (scratch is per stream, so the buffer of
    the calling stream would be the wrong one after a stream switch); no other route may have run
    on that buffer in between."""
    _require_cuda(x)
    t, d = x.shape
    k = out["idx"].size(1)
    with torch.cuda.device(x.device):
        ws = out["workspace"]
        check(lib.moe_pack_scatter(x.data_ptr(), x.element_size(), out["idx"].data_ptr(), t, d, int(experts), k,
                                   out["counts"].data_ptr(), out["offsets"].data_ptr(), out["packed"].data_ptr(),
                                   out["row_route"].data_ptr(), out["route_row"].data_ptr(), ws.data_ptr(),
                                   ws.numel(), _stream()))
    return out


def route_plan(x: torch.Tensor, idx: torch.Tensor, experts: int, *, hist_ready: bool = False) -> dict:
    """Counts, offsets and the route <-> row maps of a pack, without copying a row.

    `hist_ready`: the per-tile histograms of `idx` are already in the calling stream's scratch buffer
    (router_gemm_select has just produced idx on this stream); otherwise they are computed from idx.
    Returns dict(idx, counts, offsets, row_route, route_row, workspace) for `pack_scatter_to`."""
    _require_cuda(x, idx)
    idx = idx.to(torch.int32).contiguous()
    t, d = x.shape
    k = idx.size(1)
    dev = x.device
    with torch.cuda.device(dev):
        o = dict(idx=idx, counts=torch.empty(experts, dtype=torch.int32, device=dev),
                 offsets=torch.empty(experts + 1, dtype=torch.int32, device=dev),
                 row_route=torch.empty(t * k, dtype=torch.int32, device=dev),
                 route_row=torch.empty(t * k, dtype=torch.int32, device=dev))
        ws = o["workspace"] = workspace(dev, t, experts, k)
        fn = lib.moe_pack_scatter if hist_ready else lib.moe_pack
        check(fn(x.data_ptr(), x.element_size(), idx.data_ptr(), t, d, int(experts), k, o["counts"].data_ptr(),
                 o["offsets"].data_ptr(), None, o["row_route"].data_ptr(), o["route_row"].data_ptr(),
                 ws.data_ptr(), ws.numel(), _stream()))
    return o


def pack_scatter_to(x: torch.Tensor, experts: int, plan: dict, seg_base: torch.Tensor) -> dict:
    """Scatter the token rows of a planned route to one destination segment per expert: rows of expert
    e go, in canonical order, to the address seg_base[e] onwards (int64 [experts] on the device;
    16-byte aligned; peers' mapped memory allowed).  `plan` comes from `route_plan` (or route_fused)
    for the same x; its histograms must still be in plan["workspace"]."""
    _require_cuda(x, seg_base)
    if seg_base.dtype != torch.int64 or seg_base.numel() < experts:
        raise RuntimeError("seg_base must be an int64 tensor with one address per expert")
    x = x.contiguous()
    t, d = x.shape
    k = plan["idx"].size(1)
    ws = plan["workspace"]
    with torch.cuda.device(x.device):
        check(lib.moe_pack_scatter_to(x.data_ptr(), x.element_size(), plan["idx"].data_ptr(), t, d, int(experts), k,
                                      plan["counts"].data_ptr(), plan["offsets"].data_ptr(), seg_base.data_ptr(),
                                      plan["row_route"].data_ptr(), plan["route_row"].data_ptr(), ws.data_ptr(),
                                      ws.numel(), _stream()))
    return plan


def fused_select(logits: torch.Tensor, x: torch.Tensor, experts: int, top_k: int, out: Optional[tuple] = None):
    """Select + count + scan + pack from given logits in two launches.
    Returns (idx, gates, counts, offsets, packed, row_route, route_row); `out` may be the tuple a
    previous call returned, to reuse its buffers."""
    _require_cuda(logits, x)
    if logits.dtype not in _DTYPE_CODE:
        raise RuntimeError("logits must be fp16/bf16/fp32")
    logits = logits.contiguous()
    x = x.contiguous()
    t, d = x.shape
    dev = x.device
    with torch.cuda.device(dev):
        if out is None:
            out = (torch.empty((t, top_k), dtype=torch.int32, device=dev),
                   torch.empty((t, top_k), dtype=torch.float32, device=dev),
                   torch.empty(experts, dtype=torch.int32, device=dev),
                   torch.empty(experts + 1, dtype=torch.int32, device=dev),
                   torch.empty((t * top_k, d), dtype=x.dtype, device=dev),
                   torch.empty(t * top_k, dtype=torch.int32, device=dev),
                   torch.empty(t * top_k, dtype=torch.int32, device=dev))
        idx, gates, counts, offsets, packed, row_route, route_row = out
        ws = workspace(dev, t, experts, top_k)
        check(lib.moe_fused_select(logits.data_ptr(), _DTYPE_CODE[logits.dtype], x.data_ptr(), x.element_size(), t, d,
                                   int(experts), int(top_k), idx.data_ptr(), gates.data_ptr(), counts.data_ptr(),
                                   offsets.data_ptr(), packed.data_ptr(), row_route.data_ptr(), route_row.data_ptr(),
                                   ws.data_ptr(), ws.numel(), _stream()))
    return out


def combine(y: torch.Tensor, gates: torch.Tensor, route_row: torch.Tensor, top_k: int) -> torch.Tensor:
    """out[t] = sum_j gates[t,j] * y[route_row[t*k+j]]."""
    _require_cuda(y, gates, route_row)
    if y.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("y must be fp16 or bf16")
    y = y.contiguous()
    gates = gates.to(torch.float32).contiguous()
    route_row = route_row.to(torch.int32).contiguous()
    rows, d = y.shape
    t = rows // top_k
    with torch.cuda.device(y.device):
        out = torch.empty((t, d), dtype=y.dtype, device=y.device)
        check(lib.moe_combine(y.data_ptr(), _DTYPE_CODE[y.dtype], gates.data_ptr(), route_row.data_ptr(),
                              t, d, int(top_k), out.data_ptr(), _stream()))
    return out


def router_gemm_select(x: torch.Tensor, w_router: torch.Tensor, top_k: int, *, skew_experts: int = 0,
                       skew_bias: float = 0.0, return_logits: bool = False):
    """Fused logit GEMM + skew + top-k + gates.  Returns (idx, gates[, logits fp32])."""
    _require_cuda(x, w_router)
    if x.dtype not in (torch.float16, torch.bfloat16) or w_router.dtype != x.dtype:
        raise RuntimeError("x and the router weight must both be fp16 (Half) or both bf16")
    x = x.contiguous()
    w_router = w_router.contiguous()
    t, d = x.shape
    e = w_router.size(0)
    dev = x.device
    with torch.cuda.device(dev):
        idx = torch.empty((t, top_k), dtype=torch.int32, device=dev)
        gates = torch.empty((t, top_k), dtype=torch.float32, device=dev)
        logits = torch.empty((t, e), dtype=torch.float32, device=dev) if return_logits else None
        ws = workspace(dev, t, e, top_k)
        check(lib.moe_router_gemm_select(x.data_ptr(), w_router.data_ptr(), _DTYPE_CODE[x.dtype], t, d, e, int(top_k),
                                         int(skew_experts), float(skew_bias), idx.data_ptr(),
                                         gates.data_ptr(), logits.data_ptr() if return_logits else None,
                                         ws.data_ptr(), ws.numel(), _stream()))
    return (idx, gates, logits) if return_logits else (idx, gates)


def route_fused(x: torch.Tensor, w_router: torch.Tensor, top_k: int, *, skew_experts: int = 0,
                skew_bias: float = 0.0, return_logits: bool = False, out: Optional[dict] = None):
    """The whole fused_select strategy: logit GEMM + select + count/scan/pack.

    Returns a dict with idx, gates, counts, offsets, packed, row_route,
    route_row (and logits when asked), plus `workspace`: the scratch buffer
    of the calling stream, which holds the per-tile histograms of this call
    until the next route on that stream.  `out` may carry pre-allocated
    tensors from a previous call to avoid re-allocation.
    """
    _require_cuda(x, w_router)
    if x.dtype not in (torch.float16, torch.bfloat16) or w_router.dtype != x.dtype:
        raise RuntimeError("x and the router weight must both be fp16 (Half) or both bf16")
    x = x.contiguous()
    w_router = w_router.contiguous()
    t, d = x.shape
    e = w_router.size(0)
    dev = x.device
    with torch.cuda.device(dev):
        o = out if out is not None else {}
        if "idx" not in o:
            o["idx"] = torch.empty((t, top_k), dtype=torch.int32, device=dev)
            o["gates"] = torch.empty((t, top_k), dtype=torch.float32, device=dev)
            o["counts"] = torch.empty(e, dtype=torch.int32, device=dev)
            o["offsets"] = torch.empty(e + 1, dtype=torch.int32, device=dev)
            o["packed"] = torch.empty((t * top_k, d), dtype=x.dtype, device=dev)
            o["row_route"] = torch.empty(t * top_k, dtype=torch.int32, device=dev)
            o["route_row"] = torch.empty(t * top_k, dtype=torch.int32, device=dev)
        if return_logits and "logits" not in o:
            o["logits"] = torch.empty((t, e), dtype=torch.float32, device=dev)
        ws = o["workspace"] = workspace(dev, t, e, top_k)
        check(lib.moe_route_fused(x.data_ptr(), w_router.data_ptr(), _DTYPE_CODE[x.dtype], t, d, e, int(top_k),
                                  int(skew_experts), float(skew_bias), o["idx"].data_ptr(),
                                  o["gates"].data_ptr(), o["counts"].data_ptr(), o["offsets"].data_ptr(),
                                  o["packed"].data_ptr(), o["row_route"].data_ptr(),
                                  o["route_row"].data_ptr(),
                                  o["logits"].data_ptr() if return_logits else None,
                                  ws.data_ptr(), ws.numel(), _stream()))
    return o


def sinkhorn(logits: torch.Tensor, top_k: int, *, iters: int = 10, epsilon: float = 1e-6,
             temperature: float = 1.0):
    """Sinkhorn-balanced top-k: (idx int32 [T,k], gates float32 [T,k])."""
    _require_cuda(logits)
    if logits.dim() != 2:
        raise ValueError("SinkhornRouter expects logits of shape [tokens, experts]")
    if logits.dtype not in _DTYPE_CODE:
        raise RuntimeError("logits must be fp16/bf16/fp32")
    logits = logits.contiguous()
    t, e = logits.shape
    dev = logits.device
    with torch.cuda.device(dev):
        idx = torch.empty((t, top_k), dtype=torch.int32, device=dev)
        gates = torch.empty((t, top_k), dtype=torch.float32, device=dev)
        ws = workspace(dev, t, e, top_k)
        check(lib.moe_sinkhorn(logits.data_ptr(), _DTYPE_CODE[logits.dtype], t, e, int(top_k), int(iters),
                               float(epsilon), float(temperature), idx.data_ptr(), gates.data_ptr(),
                               ws.data_ptr(), ws.numel(), _stream()))
    return idx, gates


_ACT = {None: _lib.MOE_ACT_NONE, "none": _lib.MOE_ACT_NONE, "gelu": _lib.MOE_ACT_GELU,
        "silu": _lib.MOE_ACT_SILU, "swiglu": _lib.MOE_ACT_SWIGLU}


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, *, layout: str = "nk",
                 activation: Optional[str] = None, row_scale: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, sm_margin: int = 0,
                 bias: Optional[torch.Tensor] = None, out_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """c[offsets[e]:offsets[e+1]] = act(a[offsets[e]:offsets[e+1]] @ W[e]) for every expert.

    a [rows, K]; w [E, N, K] (layout "nk") or [E, K, N] (layout "kn"); both fp16 or both bf16;
    offsets int32 [E+1] on the device; bias [E, output features] (same dtype) is added before the
    activation.  With activation "swiglu" the weight has
    2N output features (gate rows first, then up) and the result has N columns.
    With `out_rows` (int64 [rows] on the device: one 16-byte aligned address per result row, possibly
    in a mapped peer buffer) the rows are stored there instead of in a dense result, and the table
    itself is returned.
    """
    _require_cuda(a, w, offsets)
    if a.dtype not in (torch.float16, torch.bfloat16) or w.dtype != a.dtype:
        raise RuntimeError("grouped_gemm: a and w must both be fp16 or both bf16")
    if bias is not None and (bias.dtype != a.dtype or not bias.is_cuda):
        raise RuntimeError("grouped_gemm: bias must be a CUDA tensor of the same dtype")
    if w.dim() != 3:
        raise RuntimeError("grouped_gemm: w must be [E, N, K] or [E, K, N]")
    a = a.contiguous()
    w = w.contiguous()
    offsets = offsets.to(torch.int32).contiguous()
    rows, k_dim = a.shape
    e = w.size(0)
    n_w = w.size(1) if layout == "nk" else w.size(2)
    if (w.size(2) if layout == "nk" else w.size(1)) != k_dim:
        raise RuntimeError("grouped_gemm: inner dimensions differ")
    act = _ACT[activation]
    n_out = n_w // 2 if act == _lib.MOE_ACT_SWIGLU else n_w
    dev = a.device
    with torch.cuda.device(dev):
        ws = workspace(dev, 1, e, 1)
        rs = row_scale.to(torch.float32).contiguous() if row_scale is not None else None
        if out_rows is not None:
            if out_rows.dtype != torch.int64 or not out_rows.is_cuda or out_rows.numel() < rows:
                raise RuntimeError("grouped_gemm: out_rows must be a CUDA int64 tensor with one address per row")
            check(lib.moe_grouped_gemm_rows(a.data_ptr(), w.data_ptr(), out_rows.data_ptr(), offsets.data_ptr(), e,
                                            rows, k_dim, n_out,
                                            _lib.MOE_W_NK if layout == "nk" else _lib.MOE_W_KN, w.stride(0), act,
                                            rs.data_ptr() if rs is not None else None,
                                            bias.contiguous().data_ptr() if bias is not None else None,
                                            _DTYPE_CODE[a.dtype], int(sm_margin), ws.data_ptr(), ws.numel(),
                                            _stream()))
            return out_rows
        c = out if out is not None else torch.empty((rows, n_out), dtype=a.dtype, device=dev)
        check(lib.moe_grouped_gemm(a.data_ptr(), w.data_ptr(), c.data_ptr(), offsets.data_ptr(), e, rows,
                                   k_dim, n_out, _lib.MOE_W_NK if layout == "nk" else _lib.MOE_W_KN,
                                   w.stride(0), act, rs.data_ptr() if rs is not None else None,
                                   bias.contiguous().data_ptr() if bias is not None else None,
                                   _DTYPE_CODE[a.dtype], int(sm_margin),
                                   ws.data_ptr(), ws.numel(), _stream()))
    return c
