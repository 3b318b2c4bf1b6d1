"""Expert-parallel MoE layer over `torch.distributed` (one process per GPU, NCCL over NVLink).

Generalises the reference's 2-GPU benchmark pipeline (bench_2gpu_pcie.py:258-599) to any world
size W that divides the expert count, and completes it with the combine step the reference omits:

    route (logit GEMM + select + pack)        every rank on its own tokens            [CUDA]
    all-gather of the per-expert counts        256 B per rank, one host read           [NCCL]
    dispatch all-to-all of the packed rows     remote rows only, self split = 0        [NCCL, comm stream]
    expert FFN on the rank's own rows          overlaps the dispatch                   [CUDA, main stream]
    re-bucket received rows by local expert    source-major -> expert-major            [CUDA]
    expert FFN on the received rows
    re-bucket back, combine all-to-all         rows return in the order they were sent [NCCL]
    gate-weighted combine                                                               [CUDA]

Experts are split contiguously: owner(e) = e // (E / W) (bench_2gpu_pcie.py:216-219, :372).  The
packed buffer is expert-sorted, so the rows for destination r are one slice of it and the send
splits are differences of `offsets` (bench_2gpu_pcie.py:305-322) - no extra permutation.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import ops
from ._lib import check, lib


def plan_exchange(counts_all: torch.Tensor, rank: int, world: int, *, skip_self: bool = True):
    """Row counts of the dispatch all-to-all from the all-gathered counts [W, E] (host tensor).

    Returns (send_splits, recv_splits): rows this rank sends to / receives from every rank; the
    entry for the rank itself is 0 when `skip_self` (its rows never leave the GPU).
    """
    w, e = counts_all.shape
    if w != world or e % world != 0:
        raise ValueError("experts must be divisible by world_size")
    el = e // world
    per_dest = counts_all.view(world, world, el).sum(dim=2)  # [src, dst]
    send = [int(v) for v in per_dest[rank].tolist()]
    recv = [int(v) for v in per_dest[:, rank].tolist()]
    if skip_self:
        send[rank] = 0
        recv[rank] = 0
    return send, recv


def exchange_rows(send_slices, recv_slices, rank: int, world: int, group=None) -> None:
    """Grouped point-to-point exchange with every other rank: an all-to-all without the self block,
    straight from / into slices of the packed buffers (no staging copies).  Zero-length messages
    are skipped on both sides (both sides derive the lengths from the same gathered counts)."""
    p2p = []
    for peer in range(world):
        if peer == rank:
            continue
        g_peer = dist.get_global_rank(group, peer) if group is not None else peer
        if recv_slices[peer].numel():
            p2p.append(dist.P2POp(dist.irecv, recv_slices[peer], g_peer, group))
        if send_slices[peer].numel():
            p2p.append(dist.P2POp(dist.isend, send_slices[peer], g_peer, group))
    if p2p:
        for work in dist.batch_isend_irecv(p2p):
            work.wait()


def split_rows(buf, splits):
    """Consecutive row slices of `buf` with the given lengths."""
    out, pos = [], 0
    for n in splits:
        out.append(buf[pos:pos + n])
        pos += n
    return out


class EPMoELayer:
    """One MoE layer with its experts sharded over the ranks of `group`.

    w_router [E, d] fp16 (replicated); w1_local [E/W, h, d], w2_local [E/W, d, h] fp16 (this rank's
    experts, nn.Linear layout); activation "gelu" (2-layer FFN) or "swiglu" (w1_local then holds
    gate rows followed by up rows: [E/W, 2h, d]).  strategy: "fused_select" / "naive_topk" (fused
    router GEMM + top-k) or "sinkhorn".
    """

    def __init__(self, w_router, w1_local, w2_local, top_k: int = 2, *, activation: str = "gelu",
                 strategy: str = "fused_select", sinkhorn_iters: int = 10, sinkhorn_temperature: float = 1.0,
                 skew_experts: int = 0, skew_bias: float = 0.0, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.e = w_router.size(0)
        if self.e % self.world != 0:
            raise ValueError("experts must be divisible by world_size")
        self.el = self.e // self.world
        if w1_local.size(0) != self.el or w2_local.size(0) != self.el:
            raise ValueError("local expert weights must hold experts/world experts")
        if strategy not in ("fused_select", "naive_topk", "sinkhorn"):
            raise ValueError(f"Unknown strategies: {[strategy]}")
        self.w_router, self.w1, self.w2 = w_router, w1_local, w2_local
        self.k = int(top_k)
        self.activation = activation
        self.strategy = strategy
        self.sinkhorn_iters, self.sinkhorn_temperature = sinkhorn_iters, sinkhorn_temperature
        self.skew_experts, self.skew_bias = skew_experts, skew_bias
        self.comm_stream = torch.cuda.Stream()
        self.last = {}

    # ---- stages (each usable on its own by the benchmark) -----------------------------------
    def route(self, x):
        if self.strategy == "sinkhorn":
            _, _, logits = ops.router_gemm_select(x, self.w_router, self.k, skew_experts=self.skew_experts,
                                                  skew_bias=self.skew_bias, return_logits=True)
            idx, gates = ops.sinkhorn(logits, self.k, iters=self.sinkhorn_iters,
                                      temperature=self.sinkhorn_temperature)
            counts, offsets, packed, row_route, route_row = ops.pack(x, idx, self.e)
            return dict(idx=idx, gates=gates, counts=counts, offsets=offsets, packed=packed,
                        row_route=row_route, route_row=route_row)
        return ops.route_fused(x, self.w_router, self.k, skew_experts=self.skew_experts, skew_bias=self.skew_bias)

    def exchange_counts(self, counts):
        """All-gather the per-expert counts; returns (device [W,E] int32, host copy).  One host sync,
        as in the reference (bench_2gpu_pcie.py:460-463)."""
        all_counts = torch.empty((self.world, self.e), dtype=torch.int32, device=counts.device)
        dist.all_gather_into_tensor(all_counts, counts, group=self.group)
        return all_counts, all_counts.cpu()

    def _ffn(self, rows, offsets, out):
        h = ops.grouped_gemm(rows, self.w1, offsets, layout="nk", activation=self.activation)
        return ops.grouped_gemm(h, self.w2, offsets, layout="nk", out=out)

    def _rebucket(self, src, dst, counts_all, backward, local_offsets):
        check(lib.moe_ep_rebucket(src.data_ptr(), dst.data_ptr(), counts_all.data_ptr(), self.e, self.world,
                                  self.rank, self.rank, 1 if backward else 0, src.size(1), src.element_size(),
                                  local_offsets.data_ptr() if local_offsets is not None else None,
                                  torch.cuda.current_stream().cuda_stream))

    def _exchange(self, send_slices, recv_slices):
        exchange_rows(send_slices, recv_slices, self.rank, self.world, self.group)

    _slices = staticmethod(split_rows)

    # ---- the layer --------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, *, overlap: bool = True) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("inputs must be CUDA")
        main = torch.cuda.current_stream()
        comm = self.comm_stream if overlap else main
        r, el, d = self.rank, self.el, x.size(1)

        o = self.route(x)
        counts_all, counts_host = self.exchange_counts(o["counts"])
        send, recv = plan_exchange(counts_host, r, self.world)
        off = [0] + [int(v) for v in counts_host[r].to(torch.int64).cumsum(0).tolist()]
        packed = o["packed"]
        y_packed = torch.empty_like(packed)
        # rows for destination p are packed[off[p*el] : off[(p+1)*el]]
        dest_slices = [packed[off[p * el]:off[(p + 1) * el]] for p in range(self.world)]
        ret_slices = [y_packed[off[p * el]:off[(p + 1) * el]] for p in range(self.world)]
        recv_buf = torch.empty((sum(recv), d), dtype=x.dtype, device=x.device)
        ret_buf = torch.empty_like(recv_buf)

        # dispatch of the remote rows on the communication stream ...
        comm.wait_stream(main)
        with torch.cuda.stream(comm):
            self._exchange(dest_slices, self._slices(recv_buf, recv))
        # ... while the rank's own rows (already expert-sorted for its experts) go through the FFN
        lo, hi = off[r * el], off[(r + 1) * el]
        if hi > lo:
            local_off = (o["offsets"][r * el:(r + 1) * el + 1] - o["offsets"][r * el]).contiguous()
            self._ffn(packed[lo:hi], local_off, y_packed[lo:hi])

        # received rows: bucket by local expert, FFN, restore the order they arrived in
        main.wait_stream(comm)
        if recv_buf.size(0) > 0:
            bucketed = torch.empty_like(recv_buf)
            remote_off = torch.empty(el + 1, dtype=torch.int32, device=x.device)
            self._rebucket(recv_buf, bucketed, counts_all, False, remote_off)
            y_b = self._ffn(bucketed, remote_off, torch.empty_like(bucketed))
            self._rebucket(y_b, ret_buf, counts_all, True, None)
        # combine all-to-all: every result row returns to the packed position it was sent from
        comm.wait_stream(main)
        with torch.cuda.stream(comm):
            self._exchange(self._slices(ret_buf, recv), ret_slices)
        main.wait_stream(comm)
        out = ops.combine(y_packed, o["gates"], o["route_row"], self.k)
        self.last = dict(counts_all=counts_host, send=send, recv=recv, route=o)
        return out

    __call__ = forward
