"""Expert-parallel MoE layer over `torch.distributed` (one process per GPU, NCCL over NVLink).

Generalises the reference's 2-GPU benchmark pipeline (bench_2gpu_pcie.py:258-599) to any world
size W that divides the expert count, and completes it with the combine step the reference omits:

    route (logit GEMM + select + pack)        every rank on its own tokens            [CUDA]
    all-gather of the per-expert counts        256 B per rank, one host read           [NCCL]
    for each group c of the local experts (pipelined, exchanges on a second stream):
      dispatch all-to-all of the packed rows   grouped send/recv straight from `packed` [NCCL]
      re-bucket received rows by local expert  source-major -> expert-major             [CUDA]
      expert FFN (grouped GEMM x2)             every expert's weights are read once     [CUDA]
      re-bucket back, combine all-to-all       rows return to the slot they came from   [NCCL]
    gate-weighted combine                                                                [CUDA]

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
                 skew_experts: int = 0, skew_bias: float = 0.0, group=None, transport: str = "peer",
                 max_tokens: Optional[int] = None):
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
        if transport not in ("peer", "nccl"):
            raise ValueError("transport must be 'peer' or 'nccl'")
        # "peer": device-initiated dispatch/combine, rows stored straight into the owner's expert-major
        # inbox over NVLink (CUDA IPC mappings), no host synchronisation in the layer.
        # "nccl": grouped NCCL send/recv plus re-bucketing on the owner.
        self.transport = transport
        # peer transport: the second expert GEMM stores its result rows straight into the home ranks'
        # packed slots (one kernel computes and returns); False: dense result + a separate push
        self.fuse_combine = True
        # peer transport: the pack stores every row straight into the owner's inbox (no local packed
        # copy, no push kernel); False: pack locally, then push
        self.direct_dispatch = True
        self._peer = None
        # peer transport: the inbox / result buffers are sized ONCE, at the first call (a collective
        # set-up), for `max_tokens` tokens per rank (default: the first batch; ranks may differ, the
        # largest counts); a later batch with more tokens is refused instead of re-sized, because a
        # re-size decided by one rank alone would leave the others in a different collective
        self.max_tokens = max_tokens
        self._calls = 0
        self.comm_stream = torch.cuda.Stream()
        # Expert groups pipelined against the exchanges, and SMs the persistent GEMM leaves to the
        # exchange kernels while it runs.  Measured on 2 B200s (T=4096/rank, d=4096, h=8192, E=64):
        # one group with no margin is fastest (1.95 ms); 2 groups / 16 SMs costs more in GEMM wave
        # tails and lost SMs (2.2 ms) than the ~0.09 ms per exchange it hides.  Raise both where the
        # exchange is a larger share of the layer.
        self.chunks = 1
        self.sm_margin = 0
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

    def route_select(self, x):
        """Select + pack plan without copying a row: idx, gates, counts, offsets, the route <-> row maps
        and the scratch buffer holding the tile histograms (input of the direct dispatch)."""
        if self.strategy == "sinkhorn":
            _, _, logits = ops.router_gemm_select(x, self.w_router, self.k, skew_experts=self.skew_experts,
                                                  skew_bias=self.skew_bias, return_logits=True)
            idx, gates = ops.sinkhorn(logits, self.k, iters=self.sinkhorn_iters,
                                      temperature=self.sinkhorn_temperature)
            o = ops.route_plan(x, idx, self.e)
        else:
            idx, gates = ops.router_gemm_select(x, self.w_router, self.k, skew_experts=self.skew_experts,
                                                skew_bias=self.skew_bias)
            o = ops.route_plan(x, idx, self.e, hist_ready=True)
        o["gates"] = gates
        return o

    def dispatch_direct(self, x, o, counts_all):
        """Store every routed row of x straight into its owner's expert-major inbox."""
        pr = self._peer
        check(lib.moe_ep_segment_bases(pr["inbox_ptrs"].data_ptr(), counts_all.data_ptr(), self.e, self.world,
                                       self.rank, pr["d"], x.element_size(), pr["seg_base"].data_ptr(),
                                       pr["offsets"].data_ptr(), torch.cuda.current_stream().cuda_stream))
        ops.pack_scatter_to(x, self.e, o, pr["seg_base"])

    def exchange_counts(self, counts):
        """All-gather the per-expert counts; returns (device [W,E] int32, host copy).  One host sync,
        as in the reference (bench_2gpu_pcie.py:460-463)."""
        all_counts = torch.empty((self.world, self.e), dtype=torch.int32, device=counts.device)
        dist.all_gather_into_tensor(all_counts, counts, group=self.group)
        return all_counts, all_counts.cpu()

    def _ffn(self, rows, offsets, out, e_lo=0, e_cnt=None, sm_margin=0, out_rows=None):
        """Both expert GEMMs; with `out_rows` the second one stores every result row at its own
        address (the packed slot of the rank it came from) instead of into `out`."""
        e_hi = self.el if e_cnt is None else e_lo + e_cnt
        h = ops.grouped_gemm(rows, self.w1[e_lo:e_hi], offsets, layout="nk", activation=self.activation,
                             sm_margin=sm_margin)
        return ops.grouped_gemm(h, self.w2[e_lo:e_hi], offsets, layout="nk", out=out, sm_margin=sm_margin,
                                out_rows=out_rows)

    def _rebucket(self, src, dst, counts_all, backward, local_offsets, e_lo, e_cnt):
        check(lib.moe_ep_rebucket(src.data_ptr(), dst.data_ptr(), counts_all.data_ptr(), self.e, self.world,
                                  self.rank, -1, 1 if backward else 0, src.size(1), src.element_size(),
                                  int(e_lo), int(e_cnt),
                                  local_offsets.data_ptr() if local_offsets is not None else None,
                                  torch.cuda.current_stream().cuda_stream))

    def _exchange(self, send_slices, recv_slices):
        exchange_rows(send_slices, recv_slices, self.rank, self.world, self.group)

    _slices = staticmethod(split_rows)

    # ---- the layer, in stages ---------------------------------------------------------------
    def plan(self, o, counts_all, counts_host, chunks: int):
        """Buffers and slices of one forward pass.  The local experts are handled in `chunks` groups:
        the exchange of one group overlaps the FFN of another, and every expert's weights are read
        once.  Rows for (destination p, group c) are one slice of the expert-sorted packed buffer."""
        r, el, w = self.rank, self.el, self.world
        if chunks < 1 or el % chunks != 0:
            chunks = 1
        ec = el // chunks
        packed = o["packed"]
        d = packed.size(1)
        off = [0] + [int(v) for v in counts_host[r].to(torch.int64).cumsum(0).tolist()]
        cnt = counts_host.view(w, w, chunks, ec).sum(dim=3)  # [src, dst, chunk] rows
        y_packed = torch.empty_like(packed)
        pl = dict(o=o, counts_all=counts_all, chunks=chunks, ec=ec, y_packed=y_packed, send=[], back=[], recv=[],
                  recv_buf=[], ret_buf=[], rows=[])
        for c in range(chunks):
            rows_from = [int(cnt[s_, r, c]) for s_ in range(w)]
            recv_buf = torch.empty((sum(rows_from), d), dtype=packed.dtype, device=packed.device)
            ret_buf = torch.empty_like(recv_buf)
            lohi = [(off[p * el + c * ec], off[p * el + (c + 1) * ec]) for p in range(w)]
            pl["send"].append([packed[lo:hi] for lo, hi in lohi])
            pl["back"].append([y_packed[lo:hi] for lo, hi in lohi])
            pl["recv"].append(split_rows(recv_buf, rows_from))
            pl["recv_buf"].append(recv_buf)
            pl["ret_buf"].append(ret_buf)
            pl["rows"].append(rows_from)
        return pl

    def dispatch(self, pl, c):
        """Rows of expert group c go to their owners (the rank's own rows by a device copy)."""
        r = self.rank
        if pl["recv"][c][r].numel():
            pl["recv"][c][r].copy_(pl["send"][c][r])
        self._exchange(pl["send"][c], pl["recv"][c])

    def compute(self, pl, c, sm_margin=0):
        """Bucket the received rows of group c by expert, run the expert FFN, restore arrival order."""
        recv_buf = pl["recv_buf"][c]
        if recv_buf.size(0) == 0:
            return
        ec = pl["ec"]
        bucketed = torch.empty_like(recv_buf)
        loc_off = torch.empty(ec + 1, dtype=torch.int32, device=recv_buf.device)
        self._rebucket(recv_buf, bucketed, pl["counts_all"], False, loc_off, c * ec, ec)
        y_b = self._ffn(bucketed, loc_off, torch.empty_like(bucketed), c * ec, ec, sm_margin)
        self._rebucket(y_b, pl["ret_buf"][c], pl["counts_all"], True, None, c * ec, ec)

    def give_back(self, pl, c):
        """Combine exchange of group c: every result row returns to the packed slot it came from."""
        r = self.rank
        ret = split_rows(pl["ret_buf"][c], pl["rows"][c])
        if ret[r].numel():
            pl["back"][c][r].copy_(ret[r])
        self._exchange(ret, pl["back"][c])

    # ---- device-initiated transport ------------------------------------------------------------
    def _setup_peer(self, rows_home: int, d: int, dtype, device):
        """Allocate this rank's inbox / result / flag buffers and map every peer's into this process
        (collective: every rank calls it once, at its first forward).  inbox: worst case all
        W * max_rows routes of the job land on this rank."""
        import ctypes

        w = self.world
        want = max(int(rows_home), int(self.max_tokens) * self.k if self.max_tokens is not None else 0)
        sizes = [None] * w
        dist.all_gather_object(sizes, want, group=self.group)
        max_rows = max(sizes)  # ranks may hold different numbers of tokens
        cap = w * max_rows
        inbox = torch.empty((cap, d), dtype=dtype, device=device)
        y_home = torch.empty((max_rows, d), dtype=dtype, device=device)
        # rank-to-rank signals: flag table int32 [3 slots][W] and the counts of both call parities
        # int32 [2][W][E] in one allocation the peers map
        sync = torch.zeros(3 * w + 2 * w * self.e, dtype=torch.int32, device=device)

        def export(t):
            """(64-byte IPC handle of the allocation holding `t`, offset of `t` inside it)"""
            handle = ctypes.create_string_buffer(64)
            offset = ctypes.c_size_t(0)
            with torch.cuda.device(device):
                check(lib.moe_ipc_export(t.data_ptr(), handle, ctypes.byref(offset)))
            return handle.raw, int(offset.value)

        gathered = [None] * w
        if w > 1:
            torch.cuda.synchronize(device)  # the flag table is zero before any peer can see it
            dist.all_gather_object(gathered, (export(inbox), export(y_home), export(sync)), group=self.group)
        opened = {}  # one mapping per distinct allocation

        def map_peer(handle, offset):
            if handle not in opened:
                base = ctypes.c_void_p()
                with torch.cuda.device(device):  # opened with THIS rank's device current
                    check(lib.moe_ipc_open(handle, ctypes.byref(base)))
                opened[handle] = base.value
            return opened[handle] + offset

        in_ptrs, home_ptrs, sync_ptrs = [], [], []
        for p_ in range(w):
            if p_ == self.rank:
                in_ptrs.append(inbox.data_ptr())
                home_ptrs.append(y_home.data_ptr())
                sync_ptrs.append(sync.data_ptr())
            else:
                (h_i, o_i), (h_h, o_h), (h_s, o_s) = gathered[p_]
                in_ptrs.append(map_peer(h_i, o_i))
                home_ptrs.append(map_peer(h_h, o_h))
                sync_ptrs.append(map_peer(h_s, o_s))
        counts_base = 3 * w  # word offset of the counts inside `sync`
        self._peer = dict(
            rows_home=max_rows, d=d, dtype=dtype, cap=cap, inbox=inbox, y_home=y_home, mappings=opened, sync=sync,
            inbox_ptrs=torch.tensor(in_ptrs, dtype=torch.int64, device=device),
            home_ptrs=torch.tensor(home_ptrs, dtype=torch.int64, device=device),
            flag_ptrs=torch.tensor(sync_ptrs, dtype=torch.int64, device=device),
            counts_ptrs=torch.tensor([p_ + 4 * counts_base for p_ in sync_ptrs], dtype=torch.int64, device=device),
            counts_all=sync[counts_base:].view(2, w, self.e),
            yb=torch.empty((cap, d), dtype=dtype, device=device),
            targets=torch.zeros(cap, dtype=torch.int64, device=device),
            seg_base=torch.zeros(self.e, dtype=torch.int64, device=device),
            offsets=torch.zeros(self.el + 1, dtype=torch.int32, device=device),
        )
        dist.barrier(group=self.group)

    def close(self):
        """Unmap the peers' buffers (collective in effect: call it on every rank, before the process
        group goes away; no rank may still be inside a forward)."""
        if self._peer is not None:
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=self.group)  # nobody unmaps memory a peer's kernel may still store into
            for base in self._peer["mappings"].values():
                check(lib.moe_ipc_close(base))
            self._peer = None

    def _push(self, local, ptrs, counts_all, combine, local_offsets):
        check(lib.moe_ep_push(local.data_ptr(), ptrs.data_ptr(), counts_all.data_ptr(), self.e, self.world, self.rank,
                              1 if combine else 0, local.size(1), local.element_size(),
                              local_offsets.data_ptr() if local_offsets is not None else None,
                              torch.cuda.current_stream().cuda_stream))

    def _row_targets(self, counts_all):
        pr = self._peer
        check(lib.moe_ep_row_targets(pr["home_ptrs"].data_ptr(), counts_all.data_ptr(), self.e, self.world, self.rank,
                                     pr["d"], pr["inbox"].element_size(), pr["targets"].data_ptr(),
                                     torch.cuda.current_stream().cuda_stream))
        return pr["targets"]

    def _rank_sync(self, slot: int, value: int, payload=None, payload_offset_words: int = 0):
        """Tell every rank that this rank has reached phase `slot` of call `value` (its earlier stores, the
        optional payload included, are visible to them before the flag is) and wait, on the stream, until
        every rank has done the same: one launch, no host wait.  The wait is bounded on the device; a
        rank that never arrives shows up in ops.read_status()."""
        pr = self._peer
        ws = ops.workspace(pr["sync"].device, 1, self.e, self.k)
        check(lib.moe_ep_sync(pr["flag_ptrs"].data_ptr(), pr["sync"].data_ptr(), self.world, self.rank, slot, value,
                              payload.data_ptr() if payload is not None else None,
                              pr["counts_ptrs"].data_ptr() if payload is not None else None,
                              payload_offset_words, payload.numel() if payload is not None else 0,
                              ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream))

    def exchange_counts_peer(self, counts, call: int):
        """Every rank's per-expert counts into every rank's table (peer stores + a flag; replaces the
        all-gather): returns the device tensor [W, E] of this call's parity."""
        pr = self._peer
        par = call & 1
        self._rank_sync(0, call, payload=counts, payload_offset_words=(par * self.world + self.rank) * self.e)
        return pr["counts_all"][par]

    def forward_peer(self, x: torch.Tensor, *, overlap: bool = True) -> torch.Tensor:
        """overlap=True: the exchanges ride inside the kernels that produce the rows (the pack stores
        into the owners' inboxes, the second expert GEMM stores its rows into their home slots).
        overlap=False: every stage on its own, in series (local pack, push, FFN, push back)."""
        x = x.contiguous()
        rows_home, d = x.size(0) * self.k, x.size(1)
        if self._peer is None:
            self._setup_peer(rows_home, d, x.dtype, x.device)
        pr = self._peer
        if rows_home > pr["rows_home"] or d != pr["d"] or x.dtype != pr["dtype"]:
            raise RuntimeError(f"EPMoELayer: batch of {x.size(0)} tokens x {d} does not fit the buffers set up for "
                               f"{pr['rows_home'] // self.k} tokens x {pr['d']} per rank (pass max_tokens)")
        self._calls += 1
        call = self._calls
        direct = overlap and self.direct_dispatch and (d * x.element_size()) % 16 == 0 and x.data_ptr() % 16 == 0
        fuse = overlap and self.fuse_combine
        o = self.route_select(x) if direct else self.route(x)
        # Slot 0 doubles as the barrier that frees the buffers of the previous call: a rank signals it
        # only after its own previous combine (stream order), and nobody stores into an inbox before
        # every rank has signalled.
        counts_all = self.exchange_counts_peer(o["counts"], call)
        if direct:
            self.dispatch_direct(x, o, counts_all)
        else:
            self._push(o["packed"], pr["inbox_ptrs"], counts_all, False, pr["offsets"])
        if fuse:
            targets = self._row_targets(counts_all)
            self._rank_sync(1, call)  # all rows have arrived in every inbox
            self._ffn(pr["inbox"], pr["offsets"], None, out_rows=targets)  # computes and returns the rows
        else:
            self._rank_sync(1, call)
            self._ffn(pr["inbox"], pr["offsets"], pr["yb"])
            self._push(pr["yb"], pr["home_ptrs"], counts_all, True, None)
        self._rank_sync(2, call)  # all results are back in their home slots
        out = ops.combine(pr["y_home"][:rows_home], o["gates"], o["route_row"], self.k)
        self.last = dict(counts_dev=counts_all, route=o)
        return out

    def forward(self, x: torch.Tensor, *, overlap: bool = True, chunks: Optional[int] = None) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("inputs must be CUDA")
        if self.transport == "peer":
            return self.forward_peer(x, overlap=overlap)
        main = torch.cuda.current_stream()
        comm = self.comm_stream if overlap else main
        if chunks is None:
            chunks = self.chunks if overlap else 1
        margin = self.sm_margin if overlap else 0

        o = self.route(x)
        counts_all, counts_host = self.exchange_counts(o["counts"])
        pl = self.plan(o, counts_all, counts_host, chunks)
        n = pl["chunks"]
        arrived = [torch.cuda.Event() for _ in range(n)]
        computed = [torch.cuda.Event() for _ in range(n)]
        comm.wait_stream(main)
        with torch.cuda.stream(comm):
            for c in range(n):
                self.dispatch(pl, c)
                arrived[c].record(comm)
        for c in range(n):
            main.wait_event(arrived[c])
            self.compute(pl, c, margin)
            computed[c].record(main)
        with torch.cuda.stream(comm):
            for c in range(n):
                comm.wait_event(computed[c])
                self.give_back(pl, c)
        main.wait_stream(comm)
        out = ops.combine(pl["y_packed"], o["gates"], o["route_row"], self.k)
        self.last = dict(counts_all=counts_host, route=o, plan=pl)
        return out

    __call__ = forward
