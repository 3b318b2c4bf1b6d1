"""Expert-parallel host logic on CPU: two gloo ranks route with the oracle, exchange counts, plan
the all-to-all and move rows with the same grouped point-to-point exchange the GPU layer uses.
Checks that every owner receives exactly the rows the oracle says it should, and that the
combine exchange returns every row to the position it was sent from."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, e, k, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from moe_routers_b200.ep import exchange_rows, plan_exchange, split_rows

        t, d = 96 + 17 * rank, 24
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(t, d, generator=g)
        gw = torch.Generator().manual_seed(7)
        w = torch.randn(e, d, generator=gw) / d ** 0.5
        logits = oracle.router_logits(x.numpy(), w.numpy(), skew_experts=2, skew_bias=1.0, out_dtype=np.float32)
        idx, gates, _ = oracle.topk_select(logits, k)
        packed, counts, offsets, row_route, route_row = oracle.pack_canonical(x.numpy(), idx, e)
        el = e // world

        gathered = [torch.zeros(e, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(counts))
        counts_all = torch.stack(gathered)
        send, recv = plan_exchange(counts_all, rank, world)
        assert send[rank] == 0 and recv[rank] == 0
        assert send == [0 if p == rank else int(offsets[(p + 1) * el] - offsets[p * el]) for p in range(world)]
        assert oracle.ep_send_splits(offsets, e, world)[1 - rank] == send[1 - rank]

        packed_t = torch.from_numpy(packed.copy())
        dest = [packed_t[int(offsets[p * el]):int(offsets[(p + 1) * el])] for p in range(world)]
        recv_buf = torch.zeros(sum(recv), d)
        exchange_rows(dest, split_rows(recv_buf, recv), rank, world)

        # what the peer must have sent: its rows for my experts, in its packed order
        other = 1 - rank
        to, do = 96 + 17 * other, 24
        go = torch.Generator().manual_seed(100 + other)
        xo = torch.randn(to, do, generator=go)
        lo_ = oracle.router_logits(xo.numpy(), w.numpy(), skew_experts=2, skew_bias=1.0, out_dtype=np.float32)
        idxo, _, _ = oracle.topk_select(lo_, k)
        po, co, oo, _, _ = oracle.pack_canonical(xo.numpy(), idxo, e)
        expect = po[int(oo[rank * el]):int(oo[(rank + 1) * el])]
        np.testing.assert_array_equal(recv_buf.numpy(), expect)
        assert counts_all[other].numpy().tolist() == co.tolist()

        # "expert FFN" stand-in: y = 2 * row; the return exchange puts results back in packed order
        y_packed = torch.full_like(packed_t, -1.0)
        lo, hi = int(offsets[rank * el]), int(offsets[(rank + 1) * el])
        y_packed[lo:hi] = 2 * packed_t[lo:hi]
        ret = [y_packed[int(offsets[p * el]):int(offsets[(p + 1) * el])] for p in range(world)]
        exchange_rows(split_rows(2 * recv_buf, recv), ret, rank, world)
        np.testing.assert_array_equal(y_packed.numpy(), 2 * packed)
        out = oracle.combine(y_packed.numpy(), gates, route_row, k, out_dtype=np.float32)
        np.testing.assert_allclose(out, 2 * x.numpy(), rtol=1e-5, atol=1e-6)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as exc:  # pragma: no cover
        import traceback

        q.put((rank, "".join(traceback.format_exception(exc))))


def test_two_rank_dispatch_and_combine_on_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 8, 2, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def test_plan_exchange_shapes():
    from moe_routers_b200.ep import plan_exchange

    counts_all = torch.arange(4 * 8, dtype=torch.int32).view(4, 8)
    send, recv = plan_exchange(counts_all, 1, 4)
    assert send == [int(counts_all[1, 0:2].sum()), 0, int(counts_all[1, 4:6].sum()), int(counts_all[1, 6:8].sum())]
    assert recv == [int(counts_all[0, 2:4].sum()), 0, int(counts_all[2, 2:4].sum()), int(counts_all[3, 2:4].sum())]
    with pytest.raises(ValueError):
        plan_exchange(torch.zeros(3, 8, dtype=torch.int32), 0, 3)
