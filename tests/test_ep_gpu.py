"""GPU tests of the expert-parallel layer: the re-bucket kernel against numpy, the layer on one
rank, and (when the box has two GPUs) two NCCL ranks against the single-process oracle."""
import os
import socket

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _need_cuda(n=1):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} CUDA device(s)")


@pytest.mark.parametrize("world,rank,e,d,skip", [(4, 1, 16, 64, 1), (2, 0, 8, 40, -1), (8, 7, 64, 128, 7), (1, 0, 4, 8, -1)])
def test_rebucket_matches_numpy(world, rank, e, d, skip):
    _need_cuda()
    from moe_routers_b200 import _lib

    el = e // world
    rng = np.random.default_rng(world * 100 + rank)
    counts_all = rng.integers(0, 40, size=(world, e)).astype(np.int32)
    if world > 1:
        counts_all[rng.integers(0, world), :] = 0  # a rank that sends nothing
    lens = counts_all[:, rank * el:(rank + 1) * el].copy()  # [src, e_local]
    if skip >= 0:
        lens[skip] = 0
    total = int(lens.sum())
    src = rng.standard_normal((total, d)).astype(np.float16)
    # expected expert-major order
    a_off = np.concatenate([[0], np.cumsum(lens.reshape(-1))])
    expect = np.concatenate([src[a_off[s * el + ee]:a_off[s * el + ee + 1]] for ee in range(el) for s in range(world)]
                            + [np.zeros((0, d), np.float16)])
    exp_off = np.concatenate([[0], np.cumsum(lens.sum(axis=0))]).astype(np.int32)

    s_t = torch.from_numpy(src).cuda()
    dst = torch.zeros_like(s_t)
    back = torch.zeros_like(s_t)
    c_t = torch.from_numpy(counts_all).cuda()
    off_t = torch.full((el + 1,), -1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib.moe_ep_rebucket(s_t.data_ptr(), dst.data_ptr(), c_t.data_ptr(), e, world, rank, skip, 0, d, 2,
                                        0, el, off_t.data_ptr(), st))
    _lib.check(_lib.lib.moe_ep_rebucket(dst.data_ptr(), back.data_ptr(), c_t.data_ptr(), e, world, rank, skip, 1, d, 2,
                                        0, el, None, st))
    np.testing.assert_array_equal(dst.cpu().numpy(), expect)
    np.testing.assert_array_equal(off_t.cpu().numpy(), exp_off)
    np.testing.assert_array_equal(back.cpu().numpy(), src)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world,e,d", [(4, 16, 64), (2, 8, 40), (8, 64, 128), (1, 4, 8)])
def test_push_kernel_emulated_ranks(world, e, d):
    """Device-initiated dispatch and combine with all ranks emulated on one GPU: every "rank" pushes
    its packed rows into the owners' inboxes, then every owner pushes its inbox back; rows must land
    expert-major in the inbox and return to the exact packed slot they came from."""
    _need_cuda()
    from moe_routers_b200 import _lib

    el = e // world
    rng = np.random.default_rng(world + e)
    counts_all = rng.integers(0, 30, size=(world, e)).astype(np.int32)
    if world > 1:
        counts_all[rng.integers(0, world), rng.integers(0, e)] = 0
    c_t = torch.from_numpy(counts_all).cuda()
    packed = [torch.from_numpy(rng.standard_normal((int(counts_all[r].sum()) + 1, d)).astype(np.float16)).cuda()
              for r in range(world)]
    cap = int(counts_all.sum()) + 1
    inbox = [torch.zeros((cap, d), dtype=torch.float16, device="cuda") for _ in range(world)]
    home = [torch.zeros_like(packed[r]) for r in range(world)]
    in_ptrs = torch.tensor([t.data_ptr() for t in inbox], dtype=torch.int64, device="cuda")
    home_ptrs = torch.tensor([t.data_ptr() for t in home], dtype=torch.int64, device="cuda")
    offs = [torch.full((el + 1,), -1, dtype=torch.int32, device="cuda") for _ in range(world)]
    st = torch.cuda.current_stream().cuda_stream
    for r in range(world):
        _lib.check(_lib.lib.moe_ep_push(packed[r].data_ptr(), in_ptrs.data_ptr(), c_t.data_ptr(), e, world, r, 0, d, 2,
                                        offs[r].data_ptr(), st))
    off_r = np.concatenate([np.zeros((world, 1), np.int64), np.cumsum(counts_all, axis=1)], axis=1)
    for p_ in range(world):
        segs = [packed[s_].cpu().numpy()[off_r[s_, p_ * el + ee]:off_r[s_, p_ * el + ee + 1]]
                for ee in range(el) for s_ in range(world)]
        expect = np.concatenate(segs + [np.zeros((0, d), np.float16)])
        np.testing.assert_array_equal(inbox[p_].cpu().numpy()[:len(expect)], expect)
        exp_off = np.concatenate([[0], np.cumsum(counts_all[:, p_ * el:(p_ + 1) * el].sum(axis=0))]).astype(np.int32)
        np.testing.assert_array_equal(offs[p_].cpu().numpy(), exp_off)
    for r in range(world):
        _lib.check(_lib.lib.moe_ep_push(inbox[r].data_ptr(), home_ptrs.data_ptr(), c_t.data_ptr(), e, world, r, 1, d, 2,
                                        None, st))
    for r in range(world):
        n = int(counts_all[r].sum())
        np.testing.assert_array_equal(home[r].cpu().numpy()[:n], packed[r].cpu().numpy()[:n])


@pytest.mark.parametrize("world,e,d", [(4, 16, 64), (2, 8, 128), (8, 64, 256), (1, 4, 64)])
def test_row_targets_and_gemm_return_emulated_ranks(world, e, d):
    """Combine direction fused into the expert GEMM, all ranks emulated on one GPU: the row-target
    table must send inbox row i to the packed slot it came from (checked against moe_ep_push in
    combine mode), and moe_grouped_gemm_rows through that table must leave in every home buffer
    exactly what the dense GEMM followed by the combine push leaves."""
    _need_cuda()
    from moe_routers_b200 import _lib, ops

    el = e // world
    rng = np.random.default_rng(3 * world + e)
    counts_all = rng.integers(0, 70, size=(world, e)).astype(np.int32)
    if world > 1:
        counts_all[rng.integers(0, world), rng.integers(0, e)] = 0
    c_t = torch.from_numpy(counts_all).cuda()
    n_home = [int(counts_all[r].sum()) for r in range(world)]
    n_in = [int(counts_all[:, r * el:(r + 1) * el].sum()) for r in range(world)]
    inbox = [torch.from_numpy(rng.standard_normal((n_in[r] + 1, d)).astype(np.float16)).cuda() for r in range(world)]
    w = [torch.from_numpy((rng.standard_normal((el, d, d)) / d ** 0.5).astype(np.float16)).cuda() for _ in range(world)]
    home_a = [torch.zeros((n_home[r] + 1, d), dtype=torch.float16, device="cuda") for r in range(world)]
    home_b = [torch.zeros_like(t) for t in home_a]
    ptr_a = torch.tensor([t.data_ptr() for t in home_a], dtype=torch.int64, device="cuda")
    ptr_b = torch.tensor([t.data_ptr() for t in home_b], dtype=torch.int64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for r in range(world):
        off = np.concatenate([[0], np.cumsum(counts_all[:, r * el:(r + 1) * el].sum(axis=0))]).astype(np.int32)
        off_t = torch.from_numpy(off).cuda()
        # path A: dense GEMM, then the combine push
        y = ops.grouped_gemm(inbox[r][:n_in[r]], w[r], off_t, layout="nk")
        if n_in[r]:
            _lib.check(_lib.lib.moe_ep_push(y.data_ptr(), ptr_a.data_ptr(), c_t.data_ptr(), e, world, r, 1, d, 2,
                                            None, st))
        # path B: row targets, then the GEMM storing through them
        table = torch.zeros(n_in[r] + 1, dtype=torch.int64, device="cuda")
        _lib.check(_lib.lib.moe_ep_row_targets(ptr_b.data_ptr(), c_t.data_ptr(), e, world, r, d, 2,
                                               table.data_ptr(), st))
        assert int(table[n_in[r]]) == 0  # nothing written past the last inbox row
        if n_in[r]:
            ops.grouped_gemm(inbox[r][:n_in[r]], w[r], off_t, layout="nk", out_rows=table)
    torch.cuda.synchronize()
    assert ops.read_status() == 0
    for r in range(world):
        assert torch.equal(home_a[r], home_b[r])
        assert home_a[r][:n_home[r]].abs().sum() > 0 or n_home[r] == 0


@pytest.mark.parametrize("world,e,d,k", [(4, 16, 64, 2), (2, 8, 128, 1), (8, 64, 4096, 2), (1, 4, 64, 3)])
def test_direct_dispatch_emulated_ranks(world, e, d, k):
    """Dispatch fused into the pack, all ranks emulated on one GPU: moe_pack_scatter_to with the
    segment bases of moe_ep_segment_bases must fill every owner's inbox exactly as pack + dispatch
    push does (itself checked against numpy above), and the plan must equal the pack's outputs."""
    _need_cuda()
    from moe_routers_b200 import _lib, ops

    el = e // world
    rng = np.random.default_rng(7 * world + e + k)
    tokens = [int(rng.integers(40, 300)) for _ in range(world)]
    xs = [torch.from_numpy(rng.standard_normal((t, d)).astype(np.float16)).cuda() for t in tokens]
    idxs = []
    for t in tokens:
        scores = rng.random((t, e))
        scores[:, 0] += 0.5  # a hot expert
        idxs.append(torch.from_numpy(np.argsort(-scores, axis=1)[:, :k].astype(np.int32)).cuda())
    counts_all = np.stack([np.bincount(i.cpu().numpy().reshape(-1), minlength=e) for i in idxs]).astype(np.int32)
    c_t = torch.from_numpy(counts_all).cuda()
    cap = int(counts_all.sum()) + 1
    inbox_a = [torch.zeros((cap, d), dtype=torch.float16, device="cuda") for _ in range(world)]
    inbox_b = [torch.zeros_like(t) for t in inbox_a]
    ptr_a = torch.tensor([t.data_ptr() for t in inbox_a], dtype=torch.int64, device="cuda")
    ptr_b = torch.tensor([t.data_ptr() for t in inbox_b], dtype=torch.int64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for r in range(world):
        counts, offsets, packed, row_route, route_row = ops.pack(xs[r], idxs[r], e)
        off_a = torch.full((el + 1,), -1, dtype=torch.int32, device="cuda")
        _lib.check(_lib.lib.moe_ep_push(packed.data_ptr(), ptr_a.data_ptr(), c_t.data_ptr(), e, world, r, 0, d, 2,
                                        off_a.data_ptr(), st))
        plan = ops.route_plan(xs[r], idxs[r], e)
        for key, ref in (("counts", counts), ("offsets", offsets), ("row_route", row_route), ("route_row", route_row)):
            assert torch.equal(plan[key], ref), key
        seg = torch.zeros(e, dtype=torch.int64, device="cuda")
        off_b = torch.full((el + 1,), -1, dtype=torch.int32, device="cuda")
        _lib.check(_lib.lib.moe_ep_segment_bases(ptr_b.data_ptr(), c_t.data_ptr(), e, world, r, d, 2, seg.data_ptr(),
                                                 off_b.data_ptr(), st))
        ops.pack_scatter_to(xs[r], e, plan, seg)
        assert torch.equal(off_a, off_b)
        for key, ref in (("counts", counts), ("offsets", offsets), ("row_route", row_route), ("route_row", route_row)):
            assert torch.equal(plan[key], ref), key
    torch.cuda.synchronize()
    assert ops.read_status() == 0
    for p_ in range(world):
        assert torch.equal(inbox_a[p_], inbox_b[p_])
        assert inbox_a[p_].abs().sum() > 0


def test_scatter_to_and_gemm_rows_edge_cases():
    """Rows that are not a multiple of 16 bytes are refused (no silent slow path to peer memory);
    zero tokens give zero counts; an expert nobody routes to leaves its segment untouched."""
    _need_cuda()
    from moe_routers_b200 import _lib, ops

    e, k = 8, 2
    # 1) 6-byte rows: unsupported, with a message
    x = torch.randn(64, 3).half().cuda()
    idx = torch.randint(0, e, (64, k), dtype=torch.int32).cuda()
    plan = ops.route_plan(x, idx, e)
    seg = torch.zeros(e, dtype=torch.int64, device="cuda")
    with pytest.raises(_lib.MoeError) as err:
        ops.pack_scatter_to(x, e, plan, seg)
    assert err.value.code == _lib.MOE_ERR_UNSUPPORTED
    # 2) zero tokens
    x0 = torch.zeros((0, 64), dtype=torch.float16, device="cuda")
    i0 = torch.zeros((0, k), dtype=torch.int32, device="cuda")
    p0 = ops.route_plan(x0, i0, e)
    ops.pack_scatter_to(x0, e, p0, seg)
    assert int(p0["counts"].sum()) == 0 and int(p0["offsets"][-1]) == 0
    # 3) experts 3 and 5 get nothing: their segments keep the fill value, the others hold the rows
    t, d = 200, 64
    g = torch.Generator().manual_seed(5)
    x = torch.randn(t, d, generator=g).half().cuda()
    choices = torch.tensor([0, 1, 2, 4, 6, 7])
    idx = choices[torch.stack([torch.randperm(6, generator=g)[:k] for _ in range(t)])].to(torch.int32).cuda()
    plan = ops.route_plan(x, idx, e)
    segs = [torch.full((t * k, d), 9.0, dtype=torch.float16, device="cuda") for _ in range(e)]
    seg = torch.tensor([s_.data_ptr() for s_ in segs], dtype=torch.int64, device="cuda")
    ops.pack_scatter_to(x, e, plan, seg)
    counts, offsets, packed, _, _ = ops.pack(x, idx, e)
    torch.cuda.synchronize()
    assert ops.read_status() == 0
    for ee in range(e):
        n = int(counts[ee])
        lo = int(offsets[ee])
        assert torch.equal(segs[ee][:n], packed[lo:lo + n])
        assert (segs[ee][n:] == 9.0).all()
    assert int(counts[3]) == 0 and int(counts[5]) == 0
    # 4) grouped GEMM with a row table and zero rows: nothing happens, no error
    a0 = torch.zeros((0, 64), dtype=torch.float16, device="cuda")
    w = torch.zeros((e, 64, 64), dtype=torch.float16, device="cuda")
    ops.grouped_gemm(a0, w, torch.zeros(e + 1, dtype=torch.int32, device="cuda"), layout="nk",
                     out_rows=torch.zeros(1, dtype=torch.int64, device="cuda"))


def test_rank_signals_emulated_ranks():
    """moe_ep_signal / moe_ep_wait with all ranks emulated on one GPU.  Kernels that wait on one
    another must not share a GPU, so every rank signals first and only then do the ranks wait: each
    wait finds its flags already set.  Checks the payload (per-expert counts) in every rank's table,
    two calls in a row (values grow, nothing is cleared) and a clean status."""
    _need_cuda()
    from moe_routers_b200 import _lib, ops

    world, e = 4, 16
    tables = [torch.zeros(3 * world + 2 * world * e, dtype=torch.int32, device="cuda") for _ in range(world)]
    flag_ptrs = torch.tensor([t.data_ptr() for t in tables], dtype=torch.int64, device="cuda")
    counts_ptrs = torch.tensor([t.data_ptr() + 4 * 3 * world for t in tables], dtype=torch.int64, device="cuda")
    ws = ops.workspace(torch.device("cuda", torch.cuda.current_device()), 1, e, 2)
    st = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(0)
    for call in (1, 2):
        par = call & 1
        counts = [torch.from_numpy(rng.integers(0, 99, size=e).astype(np.int32)).cuda() for _ in range(world)]
        for r in range(world):
            _lib.check(_lib.lib.moe_ep_signal(flag_ptrs.data_ptr(), world, r, 0, call, counts[r].data_ptr(),
                                              counts_ptrs.data_ptr(), (par * world + r) * e, e, st))
            _lib.check(_lib.lib.moe_ep_signal(flag_ptrs.data_ptr(), world, r, 2, call, None, None, 0, 0, st))
        for r in range(world):
            _lib.check(_lib.lib.moe_ep_wait(tables[r].data_ptr(), world, 0, call, ws.data_ptr(), ws.numel(), st))
            _lib.check(_lib.lib.moe_ep_wait(tables[r].data_ptr(), world, 2, call, ws.data_ptr(), ws.numel(), st))
        torch.cuda.synchronize()
        for r in range(world):
            tab = tables[r].cpu().numpy()
            np.testing.assert_array_equal(tab[0:world], call)                 # slot 0
            np.testing.assert_array_equal(tab[world:2 * world], 0)            # slot 1 untouched
            np.testing.assert_array_equal(tab[2 * world:3 * world], call)     # slot 2
            got = tab[3 * world:].reshape(2, world, e)[par]
            np.testing.assert_array_equal(got, np.stack([c.cpu().numpy() for c in counts]))
    assert ops.read_status() == 0


def test_wait_that_runs_out_reports_instead_of_hanging():
    """Failure detection without a GPU fault: a wait for a rank that never signals runs out after the
    workspace's wait limit (set to 2 ms here), the kernel returns, the status block names the rank,
    moe_read_status maps it to MOE_ERR_DEVICE, and the context stays usable."""
    _need_cuda()
    import ctypes
    import time

    from moe_routers_b200 import _lib

    world = 4
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    table = torch.zeros(3 * world, dtype=torch.int32, device="cuda")
    table[0:world] = torch.tensor([1, 1, 0, 1], dtype=torch.int32)  # rank 2 never arrived at call 1
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib.moe_workspace_init(ws.data_ptr(), ws.numel(), st))
    _lib.check(_lib.lib.moe_set_wait_limit(ws.data_ptr(), ws.numel(), 2_000_000, st))
    t0 = time.time()
    _lib.check(_lib.lib.moe_ep_wait(table.data_ptr(), world, 0, 1, ws.data_ptr(), ws.numel(), st))
    out = ctypes.c_int(0)
    rc = _lib.lib.moe_read_status(ws.data_ptr(), st, ctypes.byref(out))
    assert time.time() - t0 < 5.0
    assert rc == _lib.MOE_ERR_DEVICE and out.value == (0x400 | 2)
    assert "peer rank" in _lib.last_error()
    with pytest.raises(_lib.MoeError):
        _lib.check(rc)
    # the context is alive: clear the status block and run a wait that is satisfied
    _lib.check(_lib.lib.moe_workspace_init(ws.data_ptr(), ws.numel(), st))
    table[2] = 1
    _lib.check(_lib.lib.moe_ep_wait(table.data_ptr(), world, 0, 1, ws.data_ptr(), ws.numel(), st))
    assert _lib.lib.moe_read_status(ws.data_ptr(), st, ctypes.byref(out)) == 0 and out.value == 0


def _ep_worker(rank, world, port, strategy, q):
    try:
        import torch.distributed as dist

        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        import datetime

        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                                timeout=datetime.timedelta(seconds=90))
        from moe_routers_b200.ep import EPMoELayer

        strategy, _, dt_name = strategy.partition(":")
        dt = torch.bfloat16 if dt_name == "bf16" else torch.float16
        tol = 6e-2 if dt == torch.bfloat16 else 2e-2  # bf16 keeps 8 significand bits, fp16 11
        t, d, h, e, k = 512 + 64 * rank, 256, 512, 16, 2
        el = e // world
        gw = torch.Generator().manual_seed(0)
        w_router = (torch.randn(e, d, generator=gw) / d ** 0.5).to(dt)
        w1 = (torch.randn(e, h, d, generator=gw) / d ** 0.5).to(dt)
        w2 = (torch.randn(e, d, h, generator=gw) / h ** 0.5).to(dt)
        gx = torch.Generator().manual_seed(10 + rank)
        x = torch.randn(t, d, generator=gx).to(dt)
        layers = {tr: EPMoELayer(w_router.cuda(), w1[rank * el:(rank + 1) * el].cuda().contiguous(),
                                 w2[rank * el:(rank + 1) * el].cuda().contiguous(), k, activation="gelu",
                                 strategy=strategy, skew_experts=4, skew_bias=2.0, transport=tr)
                  for tr in ("peer", "nccl")}
        outs = {}
        # peer: fused exchanges twice in a row (buffers and flags are reused), the unfused kernels under
        # overlap=True, and the serial chain (overlap=False); nccl: two streams and one stream
        for tr, overlap, fuse in (("peer", True, True), ("peer", True, True), ("peer", True, False),
                                  ("peer", False, True), ("nccl", True, None), ("nccl", False, None)):
            layer = layers[tr]
            if fuse is not None:
                layer.fuse_combine = fuse  # second GEMM returns its rows itself / dense result + push
                layer.direct_dispatch = fuse  # pack stores into the owners' inboxes / local pack + push
            out = layer(x.cuda(), overlap=overlap)
            torch.cuda.synchronize()
            outs[(tr, fuse, overlap)] = out.clone()
            o = layer.last["route"]
            experts = {"w1": w1.float().numpy(), "w2": w2.float().numpy()}
            ref, _ = oracle.moe_layer(x.float().numpy(), o["idx"].cpu().numpy(), o["gates"].cpu().numpy(), experts,
                                      kind="gelu", layout="nk")
            ref = ref.astype(np.float32)
            scale = np.abs(ref).max()
            # layer outputs: 2e-2 relative to the output scale (fp16), 6e-2 for bf16
            np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=tol, atol=tol * scale)
        # the same kernels did the arithmetic in both peer variants: identical bits
        assert torch.equal(outs[("peer", True, True)], outs[("peer", False, True)])
        assert torch.equal(outs[("peer", True, True)], outs[("peer", True, False)])
        from moe_routers_b200 import ops as _ops

        assert _ops.read_status() == 0  # no bounded wait (mbarrier, rank signal) gave up
        # a batch larger than the buffers set up at the first call is refused, on every rank alike
        big = torch.zeros((t + 2048, d), dtype=dt, device="cuda")
        try:
            layers["peer"](big)
            raise AssertionError("oversized batch was accepted")
        except RuntimeError as exc:
            assert "max_tokens" in str(exc)
        dist.barrier()
        for layer in layers.values():
            layer.close()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as exc:  # pragma: no cover
        import traceback

        q.put((rank, "".join(traceback.format_exception(exc))))


def _run_ranks(world, strategy):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, world, port, strategy, q)) for r in range(world)]
    for p in procs:
        p.start()
    # A rank that raises leaves its peers waiting in a collective: stop them as soon as the first
    # failure is known (or nothing has been heard for two minutes) instead of waiting them out.
    import queue

    results = []
    try:
        while len(results) < world:
            results.append(q.get(timeout=120))
            if results[-1][1] != "ok":
                break
    except queue.Empty:
        results.append((-1, "no result from the remaining ranks within 120 s"))
    for p in procs:
        p.join(timeout=20 if all(m == "ok" for _, m in results) else 1)
        if p.is_alive():
            p.terminate()
            p.join(timeout=10)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"
    assert len(results) == world


@pytest.mark.parametrize("strategy", ["fused_select", "sinkhorn", "fused_select:bf16"])
def test_ep_layer_single_rank(strategy):
    _need_cuda(1)
    _run_ranks(1, strategy)


@pytest.mark.parametrize("strategy", ["fused_select", "sinkhorn", "fused_select:bf16"])
def test_ep_layer_two_ranks(strategy):
    _need_cuda(2)
    _run_ranks(2, strategy)
