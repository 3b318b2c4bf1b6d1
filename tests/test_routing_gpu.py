"""GPU parity of select / pack / combine against the CPU oracle and the golden
vectors of the reference.  Every call goes through the C ABI."""
import os

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from moe_routers_b200 import ops as _ops

    return _ops


def _rand_logits(t, e, dtype, seed, ties=False):
    g = torch.Generator().manual_seed(seed)
    v = torch.randn(t, e, generator=g)
    if ties:
        v = torch.round(v * 2) / 2  # many exact ties
    return v.to(dtype)


@pytest.mark.parametrize("t,e,k,dtype,ties", [
    (4096, 64, 2, torch.float16, False), (4096, 64, 2, torch.float32, False),
    (1000, 64, 2, torch.bfloat16, False), (513, 64, 2, torch.float16, True),
    (129, 64, 8, torch.float32, True), (127, 8, 2, torch.float32, False),
    (1, 64, 2, torch.float16, False), (3, 48, 3, torch.float32, True),
    (65, 256, 4, torch.float16, True), (33, 1000, 8, torch.float32, False),
    (17, 5, 5, torch.float32, True), (64, 16, 1, torch.bfloat16, True),
])
def test_topk_select_bit_exact(ops, t, e, k, dtype, ties):
    logits = _rand_logits(t, e, dtype, 100 + t + e + k, ties)
    idx, gates = ops.topk_select(logits.cuda(), k)
    ref_idx, ref_g, _ = oracle.topk_select(logits.float().numpy(), k)
    np.testing.assert_array_equal(idx.cpu().numpy(), ref_idx.astype(np.int32))
    # fp32 gate tolerance: 1e-5 relative
    np.testing.assert_allclose(gates.cpu().numpy(), ref_g, rtol=1e-5, atol=1e-7)
    assert ops.read_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_topk_select_16bit_special_values(ops, dtype):
    """The key-based kernel for 16-bit logits: -inf rows select in index order, +inf wins, -0 ties +0
    (lower index first), all-equal rows pick the first columns; E = 8 ... 1024, k = 1 ... 8."""
    logits = torch.full((5, 64), float("-inf"), dtype=dtype)
    logits[1, 7] = 1.0
    logits[2, 63] = float("inf")
    logits[3, :] = 0.0
    logits[4, :] = -0.0
    logits[4, 9] = 0.0
    logits[4, 3] = -1.0
    idx, gates = ops.topk_select(logits.cuda(), 2)
    np.testing.assert_array_equal(idx.cpu().numpy(), [[0, 1], [7, 0], [63, 0], [0, 1], [0, 1]])
    np.testing.assert_allclose(gates.cpu().numpy()[3:], 0.5)
    np.testing.assert_allclose(gates.cpu().numpy()[1], [1.0, 0.0])
    for t, e, k in [(100, 8, 2), (33, 1024, 8), (257, 128, 4), (64, 40, 1), (1000, 512, 3)]:
        g = torch.Generator().manual_seed(t + e)
        v = (torch.round(torch.randn(t, e, generator=g) * 4) / 4).to(dtype)  # many ties
        idx, gates = ops.topk_select(v.cuda(), k)
        ref_idx, ref_g, _ = oracle.topk_select(v.float().numpy(), k)
        np.testing.assert_array_equal(idx.cpu().numpy(), ref_idx.astype(np.int32))
        np.testing.assert_allclose(gates.cpu().numpy(), ref_g, rtol=1e-5, atol=1e-7)
    # a view that starts 2 bytes into an allocation is not 16-byte aligned: the generic kernel takes it
    base = torch.randn(65 * 64 + 8, generator=torch.Generator().manual_seed(1)).to(dtype).cuda()
    off = base[1:1 + 64 * 64].view(64, 64)
    idx, _ = ops.topk_select(off, 2)
    ref_idx, _, _ = oracle.topk_select(off.float().cpu().numpy(), 2)
    np.testing.assert_array_equal(idx.cpu().numpy(), ref_idx.astype(np.int32))


def test_topk_select_handles_infinities(ops):
    logits = torch.full((4, 64), float("-inf"))
    logits[1, 7] = 1.0
    logits[2, 63] = float("inf")
    logits[3, :] = 0.0
    idx, gates = ops.topk_select(logits.cuda(), 2)
    np.testing.assert_array_equal(idx.cpu().numpy(), [[0, 1], [7, 0], [63, 0], [0, 1]])


@pytest.mark.parametrize("tag,k", [("f32_e64_k2", 2), ("f32_e64_k8", 8), ("f32_e8_k2", 2),
                                   ("f32_e64_k1", 1), ("f16_e64_k2", 2), ("f32_e48_k3", 3)])
def test_topk_select_matches_reference_golden(ops, golden_dir, tag, k):
    g = np.load(os.path.join(golden_dir, "topk_router.npz"))
    logits, ref_idx, ref_w = g[f"{tag}_logits"], g[f"{tag}_idx"], g[f"{tag}_w"]
    idx, gates = ops.topk_select(torch.from_numpy(logits).cuda(), k)
    idx = idx.cpu().numpy()
    v = np.sort(logits.astype(np.float32), axis=1)[:, ::-1]
    rows = np.all(v[:, :k] != v[:, 1:k + 1], axis=1) if logits.shape[1] > k else np.ones(len(v), bool)
    np.testing.assert_array_equal(idx[rows], ref_idx[rows].astype(np.int32))
    tol = 1e-3 if logits.dtype == np.float16 else 1e-5
    np.testing.assert_allclose(gates.cpu().numpy()[rows], ref_w[rows].astype(np.float32), rtol=tol, atol=tol * 0.1)


def _random_routes(t, e, k, seed, skew=False):
    rng = np.random.default_rng(seed)
    if skew:
        p = np.ones(e)
        p[: max(1, e // 8)] = 40.0
        p /= p.sum()
    else:
        p = None
    idx = np.stack([rng.choice(e, size=k, replace=False, p=p) for _ in range(t)]).astype(np.int32) if t else np.zeros((0, k), np.int32)
    return idx


@pytest.mark.parametrize("t,d,e,k,dtype,skew", [
    (4096, 4096, 64, 2, torch.float16, False), (4096, 4096, 64, 2, torch.float16, True),
    (1, 64, 64, 2, torch.float16, False), (3, 40, 8, 2, torch.float16, False),
    (127, 72, 64, 2, torch.float16, True), (129, 100, 16, 4, torch.float32, False),
    (1000, 250, 64, 8, torch.bfloat16, True), (33, 3, 4, 1, torch.float16, False),
    (257, 36, 300, 3, torch.float16, False), (0, 64, 64, 2, torch.float16, False),
    # more than 256 tiles of 32 tokens: the separate per-expert scan kernel computes the tile bases
    (10000, 64, 64, 2, torch.float16, True), (8193, 24, 8, 4, torch.float16, False),
    (20000, 128, 256, 1, torch.bfloat16, False),
])
def test_pack_bit_exact(ops, t, d, e, k, dtype, skew):
    idx = _random_routes(t, e, k, 7 + t + d, skew)
    x = torch.randn(t, d, generator=torch.Generator().manual_seed(t + d)).to(dtype)
    counts, offsets, packed, row_route, route_row = ops.pack(x.cuda(), torch.from_numpy(idx).cuda(), e)
    xr = x.view(torch.int16 if x.element_size() == 2 else torch.int32).numpy()
    ref_packed, ref_counts, ref_offsets, ref_rr, ref_inv = oracle.pack_canonical(xr, idx, e)
    np.testing.assert_array_equal(counts.cpu().numpy(), ref_counts)
    np.testing.assert_array_equal(offsets.cpu().numpy(), ref_offsets)
    np.testing.assert_array_equal(row_route.cpu().numpy(), ref_rr)
    np.testing.assert_array_equal(route_row.cpu().numpy(), ref_inv)
    got = packed.view(torch.int16 if x.element_size() == 2 else torch.int32).cpu().numpy()
    np.testing.assert_array_equal(got, ref_packed)
    assert int(offsets[-1]) == t * k  # kernels/fused_select.cu:292
    assert ops.read_status() == 0


def test_pack_all_routes_to_one_expert_and_empty_experts(ops):
    t, d, e, k = 300, 64, 64, 2
    idx = np.zeros((t, k), np.int32)
    idx[:, 0] = 5
    idx[:, 1] = 63
    x = torch.randn(t, d).half()
    counts, offsets, packed, row_route, _ = ops.pack(x.cuda(), torch.from_numpy(idx).cuda(), e)
    c = counts.cpu().numpy()
    assert c[5] == t and c[63] == t and c.sum() == 2 * t
    np.testing.assert_array_equal(packed[:t].cpu().numpy(), x.numpy())
    np.testing.assert_array_equal(packed[t:].cpu().numpy(), x.numpy())


def test_pack_is_deterministic_and_guards_output(ops):
    t, d, e, k = 2048, 512, 64, 2
    idx = torch.from_numpy(_random_routes(t, e, k, 3)).cuda()
    x = torch.randn(t, d, device="cuda").half()
    a = ops.pack(x, idx, e)
    b = ops.pack(x, idx, e)
    for u, v in zip(a, b):
        assert torch.equal(u, v)


def test_pack_reports_bad_expert_index(ops):
    idx = torch.tensor([[0, 99], [1, 2]], dtype=torch.int32).cuda()
    x = torch.randn(2, 16).half().cuda()
    ops.pack(x, idx, 8)
    from moe_routers_b200 import _lib
    with pytest.raises(_lib.MoeError, match="out of range"):
        ops.read_status()
    # clear the status block again for later tests
    ws = ops.workspace(x.device, 1, 1, 1)
    _lib.check(_lib.lib.moe_workspace_init(ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream))
    assert ops.read_status() == 0


@pytest.mark.parametrize("t,d,k,dtype", [
    (4096, 4096, 2, torch.float16), (1000, 520, 2, torch.bfloat16), (129, 100, 4, torch.float16),
    (1, 8, 1, torch.float16), (65, 36, 8, torch.float16), (333, 4096, 3, torch.float16),
])
def test_combine_matches_oracle(ops, t, d, k, dtype):
    g = torch.Generator().manual_seed(t + d + k)
    y = torch.randn(t * k, d, generator=g).to(dtype)
    gates = torch.rand(t, k, generator=g)
    gates = gates / gates.sum(-1, keepdim=True)
    route_row = torch.randperm(t * k, generator=g).to(torch.int32)
    out = ops.combine(y.cuda(), gates.cuda(), route_row.cuda(), k)
    ref = oracle.combine(y.float().numpy(), gates.numpy(), route_row.numpy(), k, out_dtype=np.float32)
    # one rounding to the storage type: 2^-11 (fp16) / 2^-8 (bf16) relative
    tol = 1e-3 if dtype == torch.float16 else 8e-3
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=tol, atol=tol)


def test_pack_then_combine_round_trip_is_identity(ops):
    """Size-independent property at the benchmark size: packing x and combining
    the packed rows with gates that sum to one returns x."""
    t, d, e, k = 4096, 4096, 64, 2
    x = torch.randn(t, d, device="cuda").half()
    logits = torch.randn(t, e, device="cuda").half()
    idx, gates = ops.topk_select(logits, k)
    counts, offsets, packed, row_route, route_row = ops.pack(x, idx, e)
    half = torch.full_like(gates, 0.5)
    out = ops.combine(packed, half, route_row, k)
    assert torch.equal(out, x)
    assert int(counts.sum()) == t * k
    # every packed row sits inside its expert's segment
    eid = torch.repeat_interleave(torch.arange(e, device="cuda"), counts.long())
    assert torch.equal(eid, idx.reshape(-1)[row_route.long()].long())


@pytest.mark.parametrize("t,d,e,k,dtype", [(4096, 1024, 64, 2, torch.float16), (1000, 72, 48, 3, torch.float32),
                                           (33, 8, 1000, 8, torch.bfloat16), (9000, 64, 64, 2, torch.float16),
                                           (1, 16, 2, 1, torch.float16)])
def test_fused_select_equals_select_then_pack(ops, t, d, e, k, dtype):
    """moe_fused_select (select + tile histograms in one launch, then scatter) gives exactly what
    the standalone select followed by the standalone pack gives."""
    logits = _rand_logits(t, e, dtype, 5 + t + e, ties=True).cuda()
    x = torch.randn(t, d, generator=torch.Generator().manual_seed(t)).half().cuda()
    idx, gates, counts, offsets, packed, row_route, route_row = ops.fused_select(logits, x, e, k)
    idx2, gates2 = ops.topk_select(logits, k)
    c2, o2, p2, rr2, ir2 = ops.pack(x, idx2, e)
    assert torch.equal(idx, idx2) and torch.equal(gates, gates2)
    assert torch.equal(counts, c2) and torch.equal(offsets, o2) and torch.equal(packed, p2)
    assert torch.equal(row_route, rr2) and torch.equal(route_row, ir2)
    assert ops.read_status() == 0
