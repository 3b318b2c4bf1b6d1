"""GPU parity of the fused router GEMM + select (tcgen05) and of the whole
fused route against the CPU oracle.  Calls go through the C ABI."""
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


def _inputs(t, d, e, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(t, d, generator=g).half()
    w = (torch.randn(e, d, generator=g) / d ** 0.5).half()
    return x, w


SHAPES = [
    (4096, 4096, 64, 2, 8, 2.0), (4096, 4096, 64, 2, 0, 0.0), (1000, 512, 64, 2, 8, 2.0),
    (130, 64, 16, 1, 0, 0.0), (257, 4096, 128, 4, 3, -1.5), (64, 200, 32, 2, 0, 0.0),
    (300, 1024, 256, 8, 16, 0.5), (1, 4096, 64, 2, 0, 0.0), (127, 136, 48, 3, 0, 0.0),
    (4096, 4096, 8, 2, 0, 0.0), (333, 512, 40, 5, 3, 1.0), (64, 64, 2, 2, 0, 0.0),
]


@pytest.mark.parametrize("t,d,e,k,skew_n,skew_b", SHAPES)
def test_router_gemm_select(ops, t, d, e, k, skew_n, skew_b):
    x, w = _inputs(t, d, e, 11 + t + d + e)
    idx, gates, logits = ops.router_gemm_select(x.cuda(), w.cuda(), k, skew_experts=skew_n, skew_bias=skew_b,
                                                return_logits=True)
    assert ops.read_status() == 0
    logits = logits.cpu().numpy()
    ref = oracle.router_logits(x.numpy(), w.numpy(), skew_experts=skew_n, skew_bias=skew_b).astype(np.float32)
    # (1) logits: fp32 accumulation in a different order, rounded to fp16: equal up to one fp16 ulp
    # on a small fraction of entries (tolerance: one fp16 ulp = 2^-10 relative, doubled for the
    # second rounding after the skew add)
    np.testing.assert_allclose(logits, ref, rtol=2e-3, atol=1e-3)
    assert (logits != ref).mean() < 0.02
    # (2) selection is bit-exact given the logits the kernel selected from
    ref_idx, ref_g, _ = oracle.topk_select(logits, k)
    np.testing.assert_array_equal(idx.cpu().numpy(), ref_idx.astype(np.int32))
    np.testing.assert_allclose(gates.cpu().numpy(), ref_g, rtol=1e-5, atol=1e-7)
    # (3) against the oracle's own logits: rows whose selection margin exceeds the rounding noise agree
    o_idx, _, _ = oracle.topk_select(ref, k)
    srt = -np.sort(-ref, axis=1)
    margin = np.min(srt[:, :k] - srt[:, 1:k + 1], axis=1) if e > k else np.ones(t)
    rows = margin > 4e-3 * np.maximum(1.0, np.abs(srt[:, 0]))
    np.testing.assert_array_equal(idx.cpu().numpy()[rows], o_idx[rows].astype(np.int32))


@pytest.mark.parametrize("t,d,e,k,skew_n,skew_b", SHAPES[:5] + [(0, 64, 64, 2, 0, 0.0), (4736, 1024, 64, 2, 8, 2.0),
                                                    (5000, 1024, 64, 2, 0, 0.0), (31, 2048, 64, 8, 0, 0.0),
                                                    (1000, 8192, 32, 2, 0, 0.0), (513, 1024, 256, 3, 0, 0.0),
                                                    (9000, 256, 64, 2, 8, 2.0)])
def test_route_fused(ops, t, d, e, k, skew_n, skew_b):
    x, w = _inputs(t, d, e, 5 + t + d + e)
    o = ops.route_fused(x.cuda(), w.cuda(), k, skew_experts=skew_n, skew_bias=skew_b, return_logits=t > 0)
    assert ops.read_status() == 0
    idx = o["idx"].cpu().numpy()
    if t > 0:
        ref_idx, ref_g, _ = oracle.topk_select(o["logits"].cpu().numpy(), k)
        np.testing.assert_array_equal(idx, ref_idx.astype(np.int32))
    xr = x.view(torch.int16).numpy()
    packed, counts, offsets, row_route, route_row = oracle.pack_canonical(xr, idx, e)
    np.testing.assert_array_equal(o["counts"].cpu().numpy(), counts)
    np.testing.assert_array_equal(o["offsets"].cpu().numpy(), offsets)
    np.testing.assert_array_equal(o["row_route"].cpu().numpy(), row_route)
    np.testing.assert_array_equal(o["route_row"].cpu().numpy(), route_row)
    np.testing.assert_array_equal(o["packed"].view(torch.int16).cpu().numpy(), packed)
    assert int(o["offsets"][-1]) == t * k


def test_route_fused_matches_two_step_path(ops):
    """fused route == logits kernel output fed through the standalone select + pack."""
    x, w = _inputs(2048, 1024, 64, 3)
    xc, wc = x.cuda(), w.cuda()
    o = ops.route_fused(xc, wc, 2, skew_experts=8, skew_bias=2.0, return_logits=True)
    idx2, g2 = ops.topk_select(o["logits"], 2)
    assert torch.equal(idx2, o["idx"])
    torch.testing.assert_close(g2, o["gates"], rtol=1e-6, atol=1e-7)
    c, off, packed, rr, inv = ops.pack(xc, idx2, 64)
    assert torch.equal(packed, o["packed"]) and torch.equal(off, o["offsets"]) and torch.equal(rr, o["row_route"])


@pytest.mark.parametrize("t,d,e,k,skew_n,skew_b", [(1000, 1024, 64, 2, 8, 2.0), (300, 512, 48, 4, 0, 0.0)])
def test_route_fused_bf16(ops, t, d, e, k, skew_n, skew_b):
    """bf16 tokens and router weight: logits are rounded to bf16 (the dtype the reference's
    `x @ w.t()` yields for bf16 inputs); the selection is bit-exact given those logits."""
    g = torch.Generator().manual_seed(t + e)
    x = torch.randn(t, d, generator=g).bfloat16()
    w = (torch.randn(e, d, generator=g) / d ** 0.5).bfloat16()
    o = ops.route_fused(x.cuda(), w.cuda(), k, skew_experts=skew_n, skew_bias=skew_b, return_logits=True)
    assert ops.read_status() == 0
    ref = (x.float() @ w.float().t()).bfloat16()
    if skew_n:
        ref[:, :skew_n] += skew_b
    logits = o["logits"].cpu()
    # one bf16 ulp (2^-8 relative), twice when the skew add rounds again
    torch.testing.assert_close(logits, ref.float(), rtol=2 ** -7, atol=2 ** -7)
    ref_idx, ref_g, _ = oracle.topk_select(logits.numpy(), k)
    np.testing.assert_array_equal(o["idx"].cpu().numpy(), ref_idx.astype(np.int32))
    np.testing.assert_allclose(o["gates"].cpu().numpy(), ref_g, rtol=1e-5, atol=1e-7)
    packed, counts, offsets, row_route, _ = oracle.pack_canonical(x.view(torch.int16).numpy(), ref_idx, e)
    np.testing.assert_array_equal(o["packed"].view(torch.int16).cpu().numpy(), packed)
    np.testing.assert_array_equal(o["offsets"].cpu().numpy(), offsets)


def test_pack_scatter_reuses_the_histograms_of_the_route(ops):
    """moe_pack_scatter after moe_route_fused on the same workspace reproduces the pack into fresh buffers."""
    x, w = _inputs(2000, 512, 64, 9)
    xc, wc = x.cuda(), w.cuda()
    o = ops.route_fused(xc, wc, 2, skew_experts=8, skew_bias=2.0)
    fresh = dict(o, packed=torch.zeros_like(o["packed"]), counts=torch.zeros_like(o["counts"]),
                 offsets=torch.zeros_like(o["offsets"]), row_route=torch.zeros_like(o["row_route"]),
                 route_row=torch.zeros_like(o["route_row"]))
    ops.pack_scatter(xc, 64, fresh)
    for key in ("packed", "counts", "offsets", "row_route", "route_row"):
        assert torch.equal(fresh[key], o[key]), key
    # from another stream: the histograms are taken from o["workspace"], not from that stream's scratch
    other = dict(o, packed=torch.zeros_like(o["packed"]), counts=torch.zeros_like(o["counts"]),
                 offsets=torch.zeros_like(o["offsets"]))
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        ops.pack_scatter(xc, 64, other)
    side.synchronize()
    for key in ("packed", "counts", "offsets"):
        assert torch.equal(other[key], o[key]), key
