"""Pin the CPU oracle against golden vectors produced by the reference itself
(tests/golden/make_golden.py).  CPU only."""
import os

import numpy as np
import pytest
import torch

import oracle


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def _tie_free_rows(logits, k):
    """Rows whose k-th and (k+1)-th largest values differ (torch.topk leaves
    the order among equal values unspecified)."""
    v = np.sort(logits.astype(np.float32), axis=1)[:, ::-1]
    ok = np.ones(v.shape[0], dtype=bool)
    for j in range(min(k, v.shape[1] - 1)):
        ok &= v[:, j] != v[:, j + 1]
    return ok


@pytest.mark.parametrize("tag,k", [("f32_e64_k2", 2), ("f32_e64_k8", 8), ("f32_e8_k2", 2),
                                   ("f32_e64_k1", 1), ("f16_e64_k2", 2), ("f32_e48_k3", 3)])
def test_topk_router_matches_reference(golden_dir, tag, k):
    g = _load(golden_dir, "topk_router.npz")
    logits, ref_idx, ref_w = g[f"{tag}_logits"], g[f"{tag}_idx"], g[f"{tag}_w"]
    idx, w, _ = oracle.topk_select(logits, k)
    rows = _tie_free_rows(logits, k)
    assert rows.sum() >= 0.9 * len(rows)
    np.testing.assert_array_equal(idx[rows], ref_idx[rows])
    if logits.dtype == np.float16:
        np.testing.assert_allclose(w[rows], ref_w[rows].astype(np.float32), rtol=1e-3, atol=1e-4)
    else:
        np.testing.assert_allclose(w[rows], ref_w[rows], rtol=1e-5, atol=1e-7)
    # on tie rows the contract is "lowest index wins": the selected VALUES still match
    vals = np.take_along_axis(logits.astype(np.float32), idx, 1)
    ref_vals = np.take_along_axis(logits.astype(np.float32), ref_idx, 1)
    np.testing.assert_array_equal(vals, ref_vals)


def test_topk_lowest_index_wins():
    logits = np.zeros((3, 8), dtype=np.float32)
    logits[1, [5, 2, 7]] = 1.0
    logits[2, 3] = -1.0
    idx, w, _ = oracle.topk_select(logits, 2)
    np.testing.assert_array_equal(idx, [[0, 1], [2, 5], [0, 1]])
    np.testing.assert_allclose(w, 0.5)


def test_fused_select_gates_match_softmax():
    rng = np.random.default_rng(0)
    v = rng.standard_normal((100, 2)).astype(np.float32) * 5
    v = -np.sort(-v, axis=1)
    ref = torch.softmax(torch.from_numpy(v), dim=-1).numpy()
    np.testing.assert_allclose(oracle.fused_select_gates(v), ref, rtol=1e-6)


@pytest.mark.parametrize("tag", ["f32_it10", "f16_it10", "f16_it10_skew", "f32_it3_t07"])
def test_sinkhorn_router_matches_reference(golden_dir, tag):
    g = _load(golden_dir, "sinkhorn_router.npz")
    logits, ref_idx, ref_w = g[f"{tag}_logits"], g[f"{tag}_idx"], g[f"{tag}_w"]
    k, iters, temp, eps = g[f"{tag}_cfg"]
    idx, w, q = oracle.sinkhorn_route(logits, int(k), iters=int(iters), epsilon=float(eps), temperature=float(temp))
    # rows whose selection margin in q is far above fp32 summation noise must agree exactly
    qs = -np.sort(-q, axis=1)
    kk = int(k)
    margin = np.min(qs[:, :kk] - qs[:, 1 : kk + 1], axis=1) / qs[:, 0]
    rows = margin > 1e-4
    assert rows.mean() > 0.95
    np.testing.assert_array_equal(idx[rows], ref_idx[rows])
    tol = 2e-3 if logits.dtype == np.float16 else 1e-4
    np.testing.assert_allclose(w[rows], ref_w[rows].astype(np.float32), rtol=tol, atol=tol)


def test_sinkhorn_is_invariant_to_a_column_bias(golden_dir):
    g = _load(golden_dir, "sinkhorn_router.npz")
    logits = g["f32_it10_logits"]
    biased = logits.copy()
    biased[:, :8] += 2.0
    a, _, qa = oracle.sinkhorn_route(logits, 2)
    b, _, qb = oracle.sinkhorn_route(biased, 2)
    ca, _ = oracle.counts_offsets(a, 64)
    cb, _ = oracle.counts_offsets(b, 64)
    assert oracle.load_skew(ca)[1] < 0.35 and oracle.load_skew(cb)[1] < 0.35
    assert (a == b).mean() > 0.9


def test_pack_matches_reference_up_to_segment_order(golden_dir):
    g = _load(golden_dir, "pack_routes.npz")
    x, idx, w = g["x"], g["idx"], g["w"]
    packed, counts, offsets, row_route, route_row = oracle.pack_canonical(x, idx, 8)
    k = idx.shape[1]
    ref_exp, ref_tok = g["expert_ids_sorted"], g["token_ids_sorted"]
    # expert ids of the packed rows are identical; token multisets per segment are identical
    np.testing.assert_array_equal(np.repeat(np.arange(8), counts), ref_exp)
    for e in range(8):
        lo, hi = offsets[e], offsets[e + 1]
        np.testing.assert_array_equal(np.sort(row_route[lo:hi] // k), np.sort(ref_tok[lo:hi]))
        # the reference packs gate-weighted rows; undo the order and compare values
        order = np.argsort(ref_tok[lo:hi], kind="stable")
        mine = packed[lo:hi] * w.reshape(-1)[row_route[lo:hi], None]
        np.testing.assert_allclose(mine, g["x_route_sorted"][lo:hi][order], rtol=1e-6)
    assert offsets[-1] == idx.size
    np.testing.assert_array_equal(route_row[row_route], np.arange(idx.size))
    np.testing.assert_array_equal(packed, x[row_route // k])


def test_moe_layer_matches_reference(golden_dir):
    g = _load(golden_dir, "moe_layer.npz")
    x = g["x"].reshape(-1, g["x"].shape[-1])
    logits = oracle.router_logits(x, g["router_w"], out_dtype=np.float32)
    idx, gates, _ = oracle.topk_select(logits, 2)
    np.testing.assert_array_equal(idx, g["idx"])
    np.testing.assert_allclose(gates, g["gates"], rtol=1e-5)
    experts = {"w1": g["w1"], "w3": g["w3"], "w2": g["w2"]}
    # fp32 experts: evaluate the oracle without fp16 storage roundings
    import oracle.experts as ex
    packed, counts, offsets, _, route_row = oracle.pack_canonical(x, idx, 8)
    y = np.zeros_like(packed)
    for e in range(8):
        lo, hi = offsets[e], offsets[e + 1]
        y[lo:hi] = ex.swiglu_ffn(packed[lo:hi], g["w1"][e], g["w3"][e], g["w2"][e], store=np.float32)
    out = oracle.combine(y, gates, route_row, 2, out_dtype=np.float32)
    np.testing.assert_allclose(out, g["y"].reshape(out.shape), rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("tag,skew", [("plain", 0.0), ("skew", 2.0)])
def test_full_size_cpu_route_matches_reference(golden_dir, tag, skew):
    """T=4096, d=4096, E=64, k=2 on the benchmark distribution (inputs are
    regenerated from the seed; the fp32 product may differ in the last bits
    between hosts, so rows with a top-2 margin below 1e-4 are exempt)."""
    g = _load(golden_dir, "route_c1.npz")
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(4096, 4096, generator=gen)
    w = torch.randn(64, 4096, generator=gen) / 64.0
    logits = oracle.router_logits(x, w, skew_experts=8 if skew else 0, skew_bias=skew, out_dtype=np.float32)
    idx, gates, _ = oracle.topk_select(logits, 2)
    rows = g[f"{tag}_margin"] > 1e-4
    assert rows.mean() > 0.99
    np.testing.assert_array_equal(idx[rows], g[f"{tag}_idx"][rows].astype(np.int64))
    np.testing.assert_allclose(gates[rows], g[f"{tag}_w"][rows], rtol=1e-4, atol=1e-6)
    counts, offsets = oracle.counts_offsets(idx, 64)
    assert np.abs(counts - g[f"{tag}_counts"]).sum() <= 2 * (~rows).sum()
    mx, cv = oracle.load_skew(counts)
    if skew:
        assert 6.5 < mx < 8.5 and 2.0 < cv < 2.7
    else:
        assert 1.1 < mx < 1.4 and 0.05 < cv < 0.15
    sidx, _, _ = oracle.sinkhorn_route(logits, 2)
    scounts, _ = oracle.counts_offsets(sidx, 64)
    assert np.abs(scounts - g[f"{tag}_sinkhorn_counts"]).sum() <= 40
    assert oracle.load_skew(scounts)[1] < 0.1
