"""Host-side pieces that need no GPU: the routing-metric helpers (the names models/decoder_moe.py:22-35
imports) against their formulas in numpy, and the permutation sweep's CSV schema and DRAM model
(bench_router.py:303-316, :355-358)."""
import csv
import math

import numpy as np
import torch


def test_metric_helpers_match_their_formulas():
    from moe_routers_b200 import metrics as M

    rng = np.random.default_rng(0)
    s, e, k = 200, 16, 3
    logits = torch.from_numpy(rng.standard_normal((s, e)).astype(np.float32))
    idx = torch.from_numpy(np.stack([rng.permutation(e)[:k] for _ in range(s)]).astype(np.int64))
    idx[:, 0] = torch.where(torch.arange(s) % 5 == 0, torch.zeros(s, dtype=torch.int64), idx[:, 0])  # skew to expert 0
    p = M.route_distribution_from_topk(idx, e)
    counts = np.bincount(idx.numpy().reshape(-1), minlength=e)
    np.testing.assert_allclose(p.numpy(), counts / (s * k), atol=1e-7)
    assert abs(float(p.sum()) - 1.0) < 1e-6
    nz = p.numpy()[p.numpy() > 0]
    h = float(-(nz * np.log(nz)).sum())
    assert abs(M.routing_entropy_from_distribution(p) - h) < 1e-5
    assert abs(M.normalized_entropy(p) - h / math.log(e)) < 1e-5
    assert abs(M.normalized_entropy(torch.full((e,), 1.0 / e)) - 1.0) < 1e-6
    assert M.routing_entropy_from_distribution(torch.tensor([1.0, 0.0, 0.0])) == 0.0
    pr = np.exp(logits.numpy() - logits.numpy().max(axis=1, keepdims=True))
    pr /= pr.sum(axis=1, keepdims=True)
    assert abs(M.mean_topk_probability_from_logits(logits, k) - np.sort(pr, axis=1)[:, -k:].sum(axis=1).mean()) < 1e-5
    dup = idx.clone()
    dup[:, 1] = dup[:, 0]  # every token repeats a pick: k - 1 distinct experts (or fewer)
    want = np.mean([len(set(r)) for r in dup.numpy().tolist()])
    assert abs(M.avg_unique_experts_per_token(dup) - want) < 1e-6
    uniform = torch.full((e,), 1.0 / e)
    assert abs(M.aux_load_balance_loss(route_frac=uniform, importance=uniform, alpha=1.0) - 1.0) < 1e-6
    imp = torch.from_numpy(pr.mean(axis=0).astype(np.float32))
    assert abs(M.aux_load_balance_loss(route_frac=p, importance=imp, alpha=0.5)
               - 0.5 * e * float((p.numpy() * pr.mean(axis=0)).sum())) < 1e-5
    mean, std = M.unique_tokens_per_expert(idx, e)
    per = np.array([(idx.numpy() == ex).any(axis=1).sum() for ex in range(e)], dtype=np.float64)
    assert abs(mean - per.mean()) < 1e-4 and abs(std - per.std()) < 1e-4
    assert M.unique_tokens_per_expert(idx[:0], e) is None
    out = torch.from_numpy(rng.standard_normal((s, 8)).astype(np.float32))
    st = M.output_distribution_stats(out)
    assert abs(st["mean"] - out.numpy().mean()) < 1e-6 and abs(st["abs_max"] - np.abs(out.numpy()).max()) < 1e-6
    rec = M.MoEMetrics(router_backend="X", performance=M.PerformanceEfficiencyMetrics(1, 0.0, 0.0, 0.0, 0.0),
                       routing=None, usage=None, output=st)
    assert rec.router_backend == "X" and rec.performance.tokens == 1


def test_perm_sweep_model_and_csv_schema(tmp_path):
    from moe_routers_b200 import bench_router as br

    # the reference's columns come first, in its order (bench_router.py:303-316)
    assert br.PERM_SWEEP_FIELDS[:12] == ["batch_size", "seq_len", "tokens", "experts", "top_k", "d_model", "dtype",
                                         "t_perm_naive_ms", "t_perm_sorted_ms", "t_theory_ms", "peak_bw_gbs",
                                         "sorted_achieved_bw_gbs"]
    tokens, k, d, elem, bw = 8192, 2, 4096, 2, 6548.8
    m = br.perm_model(tokens, k, d, elem, bw, t_sorted_ms=0.05)
    ideal = 2.0 * tokens * k * d * elem  # read + write of every routed row (bench_router.py:355-358)
    assert abs(m["t_theory_ms"] - ideal / (bw * 1e9) * 1e3) < 1e-12
    assert abs(m["sorted_achieved_bw_gbs"] - ideal / 0.05e-3 / 1e9) < 1e-6
    assert m["compulsory_bytes"] == (1 + k) * tokens * d * elem
    nan = br.perm_model(tokens, k, d, elem, 0.0, t_sorted_ms=0.05)
    assert math.isnan(nan["t_theory_ms"]) and math.isnan(nan["sorted_achieved_bw_gbs"])
    row = dict(batch_size=4, seq_len=128, tokens=512, experts=64, top_k=2, d_model=4096, dtype="float16",
               t_perm_naive_ms=1.0, t_perm_sorted_ms=0.01, t_perm_torch_sorted_ms=0.2, peak_bw_gbs=bw)
    row.update(br.perm_model(512, 2, 4096, 2, bw, 0.01))
    path = tmp_path / "perm.csv"
    br.write_perm_csv(str(path), [row])
    with open(path) as f:
        rows = list(csv.DictReader(f))
    assert list(rows[0].keys()) == br.PERM_SWEEP_FIELDS and float(rows[0]["t_perm_naive_ms"]) == 1.0


def test_naive_mask_scan_pack_orders_rows_by_expert():
    """The baseline leg of the sweep (bench_router.py:81-120) on CPU tensors: same rows as the sorted
    pack, grouped by expert, ascending route id inside a group."""
    from moe_routers_b200 import bench_router as br

    g = torch.Generator().manual_seed(1)
    x = torch.randn(50, 8, generator=g)
    idx = torch.randint(0, 6, (50, 2), generator=g, dtype=torch.int32)
    got = br._torch_pack_mask_scan(x, idx, 6)
    order = np.argsort(idx.numpy().reshape(-1), kind="stable")
    np.testing.assert_array_equal(got.numpy(), x.numpy()[order // 2])
    torch.testing.assert_close(br._torch_pack(x, idx).sum(dim=0), got.sum(dim=0))
