"""Generate the golden vectors under tests/golden/ from the REFERENCE itself.

Run where a checkout of santiweide/moe-routers is available:

    python tests/golden/make_golden.py --reference /path/to/moe-routers

The reference's Python classes are imported unmodified.  `models/__init__.py`
and `models/decoder_moe.py` import two files that are missing from the
reference tree (`models/model.py`, `models/metrics.py`); two stub modules are
registered in `sys.modules` first so that the import succeeds (the stubs are
never called: metrics tracking stays off).

The committed `.npz` files are what the tests read; this script is not needed
at test time and the reference checkout is not needed either.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(ref_root: str):
    sys.path.insert(0, ref_root)
    model_stub = types.ModuleType("models.model")
    model_stub.OneLayerModel = object
    model_stub._parse_dtype = lambda s: s
    metrics_stub = types.ModuleType("models.metrics")
    for name in (
        "MoEMetrics PerformanceEfficiencyMetrics RoutingBehaviorMetrics ExpertUsageMetrics "
        "avg_unique_experts_per_token aux_load_balance_loss mean_topk_probability_from_logits "
        "normalized_entropy output_distribution_stats route_distribution_from_topk "
        "routing_entropy_from_distribution unique_tokens_per_expert"
    ).split():
        setattr(metrics_stub, name, object)
    sys.modules["models.model"] = model_stub
    sys.modules["models.metrics"] = metrics_stub
    import models.decoder_moe as dm  # noqa: E402
    import bench_router as br  # noqa: E402

    return dm, br


def gen_inputs(seed: int, t: int, d: int, e: int, dtype=torch.float32):
    """x ~ N(0,1) [t,d], W ~ N(0,1/d) [e,d] from one seeded CPU generator."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(t, d, generator=g)
    w = torch.randn(e, d, generator=g) / (d ** 0.5)
    return x.to(dtype), w.to(dtype)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of santiweide/moe-routers to import the routers from")
    args = ap.parse_args()
    dm, br = import_reference(args.reference)
    torch.set_num_threads(4)

    # ---- 1. TorchTopKRouter, fp32 and fp16 logits, several (E, k) ----
    out = {}
    for tag, (t, e, k, dtype) in {
        "f32_e64_k2": (257, 64, 2, torch.float32),
        "f32_e64_k8": (129, 64, 8, torch.float32),
        "f32_e8_k2": (127, 8, 2, torch.float32),
        "f32_e64_k1": (33, 64, 1, torch.float32),
        "f16_e64_k2": (513, 64, 2, torch.float16),
        "f32_e48_k3": (65, 48, 3, torch.float32),
    }.items():
        g = torch.Generator().manual_seed(1234 + t + e + k)
        logits = torch.randn(t, e, generator=g).to(dtype)
        idx, w = dm.TorchTopKRouter()(logits, k)
        out[f"{tag}_logits"] = logits.numpy()
        out[f"{tag}_idx"] = idx.numpy()
        out[f"{tag}_w"] = w.numpy()
    np.savez_compressed(os.path.join(HERE, "topk_router.npz"), **out)

    # ---- 2. SinkhornRouter ----
    out = {}
    for tag, (t, e, k, dtype, iters, temp, skew) in {
        "f32_it10": (256, 64, 2, torch.float32, 10, 1.0, 0.0),
        "f16_it10": (256, 64, 2, torch.float16, 10, 1.0, 0.0),
        "f16_it10_skew": (256, 64, 2, torch.float16, 10, 1.0, 2.0),
        "f32_it3_t07": (96, 16, 4, torch.float32, 3, 0.7, 0.0),
    }.items():
        x, w = gen_inputs(77 + t + e, t, 128, e)
        logits = x @ w.t()
        if skew:
            logits[:, :8] += skew
        logits = logits.to(dtype)
        router = dm.SinkhornRouter(iters=iters, temperature=temp)
        idx, wgt = router(logits, k)
        out[f"{tag}_logits"] = logits.numpy()
        out[f"{tag}_idx"] = idx.numpy()
        out[f"{tag}_w"] = wgt.numpy()
        out[f"{tag}_cfg"] = np.array([k, iters, temp, router.epsilon], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "sinkhorn_router.npz"), **out)

    # ---- 3. bench_router._pack_routes (gate-weighted, unstable order) ----
    t, d, e, k = 96, 32, 8, 2
    x, w = gen_inputs(5, t, d, e)
    logits = x @ w.t()
    idx, wgt = dm.TorchTopKRouter()(logits, k)
    xs, toks, exps = br._pack_routes(x, idx, wgt)
    np.savez_compressed(
        os.path.join(HERE, "pack_routes.npz"),
        x=x.numpy(), idx=idx.numpy(), w=wgt.numpy(),
        x_route_sorted=xs.numpy(), token_ids_sorted=toks.numpy(), expert_ids_sorted=exps.numpy(),
    )

    # ---- 4. MoELayer (SwiGLU experts), fp32 ----
    torch.manual_seed(11)
    d, h, e, k = 32, 64, 8, 2
    layer = dm.MoELayer(d, h, e, k)
    xin = torch.randn(2, 24, d)
    with torch.no_grad():
        y = layer(xin)
        flat = xin.view(-1, d)
        logits = layer.router(flat)
        idx, wgt = layer.router_impl(logits, k)
    np.savez_compressed(
        os.path.join(HERE, "moe_layer.npz"),
        x=xin.numpy(), y=y.numpy(), router_w=layer.router.weight.detach().numpy(),
        idx=idx.numpy(), gates=wgt.numpy(),
        w1=np.stack([ex.w1.weight.detach().numpy() for ex in layer.experts]),
        w3=np.stack([ex.w3.weight.detach().numpy() for ex in layer.experts]),
        w2=np.stack([ex.w2.weight.detach().numpy() for ex in layer.experts]),
    )

    # ---- 5. Full-size CPU fp32 naive_topk route (T=4096, d=4096, E=64, k=2) ----
    # The reference's CPU path (bench_router.py:484-505) on the benchmark
    # distribution W ~ N(0, 1/d); inputs are regenerated from the seed by the
    # test, only the outputs are stored.
    out = {}
    for tag, skew in (("plain", 0.0), ("skew", 2.0)):
        x, w = gen_inputs(0, 4096, 4096, 64)
        logits = x.float() @ w.float().t()
        if skew:
            logits[:, :8] += skew
        idx, wgt = dm.TorchTopKRouter()(logits, 2)
        vals = torch.topk(logits, 3, dim=-1).values
        out[f"{tag}_idx"] = idx.numpy().astype(np.uint8)
        out[f"{tag}_w"] = wgt.numpy().astype(np.float32)
        out[f"{tag}_margin"] = (vals[:, 1] - vals[:, 2]).numpy().astype(np.float32)
        out[f"{tag}_counts"] = torch.bincount(idx.reshape(-1), minlength=64).numpy().astype(np.int32)
        sidx, swgt = dm.SinkhornRouter(iters=10)(logits, 2)
        out[f"{tag}_sinkhorn_counts"] = torch.bincount(sidx.reshape(-1), minlength=64).numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "route_c1.npz"), **out)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
