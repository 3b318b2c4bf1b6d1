"""Run the reference's own `bench_router.py --device cpu` (staged under oracle/_ref/) in process.

TEST / BENCHMARK INFRASTRUCTURE ONLY (see the package docstring).

The staged files are the reference's, unmodified.  Two modules they import are missing from the
reference tree (`models/model.py`, `models/metrics.py`); empty stand-ins are registered in
`sys.modules` first so that the imports succeed (the CPU benchmark path never calls them).  The
script is started with `runpy` under its own command line, its printed `T_*_ms` lines are parsed.
"""
from __future__ import annotations

import contextlib
import io
import os
import re
import runpy
import sys
import types

from .build_ref import REF_DIR, staged

_METRIC_NAMES = (
    "MoEMetrics PerformanceEfficiencyMetrics RoutingBehaviorMetrics ExpertUsageMetrics "
    "avg_unique_experts_per_token aux_load_balance_loss mean_topk_probability_from_logits "
    "normalized_entropy output_distribution_stats route_distribution_from_topk "
    "routing_entropy_from_distribution unique_tokens_per_expert"
).split()


def available() -> bool:
    return staged()


def _stubs() -> dict:
    model_stub = types.ModuleType("models.model")
    model_stub.OneLayerModel = object
    model_stub._parse_dtype = lambda s: s
    metrics_stub = types.ModuleType("models.metrics")
    for name in _METRIC_NAMES:
        setattr(metrics_stub, name, object)
    return {"models.model": model_stub, "models.metrics": metrics_stub}


def run_cpu(*, tokens: int, d_model: int, experts: int, top_k: int, strategy: str = "naive_topk",
            skew_experts: int = 0, skew_bias: float = 0.0, warmup: int = 1, iters: int = 3) -> dict:
    """One run of the reference's CPU benchmark (bench_router.py:484-505, fp32); returns its mean
    stage times in milliseconds: t_logit_ms, t_select_ms, t_pack_ms, t_route_ms."""
    if not staged():
        raise RuntimeError("oracle/_ref is empty: run `python -m oracle.build_ref` where the reference is checked out")
    argv = ["bench_router.py", "--device", "cpu", "--dtype", "fp32", "--tokens", str(tokens), "--d_model", str(d_model),
            "--experts", str(experts), "--top_k", str(top_k), "--strategy", strategy, "--warmup", str(warmup),
            "--iters", str(iters), "--skew_experts", str(skew_experts), "--skew_bias", str(skew_bias)]
    saved_argv, saved_path = sys.argv, list(sys.path)
    saved_mods = {k: v for k, v in sys.modules.items() if k == "models" or k.startswith("models.") or k == "bench_router"}
    for k in saved_mods:
        del sys.modules[k]
    buf = io.StringIO()
    try:
        sys.argv = argv
        sys.path.insert(0, REF_DIR)
        sys.modules.update(_stubs())
        with contextlib.redirect_stdout(buf):
            runpy.run_path(os.path.join(REF_DIR, "bench_router.py"), run_name="__main__")
    finally:
        sys.argv = saved_argv
        sys.path[:] = saved_path
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.") or k == "bench_router"]:
            del sys.modules[k]
        sys.modules.update(saved_mods)
    text = buf.getvalue()
    out = {}
    for key in ("T_logit_ms", "T_select_ms", "T_pack_ms", "T_route_ms"):
        m = re.search(rf"^{key}:\s*([0-9.eE+-]+)\s*$", text, re.M)
        if not m:
            raise RuntimeError(f"reference output has no {key} line:\n{text[-1000:]}")
        out[key.lower()] = float(m.group(1))
    return out
