"""B200-native MoE routing and dispatch path (drop-in for santiweide/moe-routers).

Sub-modules are imported on first use so that `python -m moe_routers_b200.build`
can run before the shared library exists.  Everything except `build` loads
libmoe_b200.so on import; a missing library is an error, never a fallback.
"""
import importlib

_SUBMODULES = ("ops", "routers", "moe_layer", "fused_select_cuda", "grouped_ffn_cuda", "ep", "bench_ep", "bench_router", "strategies", "build", "_lib")


def __getattr__(name):
    if name in _SUBMODULES:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def install_dropin_modules() -> None:
    """Register `fused_select_cuda` and `grouped_ffn_cuda` in sys.modules so that
    the reference's own `import fused_select_cuda` resolves to this library."""
    import sys

    sys.modules["fused_select_cuda"] = importlib.import_module(f"{__name__}.fused_select_cuda")
    sys.modules["grouped_ffn_cuda"] = importlib.import_module(f"{__name__}.grouped_ffn_cuda")
