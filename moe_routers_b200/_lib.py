"""ctypes binding of libmoe_b200.so (the C ABI declared in include/moe_b200.h).

There is no fallback: if the shared library is missing or a symbol cannot be
resolved, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB_PATH

MOE_OK = 0
MOE_ERR_ARG, MOE_ERR_UNSUPPORTED, MOE_ERR_WORKSPACE, MOE_ERR_LAUNCH, MOE_ERR_DEVICE = 1, 2, 3, 4, 5  # include/moe_b200.h
MOE_F16, MOE_BF16, MOE_F32 = 0, 1, 2
MOE_ACT_NONE, MOE_ACT_GELU, MOE_ACT_SILU, MOE_ACT_SWIGLU = 0, 1, 2, 3
MOE_W_KN, MOE_W_NK = 0, 1

_p = C.c_void_p
_i = C.c_int
_sz = C.c_size_t
_f = C.c_float

# name -> (restype, argtypes); mirrors include/moe_b200.h one to one
SIGNATURES = {
    "moe_version": (_i, []),
    "moe_last_error": (C.c_char_p, []),
    "moe_workspace_bytes": (_sz, [_i, _i, _i]),
    "moe_workspace_init": (_i, [_p, _sz, _p]),
    "moe_read_status": (_i, [_p, _p, C.POINTER(C.c_int)]),
    "moe_set_wait_limit": (_i, [_p, _sz, C.c_ulonglong, _p]),
    "moe_launch_count": (C.c_longlong, []),
    "moe_set_pdl": (_i, [_i]),
    "moe_set_gemm_mode": (_i, [_i]),
    "moe_topk_select": (_i, [_p, _i, _i, _i, _i, _p, _p, _p]),
    "moe_pack": (_i, [_p, _i, _p, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "moe_fused_select": (_i, [_p, _i, _p, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "moe_pack_scatter": (_i, [_p, _i, _p, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "moe_pack_static": (_i, [_p, _i, _p, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p]),
    "moe_combine": (_i, [_p, _i, _p, _p, _i, _i, _i, _p, _p]),
    "moe_route_fused": (_i, [_p, _p, _i, _i, _i, _i, _i, _i, _f, _p, _p, _p, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "moe_router_gemm_select": (_i, [_p, _p, _i, _i, _i, _i, _i, _i, _f, _p, _p, _p, _p, _sz, _p]),
    "moe_ep_rebucket": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p]),
    "moe_enable_peer_access": (_i, [_i]),
    "moe_ipc_open": (_i, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "moe_ipc_close": (_i, [_p]),
    "moe_ipc_export": (_i, [_p, C.c_char_p, C.POINTER(C.c_size_t)]),
    "moe_device_pci_bus_id": (_i, [_i, C.c_char_p, _i]),
    "moe_ep_push": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _p, _p]),
    "moe_ep_signal": (_i, [_p, _i, _i, _i, _i, _p, _p, _sz, _i, _p]),
    "moe_ep_wait": (_i, [_p, _i, _i, _i, _p, _sz, _p]),
    "moe_ep_sync": (_i, [_p, _p, _i, _i, _i, _i, _p, _p, _sz, _i, _p, _sz, _p]),
    "moe_sinkhorn": (_i, [_p, _i, _i, _i, _i, _i, _f, _f, _p, _p, _p, _sz, _p]),
    "moe_grouped_gemm": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, C.c_int64, _i, _p, _p, _i, _i, _p, _sz, _p]),
    "moe_grouped_gemm_rows": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, C.c_int64, _i, _p, _p, _i, _i, _p, _sz, _p]),
    "moe_pack_scatter_to": (_i, [_p, _i, _p, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "moe_ep_segment_bases": (_i, [_p, _p, _i, _i, _i, _i, _i, _p, _p, _p]),
    "moe_ep_row_targets": (_i, [_p, _p, _i, _i, _i, _i, _i, _p, _p]),
}


class MoeError(RuntimeError):
    """A libmoe_b200 entry point returned a non-zero status."""

    def __init__(self, code: int, text: str):
        super().__init__(f"libmoe_b200 error {code}: {text}")
        self.code = code


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m moe_routers_b200.build` "
            "(there is no CPU or PyTorch fallback for this library)"
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the export is missing
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    return (lib.moe_last_error() or b"").decode()


def check(rc: int) -> None:
    if rc != MOE_OK:
        raise MoeError(rc, last_error())
