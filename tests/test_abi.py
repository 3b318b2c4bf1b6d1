"""The C-ABI library loads and exports every symbol that include/moe_b200.h
declares; argument validation works without a GPU (no kernel is launched)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from moe_routers_b200 import build

    build.build_library()
    from moe_routers_b200 import _lib

    return _lib


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "moe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moe_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = _declared_functions()
    assert len(names) >= 12
    raw = ctypes.CDLL(lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in moe_b200.h but not exported"
    assert sorted(lib.SIGNATURES) == names


def test_version_and_workspace_size(lib):
    assert lib.lib.moe_version() >= 100
    small = lib.lib.moe_workspace_bytes(32, 64, 2)
    big = lib.lib.moe_workspace_bytes(4096, 64, 2)
    assert 512 < small <= big
    assert lib.lib.moe_workspace_bytes(-1, 64, 2) == 0


def test_argument_errors_do_not_launch(lib):
    L = lib.lib
    # top_k out of range -> MOE_ERR_UNSUPPORTED with a readable text
    rc = L.moe_topk_select(None, lib.MOE_F16, 4, 64, 9, None, None, None)
    assert rc == 2 and "top_k" in lib.last_error()
    rc = L.moe_topk_select(None, 7, 4, 64, 2, None, None, None)
    assert rc == 1
    rc = L.moe_pack(None, 3, None, 4, 8, 64, 2, None, None, None, None, None, None, 0, None)
    assert rc == 1 and "elem_bytes" in lib.last_error()
    rc = L.moe_combine(None, lib.MOE_F32, None, None, 4, 8, 2, None, None)
    assert rc == 1
    with pytest.raises(lib.MoeError):
        lib.check(rc)
    # the expert-parallel entry points validate before they touch the device
    rc = L.moe_pack_scatter_to(None, 2, None, 4, 8, 64, 2, None, None, None, None, None, None, 0, None)
    assert rc == 1 and "seg_base" in lib.last_error()
    rc = L.moe_grouped_gemm_rows(None, None, None, None, 4, 16, 64, 64, lib.MOE_W_NK, 0, lib.MOE_ACT_NONE, None, None,
                                 lib.MOE_F16, 0, None, 0, None)
    assert rc == 1 and "row table" in lib.last_error()
    rc = L.moe_ep_row_targets(None, None, 6, 4, 0, 64, 2, None, None)
    assert rc == 1 and "divisible" in lib.last_error()
    rc = L.moe_ep_segment_bases(None, None, 8, 4, 5, 64, 2, None, None, None)
    assert rc == 1 and "rank" in lib.last_error()
    rc = L.moe_ep_segment_bases(None, None, 8, 4, 0, 3, 2, None, None, None)
    assert rc == 1 and "16 bytes" in lib.last_error()
    assert L.moe_grouped_gemm(None, None, None, None, 4, 0, 64, 64, lib.MOE_W_NK, 0, lib.MOE_ACT_NONE, None, None,
                              lib.MOE_F16, 0, None, 0, None) == 0  # zero rows: nothing to do
    # host-visible pointers that the kernels access 128 bits at a time must be 16-byte aligned
    rc = L.moe_grouped_gemm(ctypes.c_void_p(4096), ctypes.c_void_p(4096), ctypes.c_void_p(4096 + 8), ctypes.c_void_p(4096),
                            4, 16, 64, 64, lib.MOE_W_NK, 0, lib.MOE_ACT_NONE, None, None, lib.MOE_F16, 0,
                            ctypes.c_void_p(4096), 1 << 20, None)
    assert rc == 1 and "aligned" in lib.last_error()
    rc = L.moe_ep_push(ctypes.c_void_p(4096 + 2), ctypes.c_void_p(4096), ctypes.c_void_p(4096), 8, 4, 0, 0, 64, 2, None, None)
    assert rc == 1 and "aligned" in lib.last_error()
    rc = L.moe_ep_signal(None, 4, 0, 0, 1, None, None, 0, 0, None)
    assert rc == 1 and "flag table" in lib.last_error()
    rc = L.moe_ep_wait(None, 4, 0, 1, None, 0, None)
    assert rc == 1
    assert L.moe_ipc_export(None, None, None) == 1 and "null" in lib.last_error()
    assert L.moe_set_wait_limit(None, 0, 1000, None) == 3
    assert L.moe_launch_count() >= 0 and L.moe_set_pdl(1) == 0
    # grouped GEMM variants: the setter returns the previous set, a negative mode only reads
    before = L.moe_set_gemm_mode(-1)
    assert 0 <= before <= 31
    assert L.moe_set_gemm_mode(5) == before and L.moe_set_gemm_mode(-1) == 5
    assert L.moe_set_gemm_mode(before) == 5 and L.moe_set_gemm_mode(-1) == before
    # zero tokens is a valid no-op that needs no pointers
    assert L.moe_topk_select(None, lib.MOE_F16, 0, 64, 2, None, None, None) == 0
    assert L.moe_combine(None, lib.MOE_F16, None, None, 0, 8, 2, None, None) == 0


def test_ops_reject_cpu_tensors(lib):
    import torch
    from moe_routers_b200 import ops

    with pytest.raises(RuntimeError, match="inputs must be CUDA"):
        ops.topk_select(torch.zeros(4, 64), 2)
    with pytest.raises(RuntimeError, match="inputs must be CUDA"):
        ops.pack(torch.zeros(4, 8, dtype=torch.float16), torch.zeros(4, 2, dtype=torch.int32), 64)
