"""moe_pack_static: the pack entry point for callers that cannot allocate device memory (a fixed
memory plan, a host hook that forbids cudaMalloc).  Its scratch is an array inside the library
image.  The test drives it through the C ABI and compares every output, bit for bit, with
moe_pack on the same inputs and with the CPU oracle, on calls in a row with different inputs (the
array keeps the previous call's contents, which must not leak into the next result).

This file is collected last on purpose, so that a run that stops at the first failure has
already run every other test; it passes on its own in a fresh process as well.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _call_static(lib, x, idx, experts, status):
    """`status` may be None: the entry point accepts a NULL device_status."""
    t, d = x.shape
    k = idx.size(1)
    dev = x.device
    out = dict(
        counts=torch.empty(experts, dtype=torch.int32, device=dev),
        offsets=torch.empty(experts + 1, dtype=torch.int32, device=dev),
        packed=torch.empty((t * k, d), dtype=x.dtype, device=dev),
        row_route=torch.empty(t * k, dtype=torch.int32, device=dev),
        route_row=torch.empty(t * k, dtype=torch.int32, device=dev),
    )
    rc = lib.lib.moe_pack_static(x.data_ptr(), x.element_size(), idx.data_ptr(), t, d, experts, k,
                                 out["counts"].data_ptr(), out["offsets"].data_ptr(), out["packed"].data_ptr(),
                                 out["row_route"].data_ptr(), out["route_row"].data_ptr(),
                                 status.data_ptr() if status is not None else None,
                                 torch.cuda.current_stream().cuda_stream)
    lib.check(rc)
    return out


def test_pack_static_matches_pack_on_two_calls_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from moe_routers_b200 import _lib, ops

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    g = torch.Generator().manual_seed(0)
    # (777, 100): 200-byte rows are not a multiple of 16 bytes -> the load/store scatter, not the bulk one
    for t, d, e, k, st in [(4096, 1024, 64, 2, status), (777, 200, 256, 3, status), (777, 100, 48, 2, None),
                           (8192, 64, 256, 1, status)]:
        x = torch.randn(t, d, generator=g).half().cuda()
        idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(torch.int32).cuda()
        got = _call_static(_lib, x, idx, e, st)
        counts, offsets, packed, row_route, route_row = ops.pack(x, idx, e)
        torch.cuda.synchronize()
        assert torch.equal(got["counts"], counts)
        assert torch.equal(got["offsets"], offsets)
        assert torch.equal(got["row_route"], row_route)
        assert torch.equal(got["route_row"], route_row)
        assert torch.equal(got["packed"], packed)
        assert int(got["offsets"][-1]) == t * k
        # and against the CPU restatement of the reference's pack (canonical order), bit for bit
        ref_packed, ref_counts, ref_offsets, ref_rr, ref_inv = oracle.pack_canonical(
            x.cpu().view(torch.int16).numpy(), idx.cpu().numpy(), e)
        np.testing.assert_array_equal(got["counts"].cpu().numpy(), ref_counts)
        np.testing.assert_array_equal(got["offsets"].cpu().numpy(), ref_offsets)
        np.testing.assert_array_equal(got["row_route"].cpu().numpy(), ref_rr)
        np.testing.assert_array_equal(got["route_row"].cpu().numpy(), ref_inv)
        np.testing.assert_array_equal(got["packed"].view(torch.int16).cpu().numpy(), ref_packed)
    assert int(status.item()) == 0


def test_pack_static_edge_cases():
    """Zero tokens give zero counts and offsets without touching the other outputs; an expert id
    outside [0, experts) is reported in device_status (and skipped), never followed."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from moe_routers_b200 import _lib

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x0 = torch.zeros((0, 64), dtype=torch.float16, device="cuda")
    i0 = torch.zeros((0, 2), dtype=torch.int32, device="cuda")
    got = _call_static(_lib, x0, i0, 16, status)
    torch.cuda.synchronize()
    assert int(got["counts"].abs().sum()) == 0 and int(got["offsets"].abs().sum()) == 0

    t, d, e, k = 96, 64, 8, 2
    g = torch.Generator().manual_seed(3)
    x = torch.randn(t, d, generator=g).half().cuda()
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(torch.int32)
    idx[5, 1] = e + 3   # out of range
    idx[40, 0] = -1     # negative
    got = _call_static(_lib, x, idx.cuda(), e, status)
    torch.cuda.synchronize()
    assert int(status.item()) != 0
    valid = (idx >= 0) & (idx < e)
    np.testing.assert_array_equal(got["counts"].cpu().numpy(),
                                  np.bincount(idx[valid].numpy().reshape(-1), minlength=e))
    assert int(got["offsets"][-1]) == int(valid.sum())


def test_pack_static_rejects_sizes_beyond_its_scratch():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from moe_routers_b200 import _lib

    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    p = z.data_ptr()
    rc = _lib.lib.moe_pack_static(p, 2, p, 8193, 8, 64, 2, p, p, p, p, p, None, None)
    assert rc == 2 and "8192 tokens" in _lib.last_error()
    rc = _lib.lib.moe_pack_static(p, 2, p, 16, 8, 257, 2, p, p, p, p, p, None, None)
    assert rc == 2 and "256 experts" in _lib.last_error()
