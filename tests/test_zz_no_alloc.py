"""moe_pack_static: the pack entry point for callers that cannot allocate device memory (a fixed
memory plan, a host hook that forbids cudaMalloc).  Its scratch is an array inside the library
image.  The test drives it through the C ABI and compares every output, bit for bit, with
moe_pack on the same inputs, on two calls in a row with different inputs (the array keeps the
first call's contents, which must not leak into the second result).

This file is collected last on purpose, so that a run that stops at the first failure has
already run every other test; it passes on its own in a fresh process as well.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, x, idx, experts, status):
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
                                 out["row_route"].data_ptr(), out["route_row"].data_ptr(), status.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
    lib.check(rc)
    return out


def test_pack_static_matches_pack_on_two_calls_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from moe_routers_b200 import _lib, ops

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    g = torch.Generator().manual_seed(0)
    for t, d, e, k in [(4096, 1024, 64, 2), (777, 200, 256, 3)]:
        x = torch.randn(t, d, generator=g).half().cuda()
        idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(torch.int32).cuda()
        got = _call_static(_lib, x, idx, e, status)
        counts, offsets, packed, row_route, route_row = ops.pack(x, idx, e)
        torch.cuda.synchronize()
        assert torch.equal(got["counts"], counts)
        assert torch.equal(got["offsets"], offsets)
        assert torch.equal(got["row_route"], row_route)
        assert torch.equal(got["route_row"], route_row)
        assert torch.equal(got["packed"], packed)
        assert int(got["offsets"][-1]) == t * k
    assert int(status.item()) == 0


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
