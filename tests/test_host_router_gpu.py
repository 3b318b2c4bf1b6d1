"""HostRouter: host-resident batches through upload -> route kernels -> download on alternating slots."""
import numpy as np
import pytest
import torch

from oracle import routing

pytestmark = pytest.mark.gpu


def _clear_rows(logits, k, margin=2e-2):
    """Rows whose k-th and (k+1)-th logits differ by more than the rounding of an fp16 product."""
    srt = np.sort(logits.astype(np.float32), axis=1)[:, ::-1]
    gaps = np.abs(np.diff(srt[:, : k + 1], axis=1))
    return (gaps > margin).all(axis=1)


@pytest.mark.parametrize("depth", [1, 2, 3])
def test_host_router_matches_oracle_in_order(depth):
    from moe_routers_b200.host import HostRouter

    t, d, e, k = 512, 256, 64, 2
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(e, d, generator=g) / d ** 0.5).half()
    batches = [torch.randn(t, d, generator=g).half() for _ in range(5)]
    r = HostRouter(t, d, w, k, depth=depth)
    tickets, got = [], []
    for b in batches:  # keep `depth` batches in flight
        if len(tickets) == depth:
            got.append({n: v.clone() for n, v in r.result(tickets.pop(0)).items()})
        tickets.append(r.submit(b.pin_memory()))
    while tickets:
        got.append({n: v.clone() for n, v in r.result(tickets.pop(0)).items()})
    assert len(got) == len(batches)
    for b, o in zip(batches, got):
        logits = routing.router_logits(b.numpy(), w.numpy())
        idx, gates, _ = routing.topk_select(logits, k)
        clear = _clear_rows(logits, k)
        assert clear.mean() > 0.5
        np.testing.assert_array_equal(o["idx"].numpy()[clear], idx[clear])
        np.testing.assert_allclose(o["gates"].numpy()[clear], gates[clear], rtol=2e-3, atol=1e-3)
        # integer structure: bit-exact against the oracle's pack of the selection that was made
        packed, counts, offsets, row_route, route_row = routing.pack_canonical(
            b.numpy().view(np.uint16), o["idx"].numpy(), e)
        np.testing.assert_array_equal(o["counts"].numpy(), counts)
        np.testing.assert_array_equal(o["offsets"].numpy(), offsets)
        np.testing.assert_array_equal(o["row_route"].numpy(), row_route)
        np.testing.assert_array_equal(o["route_row"].numpy(), route_row)
        np.testing.assert_array_equal(o["packed"].numpy().view(np.uint16), packed)


def test_host_router_rejects_misuse():
    from moe_routers_b200.host import HostRouter

    w = torch.zeros(64, 128).half()
    r = HostRouter(64, 128, w, 2, depth=1)
    x = torch.zeros(64, 128).half()
    with pytest.raises(RuntimeError):
        r.submit(x.cuda())
    with pytest.raises(RuntimeError):
        r.submit(torch.zeros(32, 128).half())
    tk = r.submit(x)
    with pytest.raises(RuntimeError):
        r.submit(x)  # the only slot is still unread
    r.result(tk)
    with pytest.raises(RuntimeError):
        r.result(tk)


def test_host_router_download_subset():
    """`download=` brings back only the routing decision; the packed rows stay on the device, where
    `device_outputs` hands them to the expert GEMMs; the byte counts the benchmark declares follow."""
    from moe_routers_b200.host import HostRouter

    t, d, e, k = 256, 128, 16, 2
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(e, d, generator=g) / d ** 0.5).half()
    x = torch.randn(t, d, generator=g).half().pin_memory()
    names = ("idx", "gates", "counts", "offsets", "row_route", "route_row")
    r = HostRouter(t, d, w, k, depth=2, download=names)
    full = HostRouter(t, d, w, k, depth=1)
    tk = r.submit(x)
    o = r.result(tk)
    ref = full.route(x)
    assert sorted(o) == sorted(names)
    for n in names:
        assert torch.equal(o[n], ref[n]), n
    dev = r.device_outputs(tk)
    assert torch.equal(dev["packed"].cpu(), ref["packed"])
    assert r.d2h_bytes == sum(ref[n].numel() * ref[n].element_size() for n in names)
    assert full.d2h_bytes == r.d2h_bytes + ref["packed"].numel() * 2
    assert r.h2d_bytes == t * d * 2
    with pytest.raises(ValueError):
        HostRouter(t, d, w, k, download=("idx", "nonsense"))
