"""Route batches whose tokens live in HOST memory.

The reference's operator takes device tensors (kernels/fused_select.cu:203-215); a caller that
keeps activations on the host pays one upload of `x` and one download of the five results per
call.  `HostRouter` keeps `depth` slots, each with its own stream, device buffers and pinned host
result buffers (allocated on the NUMA node the GPU is attached to; `pin_near` does the same for a
caller's input batches), so that the download of batch i (device -> host copy engine) runs while batch
i+1 uploads (host -> device copy engine) and routes:

    r = HostRouter(tokens, d_model, w_router_host, top_k=2)
    t0 = r.submit(x0)            # returns at once; x0 must stay untouched until result(t0)
    t1 = r.submit(x1)
    out0 = r.result(t0)          # dict of pinned host tensors: idx, gates, counts, offsets, packed, ...

All compute is the library's route kernels; nothing here falls back to the CPU.
"""
from __future__ import annotations

import contextlib
import ctypes
import os

import torch

from . import ops


def parse_cpulist(text: str) -> set:
    """CPU numbers of a sysfs cpulist ("0-31,64-95")."""
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def local_cpus(device, sysfs: str = "/sys") -> set:
    """CPUs of the NUMA node that CUDA device `device` is attached to; empty when the platform does
    not say (no sysfs entry, node -1) - the caller then leaves the thread where it is."""
    from ._lib import lib

    try:
        buf = ctypes.create_string_buffer(32)
        if lib.moe_device_pci_bus_id(int(torch.device(device).index or 0), buf, 32) != 0:
            return set()
        bdf = buf.value.decode().lower()
        with open(os.path.join(sysfs, "bus/pci/devices", bdf, "numa_node")) as f:
            node = int(f.read().strip())
        if node < 0:
            return set()
        with open(os.path.join(sysfs, "devices/system/node", f"node{node}", "cpulist")) as f:
            return parse_cpulist(f.read())
    except (OSError, ValueError):
        return set()


@contextlib.contextmanager
def numa_local(device, cpus=None):
    """Run the body on CPUs next to the GPU, so that host memory pinned inside it lands on the GPU's
    own NUMA node (first touch): with one rank per GPU on a two-socket host, staging buffers on the
    far socket share the inter-socket link with every other rank's copies.  No-op where the CPUs are
    unknown or not in the thread's allowed set."""
    before = None
    try:
        want = (local_cpus(device) if cpus is None else set(cpus)) & os.sched_getaffinity(0)
        if want:
            before = os.sched_getaffinity(0)
            os.sched_setaffinity(0, want)
    except (OSError, AttributeError):
        before = None
    try:
        yield
    finally:
        if before is not None:
            os.sched_setaffinity(0, before)


def pin_near(t: torch.Tensor, device) -> torch.Tensor:
    """A pinned host copy of `t` allocated on the NUMA node of `device`."""
    with numa_local(device):
        return t.contiguous().pin_memory()


class HostRouter:
    def __init__(self, tokens: int, d_model: int, w_router: torch.Tensor, top_k: int = 2, *, depth: int = 2,
                 skew_experts: int = 0, skew_bias: float = 0.0, device=None, upload_weight_each_call: bool = False,
                 download=None):
        """`download`: names of the route outputs copied back to the host every call (default: all
        seven: idx, gates, counts, offsets, packed, row_route, route_row).  A caller whose experts run
        on the device leaves `packed` (k*T*d elements, almost all of the bytes) there and downloads
        only the routing decision; the device tensors of the last call stay reachable through
        `device_outputs(ticket)`."""
        if depth < 1:
            raise ValueError("depth must be >= 1")
        if w_router.dim() != 2 or w_router.size(1) != d_model:
            raise RuntimeError("w_router shape must be [E, d_model]")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.tokens, self.d, self.k = int(tokens), int(d_model), int(top_k)
        self.skew = (int(skew_experts), float(skew_bias))
        self.upload_w = bool(upload_weight_each_call)
        self.w_host = w_router if w_router.is_pinned() else pin_near(w_router, self.device)
        self.slots = []
        for _ in range(depth):
            s = torch.cuda.Stream(device=self.device)
            x_dev = torch.zeros((tokens, d_model), dtype=w_router.dtype, device=self.device)
            w_dev = self.w_host.to(self.device)  # one copy per slot: a per-call upload never races another slot
            torch.cuda.synchronize(self.device)
            with torch.cuda.stream(s):
                dev_out = ops.route_fused(x_dev, w_dev, self.k)  # allocates the outputs once
            names = [n for n in dev_out if n != "workspace"] if download is None else list(download)
            unknown = [n for n in names if n not in dev_out or n == "workspace"]
            if unknown:
                raise ValueError(f"unknown route outputs: {unknown}")
            with numa_local(self.device):  # pinned result buffers next to the GPU
                host_out = {n: torch.empty(dev_out[n].shape, dtype=dev_out[n].dtype).pin_memory() for n in names}
            self.slots.append(dict(stream=s, x=x_dev, w=w_dev, dev=dev_out, host=host_out,
                                   done=torch.cuda.Event(), busy=False))
        torch.cuda.synchronize(self.device)
        self._next = 0
        self.h2d_bytes = tokens * d_model * w_router.element_size() + (self.w_host.numel() * self.w_host.element_size()
                                                                       if self.upload_w else 0)
        self.d2h_bytes = sum(v.numel() * v.element_size() for v in self.slots[0]["host"].values())

    def submit(self, x_host: torch.Tensor) -> int:
        """Queue upload + route + download of one batch; returns the ticket for `result`."""
        if x_host.is_cuda:
            raise RuntimeError("x must be a host tensor")
        if tuple(x_host.shape) != (self.tokens, self.d) or x_host.dtype != self.w_host.dtype:
            raise RuntimeError("x shape must be [T, d_model] in the router weight's dtype")
        ticket = self._next
        slot = self.slots[ticket % len(self.slots)]
        if slot["busy"]:
            raise RuntimeError("slot still holds an unread result: call result() on the oldest ticket first")
        self._next += 1
        with torch.cuda.stream(slot["stream"]):
            slot["x"].copy_(x_host, non_blocking=True)
            if self.upload_w:
                slot["w"].copy_(self.w_host, non_blocking=True)
            o = ops.route_fused(slot["x"], slot["w"], self.k, skew_experts=self.skew[0], skew_bias=self.skew[1],
                                out=slot["dev"])
            for n, h in slot["host"].items():
                h.copy_(o[n], non_blocking=True)
            slot["done"].record(slot["stream"])
        slot["busy"] = True
        return ticket

    def result(self, ticket: int) -> dict:
        """Wait for a ticket; the returned pinned tensors are reused by ticket + depth."""
        slot = self.slots[ticket % len(self.slots)]
        if not slot["busy"]:
            raise RuntimeError("no pending result for this ticket")
        slot["done"].synchronize()
        slot["busy"] = False
        return slot["host"]

    def device_outputs(self, ticket: int) -> dict:
        """The device-side outputs of a ticket's slot (valid until ticket + depth is submitted)."""
        return self.slots[ticket % len(self.slots)]["dev"]

    def route(self, x_host: torch.Tensor) -> dict:
        return self.result(self.submit(x_host))
