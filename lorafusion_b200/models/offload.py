"""Activation offloading to pinned host memory over PCIe, overlapped with compute.

A 70B layer's gate|up projection output is 1.9 GB per 16K-token microbatch; keeping it for
every layer does not fit next to the base weights, and rebuilding it costs one of the four big
GEMMs of the layer.  A B200's PCIe 5 link moves about 50 GB/s in each direction at the same
time, which is idle during training -- enough to park that tensor of two layers out of three
in host memory during the forward pass and to bring it back one layer ahead of its backward.

The reference has no counterpart (it relies on gradient checkpointing only,
``lorafusion/utils/gradient_checkpointing.py``).

Streams and ordering: device->host copies run on one side stream, host->device copies on
another; CUDA events order them against the compute stream in both directions.  A tensor
being copied out is held (a plain reference) until its copy has finished and only then handed
back to the caching allocator, so the allocator never has to track cross-stream use and the
device memory taken by copies in flight is bounded (``max_backlog`` tensors).  Returning copies
land in a small ring of preallocated device buffers.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch


def host_memory_available_bytes() -> int:
    """``MemAvailable`` of this machine (0 if unknown)."""
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) * 1024
    except OSError:
        pass
    return 0


def default_host_budget_bytes() -> int:
    """Share of the host memory one rank may pin: 45 % of what is available, divided by the
    number of ranks on this node."""
    local = int(os.environ.get("LOCAL_WORLD_SIZE", "0")) or max(1, torch.cuda.device_count())
    return int(0.45 * host_memory_available_bytes() / local)


def host_slot_bytes(nbytes: int) -> int:
    """Host bytes one offload slot of ``nbytes`` really takes: the size rounded up to whole
    pages.  (``torch.empty(pin_memory=True)`` would round it up to a power of two -- 2 GiB for
    the 1.75 GiB gate|up output of a 16K-token 70B microbatch, one slot in seven wasted.)"""
    page = 4096
    return (int(nbytes) + page - 1) // page * page


class PinnedSlot:
    """A host buffer of exactly the requested size, page-locked with ``cudaHostRegister`` so that
    copies to and from it are asynchronous.  ``close()`` (or garbage collection) unlocks it."""

    def __init__(self, numel: int, dtype):
        self.tensor = torch.empty(int(numel), dtype=dtype)
        self._ptr = self.tensor.data_ptr()
        nbytes = self.tensor.numel() * self.tensor.element_size()
        rt = torch.cuda.cudart()
        err = rt.cudaHostRegister(self._ptr, nbytes, 0)
        ok = (err == rt.cudaError.success) if hasattr(rt, "cudaError") else int(err) == 0
        if not ok:
            self._ptr = None
            raise RuntimeError(f"cudaHostRegister of {nbytes} bytes failed: {err}")

    def close(self) -> None:
        if self._ptr is not None:
            try:
                torch.cuda.cudart().cudaHostUnregister(self._ptr)
            except Exception:   # interpreter shutdown: the driver unlocks the pages with the process
                pass
            self._ptr = None

    def __del__(self):
        self.close()


@dataclass
class OffloadedTensor:
    key: int
    shape: tuple
    numel: int
    done: torch.cuda.Event  # device->host copy finished


def measure_pcie_bandwidth(device, group=None, nbytes: int = 1 << 30, repeats: int = 3) -> tuple[float, float]:
    """``(device->host, host->device)`` bytes per second of this GPU's host link with both
    directions busy at once -- and, when ``group`` is given, with every rank of the group doing
    the same at the same time; the slowest rank's figures are returned on all of them.  GPUs of
    one node share the host's memory bandwidth and often PCIe switches, so the rate a rank gets
    alone says little about what it gets next to seven others."""
    import torch.distributed as dist

    device = torch.device(device)
    dev_a = torch.empty(nbytes, dtype=torch.uint8, device=device)
    dev_b = torch.empty(nbytes, dtype=torch.uint8, device=device)
    host_a = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    host_b = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    s_out, s_in = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def one_round(n):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        with torch.cuda.stream(s_out):
            ev[0].record(s_out)
            for _ in range(n):
                host_a.copy_(dev_a, non_blocking=True)
            ev[1].record(s_out)
        with torch.cuda.stream(s_in):
            ev[2].record(s_in)
            for _ in range(n):
                dev_b.copy_(host_b, non_blocking=True)
            ev[3].record(s_in)
        torch.cuda.synchronize(device)
        return ev[0].elapsed_time(ev[1]) / 1e3, ev[2].elapsed_time(ev[3]) / 1e3

    one_round(1)  # first touch of the pinned pages
    multi = group is not None and dist.is_initialized() and dist.get_world_size(group) > 1
    if multi:
        dist.barrier(group)
    t_out, t_in = one_round(repeats)
    rates = torch.tensor([repeats * nbytes / max(t_out, 1e-9), repeats * nbytes / max(t_in, 1e-9)],
                         dtype=torch.float64, device=device)
    if multi:
        dist.all_reduce(rates, op=dist.ReduceOp.MIN, group=group)
    del dev_a, dev_b, host_a, host_b
    return float(rates[0]), float(rates[1])


class ActivationOffloader:
    RING = 2          # device buffers that returning copies land in (one in use, one arriving)
    MAX_BACKLOG = 2   # tensors held on the device while their outgoing copy is in flight

    def __init__(self, device, slot_numel: int, dtype=torch.bfloat16, ring: int = RING,
                 max_backlog: int = MAX_BACKLOG):
        self.device = torch.device(device)
        self.slot_numel, self.dtype = int(slot_numel), dtype
        self.d2h = torch.cuda.Stream(self.device)
        self.h2d = torch.cuda.Stream(self.device)
        self.host: dict[int, torch.Tensor] = {}
        self._slots: dict[int, PinnedSlot] = {}   # owners of the page-locked memory behind `host`
        self.ring = [torch.empty(self.slot_numel, dtype=dtype, device=self.device) for _ in range(ring)]
        self.ring_free: list[Optional[torch.cuda.Event]] = [None] * ring
        self.next_slot = 0
        self.bytes_out = 0
        self.max_backlog = max_backlog
        self.pending: list = []  # (copy-finished event, tensor being copied out)
        self.backlog_waits = 0

    def reap(self) -> None:
        """Drop the references to tensors whose device->host copy has finished."""
        while self.pending and self.pending[0][0].query():
            self.pending.pop(0)

    def reserve_host(self, keys) -> None:
        """Pin the host slots up front (about 0.65 s per GB); raises if the host refuses."""
        for k in keys:
            if k not in self.host:
                slot = PinnedSlot(self.slot_numel, self.dtype)
                self._slots[k], self.host[k] = slot, slot.tensor

    def close(self) -> None:
        """Wait for the copies in flight and unlock the host memory."""
        self.d2h.synchronize()
        self.h2d.synchronize()
        self.pending.clear()
        self.host.clear()
        for slot in self._slots.values():
            slot.close()
        self._slots.clear()

    def store(self, key: int, t: torch.Tensor) -> OffloadedTensor:
        """Queue the copy of ``t`` (produced on the current stream) to host slot ``key``."""
        if t.numel() > self.slot_numel:
            raise ValueError("tensor larger than the offload slot")
        self.reserve_host([key])
        self.reap()
        while len(self.pending) >= self.max_backlog:  # PCIe is behind: wait on the host
            self.pending.pop(0)[0].synchronize()
            self.backlog_waits += 1
        host = self.host[key][:t.numel()].view(t.shape)
        produced = torch.cuda.Event()
        produced.record()
        self.d2h.wait_event(produced)
        done = torch.cuda.Event()
        with torch.cuda.stream(self.d2h):
            host.copy_(t, non_blocking=True)
            done.record(self.d2h)
        self.pending.append((done, t))
        self.bytes_out += t.numel() * t.element_size()
        return OffloadedTensor(key, tuple(t.shape), t.numel(), done)

    def prefetch(self, off: OffloadedTensor):
        """Start bringing ``off`` back into the next ring buffer.  Returns
        ``(device tensor, ready event, ring slot)``; the consumer waits for the event, uses
        the tensor, then calls :meth:`release`."""
        slot = self.next_slot
        self.next_slot = (slot + 1) % len(self.ring)
        if self.ring_free[slot] is not None:
            self.h2d.wait_event(self.ring_free[slot])
        self.h2d.wait_event(off.done)
        dev = self.ring[slot][:off.numel].view(off.shape)
        ready = torch.cuda.Event()
        with torch.cuda.stream(self.h2d):
            dev.copy_(self.host[off.key][:off.numel].view(off.shape), non_blocking=True)
            ready.record(self.h2d)
        return dev, ready, slot

    def release(self, slot: int) -> None:
        """The consumer (current stream) is done with ring buffer ``slot``."""
        ev = torch.cuda.Event()
        ev.record()
        self.ring_free[slot] = ev
