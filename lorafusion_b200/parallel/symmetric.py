"""Symmetric (peer-addressable) device memory for kernels that talk over NVLink.

A :class:`SymmetricBuffer` is the same-sized allocation on every rank of a group together
with every peer's device pointer to it and, when NVSwitch multicast (NVLS) is available, one
multicast address that reaches all copies at once.  Allocation and handle exchange go through
``torch.distributed._symmetric_memory`` (the plumbing); the kernels of ``csrc/comm`` do the
transfers themselves with P2P loads/stores or ``multimem`` instructions.

Role in the design: the runtime's "symmetric heap" -- peer pointers, multicast pointer,
epoch flags -- that the reference, which only ever calls NCCL through Megatron, has no
counterpart for.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class SymmetricBuffer:
    tensor: torch.Tensor
    peer_ptrs: list
    multicast_ptr: int
    rank: int
    world: int

    @property
    def has_multicast(self) -> bool:
        return self.multicast_ptr != 0


def allocate_symmetric(numel: int, dtype: torch.dtype, device, group) -> SymmetricBuffer:
    """Collective: every rank of ``group`` must call with the same ``numel`` / ``dtype``."""
    import torch.distributed._symmetric_memory as symm_mem

    t = symm_mem.empty(numel, dtype=dtype, device=device)
    hdl = symm_mem.rendezvous(t, group)
    mc = int(hdl.multicast_ptr) if getattr(hdl, "multicast_ptr", 0) else 0
    return SymmetricBuffer(t, [int(p) for p in hdl.buffer_ptrs], mc, hdl.rank, hdl.world_size)


def local_buffer(numel: int, dtype: torch.dtype, device) -> SymmetricBuffer:
    """Single-rank stand-in (world 1) backed by ordinary device memory."""
    t = torch.zeros(numel, dtype=dtype, device=device)
    return SymmetricBuffer(t, [t.data_ptr()], 0, 0, 1)


class SymmetricAllocator:
    """Hands out symmetric tensors and remembers their handles by data pointer."""

    def __init__(self, device, group):
        self.device, self.group = torch.device(device), group
        self.buffers: dict[int, SymmetricBuffer] = {}

    def __call__(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        world = dist.get_world_size(self.group) if (dist.is_initialized() and self.group is not None) else 1
        buf = allocate_symmetric(numel, dtype, self.device, self.group) if world > 1 \
            else local_buffer(numel, dtype, self.device)
        self.buffers[buf.tensor.data_ptr()] = buf
        return buf.tensor

    def handle_of(self, t: torch.Tensor) -> SymmetricBuffer:
        return self.buffers[t.data_ptr()]
