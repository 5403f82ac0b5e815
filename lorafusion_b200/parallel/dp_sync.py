"""Data-parallel gradient synchronisation for LoRA adapters.

``FusedGradSync`` drives ``csrc/comm/allreduce_adam.cu``: one kernel per adapter does the
reduce-scatter of its gradients over NVLink peer memory, scales them, applies AdamW to the
rank's shard of the optimizer state and writes the new bf16 weights into every rank's
working copy.  ``NcclGradSync`` is the unfused baseline (NCCL all-reduce of the gradient
arena followed by the local Adam kernel), which is what the reference's Megatron DDP + torch
AdamW path amounts to (``lorafusion/ops/multi_lora.py:166-184``).
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from ..models.adapters import LoRAArena
from ..ops import _native as nv
from .symmetric import SymmetricAllocator, SymmetricBuffer, allocate_symmetric, local_buffer


class LfArAdamArgs(C.Structure):
    _fields_ = [
        ("chunks", C.c_void_p),
        ("items", C.c_void_p),
        ("num_items", C.c_int64),
        ("grad", C.c_void_p * 8),
        ("work", C.c_void_p * 8),
        ("grad_mc", C.c_void_p),
        ("work_mc", C.c_void_p),
        ("master", C.c_void_p),
        ("m", C.c_void_p),
        ("v", C.c_void_p),
        ("flags", C.c_void_p * 8),
        ("done_counter", C.c_void_p),
        ("err", C.c_void_p),
        ("stream", C.c_void_p),
        ("num_chunks", C.c_int), ("rank", C.c_int), ("world", C.c_int), ("epoch", C.c_int),
        ("sync_mode", C.c_int), ("use_multimem", C.c_int), ("step", C.c_int), ("wait_ms", C.c_int),
        ("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
        ("weight_decay", C.c_float), ("grad_scale", C.c_float),
        ("trace", C.c_void_p),
    ]


def launch_allreduce_adam(*, chunks: torch.Tensor, items: Optional[torch.Tensor] = None, grad_ptrs, work_ptrs, grad_mc: int, work_mc: int,
                          master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, flag_ptrs,
                          done_counter: Optional[torch.Tensor], rank: int, world: int, epoch: int,
                          sync: bool, use_multimem: bool, step: int, lr: float, beta1: float, beta2: float,
                          eps: float, weight_decay: float, grad_scale: float, device, wait_ms: int = 0,
                          trace: Optional[torch.Tensor] = None) -> None:
    """``trace`` (optional, int64 ``[num_items, 3]`` on the device) receives per block the
    ``globaltimer`` nanoseconds at entry, when every rank's gradients were seen complete, and at
    exit (see :func:`summarize_sync_trace`)."""
    lib = nv.cuda_lib()
    if not getattr(lib, "_lf_ar_declared", False):
        lib.lf_allreduce_adam.argtypes = [C.POINTER(LfArAdamArgs)]
        lib.lf_allreduce_adam.restype = C.c_int
        lib._lf_ar_declared = True
    if items is None:  # tests; the trainer passes the arena's cached table
        from ..ops.elementwise import build_adam_work_items

        items = build_adam_work_items(chunks.cpu().tolist(), rank=rank, world=world).to(chunks.device)
    a = LfArAdamArgs()
    a.chunks = chunks.data_ptr()
    a.items, a.num_items = items.data_ptr(), items.shape[0]
    for r in range(world):
        a.grad[r] = grad_ptrs[r]
        a.work[r] = work_ptrs[r]
        a.flags[r] = flag_ptrs[r] if flag_ptrs else None
    a.grad_mc, a.work_mc = (grad_mc or None), (work_mc or None)
    a.master, a.m, a.v = master.data_ptr(), m.data_ptr(), v.data_ptr()
    a.done_counter = done_counter.data_ptr() if done_counter is not None else None
    a.err = nv.err_word(device).data_ptr()
    a.stream = nv.current_stream_ptr()
    a.num_chunks, a.rank, a.world, a.epoch = chunks.shape[0], rank, world, epoch
    a.sync_mode, a.use_multimem, a.step = int(sync), int(use_multimem), step
    a.wait_ms = int(wait_ms)  # 0 = default limit (10 s) of the cross-rank flag waits
    a.lr, a.beta1, a.beta2, a.eps = lr, beta1, beta2, eps
    a.weight_decay, a.grad_scale = weight_decay, grad_scale
    if trace is not None:
        if trace.dtype != torch.int64 or trace.numel() < 3 * items.shape[0]:
            raise ValueError("trace must be int64 with at least 3 entries per work item")
        a.trace = trace.data_ptr()
    nv.note_launch()
    rc = lib.lf_allreduce_adam(C.byref(a))
    if rc != 0:
        raise RuntimeError(f"lf_allreduce_adam failed with code {rc}")


def summarize_sync_trace(trace: torch.Tensor, num_items: int) -> dict:
    """Microseconds from the in-kernel stamps of one launch: how long the first block waited
    for the peers' gradients, how long the reduce + Adam + broadcast part took, and the span of
    the whole kernel on the device (same clock for every kernel of a GPU, so spans of different
    kernels can be laid over each other to see overlap)."""
    t = trace[:3 * num_items].view(num_items, 3).cpu()
    t0, t1, t2 = t[:, 0], t[:, 1], t[:, 2]
    return {"start_ns": int(t0.min()), "end_ns": int(t2.max()),
            "span_us": float(t2.max() - t0.min()) / 1e3,
            "max_wait_for_peers_us": float((t1 - t0).max()) / 1e3,
            "mean_work_us": float((t2 - t1).double().mean()) / 1e3}


class FusedGradSync:
    """Reduce + Adam + broadcast in one kernel per adapter.  The arena's ``grad`` and ``work``
    tensors must come from ``allocator`` (a :class:`SymmetricAllocator`)."""

    def __init__(self, arena: LoRAArena, allocator: SymmetricAllocator, group, optim, *,
                 use_multimem: bool = False):
        self.arena, self.optim, self.group = arena, optim, group
        self.grad_h: SymmetricBuffer = allocator.handle_of(arena.grad)
        self.work_h: SymmetricBuffer = allocator.handle_of(arena.work)
        self.world, self.rank = self.grad_h.world, self.grad_h.rank
        dev = arena.device
        self.flags_h = allocate_symmetric(16, torch.int32, dev, group) if self.world > 1 \
            else local_buffer(16, torch.int32, dev)
        self.flags_h.tensor.zero_()
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        self.epoch = 0
        self.trace: Optional[torch.Tensor] = None   # set to an int64 device tensor to collect in-kernel stamps
        self.last_num_items = 0
        self.use_multimem = bool(use_multimem and self.grad_h.has_multicast and self.work_h.has_multicast)
        if self.world > 1:
            torch.cuda.synchronize(dev)
            dist.barrier(group)  # flags are zeroed everywhere before the first kernel

    def begin_step(self, adapter: int) -> int:
        """Count one optimizer step of ``adapter`` (once per step, however many layer groups the
        step is launched in) and return its number."""
        self.arena.steps[adapter] += 1
        return self.arena.steps[adapter]

    def reduce_and_step(self, adapter: int, grad_scale: float, *, layers: Optional[tuple] = None,
                        step: Optional[int] = None) -> None:
        """Launch the fused kernel for ``adapter`` on the current stream.  ``layers = (lo, hi)``
        limits it to the regions of those layers, with ``step`` from :meth:`begin_step`; every
        rank must launch the same sequence of groups."""
        o, ar = self.optim, self.arena
        if step is None:
            step = self.begin_step(adapter)
        items = ar.work_items(adapter, self.rank, self.world, layers=layers)
        if items.shape[0] == 0:
            if self.world == 1:
                return
            raise RuntimeError("this rank owns no part of the requested layer group; the ranks would fall out of step")
        self.epoch += 1
        launch_allreduce_adam(
            chunks=ar.chunk_table(adapter), items=items,
            grad_ptrs=self.grad_h.peer_ptrs, work_ptrs=self.work_h.peer_ptrs,
            grad_mc=self.grad_h.multicast_ptr, work_mc=self.work_h.multicast_ptr, master=ar.master, m=ar.m,
            v=ar.v, flag_ptrs=self.flags_h.peer_ptrs, done_counter=self.done, rank=self.rank, world=self.world,
            epoch=self.epoch, sync=self.world > 1, use_multimem=self.use_multimem, step=step,
            lr=o.lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps, weight_decay=o.weight_decay,
            grad_scale=grad_scale, device=ar.device, trace=self.trace)
        self.last_num_items = int(items.shape[0])


class NcclGradSync:
    """Baseline: NCCL all-reduce of the whole gradient arena, then the local Adam kernel."""

    def __init__(self, arena: LoRAArena, group, optim):
        self.arena, self.group, self.optim = arena, group, optim
        self._reduced_for_step = -1

    def all_reduce(self) -> None:
        dist.all_reduce(self.arena.grad, group=self.group)

    def reduce_and_step(self, adapter: int, grad_scale: float) -> None:
        o = self.optim
        self.arena.adam_step(adapter, lr=o.lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps,
                             weight_decay=o.weight_decay, grad_scale=grad_scale)
