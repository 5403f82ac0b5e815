"""Storage of every LoRA adapter of a model (or pipeline stage) in flat arenas.

The reference keeps adapters as PEFT modules named ``lora_{i}`` and, for multi-LoRA data
parallelism, wraps each adapter's parameters in a fake ``nn.Module`` with its own Megatron
DDP grad buffer and AdamW (``benchmarks_paper/bench_multi_gpu.py:162-203,276-287``).  Here
all adapters live in flat 1-D arenas.  Two of them share one rank-padded layout, the one
the GEMM kernels address:

    work (bf16, read by the GEMM kernels) | grad (fp32, accumulated by the GEMM kernels)

and three hold ONLY the trainable elements, packed densely (a rank-16 adapter fills a quarter
of its rank-64 slot, so the padded layout would quadruple the optimizer state):

    master | m | v   (fp32, indexed through the ``state`` field of the chunk table)

Per merged projection the arena holds stacks ``A [n, R, K]`` and ``B [n, N, R]``
(``ops/lora.py``).  Merged projections (q|k|v and gate|up) keep one LoRA per sub-projection:
adapter ``i`` with rank ``r_i`` uses rows ``[j * slot, j * slot + r_i)`` of ``A`` for
sub-projection ``j`` and the matching columns of the rows of ``B`` that belong to ``j``
(block-diagonal ``B``); everything else stays zero and is excluded from the optimizer through
the chunk table (``AdamChunk`` regions: offset, rows, ld, col0, cols, state -- element
``(row, col)`` of the trainable window has its optimizer state at
``state + row * cols + (col - col0)``).

One chunk table per adapter lets a single kernel launch apply Adam to -- or a single fused
kernel reduce across data-parallel ranks -- all tensors of that adapter.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from ..ops.lora import LoRAStack, rank_pad
from .config import AdapterSpec, ModelConfig

# merged projection -> (sub-projection names, output sizes) resolved per model
PROJECTIONS = ("qkv", "o", "gate_up", "down")


def projection_layout(cfg: ModelConfig) -> dict[str, dict]:
    h, i = cfg.hidden_size, cfg.intermediate_size
    return {
        "qkv": dict(K=h, subs=[("q_proj", cfg.q_size), ("k_proj", cfg.kv_size), ("v_proj", cfg.kv_size)]),
        "o": dict(K=cfg.q_size, subs=[("o_proj", h)]),
        "gate_up": dict(K=h, subs=[("gate_proj", i), ("up_proj", i)]),
        "down": dict(K=i, subs=[("down_proj", h)]),
    }


@dataclass
class StackView:
    """Location of one (layer, projection) stack inside the arenas."""

    layer: int
    proj: str
    K: int
    N: int
    R: int
    slot: int
    subs: list  # [(name, out_size)]
    a_offset: int
    b_offset: int
    stack: Optional[LoRAStack] = None


class LoRAArena:
    def __init__(self, cfg: ModelConfig, adapters: Sequence[AdapterSpec], layers: Sequence[int],
                 device, *, init_b_std: float = 0.0, seed: int = 0, with_optimizer_state: bool = True,
                 shared_alloc=None):
        """``shared_alloc(numel, dtype) -> 1-D tensor`` (optional) provides the memory of the
        two arenas other ranks must reach -- the fp32 gradients and the bf16 working copy --
        e.g. from NVLink symmetric memory; everything else is ordinary device memory."""
        self.cfg = cfg
        self.adapters = list(adapters)
        self.layers = list(layers)
        self.device = torch.device(device)
        n = len(self.adapters)
        self.num_adapters = n
        self.slot = max([a.r for a in self.adapters], default=16)
        layout = projection_layout(cfg)
        self.views: dict[tuple[int, str], StackView] = {}
        off = 0
        for l in self.layers:
            for proj in PROJECTIONS:
                K, subs = layout[proj]["K"], layout[proj]["subs"]
                N = sum(s for _, s in subs)
                R = rank_pad(len(subs) * self.slot)
                a_off = off
                off += n * R * K
                b_off = off
                off += n * N * R
                self.views[(l, proj)] = StackView(l, proj, K, N, R, self.slot, list(subs), a_off, b_off)
        off = (off + 127) // 128 * 128
        self.numel = off
        if shared_alloc is not None:
            self.work = shared_alloc(off, torch.bfloat16)
            self.grad = shared_alloc(off, torch.float32)
            self.work.zero_()
            self.grad.zero_()
        else:
            self.work = torch.zeros(off, dtype=torch.bfloat16, device=self.device)
            self.grad = torch.zeros(off, dtype=torch.float32, device=self.device)
        self._build_chunk_rows()
        if with_optimizer_state:
            self.master = torch.zeros(self.state_numel, dtype=torch.float32, device=self.device)
            self.m = torch.zeros(self.state_numel, dtype=torch.float32, device=self.device)
            self.v = torch.zeros(self.state_numel, dtype=torch.float32, device=self.device)
        else:
            self.master = self.m = self.v = None
        for v in self.views.values():
            n_a, n_b = n * v.R * v.K, n * v.N * v.R
            v.stack = LoRAStack(
                self.work[v.a_offset:v.a_offset + n_a].view(n, v.R, v.K),
                self.work[v.b_offset:v.b_offset + n_b].view(n, v.N, v.R),
                self.grad[v.a_offset:v.a_offset + n_a].view(n, v.R, v.K),
                self.grad[v.b_offset:v.b_offset + n_b].view(n, v.N, v.R))
        self.steps = [0] * n
        self._chunks: dict[int, torch.Tensor] = {}
        self._work_items: dict[tuple, torch.Tensor] = {}
        self._init_weights(init_b_std, seed)

    # ------------------------------------------------------------------ layout helpers
    def targets(self, adapter: int, sub_name: str) -> bool:
        return sub_name in self.adapters[adapter].target_modules

    def sub_slices(self, view: StackView, adapter: int):
        """Yield ``(sub_name, row0_of_B, out_size, rank_col0, rank)`` for the sub-projections
        adapter ``adapter`` is attached to."""
        r = self.adapters[adapter].r
        n0 = 0
        for j, (name, size) in enumerate(view.subs):
            if self.targets(adapter, name):
                yield name, n0, size, j * view.slot, r
            n0 += size

    def stack(self, layer: int, proj: str) -> LoRAStack:
        return self.views[(layer, proj)].stack

    # ------------------------------------------------------------------ init
    def _init_weights(self, init_b_std: float, seed: int) -> None:
        """PEFT's default LoRA init: A ~ kaiming-uniform(a = sqrt 5) i.e. U(-1/sqrt K, 1/sqrt K),
        B = 0 (or N(0, init_b_std) when a non-zero B is wanted for testing/benchmarks).  The
        fp32 master starts as the bf16-rounded value the kernels read."""
        g = torch.Generator(device=self.device).manual_seed(seed)
        n = self.num_adapters
        for v in self.views.values():
            bound = 1.0 / math.sqrt(v.K)
            for i in range(n):
                for name, n0, size, c0, r in self.sub_slices(v, i):
                    a = torch.empty(r, v.K, dtype=torch.float32, device=self.device)
                    a.uniform_(-bound, bound, generator=g)
                    v.stack.a[i, c0:c0 + r].copy_(a)
                    if init_b_std > 0:
                        b = torch.empty(size, r, dtype=torch.float32, device=self.device)
                        b.normal_(0.0, init_b_std, generator=g)
                        v.stack.b[i, n0:n0 + size, c0:c0 + r].copy_(b)
        self.sync_master_from_work()

    def sync_master_from_work(self, adapter: Optional[int] = None) -> None:
        """Set the fp32 master weights to the current bf16 working values."""
        if self.master is None:
            return
        for i in (range(self.num_adapters) if adapter is None else [adapter]):
            for v in self.views.values():
                for name, n0, size, c0, r in self.sub_slices(v, i):
                    sa, sb = self.state_offsets[(v.layer, v.proj, i, name)]
                    self.master[sa:sa + r * v.K].view(r, v.K).copy_(v.stack.a[i, c0:c0 + r])
                    self.master[sb:sb + size * r].view(size, r).copy_(v.stack.b[i, n0:n0 + size, c0:c0 + r])

    # ------------------------------------------------------------------ chunk tables
    def _build_chunk_rows(self) -> None:
        """Lay out every adapter's regions and assign its dense optimizer-state offsets.
        Adapter ``i`` owns the contiguous state range ``state_range[i]``."""
        self._chunk_rows: dict[int, list] = {}
        self._chunk_layers: dict[int, list] = {}   # layer of every chunk row (rows are layer-major)
        self.state_offsets: dict[tuple, tuple[int, int]] = {}
        self.state_range: dict[int, tuple[int, int]] = {}
        state = 0

        def take(count: int) -> int:
            nonlocal state
            at = state
            state += (count + 3) // 4 * 4  # keep every region 16-byte aligned
            return at

        for adapter in range(self.num_adapters):
            rows = []
            row_layers: list = []
            lo = state
            for v in self.views.values():
                n_before = len(rows)
                a_base = v.a_offset + adapter * v.R * v.K
                b_base = v.b_offset + adapter * v.N * v.R
                a_state = {}
                # A: whole [R, K] block is cleared; trainable rows are contiguous per sub
                covered = 0
                for name, _, _, c0, r in self.sub_slices(v, adapter):
                    if c0 > covered:  # untargeted slot rows: clear only
                        rows.append((a_base + covered * v.K, 1, (c0 - covered) * v.K, 0, 0, 0))
                    a_state[name] = take(r * v.K)
                    rows.append((a_base + c0 * v.K, 1, r * v.K, 0, r * v.K, a_state[name]))
                    covered = c0 + r
                if covered < v.R:
                    rows.append((a_base + covered * v.K, 1, (v.R - covered) * v.K, 0, 0, 0))
                # B: per sub-projection a row block with a column window
                n0 = 0
                for j, (name, size) in enumerate(v.subs):
                    if self.targets(adapter, name):
                        r = self.adapters[adapter].r
                        b_state = take(size * r)
                        rows.append((b_base + n0 * v.R, size, v.R, j * v.slot, r, b_state))
                        self.state_offsets[(v.layer, v.proj, adapter, name)] = (a_state[name], b_state)
                    else:
                        rows.append((b_base + n0 * v.R, size, v.R, 0, 0, 0))
                    n0 += size
                row_layers += [v.layer] * (len(rows) - n_before)
            if any(r[1] * r[2] >= 2 ** 31 for r in rows):
                raise ValueError("an adapter region of 2^31 elements or more is not supported by the optimizer kernels")
            self._chunk_rows[adapter] = rows
            self._chunk_layers[adapter] = row_layers
            self.state_range[adapter] = (lo, state)
        self.state_numel = max(state, 4)

    def chunk_table(self, adapter: int) -> torch.Tensor:
        """int64 ``[n_chunks, 6]`` regions (offset, rows, ld, col0, cols, state) covering every
        tensor of ``adapter``; the gradient of the whole region is consumed, only the
        trainable window is updated, with its optimizer state at ``state``."""
        t = self._chunks.get(adapter)
        if t is None:
            t = torch.tensor(self._chunk_rows[adapter], dtype=torch.int64, device=self.device).view(-1, 6)
            self._chunks[adapter] = t
        return t

    def work_items(self, adapter: int, rank: int = 0, world: int = 1,
                   layers: Optional[tuple] = None) -> torch.Tensor:
        """Device table of equal-sized pieces of ``adapter``'s regions for the optimizer
        kernels (``ops.elementwise.build_adam_work_items``); slice ``rank`` of ``world`` for the
        fused data-parallel kernel.  ``layers = (lo, hi)`` restricts the table to the regions of
        layers ``lo <= l < hi`` (the gradient sync of a layer group can start as soon as the
        last backward has passed those layers)."""
        from ..ops.elementwise import build_adam_work_items

        key = (adapter, rank, world, layers)
        t = self._work_items.get(key)
        if t is None:
            t = build_adam_work_items(self._chunk_rows[adapter], rank=rank, world=world)
            if layers is not None:
                lay = torch.tensor(self._chunk_layers[adapter], dtype=torch.int64)
                keep = (lay[t[:, 0].long()] >= layers[0]) & (lay[t[:, 0].long()] < layers[1])
                t = t[keep].contiguous()
            t = t.to(self.device)
            self._work_items[key] = t
        return t

    def trainable_numel(self, adapter: int) -> int:
        tot = 0
        for v in self.views.values():
            for _, _, size, _, r in self.sub_slices(v, adapter):
                tot += r * v.K + size * r
        return tot

    # ------------------------------------------------------------------ optimizer
    def adam_step(self, adapter: int, *, lr: float, beta1: float = 0.9, beta2: float = 0.999,
                  eps: float = 1e-8, weight_decay: float = 0.0, grad_scale: float = 1.0) -> None:
        from ..ops.elementwise import adam_chunks

        if self.master is None:
            raise RuntimeError("arena was created without optimizer state")
        self.steps[adapter] += 1
        adam_chunks(self.chunk_table(adapter), self.grad, self.master, self.m, self.v, self.work,
                    lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay,
                    step=self.steps[adapter], grad_scale=grad_scale, items=self.work_items(adapter))

    def zero_grad(self) -> None:
        self.grad.zero_()

    def adapter_grad_regions(self, adapter: int) -> list:
        """1-D views of the gradient arena covering every region of ``adapter``."""
        return [self.grad[off:off + rows * ld] for off, rows, ld, _, _, _ in self._chunk_rows[adapter]]

    def all_reduce_adapter_grads(self, adapter: int, group) -> None:
        """NCCL all-reduce of one adapter's gradients (the unfused data-parallel baseline)."""
        import torch.distributed as dist

        views = self.adapter_grad_regions(adapter)
        flat = torch.cat(views)
        dist.all_reduce(flat, group=group)
        off = 0
        for v in views:
            v.copy_(flat[off:off + v.numel()])
            off += v.numel()

    # ------------------------------------------------------------------ per-adapter tensors
    def _source(self, source: str) -> Optional[torch.Tensor]:
        if source not in ("master", "m", "v", "work"):
            raise ValueError(f"unknown adapter tensor source {source!r}")
        return None if source == "work" else getattr(self, source)

    def export_adapter(self, adapter: int, source: Optional[str] = None) -> dict[str, torch.Tensor]:
        """``{"layers.{l}.{sub}.lora_A": [r, K], "...lora_B": [N_sub, r]}``.  ``source`` picks
        what is read: ``"master"`` (fp32 weights), ``"m"`` / ``"v"`` (Adam moments, same shapes),
        ``"work"`` (the bf16 copy the kernels read); default = master if present, else work."""
        if source is None:
            source = "master" if self.master is not None else "work"
        dense = self._source(source)
        out = {}
        for (l, _), v in self.views.items():
            for name, n0, size, c0, r in self.sub_slices(v, adapter):
                if dense is not None:
                    sa, sb = self.state_offsets[(v.layer, v.proj, adapter, name)]
                    a = dense[sa:sa + r * v.K].view(r, v.K)
                    b = dense[sb:sb + size * r].view(size, r)
                else:
                    a = v.stack.a[adapter, c0:c0 + r]
                    b = v.stack.b[adapter, n0:n0 + size, c0:c0 + r]
                out[f"layers.{l}.{name}.lora_A"] = a.clone()
                out[f"layers.{l}.{name}.lora_B"] = b.clone()
        return out

    def import_adapter(self, adapter: int, tensors: dict[str, torch.Tensor], target: str = "weights") -> None:
        """``target="weights"`` writes the bf16 working copy and the fp32 master; ``"m"`` /
        ``"v"`` write an Adam moment (same keys and shapes)."""
        if target not in ("weights", "m", "v"):
            raise ValueError(f"unknown import target {target!r}")
        for (l, _), v in self.views.items():
            for name, n0, size, c0, r in self.sub_slices(v, adapter):
                ka, kb = f"layers.{l}.{name}.lora_A", f"layers.{l}.{name}.lora_B"
                if ka not in tensors or kb not in tensors:
                    raise KeyError(f"missing {ka} / {kb}")
                if target == "weights":
                    v.stack.a[adapter, c0:c0 + r].copy_(tensors[ka])
                    v.stack.b[adapter, n0:n0 + size, c0:c0 + r].copy_(tensors[kb])
                dense = self.master if target == "weights" else getattr(self, target)
                if dense is not None:
                    sa, sb = self.state_offsets[(v.layer, v.proj, adapter, name)]
                    dense[sa:sa + r * v.K].view(r, v.K).copy_(tensors[ka])
                    dense[sb:sb + size * r].view(size, r).copy_(tensors[kb])

    # ------------------------------------------------------------------ sharded optimizer state
    def owned_state_mask(self, adapter: int, rank: int, world: int) -> torch.Tensor:
        """Which elements of ``adapter``'s dense optimizer-state range data-parallel rank
        ``rank`` owns under the fused gradient sync (bool ``[hi - lo]``).  That kernel updates
        ``master`` / ``m`` / ``v`` only on the owner of each slice of each region (the same split
        as :func:`lorafusion_b200.ops.elementwise.dp_slice`); everywhere else they keep their
        old values, so a checkpoint must be stitched from the owners."""
        from ..ops.elementwise import dp_slice

        lo_s, hi_s = self.state_range[adapter]
        mask = torch.zeros(hi_s - lo_s, dtype=torch.bool, device=self.device)
        for _, rows, ld, col0, cols, state in self._chunk_rows[adapter]:
            if cols == 0:
                continue
            lo, hi = dp_slice(rows * ld, rank, world)
            if hi <= lo:
                continue
            r0, r1 = lo // ld, (hi - 1) // ld
            base = state - lo_s
            for row in {r0, r1}:  # first and last row may be covered in part
                c_lo, c_hi = max(col0, lo - row * ld), min(col0 + cols, hi - row * ld)
                if c_hi > c_lo:
                    mask[base + row * cols + (c_lo - col0):base + row * cols + (c_hi - col0)] = True
            if r1 - r0 >= 2:
                mask[base + (r0 + 1) * cols:base + r1 * cols] = True
        return mask

    def gather_owned_state(self, group, rank: int, world: int) -> None:
        """Collective over the data-parallel ``group``: make ``master`` / ``m`` / ``v`` complete
        on every rank by taking each element from its owner (non-owned elements are zeroed and
        the group sums).  Needed before saving a checkpoint under the fused gradient sync."""
        import torch.distributed as dist

        if world <= 1 or self.master is None:
            return
        for adapter in range(self.num_adapters):
            lo, hi = self.state_range[adapter]
            mask = self.owned_state_mask(adapter, rank, world)
            for t in (self.master, self.m, self.v):
                seg = t[lo:hi]
                seg.masked_fill_(~mask, 0.0)
                dist.all_reduce(seg, group=group)
