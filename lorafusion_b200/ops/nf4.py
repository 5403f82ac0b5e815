"""NF4 storage of frozen base weights: quantiser, standalone dequantiser and the
``NF4Weight`` container.

Layout (the bitsandbytes one the reference's Triton dequantiser reads,
``lorafusion/ops/triton_ops/dequantize_nf4.py:16-161``): 64-element blocks over the
row-major flattened ``[N, K]`` weight, one absmax per block, two 4-bit codes per byte with
the even element in the high nibble; with ``double_quant`` the absmax vector is stored as
8-bit indices into a 256-entry code table with one fp32 scale per 256 blocks and a global
offset (its mean).

The 4-bit quantise/dequantise passes are CUDA kernels (``csrc/nf4/nf4_codec.cu``); the
second-level quantisation of the small absmax vector runs once at load time with torch ops.
A pure-PyTorch implementation of both directions is the CPU oracle.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _native as nv

NF4_CODE = torch.tensor([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
], dtype=torch.float32)

BLOCK = 64
NESTED_BLOCK = 256


def dynamic_code_8bit() -> torch.Tensor:
    """Signed 8-bit "dynamic" code table used for the second-level absmax quantisation:
    for each of 7 decades a linearly spaced set of mantissa midpoints (more points for the
    larger decades), mirrored for negative values, plus 0 and 1; 256 sorted entries."""
    data: list[float] = []
    max_exp_bits, non_sign_bits = 7, 7
    for i in range(max_exp_bits):
        items = int(2 ** (i + non_sign_bits - max_exp_bits) + 1)
        bounds = torch.linspace(0.1, 1, items)
        means = (bounds[:-1] + bounds[1:]) / 2.0
        scale = 10 ** (-(max_exp_bits - 1) + i)
        data += (scale * means).tolist()
        data += (-scale * means).tolist()
    data += [0.0, 1.0]
    data += [0.0] * (256 - len(data))
    return torch.tensor(sorted(data), dtype=torch.float32)


@dataclass
class NF4Weight:
    """A frozen ``[N, K]`` weight in NF4."""

    packed: torch.Tensor               # uint8 [N, K // 2]
    shape: tuple[int, int]
    absmax: Optional[torch.Tensor]     # fp32 [N * K / 64] (None when double-quantised)
    absmax_q: Optional[torch.Tensor] = None   # uint8 [N * K / 64]
    code256: Optional[torch.Tensor] = None    # fp32 [256]
    nested: Optional[torch.Tensor] = None     # fp32 [ceil(nblocks / 256)]
    offset: float = 0.0

    @property
    def device(self):
        return self.packed.device

    def nbytes(self) -> int:
        n = self.packed.numel()
        for t in (self.absmax, self.absmax_q, self.code256, self.nested):
            if t is not None:
                n += t.numel() * t.element_size()
        return n

    def fp32_block_scales(self) -> torch.Tensor:
        """:meth:`block_scales`, computed once and kept (the fused NF4 GEMM reads one fp32
        scale per 64-element block; costs 1/16 byte per weight on top of the 0.5 of NF4)."""
        cached = getattr(self, "_fp32_scales", None)
        if cached is None:
            cached = self.block_scales().contiguous()
            object.__setattr__(self, "_fp32_scales", cached)
        return cached

    def block_scales(self) -> torch.Tensor:
        """fp32 scale of every 64-element block (second level undone)."""
        if self.absmax_q is None:
            return self.absmax
        idx = torch.arange(self.absmax_q.numel(), device=self.device) // NESTED_BLOCK
        return self.code256[self.absmax_q.long()] * self.nested[idx] + self.offset


def _nearest_code(x: torch.Tensor, code: torch.Tensor) -> torch.Tensor:
    mids = (code[:-1] + code[1:]) / 2
    return torch.bucketize(x, mids.to(x.device), right=False)


def _double_quantize(absmax: torch.Tensor):
    code = dynamic_code_8bit().to(absmax.device)
    offset = float(absmax.mean())
    centered = absmax - offset
    n = centered.numel()
    pad = (-n) % NESTED_BLOCK
    padded = torch.nn.functional.pad(centered, (0, pad)).view(-1, NESTED_BLOCK)
    nested = padded.abs().amax(dim=1).clamp_min(1e-12)
    q = _nearest_code((padded / nested[:, None]).reshape(-1)[:n], code).to(torch.uint8)
    return q, code, nested.contiguous(), offset


def quantize_nf4(w: torch.Tensor, double_quant: bool = True) -> NF4Weight:
    """Quantise a bf16 ``[N, K]`` weight (``K % 64 == 0``).  CUDA tensors use the native
    kernel, CPU tensors the torch oracle (bit-identical codes)."""
    N, K = w.shape
    if K % BLOCK:
        raise ValueError("K must be a multiple of 64")
    w = w.contiguous()
    if w.is_cuda:
        packed = torch.empty((N, K // 2), dtype=torch.uint8, device=w.device)
        absmax = torch.empty(N * K // BLOCK, dtype=torch.float32, device=w.device)
        nv.call("lf_nf4_quantize", w.to(torch.bfloat16).data_ptr(), packed.data_ptr(),
                absmax.data_ptr(), N * K, nv.current_stream_ptr())
    else:
        blocks = w.float().view(-1, BLOCK)
        absmax = blocks.abs().amax(dim=1)
        inv = torch.where(absmax > 0, 1.0 / absmax, torch.zeros_like(absmax))
        q = _nearest_code(blocks * inv[:, None], NF4_CODE).to(torch.uint8).view(N, K)
        packed = (q[:, 0::2] << 4) | q[:, 1::2]
    if not double_quant:
        return NF4Weight(packed, (N, K), absmax)
    q8, code, nested, offset = _double_quantize(absmax)
    return NF4Weight(packed, (N, K), None, q8, code, nested, offset)


def dequantize_nf4_reference(qw: NF4Weight, dtype=torch.bfloat16) -> torch.Tensor:
    """Plain PyTorch dequantisation (CPU or GPU) -- the oracle for the kernels."""
    N, K = qw.shape
    p = qw.packed
    q = torch.stack([(p >> 4) & 0xF, p & 0xF], dim=-1).view(N, K).long()
    vals = NF4_CODE.to(p.device)[q].view(-1, BLOCK)
    return (vals * qw.block_scales()[:, None]).view(N, K).to(dtype)


def dequantize_nf4(qw: NF4Weight, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 ``[N, K]`` from NF4 with the native kernel."""
    N, K = qw.shape
    if not qw.packed.is_cuda:
        return dequantize_nf4_reference(qw)
    if out is None:
        out = torch.empty((N, K), dtype=torch.bfloat16, device=qw.device)
    p = lambda t: None if t is None else t.data_ptr()  # noqa: E731
    nv.call("lf_nf4_dequantize", qw.packed.data_ptr(), p(qw.absmax), p(qw.absmax_q),
            p(qw.code256), p(qw.nested), qw.offset, out.data_ptr(), N * K,
            nv.current_stream_ptr())
    return out
