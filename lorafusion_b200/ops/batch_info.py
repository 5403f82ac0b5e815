"""Per-microbatch description of which adapter owns which tokens.

``prepare_multi_lora_batch_info`` keeps the call signature and the dataclass fields of the
reference (``lorafusion/ops/multi_lora.py:295-453``) -- ``block_to_lookup_table`` rows are
``(rank, valid_rows, first_block_of_segment)`` -- and adds what the sm_100a kernels consume:

* ``tile_adapter``   int32 ``[n_blocks]``  adapter id of every 128-token tile (-1 = none)
* ``adapter_scale``  fp32  ``[n_adapters]`` LoRA scaling (fp32, not bf16 as in the reference)
* ``adapter_thresh16`` / ``adapter_inv_keep``  per-adapter dropout threshold and 1/(1-p)
* ``segments``       host list ``(adapter, start_row, end_row)``

Everything is assembled vectorised in ONE pinned staging buffer and moved with ONE
host-to-device copy (the reference fills its tables element by element in a Python loop and
rebuilds device pointer tables in every linear call).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

import numpy as np
import torch

from .lora_kernels import DropoutSpec, SegmentTable, TILE_M
from .philox import dropout_threshold


@dataclass
class MultiLoRABatchInfo:
    # inputs (reference field names)
    seq_len_list: list[int]
    lora_idx_list: list[int]
    lora_rank_list: list[int]
    dropout_p_list: list[float]
    alpha_list: list[float]
    block_size_m: int
    # derived (reference field names)
    padded_seq_len_list: list[int]
    block_to_lookup_table: torch.Tensor
    block_to_dropout_p: torch.Tensor
    block_to_alpha: torch.Tensor
    enable_dropout: bool
    same_dropout_p_value: Optional[float]
    max_r: int
    microbatch_idx: Optional[int] = None
    micro_batch_info: Any = None
    allow_empty_micro_batch_info: bool = False
    # native additions
    tile_adapter: Optional[torch.Tensor] = None
    adapter_scale: Optional[torch.Tensor] = None
    adapter_thresh16: Optional[torch.Tensor] = None
    adapter_inv_keep: Optional[torch.Tensor] = None
    segments: list[tuple[int, int, int]] = field(default_factory=list)
    segment_table: Optional[SegmentTable] = None
    seed: int = 0
    total_padded_tokens: int = 0

    @property
    def alpha_by_adapter(self) -> dict:
        """Host-side ``{adapter id: LoRA scaling}`` (no device read)."""
        return {a: self.alpha_list[i] for i, a in enumerate(self.lora_idx_list) if a >= 0}

    @property
    def dropout_by_adapter(self) -> dict:
        return {a: self.dropout_p_list[i] for i, a in enumerate(self.lora_idx_list) if a >= 0}

    @property
    def num_active_adapters(self) -> int:
        return len({i for i in self.lora_idx_list if i >= 0})

    def dropout_spec(self, stream_id: int, training: bool = True) -> DropoutSpec:
        """Dropout description for one linear call site (``stream_id`` distinguishes layers
        and projections so that they draw independent masks)."""
        if not (training and self.enable_dropout):
            return DropoutSpec()
        if self.same_dropout_p_value is not None:
            return DropoutSpec(seed=self.seed, stream_id=stream_id, p=self.same_dropout_p_value)
        return DropoutSpec(seed=self.seed, stream_id=stream_id, p=0.0,
                           adapter_thresh16=self.adapter_thresh16,
                           adapter_inv_keep=self.adapter_inv_keep)


def prepare_multi_lora_batch_info(
    seq_len_list: Sequence[int],
    lora_idx_list: Sequence[int],
    lora_rank_list: Sequence[int],
    dropout_p_list: Sequence[float],
    alpha_list: Sequence[float],
    block_size_m: int = TILE_M,
    output_dtype: torch.dtype = torch.bfloat16,
    micro_batch_info: Any = None,
    *,
    allow_empty_micro_batch_info: bool = False,
    device: Optional[torch.device | str] = None,
    seed: int = 0,
    num_adapters: Optional[int] = None,
) -> MultiLoRABatchInfo:
    """Build the block table of one packed microbatch.

    Segment ``i`` holds ``seq_len_list[i]`` tokens of adapter ``lora_idx_list[i]`` padded up
    to a multiple of ``block_size_m`` (which must be 128, the kernels' M tile)."""
    del output_dtype  # scalars stay fp32 here
    if block_size_m != TILE_M:
        raise ValueError(f"block_size_m must be {TILE_M} for the sm_100a kernels")
    n_seg = len(seq_len_list)
    if not (len(lora_idx_list) == len(lora_rank_list) == len(dropout_p_list) == len(alpha_list) == n_seg):
        raise ValueError("per-segment lists must have the same length")
    if device is None:
        device = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
    device = torch.device(device)
    seq = np.asarray(seq_len_list, dtype=np.int64)
    padded = ((seq + block_size_m - 1) // block_size_m) * block_size_m
    padded[seq <= 0] = 0
    blocks = padded // block_size_m
    n_blk = int(blocks.sum())
    seg_of_block = np.repeat(np.arange(n_seg), blocks)
    first_block = np.concatenate([[0], np.cumsum(blocks)[:-1]]).astype(np.int64)
    idx_in_seg = np.arange(n_blk) - first_block[seg_of_block]
    valid = np.minimum(block_size_m, seq[seg_of_block] - idx_in_seg * block_size_m)

    idx_arr = np.asarray(lora_idx_list, dtype=np.int64)
    n_ad = int(num_adapters if num_adapters is not None else (max(idx_arr.max() + 1, 1) if n_seg else 1))
    ranks = np.asarray(lora_rank_list, dtype=np.int64)
    p_arr = np.asarray(dropout_p_list, dtype=np.float64)
    alpha_arr = np.asarray(alpha_list, dtype=np.float64)

    # one staging buffer: int32 words [tile_adapter | lookup (3/blk) | thresh (n_ad)]
    # followed by fp32 words [scale (n_ad) | inv_keep (n_ad) | blk_p | blk_alpha]
    n_int = n_blk + 3 * n_blk + n_ad
    n_flt = 2 * n_ad + 2 * n_blk
    stage = torch.empty(n_int + n_flt, dtype=torch.int32,
                        pin_memory=(device.type == "cuda" and torch.cuda.is_available()))
    words = stage.numpy()
    fwords = words.view(np.float32)
    words[:n_blk] = idx_arr[seg_of_block] if n_blk else 0
    lookup = words[n_blk:4 * n_blk].reshape(n_blk, 3)
    lookup[:, 0] = ranks[seg_of_block]
    lookup[:, 1] = valid
    lookup[:, 2] = first_block[seg_of_block]
    thresh = np.zeros(n_ad, dtype=np.int64)
    scale = np.zeros(n_ad, dtype=np.float32)
    inv_keep = np.ones(n_ad, dtype=np.float32)
    for i in range(n_seg):
        a = int(idx_arr[i])
        if a < 0:
            continue
        thresh[a] = dropout_threshold(float(p_arr[i]))
        scale[a] = alpha_arr[i]
        inv_keep[a] = 1.0 / (1.0 - p_arr[i]) if p_arr[i] > 0 else 1.0
    words[4 * n_blk:n_int] = thresh
    fwords[n_int:n_int + n_ad] = scale
    fwords[n_int + n_ad:n_int + 2 * n_ad] = inv_keep
    fwords[n_int + 2 * n_ad:n_int + 2 * n_ad + n_blk] = p_arr[seg_of_block] if n_blk else 0
    fwords[n_int + 2 * n_ad + n_blk:] = alpha_arr[seg_of_block] if n_blk else 0

    dev = stage.to(device, non_blocking=True)
    fdev = dev.view(torch.float32)
    segments = []
    start = 0
    for i in range(n_seg):
        if padded[i] > 0:
            segments.append((int(idx_arr[i]), start, start + int(padded[i])))
        start += int(padded[i])
    active = [float(p_arr[i]) for i in range(n_seg) if idx_arr[i] >= 0 and padded[i] > 0]
    enable_dropout = any(p > 0 for p in active)
    same = (len(set(active)) <= 1)
    info = MultiLoRABatchInfo(
        seq_len_list=[int(v) for v in seq_len_list],
        lora_idx_list=[int(v) for v in lora_idx_list],
        lora_rank_list=[int(v) for v in lora_rank_list],
        dropout_p_list=[float(v) for v in dropout_p_list],
        alpha_list=[float(v) for v in alpha_list],
        block_size_m=block_size_m,
        padded_seq_len_list=[int(v) for v in padded],
        block_to_lookup_table=dev[n_blk:4 * n_blk].view(n_blk, 3),
        block_to_dropout_p=fdev[n_int + 2 * n_ad:n_int + 2 * n_ad + n_blk],
        block_to_alpha=fdev[n_int + 2 * n_ad + n_blk:],
        enable_dropout=enable_dropout,
        same_dropout_p_value=(active[0] if (same and active) else (0.0 if not active else None)),
        max_r=int(ranks.max()) if n_seg else 0,
        micro_batch_info=micro_batch_info,
        allow_empty_micro_batch_info=allow_empty_micro_batch_info,
        tile_adapter=dev[:n_blk],
        adapter_scale=fdev[n_int:n_int + n_ad],
        adapter_thresh16=dev[4 * n_blk:n_int],
        adapter_inv_keep=fdev[n_int + n_ad:n_int + 2 * n_ad],
        segments=segments,
        segment_table=SegmentTable(segments, device, total_rows=start),
        seed=seed,
        total_padded_tokens=start,
    )
    return info


def single_adapter_batch_info(num_tokens: int, rank: int, alpha: float, dropout_p: float, *,
                              device=None, seed: int = 0) -> MultiLoRABatchInfo:
    """Block table of a batch in which every token uses adapter 0 (plain FusedLoRA)."""
    return prepare_multi_lora_batch_info([num_tokens], [0], [rank], [dropout_p], [alpha],
                                         device=device, seed=seed, num_adapters=1)
