"""Small shared helpers: seeding, dtype names, distributed bring-up, device names, memory."""

from __future__ import annotations

import os
import random
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16, "fp16": torch.float16,
          "float32": torch.float32, "fp32": torch.float32}


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def str_to_dtype(name: str) -> torch.dtype:
    return DTYPES[name.lower()]


def maybe_setup_distributed(backend: str | None = None) -> tuple:
    """Initialise ``torch.distributed`` from the torchrun environment; returns
    ``(rank, local_rank, world_size)``.  Rendezvous always uses 127.0.0.1 on one node."""
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
            dist.init_process_group(backend, device_id=torch.device("cuda", local_rank))
        else:
            dist.init_process_group(backend)
    return rank, local_rank, world


def get_device_short_name() -> str:
    if not torch.cuda.is_available():
        return "cpu"
    return torch.cuda.get_device_name().lower().replace("nvidia ", "").replace(" ", "-")


def peak_memory_gib(device=None, reset: bool = False) -> float:
    if not torch.cuda.is_available():
        return 0.0
    v = torch.cuda.max_memory_allocated(device) / 2**30
    if reset:
        torch.cuda.reset_peak_memory_stats(device)
    return v


def list_of_ints(text) -> list:
    return [int(v) for v in str(text).replace(",", " ").split()]


def list_of_floats(text) -> list:
    return [float(v) for v in str(text).replace(",", " ").split()]


def create_packed_dummy_inputs(hidden_size: int, seq_len_list, multiple_of: Optional[int] = None,
                               dtype: torch.dtype = torch.bfloat16, device=None, *, return_input_ids: bool = True,
                               return_inputs_embeds: bool = False, return_labels: bool = False,
                               seed: Optional[int] = None) -> dict:
    """Random inputs of one packed microbatch, in the layout a varlen attention call expects:
    ``input_ids`` / ``labels`` ``[1, T]`` (ids below 10000), ``position_ids`` ``[1, T]`` restarting
    at every sequence, ``cu_seq_lens_q`` / ``cu_seq_lens_k`` (int32, length ``n + 1``) and
    ``max_length_q`` / ``max_length_k``.  With ``multiple_of`` the total is padded up and the
    padding forms one more sequence.  Same keys as the reference's helper of the same name
    (``lorafusion/utils/hf.py:6-121``), used by its layer and kernel benchmarks."""
    if not isinstance(seq_len_list, (list, tuple)) or not seq_len_list:
        raise ValueError(f"seq_len_list must be a non-empty list, got {seq_len_list!r}")
    lens = [int(v) for v in seq_len_list]
    total = sum(lens)
    if multiple_of:
        pad = (-total) % int(multiple_of)
        if pad:
            lens.append(pad)
            total += pad
    device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    gen = torch.Generator(device="cpu")
    if seed is not None:
        gen.manual_seed(int(seed))
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens, dtype=torch.int32).cumsum(0)
    out = {
        "position_ids": torch.cat([torch.arange(n, dtype=torch.long) for n in lens]).unsqueeze(0).to(device),
        "cu_seq_lens_q": cu.to(device),
        "cu_seq_lens_k": cu.to(device),
        "max_length_q": max(lens),
        "max_length_k": max(lens),
    }
    if return_input_ids:
        out["input_ids"] = torch.randint(0, 10000, (1, total), generator=gen).to(device)
    if return_inputs_embeds:
        out["inputs_embeds"] = torch.randn(1, total, hidden_size, generator=gen).to(dtype).to(device)
    if return_labels:
        out["labels"] = torch.randint(0, 10000, (1, total), generator=gen).to(device)
    return out
