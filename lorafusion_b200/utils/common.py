"""Small shared helpers: seeding, dtype names, distributed bring-up, device names, memory."""

from __future__ import annotations

import os
import random

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
