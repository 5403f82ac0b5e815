"""Launch-parameter registry of the tcgen05 GEMM family: what the tuner writes, the launchers read.

Counterpart of the reference's per-GPU tile table and its accessor
(``lorafusion/ops/triton_ops/config.py:14-152``: ``LoRATritonConfig`` per kernel and GPU,
``get_lora_kernel_config(name)``; ``tools/tune_kernels.py:442-484`` prints what to paste into
it).  Here the table is a JSON file, one per GPU model, that ``python -m
lorafusion_b200.cli.tune`` writes and :func:`get_kernel_config` serves -- no source edit is
needed after tuning, and an unknown GPU or shape falls back to built-in defaults instead of
raising.

Key: ``(kernel, M bucket, K, N)``.  ``kernel`` is one of ``fwd`` (base + LoRA slab),
``dx`` (input gradient without dropout), ``dx_dropout`` (input gradient with the mask
regenerated in the epilogue); the M bucket is the token count rounded up to a power of two.
Value: ``group_m`` (how many M tiles share a weight tile in L2 before the next N tile starts),
``max_ctas`` (0 = one persistent CTA per SM) and, for kernels that have a choice, ``bn``.

File search order: ``LORAFUSION_B200_TUNING`` (a path), then
``lorafusion_b200/ops/tuned/<gpu name>.json``.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Optional

import torch

TUNED_DIR = Path(__file__).resolve().parent / "tuned"
KERNELS = ("fwd", "dx", "dx_dropout")


@dataclass(frozen=True)
class KernelConfig:
    group_m: int = 8
    max_ctas: int = 0
    bn: Optional[int] = None     # None = the launcher's own choice for the shape
    source: str = "default"


DEFAULTS = {k: KernelConfig() for k in KERNELS}

_table: Optional[dict] = None
_table_path: Optional[str] = None


def gpu_key(device=None) -> str:
    """Lower-case device name with spaces turned into dashes (``nvidia-b200``); ``cpu`` when no
    GPU is present."""
    if not torch.cuda.is_available():
        return "cpu"
    return torch.cuda.get_device_name(device).lower().replace(" ", "-")


def m_bucket(m: int) -> int:
    return 1 << max(0, int(m - 1).bit_length())


def entry_key(kernel: str, m: int, k: int, n: int) -> str:
    return f"{kernel}:{m_bucket(m)}:{k}:{n}"


def _load() -> dict:
    global _table, _table_path
    if _table is not None:
        return _table
    path = os.environ.get("LORAFUSION_B200_TUNING")
    cand = Path(path) if path else TUNED_DIR / f"{gpu_key()}.json"
    _table, _table_path = {}, None
    if cand.exists():
        try:
            data = json.loads(cand.read_text())
            if not path and data.get("gpu") not in (None, gpu_key()):
                return _table
            _table = {k: KernelConfig(group_m=int(v.get("group_m", 8)), max_ctas=int(v.get("max_ctas", 0)),
                                      bn=v.get("bn"), source=str(cand))
                      for k, v in data.get("entries", {}).items()}
            _table_path = str(cand)
        except (OSError, ValueError, AttributeError):
            _table = {}
    return _table


def reload() -> None:
    """Forget the cached table (tests, or after the tuner wrote a new file)."""
    global _table
    _table = None


def get_kernel_config(kernel: str, m: int, k: int, n: int) -> KernelConfig:
    """Tuned launch parameters for ``kernel`` on an ``m x k x n`` problem, or the defaults."""
    if kernel not in DEFAULTS:
        raise KeyError(f"unknown kernel {kernel!r}; known: {KERNELS}")
    return _load().get(entry_key(kernel, m, k, n), DEFAULTS[kernel])


def write_table(entries: dict, path: Optional[str | Path] = None, gpu: Optional[str] = None) -> Path:
    """Write ``{entry_key: {"group_m", "max_ctas", "bn", ...}}`` as the table of ``gpu``
    (default: the current one), merged over what the file already holds."""
    gpu = gpu or gpu_key()
    out = Path(path) if path else TUNED_DIR / f"{gpu}.json"
    old = {}
    if out.exists():
        try:
            old = json.loads(out.read_text()).get("entries", {})
        except (OSError, ValueError):
            old = {}
    old.update({k: (asdict(v) if isinstance(v, KernelConfig) else dict(v)) for k, v in entries.items()})
    out.parent.mkdir(parents=True, exist_ok=True)
    out.write_text(json.dumps({"gpu": gpu, "entries": old}, indent=1, sort_keys=True))
    reload()
    return out
