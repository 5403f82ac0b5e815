"""Rank-aware logging helpers (loguru when available, stdlib logging otherwise); the
counterpart of the ``log_rank0`` / rank-prefixed helpers in ``lorafusion/utils/common.py:190-241``."""

from __future__ import annotations

import logging
import os
import sys

_RANK = int(os.environ.get("RANK", "0"))

try:  # pragma: no cover - depends on the environment
    from loguru import logger as _logger

    _HAVE_LOGURU = True
except ImportError:  # pragma: no cover
    _logger = logging.getLogger("lorafusion_b200")
    _HAVE_LOGURU = False


def setup_logging(rank: int | None = None, level: str = "INFO") -> None:
    global _RANK
    _RANK = int(os.environ.get("RANK", "0")) if rank is None else rank
    if _HAVE_LOGURU:
        _logger.remove()
        _logger.add(sys.stderr, level=level, format=f"<green>{{time:HH:mm:ss}}</green> [rank {_RANK}] {{message}}")
    else:
        logging.basicConfig(level=getattr(logging, level), format=f"%(asctime)s [rank {_RANK}] %(message)s")


def log_rank0(msg: str) -> None:
    if _RANK == 0:
        _logger.info(msg)


def log_all_ranks(msg: str) -> None:
    _logger.info(msg)


def warn_rank0(msg: str) -> None:
    if _RANK == 0:
        _logger.warning(msg)
