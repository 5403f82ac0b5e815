"""ctypes bridge to the in-tree native libraries.

``cuda_lib()`` returns the handle of ``_lf_cuda.so`` (all sm_100a kernels) and
``host_lib()`` the handle of ``_lf_host.so`` (C++ solver / simulator cores).  Loading fails
loudly: on a machine with a GPU a missing or unloadable kernel library is an error, never a
silent fallback to eager PyTorch.
"""

from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent
_LOCK = threading.Lock()
_CUDA = None
_HOST = None


class NativeLibraryError(RuntimeError):
    pass


def _load(path: Path, builder: str) -> C.CDLL:
    if not path.exists():
        if os.environ.get("LORAFUSION_B200_NO_AUTOBUILD", "0") == "1":
            raise NativeLibraryError(f"{path} is missing and auto-build is disabled")
        from lorafusion_b200 import build as _build

        getattr(_build, builder)()
    try:
        return C.CDLL(str(path))
    except OSError as exc:  # pragma: no cover - depends on the machine
        raise NativeLibraryError(f"cannot load {path}: {exc}") from exc


def cuda_lib() -> C.CDLL:
    global _CUDA
    with _LOCK:
        if _CUDA is None:
            _CUDA = _load(_PKG / "_lf_cuda.so", "build_cuda")
            _declare_cuda(_CUDA)
        return _CUDA


def host_lib() -> C.CDLL:
    global _HOST
    with _LOCK:
        if _HOST is None:
            _HOST = _load(_PKG / "_lf_host.so", "build_host")
        return _HOST


def cuda_available() -> bool:
    return torch.cuda.is_available()


# ----------------------------------------------------------------------------------------
# struct mirrors (keep in sync with csrc/gemm/gemm_api.h)
# ----------------------------------------------------------------------------------------
class LfNf4Args(C.Structure):
    _fields_ = [("block_scales", C.c_void_p), ("w_rows", C.c_int64), ("w_cols", C.c_int64)]


class LfGemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("a_rows", C.c_int64), ("a_cols", C.c_int64), ("a_ld", C.c_int64),
        ("b", C.c_void_p), ("b_rows", C.c_int64), ("b_cols", C.c_int64), ("b_ld", C.c_int64),
        ("a2", C.c_void_p), ("a2_rows", C.c_int64), ("a2_cols", C.c_int64), ("a2_ld", C.c_int64),
        ("b2", C.c_void_p), ("b2_rows", C.c_int64), ("b2_cols", C.c_int64), ("b2_ld", C.c_int64),
        ("tile_adapter", C.c_void_p),
        ("seg_tiles", C.c_void_p),
        ("out", C.c_void_p),
        ("ldo", C.c_int64),
        ("out_adapter_stride", C.c_int64),
        ("adapter_scale", C.c_void_p),
        ("bias", C.c_void_p),
        ("adapter_thresh16", C.c_void_p),
        ("adapter_inv_keep", C.c_void_p),
        ("err", C.c_void_p),
        ("stream", C.c_void_p),
        ("a_mn", C.c_int32), ("b_mn", C.c_int32), ("b2_mn", C.c_int32),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("K2", C.c_int32),
        ("bn", C.c_int32), ("nacc", C.c_int32), ("epi", C.c_int32), ("mask_a", C.c_int32),
        ("b_adapter_rows", C.c_int32), ("b2_adapter_rows", C.c_int32),
        ("num_seg_tiles", C.c_int32),
        ("out_transposed", C.c_int32),
        ("scale", C.c_float),
        ("inv_keep", C.c_float),
        ("thresh16", C.c_uint32),
        ("seed_lo", C.c_uint32), ("seed_hi", C.c_uint32), ("stream_id", C.c_uint32),
        ("row_offset", C.c_int32), ("col_offset", C.c_int32),
        ("group_m", C.c_int32), ("max_ctas", C.c_int32),
    ]


EPI_BF16 = 0
EPI_BF16_DROPMIX = 1
EPI_F32_ACCUM = 2
EPI_BF16_ADAPTER_SCALE = 3


_VP, _LL, _I, _F = C.c_void_p, C.c_longlong, C.c_int, C.c_float

_SIGNATURES = {
    "lf_rmsnorm_fwd": [_VP, _VP, _VP, _VP, _VP, _VP, _LL, _I, _F, _VP],
    "lf_rmsnorm_bwd": [_VP, _VP, _VP, _VP, _VP, _VP, _LL, _I, _VP],
    "lf_rope_inplace": [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _VP],
    "lf_swiglu_fwd": [_VP, _VP, _LL, _I, _VP],
    "lf_swiglu_bwd": [_VP, _VP, _VP, _LL, _I, _VP],
    "lf_embedding": [_VP, _VP, _VP, _LL, _I, _I, _VP],
    "lf_add": [_VP, _VP, _VP, _LL, _VP],
    "lf_cross_entropy": [_VP, _VP, _VP, _LL, _I, _LL, _F, _VP],
    "lf_adam_chunks": [_VP, _VP, _I, _VP, _VP, _VP, _VP, _VP, _F, _F, _F, _F, _F, _I, _F, _VP],
    "lf_nf4_quantize": [_VP, _VP, _VP, _LL, _VP],
    "lf_nf4_dequantize": [_VP, _VP, _VP, _VP, _VP, _F, _VP, _LL, _VP],
    "lf_attn_fwd": [_VP, _LL, _LL, _I, _I, _I, _I, _I, _VP, _I, _VP, _LL, _VP, _F, _VP, _VP],
    "lf_attn_bwd": [_VP, _VP, _VP, _VP, _LL, _LL, _I, _I, _I, _I, _I, _VP, _I, _LL, _VP, _VP,
                    _F, _VP, _VP],
}


def _declare_cuda(lib: C.CDLL) -> None:
    lib.lf_gemm.argtypes = [C.POINTER(LfGemmArgs)]
    lib.lf_gemm.restype = C.c_int
    lib.lf_gemm_pair.argtypes = [C.POINTER(LfGemmArgs)]
    lib.lf_gemm_pair.restype = C.c_int
    lib.lf_gemm_nf4.argtypes = [C.POINTER(LfGemmArgs), C.POINTER(LfNf4Args)]
    lib.lf_gemm_nf4.restype = C.c_int
    for name, sig in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = sig
        fn.restype = C.c_int


# kernels launched per C entry point (for launch accounting in benchmarks)
_LAUNCHES_PER_CALL = {"lf_attn_bwd": 3}
_LAUNCHES = 0


def launch_count() -> int:
    """Number of kernels of this library launched so far by this process."""
    return _LAUNCHES


def note_launch(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def call(name: str, *args) -> None:
    """Call an ``int``-returning C entry point and raise on a non-zero status."""
    global _LAUNCHES
    _LAUNCHES += _LAUNCHES_PER_CALL.get(name, 1)
    rc = getattr(cuda_lib(), name)(*args)
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")


# ----------------------------------------------------------------------------------------
# device error word: kernels record bounded-wait timeouts here instead of hanging
# ----------------------------------------------------------------------------------------
_ERR_WORDS: dict[int, torch.Tensor] = {}

ERR_NAMES = {
    0: "ok",
    1: "timeout waiting for a TMA stage",
    2: "timeout waiting for a free pipeline stage",
    3: "timeout waiting for a TMEM accumulator",
    4: "timeout waiting for a drained TMEM accumulator",
    5: "timeout waiting for a transformed stage",
    6: "timeout waiting for a peer flag",
    7: "bad kernel argument",
    8: "timeout (misc)",
}


def err_word(device: torch.device | int | None = None) -> torch.Tensor:
    dev = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    t = _ERR_WORDS.get(dev)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
        _ERR_WORDS[dev] = t
    return t


def check_device_errors(device=None, *, reset: bool = True) -> None:
    """Synchronise and raise if any kernel recorded a bounded-wait failure."""
    t = err_word(device)
    code = int(t.item())
    if code != 0:
        if reset:
            t.zero_()
        raise RuntimeError(f"lorafusion_b200 kernel error {code}: {ERR_NAMES.get(code, '?')}")


def current_stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream
