"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``_lf_cuda.so``  -- every CUDA kernel (``csrc/**/*.cu``), compiled for sm_100a only with
  ``nvcc -gencode arch=compute_100a,code=sm_100a``.  It exposes a plain C ABI that
  ``lorafusion_b200.ops._native`` loads through ``ctypes`` (no dependency on the torch
  headers, so a file compiles in seconds and cross-compiles on a machine without a GPU).
* ``_lf_host.so``  -- the C++ host runtime (solver / pipeline simulator cores), g++ only.

Objects are cached under ``build/`` keyed by a hash of the source, its local headers and the
flags; ``python -m lorafusion_b200.build`` rebuilds what changed.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR.parent / "build"
CUDA_LIB = PKG_DIR / "_lf_cuda.so"
HOST_LIB = PKG_DIR / "_lf_host.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build lorafusion_b200 CUDA kernels")
    return cand


def _headers() -> list[Path]:
    return sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.hpp")))


def _digest(src: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hdr in _headers():
        h.update(hdr.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _compile_one(cmd: list[str], log: Path) -> tuple[int, str]:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(proc.stdout + proc.stderr)
    return proc.returncode, proc.stdout + proc.stderr


def _build_lib(sources: list[Path], compiler: list[str], flags: list[str], out: Path,
               link_cmd: list[str], verbose: bool) -> bool:
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    jobs = []
    objs = []
    for src in sources:
        tag = _digest(src, flags)
        rel = "_".join(src.relative_to(CSRC).with_suffix("").parts)
        obj = BUILD_DIR / f"{rel}.{tag}.o"
        objs.append(obj)
        if not obj.exists():
            for stale in BUILD_DIR.glob(f"{rel}.*.o"):
                stale.unlink()
            jobs.append((src, compiler + flags + ["-c", str(src), "-o", str(obj)],
                         BUILD_DIR / f"{rel}.log"))
    changed = bool(jobs)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            results = list(pool.map(lambda j: (j[0], *_compile_one(j[1], j[2])), jobs))
        for src, rc, text in results:
            if verbose or rc != 0:
                sys.stderr.write(f"[build] {src.name}: rc={rc}\n")
            if rc != 0:
                sys.stderr.write(text)
                raise RuntimeError(f"compilation of {src} failed")
    if changed or not out.exists():
        # link next to the target and swap it in with one rename: whoever copies or loads the
        # library meanwhile sees either the old file or the new one, never a half-written one
        tmp = out.with_name(out.name + f".tmp{os.getpid()}")
        cmd = link_cmd + [str(o) for o in objs] + ["-o", str(tmp)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            tmp.unlink(missing_ok=True)
            raise RuntimeError(f"link of {out} failed")
        os.replace(tmp, out)
        changed = True
    return changed


def build_cuda(verbose: bool = False) -> Path:
    sources = sorted(CSRC.rglob("*.cu"))
    nvcc = _nvcc()
    _build_lib(sources, [nvcc], NVCC_FLAGS, CUDA_LIB,
               [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"],
               verbose)
    return CUDA_LIB


def build_host(verbose: bool = False) -> Path:
    sources = sorted(CSRC.rglob("*.cpp"))
    if not sources:
        return HOST_LIB
    gxx = shutil.which("g++") or "g++"
    _build_lib(sources, [gxx], CXX_FLAGS, HOST_LIB, [gxx, "-shared", "-pthread"], verbose)
    return HOST_LIB


def build_all(verbose: bool = False) -> None:
    build_host(verbose)
    build_cuda(verbose)


def ptxas_report() -> str:
    """Concatenate the ``-Xptxas -v`` output of the last compilation of every file."""
    out = []
    for log in sorted(BUILD_DIR.glob("*.log")):
        out.append(f"==== {log.name}\n{log.read_text()}")
    return "\n".join(out)


if __name__ == "__main__":
    build_all(verbose=True)
    print(f"built {CUDA_LIB} and {HOST_LIB}")
