"""Build and load the native libraries (sm_100a CUDA kernels and the C++ engine core).

The libraries are plain shared objects with a C ABI, built in-tree under
``research_b200/lib`` and loaded with ``ctypes``. Nothing is JIT-compiled at import time:
``build_all()`` is the explicit build step (``python -m research_b200._native``), and
``load(name)`` fails loudly when a library is missing instead of falling back to PyTorch.
"""

from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SRC_DIR = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-shared",
    "-Xcompiler",
    "-fPIC",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-Wall"]

# library name -> (compiler, [sources])
LIBRARIES: dict[str, tuple[str, list[str]]] = {
    "rb_gemm": ("nvcc", ["gemm_sm100.cu"]),
    "rb_gemm2": ("nvcc", ["gemm2_sm100.cu"]),
    "rb_ops": ("nvcc", ["ops_sm100.cu"]),
    "rb_attn": ("nvcc", ["attn_sm100.cu"]),
    "rb_flash": ("nvcc", ["flash_sm100.cu"]),
    "rb_quant": ("nvcc", ["quant_sm100.cu"]),
    "rb_train": ("nvcc", ["train_sm100.cu"]),
    "rb_comm": ("nvcc", ["comm_sm100.cu"]),
    "rb_moe": ("nvcc", ["moe_sm100.cu"]),
    "rb_engine_core": ("g++", ["engine_core.cpp"]),
}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def lib_path(name: str) -> Path:
    return LIB_DIR / f"lib{name}.so"


def _sources_mtime(sources: list[str]) -> float:
    newest = 0.0
    for s in sources:
        p = SRC_DIR / s
        if p.exists():
            newest = max(newest, p.stat().st_mtime)
    for h in list(SRC_DIR.glob("*.h")) + list(SRC_DIR.glob("*.cuh")) + list(SRC_DIR.glob("*.hpp")):
        newest = max(newest, h.stat().st_mtime)
    return newest


def _find(tool: str) -> str | None:
    found = shutil.which(tool)
    if found:
        return found
    if tool == "nvcc" and os.path.exists("/usr/local/cuda/bin/nvcc"):
        return "/usr/local/cuda/bin/nvcc"
    return None


def build_one(name: str, force: bool = False, verbose: bool = False) -> Path | None:
    """Compile one library if it is missing or older than its sources."""
    compiler, sources = LIBRARIES[name]
    srcs = [SRC_DIR / s for s in sources]
    if not all(s.exists() for s in srcs):
        return None  # component not present in this checkout
    out = lib_path(name)
    if not force and out.exists() and out.stat().st_mtime >= _sources_mtime(sources):
        return out
    tool = _find(compiler)
    if tool is None:
        raise RuntimeError(f"{compiler} not found; cannot build {name}")
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    flags = NVCC_FLAGS if compiler == "nvcc" else CXX_FLAGS
    cmd = [tool, *flags, "-I", str(SRC_DIR), "-o", str(tmp), *[str(s) for s in srcs]]
    if compiler == "g++":
        cmd.append("-lpthread")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"building {name} failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, out)
    if verbose:
        print(f"built {out}", file=sys.stderr)
    return out


def build_all(force: bool = False, verbose: bool = False) -> list[Path]:
    """Compile every native library for sm_100a (cross-compiles without a GPU)."""
    with ThreadPoolExecutor(max_workers=min(8, len(LIBRARIES))) as ex:
        results = list(ex.map(lambda n: build_one(n, force, verbose), LIBRARIES))
    return [r for r in results if r is not None]


def load(name: str) -> ctypes.CDLL:
    """Load a built library. Raises if it is absent: there is no silent fallback."""
    with _lock:
        if name in _loaded:
            return _loaded[name]
        path = lib_path(name)
        if not path.exists():
            raise RuntimeError(
                f"native library {path} is missing; run `python -m research_b200._native` to build it"
            )
        lib = ctypes.CDLL(str(path))
        _loaded[name] = lib
        return lib


def available(name: str) -> bool:
    return lib_path(name).exists()


if __name__ == "__main__":
    built = build_all(force="--force" in sys.argv, verbose=True)
    for b in built:
        print(b)
