"""Pin a process to the CPUs closest to its GPU (miniray/gpu_affinity.py:12-110).

Reads the topology through NVML; never changes a GPU setting. ``nvml`` can be injected (tests
use a fake), otherwise ``pynvml`` is imported lazily and absence is tolerated."""

from __future__ import annotations

import os


def _load_nvml(nvml=None):
    if nvml is not None:
        return nvml
    try:
        import pynvml  # provided by nvidia-ml-py

        return pynvml
    except ImportError:
        return None


def get_gpu_cpu_set(gpu_index: int, nvml=None) -> list[int] | None:
    """CPU ids NVML reports as local to the GPU, or None when unavailable."""
    nv = _load_nvml(nvml)
    if nv is None:
        return None
    try:
        nv.nvmlInit()
        handle = nv.nvmlDeviceGetHandleByIndex(gpu_index)
        n_cpu = os.cpu_count() or 1
        words = nv.nvmlDeviceGetCpuAffinity(handle, (n_cpu + 63) // 64)
        cpus = [w * 64 + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1]
        return [c for c in cpus if c < n_cpu] or None
    except Exception:
        return None
    finally:
        try:
            nv.nvmlShutdown()
        except Exception:
            pass


def set_gpu_affinity(gpu_index: int, nvml=None) -> list[int] | None:
    """Bind the calling process to the GPU-local CPUs; returns the CPU list applied (or None)."""
    cpus = get_gpu_cpu_set(gpu_index, nvml)
    if not cpus:
        return None
    try:
        os.sched_setaffinity(0, set(cpus) & set(os.sched_getaffinity(0)) or set(cpus))
    except (OSError, AttributeError):
        return None
    return cpus


def get_gpu_numa_node(gpu_index: int) -> int | None:
    """NUMA node of the GPU from sysfs (None when it cannot be determined)."""
    try:
        import glob

        for path in sorted(glob.glob("/sys/bus/pci/drivers/nvidia/*/numa_node")):
            idx = sorted(glob.glob("/sys/bus/pci/drivers/nvidia/*/numa_node")).index(path)
            if idx == gpu_index:
                v = int(open(path).read().strip())
                return v if v >= 0 else None
    except Exception:
        return None
    return None
