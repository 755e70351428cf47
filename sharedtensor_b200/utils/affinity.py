"""Keeps a process's host threads and its pinned staging buffers on the CPU socket next to its GPU.

On a two-socket 8-GPU host a pinned buffer that was first touched on the far socket is copied to the GPU through
the socket interconnect; with one process per GPU all copying at once that, not PCIe, bounds the host->device
rate.  Binding the process to the CPUs NVML reports as local to the GPU (before the buffers are allocated) avoids
it.  This changes the calling process's CPU affinity only; nothing on the GPU is touched.
"""
from __future__ import annotations

import os


def local_cpus(device_index: int) -> list[int]:
    """CPUs local to the GPU according to NVML (empty if NVML or the query is not available)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = [w * 64 + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1]
        return cpus
    except Exception:
        return []


def bind_to_gpu(device_index: int) -> list[int]:
    """Restricts this process to the intersection of its current CPU set and the GPU's local CPUs; returns the new
    set (or the unchanged one if there is nothing to intersect with)."""
    try:
        allowed = os.sched_getaffinity(0)
    except AttributeError:
        return []
    want = allowed & set(local_cpus(device_index))
    if want and want != allowed:
        try:
            os.sched_setaffinity(0, want)
            return sorted(want)
        except OSError:
            pass
    return sorted(allowed)
