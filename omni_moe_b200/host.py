"""Host-side placement for the end-to-end path: run a rank's process on the CPU cores next to its GPU.

Pinned host buffers are placed on the memory node of the thread that allocates them.  With one
process per GPU and no placement, several ranks end up on one node and their host<->device copies
share that node's memory and its link to the other socket.  `bind_near_gpu` reads (never writes) the
GPU's CPU affinity from NVML and restricts the calling process to those cores, so buffers pinned
afterwards are local to the GPU's PCIe root.
"""
from __future__ import annotations

import os

import torch


def gpu_cpu_set(device_index: int) -> set[int]:
    """CPU cores NVML reports as local to CUDA device `device_index` (empty if NVML cannot tell)."""
    try:
        import pynvml
    except ImportError:
        return set()
    try:
        pynvml.nvmlInit()
        p = torch.cuda.get_device_properties(device_index)
        bus = f"{p.pci_domain_id:08x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        return {w * 64 + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1}
    except Exception:
        return set()


def bind_near_gpu(device_index: int) -> dict:
    """Restrict this process to the cores local to the GPU, within the cores it is already allowed.
    Returns what was done: {"bound": bool, "cores": count, "reason": str}."""
    if not hasattr(os, "sched_setaffinity"):
        return {"bound": False, "cores": 0, "reason": "no sched_setaffinity on this platform"}
    allowed = os.sched_getaffinity(0)
    near = gpu_cpu_set(device_index) & allowed
    if not near:
        return {"bound": False, "cores": len(allowed), "reason": "NVML reports no local cores among the allowed ones"}
    if near == allowed:
        return {"bound": False, "cores": len(allowed), "reason": "already local"}
    os.sched_setaffinity(0, near)
    return {"bound": True, "cores": len(near), "reason": "restricted to the GPU's local cores"}
