"""Pinned host memory allocated on the NUMA node the GPU hangs off.

A host<->device copy whose pinned buffer lives on the other socket crosses the inter-socket
link before it reaches the GPU's PCIe root port; with several GPUs copying at once that link
is what saturates.  `pinned_near(device, ...)` asks the kernel to prefer the GPU's own node
(`set_mempolicy(MPOL_PREFERRED)`, a per-thread policy of this process) while PyTorch allocates
and pins the buffer, then restores the default policy.  Everything is best effort: without
sysfs, on a single-node host, or where the policy call is refused, it is a plain pinned
allocation.  Nothing about the GPU is changed.
"""

from __future__ import annotations

import ctypes
import os
import platform
from contextlib import contextmanager

import torch

_MPOL_DEFAULT, _MPOL_PREFERRED = 0, 1
_SYS_SET_MEMPOLICY = {"x86_64": 238, "aarch64": 237}.get(platform.machine())


def numa_node_of(device: torch.device | int) -> int | None:
    """The NUMA node of a CUDA device's PCI function, or None if the host does not say."""
    try:
        index = device if isinstance(device, int) else (device.index if device.index is not None
                                                        else torch.cuda.current_device())
        props = torch.cuda.get_device_properties(index)
        bus_id = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus_id}/numa_node") as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


def _set_mempolicy(mode: int, node: int | None) -> bool:
    if _SYS_SET_MEMPOLICY is None:
        return False
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        if node is None:
            return libc.syscall(_SYS_SET_MEMPOLICY, mode, None, 0) == 0
        words = node // 64 + 1
        mask = (ctypes.c_ulong * words)()
        mask[node // 64] = 1 << (node % 64)
        return libc.syscall(_SYS_SET_MEMPOLICY, mode, mask, words * 64 + 1) == 0
    except (OSError, AttributeError):
        return False


@contextmanager
def prefer_node_of(device: torch.device | int):
    """Inside the block, this thread's new pages come from the device's NUMA node if possible.
    Yields the node number in force, or None when nothing was changed."""
    node = numa_node_of(device)
    applied = node is not None and _set_mempolicy(_MPOL_PREFERRED, node)
    try:
        yield node if applied else None
    finally:
        if applied:
            _set_mempolicy(_MPOL_DEFAULT, None)


def pinned_near(device: torch.device | int, shape, dtype=torch.float32) -> torch.Tensor:
    """An uninitialised pinned host tensor, on the device's NUMA node when the host allows it."""
    with prefer_node_of(device):
        out = torch.empty(shape, dtype=dtype, pin_memory=True)
        # pages of a fresh pinned allocation are resident already; touching them is not needed
    return out


_WRITE_COMBINED = 0x04   # cudaHostAllocWriteCombined
_wc_keepalive: list = []


def pinned_write_combined(device: torch.device | int, shape, dtype=torch.float32) -> torch.Tensor:
    """A pinned host tensor in write-combined memory (`cudaHostAlloc(..., cudaHostAllocWriteCombined)`
    of the CUDA runtime PyTorch has loaded): the device reads it over PCIe without snooping the
    CPU caches, the host should only ever WRITE it (host reads are uncached and slow).  For
    staging buffers that the host fills and the GPU consumes.  The allocation lives until the
    process exits."""
    import math

    n_bytes = max(1, math.prod(shape) * torch.empty((), dtype=dtype).element_size())
    runtime = ctypes.CDLL("libcudart.so.12")
    runtime.cudaHostAlloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t, ctypes.c_uint]
    runtime.cudaHostAlloc.restype = ctypes.c_int
    ptr = ctypes.c_void_p()
    with torch.cuda.device(device), prefer_node_of(device):
        status = runtime.cudaHostAlloc(ctypes.byref(ptr), n_bytes, _WRITE_COMBINED)
    if status != 0 or not ptr.value:
        raise RuntimeError(f"cudaHostAlloc(write-combined, {n_bytes} bytes) failed with status {status}")
    raw = (ctypes.c_char * n_bytes).from_address(ptr.value)
    _wc_keepalive.append(raw)
    return torch.frombuffer(raw, dtype=dtype, count=math.prod(shape)).reshape(shape)


def describe(device: torch.device | int) -> dict:
    """What the host says about placement (for benchmark records)."""
    nodes = None
    try:
        nodes = len([d for d in os.listdir("/sys/devices/system/node") if d.startswith("node")])
    except OSError:
        pass
    return {"gpu_numa_node": numa_node_of(device), "host_numa_nodes": nodes,
            "cpus_allowed": len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else None}
