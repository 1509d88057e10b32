"""NUMA placement of the host-pinned KV pools.

A pool that a GPU streams over PCIe should live in the memory of the CPU socket that GPU hangs off: pages on
the other socket cross the inter-socket link first, and with all GPUs of a box streaming at once that link, not
PCIe, becomes the ceiling.  ``cudaHostAlloc`` places pages by the calling thread's memory policy, so
:func:`local_to_gpu` sets a preferred node (``set_mempolicy``) and, where the process is allowed those CPUs, the
thread's affinity for the duration of the allocation, and puts both back afterwards.  Everything here is
per-process state of the calling process; where the kernel, the container or the machine does not allow or need
it (one node, no permission, no sysfs) the context manager does nothing.
"""

from __future__ import annotations

import contextlib
import ctypes
import os
from typing import List, Optional

_SYS_NODE = "/sys/devices/system/node"
_SYS_PCI = "/sys/bus/pci/devices"
_MPOL_DEFAULT, _MPOL_PREFERRED = 0, 1
_SYS_SET_MEMPOLICY = {"x86_64": 238, "aarch64": 237}


def _read(path: str) -> Optional[str]:
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return None


def parse_cpulist(text: str) -> List[int]:
    """``"0-3,8,10-11"`` -> ``[0, 1, 2, 3, 8, 10, 11]``."""
    cpus: List[int] = []
    for part in text.split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-", 1)
            cpus.extend(range(int(lo), int(hi) + 1))
        else:
            cpus.append(int(part))
    return cpus


def node_count(sys_node: str = _SYS_NODE) -> int:
    try:
        return sum(1 for d in os.listdir(sys_node) if d.startswith("node") and d[4:].isdigit())
    except OSError:
        return 0


def node_cpus(node: int, sys_node: str = _SYS_NODE) -> List[int]:
    text = _read(os.path.join(sys_node, f"node{node}", "cpulist"))
    return parse_cpulist(text) if text else []


def gpu_pci_bus_id(device_index: int) -> Optional[str]:
    """``0000:1b:00.0`` of a CUDA device, lower case as sysfs spells it."""
    try:
        import torch

        p = torch.cuda.get_device_properties(device_index)
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except Exception:
        return None


def gpu_numa_node(device_index: int, sys_pci: str = _SYS_PCI) -> Optional[int]:
    """NUMA node the GPU's PCIe root belongs to, or ``None`` when unknown (sysfs reports -1 on one-node machines)."""
    bus = gpu_pci_bus_id(device_index)
    if bus is None:
        return None
    text = _read(os.path.join(sys_pci, bus, "numa_node"))
    try:
        node = int(text) if text is not None else -1
    except ValueError:
        node = -1
    return node if node >= 0 else None


def set_preferred_node(node: Optional[int]) -> bool:
    """``set_mempolicy(MPOL_PREFERRED, {node})`` for the calling thread (``None``: back to the default policy).
    Returns whether the kernel accepted it."""
    nr = _SYS_SET_MEMPOLICY.get(os.uname().machine)
    if nr is None:
        return False
    try:
        libc = ctypes.CDLL(None, use_errno=True)
    except OSError:
        return False
    if node is None:
        rc = libc.syscall(ctypes.c_long(nr), ctypes.c_int(_MPOL_DEFAULT), ctypes.c_void_p(None), ctypes.c_ulong(0))
        return rc == 0
    words = node // 64 + 1
    mask = (ctypes.c_ulong * words)()
    mask[node // 64] = 1 << (node % 64)
    rc = libc.syscall(ctypes.c_long(nr), ctypes.c_int(_MPOL_PREFERRED), mask, ctypes.c_ulong(words * 64 + 1))
    return rc == 0


@contextlib.contextmanager
def local_to_gpu(device_index: Optional[int], sys_node: str = _SYS_NODE, sys_pci: str = _SYS_PCI):
    """Allocations made inside the block prefer the memory of the GPU's socket.  Yields the node, or ``None`` when
    nothing was changed."""
    node = None
    if device_index is not None and node_count(sys_node) > 1:
        node = gpu_numa_node(device_index, sys_pci)
    if node is None:
        yield None
        return
    old_affinity = None
    policy_set = set_preferred_node(node)
    try:
        allowed = os.sched_getaffinity(0)
        local = allowed & set(node_cpus(node, sys_node))
        if local and local != allowed:
            old_affinity = allowed
            os.sched_setaffinity(0, local)      # first touch happens on the GPU's socket as well
    except (AttributeError, OSError):
        old_affinity = None
    try:
        yield node if (policy_set or old_affinity is not None) else None
    finally:
        if old_affinity is not None:
            try:
                os.sched_setaffinity(0, old_affinity)
            except OSError:
                pass
        if policy_set:
            set_preferred_node(None)
