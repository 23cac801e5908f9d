"""Bind a trainer process to the NUMA node of its GPU (CPU affinity and memory policy), without ``numactl``.

The reference re-executes each trainer under ``numactl --cpunodebind --membind`` when ``BIND_TRAINER_NUMA=1`` and maps
local ranks 0-3 to two nodes by hand (paddleformers/cli/launcher.py:22-69). Here the node is read from the machine: the
GPU's PCI address -> ``/sys/bus/pci/devices/<address>/numa_node`` -> that node's CPU list; the process pins itself with
``sched_setaffinity`` and asks for node-local memory with the ``set_mempolicy`` system call (preferred, not strict, so an
exhausted node does not kill the job). Pinned host buffers (input pipeline, checkpoint snapshots) then live next to the
GPU that reads them. Everything degrades to a logged no-op when the information is not there (containers often hide it).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

SYSFS_PCI = "/sys/bus/pci/devices"
SYSFS_NODE = "/sys/devices/system/node"
_MPOL_PREFERRED = 1
_SYS_SET_MEMPOLICY = {"x86_64": 238, "aarch64": 237}


def parse_cpulist(text: str) -> List[int]:
    """``"0-3,8,10-11"`` -> [0, 1, 2, 3, 8, 10, 11]."""
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-", 1)
            cpus.extend(range(int(lo), int(hi) + 1))
        else:
            cpus.append(int(part))
    return cpus


def gpu_pci_address(index: int) -> Optional[str]:
    """PCI address of CUDA device ``index`` as sysfs spells it (``0000:1b:00.0``), or None."""
    try:
        import torch

        p = torch.cuda.get_device_properties(index)
        dom, bus, dev = getattr(p, "pci_domain_id", None), getattr(p, "pci_bus_id", None), getattr(p, "pci_device_id", None)
        if bus is not None and dev is not None:
            return f"{int(dom or 0):04x}:{int(bus):02x}:{int(dev):02x}.0"
    except Exception:  # noqa: BLE001
        pass
    try:
        import pynvml

        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
        bus_id = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(phys)).busId
        bus_id = bus_id.decode() if isinstance(bus_id, bytes) else bus_id
        return bus_id.lower()[-12:]          # NVML prints an 8-digit domain; sysfs uses 4
    except Exception:  # noqa: BLE001
        return None


def numa_node_of_pci(address: str, sysfs_pci: str = SYSFS_PCI) -> Optional[int]:
    try:
        with open(os.path.join(sysfs_pci, address, "numa_node")) as f:
            node = int(f.read().strip())
        return node if node >= 0 else None       # -1: the platform does not say
    except (OSError, ValueError):
        return None


def cpus_of_node(node: int, sysfs_node: str = SYSFS_NODE) -> List[int]:
    try:
        with open(os.path.join(sysfs_node, f"node{node}", "cpulist")) as f:
            return parse_cpulist(f.read())
    except OSError:
        return []


def prefer_node_memory(node: int) -> bool:
    """``set_mempolicy(MPOL_PREFERRED, {node})`` for this process; False when the call is not available or refused."""
    nr = _SYS_SET_MEMPOLICY.get(os.uname().machine)
    if nr is None or node < 0 or node >= 1024:
        return False
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        words = node // 64 + 1
        mask = (ctypes.c_ulong * words)()
        mask[node // 64] = 1 << (node % 64)
        rc = libc.syscall(ctypes.c_long(nr), ctypes.c_int(_MPOL_PREFERRED), ctypes.byref(mask), ctypes.c_ulong(words * 64 + 1))
        return rc == 0
    except Exception:  # noqa: BLE001
        return False


def bind_to_gpu_node(local_rank: int, sysfs_pci: str = SYSFS_PCI, sysfs_node: str = SYSFS_NODE, set_memory: bool = True) -> dict:
    """Pin the calling process to the CPUs (and memory) of the NUMA node next to GPU ``local_rank``. Returns what was done:
    {"node": int | None, "cpus": int, "memory": bool, "reason": str}."""
    addr = gpu_pci_address(local_rank)
    if addr is None:
        return {"node": None, "cpus": 0, "memory": False, "reason": "no PCI address for the GPU"}
    node = numa_node_of_pci(addr, sysfs_pci)
    if node is None:
        return {"node": None, "cpus": 0, "memory": False, "reason": f"no numa_node for {addr}"}
    cpus = cpus_of_node(node, sysfs_node)
    allowed = set(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else set()
    target = sorted(set(cpus) & allowed) if allowed else cpus
    if not target:
        return {"node": node, "cpus": 0, "memory": False, "reason": "none of the node's CPUs is available to this process"}
    os.sched_setaffinity(0, target)
    mem = prefer_node_memory(node) if set_memory else False
    return {"node": node, "cpus": len(target), "memory": mem, "reason": "ok"}


def maybe_bind_trainer() -> Optional[dict]:
    """The hook the trainer entry points call: acts when ``BIND_TRAINER_NUMA`` is 1 / true / on / yes."""
    if os.environ.get("BIND_TRAINER_NUMA", "0").lower() not in ("1", "true", "on", "yes"):
        return None
    from .log import logger

    res = bind_to_gpu_node(int(os.environ.get("LOCAL_RANK", "0")))
    logger.info(f"trainer NUMA affinity: local_rank={os.environ.get('LOCAL_RANK', '0')} node={res['node']} cpus={res['cpus']} "
                f"memory_policy={'preferred' if res['memory'] else 'unchanged'} ({res['reason']})")
    return res
