"""Keep a rank's host threads (and therefore its pinned staging memory, which is placed on the node of the thread that
first touches it) on the NUMA node its GPU hangs off.

With one process per GPU and a pinned uint8 batch copied host-to-device every step, eight ranks read some tens of
GB/s from host memory; a rank whose staging buffers sit on the other socket pays the inter-socket link for every copy.
`bind_to_gpu_node` reads the GPU's PCI bus id from torch, the node from sysfs, and restricts the process to that node's
CPUs. It changes nothing that outlives the process, and does nothing when the topology cannot be read (containers
without sysfs, single-node machines, CPU runs)."""
from __future__ import annotations

import os
from typing import List, Optional


def _parse_cpulist(text: str) -> List[int]:
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-")
            cpus.extend(range(int(lo), int(hi) + 1))
        else:
            cpus.append(int(part))
    return cpus


def gpu_numa_node(device_index: int, sysfs: str = "/sys") -> Optional[int]:
    """NUMA node of a CUDA device, or None when it cannot be determined (or the machine has one node)."""
    try:
        import torch
        p = torch.cuda.get_device_properties(device_index)
        bus = f"{int(p.pci_domain_id):04x}:{int(p.pci_bus_id):02x}:{int(p.pci_device_id):02x}.0"     # 0000:1b:00.0
    except (AttributeError, RuntimeError, AssertionError, TypeError, ValueError):
        return None
    return numa_node_of_bus(str(bus), sysfs)


def numa_node_of_bus(bus: str, sysfs: str = "/sys") -> Optional[int]:
    path = os.path.join(sysfs, "bus", "pci", "devices", bus.lower(), "numa_node")
    try:
        with open(path) as f:
            node = int(f.read().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def node_cpus(node: int, sysfs: str = "/sys") -> List[int]:
    try:
        with open(os.path.join(sysfs, "devices", "system", "node", f"node{node}", "cpulist")) as f:
            return _parse_cpulist(f.read())
    except (OSError, ValueError):
        return []


def bind_to_gpu_node(device_index: int, sysfs: str = "/sys") -> Optional[int]:
    """Restrict this process to the CPUs of the GPU's NUMA node; returns the node, or None if nothing was changed."""
    node = gpu_numa_node(device_index, sysfs)
    if node is None:
        return None
    cpus = set(node_cpus(node, sysfs))
    try:
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
    except (AttributeError, OSError):
        return None
    return node
