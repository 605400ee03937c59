"""Host-side placement helpers for the step runner.

Pinned staging buffers should live on the NUMA node the GPU hangs off: with one process per GPU and
eight GPUs on two sockets, host-to-device copies from the far socket share the inter-socket link.
``bind_to_gpu_numa_node`` restricts the calling process to the CPUs of the GPU's node (pinned memory
allocated afterwards follows the first-touch policy).  Every step is best effort: on any error the
process keeps its affinity."""
from __future__ import annotations

import os
from typing import Optional

import torch


def _parse_cpulist(text: str) -> set:
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            cpus.update(range(int(a), int(b) + 1))
        else:
            cpus.add(int(part))
    return cpus


def gpu_numa_node(device_index: int) -> Optional[int]:
    try:
        p = torch.cuda.get_device_properties(device_index)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except Exception:  # noqa: BLE001
        return None


def bind_to_gpu_numa_node(device_index: int) -> Optional[int]:
    """Returns the NUMA node the process was bound to, or None when nothing was changed."""
    node = gpu_numa_node(device_index)
    if node is None or not hasattr(os, "sched_setaffinity"):
        return None
    try:
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = _parse_cpulist(f.read())
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:  # noqa: BLE001
        return None
