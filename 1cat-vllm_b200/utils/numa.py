"""CPU placement of a worker process next to its GPU: the cores of the NUMA node the GPU's PCIe function hangs off
(reference: vllm/utils/numa_utils.py; v1/executor/multiproc_executor.py:686-690,817-818).

Off by default (``ONECAT_NUMA_BIND=1`` turns it on): a host may already pin its containers, and a wrong mask costs more than none."""
from __future__ import annotations

import os
from typing import Optional

from onecat_vllm.logger import init_logger

log = init_logger(__name__)


def parse_cpulist(text: str) -> list[int]:
    """``"0-3,8,10-11"`` -> [0, 1, 2, 3, 8, 10, 11]."""
    cpus: list[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.extend(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_local_cpus(pci_domain: int, pci_bus: int, pci_device: int, sysfs_root: str = "/sys") -> Optional[list[int]]:
    """Cores local to a PCIe function, from ``local_cpulist`` (or the cpulist of its ``numa_node``); None when the host does not say."""
    dev = os.path.join(sysfs_root, "bus", "pci", "devices", f"{pci_domain:04x}:{pci_bus:02x}:{pci_device:02x}.0")
    try:
        with open(os.path.join(dev, "local_cpulist")) as f:
            cpus = parse_cpulist(f.read())
        if cpus:
            return cpus
    except OSError:
        pass
    try:
        with open(os.path.join(dev, "numa_node")) as f:
            node = int(f.read().strip())
        if node >= 0:
            with open(os.path.join(sysfs_root, "devices", "system", "node", f"node{node}", "cpulist")) as f:
                return parse_cpulist(f.read()) or None
    except (OSError, ValueError):
        pass
    return None


def bind_to_gpu(device_index: int, sysfs_root: str = "/sys", setaffinity=None) -> Optional[list[int]]:
    """Restrict this process to the cores local to CUDA device ``device_index`` (intersected with what it may already use).
    Returns the cores taken, or None when nothing was changed."""
    import torch
    try:
        p = torch.cuda.get_device_properties(device_index)
        ids = (int(getattr(p, "pci_domain_id", 0)), int(p.pci_bus_id), int(p.pci_device_id))
    except Exception as e:  # no such attribute / no device
        log.info_once(f"NUMA binding skipped: {e}")
        return None
    cpus = gpu_local_cpus(*ids, sysfs_root=sysfs_root)
    if not cpus:
        return None
    allowed = set(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else set(cpus)
    take = sorted(set(cpus) & allowed)
    if not take:
        return None
    (setaffinity or os.sched_setaffinity)(0, take)
    log.info_once(f"worker for cuda:{device_index} bound to {len(take)} cores of its NUMA node")
    return take
