"""CPU placement of GPU workers: cpulist parsing, the sysfs lookups, and the affinity call (against a made-up sysfs tree)."""
import os
from types import SimpleNamespace

from onecat_vllm.utils import numa


def test_parse_cpulist():
    assert numa.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert numa.parse_cpulist("") == []


def test_gpu_local_cpus_and_binding(tmp_path, monkeypatch):
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "local_cpulist").write_text("0-1,4\n")
    assert numa.gpu_local_cpus(0, 0x1b, 0, str(tmp_path)) == [0, 1, 4]
    # a function that only names its node: the node's cpulist is used
    dev2 = tmp_path / "bus" / "pci" / "devices" / "0001:9c:00.0"
    dev2.mkdir(parents=True)
    (dev2 / "numa_node").write_text("1\n")
    node = tmp_path / "devices" / "system" / "node" / "node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("2-3\n")
    assert numa.gpu_local_cpus(1, 0x9c, 0, str(tmp_path)) == [2, 3]
    assert numa.gpu_local_cpus(0, 0x55, 0, str(tmp_path)) is None
    import torch
    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda i: SimpleNamespace(pci_domain_id=0, pci_bus_id=0x1b, pci_device_id=0))
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: {0, 1, 2, 3})
    calls = []
    took = numa.bind_to_gpu(0, str(tmp_path), setaffinity=lambda pid, cpus: calls.append((pid, list(cpus))))
    assert took == [0, 1] and calls == [(0, [0, 1])]           # core 4 is outside what the process may use
    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda i: SimpleNamespace(pci_domain_id=0, pci_bus_id=0x55, pci_device_id=0))
    assert numa.bind_to_gpu(0, str(tmp_path), setaffinity=lambda *a: calls.append(a)) is None and len(calls) == 1
