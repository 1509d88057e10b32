"""NUMA placement helper for the pinned pools, against a fabricated sysfs tree."""

import os

import pytest

from directkv_b200 import numa


def _fake_sysfs(tmp_path, node_cpulists, gpu_node):
    node_dir = tmp_path / "node"
    for i, cpus in enumerate(node_cpulists):
        d = node_dir / f"node{i}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(cpus + "\n")
    (node_dir / "possible").write_text("0-1\n")           # a file that is not a node directory
    pci = tmp_path / "pci" / "0000:1b:00.0"
    pci.mkdir(parents=True)
    (pci / "numa_node").write_text(f"{gpu_node}\n")
    return str(node_dir), str(tmp_path / "pci")


def test_parse_cpulist():
    assert numa.parse_cpulist("0-3,8,10-11") == [0, 1, 2, 3, 8, 10, 11]
    assert numa.parse_cpulist("5") == [5]
    assert numa.parse_cpulist("") == []


def test_sysfs_readers(tmp_path, monkeypatch):
    sys_node, sys_pci = _fake_sysfs(tmp_path, ["0-3", "4-7"], 1)
    monkeypatch.setattr(numa, "gpu_pci_bus_id", lambda idx: "0000:1b:00.0")
    assert numa.node_count(sys_node) == 2
    assert numa.node_cpus(1, sys_node) == [4, 5, 6, 7]
    assert numa.gpu_numa_node(0, sys_pci) == 1
    assert numa.node_count(str(tmp_path / "missing")) == 0
    (tmp_path / "pci" / "0000:1b:00.0" / "numa_node").write_text("-1\n")       # what one-node machines report
    assert numa.gpu_numa_node(0, sys_pci) is None
    monkeypatch.setattr(numa, "gpu_pci_bus_id", lambda idx: None)
    assert numa.gpu_numa_node(0, sys_pci) is None


def test_single_node_machine_is_left_alone(tmp_path, monkeypatch):
    sys_node, sys_pci = _fake_sysfs(tmp_path, ["0-63"], 0)
    monkeypatch.setattr(numa, "gpu_pci_bus_id", lambda idx: "0000:1b:00.0")
    before = os.sched_getaffinity(0)
    with numa.local_to_gpu(0, sys_node, sys_pci) as node:
        assert node is None and os.sched_getaffinity(0) == before
    with numa.local_to_gpu(None, sys_node, sys_pci) as node:
        assert node is None


def test_affinity_and_policy_are_restored(tmp_path, monkeypatch):
    allowed = sorted(os.sched_getaffinity(0))
    if len(allowed) < 2:
        pytest.skip("needs two CPUs")
    half = allowed[: len(allowed) // 2]
    rest = allowed[len(allowed) // 2:]
    sys_node, sys_pci = _fake_sysfs(tmp_path, [",".join(map(str, rest)), ",".join(map(str, half))], 1)
    monkeypatch.setattr(numa, "gpu_pci_bus_id", lambda idx: "0000:1b:00.0")
    calls = []
    monkeypatch.setattr(numa, "set_preferred_node", lambda node: calls.append(node) or True)
    with numa.local_to_gpu(0, sys_node, sys_pci) as node:
        assert node == 1
        assert os.sched_getaffinity(0) == set(half)
    assert os.sched_getaffinity(0) == set(allowed)
    assert calls == [1, None]


def test_cpus_outside_the_cpuset_are_not_requested(tmp_path, monkeypatch):
    allowed = set(os.sched_getaffinity(0))
    foreign = ",".join(str(c) for c in range(max(allowed) + 1, max(allowed) + 5))
    sys_node, sys_pci = _fake_sysfs(tmp_path, ["0", foreign], 1)
    monkeypatch.setattr(numa, "gpu_pci_bus_id", lambda idx: "0000:1b:00.0")
    monkeypatch.setattr(numa, "set_preferred_node", lambda node: False)      # e.g. seccomp refuses the call
    with numa.local_to_gpu(0, sys_node, sys_pci) as node:
        assert node is None and os.sched_getaffinity(0) == allowed


def test_set_preferred_node_round_trip():
    """The real system call on the current (always existing) node 0: accepted or refused, never raising."""
    ok = numa.set_preferred_node(0)
    assert ok in (True, False)
    assert numa.set_preferred_node(None) in (True, False)
