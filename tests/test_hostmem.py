"""Host-side placement helper: sysfs parsing and affinity narrowing against a fake sysfs tree."""
import os

import pytest

from cudeep_b200 import hostmem


def fake_sysfs(root, pci, node, cpulists):
    dev = root / "bus" / "pci" / "devices" / pci
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text(f"{node}\n")
    for n, text in cpulists.items():
        d = root / "devices" / "system" / "node" / f"node{n}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(text + "\n")
    return root


def test_parse_cpulist():
    assert hostmem.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert hostmem.parse_cpulist("5") == {5}
    assert hostmem.parse_cpulist("") == set()


def test_numa_node_lookup(tmp_path):
    root = fake_sysfs(tmp_path, "0000:1b:00.0", 1, {0: "0-3", 1: "4-7"})
    assert hostmem.numa_node_of("0000:1b:00.0", root) == 1
    assert hostmem.cpus_of_node(1, root) == {4, 5, 6, 7}
    assert hostmem.numa_node_of("0000:ff:00.0", root) is None           # unknown device
    single = fake_sysfs(tmp_path / "single", "0000:01:00.0", -1, {})
    assert hostmem.numa_node_of("0000:01:00.0", single) is None         # a machine without NUMA


@pytest.mark.skipif(not hasattr(os, "sched_getaffinity"), reason="no CPU affinity on this platform")
def test_near_gpu_narrows_and_restores(tmp_path):
    allowed = sorted(os.sched_getaffinity(0))
    if len(allowed) < 2:
        pytest.skip("one CPU: nothing to narrow")
    half = allowed[: len(allowed) // 2]
    root = fake_sysfs(tmp_path, "0000:1b:00.0", 0, {0: ",".join(map(str, half))})
    with hostmem.near_gpu(0, sysfs=root, pci="0000:1b:00.0") as info:
        assert info["bound"] and info["numa_node"] == 0 and info["cpus"] == len(half)
        assert os.sched_getaffinity(0) == set(half)
    assert sorted(os.sched_getaffinity(0)) == allowed


@pytest.mark.skipif(not hasattr(os, "sched_getaffinity"), reason="no CPU affinity on this platform")
def test_near_gpu_does_nothing_without_an_answer(tmp_path):
    allowed = os.sched_getaffinity(0)
    with hostmem.near_gpu(0, sysfs=tmp_path, pci="0000:1b:00.0") as info:
        assert not info["bound"] and info["numa_node"] is None
        assert os.sched_getaffinity(0) == allowed
    # a node whose CPUs this process may not use at all: left alone as well
    root = fake_sysfs(tmp_path / "other", "0000:1b:00.0", 0, {0: "100000-100003"})
    with hostmem.near_gpu(0, sysfs=root, pci="0000:1b:00.0") as info:
        assert not info["bound"]
        assert os.sched_getaffinity(0) == allowed
