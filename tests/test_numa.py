"""CPU affinity next to the GPU: parsing and the decisions, against a fake sysfs tree."""
import os

from tileccl_b200.utils import numa


def _fake_sysfs(tmp_path, node_of_gpu, cpulists):
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text(f"{node_of_gpu}\n")
    for n, text in cpulists.items():
        d = tmp_path / "devices" / "system" / "node" / f"node{n}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(text + "\n")
    return str(tmp_path)


def test_cpulist_and_node_lookup(tmp_path):
    assert numa.parse_cpulist("0-3,8,10-11") == {0, 1, 2, 3, 8, 10, 11}
    assert numa.parse_cpulist("") == set()
    root = _fake_sysfs(tmp_path, 1, {0: "0-55,112-167", 1: "56-111,168-223"})
    assert numa.gpu_numa_node("0000:1B:00.0", root) == 1
    assert numa.gpu_numa_node("00000000:1B:00.0", root) == 1          # NVML's 8-digit domain
    assert numa.gpu_numa_node("0000:99:00.0", root) == -1
    assert 56 in numa.node_cpus(1, root) and 0 not in numa.node_cpus(1, root)
    assert numa.node_cpus(7, root) == set()


def test_bind_decisions_leave_the_process_alone_when_unsure(tmp_path, monkeypatch):
    before = os.sched_getaffinity(0)
    try:
        # unknown node
        root = _fake_sysfs(tmp_path / "a", -1, {0: "0-3"})
        r = numa.bind_to_gpu_node(sysfs=root, pci_bus_id="0000:1b:00.0")
        assert not r["bound"] and r["node"] == -1 and os.sched_getaffinity(0) == before
        # the node's CPUs are not ours
        root = _fake_sysfs(tmp_path / "b", 0, {0: "100000-100003"})
        r = numa.bind_to_gpu_node(sysfs=root, pci_bus_id="0000:1b:00.0")
        assert not r["bound"] and "outside" in r["why"] and os.sched_getaffinity(0) == before
        # switched off
        monkeypatch.setenv("TILECCL_NO_NUMA_BIND", "1")
        root = _fake_sysfs(tmp_path / "c", 0, {0: ",".join(str(c) for c in sorted(before))})
        assert not numa.bind_to_gpu_node(sysfs=root, pci_bus_id="0000:1b:00.0")["bound"]
        monkeypatch.delenv("TILECCL_NO_NUMA_BIND")
        # the node holds one of our CPUs: bound to it
        one = min(before)
        root = _fake_sysfs(tmp_path / "d", 0, {0: str(one)})
        r = numa.bind_to_gpu_node(sysfs=root, pci_bus_id="0000:1b:00.0")
        assert r["bound"] and r["cpus"] == 1 and os.sched_getaffinity(0) == {one}
        # a broken tree never raises
        assert numa.bind_to_gpu_node(sysfs="/nonexistent", pci_bus_id="zz")["bound"] is False
    finally:
        os.sched_setaffinity(0, before)
