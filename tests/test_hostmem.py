"""Host-side NUMA placement helper: sysfs parsing and the decision, against a fake sysfs tree (no GPU, no affinity
change)."""
import os

from strata_b200 import hostmem


def fake_sysfs(tmp_path, node_of_device, cpulists):
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("%d\n" % node_of_device)
    for node, text in cpulists.items():
        d = tmp_path / "devices" / "system" / "node" / ("node%d" % node)
        d.mkdir(parents=True)
        (d / "cpulist").write_text(text + "\n")
    return str(tmp_path)


def test_cpu_list_format():
    assert hostmem.parse_cpu_list("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert hostmem.parse_cpu_list("") == []
    assert hostmem.parse_cpu_list("5,x-2,7") == [5, 7]


def test_binds_to_the_allowed_cpus_of_the_device_node(tmp_path):
    sysfs = fake_sysfs(tmp_path, 1, {0: "0-13,28-41", 1: "14-27,42-55"})
    rec = hostmem.bind_to_node_of("0000:1B:00.0", sysfs=sysfs, allowed=set(range(10, 20)), apply=False)
    assert rec == {"node": 1, "cpus": 6, "bound": True}


def test_leaves_the_process_alone_when_it_cannot_help(tmp_path):
    sysfs = fake_sysfs(tmp_path, 1, {0: "0-13", 1: "14-27"})
    rec = hostmem.bind_to_node_of("0000:1b:00.0", sysfs=sysfs, allowed=set(range(0, 8)), apply=False)
    assert not rec["bound"] and "no allowed CPU" in rec["why"]
    rec = hostmem.bind_to_node_of("0000:1b:00.0", sysfs=sysfs, allowed=set(range(14, 20)), apply=False)
    assert not rec["bound"] and "already confined" in rec["why"]
    rec = hostmem.bind_to_node_of("0000:ff:00.0", sysfs=sysfs, allowed={0}, apply=False)
    assert not rec["bound"] and rec["node"] is None
    sysfs2 = fake_sysfs(tmp_path / "b", -1, {})
    rec = hostmem.bind_to_node_of("0000:1b:00.0", sysfs=sysfs2, allowed={0}, apply=False)
    assert not rec["bound"]


def test_a_dry_run_changes_nothing():
    before = os.sched_getaffinity(0)
    rec = hostmem.bind_near_gpu(0, apply=False)
    assert os.sched_getaffinity(0) == before
    assert isinstance(rec["bound"], bool)
