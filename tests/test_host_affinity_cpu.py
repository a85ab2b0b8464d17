"""core.bind_host_threads_to_node_of: the CPUs of the NUMA node a PCI device
hangs off, read from a sysfs tree (a made-up one here), become the affinity
of the calling thread.  Runs in a child process, whose affinity dies with it."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import os, sys
sys.path.insert(0, sys.argv[1])
from __graft_entry__ import load_package
core = load_package().core
before = sorted(os.sched_getaffinity(0))
print("R", core.bind_host_threads_to_node_of(sys.argv[3], sys.argv[2]), sorted(os.sched_getaffinity(0)) == before)
print("A", sorted(os.sched_getaffinity(0)))
"""


def _run(tmp, bus):
    out = subprocess.run([sys.executable, "-c", CHILD, ROOT, str(tmp), bus], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = dict(l.split(" ", 1) for l in out.stdout.strip().splitlines())
    return lines


def _tree(tmp, node, cpulist):
    dev = tmp / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("%d\n" % node)
    if cpulist is not None:
        nd = tmp / "devices" / "system" / "node" / ("node%d" % max(node, 0))
        nd.mkdir(parents=True)
        (nd / "cpulist").write_text(cpulist + "\n")


def test_binds_to_the_nodes_cpus(tmp_path):
    allowed = sorted(os.sched_getaffinity(0))
    if len(allowed) < 2:
        pytest.skip("needs two usable CPUs")
    keep = allowed[:1] + allowed[-1:]
    # the list names the two CPUs as ranges plus one CPU this process may not use
    _tree(tmp_path, 1, "%d-%d,%d,100000" % (keep[0], keep[0], keep[1]))
    got = _run(tmp_path, "0000:1B:00.0")          # CUDA reports the address in upper case
    assert got["R"].startswith("(1, 2)")
    assert got["A"] == str(keep)


@pytest.mark.parametrize("node,cpulist", [(-1, None), (0, None), (0, "100000-100001")])
def test_leaves_the_affinity_alone_when_the_node_is_unknown(tmp_path, node, cpulist):
    _tree(tmp_path, node, cpulist)
    got = _run(tmp_path, "0000:1b:00.0")
    assert got["R"].endswith("True")              # affinity unchanged
    assert got["R"].startswith("(-1, 0)") or got["R"].startswith("(0, 0)")


def test_unknown_device_directory(tmp_path):
    got = _run(tmp_path, "0000:ff:00.0")
    assert got["R"].startswith("(-1, 0)") and got["R"].endswith("True")
