"""Host logic of the benchmark that needs no GPU: reading the GPUs' local cores from the driver's
topology table and dividing them among the ranks of a node."""
import os
import subprocess
import sys
import types

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402

TOPO_ONE_NODE = (
    "\t\x1b[4mGPU0\tGPU1\tGPU2\tGPU3\tCPU Affinity\tNUMA Affinity\tGPU NUMA ID\x1b[0m\n"
    "GPU0\t X \tNV18\tNV18\tNV18\t0-31\t0\t\tN/A\n"
    "GPU1\tNV18\t X \tNV18\tNV18\t0-31\t0\t\tN/A\n"
    "GPU2\tNV18\tNV18\t X \tNV18\t0-31\t0\t\tN/A\n"
    "GPU3\tNV18\tNV18\tNV18\t X \t0-31\t0\t\tN/A\n"
    "\nLegend:\n\n  X    = Self\n")
TOPO_TWO_SOCKETS = (
    "\tGPU0\tGPU1\tGPU2\tGPU3\tCPU Affinity\tNUMA Affinity\n"
    "GPU0\t X \tNV18\tSYS\tSYS\t0-15,64-79\t0\n"
    "GPU1\tNV18\t X \tSYS\tSYS\t0-15,64-79\t0\n"
    "GPU2\tSYS\tSYS\t X \tNV18\t16-31,80-95\t1\n"
    "GPU3\tSYS\tSYS\tNV18\t X \t16-31,80-95\t1\n")


def fake_topo(monkeypatch, text):
    def run(cmd, **kwargs):
        assert cmd[:3] == ["nvidia-smi", "topo", "-m"]
        return types.SimpleNamespace(stdout=text)
    monkeypatch.setattr(subprocess, "run", run)


def test_local_cores_are_read_from_the_topology_table(monkeypatch):
    fake_topo(monkeypatch, TOPO_ONE_NODE)
    aff = bench.gpu_cpu_affinities()
    assert sorted(aff) == [0, 1, 2, 3] and all(v == list(range(32)) for v in aff.values())
    fake_topo(monkeypatch, TOPO_TWO_SOCKETS)
    aff = bench.gpu_cpu_affinities()
    assert aff[0] == list(range(16)) + list(range(64, 80)) and aff[3] == list(range(16, 32)) + list(range(80, 96))
    fake_topo(monkeypatch, "no table here\n")
    assert bench.gpu_cpu_affinities() == {}


@pytest.mark.parametrize("topo,world,expected", [
    # one socket: the ranks divide its cores evenly
    (TOPO_ONE_NODE, 4, [list(range(0, 8)), list(range(8, 16)), list(range(16, 24)), list(range(24, 32))]),
    (TOPO_ONE_NODE, 2, [list(range(0, 16)), list(range(16, 32))]),
    # two sockets: the two ranks of a socket divide that socket's cores
    (TOPO_TWO_SOCKETS, 4, [list(range(0, 16)), list(range(64, 80)), list(range(16, 32)), list(range(80, 96))]),
])
def test_ranks_divide_the_cores_their_gpus_share(monkeypatch, topo, world, expected):
    fake_topo(monkeypatch, topo)
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: set(range(96)), raising=False)
    bound = {}
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cores: bound.setdefault("cores", list(cores)), raising=False)
    for rank in range(world):
        bound.clear()
        text = bench.pin_rank_to_cores(rank, world, rank)
        assert bound["cores"] == expected[rank], (rank, bound)
        assert text.startswith("cores local to the GPU")


def test_without_a_topology_table_all_cores_are_split_evenly(monkeypatch):
    fake_topo(monkeypatch, "")
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: set(range(8)), raising=False)
    bound = {}
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cores: bound.setdefault("cores", list(cores)), raising=False)
    assert bench.pin_rank_to_cores(1, 4, 1).startswith("even split of all cores")
    assert bound["cores"] == [2, 3]
