"""Command-line tools on GPU buffers: dccl_cli --verify for every entry point, its stock-NCCL twin on the
same workload (both are checked against the same serial fold, which is the differential test), the
p2p_perf window test and the C++ sweep tool."""
import glob
import os
import sys

import pytest

from conftest import gpu_count
from dccl_b200.utils.launch import spawn_ranks

pytestmark = pytest.mark.gpu


def nccl_env():
    c = glob.glob(os.path.join(sys.prefix, "lib", "python*", "site-packages", "nvidia", "nccl", "lib", "libnccl.so.2"))
    return {"DCCL_NCCL_LIB": c[0]} if c else {}


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_dccl_cli_verifies_every_api_on_gpus(build_dir, tmp_path):
    world = min(gpu_count(), 8)
    cli = os.path.join(build_dir, "dccl_cli")
    for api, dtype, op, count in [("all_reduce", "bfloat16", "avg", 8 * 100003), ("all_reduce", "float32", "sum", 1024),
                                  ("reduce_scatter", "float32", "max", 8 * 4096), ("all_gather", "int32", "sum", 8 * 50000),
                                  ("reduce", "float64", "sum", 30000), ("broadcast", "uint8", "sum", 70001)]:
        res = spawn_ranks([cli, "-a", api, "-g", "auto", "-t", dtype, "-o", op, "-c", str(count), "-r", "20", "-w", "2", "-i", "uniform", "--verify",
                           "--tt-per-rank"], world, cwd=str(tmp_path), gpus=True, timeout=180)
        for r, p in enumerate(res):
            assert p.returncode == 0, (api, r, p.stdout[-800:], p.stderr[-800:])
            if api != "reduce" or r == 0:
                assert "verify: ok" in p.stdout, (api, r, p.stdout[-500:])
    # send / recv between rank 0 and rank 1, like the original's test: rank 0 runs 'send', rank 1 'recv'; --verify on both
    # so that both make the same (collective) registration calls
    base = [cli, "-g", "auto", "-t", "float32", "-c", "100000", "-r", "5", "-i", "uniform"]
    res = spawn_ranks(base + ["-a", "send", "--verify"], 2, cwd=str(tmp_path), gpus=True, timeout=120, per_rank_argv={1: base + ["-a", "recv", "--verify"]})
    assert all(p.returncode == 0 for p in res), [(p.stdout[-400:], p.stderr[-400:]) for p in res]
    assert "verify: ok" in res[1].stdout


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_stock_nccl_twin_agrees(build_dir, tmp_path):
    world = min(gpu_count(), 8)
    res = spawn_ranks([os.path.join(build_dir, "nccl_cli"), "-a", "all_reduce", "-g", "auto", "-t", "float32", "-o", "sum", "-c", "100003", "-r", "10",
                       "-i", "uniform", "--verify"], world, cwd=str(tmp_path), gpus=True, timeout=180, env_extra=nccl_env())
    for r, p in enumerate(res):
        assert p.returncode == 0, (r, p.stdout[-800:], p.stderr[-800:])
        assert "verify: ok" in p.stdout
    assert (tmp_path / "nccl_cli.0.tt").exists()


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_p2p_perf_and_sweep_tool_on_gpus(build_dir, tmp_path):
    res = spawn_ranks([os.path.join(build_dir, "p2p_perf"), "-t", "p2p", "-c", "0", "-s", "1048576", "-d", "4", "-w", "0.2", "-D", "0.5"], 2,
                      cwd=str(tmp_path), timeout=120, per_rank_env={0: {"CUDA_VISIBLE_DEVICES": "0"}, 1: {"CUDA_VISIBLE_DEVICES": "1"}})
    # each rank sees one device as device 0; peer mapping still goes through the file-descriptor handles
    assert all(p.returncode == 0 for p in res), [(p.stdout[-400:], p.stderr[-400:]) for p in res]
    assert "GB/s" in res[0].stdout
    res = spawn_ranks([os.path.join(build_dir, "dccl_sweep"), "--gpu", "auto", "--min", "4096", "--max", "4194304", "--factor", "32", "--impls", "dccl",
                       "--out", str(tmp_path / "sweep.json")], 2, cwd=str(tmp_path), gpus=True, timeout=180)
    assert all(p.returncode == 0 for p in res), [(p.stdout[-400:], p.stderr[-400:]) for p in res]
    import json
    rows = json.load(open(tmp_path / "sweep.json"))["rows"]
    assert len(rows) == 9 and all(r["us"] > 0 for r in rows)


def test_topology_tool_lists_the_visible_gpus(build_dir):
    """dccl_topo: one entry per visible GPU, every pair peer-accessible on an NVSwitch box, a one-line summary."""
    import json
    import subprocess
    p = subprocess.run([os.path.join(build_dir, "dccl_topo")], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr
    out = json.loads(p.stdout)
    n = min(gpu_count(), 8)
    topo = out["topology"]
    assert topo["nranks"] == n and all(g["sm_count"] > 0 for g in topo["gpus"])
    assert all(topo["peer_access"][a][b] == (2 if a == b else 1) for a in range(n) for b in range(n))
    assert str(n) + " x " in out["summary"]
