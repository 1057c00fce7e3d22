"""Host-buffer collectives among real processes on this machine (shared-memory backend).

Covers the configuration the baseline names (4 processes, all-reduce sum fp32, 1024 elements per
rank, uniform[-1,1] seeded by rank, 1000 repeats, checked against a serial sum with rtol 1e-5; the
same shapes for reduce-scatter and all-gather) plus every dtype x operator, world sizes that are not
powers of two, counts that the world size does not divide, unaligned buffers, both algorithms.
"""
import os
import subprocess

import pytest

from dccl_b200.utils.launch import python_ranks, spawn_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "workers", "cpu_worker.py")


def run_worker(world, args, env=None, timeout=240):
    res = python_ranks(WORKER, args, world, env_extra=env, timeout=timeout)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d: %s\n%s" % (r, p.stdout[-2000:], p.stderr[-2000:])
        assert p.stdout.strip().startswith("OK"), p.stdout
    return res


@pytest.mark.parametrize("world", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("algo", ["ring", "rabenseifner"])
def test_all_dtypes_ops_and_shapes(world, algo):
    res = run_worker(world, ["--suite", "basic", "--algo", algo])
    assert res[0].stdout.split()[2] == algo


@pytest.mark.parametrize("world", [6, 7])
def test_large_odd_counts_non_power_of_two(world):
    # messages larger than one FIFO, tiny FIFO: exercises wrap-around and back pressure
    run_worker(world, ["--suite", "large", "--algo", "rabenseifner"], env={"DCCL_SHM_CHANNEL_BYTES": "8192"})
    run_worker(world, ["--suite", "large", "--algo", "ring"], env={"DCCL_SHM_CHANNEL_BYTES": "8192"})


def test_baseline_config_python_api():
    run_worker(4, ["--suite", "baseline", "--algo", "ring", "--repeat", "1000"])


@pytest.mark.parametrize("api", ["all_reduce", "reduce_scatter", "all_gather"])
def test_baseline_config_dccl_cli(build_dir, tmp_path, api):
    """4 processes x dccl_cli --verify, 1000 repeats, and the .tt files it leaves behind."""
    cli = os.path.join(build_dir, "dccl_cli")
    count = "1024" if api == "all_reduce" else "4096"   # 1024 elements per rank
    res = spawn_ranks([cli, "-a", api, "-t", "float32", "-c", count, "-r", "1000", "-i", "uniform", "--verify", "--tt-per-rank"],
                      4, cwd=str(tmp_path), timeout=240)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d: %s\n%s" % (r, p.stdout[-1500:], p.stderr[-1500:])
        assert "verify: ok" in p.stdout
        assert "dccl api evaluation with the following configuration:" in p.stdout
        assert "\tapi:%s" % api in p.stdout and "\trepeat:1000" in p.stdout and "\ttype:7" in p.stdout
    from dccl_b200.utils import tt
    for r in range(4):
        declared, rows = tt.read_tt(str(tmp_path / ("dccl_cli.%d.tt" % r)))
        assert declared == len(rows)
        tags = [x[0] for x in rows]
        assert tags[:3] == [1000001, 1000002, 1000003] and tags[-1] == 1000004
        assert all(x[1] == r for x in rows)
        if api == "all_reduce":
            assert tags.count(1001001) == 1000 and tags.count(1001100) == 1000


@pytest.mark.parametrize("api", ["all_to_all", "gather", "scatter"])
def test_dccl_cli_composed_collectives(build_dir, tmp_path, api):
    """The entry points composed of grouped send / recv, 3 host processes, messages longer than a FIFO."""
    cli = os.path.join(build_dir, "dccl_cli")
    res = spawn_ranks([cli, "-a", api, "-t", "int64", "-c", str(3 * 200001), "-r", "5", "-w", "1", "-i", "uniform", "--verify", "--root", "2"],
                      3, cwd=str(tmp_path), timeout=240)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d: %s\n%s" % (r, p.stdout[-1500:], p.stderr[-1500:])
        if api != "gather" or r == 2:
            assert "verify: ok" in p.stdout, (api, r, p.stdout[-500:])


def test_nccl_spellings_compile_and_run(build_dir, tmp_path):
    """examples/nccl_names: the inline NCCL-style aliases of the header (built by make)."""
    p = subprocess.run([os.path.join(build_dir, "nccl_names")], cwd=str(tmp_path), capture_output=True, text=True, timeout=60)
    assert p.returncode == 0 and p.stdout.strip() == "1 0 no error 2.0", (p.stdout, p.stderr)


def test_flat_c_interface_from_plain_c(build_dir, tmp_path):
    """examples/c_api/main.c compiled as C against include/dccl/dccl_c.h (built by make)."""
    p = subprocess.run([os.path.join(build_dir, "c_api_example")], cwd=str(tmp_path), capture_output=True, text=True, timeout=60)
    assert p.returncode == 0 and p.stdout.strip() == "rank 0 of 1: 1 2 3 4 (no error)", (p.stdout, p.stderr)


def test_cli_defaults_match_the_original(build_dir, tmp_path):
    cli = os.path.join(build_dir, "dccl_cli")
    p = spawn_ranks([cli, "-a", "all_reduce", "-r", "3"], 1, cwd=str(tmp_path))[0]
    assert p.returncode == 0
    lines = p.stdout.splitlines()
    assert lines[0] == "dccl api evaluation with the following configuration:"
    assert "\twarmup:0" in lines and "\ttype:3" in lines and "\top:0" in lines and "\tcount:1024" in lines
    assert lines[lines.index("warm up...") + 1] == "done."
    assert "flush timestamp..." in lines and lines[-1] == "...done"
    assert (tmp_path / "dccl_cli.tt").exists()
    # no --api: help text, exit status -1
    p = spawn_ranks([cli], 1, cwd=str(tmp_path))[0]
    assert p.returncode == 255 and "--api NAME" in p.stdout
    # operators are parsed by name (max is max, not prod)
    p = spawn_ranks([cli, "-a", "all_reduce", "-o", "max", "-r", "1"], 1, cwd=str(tmp_path))[0]
    assert "\top:2" in p.stdout


def test_cli_save_hex_dump_layout(build_dir, tmp_path):
    """--save writes the 32-bytes-per-line hex dumps of the original's save_mem."""
    cli = os.path.join(build_dir, "dccl_cli")
    p = spawn_ranks([cli, "-a", "all_reduce", "-t", "uint32", "-c", "20", "-r", "1", "-s"], 1, cwd=str(tmp_path), timeout=60)[0]
    assert p.returncode == 0
    for name in ("sendbuf.host.before.txt", "recvbuf.host.txt", "sendbuf.host.after.txt"):
        assert (tmp_path / name).exists(), name
    lines = (tmp_path / "sendbuf.host.before.txt").read_text().split("\n")
    assert lines[0] == "0x00000000: " + "  ".join(" ".join(["00"] * 8) for _ in range(4))
    assert lines[1].startswith("0x00000020: 00 00 00 00 00 00 00 00  00")
    assert len(lines[2].split(":")[1].split()) == 16          # 80 bytes = 32 + 32 + 16


def test_cfg_directory_recipe(build_dir, tmp_path):
    """cd cfg/n<k> && helloworld: rank from local_id, world from layout.json, no environment variables."""
    from dccl_b200.utils.launch import free_port
    import subprocess
    port = free_port()
    (tmp_path / "layout.json").write_text('[{"type_alias":"DCCLSubgroupType","layout":[{"min_nodes_by_shard":["3"],"max_nodes_by_shard":["3"]}]}]')
    procs = []
    env = {k: v for k, v in os.environ.items() if not k.startswith("DCCL_") and k not in ("RANK", "WORLD_SIZE")}
    for r in range(3):
        d = tmp_path / ("n%d" % r)
        d.mkdir()
        (d / "derecho.cfg").write_text("[DERECHO]\ncontact_ip = 127.0.0.1\ncontact_port = %d\nlocal_id = %d\nlocal_ip = 127.0.0.1\n"
                                       "[DCCL]\nallreduce_algorithm = rabenseifner\n[LAYOUT]\njson_layout_file = ../layout.json\n" % (port, r))
        procs.append(subprocess.Popen([os.path.join(build_dir, "helloworld")], cwd=str(d), env=env, stdout=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=60)[0] for p in procs]
    for r, o in enumerate(outs):
        assert "world size = 3, my rank = %d" % r in o


def test_p2p_perf_host_mode(build_dir, tmp_path):
    """Windowed send/recv throughput tool between rank 0 and 1 over the host path; writes oob.dat."""
    tool = os.path.join(build_dir, "p2p_perf")
    dirs = []
    for r in range(2):
        d = tmp_path / ("r%d" % r)
        d.mkdir()
        dirs.append(d)
    import subprocess
    from dccl_b200.utils.launch import free_port
    port = free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, DCCL_RANK=str(r), DCCL_WORLD_SIZE="2", DCCL_MASTER_PORT=str(port), DCCL_MASTER_ADDR="127.0.0.1")
        procs.append(subprocess.Popen([tool, "-t", "p2p", "-s", "65536", "-d", "4", "-w", "0.2", "-D", "0.5"], cwd=str(dirs[r]), env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=60) for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "Evaluating transport performance with the following configuration:" in outs[0][0]
    assert "GB/s" in outs[0][0] and "received" in outs[1][0]
    from dccl_b200.utils import tt
    declared, rows = tt.read_tt(str(dirs[0] / "oob.dat"))
    tags = [x[0] for x in rows]
    assert declared == len(rows) and tags[0] == 2000001 and 2000004 in tags and tags.count(2001001) >= 8
    # missing --transport: exit 1 with the help text
    p = subprocess.run([tool], capture_output=True, text=True)
    assert p.returncode == 1 and "--transport" in p.stdout + p.stderr


def test_cmake_build_install_and_find_package(tmp_path):
    """The CMake route of the original (cmake .. && make && make install, then find_package(dccl) from another
    project; reference CMakeLists.txt:108-175, examples/helloworld/CMakeLists.txt): host-only configuration here."""
    import shutil
    if shutil.which("cmake") is None:
        pytest.skip("cmake is not installed")
    bdir, prefix, hdir = tmp_path / "b", tmp_path / "inst", tmp_path / "hw"
    bdir.mkdir()
    hdir.mkdir()
    def sh(cmd, cwd):
        p = subprocess.run(cmd, cwd=str(cwd), capture_output=True, text=True, timeout=900)
        assert p.returncode == 0, " ".join(cmd) + "\n" + p.stdout[-2000:] + p.stderr[-2000:]
    sh(["cmake", ROOT, "-DDCCL_WITH_CUDA=OFF", "-DCMAKE_INSTALL_PREFIX=" + str(prefix)], bdir)
    sh(["make", "-j8"], bdir)
    sh(["make", "install"], bdir)
    for rel in ["lib/libdccl.so", "include/dccl/dccl.hpp", "include/dccl/dccl_c.h", "include/dccl/config.h", "bin/dccl_cli", "bin/p2p_perf",
                "lib/cmake/dccl/dcclConfig.cmake"]:
        assert (prefix / rel).exists(), rel
    sh(["cmake", os.path.join(ROOT, "examples", "helloworld"), "-Ddccl_DIR=" + str(prefix / "lib" / "cmake" / "dccl")], hdir)
    sh(["make"], hdir)
    env = dict(os.environ, DCCL_RANK="0", DCCL_WORLD_SIZE="1")
    p = subprocess.run([str(hdir / "helloworld")], env=env, capture_output=True, text=True, timeout=60)
    assert p.returncode == 0 and "world size = 1, my rank = 0" in p.stdout, p.stdout + p.stderr


def test_python_examples(dccl_lib):
    """examples/python: all-reduce on host arrays over 4 ranks, a tensor-parallel MLP training for a few steps on 2."""
    for script, world in (("allreduce.py", 4), ("tensor_parallel_mlp.py", 2)):
        res = python_ranks(os.path.join(ROOT, "examples", "python", script), [], world, timeout=300)
        for r, p in enumerate(res):
            assert p.returncode == 0, "%s rank %d:\n%s\n%s" % (script, r, p.stdout[-2000:], p.stderr[-2000:])
