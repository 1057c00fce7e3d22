"""Host-side unit tests: index arithmetic, conversions, configuration, timestamps, variant table."""
import ctypes
import os

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from dccl_b200.utils import oracle, tt


def test_slot_range_covers_everything(dccl_lib):
    lo, hi = ctypes.c_size_t(), ctypes.c_size_t()
    for count in [0, 1, 7, 8, 1000, 1023, 1024, 1025, 99999]:
        for n in range(1, 9):
            for align in [1, 4, 8]:
                covered = 0
                prev_hi = 0
                for i in range(n):
                    dccl_lib.dccl_slot_range(count, n, i, align, ctypes.byref(lo), ctypes.byref(hi))
                    assert lo.value == prev_hi and hi.value >= lo.value
                    if lo.value < count:
                        assert lo.value % align == 0
                    covered += hi.value - lo.value
                    prev_hi = hi.value
                assert covered == count and prev_hi == count


@given(st.integers(0, 255), st.integers(1, 8))
@settings(max_examples=200, deadline=None)
def test_reverse_bits_is_an_involution(dccl_lib, x, bits):
    x &= (1 << bits) - 1
    r = dccl_lib.dccl_reverse_bits(x, bits)
    assert dccl_lib.dccl_reverse_bits(r, bits) == x
    assert bin(r).count("1") == bin(x).count("1")


def test_log_two(dccl_lib):
    for x in range(1, 300):
        assert dccl_lib.dccl_log_two(x) == x.bit_length() - 1


def test_type_and_op_names(dccl_lib):
    names = ["int8", "uint8", "int32", "uint32", "int64", "uint64", "float16", "float32", "float64", "bfloat16"]
    sizes = [1, 1, 4, 4, 8, 8, 2, 4, 8, 2]
    for i, (nm, sz) in enumerate(zip(names, sizes)):
        assert dccl_lib.dccl_parse_type(nm.encode()) == i
        assert dccl_lib.dccl_size_of_type(i) == sz
    # every operator name maps to its own value (the original's parser mixed them up)
    for i, nm in enumerate(["sum", "prod", "max", "min", "avg"]):
        assert dccl_lib.dccl_parse_op(nm.encode()) == i
    assert dccl_lib.dccl_parse_op(b"nonsense") == 5
    assert dccl_lib.dccl_parse_type(b"nonsense") == 10


def test_half_conversion_matches_numpy(dccl_lib):
    bits = np.arange(0, 65536, 7, dtype=np.uint16)
    for b in bits:
        f = np.array([b], dtype=np.uint16).view(np.float16)[0]
        got = dccl_lib.dccl_half_to_float(int(b))
        if np.isnan(f):
            assert np.isnan(got)
        else:
            assert got == float(f)
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.normal(0, 1, 2000), rng.normal(0, 1e-6, 500), rng.normal(0, 3e4, 500), [0.0, -0.0, 65504.0, 1e6, -1e6, 6e-8]]).astype(np.float32)
    for v in vals:
        want = np.array([v], dtype=np.float32).astype(np.float16).view(np.uint16)[0]
        assert dccl_lib.dccl_float_to_half(float(v)) == int(want), v


def test_bf16_conversion_round_to_nearest_even(dccl_lib):
    rng = np.random.default_rng(1)
    vals = rng.normal(0, 10, 3000).astype(np.float32)
    want = oracle.f32_to_bf16(vals)
    for v, w in zip(vals, want):
        assert dccl_lib.dccl_float_to_bf16(float(v)) == int(w)
        assert dccl_lib.dccl_bf16_to_float(int(w)) == float(oracle.bf16_to_f32(np.array([w]))[0])


def test_config_file_env_and_layout(dccl_lib, tmp_path, monkeypatch):
    cfg = tmp_path / "derecho.cfg"
    cfg.write_text("# comment\n[DERECHO]\nlocal_id = 3\ncontact_ip = 127.0.0.1\ncontact_port = 23580 # trailing\n"
                   "[DCCL]\nallreduce_algorithm = rabenseifner\n[LOGGER]\ndefault_log_level = info\n")
    (tmp_path / "layout.json").write_text('[{"layout":[{"min_nodes_by_shard": ["8"], "max_nodes_by_shard": ["8"]}]}]')
    monkeypatch.chdir(tmp_path)
    monkeypatch.delenv("DCCL_ALLREDUCE_ALGORITHM", raising=False)
    dccl_lib.dccl_config_reload()
    out = ctypes.create_string_buffer(64)
    assert dccl_lib.dccl_config_get(b"DCCL/allreduce_algorithm", out, 64) == 1 and out.value == b"rabenseifner"
    assert dccl_lib.dccl_config_get(b"DERECHO/contact_port", out, 64) == 1 and out.value == b"23580"
    assert dccl_lib.dccl_config_get(b"DERECHO/nothing", out, 64) == 0
    # environment beats the file
    monkeypatch.setenv("DCCL_ALLREDUCE_ALGORITHM", "ring")
    assert dccl_lib.dccl_config_get(b"DCCL/allreduce_algorithm", out, 64) == 1 and out.value == b"ring"
    assert dccl_lib.dccl_config_parse_world((tmp_path / "layout.json").read_text().encode()) == 8
    assert dccl_lib.dccl_config_parse_world(b"{}") == 0
    monkeypatch.chdir(os.path.dirname(__file__))
    dccl_lib.dccl_config_reload()


def test_timestamp_file_format(dccl_lib, tmp_path):
    dccl_lib.dccl_timestamp_clear()
    for i in range(5000):   # more than the first buffer: exercises growth
        dccl_lib.dccl_timestamp_log(1001001 + (i % 2) * 99, 3, i)
    assert dccl_lib.dccl_timestamp_size() == 5000
    path = tmp_path / "x.tt"
    dccl_lib.dccl_timestamp_flush(str(path).encode(), 1)
    assert dccl_lib.dccl_timestamp_size() == 0
    lines = path.read_text().splitlines()
    assert lines[0] == "# number of entries:5000"
    assert lines[1] == "# tag rank extra tsns"
    declared, rows = tt.read_tt(str(path))
    assert declared == 5000 and len(rows) == 5000
    assert rows[0][:3] == (1001001, 3, 0) and rows[1][:3] == (1001100, 3, 1)
    ts = [r[3] for r in rows]
    assert all(b >= a for a, b in zip(ts, ts[1:]))
    assert len(tt.durations(rows, 1001001, 1001100)) == 2500


def test_tuner_table_and_file_override(dccl_lib):
    algo = ctypes.create_string_buffer(32)
    ctas = ctypes.c_int()

    def choose(coll, n, nbytes, nvls=1):
        assert dccl_lib.dccl_tuner_choose(coll.encode(), n, nbytes, nvls, algo, 32, ctypes.byref(ctas)) == 0
        return algo.value.decode(), ctas.value

    assert choose("allreduce", 8, 1024)[0] == "oneshot"
    assert choose("allreduce", 8, 1 << 30)[0] == "nvls"
    assert choose("allreduce", 8, 1 << 30, nvls=0)[0] == "twoshot"     # no multicast: peer-to-peer variant
    assert choose("allreduce_sym", 8, 1 << 30) == ("nvls", 16)
    # two ranks: rows for an exact world size come before the wildcard rows
    assert choose("allreduce_sym", 2, 1 << 30) == ("twoshot", 128) and choose("allreduce", 2, 1 << 24) == ("twoshot", 128)
    assert choose("allreduce", 2, 50000)[0] == "oneshot" and choose("allreduce", 2, 300000)[0] == "twoshot_ll"
    assert choose("allreduce", 4, 1 << 30)[0] == "twoshot" and choose("allreduce_sym", 4, 1 << 30) == ("nvls", 16)
    assert choose("allreduce", 4, 1 << 20)[0] == "twoshot_ll" and choose("allreduce", 6, 1 << 30)[0] == "nvls"
    assert choose("reducescatter_sym", 8, 1 << 30) == ("nvls", 64) and choose("reducescatter", 8, 1 << 30)[0] == "twoshot"
    assert dccl_lib.dccl_tuner_choose(b"bogus", 8, 1, 1, algo, 32, ctypes.byref(ctas)) == -1
    text = b"# my table\nallreduce 8 4k ring 4\nallreduce * inf rabenseifner 12\nnot a rule\nallreduce 8 1m twoshot 999\n"
    assert dccl_lib.dccl_tuner_load_text(text) == 2
    assert choose("allreduce", 8, 1000) == ("ring", 4)
    assert choose("allreduce", 8, 100000) == ("rabenseifner", 12)
    assert choose("allreduce", 4, 10) == ("rabenseifner", 12)
    assert choose("reducescatter", 8, 10)[0] == "oneshot"              # untouched collective keeps the built-in rows
    # rules bound to an element width: they come before the rules for every width, for the same world size only
    def choose_w(coll, n, nbytes, esize):
        assert dccl_lib.dccl_tuner_choose_width(coll.encode(), n, nbytes, 1, esize, algo, 32, ctypes.byref(ctas)) == 0
        return algo.value.decode(), ctas.value
    text = b"allgather 8 1m ring 8 2\nallgather 8 1m twoshot 16\nallgather * inf nvls 24 4\nallgather * inf oneshot 3 *\nallgather 8 inf ring 5 3\n"
    assert dccl_lib.dccl_tuner_load_text(text) == 4                     # an element width of 3 bytes is refused
    assert choose_w("allgather", 8, 1000, 2) == ("ring", 8) and choose_w("allgather", 8, 1000, 4) == ("twoshot", 16)
    assert choose_w("allgather", 8, 1000, 0) == ("twoshot", 16) and choose_w("allgather", 8, 1 << 22, 4) == ("nvls", 24)
    assert choose_w("allgather", 4, 1000, 2) == ("oneshot", 3) and choose_w("allgather", 4, 1000, 4) == ("nvls", 24)


def test_oracle_integer_semantics():
    a = np.array([100, -100, 7], dtype=np.int8)
    b = np.array([100, -100, -2], dtype=np.int8)
    assert list(oracle.fold([a, b], "sum")) == [-56, 56, 5]            # wraps like the kernels
    assert list(oracle.fold([a, b], "prod")) == [16, 16, -14]
    assert list(oracle.fold([np.array([-7], np.int32), np.array([2], np.int32)], "avg")) == [-2]   # truncates toward zero


def test_tuning_table_from_measured_sweeps(dccl_lib, tmp_path):
    """benchmarks/make_tune_table.py: the fastest variant per size becomes a rule the native tuner accepts."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    rows = []
    for nbytes, times in [(1024, {"oneshot": 5.0, "twoshot": 12.0}), (65536, {"oneshot": 8.0, "twoshot": 13.0}),
                          (1 << 20, {"twoshot": 20.0, "nvls": 18.0}), (1 << 26, {"twoshot": 300.0, "nvls": 150.0, "ring": 500.0})]:
        for algo, us in times.items():
            for ctas in (16, 64):
                rows.append({"coll": "allreduce", "algo": algo, "ran": algo, "ctas": ctas, "unroll": 4, "bytes": nbytes,
                             "us": us + (0.5 if ctas == 16 else 0.0)})
    rows.append({"coll": "allreduce", "algo": "auto", "ran": "nvls", "ctas": 0, "bytes": 1 << 26, "us": 1.0})        # ignored
    rows.append({"coll": "allreduce", "algo": "rabenseifner", "ran": "twoshot", "ctas": 64, "bytes": 1024, "us": 1.0})  # fell back: ignored
    rows.append({"coll": "allreduce", "algo": "nvls_sym", "ran": "nvls", "ctas": 16, "bytes": 1 << 26, "us": 100.0})
    f1 = tmp_path / "sweep.json"
    f1.write_text(json.dumps({"n_gpus": 8, "impl": "ours", "rows": rows}))
    f2 = tmp_path / "ctool.json"
    f2.write_text(json.dumps({"n_gpus": 8, "symmetric": False, "rows": [
        {"coll": "reduce_scatter", "impl": "dccl", "bytes": 1 << 20, "us": 30.0, "variant": "twoshot"},
        {"coll": "reduce_scatter", "impl": "nccl", "bytes": 1 << 20, "us": 1.0, "variant": "nccl"}]}))
    out = tmp_path / "tune.txt"
    subprocess.run([sys.executable, os.path.join(root, "benchmarks", "make_tune_table.py"), "--in", str(f1), "--in", str(f2) + ":128",
                    "--out", str(out)], check=True)
    text = out.read_text()
    assert "allreduce 8 65536 oneshot 64" in text and "allreduce 8 inf nvls 64" in text
    assert "allreduce_sym 8 inf nvls 16" in text and "reducescatter 8 inf twoshot 128" in text
    assert dccl_lib.dccl_tuner_load_text(text.encode()) == 4
    algo = ctypes.create_string_buffer(32)
    ctas = ctypes.c_int()
    for nbytes, want in [(512, b"oneshot"), (65536, b"oneshot"), (65537, b"nvls"), (1 << 30, b"nvls")]:
        assert dccl_lib.dccl_tuner_choose(b"allreduce", 8, nbytes, 1, algo, 32, ctypes.byref(ctas)) == 0
        assert algo.value == want, (nbytes, algo.value)
    assert dccl_lib.dccl_tuner_choose(b"reducescatter", 8, 1 << 28, 1, algo, 32, ctypes.byref(ctas)) == 0 and (algo.value, ctas.value) == (b"twoshot", 128)


def test_launcher_command_line():
    """python -m dccl_b200.utils.launch: one process per rank, rank-tagged output, worst exit code."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "dccl_b200.utils.launch", "-n", "3", "--", "/bin/sh", "-c", "echo rank $DCCL_RANK of $DCCL_WORLD_SIZE"],
                       cwd=root, capture_output=True, text=True, timeout=60)
    assert p.returncode == 0, p.stderr
    assert sorted(p.stdout.split("\n")[:3]) == ["[0] rank 0 of 3", "[1] rank 1 of 3", "[2] rank 2 of 3"]
    p = subprocess.run([sys.executable, "-m", "dccl_b200.utils.launch", "-n", "2", "--", "/bin/sh", "-c", "exit $DCCL_RANK"],
                       cwd=root, capture_output=True, text=True, timeout=60)
    assert p.returncode == 1


def test_nvlink_report_against_a_fake_nvml(dccl_lib, tmp_path):
    """The NVML side of the topology discovery (read-only queries, library loaded at run time) against tests/fakes/fake_nvml.c."""
    import json
    import subprocess
    if not hasattr(dccl_lib, "dccl_nvml_link_report"):
        pytest.skip("host-only build")
    here = os.path.dirname(os.path.abspath(__file__))
    so = str(tmp_path / "libfake_nvml.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", so, os.path.join(here, "fakes", "fake_nvml.c")], check=True)
    buf = ctypes.create_string_buffer(4096)
    assert dccl_lib.dccl_nvml_link_report(so.encode(), buf, len(buf)) == 0, buf.value
    rep = json.loads(buf.value.decode())
    assert [g["nvlinks_active"] for g in rep["gpus"]] == [18, 17]
    assert [g["nvlinks_to_switch"] for g in rep["gpus"]] == [18, 17]
    assert rep["gpus"][0]["name"] == "Fake B200 #0" and rep["gpus"][1]["nvlink_version"] == 7
    # a library that is not there is an answer, not a crash
    assert dccl_lib.dccl_nvml_link_report(str(tmp_path / "missing.so").encode(), buf, len(buf)) == -1
    assert b"cannot load" in buf.value


def test_topology_tool_without_a_gpu(build_dir, tmp_path):
    """dccl_topo on a machine without a usable driver: an empty table, and the NVML view through the fake library."""
    import json
    import subprocess
    tool = os.path.join(build_dir, "dccl_topo")
    if not os.path.exists(tool):
        pytest.skip("host-only build")
    from conftest import gpu_count
    out = json.loads(subprocess.run([tool], capture_output=True, text=True, timeout=60, check=True).stdout)
    if gpu_count() == 0:
        assert out["summary"] == "no CUDA devices" and out["topology"]["nranks"] == 0
    else:
        assert out["topology"]["nranks"] == min(gpu_count(), 8)
    here = os.path.dirname(os.path.abspath(__file__))
    so = str(tmp_path / "libfake_nvml.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", so, os.path.join(here, "fakes", "fake_nvml.c")], check=True)
    rep = json.loads(subprocess.run([tool, "--nvml", so], capture_output=True, text=True, timeout=60, check=True).stdout)
    assert len(rep["gpus"]) == 2 and rep["gpus"][1]["nvlinks_active"] == 17


def test_guard_words_of_the_pool_layout(dccl_lib):
    """The guard words between the regions of a device pool, exercised on a host buffer with the same layout: intact
    after filling, a damaged byte right after each region (and right before the staging area) is named with its
    gap and offset, and writes that stay inside the regions never disturb them."""
    if not hasattr(dccl_lib, "dccl_selftest_canary"):
        pytest.skip("host-only build")
    assert dccl_lib.dccl_selftest_canary() == 0
    # the library the package ships is the normal build: range checks are compiled out
    assert dccl_lib.dccl_debug_bounds_build() == 0
    assert dccl_lib.dccl_emu_declare_stage_bytes(1 << 16) == -1


def test_profile_summary_from_a_raw_page():
    """benchmarks/ncu_summary.py on a hand-made raw page: metric rows in a fixed order, the three largest stalls."""
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("ncu_summary", os.path.join(root, "benchmarks", "ncu_summary.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    pre = "smsp__average_warps_issue_stalled_"
    post = "_per_issue_active.ratio"
    names = ["ID", "Kernel Name", "gpu__time_duration.sum", "dram__bytes_read.sum", "launch__registers_per_thread",
             pre + "long_scoreboard" + post, pre + "barrier" + post, pre + "wait" + post, pre + "membar" + post, "other__metric"]
    units = ["", "", "us", "Mbyte", "register/thread", "inst", "inst", "inst", "inst", ""]
    row = ["0", "k_direct<float, 0>(CollArgs)", "12.5", "64.0", "96", "30.1", "4.5", "1.25", "9.75", "7"]
    text = "==PROF== banner line\n" + "\n".join(",".join('"%s"' % v for v in r) for r in (names, units, row)) + "\n"
    launches = mod.parse_csv(text)
    assert len(launches) == 1 and launches[0][0].startswith("k_direct")
    lines = mod.summary_lines(launches[0][1])
    assert [l[0] for l in lines[:3]] == ["gpu__time_duration.sum", "dram__bytes_read.sum", "launch__registers_per_thread"]
    assert [l[0] for l in lines[3:]] == [pre + s + post for s in ("long_scoreboard", "membar", "barrier")]
    assert lines[0][1:] == ("12.5", "us")


def test_committed_table_file_is_the_built_in_table(tmp_path):
    """cfg/tune_b200_nvswitch.txt is what `make_tune_table.py --builtin` writes (a fresh process: no test has touched the
    table), and loading it over the built-in table changes no choice."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = {k: v for k, v in os.environ.items() if k != "DCCL_TUNE_FILE"}
    p = subprocess.run([sys.executable, os.path.join(root, "benchmarks", "make_tune_table.py"), "--builtin"], capture_output=True, text=True,
                       env=env, check=True)
    committed = open(os.path.join(root, "cfg", "tune_b200_nvswitch.txt")).read()
    assert p.stdout == committed
    rules = [line for line in committed.splitlines() if line and not line.startswith("#")]
    assert len(rules) >= 30 and all(len(r.split()) in (5, 6) for r in rules)
    code = ("import ctypes, sys\n"
            "from dccl_b200._lib import lib\n"
            "L = lib()\n"
            "def pick(coll, n, b, w):\n"
            "    a = ctypes.create_string_buffer(32); c = ctypes.c_int()\n"
            "    assert L.dccl_tuner_choose_width(coll, n, b, 1, w, a, 32, ctypes.byref(c)) == 0\n"
            "    return a.value, c.value\n"
            "grid = [(coll, n, 1 << s, w) for coll in [b'allreduce', b'allreduce_sym', b'reducescatter', b'reducescatter_sym', b'allgather', b'broadcast', b'reduce']\n"
            "        for n in (2, 3, 4, 8) for s in range(2, 31, 2) for w in (1, 2, 4, 8)]\n"
            "before = [pick(*g) for g in grid]\n"
            "assert L.dccl_tuner_load_text(open(sys.argv[1]).read().encode()) >= 30\n"
            "assert [pick(*g) for g in grid] == before\n"
            "print('same')\n")
    q = subprocess.run([sys.executable, "-c", code, os.path.join(root, "cfg", "tune_b200_nvswitch.txt")], capture_output=True, text=True, env=env, cwd=root)
    assert q.returncode == 0 and "same" in q.stdout, q.stdout + q.stderr


def test_table_dump_round_trips_rules_with_an_element_width(dccl_lib):
    """A rule bound to an element width comes back out of the dump in the file format, and the dump loads again."""
    assert dccl_lib.dccl_tuner_load_text(b"broadcast 8 3m twoshot 24 2\nbroadcast * inf nvls 48\n") == 2
    n = dccl_lib.dccl_tuner_dump(None, 0)
    buf = ctypes.create_string_buffer(n + 1)
    dccl_lib.dccl_tuner_dump(buf, n + 1)
    lines = buf.value.decode().splitlines()
    assert "broadcast 8 3m twoshot 24 2" in lines and "broadcast * inf nvls 48" in lines
    assert dccl_lib.dccl_tuner_load_text(buf.value) == len(lines)
    buf2 = ctypes.create_string_buffer(n + 1)
    dccl_lib.dccl_tuner_dump(buf2, n + 1)
    assert buf2.value == buf.value
