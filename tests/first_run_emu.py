"""Single-GPU emulation tests of paths that have not run on hardware yet. Not collected by name: they are run in a child
process by tests/test_gpu_emu.py::test_paths_not_yet_run_on_hardware_in_a_child_process, and move into that file after
their first clean run."""
import numpy as np
import pytest

from dccl_b200.utils import oracle
from test_gpu_emu import close, emu, inputs_for, np_dtype

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [2, 4, 8])
def test_ring_kernel_adds_in_ring_order(dccl_lib, n):
    """fp32 sum through the ring kernel against a fold in the order the ring adds, shard by shard (shards are whole
    16-byte vectors): the bits must match."""
    for count in [1, 3, 257, 4096, 10007, 65536 + 5]:
        ins = inputs_for("float32", "sum", count, n, seed=count % 89)
        out = emu(dccl_lib, "allreduce", "ring", n, "float32", "sum", count, ins)
        assert np.array_equal(out[0], oracle.ring_fold_sum(ins, align=4)), (n, count)


@pytest.mark.parametrize("n", [2, 3, 8])
def test_two_shot_packet_all_reduce(dccl_lib, n):
    """Shards to their owners and folded shards to everybody, both as polled packets (no barrier); up to 256 KB per shard."""
    for name in ["float32", "bfloat16", "int8", "float64"]:
        cap = (n * (256 << 10)) // np.dtype(np_dtype(name)).itemsize       # 256 KB per shard
        for count in [c for c in [1, 9, 4099, 65536 + 5, cap] if c <= cap]:
            for op in ["sum", "avg", "max"]:
                ins = inputs_for(name, op, count, n, seed=53)
                want = oracle.fold(ins, op, bf16=name == "bfloat16")
                for in_place, misalign in [(0, 0), (1, 0), (0, 4)]:
                    out = emu(dccl_lib, "allreduce", "twoshot_ll", n, name, op, count, ins, in_place=in_place, misalign=misalign, iters=4, ctas=6)
                    for r in range(n):
                        assert close(out[r], want, name, n), (n, name, op, count, r, in_place, misalign)
                    for r in range(1, n):
                        assert np.array_equal(out[r], out[0]), (n, name, op, count, "ranks differ")
    # the same kernel as a reduce: folded shards go to the root only
    for root in {0, n - 1}:
        for count in [1, 5, 4099, 65536 + 5]:
            ins = inputs_for("float32", "sum", count, n, seed=59)
            for op in ["sum", "avg"]:
                out = emu(dccl_lib, "reduce", "twoshot_ll", n, "float32", op, count, ins, root=root, iters=4, ctas=6)
                assert close(out[root], oracle.fold(ins, op), "float32", n), ("reduce", n, root, count, op)


def _capacity_fp32(algo, kind, n, stage):
    """Largest fp32 count the staged variants take with `stage` bytes per staging half (whole 16-byte vectors)."""
    elems, fl = stage // 4, lambda v: v // 4 * 4
    if algo == "ring":
        return n * fl(elems // (2 * n)) if kind == "allreduce" else fl(elems // (2 * n))
    if algo == "rabenseifner":
        return fl(elems // (n.bit_length()))                      # log2(n) + 1 areas for a power of two
    if kind in ("allreduce", "reduce"):
        return n * fl(elems // (n + 1))
    if kind == "reducescatter":
        return fl(elems // (n + 1))
    return fl(elems) if kind == "allgather" else n * fl(elems)


def test_guard_words_between_the_pool_regions_stay_intact(dccl_lib):
    """Every emulated variant at the largest message its region takes (and at a small one), with guard words in the
    unused parts of every pool: the harness returns 200 + gap when a run damaged them."""
    n, stage = 8, 1 << 20
    ll_cap = (128 << 10) // 4
    cases = [("allreduce", "oneshot", ll_cap), ("reducescatter", "oneshot", ll_cap), ("allgather", "oneshot", ll_cap),
             ("broadcast", "oneshot", ll_cap), ("reduce", "oneshot", ll_cap),
             ("allreduce", "twoshot_ll", n * (256 << 10) // 4), ("reduce", "twoshot_ll", n * (256 << 10) // 4)]
    for kind in ["allreduce", "reducescatter", "allgather", "broadcast", "reduce"]:
        for algo in ["twoshot", "ring", "rabenseifner"]:
            if algo == "rabenseifner" and kind != "allreduce" or algo == "ring" and kind in ("broadcast", "reduce"):
                continue
            cases.append((kind, algo, _capacity_fp32(algo, kind, n, stage)))
    dccl_lib.dccl_emu_set_guard(1)
    try:
        for kind, algo, cap in cases:
            for count in [5, cap]:
                in_count = count * n if kind == "reducescatter" else count
                ins = inputs_for("float32", "sum", in_count, n, seed=61)
                out = emu(dccl_lib, kind, algo, n, "float32", "sum", count, ins, root=n - 1, iters=2, stage=stage)
                want = oracle.fold(ins, "sum")
                if kind == "allreduce":
                    assert close(out[0], want, "float32", n), (kind, algo, count)
                elif kind == "reduce":
                    assert close(out[n - 1], want, "float32", n), (kind, algo, count)
        # grouped send / recv: two messages per peer, each longer than the FIFO and ending in a short chunk
        W, nbytes = 2, (4 << 20) + 4096
        hin = np.random.default_rng(5).integers(0, 255, size=n * W * nbytes, dtype=np.uint8)
        hout = np.zeros_like(hin)
        rc = dccl_lib.dccl_emu_sendrecv_ring(n, nbytes, W, 4, 2, hin.ctypes.data, hout.ctypes.data)
        assert rc == 0, rc
        got, sent = hout.reshape(n, W * nbytes), hin.reshape(n, W * nbytes)
        for r in range(n):
            assert np.array_equal(got[r], sent[(r - 1) % n]), r
    finally:
        dccl_lib.dccl_emu_set_guard(0)


def test_range_checking_build_refuses_before_it_touches_memory():
    """The library compiled with its range checks (make BOUNDS=1), in a process of its own: normal runs pass, and a
    run that is told a smaller staging area than its message needs comes back with the bounds code."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "build-bounds", "libdccl.so")
    if not os.path.exists(path):
        pytest.skip("build-bounds/libdccl.so is not built (make BOUNDS=1 lib)")
    env = dict(os.environ, DCCL_LIBRARY=path)
    probe = subprocess.run([sys.executable, "-c", "import sys; sys.path.insert(0, %r); from dccl_b200 import _lib; _lib.lib()" % root],
                           env=env, capture_output=True, text=True, timeout=300)
    if probe.returncode != 0:
        pytest.skip("build-bounds/libdccl.so does not match the bindings (rebuild it: make BOUNDS=1 lib)")
    p = subprocess.run([sys.executable, os.path.join(root, "tests", "workers", "bounds_worker.py")], env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "bounds worker: ok" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]


def test_all_reduce_after_other_kernels_in_the_same_world(dccl_lib):
    """Two other collectives run before every call under test, in the same virtual world and on the same buffers
    (dccl_emu_set_mix): rooted packet kernels between all-reduces, staged forms between packet forms. What they leave in
    flags, packet generations and staging halves is what the next kernel starts from."""
    import itertools
    pre = ["allreduce:oneshot", "broadcast:oneshot", "reduce:oneshot", "reducescatter:oneshot", "allgather:oneshot", "allreduce:twoshot_ll",
           "reduce:twoshot_ll", "allreduce:twoshot", "broadcast:twoshot", "reduce:twoshot", "allreduce:ring", "allreduce:rabenseifner"]
    n, count = 4, 1031
    try:
        for a, b in itertools.product(pre, pre):
            assert dccl_lib.dccl_emu_set_mix((a + "," + b).encode()) == 2
            for algo in ["oneshot", "twoshot_ll", "twoshot"]:
                ins = inputs_for("float32", "sum", count, n, seed=5)
                out = emu(dccl_lib, "allreduce", algo, n, "float32", "sum", count, ins, root=1, iters=3)
                want = oracle.fold(ins, "sum")
                for r in range(n):
                    assert close(out[r], want, "float32", n), ("after", a, b, algo, r)
    finally:
        dccl_lib.dccl_emu_set_mix(b"")


@pytest.mark.parametrize("n,ctas", [(2, 4), (4, 4), (8, 2), (5, 10)])
def test_all_to_all_as_grouped_send_recv(dccl_lib, n, ctas):
    """The launch the library composes for an all-to-all: every rank's receives from rank - k, then its sends to rank + k,
    in one launch, three times in a row; blocks shorter and longer than the FIFO, the last chunk short."""
    for nbytes in [4, 1000, 65536 + 8, (1 << 20) + 24, (5 << 20) + 8]:
        hin = np.random.default_rng(nbytes + n).integers(0, 255, size=n * n * nbytes, dtype=np.uint8)
        hout = np.zeros_like(hin)
        rc = dccl_lib.dccl_emu_all_to_all(n, nbytes, ctas, 3, hin.ctypes.data, hout.ctypes.data)
        assert rc == 0, (n, nbytes, rc)
        src, got = hin.reshape(n, n, nbytes), hout.reshape(n, n, nbytes)
        for r in range(n):
            for p in range(n):
                assert np.array_equal(got[r, p], src[p, r]), (n, nbytes, r, p)
