"""Device kernels against the serial fold, all ranks emulated on ONE GPU.

One cooperative launch plays every rank (see csrc/gpu/emu.cu), so the flag protocol, staging halves,
packet generations and the reductions are the code that runs on a multi-GPU box. Each case runs
three calls back to back, which exercises the reuse of both staging halves / packet generations.
"""
import ctypes
import os

import numpy as np
import pytest

from dccl_b200.comm import DTYPE_NAMES, OPS
from dccl_b200.utils import oracle

pytestmark = pytest.mark.gpu

FLOATS = ["float16", "float32", "float64", "bfloat16"]


def np_dtype(name):
    return np.uint16 if name == "bfloat16" else np.dtype(name)


def inputs_for(name, op, count, n, seed):
    ins = [oracle.make_input(name, count, seed=seed * 100 + r) for r in range(n)]
    if op == "prod" and name in FLOATS:   # keep products in range
        if name == "bfloat16":
            ins = [oracle.f32_to_bf16(np.where(np.abs(oracle.bf16_to_f32(x)) < 0.5, 1.0, 1.25).astype(np.float32)) for x in ins]
        else:
            ins = [np.where(np.abs(x) < 0.5, 1.0, 1.25).astype(name) for x in ins]
    return ins


def close(got, want, name, world):
    rtol, atol = oracle.tolerances(name, world)
    if rtol == 0.0:
        return np.array_equal(got, want)
    if name == "bfloat16":
        got, want = oracle.bf16_to_f32(got), oracle.bf16_to_f32(want)
    return np.allclose(got.astype(np.float64), want.astype(np.float64), rtol=rtol, atol=atol)


def emu(lib, kind, algo, n, name, op, count, ins, root=0, ctas=3, in_place=0, misalign=0, iters=3, stage=0):
    dt = DTYPE_NAMES.index(name)
    es = np_dtype(name).itemsize if name != "bfloat16" else 2
    in_elems = count * n if kind == "reducescatter" else count
    out_elems = count * n if kind == "allgather" else count
    hin = np.concatenate(ins).astype(np_dtype(name), copy=False)
    assert hin.size == in_elems * n
    hout = np.zeros(out_elems * n, dtype=np_dtype(name))
    rc = lib.dccl_emu_collective(kind.encode(), algo.encode(), n, dt, OPS[op], count, root, ctas, in_place, misalign, iters,
                                 stage, hin.ctypes.data, hout.ctypes.data)
    assert rc == 0, "emulation returned %d" % rc
    assert es * out_elems * n == hout.nbytes
    return hout.reshape(n, out_elems)


@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "ring", "rabenseifner"])
@pytest.mark.parametrize("n", [2, 4, 8])
def test_allreduce_fp32_bf16_sizes(dccl_lib, algo, n):
    for name in ["float32", "bfloat16"]:
        for count in [1, 3, 257, 4096, 10007, 65536 + 5]:
            if algo == "oneshot" and count * (4 if name == "float32" else 2) > 128 * 1024:
                continue
            for op in ["sum", "avg"]:
                ins = inputs_for(name, op, count, n, seed=count % 89)
                want = oracle.fold(ins, op, bf16=name == "bfloat16")
                out = emu(dccl_lib, "allreduce", algo, n, name, op, count, ins)
                for r in range(n):
                    assert close(out[r], want, name, n), (algo, n, name, op, count, r)
                # all ranks must hold the same bits
                for r in range(1, n):
                    assert np.array_equal(out[r], out[0]), (algo, n, name, op, count, "ranks differ")


@pytest.mark.parametrize("n", [3, 5, 6, 7])
def test_rabenseifner_on_worlds_that_are_not_a_power_of_two(dccl_lib, n):
    """n = 2^m + r: the first 2r ranks pair up (the odd one hands its vector to the even one and gets the result back),
    the rest run the halving and doubling steps on 2^m ranks. Every rank must end with the same bits, at the largest
    count the staging takes too."""
    stage = 1 << 20
    cap = _capacity_fp32("rabenseifner", "allreduce", n, stage)
    for name, op, count, in_place, misalign in [("float32", "sum", 1, 0, 0), ("float32", "avg", 10007, 0, 4), ("bfloat16", "sum", 65536 + 5, 1, 0),
                                                ("int32", "max", 4099, 0, 0), ("float64", "prod", 257, 1, 8), ("float32", "sum", cap, 0, 0)]:
        ins = inputs_for(name, op, count, n, seed=71 + n)
        want = oracle.fold(ins, op, bf16=name == "bfloat16")
        out = emu(dccl_lib, "allreduce", "rabenseifner", n, name, op, count, ins, in_place=in_place, misalign=misalign, iters=3, stage=stage)
        for r in range(n):
            assert close(out[r], want, name, n), (n, name, op, count, r)
        for r in range(1, n):
            assert np.array_equal(out[r], out[0]), (n, name, op, count, "ranks differ")


@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "ring", "rabenseifner"])
def test_allreduce_every_dtype_and_operator(dccl_lib, algo):
    n, count = 4, 1031
    for name in DTYPE_NAMES:
        for op in ["sum", "prod", "max", "min", "avg"]:
            ins = inputs_for(name, op, count, n, seed=7)
            want = oracle.fold(ins, op, bf16=name == "bfloat16")
            out = emu(dccl_lib, "allreduce", algo, n, name, op, count, ins)
            for r in range(n):
                assert close(out[r], want, name, n), (algo, name, op, r)


@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "ring", "rabenseifner", "twoshot_ll"])
def test_min_max_ignore_a_nan_when_a_number_is_there(dccl_lib, algo):
    """max / min of floats follow IEEE maxNum / minNum (fmax / fmin, as NCCL's kernels do): whichever rank holds the NaN
    and in whatever order the values meet, the number wins; only an element that is NaN on every rank stays NaN."""
    n, count = 4, 2053
    for name in ["float32", "bfloat16", "float16", "float64"]:
        ins = inputs_for(name, "max", count, n, seed=19)
        nan = np.uint16(0x7FC0) if name == "bfloat16" else np.nan
        for r in range(n):
            ins[r][r::7] = nan                  # a different pattern per rank ...
        for r in range(n):
            ins[r][5::101] = nan                # ... and some elements that are NaN everywhere
        for op in ["max", "min"]:
            want = oracle.fold(ins, op, bf16=name == "bfloat16")
            wf = oracle.bf16_to_f32(want) if name == "bfloat16" else want
            assert np.isnan(wf[5::101]).all() and not np.isnan(np.delete(wf, np.arange(5, count, 101))).any()
            out = emu(dccl_lib, "allreduce", algo, n, name, op, count, ins)
            for r in range(n):
                got = oracle.bf16_to_f32(out[r]) if name == "bfloat16" else out[r]
                assert np.array_equal(np.isnan(got), np.isnan(wf)), (algo, name, op, r)
                assert np.array_equal(got[~np.isnan(wf)], wf[~np.isnan(wf)]), (algo, name, op, r)


@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "ring", "rabenseifner"])
def test_allreduce_in_place_and_unaligned(dccl_lib, algo):
    n = 4
    for name, misalign in [("float32", 4), ("bfloat16", 2), ("float32", 0), ("int8", 1), ("float64", 8)]:
        for in_place in [0, 1]:
            count = 5003
            ins = inputs_for(name, "sum", count, n, seed=3)
            want = oracle.fold(ins, "sum", bf16=name == "bfloat16")
            out = emu(dccl_lib, "allreduce", algo, n, name, "sum", count, ins, in_place=in_place, misalign=misalign)
            for r in range(n):
                assert close(out[r], want, name, n), (algo, name, misalign, in_place, r)


@pytest.mark.parametrize("algo", ["twoshot", "ring", "oneshot"])
@pytest.mark.parametrize("n", [2, 3, 8])
def test_reduce_scatter_and_all_gather(dccl_lib, algo, n):
    for name in ["float32", "bfloat16", "int32", "float16"]:
        for count in [1, 256, 1000, 4097]:
            for op in ["sum", "max", "min", "avg"]:
                ins = inputs_for(name, op, count * n, n, seed=11)
                want = oracle.fold(ins, op, bf16=name == "bfloat16")
                for in_place in [0, 1]:
                    out = emu(dccl_lib, "reducescatter", algo, n, name, op, count, ins, in_place=in_place)
                    for r in range(n):
                        assert close(out[r], want[r * count:(r + 1) * count], name, n), ("rs", algo, n, name, op, count, r, in_place)
            ins = inputs_for(name, "sum", count, n, seed=13)
            for in_place in [0, 1]:
                out = emu(dccl_lib, "allgather", algo, n, name, "sum", count, ins, in_place=in_place)
                for r in range(n):
                    assert np.array_equal(out[r], np.concatenate(ins)), ("ag", algo, n, name, count, r, in_place)


@pytest.mark.parametrize("n", [2, 5, 8])
def test_broadcast_and_reduce_roots(dccl_lib, n):
    for root in {0, n - 1}:
        for count in [1, 4, 1000, 70001]:
            ins = inputs_for("float32", "sum", count, n, seed=17)
            for algo in ["oneshot", "twoshot"]:
                out = emu(dccl_lib, "broadcast", algo, n, "float32", "sum", count, ins, root=root, in_place=1)
                for r in range(n):
                    assert np.array_equal(out[r], ins[root]), ("bcast", algo, n, root, count, r)
            for op in ["sum", "avg", "max"]:
                want = oracle.fold(ins, op)
                for algo in ["twoshot", "oneshot"]:     # oneshot: packets up to 128 KB, else the staged variant
                    out = emu(dccl_lib, "reduce", algo if count * 4 <= 128 * 1024 else "twoshot", n, "float32", op, count, ins, root=root)
                    assert close(out[root], want, "float32", n), ("reduce", algo, n, root, count, op)


def test_many_ctas_and_small_staging(dccl_lib):
    """More CTAs than vectors, and a staging half barely larger than the message."""
    n = 8
    for ctas in [1, 7, 16]:
        for count in [5, 20000]:
            ins = inputs_for("float32", "sum", count, n, seed=ctas)
            want = oracle.fold(ins, "sum")
            for algo in ["twoshot", "ring", "rabenseifner"]:
                out = emu(dccl_lib, "allreduce", algo, n, "float32", "sum", count, ins, ctas=ctas, stage=1 << 20)
                for r in range(n):
                    assert close(out[r], want, "float32", n), (algo, ctas, count, r)


def test_send_recv_ring(dccl_lib):
    for n, window in [(2, 1), (8, 1), (2, 4), (4, 3)]:
        # window > 1: several operations of one launch address the same peer (each works on its own FIFO slot)
        for nbytes in [4, 1000, (1 << 20) + 24, 5 * (1 << 20) + 8]:   # the last one is longer than the FIFO: needs flow control
            if window > 1 and nbytes > (2 << 20):
                continue
            rng = np.random.default_rng(nbytes)
            hin = rng.integers(0, 256, n * window * nbytes, dtype=np.uint8)
            hout = np.zeros_like(hin)
            rc = dccl_lib.dccl_emu_sendrecv_ring(n, nbytes, window, 4, 3, hin.ctypes.data, hout.ctypes.data)
            assert rc == 0
            hin, hout = hin.reshape(n, window * nbytes), hout.reshape(n, window * nbytes)
            for r in range(n):
                assert np.array_equal(hout[r], hin[(r - 1) % n]), (n, window, nbytes, r)


def test_local_reduce_every_dtype_and_operator(dccl_lib):
    count = 100003
    for name in DTYPE_NAMES:
        for op in ["sum", "prod", "max", "min"]:
            a, b = inputs_for(name, op, count, 2, seed=23)
            want = oracle.fold([a, b], op, bf16=name == "bfloat16")
            acc = a.copy()
            rc = dccl_lib.dccl_local_reduce(acc.ctypes.data, b.ctypes.data, count, DTYPE_NAMES.index(name), OPS[op])
            assert rc == 0 and close(acc, want, name, 2), (name, op)


def test_bounded_wait_returns_a_status(dccl_lib):
    """A wait on a flag that nothing sets ends by itself with a timeout status; the context stays usable."""
    ms = ctypes.c_float()
    code = dccl_lib.dccl_emu_wait_probe(50, ctypes.byref(ms))
    assert code == 1, "expected the timeout status, got %d" % code
    assert 40.0 <= ms.value < 2000.0
    # the device still works
    a = np.ones(1000, dtype=np.float32)
    b = np.ones(1000, dtype=np.float32)
    assert dccl_lib.dccl_local_reduce(a.ctypes.data, b.ctypes.data, 1000, 7, 0) == 0 and np.all(a == 2.0)


def test_large_reduce_scatter_overlaps_push_and_reduce(dccl_lib):
    """Ranges above 512 KB per CTA take the pipelined path (pieces pushed ahead of the fold)."""
    for n, count, ctas in [(4, (1 << 20) + 7, 3), (8, 300000, 1), (2, (2 << 20) + 3, 2)]:
        for name, op in [("float32", "sum"), ("bfloat16", "avg"), ("int32", "max")]:
            ins = inputs_for(name, op, count * n, n, seed=29)
            want = oracle.fold(ins, op, bf16=name == "bfloat16")
            for in_place in [0, 1]:
                out = emu(dccl_lib, "reducescatter", "twoshot", n, name, op, count, ins, ctas=ctas, in_place=in_place, stage=96 << 20)
                for r in range(n):
                    assert close(out[r], want[r * count:(r + 1) * count], name, n), (n, count, name, op, r, in_place)


def test_sequence_number_kept_on_the_device(dccl_lib):
    """With the device-side counter, a launch carries no usable sequence number (as when a CUDA graph
    replays it); every variant must still run call after call, alternating staging halves."""
    dccl_lib.dccl_emu_set_device_seq(1)
    try:
        for n in [2, 8]:
            for count in [5, 4099, 70001]:
                ins = inputs_for("bfloat16", "avg", count, n, seed=31)
                want = oracle.fold(ins, "avg", bf16=True)
                for algo in ["oneshot", "twoshot", "ring", "rabenseifner"]:
                    if algo == "oneshot" and count * 2 > 128 * 1024:
                        continue
                    out = emu(dccl_lib, "allreduce", algo, n, "bfloat16", "avg", count, ins, iters=5, ctas=4)
                    for r in range(n):
                        assert close(out[r], want, "bfloat16", n), ("allreduce", algo, n, count, r)
                ins = inputs_for("float32", "sum", count * n, n, seed=37)
                want = oracle.fold(ins, "sum")
                for algo in ["oneshot", "twoshot", "ring"]:
                    if algo == "oneshot" and count * 4 > 128 * 1024:
                        continue
                    out = emu(dccl_lib, "reducescatter", algo, n, "float32", "sum", count, ins, iters=4)
                    for r in range(n):
                        assert close(out[r], want[r * count:(r + 1) * count], "float32", n), ("rs", algo, n, count, r)
                ins = inputs_for("float32", "sum", count, n, seed=41)
                for algo in ["oneshot", "twoshot"]:
                    out = emu(dccl_lib, "allgather", algo if count * 4 <= 128 * 1024 else "twoshot", n, "float32", "sum", count, ins, iters=4)
                    for r in range(n):
                        assert np.array_equal(out[r], np.concatenate(ins)), ("ag", algo, n, count, r)
                    out = emu(dccl_lib, "broadcast", algo, n, "float32", "sum", count, ins, root=n - 1, in_place=1, iters=4)
                    for r in range(n):
                        assert np.array_equal(out[r], ins[n - 1]), ("bcast", algo, n, count, r)
    finally:
        dccl_lib.dccl_emu_set_device_seq(0)


def test_zero_copy_two_shot_on_peer_addressable_buffers(dccl_lib):
    """Buffers that every rank can address are folded straight out of / into the user memory."""
    dccl_lib.dccl_emu_set_peer_buffers(1)
    try:
        for n in [2, 3, 4, 8]:
            for name in ["bfloat16", "float32", "int32", "float64", "uint8"]:
                for count in [1, 7, 4096, 100003, (1 << 20) + 24]:
                    for op in ["sum", "avg", "min"]:
                        ins = inputs_for(name, op, count, n, seed=43)
                        want = oracle.fold(ins, op, bf16=name == "bfloat16")
                        for in_place in [0, 1]:
                            out = emu(dccl_lib, "allreduce", "twoshot", n, name, op, count, ins, in_place=in_place, ctas=5)
                            for r in range(n):
                                assert close(out[r], want, name, n), (n, name, count, op, r, in_place)
                            for r in range(1, n):
                                assert np.array_equal(out[r], out[0]), (n, name, count, op, "ranks differ")
            # reduce-scatter: slot r of every send buffer folded into rank r's receive buffer (whole vectors per slot)
            for name in ["bfloat16", "float32", "int64"]:
                for count in [16, 4096, 100000, (1 << 19) + 64]:
                    for op in ["sum", "avg", "max"]:
                        ins = inputs_for(name, op, count * n, n, seed=47)
                        want = oracle.fold(ins, op, bf16=name == "bfloat16")
                        for in_place in [0, 1]:
                            out = emu(dccl_lib, "reducescatter", "twoshot", n, name, op, count, ins, in_place=in_place, ctas=5)
                            for r in range(n):
                                assert close(out[r], want[r * count:(r + 1) * count], name, n), ("rs", n, name, count, op, r, in_place)
    finally:
        dccl_lib.dccl_emu_set_peer_buffers(0)


@pytest.mark.parametrize("n", [2, 3, 5, 8])
def test_zero_copy_broadcast_and_reduce_on_peer_addressable_buffers(dccl_lib, n):
    """Broadcast as a pipelined scatter and all-gather by peer loads (every chunk count from one to more chunks than the
    shard has vectors), reduce with one shard per rank other than the root folded into the root's buffer; every root."""
    dccl_lib.dccl_emu_set_peer_buffers(1)
    try:
        for root in sorted({0, 1, n - 1}):
            for chunks in [1, 2, 5, 24]:
                dccl_lib.dccl_emu_set_bcast_chunks(chunks)
                for name, count in [("uint8", 1), ("uint8", 4099), ("float32", 16), ("bfloat16", 100003), ("float32", (1 << 18) + 4), ("float64", 777)]:
                    ins = inputs_for(name, "sum", count, n, seed=83 + root)
                    for in_place in [0, 1]:
                        out = emu(dccl_lib, "broadcast", "twoshot", n, name, "sum", count, ins, root=root, in_place=in_place, ctas=5, iters=3)
                        for r in range(n):
                            assert np.array_equal(out[r], ins[root]), ("bcast", n, root, chunks, name, count, r, in_place)
            dccl_lib.dccl_emu_set_bcast_chunks(0)
            for name in ["bfloat16", "float32", "int32", "float64"]:
                for count in [1, 7, 4096, 100003, (1 << 19) + 24]:
                    for op in ["sum", "avg", "max"]:
                        ins = inputs_for(name, op, count, n, seed=89)
                        want = oracle.fold(ins, op, bf16=name == "bfloat16")
                        for in_place in [0, 1]:
                            out = emu(dccl_lib, "reduce", "twoshot", n, name, op, count, ins, root=root, in_place=in_place, ctas=5)
                            assert close(out[root], want, name, n), ("reduce", n, root, name, count, op, in_place)
    finally:
        dccl_lib.dccl_emu_set_bcast_chunks(0)
        dccl_lib.dccl_emu_set_peer_buffers(0)


def test_zero_copy_rooted_forms_and_odd_worlds_on_random_shapes(dccl_lib):
    """Forty shapes drawn with a fixed seed: world size, root, chunk count, grid, element count, type, in place or not.
    Every byte of a broadcast must arrive exactly once whatever the cut into shards, chunks, teams and CTA slices;
    the reduce and the halving-and-doubling all-reduce must match the serial fold."""
    rng = np.random.RandomState(20240607)
    dccl_lib.dccl_emu_set_peer_buffers(1)
    try:
        for case in range(40):
            n = int(rng.randint(2, 9))
            root = int(rng.randint(0, n))
            chunks = int(rng.choice([1, 2, 3, 7, 24]))
            ctas = int(rng.choice([1, 2, 3, 6]))
            name = str(rng.choice(["uint8", "bfloat16", "float32", "float64"]))
            count = int(rng.choice([1, 15, 16, 17, 1000, 4097, 70001, 300007]))
            in_place = int(rng.randint(0, 2))
            ins = inputs_for(name, "sum", count, n, seed=100 + case)
            dccl_lib.dccl_emu_set_bcast_chunks(chunks)
            out = emu(dccl_lib, "broadcast", "twoshot", n, name, "sum", count, ins, root=root, in_place=in_place, ctas=ctas, iters=2)
            for r in range(n):
                assert np.array_equal(out[r], ins[root]), ("bcast", case, n, root, chunks, ctas, name, count, in_place, r)
            if name != "uint8":
                op = str(rng.choice(["sum", "avg", "min"]))
                ins = inputs_for(name, op, count, n, seed=200 + case)
                want = oracle.fold(ins, op, bf16=name == "bfloat16")
                out = emu(dccl_lib, "reduce", "twoshot", n, name, op, count, ins, root=root, in_place=in_place, ctas=ctas, iters=2)
                assert close(out[root], want, name, n), ("reduce", case, n, root, ctas, name, count, op, in_place)
                out = emu(dccl_lib, "allreduce", "rabenseifner", n, name, op, count, ins, in_place=in_place, ctas=ctas, iters=2, stage=32 << 20)
                for r in range(n):
                    assert close(out[r], want, name, n), ("rabenseifner", case, n, ctas, name, count, op, in_place, r)
    finally:
        dccl_lib.dccl_emu_set_bcast_chunks(0)
        dccl_lib.dccl_emu_set_peer_buffers(0)


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
    """Shards to their owners and folded shards to everybody, both as polled packets (no barrier); up to 512 KB per shard."""
    for name in ["float32", "bfloat16", "int8", "float64"]:
        cap = (n * (512 << 10)) // np.dtype(np_dtype(name)).itemsize       # 512 KB per shard
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
        # log2(n) + 1 areas for a power of two, one more for the leader / follower pairs of any other world
        return fl(elems // (n.bit_length() + (1 if n & (n - 1) else 0)))
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
             ("allreduce", "twoshot_ll", n * (512 << 10) // 4), ("reduce", "twoshot_ll", n * (512 << 10) // 4)]
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


@pytest.mark.parametrize("n,ctas", [(2, 4), (4, 4), (8, 1), (5, 3)])
def test_all_to_all_as_grouped_send_recv(dccl_lib, n, ctas):
    """The launch the library composes for an all-to-all: every rank's receives from rank - k, then its sends to rank + k,
    in one launch, three times in a row; blocks shorter and longer than the FIFO, the last chunk short. One launch plays
    n ranks x 2 (n - 1) operations x ctas blocks, all of which must be resident at once on the one GPU (148 SMs, one
    block of this kernel per SM), which bounds the cases."""
    for nbytes in [4, 1000, 65536 + 8, (1 << 20) + 24, (5 << 20) + 8]:
        hin = np.random.default_rng(nbytes + n).integers(0, 255, size=n * n * nbytes, dtype=np.uint8)
        hout = np.zeros_like(hin)
        rc = dccl_lib.dccl_emu_all_to_all(n, nbytes, ctas, 3, hin.ctypes.data, hout.ctypes.data)
        assert rc == 0, (n, nbytes, rc)
        src, got = hin.reshape(n, n, nbytes), hout.reshape(n, n, nbytes)
        for r in range(n):
            for p in range(n):
                assert np.array_equal(got[r, p], src[p, r]), (n, nbytes, r, p)


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_large_send_recv_meet_first_and_go_zero_copy_where_mapped(dccl_lib, mode):
    """Messages of 512 KB and more are rendezvous messages: the receiver posts where its buffer lies, the sender stores
    straight into it when it has that memory mapped (mode 1), falls back to the FIFO when it has not (mode 2), and both
    happen in one launch (mode 3: only even ranks' buffers are mapped). Small messages between them keep using the FIFO,
    whose chunk numbers and credit must stay consistent across the direct messages; several rounds, windows of messages
    per peer, sizes that are not whole chunks."""
    dccl_lib.dccl_emu_set_p2p_rendezvous(mode)
    try:
        for n, window, ctas in [(2, 1, 4), (4, 2, 3), (8, 1, 2), (3, 3, 2)]:
            for nbytes in [(512 << 10), (1 << 20) + 40, (5 << 20) + 8, 1000]:
                if window > 1 and nbytes > (2 << 20):
                    continue
                hin = np.random.default_rng(nbytes + n + mode).integers(0, 256, n * window * nbytes, dtype=np.uint8)
                hout = np.zeros_like(hin)
                rc = dccl_lib.dccl_emu_sendrecv_ring(n, nbytes, window, ctas, 4, hin.ctypes.data, hout.ctypes.data)
                assert rc == 0, (mode, n, window, nbytes, rc)
                a, b = hin.reshape(n, window * nbytes), hout.reshape(n, window * nbytes)
                for r in range(n):
                    assert np.array_equal(b[r], a[(r - 1) % n]), (mode, n, window, nbytes, r)
        # the launch an all-to-all is made of: 2 (n - 1) operations per rank, more receive buffers than the table of mappings holds
        for n, ctas in [(4, 3), (8, 1)]:
            for nbytes in [(1 << 20) + 24, (600 << 10)]:
                hin = np.random.default_rng(nbytes + n).integers(0, 255, size=n * n * nbytes, dtype=np.uint8)
                hout = np.zeros_like(hin)
                rc = dccl_lib.dccl_emu_all_to_all(n, nbytes, ctas, 3, hin.ctypes.data, hout.ctypes.data)
                assert rc == 0, (mode, n, nbytes, rc)
                src, got = hin.reshape(n, n, nbytes), hout.reshape(n, n, nbytes)
                for r in range(n):
                    for p in range(n):
                        assert np.array_equal(got[r, p], src[p, r]), (mode, n, nbytes, r, p)
    finally:
        dccl_lib.dccl_emu_set_p2p_rendezvous(0)
