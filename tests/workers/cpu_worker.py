"""One rank of a host-buffer test: runs a list of collectives on numpy arrays and checks each
against the serial fold. Prints 'OK <cases>' or the first mismatches and exits non-zero."""
import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from dccl_b200 import Communicator, group_end, group_start  # noqa: E402
from dccl_b200.comm import BFLOAT16, DTYPE_SIZES, OPS  # noqa: E402
from dccl_b200._lib import lib  # noqa: E402
from dccl_b200.utils import oracle  # noqa: E402

FLOATS = ["float16", "float32", "float64", "bfloat16"]
INTS = ["int8", "uint8", "int32", "uint32", "int64", "uint64"]


def close(got, want, dtype_name, world):
    if dtype_name == "bfloat16":
        g, w = oracle.bf16_to_f32(got).astype(np.float64), oracle.bf16_to_f32(want).astype(np.float64)
    else:
        g, w = got.astype(np.float64), want.astype(np.float64)
    rtol, atol = oracle.tolerances(dtype_name, world)
    if rtol == 0.0:
        return np.array_equal(got, want)
    return np.allclose(g, w, rtol=rtol, atol=atol)


class Raw:
    """Calls the C API with explicit dtype codes, so bfloat16 (uint16 bit patterns) can be tested from numpy."""

    def __init__(self, comm):
        self.c = comm
        self.h = comm._h
        self.L = lib()

    def code(self, name):
        return ["int8", "uint8", "int32", "uint32", "int64", "uint64", "float16", "float32", "float64", "bfloat16"].index(name)

    def all_reduce(self, s, r, name, op):
        return self.L.dccl_all_reduce(s.ctypes.data, r.ctypes.data, s.size, self.code(name), OPS[op], self.h, None)

    def reduce_scatter(self, s, r, name, op):
        return self.L.dccl_reduce_scatter(s.ctypes.data, r.ctypes.data, r.size, self.code(name), OPS[op], self.h, None)

    def all_gather(self, s, r, name):
        return self.L.dccl_all_gather(s.ctypes.data, r.ctypes.data, s.size, self.code(name), self.h, None)

    def broadcast(self, s, r, name, root):
        return self.L.dccl_broadcast(s.ctypes.data, r.ctypes.data, r.size, self.code(name), root, self.h, None)

    def reduce(self, s, r, name, op, root):
        return self.L.dccl_reduce(s.ctypes.data, r.ctypes.data if r is not None else None, s.size, self.code(name), OPS[op], root, self.h, None)


def unaligned(arr, offset_elems):
    """A copy of arr that starts offset_elems elements into a larger allocation (not cache-line aligned)."""
    big = np.empty(arr.size + offset_elems + 16, dtype=arr.dtype)
    view = big[offset_elems:offset_elems + arr.size]
    view[:] = arr
    return view


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--suite", default="basic")
    ap.add_argument("--algo", default="ring")
    ap.add_argument("--repeat", type=int, default=1)
    args = ap.parse_args()
    comm = Communicator()
    raw = Raw(comm)
    rank, world = comm.rank, comm.world
    for coll in ("allreduce", "reducescatter", "allgather"):
        comm.set_algorithm(coll, args.algo)
    failures, cases = [], 0

    def check(ok, what):
        nonlocal cases
        cases += 1
        if not ok:
            failures.append(what)

    if args.suite == "basic":
        dtypes, ops, counts = FLOATS + INTS, ["sum", "prod", "max", "min", "avg"], [1, 5, 64, 1000, 1024, 4099]
    elif args.suite == "baseline":   # fp32 sum, 1024 elements per rank, uniform[-1,1], seed = rank, many repeats
        dtypes, ops, counts = ["float32"], ["sum"], [1024]
    else:
        dtypes, ops, counts = ["float32", "bfloat16", "int32"], ["sum", "avg"], [7, 100000, 300001]

    if args.suite == "basic":
        # max / min of floats: a NaN loses against a number wherever it sits (IEEE maxNum / minNum); NaN on every rank stays
        for name in ["float32", "float64", "bfloat16", "float16"]:
            count = 1031
            ins = [oracle.make_input(name, count, seed=77 + r) for r in range(world)]
            nan = np.uint16(0x7FC0) if name == "bfloat16" else np.nan
            for r in range(world):
                ins[r][r::5] = nan
                ins[r][3::97] = nan
            for op in ["max", "min"]:
                want = oracle.fold(ins, op, bf16=name == "bfloat16")
                out = np.zeros_like(ins[rank])
                rc = raw.all_reduce(ins[rank].copy(), out, name, op)
                gf = oracle.bf16_to_f32(out) if name == "bfloat16" else out.astype(np.float64)
                wf = oracle.bf16_to_f32(want) if name == "bfloat16" else want.astype(np.float64)
                check(rc == 0 and np.array_equal(np.isnan(gf), np.isnan(wf)) and np.array_equal(gf[~np.isnan(wf)], wf[~np.isnan(wf)]),
                      "all_reduce %s %s with NaN inputs" % (name, op))

    for name in dtypes:
        for count in counts:
            ins = [oracle.make_input(name, count, seed=1000 * r + count % 97) for r in range(world)]
            if args.suite == "baseline":
                ins = [oracle.make_input(name, count, seed=r) for r in range(world)]
            bf = name == "bfloat16"
            for op in ops:
                if op == "prod" and name in FLOATS:
                    pins = [np.where(np.abs(x.astype(np.float64) if not bf else oracle.bf16_to_f32(x)) < 0.5, 1.0, 1.25) for x in ins]
                    pins = [oracle.f32_to_bf16(p.astype(np.float32)) if bf else p.astype(name) for p in pins]
                else:
                    pins = ins
                want = oracle.fold(pins, op, bf16=bf)
                # all-reduce, out of place, receive buffer deliberately unaligned
                for _ in range(args.repeat):
                    s = unaligned(pins[rank], 1 + rank)
                    r = unaligned(np.zeros_like(pins[rank]), 3)
                    rc = raw.all_reduce(s, r, name, op)
                    check(rc == 0 and close(r, want, name, world), "all_reduce %s %s n=%d rc=%d" % (name, op, count, rc))
                    if args.algo == "ring" and op == "sum" and name in ("float32", "float64"):
                        # same additions in the same order as the ring: the bits must match, on every rank
                        check(np.array_equal(r, oracle.ring_fold_sum(pins)), "all_reduce %s ring order n=%d" % (name, count))
                # in place
                s = pins[rank].copy()
                rc = raw.all_reduce(s, s, name, op)
                check(rc == 0 and close(s, want, name, world), "all_reduce in place %s %s n=%d" % (name, op, count))
                # reduce to the last rank and to rank 0
                for root in {0, world - 1}:
                    s = pins[rank].copy()
                    r = np.zeros_like(s)
                    rc = raw.reduce(s, r, name, op, root)
                    check(rc == 0 and (rank != root or close(r, want, name, world)), "reduce %s %s n=%d root=%d" % (name, op, count, root))
                # reduce-scatter: every rank contributes world*count elements
                if count <= 1024:
                    big = [oracle.make_input(name, count * world, seed=77 * r + count) for r in range(world)]
                    if op == "prod" and name in FLOATS:
                        continue
                    wantb = oracle.fold(big, op, bf16=bf)
                    r = np.zeros(count, dtype=big[0].dtype)
                    rc = raw.reduce_scatter(big[rank].copy(), r, name, op)
                    check(rc == 0 and close(r, wantb[rank * count:(rank + 1) * count], name, world), "reduce_scatter %s %s n=%d" % (name, op, count))
            # all-gather and broadcast move bytes
            g = np.zeros(count * world, dtype=ins[0].dtype)
            rc = raw.all_gather(ins[rank].copy(), g, name)
            check(rc == 0 and np.array_equal(g, np.concatenate(ins)), "all_gather %s n=%d" % (name, count))
            g2 = np.zeros(count * world, dtype=ins[0].dtype)
            g2[rank * count:(rank + 1) * count] = ins[rank]
            rc = raw.all_gather(g2[rank * count:(rank + 1) * count], g2, name)
            check(rc == 0 and np.array_equal(g2, np.concatenate(ins)), "all_gather in place %s n=%d" % (name, count))
            for root in {0, world - 1}:
                r = ins[rank].copy() if rank == root else np.zeros_like(ins[rank])
                rc = raw.broadcast(r, r, name, root)
                check(rc == 0 and np.array_equal(r, ins[root]), "broadcast %s n=%d root=%d" % (name, count, root))

    # send / recv: a ring, grouped so that everybody may send first
    if world > 1:
        msg = np.full(70000, rank, dtype=np.int32)     # larger than one FIFO when the channel is small
        got = np.zeros_like(msg)
        group_start()
        comm.send(msg, (rank + 1) % world)
        comm.recv(got, (rank - 1) % world)
        group_end()
        check(np.all(got == (rank - 1) % world), "grouped ring send/recv")
        if rank < 2:   # plain blocking pair, like dccl_cli's send / recv
            if rank == 0:
                comm.send(msg, 1)
            else:
                comm.recv(got, 0)
                check(np.all(got == 0), "blocking send/recv")
    # the descriptor plane (SCM_RIGHTS over the per-rank unix sockets) that carries the GPU memory handles
    from dccl_b200._lib import lib as _native
    check(_native().dccl_selftest_fd_exchange(comm._h) == 0, "descriptor exchange between all ranks")
    check(_native().dccl_debug_check(comm._h) == 0, "pool check without a device side is a success")
    # the exchange board in the shared control segment (per-call agreement for lazy registration): 2000 skewed rounds
    check(_native().dccl_selftest_board(comm._h, 2000) == 0, "small all-gathers over the shared-memory board")
    # barrier: nobody passes before the last rank has arrived (the last rank arrives 0.3 s late)
    import time
    t0 = time.monotonic()
    if rank == world - 1:
        time.sleep(0.3)
    comm.barrier()
    check(world == 1 or rank == world - 1 or time.monotonic() - t0 > 0.25, "barrier waits for the last rank")

    # the symmetric allocator over a stand-in driver (memfd + mmap): every rank maps every peer's segment and reads it;
    # then with one rank's allocation failing: everybody must come back with a failure, nobody may hang
    if hasattr(_native(), "dccl_selftest_symmem") and world <= 8:
        check(_native().dccl_selftest_symmem(comm._h, -1) == 0, "symmetric allocator: segments of all ranks mapped and readable")
        check(_native().dccl_selftest_symmem(comm._h, world - 1) == 0, "symmetric allocator: a failing rank fails everybody")
        check(_native().dccl_selftest_symmem(comm._h, -1) == 0, "symmetric allocator: works again afterwards")

    # all-to-all (equal and uneven blocks), gather, scatter
    for n in [1, 1000, 400001]:
        src = [np.arange(n * world, dtype=np.float64) + 1e6 * r for r in range(world)]
        out = np.zeros(n * world, dtype=np.float64)
        comm.all_to_all(src[rank], out)
        check(np.array_equal(out, np.concatenate([src[p][rank * n:(rank + 1) * n] for p in range(world)])), "all_to_all n=%d" % n)
        for root in {0, world - 1}:
            got = np.zeros(n * world, dtype=np.float64) if rank == root else None
            comm.gather(src[rank][:n], got, root=root)
            check(rank != root or np.array_equal(got, np.concatenate([src[p][:n] for p in range(world)])), "gather n=%d root=%d" % (n, root))
            piece = np.zeros(n, dtype=np.float64)
            comm.scatter(src[root] if rank == root else None, piece, root=root)
            check(np.array_equal(piece, src[root][rank * n:(rank + 1) * n]), "scatter n=%d root=%d" % (n, root))
    sc = [(p + rank) % 3 * 5 for p in range(world)]              # what I send to p (some blocks are empty)
    rc = [(rank + p) % 3 * 5 for p in range(world)]              # what p sends to me
    sbuf = np.concatenate([np.full(sc[p], 100 * rank + p, dtype=np.int32) for p in range(world)] + [np.zeros(0, np.int32)])
    rbuf = np.zeros(sum(rc), dtype=np.int32)
    comm.all_to_all(sbuf, rbuf, send_counts=sc, recv_counts=rc)
    check(np.array_equal(rbuf, np.concatenate([np.full(rc[p], 100 * p + rank, dtype=np.int32) for p in range(world)] + [np.zeros(0, np.int32)])), "all_to_all with uneven blocks")
    code, msg_ = comm.last_error()
    check(code == 0, "async error " + msg_)
    algo = comm.last_algorithm("allreduce")
    comm.finalize()
    if failures:
        print("FAILED %d of %d on rank %d: %s" % (len(failures), cases, rank, "; ".join(failures[:8])))
        sys.exit(1)
    print("OK %d %s" % (cases, algo))


if __name__ == "__main__":
    main()
