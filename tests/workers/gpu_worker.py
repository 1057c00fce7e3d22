"""One rank of a multi-GPU test: device collectives on torch tensors, every variant, checked against
a fold computed on the CPU from the seeds of all ranks. Prints 'OK <cases>' or the failures."""
import argparse
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from dccl_b200 import Communicator, group_end, group_start  # noqa: E402
from dccl_b200.utils import oracle  # noqa: E402

TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16, "float64": torch.float64,
         "int32": torch.int32, "int64": torch.int64, "int8": torch.int8, "uint8": torch.uint8}


def to_torch(arr, name, dev):
    if name == "bfloat16":
        return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16).to(dev)
    return torch.from_numpy(arr.copy()).to(dev)


def to_numpy(t, name):
    if name == "bfloat16":
        return t.cpu().view(torch.int16).numpy().view(np.uint16)
    return t.cpu().numpy()


def close(got, want, name, world):
    rtol, atol = oracle.tolerances(name, world)
    if rtol == 0.0:
        return np.array_equal(got, want)
    if name == "bfloat16":
        got, want = oracle.bf16_to_f32(got), oracle.bf16_to_f32(want)
    return np.allclose(got.astype(np.float64), want.astype(np.float64), rtol=rtol, atol=atol)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--suite", default="basic")
    args = ap.parse_args()
    local = int(os.environ.get("DCCL_LOCAL_DEVICE", os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = Communicator(device=local)
    rank, world = comm.rank, comm.world
    failures, cases = [], 0

    def check(ok, what):
        nonlocal cases
        cases += 1
        if not ok:
            failures.append(what)

    if args.suite == "odd_world":
        # all-reduce of every staged peer variant on a world that is not a power of two: halving and doubling folds the
        # world onto the next lower power of two through leader / follower pairs
        for algo in ["rabenseifner", "twoshot", "ring"]:
            comm.set_algorithm("allreduce", algo)
            for name in ["float32", "bfloat16", "int32"]:
                for count in [1, 1000, 300001, 4 << 20]:
                    ins = [oracle.make_input(name, count, seed=37 * r + count % 103) for r in range(world)]
                    for op in ["sum", "avg", "max"]:
                        want = oracle.fold(ins, op, bf16=name == "bfloat16")
                        s = to_torch(ins[rank], name, dev)
                        r = torch.zeros_like(s)
                        for _ in range(3):
                            comm.all_reduce(s, r, op=op)
                        torch.cuda.synchronize()
                        check(comm.last_algorithm("allreduce") == algo, "all_reduce %s ran %s" % (algo, comm.last_algorithm("allreduce")))
                        check(close(to_numpy(r, name), want, name, world), "all_reduce %s %s %s n=%d" % (algo, name, op, count))
                        comm.all_reduce(s, op=op)   # in place
                        torch.cuda.synchronize()
                        check(close(to_numpy(s, name), want, name, world), "all_reduce in place %s %s %s n=%d" % (algo, name, op, count))
        launches = comm.stat("launches")
        comm.finalize()
        if failures:
            print("FAILED %d of %d on rank %d: %s" % (len(failures), cases, rank, "; ".join(failures[:10])))
            sys.exit(1)
        print("OK %d multicast=%d launches=%d" % (cases, 0, launches))
        return

    if args.suite == "rooted":
        # broadcast / reduce of large ordinary buffers with the pipelined switch form switched on
        if not comm.has_multicast:
            comm.finalize()
            print("OK 0 multicast=0 launches=0")
            return
        comm.set_param("rooted_pipe", 1)
        for name, count in [("float32", (8 << 20) + 3), ("bfloat16", 16 << 20), ("int32", (5 << 20) + 1)]:
            ins = [oracle.make_input(name, count, seed=500 + r) for r in range(world)]
            for root in sorted({0, world - 1}):
                for shift in (0, 1):       # 1: buffers that do not start on a 16-byte boundary
                    base = torch.zeros(count + 8, dtype=TORCH[name], device=dev)
                    b = base[shift:shift + count]
                    for _ in range(3):
                        b.copy_(to_torch(ins[rank], name, dev))
                        comm.broadcast(b, root=root)
                    torch.cuda.synchronize()
                    check(comm.last_algorithm("broadcast") == "nvls", "broadcast ran %s" % comm.last_algorithm("broadcast"))
                    check(np.array_equal(to_numpy(b.contiguous(), name), ins[root]), "pipelined broadcast %s root=%d shift=%d" % (name, root, shift))
                    if shift:
                        continue
                    for op in ["sum", "avg", "max"]:
                        s = to_torch(ins[rank], name, dev)
                        out = torch.zeros_like(s)
                        for _ in range(2):
                            comm.reduce(s, out, op=op, root=root)
                        torch.cuda.synchronize()
                        want = oracle.fold(ins, op, bf16=name == "bfloat16")
                        check(rank != root or close(to_numpy(out, name), want, name, world), "pipelined reduce %s %s root=%d" % (name, op, root))
        code, emsg = comm.last_error()
        check(code == 0, "async error: " + emsg)
        launches = comm.launches
        comm.finalize()
        if failures:
            print("FAILED %d of %d on rank %d: %s" % (len(failures), cases, rank, "; ".join(failures[:10])))
            sys.exit(1)
        print("OK %d multicast=1 launches=%d" % (cases, launches))
        return

    if args.suite == "lazy":
        # ordinary tensors that nobody registered: a large call on them exchanges the allocations between the ranks,
        # maps what is new and then runs zero-copy; a freed and re-allocated buffer is mapped afresh; a pointer that is
        # not 16-byte aligned on ONE rank sends every rank down the staged path
        comm.set_algorithm("allreduce", "twoshot")
        comm.set_algorithm("reducescatter", "twoshot")
        comm.set_param("direct_rs", 1)
        for rnd in range(3):
            for name, count in [("bfloat16", (4 << 20) + 64 * world), ("float32", (2 << 20) + 32 * world)]:
                ins = [oracle.make_input(name, count, seed=7000 + 10 * rnd + r) for r in range(world)]
                bf = name == "bfloat16"
                for op in ["sum", "avg"]:
                    want = oracle.fold(ins, op, bf16=bf)
                    s = to_torch(ins[rank], name, dev)
                    out = torch.zeros_like(s)
                    z0 = comm.stat("zero_copy_calls")
                    for _ in range(2):
                        comm.all_reduce(s, out, op=op)
                    torch.cuda.synchronize()
                    check(comm.stat("zero_copy_calls") - z0 == 2, "lazy registration: all_reduce %s ran zero-copy (%d)" % (name, comm.stat("zero_copy_calls") - z0))
                    check(close(to_numpy(out, name), want, name, world), "lazy all_reduce %s %s round %d" % (name, op, rnd))
                    comm.all_reduce(s, op=op)      # in place
                    torch.cuda.synchronize()
                    check(close(to_numpy(s, name), want, name, world), "lazy all_reduce in place %s %s" % (name, op))
                    # reduce-scatter: the peers read this rank's send buffer
                    per = count // world
                    s = to_torch(ins[rank], name, dev)
                    rs = torch.zeros(per, dtype=s.dtype, device=dev)
                    z0 = comm.stat("zero_copy_calls")
                    comm.reduce_scatter(s[:per * world], rs, op=op)
                    torch.cuda.synchronize()
                    check(comm.stat("zero_copy_calls") - z0 == 1, "lazy registration: reduce_scatter %s ran zero-copy" % name)
                    check(close(to_numpy(rs, name), want[rank * per:(rank + 1) * per], name, world), "lazy reduce_scatter %s %s" % (name, op))
                    # one rank off a 16-byte boundary: staged on every rank, same values
                    es = s.element_size()
                    shift = (4 // es) if rank == world - 1 else 0
                    base_s = torch.zeros(count + 16, dtype=s.dtype, device=dev)
                    base_o = torch.zeros(count + 16, dtype=s.dtype, device=dev)
                    v, o = base_s[shift:shift + count], base_o[shift:shift + count]
                    v.copy_(to_torch(ins[rank], name, dev))
                    z0 = comm.stat("zero_copy_calls")
                    comm.all_reduce(v, o, op=op)
                    torch.cuda.synchronize()
                    check(comm.stat("zero_copy_calls") == z0, "one unaligned rank: nobody runs zero-copy")
                    check(close(to_numpy(o.contiguous(), name), want, name, world), "all_reduce with one unaligned rank %s %s" % (name, op))
                    del s, out, rs, base_s, base_o, v, o
            # give the memory back to the driver: the next round's tensors are new allocations, often at old addresses
            torch.cuda.synchronize()
            comm.barrier()
            torch.cuda.empty_cache()
        comm.set_param("direct_rs", 0)
        comm.set_algorithm("allreduce", "auto")
        comm.set_algorithm("reducescatter", "auto")
        # broadcast and reduce from the same threshold on: the receivers load the message out of the root's buffer and out
        # of each other's; the owners of a shard fold it into the root's buffer. Ordinary tensors, a root whose source is
        # symmetric memory, every root position, in place; one unaligned rank sends everybody down the staged path.
        comm.set_param("direct_bcast_min_kb", 4096)       # by default the broadcast takes this path from 32 MB on,
        comm.set_param("direct_reduce_small_worlds", 1)   # and so does the reduce on worlds of up to four ranks
        for name, count in [("bfloat16", (4 << 20) + 72), ("float32", (3 << 20) + 4), ("uint8", (5 << 20) + 13)]:
            ins = [oracle.make_input(name, count, seed=7700 + r) for r in range(world)]
            want = oracle.fold(ins, "sum", bf16=name == "bfloat16")
            for root in sorted({0, 1 % world, world - 1}):
                for variant in ["plain", "in place", "symmetric source", "unaligned"]:
                    shift = 1 if variant == "unaligned" and rank == world - 1 else 0
                    base_s = comm.symmetric_empty(count + 16, to_torch(ins[rank][:1], name, dev).dtype, local) if variant == "symmetric source" \
                        else torch.zeros(count + 16, dtype=to_torch(ins[rank][:1], name, dev).dtype, device=dev)
                    base_o = torch.zeros(count + 16, dtype=base_s.dtype, device=dev)
                    v = base_s[shift:shift + count]
                    o = v if variant == "in place" else base_o[shift:shift + count]
                    v.copy_(to_torch(ins[rank], name, dev))
                    z0 = comm.stat("zero_copy_calls")
                    for _ in range(2):
                        comm.broadcast(v, o, root=root)
                    torch.cuda.synchronize()
                    zc = comm.stat("zero_copy_calls") - z0
                    check(zc == (0 if variant == "unaligned" else 2), "broadcast %s %s root %d: zero-copy calls %d" % (name, variant, root, zc))
                    check(np.array_equal(to_numpy(o.contiguous(), name), ins[root]), "lazy broadcast %s %s root %d" % (name, variant, root))
                    if name != "uint8":
                        v.copy_(to_torch(ins[rank], name, dev))
                        z0 = comm.stat("zero_copy_calls")
                        comm.reduce(v, o if rank == root or variant == "in place" else None, op="sum", root=root)
                        torch.cuda.synchronize()
                        zc = comm.stat("zero_copy_calls") - z0
                        check(zc == (0 if variant == "unaligned" else 1), "reduce %s %s root %d: zero-copy calls %d" % (name, variant, root, zc))
                        check(rank != root or close(to_numpy(o.contiguous(), name), want, name, world), "lazy reduce %s %s root %d" % (name, variant, root))
                    torch.cuda.synchronize()
                    comm.barrier()
                    if variant == "symmetric source":
                        comm.free_symmetric(base_s)
                    del base_s, base_o, v, o
        comm.set_param("direct_bcast_min_kb", 32 << 10)
        comm.set_param("direct_reduce_small_worlds", 0)
        # variant choices that only one rank's alignment could have changed: a reduce-scatter into an unaligned receive
        # buffer (pipelined switch form from 256 KB on) and an all-gather from an unaligned source into symmetric memory
        if comm.has_multicast:
            comm.set_param("pipe_min_mb", 1)
            name, per = "float32", (1 << 20) + 8
            ins = [oracle.make_input(name, per * world, seed=7500 + r) for r in range(world)]
            want = oracle.fold(ins, "sum")
            shift = 1 if rank == world - 1 else 0
            comm.set_algorithm("reducescatter", "nvls")
            s = to_torch(ins[rank], name, dev)
            base_o = torch.zeros(per + 8, dtype=torch.float32, device=dev)
            o = base_o[shift:shift + per]
            for _ in range(2):
                comm.reduce_scatter(s, o, op="sum")
            torch.cuda.synchronize()
            check(close(to_numpy(o.contiguous(), name), want[rank * per:(rank + 1) * per], name, world), "switch reduce_scatter, one receive buffer unaligned")
            comm.set_algorithm("reducescatter", "auto")
            comm.set_algorithm("allgather", "nvls")
            g = comm.symmetric_empty(per * world, torch.float32, local)
            base_s = torch.zeros(per + 8, dtype=torch.float32, device=dev)
            v = base_s[shift:shift + per]
            v.copy_(to_torch(ins[rank][:per], name, dev))
            comm.all_gather(v, g)
            torch.cuda.synchronize()
            check(np.array_equal(to_numpy(g, name), np.concatenate([x[:per] for x in ins])), "switch all_gather into symmetric memory, one source unaligned")
            comm.set_algorithm("allgather", "auto")
            comm.free_symmetric(g)
            # max / min inside the switch follow the same NaN rule as the peer kernels: a number beats a NaN
            for name in ["bfloat16", "float16"]:
                count = 70001
                ins = [oracle.make_input(name, count, seed=7700 + r) for r in range(world)]
                nan = np.uint16(0x7FC0) if name == "bfloat16" else np.nan
                for r in range(world):
                    ins[r][r::9] = nan
                    ins[r][4::113] = nan
                comm.set_algorithm("allreduce", "nvls")
                for op in ["max", "min"]:
                    want = oracle.fold(ins, op, bf16=name == "bfloat16")
                    wf = oracle.bf16_to_f32(want) if name == "bfloat16" else want.astype(np.float32)
                    s = to_torch(ins[rank], name, dev)
                    out = torch.zeros_like(s)
                    comm.all_reduce(s, out, op=op)
                    torch.cuda.synchronize()
                    got = to_numpy(out, name)
                    gf = oracle.bf16_to_f32(got) if name == "bfloat16" else got.astype(np.float32)
                    check(comm.last_algorithm("allreduce") == "nvls", "NaN rule: ran %s" % comm.last_algorithm("allreduce"))
                    check(np.array_equal(np.isnan(gf), np.isnan(wf)) and np.array_equal(gf[~np.isnan(wf)], wf[~np.isnan(wf)]),
                          "switch %s of %s with NaN inputs" % (op, name))
                comm.set_algorithm("allreduce", "auto")
        code, emsg = comm.last_error()
        check(code == 0, "async error: " + emsg)
        launches = comm.launches
        mc = comm.has_multicast
        comm.finalize()
        if failures:
            print("FAILED %d of %d on rank %d: %s" % (len(failures), cases, rank, "; ".join(failures[:10])))
            sys.exit(1)
        print("OK %d multicast=%d launches=%d" % (cases, int(mc), launches))
        return

    if args.suite == "extra":
        # what the communicator found out about the box
        topo = comm.topology()
        check(topo["nranks"] == world and len(topo["gpus"]) == world, "topology: one entry per rank")
        check(all(g["sm_count"] > 0 and g["mem_bytes"] > 0 and g["pci"] for g in topo["gpus"]), "topology: GPU facts")
        check(all(topo["peer_access"][a][b] in (1, 255) for a in range(world) for b in range(world) if a != b), "topology: peers reachable")
        check(all(bool(g["multicast"]) == comm.has_multicast for g in topo["gpus"]) or not comm.has_multicast, "topology: multicast flag")

    algos = ["oneshot", "twoshot", "ring", "rabenseifner"] + (["nvls"] if comm.has_multicast else [])
    if args.suite == "basic":
        names, counts = ["float32", "bfloat16", "int32", "float16"], [1, 1000, 16384, 300001, 4 << 20]
    elif args.suite == "extra":   # the two-shot packet variant, up to its capacity and beyond (falls back to the staged form)
        algos, names, counts = ["twoshot_ll"], ["float32", "bfloat16", "int32"], [1, 1000, 16384, 300001, 4 << 20]
    else:   # chunking: staging is made small through DCCL_STAGING_BYTES by the caller
        names, counts = ["float32", "bfloat16"], [3 << 20, (8 << 20) + 12345]
    for name in names:
        for count in counts:
            ins = [oracle.make_input(name, count, seed=31 * r + count % 101) for r in range(world)]
            bf = name == "bfloat16"
            for op in (["sum", "avg", "max"] if args.suite == "basic" else ["sum"]):
                want = oracle.fold(ins, op, bf16=bf)
                for algo in algos:
                    comm.set_algorithm("allreduce", algo)
                    s = to_torch(ins[rank], name, dev)
                    r = torch.zeros_like(s)
                    for _ in range(3):
                        comm.all_reduce(s, r, op=op)
                    torch.cuda.synchronize()
                    used = comm.last_algorithm("allreduce")
                    check(close(to_numpy(r, name), want, name, world), "all_reduce %s %s %s n=%d (ran %s)" % (algo, name, op, count, used))
                    comm.all_reduce(s, op=op)   # in place
                    torch.cuda.synchronize()
                    check(close(to_numpy(s, name), want, name, world), "all_reduce in place %s %s %s n=%d" % (algo, name, op, count))
                comm.set_algorithm("allreduce", "auto")
                # reduce to both ends
                for root in {0, world - 1}:
                    for algo in (["twoshot_ll"] if args.suite == "extra" else ["twoshot", "oneshot"] + (["nvls"] if comm.has_multicast else [])):
                        comm.set_algorithm("reduce", algo)
                        s = to_torch(ins[rank], name, dev)
                        r = torch.zeros_like(s)
                        comm.reduce(s, r, op=op, root=root)
                        torch.cuda.synchronize()
                        check(rank != root or close(to_numpy(r, name), want, name, world), "reduce %s %s %s n=%d root=%d" % (algo, name, op, count, root))
                # reduce-scatter (count must split)
                per = count // world
                if per:
                    wantrs = want[rank * per:(rank + 1) * per]
                    for algo in ["twoshot", "ring", "oneshot"] + (["nvls"] if comm.has_multicast else []):
                        comm.set_algorithm("reducescatter", algo)
                        s = to_torch(ins[rank][:per * world], name, dev)
                        r = torch.zeros(per, dtype=s.dtype, device=dev)
                        comm.reduce_scatter(s, r, op=op)
                        torch.cuda.synchronize()
                        check(close(to_numpy(r, name), wantrs, name, world), "reduce_scatter %s %s %s n=%d" % (algo, name, op, per))
            per = max(1, count // world)
            full = np.concatenate([x[:per] for x in ins])
            for algo in ["twoshot", "ring", "oneshot"] + (["nvls"] if comm.has_multicast else []):
                comm.set_algorithm("allgather", algo)
                s = to_torch(ins[rank][:per], name, dev)
                r = torch.zeros(per * world, dtype=s.dtype, device=dev)
                comm.all_gather(s, r)
                torch.cuda.synchronize()
                check(np.array_equal(to_numpy(r, name), full), "all_gather %s %s n=%d" % (algo, name, per))
            for root in {0, world - 1}:
                for algo in ["oneshot", "twoshot"] + (["nvls"] if comm.has_multicast else []):
                    comm.set_algorithm("broadcast", algo)
                    b = to_torch(ins[rank], name, dev)
                    comm.broadcast(b, root=root)
                    torch.cuda.synchronize()
                    check(np.array_equal(to_numpy(b, name), ins[root]), "broadcast %s %s n=%d root=%d" % (algo, name, count, root))

    # symmetric memory: zero-copy switch reduction
    if comm.has_multicast and args.suite == "basic":
        for name in ["float32", "bfloat16"]:
            count = 1 << 20
            ins = [oracle.make_input(name, count, seed=900 + r) for r in range(world)]
            want = oracle.fold(ins, "avg", bf16=name == "bfloat16")
            t = comm.symmetric_empty(count, TORCH[name], local)
            t.copy_(to_torch(ins[rank], name, dev))
            torch.cuda.synchronize()
            comm.set_algorithm("allreduce", "nvls")
            comm.all_reduce(t, op="avg")
            torch.cuda.synchronize()
            check(close(to_numpy(t, name), want, name, world), "symmetric all_reduce %s" % name)
            # reduce-scatter straight out of the symmetric buffer, all-gather straight into one
            per = count // world
            t.copy_(to_torch(ins[rank], name, dev))
            torch.cuda.synchronize()
            comm.set_algorithm("reducescatter", "nvls")
            out = torch.zeros(per, dtype=TORCH[name], device=dev)
            comm.reduce_scatter(t, out, op="sum")
            torch.cuda.synchronize()
            wsum = oracle.fold(ins, "sum", bf16=name == "bfloat16")
            check(close(to_numpy(out, name), wsum[rank * per:(rank + 1) * per], name, world), "symmetric reduce_scatter %s (ran %s)" % (name, comm.last_algorithm("reducescatter")))
            comm.set_algorithm("allgather", "nvls")
            mine = to_torch(ins[rank][:per], name, dev)
            comm.all_gather(mine, t)
            torch.cuda.synchronize()
            check(np.array_equal(to_numpy(t, name), np.concatenate([x[:per] for x in ins])), "symmetric all_gather %s" % name)
            comm.set_algorithm("reducescatter", "auto")
            comm.set_algorithm("allgather", "auto")
            comm.free_symmetric(t)
        comm.set_algorithm("allreduce", "auto")

    # buffers every rank can address (symmetric, or registered): the two-shot variant folds them without staging
    if args.suite == "basic":
        for name, count in [("bfloat16", (1 << 20) + 64), ("float32", 300001), ("int32", 4099)]:
            ins = [oracle.make_input(name, count, seed=1200 + r) for r in range(world)]
            for op in ["sum", "avg", "max"]:
                want = oracle.fold(ins, op, bf16=name == "bfloat16")
                src = comm.symmetric_empty(count, TORCH[name], local)
                dst = comm.symmetric_empty(count, TORCH[name], local)
                src.copy_(to_torch(ins[rank], name, dev))
                torch.cuda.synchronize()
                comm.set_algorithm("allreduce", "twoshot")
                before = comm.launches
                for _ in range(3):
                    comm.all_reduce(src, dst, op=op)
                torch.cuda.synchronize()
                check(comm.launches - before == 3, "zero-copy two-shot: one launch per call")
                check(close(to_numpy(dst, name), want, name, world), "zero-copy two-shot all_reduce %s %s" % (name, op))
                comm.all_reduce(src, op=op)   # in place
                torch.cuda.synchronize()
                check(close(to_numpy(src, name), want, name, world), "zero-copy two-shot all_reduce in place %s %s" % (name, op))
                if count % (8 * world) == 0:
                    per = count // world
                    src.copy_(to_torch(ins[rank], name, dev))
                    torch.cuda.synchronize()
                    comm.set_algorithm("reducescatter", "twoshot")
                    comm.reduce_scatter(src, dst[:per], op=op)
                    torch.cuda.synchronize()
                    check(close(to_numpy(dst[:per], name), want[rank * per:(rank + 1) * per], name, world), "zero-copy two-shot reduce_scatter %s %s" % (name, op))
                    comm.set_algorithm("reducescatter", "auto")
                comm.free_symmetric(src)
                comm.free_symmetric(dst)
            # ordinary allocations, registered with every rank
            # (registration wants whole cache lines: pad the allocation, use its front part)
            padded = (count + 63) // 64 * 64
            abuf = torch.zeros(padded, dtype=TORCH[name], device=dev)
            bbuf = torch.zeros(padded, dtype=TORCH[name], device=dev)
            a, b = abuf[:count], bbuf[:count]
            a.copy_(to_torch(ins[rank], name, dev))
            comm.register(abuf)
            comm.register(bbuf)
            before = comm.launches
            comm.all_reduce(a, b, op="sum")
            torch.cuda.synchronize()
            check(comm.launches - before == 1, "registered buffers: one launch")
            check(close(to_numpy(b, name), oracle.fold(ins, "sum", bf16=name == "bfloat16"), name, world), "registered buffers all_reduce %s" % name)
            comm.deregister(abuf)
            comm.deregister(bbuf)
        comm.set_algorithm("allreduce", "auto")

    # send / recv: grouped ring with 8 MB messages (longer than the FIFO), then a plain pair
    msg = torch.full((2 << 20,), float(rank), dtype=torch.float32, device=dev)
    got = torch.zeros_like(msg)
    for _ in range(2):
        group_start()
        comm.send(msg, (rank + 1) % world)
        comm.recv(got, (rank - 1) % world)
        group_end()
    torch.cuda.synchronize()
    check(bool((got == float((rank - 1) % world)).all()), "grouped ring send/recv")
    small = torch.full((1000,), float(rank + 10), dtype=torch.float32, device=dev)
    if rank == 0:
        comm.send(small, 1)
    elif rank == 1:
        comm.recv(small, 0)
        torch.cuda.synchronize()
        check(bool((small == 10.0).all()), "plain send/recv")
    torch.cuda.synchronize()

    # all-to-all, gather, scatter on device buffers: one launch of grouped sends / receives plus the own block
    if args.suite == "extra":
        for n_el in [1, 1000, (3 << 20) + 5]:      # the largest is longer than the 4 x 1 MB FIFO of a pair
            src = [torch.arange(n_el * world, dtype=torch.float32) + 1e6 * r for r in range(world)]
            mine = src[rank].to(dev)
            out = torch.zeros(n_el * world, dtype=torch.float32, device=dev)
            comm.all_to_all(mine, out)
            torch.cuda.synchronize()
            want = torch.cat([src[p][rank * n_el:(rank + 1) * n_el] for p in range(world)])
            check(torch.equal(out.cpu(), want), "all_to_all n=%d" % n_el)
            for root in sorted({0, world - 1}):
                got = torch.zeros(n_el * world, dtype=torch.float32, device=dev) if rank == root else None
                comm.gather(mine[:n_el], got, root=root)
                piece = torch.zeros(n_el, dtype=torch.float32, device=dev)
                comm.scatter(mine if rank == root else None, piece, root=root)
                torch.cuda.synchronize()
                check(rank != root or torch.equal(got.cpu(), torch.cat([src[p][:n_el] for p in range(world)])), "gather n=%d root=%d" % (n_el, root))
                check(torch.equal(piece.cpu(), src[root][rank * n_el:(rank + 1) * n_el]), "scatter n=%d root=%d" % (n_el, root))

    # CUDA graph replay: refused while the host counts sequence numbers, correct with the device-side counter
    if args.suite == "basic":
        from dccl_b200.comm import DcclError
        n_small, n_big = 1000, 1 << 20
        xs = torch.zeros(n_small, dtype=torch.float32, device=dev)
        ys = torch.zeros_like(xs)
        xb = torch.zeros(n_big, dtype=torch.bfloat16, device=dev)
        yb = torch.zeros_like(xb)
        zb = torch.zeros_like(xb)
        rs_out = torch.zeros(n_big // world, dtype=torch.bfloat16, device=dev)
        ag_out = torch.zeros(n_small * world, dtype=torch.float32, device=dev)
        side = torch.cuda.Stream(device=dev)
        refused = False
        g0 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g0, stream=side):
            ys.add_(0)   # something to capture, so that the graph is not empty
            try:
                comm.all_reduce(xs, ys, op="sum")
            except DcclError:
                refused = True
        check(refused, "capture with host-side sequence numbers must be refused")
        torch.cuda.synchronize()
        comm.set_param("device_seq", 1)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            comm.all_reduce(xs, ys, op="sum")            # packets
            comm.all_reduce(xb, yb, op="avg")            # staging half A
            comm.all_reduce(yb, zb, op="sum")            # staging half B
            comm.reduce_scatter(xb, rs_out, op="sum")
            comm.all_gather(xs, ag_out)
        for it in range(4):
            ins_s = [oracle.make_input("float32", n_small, seed=2000 + 10 * it + r) for r in range(world)]
            ins_b = [oracle.make_input("bfloat16", n_big, seed=3000 + 10 * it + r) for r in range(world)]
            xs.copy_(to_torch(ins_s[rank], "float32", dev))
            xb.copy_(to_torch(ins_b[rank], "bfloat16", dev))
            torch.cuda.synchronize()
            g.replay()
            if it == 1:
                g.replay()   # twice in a row without the host in between
            torch.cuda.synchronize()
            check(close(to_numpy(ys, "float32"), oracle.fold(ins_s, "sum"), "float32", world), "graph replay %d: small all_reduce" % it)
            avg = oracle.fold(ins_b, "avg", bf16=True)
            check(close(to_numpy(yb, "bfloat16"), avg, "bfloat16", world), "graph replay %d: all_reduce avg" % it)
            want_z = oracle.fold([to_numpy(yb, "bfloat16")] * world, "sum", bf16=True)
            check(close(to_numpy(zb, "bfloat16"), want_z, "bfloat16", world), "graph replay %d: chained all_reduce" % it)
            per = n_big // world
            wsum = oracle.fold(ins_b, "sum", bf16=True)
            check(close(to_numpy(rs_out, "bfloat16"), wsum[rank * per:(rank + 1) * per], "bfloat16", world), "graph replay %d: reduce_scatter" % it)
            check(np.array_equal(to_numpy(ag_out, "float32"), np.concatenate(ins_s)), "graph replay %d: all_gather" % it)
        # eager calls interleave with replays in this mode, and the number goes back to the host afterwards
        comm.all_reduce(xs, ys, op="max")
        g.replay()
        torch.cuda.synchronize()
        comm.set_param("device_seq", 0)
        comm.all_reduce(xs, ys, op="max")
        torch.cuda.synchronize()
        check(close(to_numpy(ys, "float32"), oracle.fold(ins_s, "max"), "float32", world), "all_reduce after leaving the device-counter mode")
        del g, g0

    code, emsg = comm.last_error()
    check(code == 0, "async error: " + emsg)
    if os.environ.get("DCCL_DEBUG_BOUNDS") == "1":   # guard words between the pool regions: nothing wrote there
        torch.cuda.synchronize()
        try:
            comm.debug_check()
        except Exception as e:  # noqa: BLE001
            check(False, "pool guard words: %s (%s)" % (e, comm.last_error()[1]))
    mc = comm.has_multicast
    launches = comm.launches
    comm.finalize()
    if failures:
        print("FAILED %d of %d on rank %d: %s" % (len(failures), cases, rank, "; ".join(failures[:10])))
        sys.exit(1)
    print("OK %d multicast=%d launches=%d" % (cases, int(mc), launches))


if __name__ == "__main__":
    main()
