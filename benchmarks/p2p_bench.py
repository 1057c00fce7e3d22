#!/usr/bin/env python
"""Send / recv between GPUs: a ring in which every rank sends to rank + 1 and receives from rank - 1 (one grouped
launch per step), over message sizes from 4 bytes to 256 MB, and an all-to-all of equal blocks; this library against
stock NCCL (torch.distributed) in the same processes. Device time per step (CUDA events around a batch of steps after
warm-up, maximum over ranks); bandwidth is bytes sent per rank and direction over that time.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        benchmarks/p2p_bench.py [--out results/p2p.json] [--no-nccl]

Messages of 512 KB and more travel zero-copy once the sender has mapped the receiver's buffer, which it does the first
time it sends after the receiver announced that buffer: the warm-up steps see to that.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def timed(torch, barrier, host_max, fn, steps, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return host_max(e0.elapsed_time(e1) / steps)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--max-mb", type=int, default=256)
    ap.add_argument("--a2a-mb", type=int, default=64, help="block size of the all-to-all, MB per peer")
    args = ap.parse_args()
    import numpy as np
    import torch
    from dccl_b200 import Communicator, group_end, group_start
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = Communicator(device=local)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    sizes = [4, 1024, 64 << 10, 256 << 10, 1 << 20, 4 << 20, 16 << 20, 64 << 20]
    if args.max_mb >= 256:
        sizes.append(256 << 20)
    maxb = max(sizes)
    sb = torch.ones(maxb, dtype=torch.uint8, device=dev)
    rb = torch.zeros(maxb, dtype=torch.uint8, device=dev)
    blk = args.a2a_mb << 20
    a_in = torch.ones(blk * world, dtype=torch.uint8, device=dev)
    a_out = torch.zeros(blk * world, dtype=torch.uint8, device=dev)
    rows = []

    def ours_barrier():
        comm.barrier()

    def ours_max(x):
        a = np.array([x], dtype=np.float64)
        comm.all_reduce(a, op="max")
        return float(a[0])

    for nbytes in sizes:
        def ring():
            group_start()
            comm.send(sb[:nbytes], nxt)
            comm.recv(rb[:nbytes], prv)
            group_end()
        ms = timed(torch, ours_barrier, ours_max, ring, 200 if nbytes <= (1 << 20) else 20)
        rows.append({"what": "ring", "impl": "dccl", "bytes": nbytes, "us": round(ms * 1e3, 2), "gbs": round(nbytes / ms / 1e6, 2)})
    ok = bool((rb[:1024] == 1).all().item())
    ms = timed(torch, ours_barrier, ours_max, lambda: comm.all_to_all(a_in, a_out), 10)
    rows.append({"what": "all_to_all", "impl": "dccl", "bytes": blk, "us": round(ms * 1e3, 2), "gbs": round(blk * (world - 1) / ms / 1e6, 2)})
    comm.finalize()

    if not args.no_nccl and world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

        def nccl_max(x):
            t = torch.tensor([x], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        for nbytes in sizes:
            def ring():
                for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, sb[:nbytes], nxt), dist.P2POp(dist.irecv, rb[:nbytes], prv)]):
                    w.wait()
            ms = timed(torch, dist.barrier, nccl_max, ring, 200 if nbytes <= (1 << 20) else 20)
            rows.append({"what": "ring", "impl": "nccl", "bytes": nbytes, "us": round(ms * 1e3, 2), "gbs": round(nbytes / ms / 1e6, 2)})
        ms = timed(torch, dist.barrier, nccl_max, lambda: dist.all_to_all_single(a_out, a_in), 10)
        rows.append({"what": "all_to_all", "impl": "nccl", "bytes": blk, "us": round(ms * 1e3, 2), "gbs": round(blk * (world - 1) / ms / 1e6, 2)})
        dist.destroy_process_group()
    if rank == 0:
        print("%-11s %-5s %12s %10s %10s" % ("pattern", "impl", "bytes", "us", "GB/s"))
        for r in rows:
            print("%-11s %-5s %12d %10.2f %10.2f" % (r["what"], r["impl"], r["bytes"], r["us"], r["gbs"]))
        print("data check:", "ok" if ok else "WRONG")
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            json.dump({"n_gpus": world, "rows": rows}, open(args.out, "w"), indent=1)
    return 0 if ok else 3


if __name__ == "__main__":
    sys.exit(main())
