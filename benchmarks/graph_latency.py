#!/usr/bin/env python
"""Small-message all-reduce latency: eager launches against CUDA-graph replay, this library and stock NCCL.

A chain of `--chain` all-reduces of one size is issued eagerly, then captured once into a CUDA graph and
replayed; both are timed on the device (CUDA events, max over ranks). Replay removes the per-call host
work (argument set-up, launch), which is what bounds a decode-style loop of many small collectives.
This library needs its device-side sequence counter for capture (`set_param("device_seq", 1)`).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/graph_latency.py
    ... benchmarks/graph_latency.py --sizes 1024,65536,1048576 --chain 32 --out results/graph_latency.json
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="1024,8192,65536,262144,1048576", help="message bytes per rank (bf16)")
    ap.add_argument("--chain", type=int, default=32, help="all-reduces per timed batch / per graph")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--out", default=os.path.join(ROOT, "results", "graph_latency.json"))
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from dccl_b200 import Communicator

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = Communicator(device=local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29571")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    def timed(fn):
        """ms per call of fn (one batch), max over ranks."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.reps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([t0.elapsed_time(t1) / args.reps], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    rows = []
    for nbytes in [int(x) for x in args.sizes.split(",")]:
        n = max(8, nbytes // 2)
        x = comm.symmetric_empty(n, torch.bfloat16, local) if world > 1 else torch.empty(n, dtype=torch.bfloat16, device=dev)
        x.fill_(0.001)
        y = torch.full((n,), 0.001, dtype=torch.bfloat16, device=dev)

        def ours_batch():
            for _ in range(args.chain):
                comm.all_reduce(x, op="avg")

        def nccl_batch():
            for _ in range(args.chain):
                dist.all_reduce(y, op=dist.ReduceOp.AVG)

        row = {"bytes": n * 2, "chain": args.chain}
        row["ours_eager_us"] = timed(ours_batch) * 1e3 / args.chain
        row["nccl_eager_us"] = timed(nccl_batch) * 1e3 / args.chain
        # capture both chains
        side = torch.cuda.Stream(device=dev)
        comm.set_param("device_seq", 1)
        row["ours_eager_devseq_us"] = timed(ours_batch) * 1e3 / args.chain   # what the device-side counter costs per call
        g_ours = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_ours, stream=side, capture_error_mode="thread_local"):
            ours_batch()
        row["ours_graph_us"] = timed(g_ours.replay) * 1e3 / args.chain
        del g_ours
        torch.cuda.synchronize()
        comm.set_param("device_seq", 0)
        g_nccl = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_nccl, stream=side, capture_error_mode="thread_local"):
            nccl_batch()
        row["nccl_graph_us"] = timed(g_nccl.replay) * 1e3 / args.chain
        del g_nccl
        torch.cuda.synchronize()
        row = {k: (round(v, 2) if isinstance(v, float) else v) for k, v in row.items()}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        if world > 1:
            comm.free_symmetric(x)
    if rank == 0:
        os.makedirs(os.path.dirname(args.out), exist_ok=True)
        with open(args.out, "w") as f:
            json.dump({"n_gpus": world, "dtype": "bf16", "rows": rows}, f, indent=1)
    dist.destroy_process_group()
    comm.finalize()


if __name__ == "__main__":
    main()
