#!/usr/bin/env python
"""Data-parallel training benchmark: Llama-style decoder, bf16 gradients in 25 MB buckets, averaged
by the library while backward still runs.

    python benchmarks/train_ddp.py --backend dccl --steps 10 --warmup 3                      # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
           --master-port 29500 benchmarks/train_ddp.py --backend dccl

Shape of the benchmark configuration: 22 layers, hidden 2048, 32 heads, 4 KV heads, FFN 5632,
vocabulary 32000 (1.1 B parameters), random init, synthetic tokens uniform over the vocabulary,
sequence 2048, micro-batch 8 per GPU. Every step copies its tokens from pinned host memory, runs
forward, backward (with the gradient all-reduce overlapped), the optimizer step, and reads the loss
back to the host. Reports tokens/s over all GPUs (CUDA-event time, max over ranks) and the exposed
communication time = step time minus the time of the same step with the all-reduce switched off.

--backend dccl      GradientAllReducer: symmetric-memory buckets, zero-copy switch reduction
--backend dccl_ddp  torch DistributedDataParallel over process group "dccl" with the library's comm hook
--backend nccl      torch DistributedDataParallel over stock NCCL (comparison)
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from dccl_b200.models.llama import LlamaConfig, LlamaDecoder  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="dccl", choices=["dccl", "dccl_ddp", "nccl"])
    ap.add_argument("--model", default="1b", choices=["1b", "tiny"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--bucket-mb", type=int, default=25)
    ap.add_argument("--plain-buckets", action="store_true",
                    help="dccl_ddp: leave DDP's gradient buckets in ordinary memory (default: they come from a memory pool of symmetric memory)")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = LlamaConfig.tinyllama_1b() if args.model == "1b" else LlamaConfig.tiny()
    seq = min(args.seq, cfg.max_seq)
    torch.manual_seed(0)
    model = LlamaDecoder(cfg).to(dev).to(torch.bfloat16)

    comm = reducer = ddp = None
    import torch.distributed as dist
    if args.backend == "dccl":
        from dccl_b200 import Communicator
        from dccl_b200.parallel.ddp import GradientAllReducer
        comm = Communicator(device=local)
        reducer = GradientAllReducer(model, comm, bucket_bytes=args.bucket_mb << 20)
        net = model
    else:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        if args.backend == "dccl_ddp":
            import dccl_b200.parallel.process_group as pgmod
            from dccl_b200.parallel.ddp import register_ddp_hook
            dist.init_process_group("dccl", rank=rank, world_size=world)
            comm = pgmod.communicator()
            comm.bind_device(local)
        else:
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        if args.backend == "dccl_ddp" and not args.plain_buckets and world > 1:
            # DDP allocates its gradient buckets while it is constructed: inside the pool they become symmetric memory,
            # which the switch reduces in place
            pool = comm.symmetric_mem_pool()
            with torch.cuda.use_mem_pool(pool):
                ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True)
        else:
            ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True)
        if args.backend == "dccl_ddp":
            register_ddp_hook(ddp, comm, dev)
        net = ddp
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)

    host_tokens = torch.randint(0, cfg.vocab_size, (args.batch, seq + 1)).pin_memory()
    tokens = torch.empty_like(host_tokens, device=dev)
    losses = []

    def step(comm_on=True):
        if reducer is not None:
            reducer.enabled = comm_on
        tokens.copy_(host_tokens, non_blocking=True)
        if ddp is not None and not comm_on:
            with ddp.no_sync():
                loss = ddp.module.loss(tokens)
                loss.backward()
        else:
            loss = net.loss(tokens) if ddp is None else _ddp_loss(ddp, tokens)
            loss.backward()
        if reducer is not None:
            reducer.finish()
        opt.step()
        if reducer is not None:
            reducer.zero_grad()
        else:
            opt.zero_grad(set_to_none=False)
        losses.append(loss.item())     # device -> host read of the step's result

    def _ddp_loss(d, t):
        logits = d(t[:, :-1])
        return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), t[:, 1:].reshape(-1))

    def barrier():
        if comm is not None and args.backend == "dccl":
            import numpy as np
            a = np.zeros(1, dtype=np.int32)
            comm.all_reduce(a)
        else:
            dist.barrier()

    def host_max(x):
        if comm is not None and args.backend == "dccl":
            import numpy as np
            a = np.array([x], dtype=np.float64)
            comm.all_reduce(a, op="max")
            return float(a[0])
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(comm_on, steps):
        torch.cuda.synchronize()
        barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step(comm_on)
        e1.record()
        torch.cuda.synchronize()
        barrier()
        return host_max(e0.elapsed_time(e1) / steps)

    for _ in range(args.warmup):
        step(True)
    l0 = comm.launches if comm is not None else 0
    ms = timed(True, args.steps)
    launches = (comm.launches - l0) if comm is not None else 0
    ms_nocomm = timed(False, max(3, args.steps // 2)) if world > 1 else ms
    tokens_per_step = world * args.batch * seq
    if rank == 0:
        print(json.dumps({
            "metric": "ddp_tokens_per_s", "value": round(tokens_per_step / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3), "ms_per_step_without_allreduce": round(ms_nocomm, 3),
            "exposed_comm_ms": round(max(0.0, ms - ms_nocomm), 3), "higher_is_better": True, "scaling": "weak", "dtype": "bf16",
            "data": "synthetic", "backend": args.backend, "gpu_launches": int(launches),
            "e2e": {"h2d_bytes_per_step": host_tokens.numel() * 8, "d2h_bytes_per_step": 4, "included": True},
            "config": {"model": "llama-1.1b" if args.model == "1b" else "llama-tiny", "params": cfg.num_params(), "global_batch": world * args.batch,
                       "seq_len": seq, "parallelism": "dp%d" % world, "bucket_mb": args.bucket_mb, "optimizer": "AdamW fused, bf16 params"},
            "final_loss": round(losses[-1], 4)}))
    if reducer is not None:
        reducer.close()
    if args.backend == "dccl":
        comm.finalize()
    else:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
