#!/usr/bin/env python
"""Tensor-parallel training benchmark: the Llama-style decoder with heads and feed-forward columns dealt out over
the GPUs (``dccl_b200.models.llama_tp``), two activation all-reduces per block forward and two backward.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
           benchmarks/train_tp.py --backend dccl
    ... benchmarks/train_tp.py --backend nccl        # the same layers, collectives through stock NCCL
    ... benchmarks/train_tp.py --backend dccl --in-place-reduce   # all-reduces zero-copy on symmetric buffers
    ... benchmarks/train_tp.py --backend dccl --sequence-parallel # all-gather + reduce-scatter instead of all-reduce

Where the data-parallel benchmark (train_ddp.py) hides a few large all-reduces behind backward, this one puts
4 x layers all-reduces of batch x seq x hidden activations (64 MB in bf16 at the default shape) on the critical
path: step time minus the time of the same step with the collectives switched off is the communication time
itself. Every rank sees the same tokens; every step copies them from pinned host memory, runs forward, backward,
the optimizer step on the rank's slices, and reads the loss back. Reports tokens/s (CUDA-event time, max over ranks).
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from dccl_b200.models.llama import LlamaConfig, LlamaDecoder  # noqa: E402
from dccl_b200.models.llama_tp import shard  # noqa: E402


class NoComm:
    """Stands in for the communicator when the collectives are switched off: same shapes, no data moved."""

    def __init__(self, comm):
        self.rank, self.world = comm.rank, comm.world

    def all_reduce(self, send, recv=None, op="sum", stream=None):
        recv = send if recv is None else recv
        if recv is not send:
            recv.copy_(send)
        return recv

    def all_gather(self, send, recv, stream=None):
        recv.view(self.world, -1).copy_(send.reshape(1, -1).expand(self.world, -1))
        return recv

    def reduce_scatter(self, send, recv, op="sum", stream=None):
        recv.view(-1).copy_(send.view(self.world, -1)[self.rank])
        return recv


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="dccl", choices=["dccl", "nccl"])
    ap.add_argument("--model", default="1b", choices=["1b", "tiny"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--in-place-reduce", action="store_true",
                    help="block exits write their product into symmetric buffers that the switch reduces in place (dccl only)")
    ap.add_argument("--vocab-parallel", action="store_true", help="embedding, head and loss split over the vocabulary as well")
    ap.add_argument("--sequence-parallel", action="store_true",
                    help="activations between the blocks split along the sequence: all-gather + reduce-scatter instead of all-reduce")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = LlamaConfig.tinyllama_1b() if args.model == "1b" else LlamaConfig.tiny()
    if cfg.kv_heads % world:
        cfg.kv_heads = world if cfg.heads % world == 0 else cfg.kv_heads      # the default shape has 4 KV heads
    seq = min(args.seq, cfg.max_seq)

    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29535")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)       # timing reductions, and the comparison arm
    if args.backend == "dccl":
        from dccl_b200 import Communicator
        comm = Communicator(device=local)
    else:
        from dccl_b200.parallel.torch_comm import TorchDistCommunicator
        comm = TorchDistCommunicator()

    torch.manual_seed(0)                                                            # the same unsplit weights on every rank
    model = shard(LlamaDecoder(cfg).to(dev).to(torch.bfloat16), comm, in_place_reduce=args.in_place_reduce and args.backend == "dccl",
                  vocab_parallel=args.vocab_parallel, sequence_parallel=args.sequence_parallel)
    params = [p for p in model.parameters()]
    opt = torch.optim.AdamW(params, lr=1e-4, fused=True)
    host_tokens = torch.randint(0, cfg.vocab_size, (args.batch, seq + 1), generator=torch.Generator().manual_seed(1)).pin_memory()
    tokens = torch.empty_like(host_tokens, device=dev)
    losses = []
    off = NoComm(comm)

    def set_comm(c):
        for blk in model.blocks:
            blk.comm = c
            blk.attn.comm = c

    def step():
        tokens.copy_(host_tokens, non_blocking=True)
        loss = model.loss(tokens)
        loss.backward()
        model.sync_replicated_grads()       # sequence parallel only; nothing otherwise
        opt.step()
        opt.zero_grad(set_to_none=False)
        losses.append(loss.item())

    def timed(steps):
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(args.warmup):
        step()
    l0 = comm.launches if args.backend == "dccl" else 0
    ms = timed(args.steps)
    launches = (comm.launches - l0) if args.backend == "dccl" else 0
    final_loss = losses[-1]
    set_comm(off)
    ms_off = timed(max(3, args.steps // 2)) if world > 1 else ms
    set_comm(comm)
    tokens_per_step = args.batch * seq
    act_bytes = args.batch * seq * cfg.hidden * 2
    if rank == 0:
        print(json.dumps({
            "metric": "tp_tokens_per_s", "value": round(tokens_per_step / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3), "ms_per_step_without_collectives": round(ms_off, 3),
            "comm_ms": round(max(0.0, ms - ms_off), 3), "allreduces_per_step": 4 * cfg.layers, "allreduce_bytes": act_bytes,
            "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic", "backend": args.backend,
            "gpu_launches": int(launches), "in_place_reduce": bool(args.in_place_reduce and args.backend == "dccl"),
            "e2e": {"h2d_bytes_per_step": host_tokens.numel() * 8, "d2h_bytes_per_step": 4, "included": True},
            "config": {"model": "llama-1.1b" if args.model == "1b" else "llama-tiny", "params": cfg.num_params(), "global_batch": args.batch,
                       "seq_len": seq, "parallelism": "tp%d" % world, "kv_heads": cfg.kv_heads, "vocab_parallel": bool(args.vocab_parallel), "sequence_parallel": bool(args.sequence_parallel), "optimizer": "AdamW fused, bf16 params"},
            "final_loss": round(final_loss, 4), "final_loss_is_rank0_share": bool(args.sequence_parallel)}))
    model.close()
    dist.destroy_process_group()
    if args.backend == "dccl":
        comm.finalize()


if __name__ == "__main__":
    main()
