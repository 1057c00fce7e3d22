"""Tensor- and sequence-parallel linear layers over the differentiable collectives of ``dccl_b200.ops``.

The original is a collectives library without model code; these layers are the smallest useful consumers of
its all-reduce / all-gather / reduce-scatter (reference src/core/dccl.cpp:344-501, 551-698, 849-862) inside a
model: a column-parallel layer followed by a row-parallel one needs one all-reduce forward and one backward
(tensor parallel), or an all-gather and a reduce-scatter each way when the activations between blocks are kept
split along the sequence (sequence parallel).

    up = ColumnParallelLinear(d, 4 * d, comm)            # weight rows [rank * 4d/n, (rank+1) * 4d/n)
    down = RowParallelLinear(4 * d, d, comm)             # weight columns likewise
    y = down(torch.nn.functional.gelu(up(x)))            # x, y: the same on every rank

Weights are created for the whole layer from the given generator seed and cut, so that every world size
starts from the same model (and a test can compare with the unsplit layer).
"""
import math

import torch

from ..ops import functional as F


def _full_weight(out_features, in_features, seed, dtype, device):
    g = torch.Generator(device="cpu").manual_seed(seed)
    w = torch.empty(out_features, in_features, dtype=torch.float32)
    bound = 1.0 / math.sqrt(in_features)
    w.uniform_(-bound, bound, generator=g)
    b = torch.empty(out_features, dtype=torch.float32).uniform_(-bound, bound, generator=g)
    return w.to(device=device, dtype=dtype), b.to(device=device, dtype=dtype)


class ColumnParallelLinear(torch.nn.Module):
    """y = x W^T + b with the output features split over the ranks; the result stays split.

    sequence_parallel: the input arrives split along ``seq_dim`` and is all-gathered first (backward:
    reduce-scatter); otherwise the input is the same on every rank (backward: all-reduce of its gradient).
    """

    def __init__(self, in_features, out_features, comm, bias=True, sequence_parallel=False, seq_dim=0, seed=0,
                 dtype=torch.float32, device="cpu"):
        super().__init__()
        if out_features % comm.world:
            raise ValueError("out_features must split evenly over the ranks")
        self.comm, self.sequence_parallel, self.seq_dim = comm, sequence_parallel, seq_dim
        per = out_features // comm.world
        w, b = _full_weight(out_features, in_features, seed, dtype, device)
        self.weight = torch.nn.Parameter(w[comm.rank * per:(comm.rank + 1) * per].clone())
        self.bias = torch.nn.Parameter(b[comm.rank * per:(comm.rank + 1) * per].clone()) if bias else None

    def forward(self, x):
        x = F.all_gather(x, self.seq_dim, self.comm) if self.sequence_parallel else F.copy_to_region(x, self.comm)
        return torch.nn.functional.linear(x, self.weight, self.bias)


class RowParallelLinear(torch.nn.Module):
    """y = x W^T + b with the input features split over the ranks (x is the split output of a column-parallel
    layer); the partial products are summed over the ranks.

    sequence_parallel: the sum is a reduce-scatter along ``seq_dim`` and the result stays split; otherwise an
    all-reduce and the result is the same on every rank. The bias is added once, after the sum.
    """

    def __init__(self, in_features, out_features, comm, bias=True, sequence_parallel=False, seq_dim=0, seed=1,
                 dtype=torch.float32, device="cpu"):
        super().__init__()
        if in_features % comm.world:
            raise ValueError("in_features must split evenly over the ranks")
        self.comm, self.sequence_parallel, self.seq_dim = comm, sequence_parallel, seq_dim
        per = in_features // comm.world
        w, b = _full_weight(out_features, in_features, seed, dtype, device)
        self.weight = torch.nn.Parameter(w[:, comm.rank * per:(comm.rank + 1) * per].clone())
        # the bias is replicated; under sequence parallelism its gradient is a partial sum per rank and has to be
        # all-reduced with the other replicated parameters (sync_replicated_grads)
        self.bias = torch.nn.Parameter(b.clone()) if bias else None

    def forward(self, x):
        y = torch.nn.functional.linear(x, self.weight)
        y = F.reduce_scatter(y, self.seq_dim, "sum", self.comm) if self.sequence_parallel else F.reduce_from_region(y, self.comm)
        return y + self.bias if self.bias is not None else y


def sync_replicated_grads(params, comm):
    """Sum the gradients of parameters that are replicated over the ranks but saw only a part of the batch or
    sequence (biases and norms under sequence parallelism). One all-reduce over the flattened gradients."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1) for g in grads])
    comm.all_reduce(flat, op="sum")
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()
