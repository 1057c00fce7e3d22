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
                 dtype=torch.float32, device="cpu", pool=None):
        super().__init__()
        if in_features % comm.world:
            raise ValueError("in_features must split evenly over the ranks")
        self.comm, self.sequence_parallel, self.seq_dim = comm, sequence_parallel, seq_dim
        self.pool = pool          # a SymmetricPool: the product is written into it and reduced in place (not with sequence_parallel)
        per = in_features // comm.world
        w, b = _full_weight(out_features, in_features, seed, dtype, device)
        self.weight = torch.nn.Parameter(w[:, comm.rank * per:(comm.rank + 1) * per].clone())
        # the bias is replicated; under sequence parallelism its gradient is a partial sum per rank and has to be
        # all-reduced with the other replicated parameters (sync_replicated_grads)
        self.bias = torch.nn.Parameter(b.clone()) if bias else None

    def forward(self, x):
        if self.pool is not None and not self.sequence_parallel:
            y = row_linear_reduce_in_place(x, self.weight, self.comm, self.pool)
            return y + self.bias if self.bias is not None else y.clone()       # a fresh tensor: the pool buffer is reused
        y = torch.nn.functional.linear(x, self.weight)
        y = F.reduce_scatter(y, self.seq_dim, "sum", self.comm) if self.sequence_parallel else F.reduce_from_region(y, self.comm)
        return y + self.bias if self.bias is not None else y


class SymmetricPool:
    """A few reusable output buffers in symmetric memory (``dcclMemAlloc``), handed out round robin.

    A matrix product that writes its result straight into one of them can be all-reduced IN PLACE by the NVSwitch
    (``multimem.ld_reduce`` / ``multimem.st`` on the buffer itself): no staging copy in, none out. A buffer is
    reused after ``depth`` further requests, so the result must be consumed before that (a residual add right
    after the layer does). Without multicast, on CPU tensors or with one rank the buffers are ordinary tensors
    and only the in-place form remains. ``close()`` gives the memory back (collective).
    """

    def __init__(self, comm, depth=4):
        self.comm, self.depth = comm, depth
        self._bufs, self._next, self._numel, self._dtype = [], 0, 0, None

    def _symmetric(self, device):
        return device.type == "cuda" and self.comm.world > 1 and getattr(self.comm, "has_multicast", False)

    def take(self, shape, dtype, device):
        numel = 1
        for s in shape:
            numel *= int(s)
        if numel > self._numel or dtype != self._dtype:          # first use, or a larger request: every rank sees the same shapes
            self.close()
            self._numel, self._dtype = numel, dtype
            for _ in range(self.depth):
                if self._symmetric(device):
                    self._bufs.append(self.comm.symmetric_empty(numel, dtype, device.index))
                else:
                    self._bufs.append(torch.empty(numel, dtype=dtype, device=device))
        buf = self._bufs[self._next]
        self._next = (self._next + 1) % self.depth
        return buf[:numel].view(shape)

    def close(self):
        for b in self._bufs:
            if hasattr(b, "_dccl_ptr"):
                self.comm.free_symmetric(b)
        self._bufs, self._next, self._numel = [], 0, 0


class _RowLinearReduceInPlace(torch.autograd.Function):
    """y = all_reduce(x W^T) with the product written into a pool buffer and reduced there."""

    @staticmethod
    def forward(ctx, x, weight, comm, pool):
        ctx.save_for_backward(x, weight)
        out = pool.take(tuple(x.shape[:-1]) + (weight.shape[0],), x.dtype, x.device)
        torch.matmul(x, weight.t(), out=out)
        comm.all_reduce(out, op="sum")
        return out

    @staticmethod
    def backward(ctx, g):
        x, weight = ctx.saved_tensors
        gx = torch.matmul(g, weight) if ctx.needs_input_grad[0] else None
        gw = torch.matmul(g.reshape(-1, g.shape[-1]).t(), x.reshape(-1, x.shape[-1])) if ctx.needs_input_grad[1] else None
        return gx, gw, None, None


def row_linear_reduce_in_place(x, weight, comm, pool):
    """Exit of a tensor-parallel block without a staging copy: ``x @ weight.T`` lands in a buffer of `pool` and the
    ranks' partial products are summed there. The result is only valid until the pool hands the buffer out again."""
    return _RowLinearReduceInPlace.apply(x, weight, comm, pool)


class _ColumnLinearsReduceGradInPlace(torch.autograd.Function):
    """(x W_1^T, ..., x W_k^T) for the column-parallel layers that share the input of a tensor-parallel block; in
    backward the input gradient sum_i g_i W_i is accumulated in a pool buffer and summed over the ranks there."""

    @staticmethod
    def forward(ctx, x, comm, pool, *weights):
        ctx.comm, ctx.pool = comm, pool
        ctx.save_for_backward(x, *weights)
        return tuple(torch.matmul(x, w.t()) for w in weights)

    @staticmethod
    def backward(ctx, *gs):
        x, *weights = ctx.saved_tensors
        gx = None
        if ctx.needs_input_grad[0]:
            gx = ctx.pool.take(tuple(x.shape), x.dtype, x.device)
            flat = gx.view(-1, x.shape[-1])
            torch.matmul(gs[0].reshape(-1, gs[0].shape[-1]), weights[0], out=flat)
            for g, w in zip(gs[1:], weights[1:]):
                flat.addmm_(g.reshape(-1, g.shape[-1]), w)
            ctx.comm.all_reduce(gx, op="sum")
        x2 = x.reshape(-1, x.shape[-1])
        gws = tuple(torch.matmul(g.reshape(-1, g.shape[-1]).t(), x2) for g in gs)
        return (gx, None, None) + gws


def column_linears_reduce_grad_in_place(x, weights, comm, pool):
    """Entry of a tensor-parallel block without a staging copy in backward: returns ``x @ W.T`` for every W in
    `weights` (no bias); the gradient of `x` is built in a buffer of `pool` and summed over the ranks in place. It is
    only valid until the pool hands the buffer out again (the backward of the preceding norm consumes it at once)."""
    return _ColumnLinearsReduceGradInPlace.apply(x, comm, pool, *weights)


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
