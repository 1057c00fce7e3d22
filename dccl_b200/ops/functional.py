"""Differentiable collectives on torch tensors.

The library itself stops at the collective calls (like the original, whose API ends at
reference include/dccl/dccl.hpp:143-420); tensor-, sequence- and expert-parallel layers need the same
calls with a backward pass. Every function here runs one collective of a ``Communicator`` in forward
and the adjoint collective in backward:

    =====================  ==========================  ==========================
    function               forward                     backward
    =====================  ==========================  ==========================
    all_reduce             all-reduce (sum / avg)      all-reduce (same operator)
    all_gather             all-gather along ``dim``    reduce-scatter (sum)
    reduce_scatter         reduce-scatter (sum / avg)  all-gather (scaled for avg)
    all_to_all             all-to-all, equal blocks    all-to-all
    broadcast              broadcast from ``root``     reduce (sum) to ``root``
    copy_to_region         identity                    all-reduce (sum)
    reduce_from_region     all-reduce (sum)            identity
    send                   send to ``peer``            receive the gradient from ``peer``
    recv                   receive from ``peer``       send the gradient to ``peer``
    ring_shift             to rank+k, from rank-k      to rank-k, from rank+k
    =====================  ==========================  ==========================

The first five are exact adjoints when every rank goes on to use its output in its own loss term.
``copy_to_region`` / ``reduce_from_region`` are the pair a tensor-parallel block is built from: its
input is the same on every rank and its loss is computed once, so the reduction belongs to the
backward of the entry and to the forward of the exit.

CUDA tensors run the device kernels on the current stream, CPU tensors the shared-memory host path,
so the same model code is tested without a GPU.

A collective in backward is still a collective: every rank has to reach it. An output that a rank does
not use must stay in that rank's autograd graph all the same (add ``0.0 * y.sum()`` to something that is
used), or the other ranks wait for an exchange that this rank never starts.
"""
import torch

_default = None


def set_default_communicator(comm):
    """The communicator used when a call does not name one."""
    global _default
    _default = comm


def get_default_communicator():
    if _default is None:
        raise RuntimeError("no communicator: pass comm= or call dccl_b200.ops.set_default_communicator first")
    return _default


def _comm(comm):
    return comm if comm is not None else get_default_communicator()


def _move_in(x, dim):
    """`dim` to the front, contiguous: the collectives cut and join along the first dimension."""
    return x.movedim(dim, 0).contiguous() if dim != 0 else x.contiguous()


def _move_out(y, dim):
    return y.movedim(0, dim) if dim != 0 else y


def _gather_dim0(comm, x):
    out = x.new_empty((comm.world * x.shape[0],) + tuple(x.shape[1:]))
    comm.all_gather(x, out)
    return out


def _scatter_dim0(comm, x, op):
    if x.shape[0] % comm.world:
        raise ValueError("reduce_scatter: dimension of size %d does not split over %d ranks" % (x.shape[0], comm.world))
    out = x.new_empty((x.shape[0] // comm.world,) + tuple(x.shape[1:]))
    comm.reduce_scatter(x, out, op=op)
    return out


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm, op):
        ctx.comm, ctx.op = comm, op
        x = x.contiguous()
        return comm.all_reduce(x, torch.empty_like(x), op=op)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        return ctx.comm.all_reduce(g, torch.empty_like(g), op=ctx.op), None, None


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm, dim):
        ctx.comm, ctx.dim = comm, dim
        return _move_out(_gather_dim0(comm, _move_in(x, dim)), dim)

    @staticmethod
    def backward(ctx, g):
        return _move_out(_scatter_dim0(ctx.comm, _move_in(g, ctx.dim), "sum"), ctx.dim), None, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm, dim, op):
        ctx.comm, ctx.dim, ctx.op = comm, dim, op
        return _move_out(_scatter_dim0(comm, _move_in(x, dim), op), dim)

    @staticmethod
    def backward(ctx, g):
        out = _gather_dim0(ctx.comm, _move_in(g, ctx.dim))
        if ctx.op == "avg":
            out = out / ctx.comm.world
        return _move_out(out, ctx.dim), None, None, None


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        x = x.contiguous()
        if x.shape[0] % comm.world:
            raise ValueError("all_to_all: first dimension of size %d does not split over %d ranks" % (x.shape[0], comm.world))
        return comm.all_to_all(x, torch.empty_like(x))

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        return ctx.comm.all_to_all(g, torch.empty_like(g)), None


class _AllToAllV(torch.autograd.Function):
    """Rows of `x` (first dimension) in per-peer runs of send_counts[p] rows; the result has recv_counts[p] rows from
    rank p, in rank order. Backward is the same exchange with the counts swapped."""

    @staticmethod
    def forward(ctx, x, comm, send_counts, recv_counts):
        ctx.comm, ctx.sc, ctx.rc = comm, list(send_counts), list(recv_counts)
        x = x.contiguous()
        row = 1
        for s in x.shape[1:]:
            row *= int(s)
        ctx.row = row
        out = x.new_empty((sum(ctx.rc),) + tuple(x.shape[1:]))
        comm.all_to_all(x, out, [c * row for c in ctx.sc], [c * row for c in ctx.rc])
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = g.new_empty((sum(ctx.sc),) + tuple(g.shape[1:]))
        ctx.comm.all_to_all(g, out, [c * ctx.row for c in ctx.rc], [c * ctx.row for c in ctx.sc])
        return out, None, None, None


class _Broadcast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm, root):
        ctx.comm, ctx.root = comm, root
        x = x.contiguous()
        return comm.broadcast(x, torch.empty_like(x), root=root)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        comm, root = ctx.comm, ctx.root
        if comm.rank == root:
            return comm.reduce(g, torch.empty_like(g), op="sum", root=root), None, None
        comm.reduce(g, None, op="sum", root=root)
        return torch.zeros_like(g), None, None


class _CopyToRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        return ctx.comm.all_reduce(g, torch.empty_like(g), op="sum"), None


class _ReduceFromRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        x = x.contiguous()
        return comm.all_reduce(x, torch.empty_like(x), op="sum")

    @staticmethod
    def backward(ctx, g):
        return g, None


class _Send(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm, peer):
        ctx.comm, ctx.peer, ctx.like = comm, peer, (x.shape, x.dtype, x.device)
        x = x.contiguous()
        comm.send(x, peer)
        return x.new_zeros(())

    @staticmethod
    def backward(ctx, g):
        shape, dtype, device = ctx.like
        grad = torch.empty(shape, dtype=dtype, device=device)
        ctx.comm.recv(grad, ctx.peer)
        return grad, None, None


class _Recv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, like, comm, peer):
        ctx.comm, ctx.peer = comm, peer
        out = torch.empty_like(like)
        return comm.recv(out, peer)

    @staticmethod
    def backward(ctx, g):
        ctx.comm.send(g.contiguous(), ctx.peer)
        return None, None, None


def _exchange(comm, x, to, frm):
    """x goes to rank `to`, the result comes from rank `frm`; one grouped call, so a ring of these cannot deadlock."""
    out = torch.empty_like(x)
    if to == comm.rank and frm == comm.rank:
        return out.copy_(x)
    comm.group_start()
    comm.send(x, to)
    comm.recv(out, frm)
    comm.group_end()
    return out


class _RingShift(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm, k):
        ctx.comm, ctx.k = comm, k
        n, r = comm.world, comm.rank
        return _exchange(comm, x.contiguous(), (r + k) % n, (r - k) % n)

    @staticmethod
    def backward(ctx, g):
        n, r, k = ctx.comm.world, ctx.comm.rank, ctx.k
        return _exchange(ctx.comm, g.contiguous(), (r - k) % n, (r + k) % n), None, None


def all_reduce(x, op="sum", comm=None):
    if op not in ("sum", "avg"):
        raise ValueError("differentiable all_reduce supports sum and avg")
    return _AllReduce.apply(x, _comm(comm), op)


def all_gather(x, dim=0, comm=None):
    """Every rank's `x` joined along `dim`, in rank order."""
    return _AllGather.apply(x, _comm(comm), dim % x.dim())


def reduce_scatter(x, dim=0, op="sum", comm=None):
    """Reduce over the ranks, keep block <rank> of the result along `dim`."""
    if op not in ("sum", "avg"):
        raise ValueError("differentiable reduce_scatter supports sum and avg")
    return _ReduceScatter.apply(x, _comm(comm), dim % x.dim(), op)


def all_to_all(x, send_counts=None, recv_counts=None, comm=None):
    """Block p of `x` (first dimension cut into world-size equal blocks) goes to rank p; block p of the result comes
    from rank p. With `send_counts` / `recv_counts` (rows per peer, both needed) the blocks have those sizes."""
    if send_counts is None and recv_counts is None:
        return _AllToAll.apply(x, _comm(comm))
    if send_counts is None or recv_counts is None:
        raise ValueError("all_to_all: give both send_counts and recv_counts")
    if sum(send_counts) != x.shape[0]:
        raise ValueError("all_to_all: send_counts add up to %d rows, the tensor has %d" % (sum(send_counts), x.shape[0]))
    return _AllToAllV.apply(x, _comm(comm), send_counts, recv_counts)


def broadcast(x, root=0, comm=None):
    return _Broadcast.apply(x, _comm(comm), root)


def send(x, peer, comm=None):
    """Send `x` to `peer` (the next pipeline stage). Returns a zero scalar that carries the graph: add it to this
    rank's loss (or call ``.backward()`` on it when the rank has no loss of its own) and backward receives the
    gradient of `x` from `peer` and continues into the graph that produced `x`."""
    return _Send.apply(x, _comm(comm), peer)


def recv(like, peer, comm=None):
    """Receive a tensor shaped like `like` from `peer` (the previous pipeline stage); backward sends its gradient
    back. `like` only gives shape, dtype and device."""
    like = like.detach().requires_grad_(True)      # the output must be part of a graph for backward to reach us
    return _Recv.apply(like, _comm(comm), peer)


def ring_shift(x, k=1, comm=None):
    """Every rank passes `x` to rank + k and gets the tensor of rank - k (same shape on all ranks)."""
    return _RingShift.apply(x, _comm(comm), k)


def copy_to_region(x, comm=None):
    """Entry of a tensor-parallel block: identity forward, all-reduce of the gradient backward."""
    return _CopyToRegion.apply(x, _comm(comm))


def reduce_from_region(x, comm=None):
    """Exit of a tensor-parallel block: all-reduce of the partial results forward, identity backward."""
    return _ReduceFromRegion.apply(x, _comm(comm))
