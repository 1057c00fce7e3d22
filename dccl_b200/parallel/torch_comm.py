"""The calls of ``dccl_b200.Communicator`` that the differentiable collectives use, served by ``torch.distributed``.

``TorchDistCommunicator(group)`` lets the layers of ``dccl_b200.ops`` / ``dccl_b200.parallel`` run over any
``torch.distributed`` backend (stock NCCL on GPUs, gloo on CPUs): the comparison arm of the benchmarks and a
differential check of the layers themselves. Only the tensor forms are covered (torch tensors, contiguous).
"""
import torch
import torch.distributed as dist

_OPS = {"sum": dist.ReduceOp.SUM, "prod": dist.ReduceOp.PRODUCT, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN,
        "avg": dist.ReduceOp.AVG}


class TorchDistCommunicator:
    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.has_multicast = False
        # gloo has no averaging operator: sum, then scale
        self._no_avg = dist.get_backend(group) == "gloo"

    def _reduce_op(self, op):
        return dist.ReduceOp.SUM if (op == "avg" and self._no_avg) else _OPS[op]

    def _fix_avg(self, t, op):
        if op == "avg" and self._no_avg:
            t.div_(self.world)
        return t

    def all_reduce(self, send, recv=None, op="sum", stream=None):
        recv = send if recv is None else recv
        if recv is not send:
            recv.copy_(send)
        dist.all_reduce(recv, op=self._reduce_op(op), group=self.group)
        return self._fix_avg(recv, op)

    def reduce_scatter(self, send, recv, op="sum", stream=None):
        if self._no_avg:      # gloo has no reduce-scatter either: all-reduce a copy and keep the own block
            tmp = send.clone()
            dist.all_reduce(tmp, op=self._reduce_op(op), group=self.group)
            recv.copy_(tmp.reshape(self.world, -1)[self.rank].view_as(recv))
            return self._fix_avg(recv, op)
        dist.reduce_scatter_tensor(recv, send, op=_OPS[op], group=self.group)
        return recv

    def all_gather(self, send, recv, stream=None):
        dist.all_gather_into_tensor(recv, send, group=self.group)
        return recv

    def broadcast(self, send, recv=None, root=0, stream=None):
        recv = send if recv is None else recv
        if recv is not send and self.rank == root:
            recv.copy_(send)
        dist.broadcast(recv, src=dist.get_global_rank(self.group, root) if self.group is not None else root, group=self.group)
        return recv

    def reduce(self, send, recv=None, op="sum", root=0, stream=None):
        tmp = send.clone()
        dist.reduce(tmp, dst=dist.get_global_rank(self.group, root) if self.group is not None else root, op=self._reduce_op(op),
                    group=self.group)
        if self.rank == root:
            recv = send if recv is None else recv
            recv.copy_(tmp)
            return self._fix_avg(recv, op)
        return recv

    def all_to_all(self, send, recv, send_counts=None, recv_counts=None, stream=None):
        if send_counts is None and recv_counts is None:
            dist.all_to_all_single(recv.view(-1), send.view(-1), group=self.group)
        else:
            dist.all_to_all_single(recv.view(-1), send.view(-1), output_split_sizes=list(recv_counts), input_split_sizes=list(send_counts),
                                   group=self.group)
        return recv

    def send(self, x, peer, stream=None):
        self._pending = getattr(self, "_pending", [])
        self._pending.append(dist.P2POp(dist.isend, x, dist.get_global_rank(self.group, peer) if self.group is not None else peer, self.group))
        self._flush()

    def recv(self, x, peer, stream=None):
        self._pending = getattr(self, "_pending", [])
        self._pending.append(dist.P2POp(dist.irecv, x, dist.get_global_rank(self.group, peer) if self.group is not None else peer, self.group))
        self._flush()
        return x

    # send / recv between group_start() and group_end() are issued together (a ring of them cannot deadlock)
    _depth = 0

    def group_start(self):
        self._depth += 1

    def group_end(self):
        self._depth -= 1
        self._flush()

    def _flush(self):
        if self._depth > 0 or not getattr(self, "_pending", None):
            return
        ops, self._pending = self._pending, []
        for w in dist.batch_isend_irecv(ops):
            w.wait()

    def finalize(self):
        pass
