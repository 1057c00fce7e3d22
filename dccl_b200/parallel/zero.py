"""Data parallelism with the optimizer state split over the ranks (ZeRO stage 1 / 2 style).

The gradient all-reduce of plain data parallelism is a reduce-scatter followed by an all-gather (the
original builds its ring all-reduce exactly so, reference src/core/all_reduce_ring.cpp:8-79). Here the
optimizer step sits between the two halves: every rank reduces only its 1/world slice of the flat gradient,
updates the matching slice of the parameters with its own slice of the optimizer state, and the updated
slices are gathered. Communication volume is that of one all-reduce; optimizer memory and update work
drop to 1/world per rank.

    params -> one flat buffer per dtype (padded to world x 16 bytes), ``p.data`` and ``p.grad`` are views
    step:    reduce_scatter(avg) flat_grad -> grad slice (fp32 copy when the parameters are 16-bit)
             inner optimizer on the master slice (fp32)
             all_gather the updated slice (cast back) into the flat parameter buffer

With ``comm.world == 1`` this is the inner optimizer on a flat buffer. CPU tensors use the host path, CUDA
tensors the device kernels on the current stream; on GPUs with NVSwitch multicast the flat buffers live in
symmetric memory (``symmetric=True``), so that both collectives run zero-copy through the switch. Call
``close()`` before the communicator is finalized to give that memory back.
"""
import torch


class ShardedOptimizer:
    """optimizer_cls(params, **kwargs) is built over ONE tensor per dtype: this rank's fp32 master slice."""

    def __init__(self, params, comm, optimizer_cls=torch.optim.AdamW, symmetric=True, **kwargs):
        self.comm = comm
        self._sym = []
        params = [p for p in params if p.requires_grad]
        if not params:
            raise ValueError("no trainable parameters")
        n, r = comm.world, comm.rank
        self.groups = []
        by_dtype = {}
        for p in params:
            by_dtype.setdefault((p.dtype, p.device), []).append(p)
        masters = []
        for (dtype, device), plist in by_dtype.items():
            itemsize = torch.empty((), dtype=dtype).element_size()
            align = 16 // itemsize
            offs, total = [], 0
            for p in plist:
                offs.append(total)
                total += -(-p.numel() // align) * align            # every view starts 16-byte aligned
            per = -(-total // (n * align)) * align                  # slice length, a whole number of 16-byte vectors
            if symmetric and device.type == "cuda" and n > 1 and comm.has_multicast:
                flat = comm.symmetric_empty(per * n, dtype, device.index).zero_()
                grad = comm.symmetric_empty(per * n, dtype, device.index).zero_()
                self._sym += [flat, grad]
            else:
                flat = torch.zeros(per * n, dtype=dtype, device=device)
                grad = torch.zeros(per * n, dtype=dtype, device=device)
            for p, off in zip(plist, offs):
                flat[off:off + p.numel()].copy_(p.data.reshape(-1))
                p.data = flat[off:off + p.numel()].view_as(p)
                p.grad = grad[off:off + p.numel()].view_as(p)
            master = flat[r * per:(r + 1) * per].detach().clone().float().requires_grad_(True)
            master.grad = torch.zeros_like(master)
            masters.append(master)
            self.groups.append({"flat": flat, "grad": grad, "per": per, "master": master, "params": plist,
                                "grad_slice": torch.empty(per, dtype=dtype, device=device),
                                "out_slice": torch.empty(per, dtype=dtype, device=device)})
        self.inner = optimizer_cls(masters, **kwargs)

    def zero_grad(self):
        for g in self.groups:
            g["grad"].zero_()

    def step(self):
        comm, n = self.comm, self.comm.world
        for g in self.groups:
            if n > 1:
                comm.reduce_scatter(g["grad"], g["grad_slice"], op="avg")
                g["master"].grad.copy_(g["grad_slice"])
            else:
                g["master"].grad.copy_(g["grad"])
        self.inner.step()
        for g in self.groups:
            if n > 1:
                g["out_slice"].copy_(g["master"].detach())
                comm.all_gather(g["out_slice"], g["flat"])
            else:
                g["flat"].copy_(g["master"].detach())

    def close(self):
        """Give symmetric buffers back (collective). The parameters keep their values in ordinary memory."""
        if not self._sym:
            return
        torch.cuda.synchronize()
        for g in self.groups:
            keep = g["flat"].clone()
            off = 0
            for p in g["params"]:
                # same layout as in __init__: every view starts 16-byte aligned
                align = 16 // keep.element_size()
                p.data = keep[off:off + p.numel()].view_as(p)
                p.grad = None
                off += -(-p.numel() // align) * align
            g["flat"], g["grad"] = keep, torch.zeros_like(keep)
        for t in self._sym:
            self.comm.free_symmetric(t)
        self._sym = []

    def state_bytes(self):
        """Bytes of optimizer state held by this rank (for reports and tests)."""
        total = 0
        for st in self.inner.state.values():
            for v in st.values():
                if torch.is_tensor(v):
                    total += v.numel() * v.element_size()
        return total
