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
tensors the device kernels on the current stream.
"""
import torch


class ShardedOptimizer:
    """optimizer_cls(params, **kwargs) is built over ONE tensor per dtype: this rank's fp32 master slice."""

    def __init__(self, params, comm, optimizer_cls=torch.optim.AdamW, **kwargs):
        self.comm = comm
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

    def state_bytes(self):
        """Bytes of optimizer state held by this rank (for reports and tests)."""
        total = 0
        for st in self.inner.state.values():
            for v in st.values():
                if torch.is_tensor(v):
                    total += v.numel() * v.element_size()
        return total
