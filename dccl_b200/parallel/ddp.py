"""Data-parallel gradient reduction through the library.

Two ways in:

``GradientAllReducer(model, comm)``
    The native path. Gradients of all parameters live in a few flat bucket
    buffers (25 MB by default) that are allocated in SYMMETRIC memory, so the
    all-reduce of a bucket is the zero-copy switch variant: the NVSwitch reduces
    the buckets of all ranks in place, with the 1/world scale fused
    (``ncclAvg``). ``param.grad`` is a view into its bucket, autograd
    accumulates straight into it, and a bucket is launched on a side stream the
    moment its last gradient has been produced, while backward continues.

``register_ddp_hook(ddp_model, comm)``
    A communication hook for ``torch.nn.parallel.DistributedDataParallel``:
    DDP keeps its own bucketing, each bucket is averaged by the library on a
    side stream and handed back as a future.
"""
import torch

from ..comm import Communicator


class GradientAllReducer:
    def __init__(self, model, comm: Communicator, bucket_bytes=25 << 20, symmetric=True, op="avg"):
        self.comm = comm
        self.op = op
        self.enabled = True
        params = [p for p in model.parameters() if p.requires_grad]
        if not params:
            raise ValueError("model has no trainable parameters")
        self.device = params[0].device
        self.stream = torch.cuda.Stream(device=self.device, priority=-1) if self.device.type == "cuda" else None
        self._sym = []
        self.buckets = []      # dicts: buffer, params, pending, event
        self._bucket_of = {}
        # gradients arrive roughly in reverse parameter order, so buckets are filled in that order
        by_dtype = {}
        for p in reversed(params):
            by_dtype.setdefault(p.dtype, []).append(p)
        for dtype, plist in by_dtype.items():
            itemsize = torch.empty((), dtype=dtype).element_size()
            cur, cur_bytes = [], 0
            groups = []
            for p in plist:
                nbytes = -(-p.numel() * itemsize // 16) * 16     # every view starts 16-byte aligned
                if cur and cur_bytes + nbytes > bucket_bytes:
                    groups.append(cur)
                    cur, cur_bytes = [], 0
                cur.append(p)
                cur_bytes += nbytes
            if cur:
                groups.append(cur)
            for g in groups:
                offs, total = [], 0
                for p in g:
                    offs.append(total)
                    total += -(-p.numel() * itemsize // 16) * 16 // itemsize
                use_sym = symmetric and self.device.type == "cuda" and comm.world > 1 and comm.has_multicast
                if use_sym:
                    buf = comm.symmetric_empty(total, dtype, self.device.index)
                    self._sym.append(buf)
                else:
                    buf = torch.empty(total, dtype=dtype, device=self.device)
                buf.zero_()
                b = {"buffer": buf, "params": g, "pending": len(g), "event": None, "launched": False}
                self.buckets.append(b)
                for p, off in zip(g, offs):
                    p.grad = buf[off:off + p.numel()].view_as(p)
                    self._bucket_of[p] = b
        self._hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in params]

    def _on_grad(self, p):
        b = self._bucket_of[p]
        b["pending"] -= 1
        if b["pending"] == 0:
            self._launch(b)

    def _launch(self, b):
        b["launched"] = True
        if not self.enabled or self.comm.world == 1:
            return
        if self.stream is None:
            self.comm.all_reduce(b["buffer"], op=self.op)
            return
        ready = torch.cuda.Event()
        ready.record()                        # on the stream backward runs on
        self.stream.wait_event(ready)
        self.comm.all_reduce(b["buffer"], op=self.op, stream=self.stream)
        done = torch.cuda.Event()
        done.record(self.stream)
        b["event"] = done

    def finish(self):
        """Call after backward: launches buckets whose parameters got no gradient, then makes the current
        stream wait for every bucket. The host does not block."""
        for b in self.buckets:
            if not b["launched"]:
                self._launch(b)
        for b in self.buckets:
            if b["event"] is not None:
                torch.cuda.current_stream(self.device).wait_event(b["event"])
                b["event"] = None
            b["pending"] = len(b["params"])
            b["launched"] = False

    def zero_grad(self):
        """Zero all gradients with one fill per bucket (instead of one per parameter)."""
        for b in self.buckets:
            b["buffer"].zero_()

    def close(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        for t in self._sym:
            self.comm.free_symmetric(t)
        self._sym = []


class _HookState:
    def __init__(self, comm, device):
        self.comm = comm
        self.stream = torch.cuda.Stream(device=device, priority=-1)
        self.events = {}          # one "gradients of this bucket are ready" event per bucket, made once


def _ddp_hook(state, bucket):
    buf = bucket.buffer()
    fut = torch.futures.Future(devices=[buf.device])
    ready = state.events.get(bucket.index())
    if ready is None:
        ready = state.events[bucket.index()] = torch.cuda.Event()
    ready.record()
    state.stream.wait_event(ready)
    with torch.cuda.stream(state.stream):
        state.comm.all_reduce(buf, op="avg", stream=state.stream)
        # The future keeps the bucket alive and records the side stream; DDP waits on it before it uses the bucket,
        # and the bucket is DDP's own long-lived buffer, so the allocator needs no note about the side stream.
        fut.set_result(buf)
    return fut


def register_ddp_hook(ddp_model, comm, device=None):
    """Route DDP's bucketed gradient all-reduce through ``comm`` (average fused into the kernel)."""
    device = device if device is not None else next(ddp_model.parameters()).device
    state = _HookState(comm, device)
    ddp_model.register_comm_hook(state, _ddp_hook)
    return state
