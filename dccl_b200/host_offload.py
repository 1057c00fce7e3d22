"""All-reduce of HOST buffers through the GPUs, with the three legs overlapped.

The original reduces host buffers on the CPUs, over its RDMA transport (reference src/core/dccl.cpp:344-501, host
branch). On an NVLink box the fast way to reduce pinned host memory is through the GPUs: copy a piece to the device,
let the NVSwitch reduce it, copy it back. Done one whole message after the other the three legs add up, and the two PCIe
copies are most of the time. ``HostAllReducer`` cuts the message into chunks and keeps three of them in flight on
three streams: while chunk k is being reduced, chunk k+1 travels host->device and chunk k-1 device->host, so the step
costs about one PCIe direction instead of two plus the collective (PCIe is full duplex).

The device slots are symmetric memory (``dcclMemAlloc``), allocated once per reducer, so the switch reduces them in
place. All ranks must create the reducer and call it in the same order, like any collective.

    red = HostAllReducer(comm, max_bytes=1 << 30)
    red(host_in, host_out, op="sum")        # pinned torch tensors of the same dtype and length; returns when host_out is complete
    red.close()
"""


class HostAllReducer:
    def __init__(self, comm, chunk_bytes=32 << 20, slots=3, device=None):
        import torch
        self.torch = torch
        self.comm = comm
        self.device = torch.cuda.current_device() if device is None else device
        self.chunk_bytes = int(chunk_bytes)
        self.nslots = int(slots)
        # byte slots; views of the right dtype are made per call
        self.slots = [comm.symmetric_empty(self.chunk_bytes, torch.uint8, self.device) for _ in range(self.nslots)]
        self.s_in = torch.cuda.Stream(device=self.device)
        self.s_red = torch.cuda.Stream(device=self.device)
        self.s_out = torch.cuda.Stream(device=self.device)
        self.slot_free = [None] * self.nslots       # event: the device->host copy out of the slot has finished

    def __call__(self, host_in, host_out, op="sum"):
        torch = self.torch
        if host_in.dtype != host_out.dtype or host_in.numel() != host_out.numel():
            raise ValueError("input and output must have the same dtype and length")
        if not (host_in.is_pinned() and host_out.is_pinned()):
            raise ValueError("host buffers must be pinned (torch.Tensor.pin_memory) for the copies to overlap")
        es = host_in.element_size()
        per = self.chunk_bytes // es
        n = host_in.numel()
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_red, self.s_out):
            s.wait_event(start)
        k = 0
        for lo in range(0, n, per):
            hi = min(n, lo + per)
            slot = self.slots[k % self.nslots][:(hi - lo) * es].view(host_in.dtype)
            with torch.cuda.stream(self.s_in):
                if self.slot_free[k % self.nslots] is not None:
                    self.s_in.wait_event(self.slot_free[k % self.nslots])
                slot.copy_(host_in[lo:hi], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(self.s_in)
            with torch.cuda.stream(self.s_red):
                self.s_red.wait_event(arrived)
                self.comm.all_reduce(slot, op=op, stream=self.s_red)
                reduced = torch.cuda.Event()
                reduced.record(self.s_red)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(reduced)
                host_out[lo:hi].copy_(slot, non_blocking=True)
                done = torch.cuda.Event()
                done.record(self.s_out)
            self.slot_free[k % self.nslots] = done
            k += 1
        # the caller's stream continues when the last copy has landed; the host waits for it too, since the result is host memory
        cur.wait_stream(self.s_out)
        self.s_out.synchronize()
        return host_out

    def close(self):
        self.torch.cuda.synchronize(self.device)
        for t in self.slots:
            self.comm.free_symmetric(t)
        self.slots = []
