"""One rank of the memory-pool test: tensors created inside a torch memory pool that the communicator serves come out
of symmetric memory, so the switch reduces them in place; and pinned host buffers are reduced through the GPUs by the
chunked helper. Prints 'OK <cases>' or the failures."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from dccl_b200 import Communicator  # noqa: E402
from dccl_b200.host_offload import HostAllReducer  # noqa: E402
from dccl_b200.utils import oracle  # noqa: E402


def main():
    local = int(os.environ.get("DCCL_LOCAL_DEVICE", os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = Communicator(device=local)
    rank, world = comm.rank, comm.world
    failures, cases = [], 0

    def check(ok, what):
        nonlocal cases
        cases += 1
        if not ok:
            failures.append(what)

    # ---- tensors from a pool of symmetric memory ----
    if comm.has_multicast:
        pool = comm.symmetric_mem_pool()
        count = (6 << 20) + 64
        with torch.cuda.use_mem_pool(pool):
            a = torch.empty(count, dtype=torch.float32, device=dev)
            b = torch.empty(count, dtype=torch.bfloat16, device=dev)
        outside = torch.empty(count, dtype=torch.float32, device=dev)
        for t, name in ((a, "float32"), (b, "bfloat16")):
            ins = [oracle.make_input(name, count, seed=4000 + r) for r in range(world)]
            src = ins[rank].view(np.int16) if name == "bfloat16" else ins[rank]
            t.copy_(torch.from_numpy(src.copy()).view(t.dtype).to(dev))
            check(comm.is_symmetric(t), "a tensor from the pool lies in symmetric memory (%s)" % name)
            s0 = comm.stat("symmetric_calls") + comm.stat("zero_copy_calls")
            comm.all_reduce(t, op="avg")
            torch.cuda.synchronize()
            # in place by the switch, or (two ranks) by the zero-copy peer form: no staging either way
            check(comm.stat("symmetric_calls") + comm.stat("zero_copy_calls") == s0 + 1, "a tensor from the pool is reduced where it lies (%s)" % name)
            got = t.cpu().view(torch.int16).numpy().view(np.uint16) if name == "bfloat16" else t.cpu().numpy()
            want = oracle.fold(ins, "avg", bf16=name == "bfloat16")
            rtol, atol = oracle.tolerances(name, world)
            g = oracle.bf16_to_f32(got) if name == "bfloat16" else got
            w = oracle.bf16_to_f32(want) if name == "bfloat16" else want
            check(np.allclose(g.astype(np.float64), w.astype(np.float64), rtol=rtol, atol=atol), "all_reduce of a pool tensor (%s)" % name)
        outside.fill_(1.0)
        comm.all_reduce(outside, op="sum")
        torch.cuda.synchronize()
        check(not comm.is_symmetric(outside) and bool((outside == float(world)).all()), "a tensor from the ordinary allocator is not symmetric, and reduces all the same")
        del a, b

    # ---- host buffers through the GPUs, three chunks in flight ----
    red = HostAllReducer(comm, chunk_bytes=1 << 20, device=local)
    for name, count in (("float32", (3 << 20) + 77), ("float32", 1000)):
        ins = [oracle.make_input(name, count, seed=4100 + r) for r in range(world)]
        hin = torch.from_numpy(ins[rank].copy()).pin_memory()
        hout = torch.zeros(count, dtype=torch.float32).pin_memory()
        for op in ("sum", "max"):
            red(hin, hout, op=op)
            check(np.allclose(hout.numpy().astype(np.float64), oracle.fold(ins, op).astype(np.float64), rtol=1e-5, atol=1e-5),
                  "host all_reduce through the GPUs (%s, %d elements)" % (op, count))
    red.close()
    code, emsg = comm.last_error()
    check(code == 0, "async error: " + emsg)
    comm.finalize()
    if failures:
        print("FAILED %d of %d on rank %d: %s" % (len(failures), cases, rank, "; ".join(failures[:10])))
        sys.exit(1)
    print("OK %d" % cases)


if __name__ == "__main__":
    main()
