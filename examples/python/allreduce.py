"""All-reduce from Python, on host arrays and (with --cuda) on device tensors.

    python -m dccl_b200.utils.launch -n 4 examples/python/allreduce.py
    python -m dccl_b200.utils.launch -n 8 --gpus examples/python/allreduce.py --cuda

The launcher starts one process per rank on this machine and sets DCCL_RANK / DCCL_WORLD_SIZE / DCCL_MASTER_*;
under torchrun the library reads RANK / WORLD_SIZE / MASTER_* instead.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from dccl_b200 import Communicator  # noqa: E402


def main():
    if "--cuda" in sys.argv[1:]:
        import torch
        local = int(os.environ.get("DCCL_LOCAL_DEVICE", os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(local)
        comm = Communicator(device=local)
        x = torch.full((1 << 20,), float(comm.rank + 1), dtype=torch.bfloat16, device="cuda")
        comm.all_reduce(x, op="avg")                       # one kernel on the current stream, 1/world fused
        torch.cuda.synchronize()
        got, variant = float(x[0]), comm.last_algorithm("allreduce")
    else:
        comm = Communicator()
        x = np.full(1 << 16, comm.rank + 1, dtype=np.float32)
        comm.all_reduce(x, op="avg")                       # shared-memory host path
        got, variant = float(x[0]), comm.last_algorithm("allreduce")
    want = (comm.world + 1) / 2.0
    print("rank %d of %d: average = %g (expected %g), variant %s" % (comm.rank, comm.world, got, want, variant))
    comm.finalize()
    sys.exit(0 if abs(got - want) < 1e-2 else 1)


if __name__ == "__main__":
    main()
