"""A tensor-parallel MLP trained for a few steps.

    python -m dccl_b200.utils.launch -n 2 examples/python/tensor_parallel_mlp.py
    python -m dccl_b200.utils.launch -n 8 --gpus examples/python/tensor_parallel_mlp.py --cuda

ColumnParallelLinear / RowParallelLinear keep a slice of the weights per rank; the differentiable collectives of
dccl_b200.ops run the all-reduce of the partial products forward and of the input gradient backward.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from dccl_b200 import Communicator  # noqa: E402
from dccl_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear  # noqa: E402


def main():
    dev = "cpu"
    if "--cuda" in sys.argv[1:]:
        local = int(os.environ.get("DCCL_LOCAL_DEVICE", os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        comm = Communicator(device=local)
    else:
        comm = Communicator()
    d, h = 64, 64 * comm.world
    up = ColumnParallelLinear(d, h, comm, seed=0, device=dev)
    down = RowParallelLinear(h, d, comm, seed=1, device=dev)
    opt = torch.optim.SGD(list(up.parameters()) + list(down.parameters()), lr=0.05)
    torch.manual_seed(0)                                   # the same batch on every rank: this is tensor, not data parallelism
    x, target = torch.randn(32, d).to(dev), torch.randn(32, d).to(dev)
    losses = []
    for _ in range(20):
        opt.zero_grad()
        loss = ((down(torch.nn.functional.gelu(up(x))) - target) ** 2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    print("rank %d of %d: loss %.4f -> %.4f (weights per rank: %d of %d)" % (
        comm.rank, comm.world, losses[0], losses[-1], up.weight.numel() + down.weight.numel(), 2 * d * h))
    comm.finalize()
    sys.exit(0 if losses[-1] < losses[0] else 1)


if __name__ == "__main__":
    main()
