"""One rank of the sharded-optimizer test: a small MLP trained for a few steps with dccl_b200.parallel.zero against the
same model trained in one piece on the mean of all ranks' losses (computed locally by every rank)."""
import copy
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from dccl_b200 import Communicator  # noqa: E402
from dccl_b200.parallel.zero import ShardedOptimizer  # noqa: E402


def main():
    dev = "cpu"
    if "--cuda" in sys.argv[1:]:                      # tensors on GPU <DCCL_LOCAL_DEVICE>: the device kernels run
        local = int(os.environ.get("DCCL_LOCAL_DEVICE", os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        comm = Communicator(device=local)
    else:
        comm = Communicator()
    n, r = comm.world, comm.rank
    torch.manual_seed(7)
    model = torch.nn.Sequential(torch.nn.Linear(10, 33), torch.nn.Tanh(), torch.nn.Linear(33, 5)).to(dev)   # odd sizes: padding is exercised
    ref = copy.deepcopy(model)
    xs = [torch.randn(6, 10).to(dev) for _ in range(n * 3)]
    ys = [torch.randn(6, 5).to(dev) for _ in range(n * 3)]
    kw = dict(lr=1e-2, weight_decay=0.01, betas=(0.9, 0.95))
    opt = ShardedOptimizer(model.parameters(), comm, torch.optim.AdamW, **kw)
    ref_opt = torch.optim.AdamW(ref.parameters(), **kw)
    ok = True
    for step in range(3):
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(xs[step * n + r]), ys[step * n + r]).backward()
        opt.step()
        ref_opt.zero_grad()
        sum(torch.nn.functional.mse_loss(ref(xs[step * n + q]), ys[step * n + q]) for q in range(n)).div(n).backward()
        ref_opt.step()
        for p, q in zip(model.parameters(), ref.parameters()):
            if not torch.allclose(p, q, rtol=1e-5, atol=1e-6):
                ok = False
                print("rank %d step %d: parameters differ by %g" % (r, step, (p - q).abs().max().item()))
    full = sum(2 * p.numel() * 4 for p in ref.parameters())
    mine = opt.state_bytes()
    opt.close()
    for p, q in zip(model.parameters(), ref.parameters()):
        if not torch.allclose(p, q, rtol=1e-5, atol=1e-6):
            ok = False
            print("rank %d: parameters changed by close()" % r)
    if n > 1 and not mine < full * 0.75:
        ok = False
        print("rank %d: optimizer state %d bytes, unsplit %d" % (r, mine, full))
    if dev != "cpu":
        torch.cuda.synchronize()
    comm.finalize()
    if not ok:
        sys.exit(1)
    print("OK zero worker rank %d (state %d of %d bytes)" % (r, mine, full))


if __name__ == "__main__":
    main()
