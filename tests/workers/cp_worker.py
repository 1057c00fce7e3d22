"""One rank of the context-parallel test: ring attention and the all-to-all (Ulysses) form against plain attention over
the whole sequence, outputs and gradients of q, k, v, with and without the causal mask."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from dccl_b200 import Communicator  # noqa: E402
from dccl_b200.parallel.context_parallel import ring_attention, ulysses_attention  # noqa: E402


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
    B, H, S, D = 2, 2 * n, 5, 8
    torch.manual_seed(2468)
    full = [torch.randn(B, H, S * n, D).to(dev) for _ in range(3)]
    w = torch.randn(B, H, S * n, D).to(dev)
    ok = True
    sl = slice(r * S, (r + 1) * S)
    for causal in (False, True):
        ref = [t.clone().requires_grad_(True) for t in full]
        ref_out = torch.nn.functional.scaled_dot_product_attention(*ref, is_causal=causal)
        (ref_out * w).sum().backward()
        for name, fn in (("ring", ring_attention), ("ulysses", ulysses_attention)):
            q, k, v = [t[:, :, sl].clone().requires_grad_(True) for t in full]
            out = fn(q, k, v, comm, causal=causal)
            (out * w[:, :, sl]).sum().backward()
            for what, got, want in [("output", out, ref_out[:, :, sl]), ("dq", q.grad, ref[0].grad[:, :, sl]),
                                    ("dk", k.grad, ref[1].grad[:, :, sl]), ("dv", v.grad, ref[2].grad[:, :, sl])]:
                if not torch.allclose(got, want.detach(), rtol=1e-4, atol=1e-5):
                    ok = False
                    print("rank %d: %s attention (causal=%s): %s differs by %g" % (r, name, causal, what, (got - want).abs().max().item()))
    if dev != "cpu":
        torch.cuda.synchronize()
    comm.finalize()
    if not ok:
        sys.exit(1)
    print("OK cp worker rank %d" % r)


if __name__ == "__main__":
    main()
