"""One rank of the expert-parallel test: every rank holds its own tokens and E / world experts; output, input
gradient, expert gradients and the (summed) router gradient are compared with all experts applied in one process."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from dccl_b200 import Communicator  # noqa: E402
from dccl_b200.parallel.expert_parallel import ExpertParallelMLP, expert_weights, router_weight  # noqa: E402
from dccl_b200.parallel.tensor_parallel import sync_replicated_grads  # noqa: E402


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
    d, h, E, T = 8, 12, 2 * n, 11
    torch.manual_seed(4321)
    xs = [torch.randn(T + p, d).to(dev) for p in range(n)]    # a different number of tokens per rank
    ts = [torch.randn(T + p, d).to(dev) for p in range(n)]
    ok = True

    def check(cond, what):
        nonlocal ok
        if not cond:
            ok = False
            print("rank %d: %s" % (r, what))

    # the unsplit layer over everybody's tokens
    router = router_weight(d, E, 0, device=dev).requires_grad_(True)
    experts = [[w.requires_grad_(True) for w in expert_weights(d, h, e, 0, device=dev)] for e in range(E)]
    ref_x = [x.clone().requires_grad_(True) for x in xs]
    ref_out = []
    for x in ref_x:
        probs = torch.softmax(x @ router.t(), -1)
        gate, top = probs.max(-1)
        rows = [torch.nn.functional.linear(torch.nn.functional.gelu(torch.nn.functional.linear(x[t:t + 1], experts[int(top[t])][0])),
                                           experts[int(top[t])][1]) * gate[t] for t in range(x.shape[0])]
        ref_out.append(torch.cat(rows, 0))
    sum(((o - t) ** 2).sum() for o, t in zip(ref_out, ts)).backward()

    moe = ExpertParallelMLP(d, h, E, comm, seed=0, device=dev)
    x = xs[r].clone().requires_grad_(True)
    out = moe(x)
    check(torch.allclose(out, ref_out[r].detach(), rtol=1e-4, atol=1e-5), "forward differs")
    ((out - ts[r]) ** 2).sum().backward()
    check(torch.allclose(x.grad, ref_x[r].grad, rtol=1e-4, atol=1e-5), "input gradient differs")
    for j in range(moe.per):
        e = r * moe.per + j
        check(torch.allclose(moe.w_in[j].grad, experts[e][0].grad, rtol=1e-4, atol=1e-5), "expert %d w_in gradient differs" % e)
        check(torch.allclose(moe.w_out[j].grad, experts[e][1].grad, rtol=1e-4, atol=1e-5), "expert %d w_out gradient differs" % e)
    sync_replicated_grads([moe.router], comm)
    check(torch.allclose(moe.router.grad, router.grad, rtol=1e-4, atol=1e-5), "router gradient differs")
    if dev != "cpu":
        torch.cuda.synchronize()
    comm.finalize()
    if not ok:
        sys.exit(1)
    print("OK moe worker rank %d" % r)


if __name__ == "__main__":
    main()
