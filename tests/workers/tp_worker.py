"""One rank of the test of the differentiable collectives and the tensor / sequence parallel layers. Every rank
also computes the unsplit reference by itself and compares. CPU tensors (shared-memory host path) by default;
with --cuda the tensors live on GPU <DCCL_LOCAL_DEVICE> and the device kernels run."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from dccl_b200 import Communicator  # noqa: E402
from dccl_b200 import ops  # noqa: E402
from dccl_b200.parallel.tensor_parallel import (ColumnParallelLinear, RowParallelLinear, _full_weight,  # noqa: E402
                                                sync_replicated_grads)

failures = []


def check(ok, what):
    if not ok:
        failures.append(what)


def close(a, b, tol=1e-5):
    return torch.allclose(a, b, rtol=tol, atol=tol)


def main():
    cuda = "--cuda" in sys.argv[1:]
    dev = "cpu"
    if cuda:
        local = int(os.environ.get("DCCL_LOCAL_DEVICE", os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        comm = Communicator(device=local)
    else:
        comm = Communicator()
    native = comm
    if "--gloo" in sys.argv[1:]:      # the same layers over torch.distributed (gloo): a differential run of the layers
        import torch.distributed as dist
        from dccl_b200.parallel.torch_comm import TorchDistCommunicator
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % (int(os.environ["DCCL_MASTER_PORT"]) + 1),
                                rank=comm.rank, world_size=comm.world)
        comm = TorchDistCommunicator()
    ops.set_default_communicator(comm)
    n, r = comm.world, comm.rank
    torch.manual_seed(1234)                          # the same "global" data on every rank
    xs = [torch.randn(4 * n, 6).to(dev) for _ in range(n)]   # rank p's input is xs[p]
    ws = [torch.randn(4 * n, 6).to(dev) for _ in range(n)]   # rank p weighs its output with ws[p] in its loss

    # all_reduce: L = sum_p <w_p, sum_q x_q>  ->  dL/dx_r = sum_p w_p
    for op in ("sum", "avg"):
        x = xs[r].clone().requires_grad_(True)
        y = ops.all_reduce(x, op)
        want = sum(xs) / (n if op == "avg" else 1)
        check(close(y, want), "all_reduce %s forward" % op)
        (y * ws[r]).sum().backward()
        check(close(x.grad, sum(ws) / (n if op == "avg" else 1)), "all_reduce %s backward" % op)

    # all_gather along dim 0 and dim 1
    for dim in (0, 1):
        x = xs[r].clone().requires_grad_(True)
        y = ops.all_gather(x, dim)
        check(close(y, torch.cat(xs, dim)), "all_gather dim %d forward" % dim)
        wfull = [torch.cat([ws[(p + q) % n] for q in range(n)], dim) for p in range(n)]   # rank p's weights for the gathered tensor
        (y * wfull[r]).sum().backward()
        want = sum(w.chunk(n, dim)[r] for w in wfull)
        check(close(x.grad, want), "all_gather dim %d backward" % dim)

    # reduce_scatter along dim 0, sum and avg
    for op in ("sum", "avg"):
        x = xs[r].clone().requires_grad_(True)
        y = ops.reduce_scatter(x, 0, op)
        want = (sum(xs) / (n if op == "avg" else 1)).chunk(n, 0)[r]
        check(close(y, want), "reduce_scatter %s forward" % op)
        wb = [w[:4] for w in ws]                                                         # rank p weighs its block with wb[p]
        (y * wb[r]).sum().backward()
        check(close(x.grad, torch.cat(wb, 0) / (n if op == "avg" else 1)), "reduce_scatter %s backward" % op)

    # all_to_all
    x = xs[r].clone().requires_grad_(True)
    y = ops.all_to_all(x)
    check(close(y, torch.cat([xs[p].chunk(n, 0)[r] for p in range(n)], 0)), "all_to_all forward")
    (y * ws[r]).sum().backward()
    check(close(x.grad, torch.cat([ws[p].chunk(n, 0)[r] for p in range(n)], 0)), "all_to_all backward")

    # broadcast from the last rank
    root = n - 1
    x = xs[r].clone().requires_grad_(True)
    y = ops.broadcast(x, root)
    check(close(y, xs[root]), "broadcast forward")
    (y * ws[r]).sum().backward()
    check(close(x.grad, sum(ws) if r == root else torch.zeros_like(x)), "broadcast backward")

    # tensor-parallel MLP against the unsplit one: same output, same input gradient, matching weight gradients
    d, h, T = 6, 8 * n, 4 * n
    w1, b1 = _full_weight(h, d, 0, torch.float32, dev)
    w2, b2 = _full_weight(d, h, 1, torch.float32, dev)
    inp = torch.randn(T, d).to(dev)
    tgt = torch.randn(T, d).to(dev)

    ref_in = inp.clone().requires_grad_(True)
    rw1, rb1, rw2, rb2 = [t.clone().requires_grad_(True) for t in (w1, b1, w2, b2)]
    ref_out = torch.nn.functional.linear(torch.nn.functional.gelu(torch.nn.functional.linear(ref_in, rw1, rb1)), rw2, rb2)
    ((ref_out - tgt) ** 2).sum().backward()

    up, down = ColumnParallelLinear(d, h, comm, seed=0, device=dev), RowParallelLinear(h, d, comm, seed=1, device=dev)
    x = inp.clone().requires_grad_(True)
    out = down(torch.nn.functional.gelu(up(x)))
    check(close(out, ref_out.detach(), 1e-4), "tensor parallel forward")
    ((out - tgt) ** 2).sum().backward()
    per = h // n
    check(close(x.grad, ref_in.grad, 1e-4), "tensor parallel input gradient")
    check(close(up.weight.grad, rw1.grad[r * per:(r + 1) * per], 1e-4), "column weight gradient")
    check(close(up.bias.grad, rb1.grad[r * per:(r + 1) * per], 1e-4), "column bias gradient")
    check(close(down.weight.grad, rw2.grad[:, r * per:(r + 1) * per], 1e-4), "row weight gradient")
    check(close(down.bias.grad, rb2.grad, 1e-4), "row bias gradient")

    # sequence parallel: activations split along the sequence outside the block; the loss is the sum over the ranks
    up = ColumnParallelLinear(d, h, comm, sequence_parallel=True, seed=0, device=dev)
    down = RowParallelLinear(h, d, comm, sequence_parallel=True, seed=1, device=dev)
    tl = T // n
    x = inp[r * tl:(r + 1) * tl].clone().requires_grad_(True)
    out = down(torch.nn.functional.gelu(up(x)))
    check(close(out, ref_out.detach()[r * tl:(r + 1) * tl], 1e-4), "sequence parallel forward")
    ((out - tgt[r * tl:(r + 1) * tl]) ** 2).sum().backward()
    sync_replicated_grads([down.bias], comm)
    check(close(x.grad, ref_in.grad[r * tl:(r + 1) * tl], 1e-4), "sequence parallel input gradient")
    check(close(up.weight.grad, rw1.grad[r * per:(r + 1) * per], 1e-4), "sequence parallel column weight gradient")
    check(close(down.weight.grad, rw2.grad[:, r * per:(r + 1) * per], 1e-4), "sequence parallel row weight gradient")
    check(close(down.bias.grad, rb2.grad, 1e-4), "sequence parallel row bias gradient after sync")

    # pipeline: stage s (one Linear + tanh) lives on rank s; activations go forward with send / recv, gradients come back
    if n > 1:
        torch.manual_seed(99)
        stages = [torch.nn.Linear(d, d).to(dev) for _ in range(n)]
        px, ptgt = torch.randn(5, d).to(dev), torch.randn(5, d).to(dev)
        h = px
        for st in stages:
            h = torch.tanh(st(h))
        ((h - ptgt) ** 2).sum().backward()                        # the unsplit reference, on every rank
        want_w, want_b = stages[r].weight.grad.clone(), stages[r].bias.grad.clone()
        mine = torch.nn.Linear(d, d).to(dev)
        mine.load_state_dict(stages[r].state_dict())
        h_in = px if r == 0 else ops.recv(px, r - 1)
        h_out = torch.tanh(mine(h_in))
        if r == n - 1:
            ((h_out - ptgt) ** 2).sum().backward()
        else:
            ops.send(h_out, r + 1).backward()
        check(close(mine.weight.grad, want_w, 1e-4), "pipeline stage %d weight gradient" % r)
        check(close(mine.bias.grad, want_b, 1e-4), "pipeline stage %d bias gradient" % r)

    if cuda:
        torch.cuda.synchronize()
    if native is not comm:
        import torch.distributed as dist
        dist.destroy_process_group()
    native.finalize()
    if failures:
        print("FAILED on rank %d: %s" % (r, "; ".join(failures)))
        sys.exit(1)
    print("OK tp worker rank %d" % r)


if __name__ == "__main__":
    main()
