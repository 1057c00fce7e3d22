"""Expert-parallel mixture-of-experts layer over the differentiable all-to-all.

The original has no all-to-all (reference include/dccl/dccl.hpp:143-420 ends at send / recv); this library
composes one from grouped send / recv (``dcclAllToAllv``), and this layer is its consumer: E experts are dealt
out E / world to a rank, every token goes to the rank that holds its top-1 expert (dispatch), runs through that
expert and comes back to where it started (combine), scaled by its gate. Backward runs the same two exchanges
with the counts swapped.

    moe = ExpertParallelMLP(d_model, d_hidden, num_experts, comm)
    y = moe(x)                         # x, y: [tokens on this rank, d_model]

The router is replicated; its gradient on a rank covers that rank's tokens only and is summed with the other
replicated parameters (``tensor_parallel.sync_replicated_grads``) when the ranks hold different tokens.
"""
import math

import torch

from ..ops import functional as F


def expert_weights(d_model, d_hidden, expert, seed, dtype=torch.float32, device="cpu"):
    """(w_in [h, d], w_out [d, h]) of one expert, the same for every world size."""
    g = torch.Generator(device="cpu").manual_seed(seed * 1000003 + expert)
    w_in = torch.empty(d_hidden, d_model).uniform_(-1 / math.sqrt(d_model), 1 / math.sqrt(d_model), generator=g)
    w_out = torch.empty(d_model, d_hidden).uniform_(-1 / math.sqrt(d_hidden), 1 / math.sqrt(d_hidden), generator=g)
    return w_in.to(device=device, dtype=dtype), w_out.to(device=device, dtype=dtype)


def router_weight(d_model, num_experts, seed, dtype=torch.float32, device="cpu"):
    g = torch.Generator(device="cpu").manual_seed(seed * 1000003 + 999983)
    return torch.empty(num_experts, d_model).uniform_(-1.0, 1.0, generator=g).to(device=device, dtype=dtype)


class ExpertParallelMLP(torch.nn.Module):
    def __init__(self, d_model, d_hidden, num_experts, comm, seed=0, dtype=torch.float32, device="cpu"):
        super().__init__()
        if num_experts % comm.world:
            raise ValueError("num_experts must split evenly over the ranks")
        self.comm, self.num_experts, self.per = comm, num_experts, num_experts // comm.world
        self.router = torch.nn.Parameter(router_weight(d_model, num_experts, seed, dtype, device))
        first = comm.rank * self.per
        ws = [expert_weights(d_model, d_hidden, first + j, seed, dtype, device) for j in range(self.per)]
        self.w_in = torch.nn.ParameterList([torch.nn.Parameter(w[0]) for w in ws])
        self.w_out = torch.nn.ParameterList([torch.nn.Parameter(w[1]) for w in ws])

    def forward(self, x):
        comm, n, per, E = self.comm, self.comm.world, self.per, self.num_experts
        probs = torch.softmax(torch.nn.functional.linear(x, self.router), dim=-1)
        gate, top = probs.max(dim=-1)
        order = torch.argsort(top, stable=True)                 # tokens grouped by expert, hence by destination rank
        counts = torch.bincount(top, minlength=E)               # per expert, on this rank
        # every rank learns how many tokens each source sends to each of its experts
        incoming = torch.empty_like(counts)
        comm.all_to_all(counts.contiguous(), incoming)          # row p: what rank p sends to my experts
        send_counts = counts.view(n, per).sum(1).tolist()
        incoming = incoming.view(n, per)
        recv_counts = incoming.sum(1).tolist()
        got = F.all_to_all(x[order], send_counts, recv_counts, comm)        # dispatch: grouped by source, then by expert
        outs, row = [], 0
        for p in range(n):
            for j in range(per):
                c = int(incoming[p, j])
                seg = got[row:row + c]
                outs.append(torch.nn.functional.linear(torch.nn.functional.gelu(torch.nn.functional.linear(seg, self.w_in[j])), self.w_out[j]))
                row += c
        done = torch.cat(outs, 0) if outs else got
        back = F.all_to_all(done, recv_counts, send_counts, comm)           # combine: the way they came
        y = torch.zeros_like(x)
        return y.index_add(0, order, back * gate[order].unsqueeze(-1))
