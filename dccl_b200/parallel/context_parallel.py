"""Attention over a sequence that is split across the ranks (context parallelism), two ways.

``ring_attention``    every rank keeps its queries; the key / value blocks travel round the ring (one grouped
                      send + recv per step, the pattern of the send/recv ring benchmark) and each arriving block
                      is folded into a running softmax. Memory per rank stays at one block; n - 1 shifts.
``ulysses_attention`` two all-to-alls: sequence-split -> head-split before attention (every rank sees the whole
                      sequence for heads / world of the heads) and back afterwards. Needs heads % world == 0.

Both take q, k, v of shape [batch, heads, local sequence, head dim], rank r holding positions
[r * local, (r + 1) * local), and return the attention output for the local positions. Backward comes from
autograd through the differentiable collectives (``dccl_b200.ops``): gradients of a key / value block travel
the ring backwards to the rank that owns it. The original has neither a sequence dimension nor an all-to-all;
its building blocks for this are send / recv (reference src/core/dccl.cpp:865-911).
"""
import math

import torch

from ..ops import functional as F


def ring_attention(q, k, v, comm, causal=False):
    n, r = comm.world, comm.rank
    B, H, S, D = q.shape
    scale = 1.0 / math.sqrt(D)
    m = q.new_full((B, H, S, 1), float("-inf"))
    l = q.new_zeros((B, H, S, 1))
    o = torch.zeros_like(q)
    kv = torch.stack([k, v], 0)
    tri = torch.ones(S, S, dtype=torch.bool, device=q.device).tril() if causal else None
    for step in range(n):
        src = (r - step) % n                         # the rank whose block is here now
        if not (causal and src > r):                 # a later block is invisible to every local query
            scores = torch.matmul(q, kv[0].transpose(-1, -2)) * scale
            if causal and src == r:
                scores = scores.masked_fill(~tri, float("-inf"))
            m_new = torch.maximum(m, scores.amax(-1, keepdim=True))
            p = torch.exp(scores - m_new)
            alpha = torch.exp(m - m_new)
            l = l * alpha + p.sum(-1, keepdim=True)
            o = o * alpha + torch.matmul(p, kv[1])
            m = m_new
        else:
            # keep the block in the graph: backward must run the matching exchange on every rank, used or not
            o = o + 0.0 * kv.sum()
        if step < n - 1:
            kv = F.ring_shift(kv, 1, comm)
    return o / l


def _seq_to_heads(x, comm):
    """[B, H, S_local, D] -> [B, H / n, S_local * n, D]: block p of the heads goes to rank p, sequences join in rank order."""
    n = comm.world
    B, H, S, D = x.shape
    x = x.reshape(B, n, H // n, S, D).permute(1, 0, 2, 3, 4).contiguous()       # [n (dest), B, H/n, S, D]
    y = F.all_to_all(x.reshape(n * B, H // n, S, D), comm=comm)                 # [n (source), B, H/n, S, D]
    return y.reshape(n, B, H // n, S, D).permute(1, 2, 0, 3, 4).reshape(B, H // n, n * S, D)


def _heads_to_seq(x, comm):
    n = comm.world
    B, Hn, Sn, D = x.shape
    S = Sn // n
    x = x.reshape(B, Hn, n, S, D).permute(2, 0, 1, 3, 4).contiguous()           # [n (dest: owner of the positions), B, H/n, S, D]
    y = F.all_to_all(x.reshape(n * B, Hn, S, D), comm=comm)                     # [n (source: owner of the heads), B, H/n, S, D]
    return y.reshape(n, B, Hn, S, D).permute(1, 0, 2, 3, 4).reshape(B, n * Hn, S, D)


def ulysses_attention(q, k, v, comm, causal=False):
    if q.shape[1] % comm.world:
        raise ValueError("ulysses_attention: the number of heads must split evenly over the ranks")
    qh, kh, vh = (_seq_to_heads(t, comm) for t in (q, k, v))
    out = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal)
    return _heads_to_seq(out, comm)
