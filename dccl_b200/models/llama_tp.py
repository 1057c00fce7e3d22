"""Tensor-parallel form of the Llama-style decoder (``dccl_b200.models.llama``).

``shard(model, comm)`` turns an unsplit ``LlamaDecoder`` into one whose attention heads and feed-forward columns
are dealt out over the ranks of ``comm`` (heads and KV heads must divide by the world size): q / k / v and
gate / up keep the rows of their own heads / columns, o and down keep the matching input columns, and each
block needs two all-reduces forward and two backward (``ops.copy_to_region`` at the entry of the attention and of
the MLP, ``ops.reduce_from_region`` at their exits). Embedding, norms and the output head stay replicated; since
every rank sees the same tokens their gradients come out identical on all ranks without further communication.
Every rank starts from the same unsplit weights, so the sharded model computes what the unsplit one does.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from ..parallel.tensor_parallel import SymmetricPool, column_linears_reduce_grad_in_place, row_linear_reduce_in_place
from .llama import LlamaDecoder, apply_rope, rope_tables


def _rows(linear, lo, hi):
    out = nn.Linear(linear.in_features, hi - lo, bias=False, device=linear.weight.device, dtype=linear.weight.dtype)
    out.weight.data.copy_(linear.weight.data[lo:hi])
    return out


def _cols(linear, lo, hi):
    out = nn.Linear(hi - lo, linear.out_features, bias=False, device=linear.weight.device, dtype=linear.weight.dtype)
    out.weight.data.copy_(linear.weight.data[:, lo:hi])
    return out


class ShardedAttention(nn.Module):
    def __init__(self, attn, comm, pool=None, sequence_parallel=False):
        super().__init__()
        self.pool, self.sp = pool, sequence_parallel
        n, r = comm.world, comm.rank
        if attn.h % n or attn.kv % n:
            raise ValueError("heads (%d) and KV heads (%d) must divide by the world size (%d)" % (attn.h, attn.kv, n))
        self.comm, self.h, self.kv, self.hd = comm, attn.h // n, attn.kv // n, attn.hd
        qw, kw = self.h * self.hd, self.kv * self.hd
        self.q = _rows(attn.q, r * qw, (r + 1) * qw)
        self.k = _rows(attn.k, r * kw, (r + 1) * kw)
        self.v = _rows(attn.v, r * kw, (r + 1) * kw)
        self.o = _cols(attn.o, r * qw, (r + 1) * qw)

    def forward(self, x, cos, sin):
        if self.sp:      # the input is this rank's part of the sequence: gather it (backward: reduce-scatter)
            x = ops.all_gather(x, 1, self.comm)
        b, s, _ = x.shape
        if self.sp:
            q, k, v = self.q(x), self.k(x), self.v(x)
        elif self.pool is not None:
            q, k, v = column_linears_reduce_grad_in_place(x, (self.q.weight, self.k.weight, self.v.weight), self.comm, self.pool)
        else:
            x = ops.copy_to_region(x, self.comm)
            q, k, v = self.q(x), self.k(x), self.v(x)
        q = q.view(b, s, self.h, self.hd).transpose(1, 2)
        k = k.view(b, s, self.kv, self.hd).transpose(1, 2)
        v = v.view(b, s, self.kv, self.hd).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.kv != self.h)
        out = out.transpose(1, 2).reshape(b, s, self.h * self.hd)
        if self.sp:      # sum the partial products and keep this rank's part of the sequence (backward: all-gather)
            return ops.reduce_scatter(self.o(out), 1, "sum", self.comm)
        if self.pool is not None:
            return row_linear_reduce_in_place(out, self.o.weight, self.comm, self.pool)
        return ops.reduce_from_region(self.o(out), self.comm)


class ShardedBlock(nn.Module):
    def __init__(self, blk, comm, pool=None, sequence_parallel=False):
        super().__init__()
        self.pool, self.sp = pool, sequence_parallel
        n, r = comm.world, comm.rank
        ffn = blk.gate.out_features
        if ffn % n:
            raise ValueError("the feed-forward width (%d) must divide by the world size (%d)" % (ffn, n))
        per = ffn // n
        self.comm = comm
        self.n1, self.n2 = blk.n1, blk.n2
        self.attn = ShardedAttention(blk.attn, comm, pool, sequence_parallel)
        self.gate = _rows(blk.gate, r * per, (r + 1) * per)
        self.up = _rows(blk.up, r * per, (r + 1) * per)
        self.down = _cols(blk.down, r * per, (r + 1) * per)

    def forward(self, x, cos, sin):
        x = x + self.attn(self.n1(x), cos, sin)
        if self.sp:
            h = ops.all_gather(self.n2(x), 1, self.comm)
            return x + ops.reduce_scatter(self.down(F.silu(self.gate(h)) * self.up(h)), 1, "sum", self.comm)
        if self.pool is not None:       # the residual add (forward) and the norm's backward consume the pool buffers at once
            g, u = column_linears_reduce_grad_in_place(self.n2(x), (self.gate.weight, self.up.weight), self.comm, self.pool)
            return x + row_linear_reduce_in_place(F.silu(g) * u, self.down.weight, self.comm, self.pool)
        h = ops.copy_to_region(self.n2(x), self.comm)
        return x + ops.reduce_from_region(self.down(F.silu(self.gate(h)) * self.up(h)), self.comm)


class VocabParallelEmbedding(nn.Module):
    """Rows [rank * V / n, (rank + 1) * V / n) of the embedding table; tokens of other ranks' rows contribute zeros and
    the partial results are summed (forward all-reduce, identity backward: every rank updates its own rows)."""

    def __init__(self, embed, comm):
        super().__init__()
        n, r = comm.world, comm.rank
        if embed.num_embeddings % n:
            raise ValueError("the vocabulary (%d) must divide by the world size (%d)" % (embed.num_embeddings, n))
        self.comm, self.per = comm, embed.num_embeddings // n
        self.lo = r * self.per
        self.weight = nn.Parameter(embed.weight.data[self.lo:self.lo + self.per].clone())

    def forward(self, tokens):
        local = tokens - self.lo
        mine = (local >= 0) & (local < self.per)
        out = F.embedding(local.clamp(0, self.per - 1), self.weight) * mine.unsqueeze(-1).to(self.weight.dtype)
        return ops.reduce_from_region(out, self.comm)


def vocab_parallel_cross_entropy(logits_local, targets, lo, comm):
    """Mean cross entropy over rows of logits whose columns are split over the ranks (this rank holds the classes
    [lo, lo + logits_local.shape[-1])). Three small all-reduces: the row maximum, the sum of exponentials and the
    logit of the target class; the full row of logits never exists on one rank."""
    x = logits_local.float()
    per = x.shape[-1]
    m = x.detach().amax(-1)
    comm.all_reduce(m, op="max")
    s = ops.reduce_from_region(torch.exp(x - m.unsqueeze(-1)).sum(-1), comm)
    local = targets - lo
    mine = (local >= 0) & (local < per)
    t = x.gather(-1, local.clamp(0, per - 1).unsqueeze(-1)).squeeze(-1) * mine.to(x.dtype)
    t = ops.reduce_from_region(t, comm)
    return (torch.log(s) + m - t).mean()


class ShardedLlamaDecoder(nn.Module):
    def __init__(self, model: LlamaDecoder, comm, in_place_reduce=False, vocab_parallel=False, sequence_parallel=False):
        super().__init__()
        if sequence_parallel and (in_place_reduce or vocab_parallel):
            raise ValueError("sequence_parallel does not combine with in_place_reduce or vocab_parallel")
        self.cfg, self.comm, self.sp = model.cfg, comm, sequence_parallel
        self.embed, self.norm, self.head = model.embed, model.norm, model.head
        self.vocab_parallel = vocab_parallel
        if vocab_parallel:
            per = model.cfg.vocab_size // comm.world
            self.embed = VocabParallelEmbedding(model.embed, comm)
            self.head = _rows(model.head, comm.rank * per, (comm.rank + 1) * per)
            self.vocab_lo = comm.rank * per
        # one pool for all blocks: both exits of a block feed a residual add, which consumes the buffer at once
        self.pool = SymmetricPool(comm) if in_place_reduce else None
        self.blocks = nn.ModuleList([ShardedBlock(b, comm, self.pool, sequence_parallel) for b in model.blocks])

    def replicated_parameters(self):
        """Embedding, norms and head: the same on every rank. Under sequence parallelism their gradients are partial
        sums after backward; ``sync_replicated_grads()`` adds them up."""
        ps = list(self.embed.parameters()) + list(self.norm.parameters()) + list(self.head.parameters())
        for blk in self.blocks:
            ps += list(blk.n1.parameters()) + list(blk.n2.parameters())
        return ps

    def sync_replicated_grads(self):
        if self.sp:
            from ..parallel.tensor_parallel import sync_replicated_grads
            sync_replicated_grads(self.replicated_parameters(), self.comm)

    def close(self):
        """Give the symmetric activation buffers back (collective); call before the communicator is finalized."""
        if self.pool is not None:
            self.pool.close()

    def _my_part(self, t):
        """This rank's part of dimension 1 (the sequence)."""
        per = t.shape[1] // self.comm.world
        return t[:, self.comm.rank * per:(self.comm.rank + 1) * per]

    def forward(self, tokens):
        x = self.embed(tokens)
        cos, sin = rope_tables(tokens.shape[1], self.cfg.hidden // self.cfg.heads, self.cfg.rope_theta, tokens.device)
        if self.sp:      # between the blocks every rank keeps 1 / world of the sequence; returns the logits of that part
            if tokens.shape[1] % self.comm.world:
                raise ValueError("the sequence length (%d) must divide by the world size" % tokens.shape[1])
            x = self._my_part(x)
        for blk in self.blocks:
            x = blk(x, cos, sin)
        x = self.norm(x)
        if self.vocab_parallel:        # this rank's slice of the classes
            return self.head(ops.copy_to_region(x, self.comm))
        return self.head(x)

    def loss(self, tokens):
        logits = self.forward(tokens[:, :-1])
        if self.sp:
            # this rank's share of the mean over ALL tokens: the shares add up to the loss of the unsplit model, and
            # after backward the gradients of the replicated parameters are partial sums (sync_replicated_grads)
            targets = self._my_part(tokens[:, 1:])
            total = tokens.shape[0] * (tokens.shape[1] - 1)
            return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1), reduction="sum") / total
        if self.vocab_parallel:
            return vocab_parallel_cross_entropy(logits.reshape(-1, logits.shape[-1]), tokens[:, 1:].reshape(-1), self.vocab_lo, self.comm)
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), tokens[:, 1:].reshape(-1))


def shard(model: LlamaDecoder, comm, in_place_reduce=False, vocab_parallel=False, sequence_parallel=False):
    """The tensor-parallel form of `model` for this rank (the unsplit blocks are not kept). in_place_reduce: the
    products at the exits of attention and MLP (forward) and the input gradients at their entries (backward) are
    written into symmetric buffers and summed there by the switch: all four all-reduces of a block run zero-copy.
    vocab_parallel: embedding table and output head are split over the vocabulary as well and the loss is computed from
    the split logits (`vocab_parallel_cross_entropy`); forward() then returns this rank's slice of the logits.
    sequence_parallel: between the blocks every rank keeps 1 / world of the sequence (norms and residuals work on that
    part); a block gathers it at its entry and reduce-scatters at its exit, which moves the same bytes as the two
    all-reduces. loss() then returns this rank's share of the loss; call sync_replicated_grads() after backward."""
    return ShardedLlamaDecoder(model, comm, in_place_reduce, vocab_parallel, sequence_parallel)
