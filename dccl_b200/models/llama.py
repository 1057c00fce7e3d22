"""Llama-style decoder used by the data-parallel training benchmark.

Plain PyTorch: RMSNorm, rotary position embedding, grouped-query attention through
``scaled_dot_product_attention``, SwiGLU MLP, untied output head. ``LlamaConfig.tinyllama_1b`` is
the benchmark's shape: 22 layers, hidden 2048, 32 heads, 4 KV heads, FFN 5632, vocabulary 32000
(about 1.1 B parameters). The model is only the workload whose gradients the library all-reduces;
the "no library GEMM" rule of this project applies to the communication paths, not to it.
"""
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden: int = 2048
    layers: int = 22
    heads: int = 32
    kv_heads: int = 4
    ffn: int = 5632
    max_seq: int = 2048
    rope_theta: float = 10000.0
    eps: float = 1e-5

    @staticmethod
    def tinyllama_1b():
        return LlamaConfig()

    @staticmethod
    def tiny():
        return LlamaConfig(vocab_size=512, hidden=128, layers=2, heads=4, kv_heads=2, ffn=256, max_seq=128)

    def num_params(self):
        hd = self.hidden // self.heads
        attn = self.hidden * self.hidden * 2 + 2 * self.hidden * hd * self.kv_heads
        mlp = 3 * self.hidden * self.ffn
        return self.layers * (attn + mlp + 2 * self.hidden) + 2 * self.vocab_size * self.hidden + self.hidden


class RMSNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return (v * self.weight.float()).to(x.dtype)


def rope_tables(seq, head_dim, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    t = torch.arange(seq, device=device, dtype=torch.float32)
    f = torch.outer(t, inv)
    return f.cos(), f.sin()


def apply_rope(x, cos, sin):
    # x: [B, H, S, D]; rotate pairs (even, odd halves)
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c, s = cos[None, None, : x.shape[2]], sin[None, None, : x.shape[2]]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.h, self.kv, self.hd = cfg.heads, cfg.kv_heads, cfg.hidden // cfg.heads
        self.q = nn.Linear(cfg.hidden, cfg.heads * self.hd, bias=False)
        self.k = nn.Linear(cfg.hidden, cfg.kv_heads * self.hd, bias=False)
        self.v = nn.Linear(cfg.hidden, cfg.kv_heads * self.hd, bias=False)
        self.o = nn.Linear(cfg.heads * self.hd, cfg.hidden, bias=False)

    def forward(self, x, cos, sin):
        b, s, _ = x.shape
        q = self.q(x).view(b, s, self.h, self.hd).transpose(1, 2)
        k = self.k(x).view(b, s, self.kv, self.hd).transpose(1, 2)
        v = self.v(x).view(b, s, self.kv, self.hd).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.kv != self.h)
        return self.o(out.transpose(1, 2).reshape(b, s, self.h * self.hd))


class Block(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.n1, self.n2 = RMSNorm(cfg.hidden, cfg.eps), RMSNorm(cfg.hidden, cfg.eps)
        self.attn = Attention(cfg)
        self.gate = nn.Linear(cfg.hidden, cfg.ffn, bias=False)
        self.up = nn.Linear(cfg.hidden, cfg.ffn, bias=False)
        self.down = nn.Linear(cfg.ffn, cfg.hidden, bias=False)

    def forward(self, x, cos, sin):
        x = x + self.attn(self.n1(x), cos, sin)
        h = self.n2(x)
        return x + self.down(F.silu(self.gate(h)) * self.up(h))


class LlamaDecoder(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden)
        self.blocks = nn.ModuleList([Block(cfg) for _ in range(cfg.layers)])
        self.norm = RMSNorm(cfg.hidden, cfg.eps)
        self.head = nn.Linear(cfg.hidden, cfg.vocab_size, bias=False)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)

    def forward(self, tokens):
        x = self.embed(tokens)
        cos, sin = rope_tables(tokens.shape[1], self.cfg.hidden // self.cfg.heads, self.cfg.rope_theta, tokens.device)
        for blk in self.blocks:
            x = blk(x, cos, sin)
        return self.head(self.norm(x))

    def loss(self, tokens):
        """Next-token cross entropy on a batch of token ids [B, S]."""
        logits = self.forward(tokens[:, :-1])
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), tokens[:, 1:].reshape(-1))
