"""Stock-PyTorch Llama decoder used only by ``bench.py --impl reference``.

Plain ``nn.Linear`` / ``nn.RMSNorm`` / eager RoPE / ``F.scaled_dot_product_attention`` /
``F.cross_entropy``: the same architecture, sizes and initialisation as the config under test, with
none of this repository's kernels, models or runtime on the path.  It is sharded by the unmodified
reference package through its public ``fully_shard`` / ``configure_optimizer``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn


def rope_tables(seq_len: int, head_dim: int, theta: float, device):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.arange(seq_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def apply_rope(x, cos, sin):
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    c, s = cos[None, :, None, :].to(x.dtype), sin[None, :, None, :].to(x.dtype)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


class RefBlock(nn.Module):
    def __init__(self, hidden, n_heads, head_dim, ffn, eps, std):
        super().__init__()
        self.n_heads, self.head_dim = n_heads, head_dim
        self.attn_norm = nn.RMSNorm(hidden, eps=eps)
        self.wq = nn.Linear(hidden, hidden, bias=False)
        self.wk = nn.Linear(hidden, hidden, bias=False)
        self.wv = nn.Linear(hidden, hidden, bias=False)
        self.wo = nn.Linear(hidden, hidden, bias=False)
        self.mlp_norm = nn.RMSNorm(hidden, eps=eps)
        self.w_gate = nn.Linear(hidden, ffn, bias=False)
        self.w_up = nn.Linear(hidden, ffn, bias=False)
        self.w_down = nn.Linear(ffn, hidden, bias=False)
        for m in (self.wq, self.wk, self.wv, self.wo, self.w_gate, self.w_up, self.w_down):
            nn.init.normal_(m.weight, mean=0.0, std=std)

    def forward(self, x, cos, sin):
        b, s, h = x.shape
        xn = self.attn_norm(x)
        q = self.wq(xn).view(b, s, self.n_heads, self.head_dim)
        k = self.wk(xn).view(b, s, self.n_heads, self.head_dim)
        v = self.wv(xn).view(b, s, self.n_heads, self.head_dim)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + self.wo(o.transpose(1, 2).reshape(b, s, h))
        xn = self.mlp_norm(x)
        return x + self.w_down(F.silu(self.w_gate(xn)) * self.w_up(xn))


class RefLlama(nn.Module):
    def __init__(self, vocab_size, hidden, n_layers, n_heads, head_dim, ffn, rope_theta=10000.0, eps=1e-5,
                 init_std=0.02, activation_checkpointing=False):
        super().__init__()
        self.head_dim, self.rope_theta = head_dim, rope_theta
        self.activation_checkpointing = activation_checkpointing
        self.embed = nn.Embedding(vocab_size, hidden)
        nn.init.normal_(self.embed.weight, mean=0.0, std=init_std)
        self.layers = nn.ModuleList([RefBlock(hidden, n_heads, head_dim, ffn, eps, init_std) for _ in range(n_layers)])
        self.final_norm = nn.RMSNorm(hidden, eps=eps)
        self.lm_head = nn.Linear(hidden, vocab_size, bias=False)
        nn.init.normal_(self.lm_head.weight, mean=0.0, std=init_std)

    def forward(self, tokens, targets=None):
        cos, sin = rope_tables(tokens.shape[1], self.head_dim, self.rope_theta, tokens.device)
        x = self.embed(tokens)
        for layer in self.layers:
            if self.activation_checkpointing and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint

                x = checkpoint(layer, x, cos, sin, use_reentrant=False)
            else:
                x = layer(x, cos, sin)
        logits = self.lm_head(self.final_norm(x))
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))
