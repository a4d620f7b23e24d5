"""Stock-PyTorch MoE decoder used only by ``bench.py --impl reference --config 5``.

Dense parameters are sharded by the unmodified reference package (``fully_shard`` with the experts
as ``ignored_params``); the experts are expert-parallel with the token dispatcher of the reference's
own EP test fixture (four ``all_to_all_single`` calls, argsort / index_select / scatter-add and a
Python loop over local experts, test/fsdp/test_deepseek_v3_ep_train.py:472-563) generalised to top-k.
None of this repository's kernels, models or runtime is on this path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from ref_llama import apply_rope, rope_tables


def _a2a(x, out_splits, in_splits, group):
    import torch.distributed.nn.functional as DF

    out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
    return DF.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)


class RefExperts(nn.Module):
    def __init__(self, hidden, ffn, n_local, std, dtype):
        super().__init__()
        self.gate_up = nn.ParameterList([nn.Parameter(torch.empty(2 * ffn, hidden, dtype=dtype).normal_(0, std))
                                         for _ in range(n_local)])
        self.down = nn.ParameterList([nn.Parameter(torch.empty(hidden, ffn, dtype=dtype).normal_(0, std))
                                      for _ in range(n_local)])
        self.ffn = ffn


class RefMoEBlock(nn.Module):
    def __init__(self, hidden, n_heads, head_dim, n_experts, expert_ffn, top_k, aux_coef, eps, std, world, dtype, ep_group=None):
        super().__init__()
        self.n_heads, self.head_dim, self.top_k, self.aux_coef = n_heads, head_dim, top_k, aux_coef
        self.n_experts, self.world, self.ep_group = n_experts, world, ep_group
        self.attn_norm = nn.RMSNorm(hidden, eps=eps)
        self.wq = nn.Linear(hidden, hidden, bias=False)
        self.wk = nn.Linear(hidden, hidden, bias=False)
        self.wv = nn.Linear(hidden, hidden, bias=False)
        self.wo = nn.Linear(hidden, hidden, bias=False)
        self.mlp_norm = nn.RMSNorm(hidden, eps=eps)
        self.router = nn.Linear(hidden, n_experts, bias=False)
        for m in (self.wq, self.wk, self.wv, self.wo, self.router):
            nn.init.normal_(m.weight, mean=0.0, std=std)
        self.experts = RefExperts(hidden, expert_ffn, n_experts // world, std, dtype)
        self.last_aux = None

    def moe(self, x):
        T, H = x.shape
        E, K, W = self.n_experts, self.top_k, self.world
        El = E // W
        probs = torch.softmax(self.router(x).float(), dim=-1)
        w, idx = probs.topk(K, dim=-1)
        flat = idx.reshape(-1)
        counts = torch.bincount(flat, minlength=E)
        self.last_aux = self.aux_coef * E * ((counts.float() / (T * K)) * probs.mean(0)).sum()
        order = torch.argsort(flat, stable=True)
        tok = order // K
        xs = x.index_select(0, tok)
        if W > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.ep_group)                     # [W * El] counts from every source
            in_splits = counts.view(W, El).sum(1).tolist()
            out_splits = recv_counts.view(W, El).sum(1).tolist()
            xr = _a2a(xs, out_splits, in_splits, self.ep_group)
            per = recv_counts.view(W, El)
            # rows arrive grouped by source rank, then by local expert: regroup by expert
            eid = torch.repeat_interleave(torch.arange(El, device=x.device).repeat(W), per.reshape(-1))
            perm = torch.argsort(eid, stable=True)
            xr = xr.index_select(0, perm)
            sizes = per.sum(0).tolist()
        else:
            xr, sizes = xs, counts.tolist()
        outs, start = [], 0
        for el, n in enumerate(sizes):
            if n:
                gu = F.linear(xr[start:start + n], self.experts.gate_up[el])
                f = self.experts.ffn
                outs.append(F.linear(F.silu(gu[:, :f]) * gu[:, f:], self.experts.down[el]))
            start += n
        yr = torch.cat(outs, 0) if outs else xr.new_zeros(0, H)
        if W > 1:
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(perm.numel(), device=perm.device)
            yr = yr.index_select(0, inv)
            ys = _a2a(yr, in_splits, out_splits, self.ep_group)
        else:
            ys = yr
        wk = w.reshape(-1).index_select(0, order).to(ys.dtype).unsqueeze(1)
        y = torch.zeros_like(x)
        return y.index_add(0, tok, ys * wk)

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
        return x + self.moe(xn.reshape(b * s, h)).view(b, s, h)


class RefMoE(nn.Module):
    def __init__(self, vocab_size, hidden, n_layers, n_heads, head_dim, n_experts, expert_ffn, top_k, aux_coef=0.01,
                 rope_theta=10000.0, eps=1e-5, init_std=0.02, world=1, expert_dtype=torch.bfloat16, ep_group=None):
        super().__init__()
        self.head_dim, self.rope_theta = head_dim, rope_theta
        self.embed = nn.Embedding(vocab_size, hidden)
        nn.init.normal_(self.embed.weight, mean=0.0, std=init_std)
        self.layers = nn.ModuleList([RefMoEBlock(hidden, n_heads, head_dim, n_experts, expert_ffn, top_k, aux_coef, eps,
                                                 init_std, world, expert_dtype, ep_group) for _ in range(n_layers)])
        self.final_norm = nn.RMSNorm(hidden, eps=eps)
        self.lm_head = nn.Linear(hidden, vocab_size, bias=False)
        nn.init.normal_(self.lm_head.weight, mean=0.0, std=init_std)

    def expert_parameters(self):
        return [p for layer in self.layers for p in layer.experts.parameters()]

    def forward(self, tokens, targets=None):
        cos, sin = rope_tables(tokens.shape[1], self.head_dim, self.rope_theta, tokens.device)
        x = self.embed(tokens)
        for layer in self.layers:
            x = layer(x, cos, sin)
        logits = self.lm_head(self.final_norm(x))
        if targets is None:
            return logits
        loss = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))
        for layer in self.layers:
            loss = loss + layer.last_aux
        return loss


class RefCombinedOptimizer:
    def __init__(self, dense, experts):
        self.dense, self.experts = dense, experts

    def step(self):
        self.dense.step()
        self.experts.step()

    def zero_grad(self, set_to_none=True):
        self.dense.zero_grad(set_to_none=set_to_none)
        self.experts.zero_grad(set_to_none=set_to_none)
