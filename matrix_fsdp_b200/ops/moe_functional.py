"""Autograd nodes of the MoE decoder block: the attention half and the expert-parallel FFN.

Both are explicit kernel sequences (tcgen05 GEMMs, attention, routing, dispatch/combine over peer
memory).  ``moe_ffn_reference`` is the same math in plain PyTorch; it is the CPU path (Gloo has no
all-to-all, so it gathers tokens, lets every rank apply its own experts, and sums) and the oracle of
the GPU tests.  The reference project ships no MoE layer; its EP test fixture is
test/fsdp/test_deepseek_v3_ep_train.py:472-563.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import functional as OF


# ---------------------------------------------------------------------------- attention half
class AttentionHalfFunction(torch.autograd.Function):
    """x + Wo·attention(rope(Wqkv·rmsnorm(x))) with a hand-written backward."""

    @staticmethod
    def forward(ctx, x, cos, sin, sinks, shape: OF.BlockShape, wn, wq, wk, wv, wo):
        from . import kernels as K

        x = x.contiguous()
        s = shape
        T, H = x.shape[0], s.hidden
        xn, rstd = K.rmsnorm_fwd(x, wn, s.eps)
        qkv = torch.empty((T, 3 * H), dtype=x.dtype, device=x.device)
        wqkv = OF._fused_weight([wq, wk, wv])
        if wqkv is not None:
            K.gemm(xn, wqkv, out=qkv)
        else:
            for i, w in enumerate((wq, wk, wv)):
                K.gemm(xn, w, out=qkv[:, i * H:(i + 1) * H])
        K.rope_(qkv, cos, sin, s.seq, 0, 2 * s.n_heads, s.head_dim)
        attn, attn_saved = OF._AttentionCore.forward(qkv, s)
        out = K.gemm(attn, wo, cin=x, beta=1.0)
        ctx.save_for_backward(x, cos, sin, wn, wq, wk, wv, wo, xn, rstd, qkv, attn)
        ctx.attn_saved, ctx.shape, ctx.sinks = attn_saved, s, sinks
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import kernels as K

        x, cos, sin, wn, wq, wk, wv, wo, xn, rstd, qkv, attn = ctx.saved_tensors
        s, sinks = ctx.shape, ctx.sinks
        H = s.hidden
        dout = dout.contiguous()
        dattn = K.gemm(dout, wo, b_mn_major=True)
        g_wo = OF._wgrad(dout, attn, sinks[4])
        dqkv = OF._AttentionCore.backward(dattn, qkv, attn, ctx.attn_saved, s).contiguous()
        K.rope_(dqkv, cos, sin, s.seq, 0, 2 * s.n_heads, s.head_dim, backward=True)
        wqkv = OF._fused_weight([wq, wk, wv])
        if wqkv is not None:
            dxn = K.gemm(dqkv, wqkv, b_mn_major=True)
        else:
            dxn = K.gemm(dqkv[:, :H], wq, b_mn_major=True)
            K.gemm(dqkv[:, H:2 * H], wk, b_mn_major=True, out=dxn, cin=dxn, beta=1.0)
            K.gemm(dqkv[:, 2 * H:], wv, b_mn_major=True, out=dxn, cin=dxn, beta=1.0)
        g_q, g_k, g_v = OF._wgrad_pair(dqkv, xn, (sinks[1], sinks[2], sinks[3]), (H, H, H))
        dx, g_n = OF._norm_bwd(dxn, x, wn, rstd, dout, sinks[0])
        return dx, None, None, None, None, g_n, g_q, g_k, g_v, g_wo


def attention_half(x: torch.Tensor, module, shape: OF.BlockShape, cos, sin) -> torch.Tensor:
    sinks = getattr(module, "_attn_sinks", None)
    params = [module.attn_norm.weight, module.wq.weight, module.wk.weight, module.wv.weight, module.wo.weight]
    if sinks is None:
        sinks = [OF.GradSink(p) for p in params]
        module._attn_sinks = sinks
    return AttentionHalfFunction.apply(x, cos, sin, sinks, shape, *params)


# ---------------------------------------------------------------------------- MoE FFN
class MoEFFNFunction(torch.autograd.Function):
    """``(res + sum_k w_k * expert_k(x), aux)`` with experts spread over the EP ranks.

    ``x`` is the normalised hidden state [T, H]; ``w_gu`` [El, 2F, H] and ``w_down`` [El, H, F] are
    this rank's experts.  ``aux`` = coef * E * sum_e (fraction of routed entries on e) * (mean prob of e).
    """

    @staticmethod
    def forward(ctx, x, res, router_w, w_gu, w_down, ep, top_k: int, aux_coef: float, router_sink):
        from . import kernels as K
        from . import moe_kernels as MK

        x = x.contiguous()
        T, H = x.shape
        E = router_w.shape[0]
        El = ep.experts_per_rank
        logits = K.gemm(x, router_w)                                   # [T, E]
        prob_sum = torch.zeros(E, dtype=torch.float32, device=x.device)
        probs, idx, w = MK.router_topk(logits, top_k, prob_sum)
        slot, counts = MK.assign_slots(idx, E)
        counts_all = ep.exchange_counts(counts)
        dest_base, group_offsets, group_rows, tile_group, stats = MK.plan(counts_all, ep.world, ep.rank, E, ep.cap_rows)
        ep.note_plan(stats, T * top_k)
        route = MK.dispatch_push(x, idx, ep.recv_addrs, El, ep.cap_rows, slot=slot, dest_base=dest_base)
        MK.zero_pad(ep.recv, H, group_offsets, group_rows)
        ep.fence(1)
        gu = K.grouped_gemm_m(ep.recv, w_gu, tile_group, groups_of_256_rows=True)              # [cap, 2F]
        h = K.swiglu_fwd(gu)
        K.grouped_gemm_m(h, w_down, tile_group, out=ep.out, groups_of_256_rows=True)
        del h
        x_recv = ep.recv.clone() if ctx.needs_input_grad[3] or ctx.needs_input_grad[0] else None
        ep.fence(2)
        y, _ = MK.combine_pull(ep.out_addrs, idx, route, H, El, weight=w, res=res)
        frac = counts.float() / float(T * top_k)
        aux = (aux_coef * E / float(T)) * (frac * prob_sum).sum()
        ctx.save_for_backward(x, router_w, w_gu, w_down, probs, idx, w, route, group_offsets, group_rows, tile_group,
                              stats, gu, x_recv, frac)
        ctx.ep, ctx.aux_coef, ctx.router_sink, ctx.has_res = ep, aux_coef, router_sink, res is not None
        ep.last_stats = stats
        return y, aux

    @staticmethod
    def backward(ctx, dy, daux):
        from . import kernels as K
        from . import moe_kernels as MK

        (x, router_w, w_gu, w_down, probs, idx, w, route, group_offsets, group_rows, tile_group, stats, gu, x_recv,
         frac) = ctx.saved_tensors
        ep = ctx.ep
        T, H = x.shape
        E, El = router_w.shape[0], ep.experts_per_rank
        dy = dy.contiguous()
        # gradient rows, weighted by the router weight, go to the expert owners
        MK.dispatch_push(dy, idx, ep.recv_addrs, El, ep.cap_rows, route=route, scale=w)
        MK.zero_pad(ep.recv, H, group_offsets, group_rows)
        ep.fence(1)
        dh = K.grouped_gemm_m(ep.recv, w_down, tile_group, b_mn_major=True, groups_of_256_rows=True)   # [cap, F]
        dgu, h = MK.swiglu_bwd_dot(dh, gu, ep.out_scalar, stats[0:1])
        del dh
        g_down = K.grouped_gemm_k(ep.recv, h, group_offsets, El)                     # [El, H, F]
        del h
        K.grouped_gemm_m(dgu, w_gu, tile_group, b_mn_major=True, out=ep.out, groups_of_256_rows=True)  # [cap, H]
        g_gu = K.grouped_gemm_k(dgu, x_recv, group_offsets, El)                      # [El, 2F, H]
        del dgu
        ep.fence(2)
        dx, rowdot = MK.combine_pull(ep.out_addrs, idx, route, H, El, scalar_addrs=ep.scalar_addrs)
        dw = rowdot / w.clamp_min(1e-20)
        aux_grad = (daux.float() * (ctx.aux_coef * E / float(T))) * frac
        dlogits = MK.router_bwd(probs, idx, dw, aux_grad.contiguous())
        K.gemm(dlogits, router_w, b_mn_major=True, out=dx, cin=dx, beta=1.0)
        g_router = OF._wgrad(dlogits, x, ctx.router_sink)
        return dx, (dy if ctx.has_res else None), g_router, g_gu, g_down, None, None, None, None


def moe_ffn(x, res, router_w, w_gu, w_down, ep, top_k: int, aux_coef: float, router_param=None):
    sink = OF.GradSink(router_param) if router_param is not None else None
    return MoEFFNFunction.apply(x, res, router_w, w_gu, w_down, ep, top_k, aux_coef, sink)


# ---------------------------------------------------------------------------- plain PyTorch
class _GatherRows(torch.autograd.Function):
    """Concatenate every rank's rows; backward sums the gradients and keeps this rank's rows
    (all-reduce based, so it also runs on Gloo, which has neither reduce-scatter nor all-to-all)."""

    @staticmethod
    def forward(ctx, t, group):
        import torch.distributed as dist

        ctx.group, ctx.rows = group, t.shape[0]
        parts = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, t.contiguous(), group=group)
        return torch.cat(parts, dim=0)

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist

        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        r = dist.get_rank(ctx.group)
        return g[r * ctx.rows:(r + 1) * ctx.rows], None


def moe_ffn_reference(x, res, router_w, w_gu, w_down, top_k: int, aux_coef: float, group=None):
    """Same result as :func:`moe_ffn` in stock ops (fp32 routing).  With ``group`` the experts in
    ``w_gu`` / ``w_down`` are this rank's slice and tokens are exchanged by gather + sum."""
    T, H = x.shape
    E = router_w.shape[0]
    logits = F.linear(x, router_w).float()
    probs = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    counts = torch.zeros(E, dtype=torch.float32, device=x.device)
    counts.scatter_add_(0, idx.reshape(-1), torch.ones(T * top_k, dtype=torch.float32, device=x.device))
    aux = (aux_coef * E / float(T)) * ((counts / float(T * top_k)) * probs.sum(0)).sum()
    world, rank = 1, 0
    if group is not None:
        import torch.distributed as dist

        world, rank = dist.get_world_size(group), dist.get_rank(group)
    if world > 1:
        import torch.distributed.nn.functional as DF

        x_all = _GatherRows.apply(x, group)
        w_all = _GatherRows.apply(w, group)
        idx_all = _GatherRows.apply(idx, group)
    else:
        x_all, w_all, idx_all = x, w, idx
    El = w_gu.shape[0]
    Fd = w_down.shape[2]
    y_all = torch.zeros(x_all.shape[0], H, dtype=torch.float32, device=x.device)
    for el in range(El):
        e = rank * El + el
        tok, kk = (idx_all == e).nonzero(as_tuple=True)
        # an expert without tokens still goes through the (empty) products: the result has to hang on ``x_all`` and
        # ``w_all`` on every rank, or a rank whose experts stay idle would leave out the collectives in the backward
        # of the gathers while the other ranks run them
        gu = F.linear(x_all[tok], w_gu[el])
        hcur = F.silu(gu[:, :Fd]) * gu[:, Fd:]
        ye = F.linear(hcur, w_down[el]).float() * w_all[tok, kk].unsqueeze(1)
        y_all = y_all.index_add(0, tok, ye)
    if world > 1:
        y_all = DF.all_reduce(y_all, group=group)
        y = y_all[rank * T:(rank + 1) * T]
    else:
        y = y_all
    y = y.to(x.dtype)
    return (y if res is None else res + y), aux
