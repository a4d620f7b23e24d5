"""Differentiable ops built on the sm_100a kernels, with a plain-PyTorch path for CPU.

The heavy object is :class:`DecoderBlockFunction`: one autograd node per transformer block with a
hand-written backward.  That keeps the host cost of a block at a couple of dozen kernel launches
(no per-op autograd bookkeeping), lets the weight gradients be written by the wgrad GEMM straight
into the FSDP unit's gradient bucket, and gives built-in activation recomputation (save only the
block input).

Every op also exists as a small standalone function (``linear``, ``rms_norm``, ``swiglu``,
``fused_cross_entropy``) for models that are not built from the block node.

The reference ships no model ops at all; its benches build blocks from ``nn.Linear`` /
``F.scaled_dot_product_attention`` / ``nn.LayerNorm`` (``test/fsdp/bench_fsdp2_compare.py:305-514``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import lib as _lib


def use_native(t: torch.Tensor) -> bool:
    """Kernels run for CUDA bf16 tensors; on a GPU box a missing library is an error."""
    if t.device.type != "cuda" or t.dtype != torch.bfloat16 or _lib.disabled_by_env():
        return False
    _lib.load(required=True)
    return True


# ---------------------------------------------------------------------------- rope tables
_ROPE_CACHE: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def rope_tables(seq_len: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    key = (seq_len, head_dim, float(theta), str(device))
    hit = _ROPE_CACHE.get(key)
    if hit is None:
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
        ang = torch.arange(seq_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
        hit = (ang.cos().contiguous(), ang.sin().contiguous())
        _ROPE_CACHE[key] = hit
    return hit


def apply_rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x``: [B, S, nH, D]; rotate-half pairing (i, i + D/2)."""
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c, s = cos[None, : x.shape[1], None, :], sin[None, : x.shape[1], None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


# ---------------------------------------------------------------------------- small ops
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, sink):
        from . import kernels as K

        ctx.save_for_backward(x, w)
        ctx.sink = sink
        x2 = x.reshape(-1, x.shape[-1])
        return K.gemm(x2, w).view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from . import kernels as K

        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = K.gemm(dy2, w, b_mn_major=True).view(x.shape) if ctx.needs_input_grad[0] else None
        dw = _wgrad(dy2, x2, ctx.sink)
        return dx, dw, None


class GradSink:
    """Where a weight gradient goes: the owning FSDP unit's bucket when there is one."""

    __slots__ = ("param",)

    def __init__(self, param: torch.nn.Parameter) -> None:
        self.param = param

    def target(self):
        ref = getattr(self.param, "_mfsdp_unit_ref", None)
        unit = ref() if ref is not None else None
        if unit is None or unit.state.value != "unsharded" or unit.flat_buffer.bucket.dtype != torch.bfloat16:
            return None
        return unit


def _wgrad(dy2: torch.Tensor, x2: torch.Tensor, sink: GradSink | None):
    """dW = dyᵀ·x; written into the FSDP bucket when possible (returns None then)."""
    from . import kernels as K

    unit = sink.target() if sink is not None else None
    if unit is None:
        return K.gemm(dy2, x2, a_mn_major=True, b_mn_major=True)
    fqn = sink.param._matrix_fsdp_fqn
    view, acc = unit.grad_target(fqn)
    K.gemm(dy2, x2, a_mn_major=True, b_mn_major=True, out=view, cin=view if acc else None, beta=1.0 if acc else 0.0)
    unit.mark_grad_written(fqn)
    return None


def linear(x: torch.Tensor, weight: torch.Tensor, param: torch.nn.Parameter | None = None) -> torch.Tensor:
    """``x @ weightᵀ`` on the tcgen05 GEMM (fwd, dgrad, wgrad)."""
    if not use_native(x) or weight.dtype != torch.bfloat16 or x.shape[-1] % 8 or weight.shape[0] % 8:
        return F.linear(x, weight)
    return _LinearFn.apply(x.contiguous(), weight, GradSink(param) if param is not None else None)


class _EmbeddingFn(torch.autograd.Function):
    """Row lookup whose backward sums the rows of equal ids with one deterministic kernel sequence and writes the
    result into the owning unit's gradient bucket (torch's backward sorts 64-bit keys, fills a fresh V x H tensor
    and the runtime then copies it into the bucket: about 0.3 ms at the very end of the backward pass, where
    nothing overlaps it)."""

    @staticmethod
    def forward(ctx, ids, w, sink):
        ctx.save_for_backward(ids)
        ctx.sink, ctx.w_shape = sink, tuple(w.shape)
        return F.embedding(ids, w)

    @staticmethod
    def backward(ctx, dy):
        from . import kernels as K

        (ids,) = ctx.saved_tensors
        V, H = ctx.w_shape
        dy2 = dy.reshape(-1, H).contiguous()
        flat_ids = ids.reshape(-1).contiguous()
        unit = ctx.sink.target() if ctx.sink is not None else None
        if unit is not None:
            fqn = ctx.sink.param._matrix_fsdp_fqn
            view, acc = unit.grad_target(fqn)
            K.embedding_bwd(dy2, flat_ids, view, accumulate=acc)
            unit.mark_grad_written(fqn)
            return None, None, None
        dw = torch.empty((V, H), dtype=torch.bfloat16, device=dy.device)
        K.embedding_bwd(dy2, flat_ids, dw)
        return None, dw, None


_EMBED_MAX_TOKENS = 32768       # the rank pass compares every position with the earlier ones


def embedding(ids: torch.Tensor, weight: torch.Tensor, param: torch.nn.Parameter | None = None) -> torch.Tensor:
    """``weight[ids]``; on CUDA with bf16 rows the backward runs :class:`_EmbeddingFn`'s kernels."""
    if use_native(weight) and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0 \
            and weight.stride(1) == 1 and ids.dtype == torch.int64 and ids.numel() <= _EMBED_MAX_TOKENS \
            and torch.is_grad_enabled() and weight.requires_grad:
        return _EmbeddingFn.apply(ids, weight, GradSink(param) if param is not None else None)
    return F.embedding(ids, weight)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        from . import kernels as K

        y, rstd = K.rmsnorm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import kernels as K

        x, w, rstd = ctx.saved_tensors
        dx, dw = K.rmsnorm_bwd(dy.contiguous(), x, w, rstd)
        return dx, dw, None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if use_native(x) and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return _RMSNormFn.apply(x.contiguous(), weight, eps)
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        from . import kernels as K

        ctx.save_for_backward(gu)
        return K.swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dh):
        from . import kernels as K

        (gu,) = ctx.saved_tensors
        return K.swiglu_bwd(dh.contiguous(), gu)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``[..., 2F]`` input laid out as [gate | up]."""
    f = gate_up.shape[-1] // 2
    if use_native(gate_up) and f % 8 == 0:
        flat = gate_up.reshape(-1, 2 * f).contiguous()
        return _SwiGLUFn.apply(flat).view(*gate_up.shape[:-1], f)
    return F.silu(gate_up[..., :f]) * gate_up[..., f:]


class _FusedCEFn(torch.autograd.Function):
    """Softmax cross-entropy whose forward also produces the logits gradient in place."""

    @staticmethod
    def forward(ctx, logits, target, ignore_index, n_valid, unit_upstream_grad):
        from . import kernels as K

        if n_valid is None:
            # the count of kept targets stays on the device; the kernel reads the scale from there
            scale = (target != ignore_index).sum().clamp_(min=1).to(torch.float32).reciprocal_().view(1)
        else:
            scale = 1.0 / float(max(int(n_valid), 1))
        loss_rows = K.cross_entropy_(logits, target, scale, ignore_index)   # logits now hold dlogits
        ctx.save_for_backward(logits)
        ctx.unit_upstream_grad = unit_upstream_grad
        total = loss_rows.sum()
        return total * (scale[0] if isinstance(scale, torch.Tensor) else scale)

    @staticmethod
    def backward(ctx, dloss):
        (dlogits,) = ctx.saved_tensors
        if not ctx.unit_upstream_grad:
            dlogits.mul_(dloss.to(dlogits.dtype))
        return dlogits, None, None, None, None


def fused_cross_entropy(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100,
                        n_valid: int | None = None, unit_upstream_grad: bool = False) -> torch.Tensor:
    """Mean token cross-entropy; the logits buffer is consumed (overwritten with its gradient).

    ``n_valid``: number of non-ignored targets when the caller knows it on the host; otherwise it is
    counted on the device and the kernel reads the scale from device memory (no host sync either way).  ``unit_upstream_grad``: promise that the returned loss is what ``backward()`` is
    called on (upstream gradient 1), which skips one pass over the logits.
    """
    v = logits.shape[-1]
    flat_t = target.reshape(-1)
    if use_native(logits) and v % 8 == 0 and v <= 8 * 1024 * 6 and logits.is_contiguous():
        return _FusedCEFn.apply(logits.view(-1, v), flat_t, ignore_index, n_valid, unit_upstream_grad)
    return F.cross_entropy(logits.reshape(-1, v).float(), flat_t, ignore_index=ignore_index)


# ---------------------------------------------------------------------------- attention
def causal_attention_reference(qkv: torch.Tensor, batch: int, seq: int, n_heads: int, head_dim: int) -> torch.Tensor:
    """``qkv``: [B*S, 3*H] (post-RoPE) → [B*S, H] via ``F.scaled_dot_product_attention``."""
    h = n_heads * head_dim
    q, k, v = (qkv[:, i * h:(i + 1) * h].view(batch, seq, n_heads, head_dim).transpose(1, 2) for i in range(3))
    o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
    return o.transpose(1, 2).reshape(batch * seq, h)


@dataclass
class BlockShape:
    batch: int
    seq: int
    hidden: int
    n_heads: int
    head_dim: int
    ffn: int
    eps: float
    rope_theta: float


class _AttentionCore:
    """Attention forward/backward used inside the block node.

    Uses this package's tcgen05 attention kernels when built; until then the library SDPA kernel
    is called through a small private autograd graph that is kept from forward to backward.
    """

    @staticmethod
    def forward(qkv: torch.Tensor, s: BlockShape):
        from . import attention as A

        if A.available() and s.head_dim == A.HEAD_DIM and A.supports(s.seq):
            out, lse = A.attention_fwd(qkv, s.batch, s.seq, s.n_heads, s.head_dim)
            return out, ("native", lse)
        h = s.n_heads * s.head_dim
        with torch.enable_grad():
            leaves = [qkv[:, i * h:(i + 1) * h].detach().requires_grad_(True) for i in range(3)]
            q, k, v = (t.view(s.batch, s.seq, s.n_heads, s.head_dim).transpose(1, 2) for t in leaves)
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
            out = o.transpose(1, 2).reshape(s.batch * s.seq, h)
        return out.detach(), ("sdpa", leaves, out)

    @staticmethod
    def backward(dout: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, saved, s: BlockShape) -> torch.Tensor:
        if saved[0] == "native":
            from . import attention as A

            return A.attention_bwd(dout, qkv, out, saved[1], s.batch, s.seq, s.n_heads, s.head_dim)
        _, leaves, graph_out = saved
        dq, dk, dv = torch.autograd.grad(graph_out, leaves, dout)
        return torch.cat([dq, dk, dv], dim=1)


# ---------------------------------------------------------------------------- the block node
def _fused_weight(parts: list[torch.Tensor]) -> torch.Tensor | None:
    """If ``parts`` are row-blocks laid out back to back in ONE storage, view them as one matrix.

    Adjacent addresses are not enough: two separate allocations can sit next to each other, and a
    view may not run past the storage it was made from.  So every part has to be a view of the
    same untyped storage, at consecutive element offsets, and that storage has to cover the whole
    stacked matrix.
    """
    first = parts[0]
    if first.dim() != 2:
        return None
    store = first.untyped_storage()
    base, esz = store.data_ptr(), first.element_size()
    off = first.storage_offset()
    cols = first.shape[1]
    rows = 0
    for p in parts:
        if (p.dim() != 2 or p.shape[1] != cols or p.dtype != first.dtype or not p.is_contiguous()
                or p.untyped_storage().data_ptr() != base or p.storage_offset() != off):
            return None
        off += p.numel()
        rows += p.shape[0]
    if off * esz > store.nbytes():
        return None
    return first.as_strided((rows, cols), (cols, 1))


class BlockParams:
    """Parameter handles of one decoder block, in flat (registration) order."""

    names = ("attn_norm", "wq", "wk", "wv", "wo", "mlp_norm", "w_gate", "w_up", "w_down")

    def __init__(self, module) -> None:
        self.module = module
        self.params = [getattr(module, n).weight if hasattr(getattr(module, n), "weight") else getattr(module, n)
                       for n in self.names]

    def sink(self, i: int) -> GradSink:
        return GradSink(self.params[i])


class DecoderBlockFunction(torch.autograd.Function):
    """Pre-norm decoder block: RMSNorm → QKV → RoPE → causal attention → O (+res) → RMSNorm →
    gate/up → SwiGLU → down (+res), forward and backward as explicit kernel sequences."""

    @staticmethod
    def forward(ctx, x, cos, sin, bp: BlockParams, shape: BlockShape, recompute: bool, *weights):
        ctx.bp, ctx.shape, ctx.recompute = bp, shape, recompute
        x = x.contiguous()
        acts = DecoderBlockFunction._forward_impl(x, cos, sin, weights, shape, bp)
        out = acts["out"]
        if recompute:
            ctx.save_for_backward(x, cos, sin, *weights)
            ctx.acts = None
        else:
            ctx.save_for_backward(x, cos, sin, *weights)
            ctx.acts = acts
        return out

    @staticmethod
    def _forward_impl(x, cos, sin, weights, s: BlockShape, bp: "BlockParams | None" = None) -> dict:
        from . import kernels as K

        wn1, wq, wk, wv, wo, wn2, wg, wu, wd = weights
        T, H, Fd = x.shape[0], s.hidden, s.ffn
        xn, rstd1 = K.rmsnorm_fwd(x, wn1, s.eps)
        qkv = torch.empty((T, 3 * H), dtype=x.dtype, device=x.device)
        wqkv = _fused_weight([wq, wk, wv])
        plan = _take_deferred_gather(bp, wqkv) if bp is not None else None
        if plan is not None:
            # the q|k|v rows of this unit's all-gather arrive inside this GEMM
            K.gemm_ag(xn, wqkv, plan, out=qkv)
        elif wqkv is not None:
            K.gemm(xn, wqkv, out=qkv)
        else:
            for i, w in enumerate((wq, wk, wv)):
                K.gemm(xn, w, out=qkv[:, i * H:(i + 1) * H])
        K.rope_(qkv, cos, sin, s.seq, 0, 2 * s.n_heads, s.head_dim)
        attn, attn_saved = _AttentionCore.forward(qkv, s)
        x1 = K.gemm(attn, wo, cin=x, beta=1.0)
        xn2, rstd2 = K.rmsnorm_fwd(x1, wn2, s.eps)
        gu = torch.empty((T, 2 * Fd), dtype=x.dtype, device=x.device)
        wgu = _fused_weight([wg, wu])
        if wgu is not None:
            K.gemm(xn2, wgu, out=gu)
        else:
            K.gemm(xn2, wg, out=gu[:, :Fd])
            K.gemm(xn2, wu, out=gu[:, Fd:])
        h = K.swiglu_fwd(gu)
        out = K.gemm(h, wd, cin=x1, beta=1.0)
        return dict(xn=xn, rstd1=rstd1, qkv=qkv, attn=attn, attn_saved=attn_saved, x1=x1, xn2=xn2, rstd2=rstd2,
                    gu=gu, h=h, out=out)

    @staticmethod
    def backward(ctx, dout):
        from . import kernels as K

        s: BlockShape = ctx.shape
        bp: BlockParams = ctx.bp
        x, cos, sin, *weights = ctx.saved_tensors
        wn1, wq, wk, wv, wo, wn2, wg, wu, wd = weights
        acts = ctx.acts
        if acts is None:
            with torch.no_grad():
                acts = DecoderBlockFunction._forward_impl(x, cos, sin, weights, s)
        ctx.acts = None
        dout = dout.contiguous()
        T, H, Fd = x.shape[0], s.hidden, s.ffn
        grads: list = [None] * 9

        # ---- MLP
        dh = K.gemm(dout, wd, b_mn_major=True)                       # [T, F]
        grads[8] = _wgrad(dout, acts["h"], bp.sink(8))
        dgu = K.swiglu_bwd(dh, acts["gu"])                            # [T, 2F]
        del dh
        wgu = _fused_weight([wg, wu])
        if wgu is not None:
            dxn2 = K.gemm(dgu, wgu, b_mn_major=True)
        else:
            dxn2 = K.gemm(dgu[:, :Fd], wg, b_mn_major=True)
            K.gemm(dgu[:, Fd:], wu, b_mn_major=True, out=dxn2, cin=dxn2, beta=1.0)
        grads[6], grads[7] = _wgrad_pair(dgu, acts["xn2"], (bp.sink(6), bp.sink(7)), (Fd, Fd))
        del dgu
        dx1, grads[5] = _norm_bwd(dxn2, acts["x1"], wn2, acts["rstd2"], dout, bp.sink(5))
        del dxn2

        # ---- attention
        dattn = K.gemm(dx1, wo, b_mn_major=True)
        grads[4] = _wgrad(dx1, acts["attn"], bp.sink(4))
        dqkv = _AttentionCore.backward(dattn, acts["qkv"], acts["attn"], acts["attn_saved"], s)
        del dattn
        dqkv = dqkv.contiguous()
        K.rope_(dqkv, cos, sin, s.seq, 0, 2 * s.n_heads, s.head_dim, backward=True)
        wqkv = _fused_weight([wq, wk, wv])
        if wqkv is not None:
            dxn = K.gemm(dqkv, wqkv, b_mn_major=True)
        else:
            dxn = K.gemm(dqkv[:, :H], wq, b_mn_major=True)
            K.gemm(dqkv[:, H:2 * H], wk, b_mn_major=True, out=dxn, cin=dxn, beta=1.0)
            K.gemm(dqkv[:, 2 * H:], wv, b_mn_major=True, out=dxn, cin=dxn, beta=1.0)
        grads[1], grads[2], grads[3] = _wgrad_pair(dqkv, acts["xn"], (bp.sink(1), bp.sink(2), bp.sink(3)), (H, H, H))
        del dqkv
        dx, grads[0] = _norm_bwd(dxn, x, wn1, acts["rstd1"], dx1, bp.sink(0))
        return (dx, None, None, None, None, None, *grads)


def _take_deferred_gather(bp: "BlockParams", wqkv: torch.Tensor | None):
    """Plan of the all-gather rows that the owning FSDP unit left to the QKV GEMM, if any."""
    ref = getattr(bp.params[1], "_mfsdp_unit_ref", None)
    unit = ref() if ref is not None else None
    if unit is None or unit.flat_buffer.deferred_gather is None:
        return None
    if wqkv is None:
        unit.flat_buffer.complete_deferred_gather()
        return None
    return unit.flat_buffer.take_deferred_gather(wqkv)


def _norm_bwd(dy, x, w, rstd, dres, sink: GradSink):
    from . import kernels as K

    unit = sink.target()
    if unit is None:
        dx, dw = K.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
        return dx, dw
    fqn = sink.param._matrix_fsdp_fqn
    view, acc = unit.grad_target(fqn)
    dx, _ = K.rmsnorm_bwd(dy, x, w, rstd, dres=dres, dw_out=view, accumulate_dw=acc)
    unit.mark_grad_written(fqn)
    return dx, None


def _wgrad_pair(dy: torch.Tensor, x: torch.Tensor, sinks, widths):
    """Weight gradients of row-stacked weights: one wide GEMM when their bucket slots are contiguous."""
    from . import kernels as K

    units = [s.target() for s in sinks]
    if all(u is not None for u in units) and len({id(u) for u in units}) == 1:
        unit = units[0]
        views, accs = zip(*(unit.grad_target(s.param._matrix_fsdp_fqn) for s in sinks))
        fused = _fused_weight(list(views))
        if fused is not None and len(set(accs)) == 1:
            acc = accs[0]
            K.gemm(dy, x, a_mn_major=True, b_mn_major=True, out=fused, cin=fused if acc else None,
                   beta=1.0 if acc else 0.0)
            for s in sinks:
                unit.mark_grad_written(s.param._matrix_fsdp_fqn)
            return (None,) * len(sinks)
    out, col = [], 0
    for s, w in zip(sinks, widths):
        out.append(_wgrad(dy[:, col:col + w], x, s))
        col += w
    return tuple(out)


def decoder_block(x: torch.Tensor, module, shape: BlockShape, cos: torch.Tensor, sin: torch.Tensor,
                  recompute: bool = False) -> torch.Tensor:
    """Run one decoder block (``x``: [B*S, H] bf16 on CUDA) through the fused node."""
    bp = getattr(module, "_block_params", None)
    if bp is None:
        bp = BlockParams(module)
        module._block_params = bp
    return DecoderBlockFunction.apply(x, cos, sin, bp, shape, recompute, *bp.params)
