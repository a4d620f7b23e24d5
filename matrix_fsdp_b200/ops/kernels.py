"""Tensor-level entry points of the sm_100a kernel library.

Each function validates shapes/dtypes, launches on the current CUDA stream and returns
torch tensors.  They are the non-differentiable building blocks; autograd wiring lives
in :mod:`matrix_fsdp_b200.ops.functional`.

The reference has two device kernels of its own, both plain copies
(``matrix_fsdp/kernels/native/matrix_copy_cuda.cu:8-36``, bound in ``matrix_copy.cpp:1-162`` and loaded by
``matrix_fsdp/kernels/native.py:1-492``); every model op there goes through PyTorch / cuBLAS.  ``copy_segments``
here is the counterpart of those copies; everything else replaces library calls of the reference's bench models
(``test/fsdp/bench_fsdp2_compare.py:456-483``) and of ``torch.optim`` (AdamW, SGD, ``torch/optim/_muon.py:276-310``).
"""
from __future__ import annotations

import torch

from . import lib as _lib

_STATUS: dict[int, torch.Tensor] = {}
_SM_COUNT: dict[int, int] = {}
_SCRATCH: dict[tuple, torch.Tensor] = {}


def _L():
    return _lib.load(required=True)


def launch_count() -> int:
    return _lib.launch_count()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait runs out."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    t = _STATUS.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _STATUS[idx] = t
    return t


def check_status(device=None, reset: bool = True) -> int:
    """Read (device->host) the status word; raises if a kernel reported a timeout."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        if reset:
            w.zero_()
        names = {1: "mbarrier wait timed out", 2: "peer flag wait timed out", 3: "bad argument",
                 4: "index out of bounds"}
        raise RuntimeError(f"device status {code}: {names.get(code, 'unknown')}")
    return code


def sm_count(device=None) -> int:
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    n = _SM_COUNT.get(idx)
    if n is None:
        n = torch.cuda.get_device_properties(idx).multi_processor_count
        _SM_COUNT[idx] = n
    return n


def _scratch_f32(n: int, device, tag: str) -> torch.Tensor:
    key = (tag, torch.device(device).index, n)
    t = _SCRATCH.get(key)
    if t is None:
        t = torch.zeros(n, dtype=torch.float32, device=device)
        _SCRATCH[key] = t
    return t


# ------------------------------------------------------------------ GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False, b_mn_major: bool = False,
         out: torch.Tensor | None = None, cin: torch.Tensor | None = None, alpha: float = 1.0,
         beta: float = 0.0, force_bn: int = 0, symmetric: bool = False) -> torch.Tensor:
    """``out[M,N] = alpha * A·Bᵀ + beta * cin`` on the tcgen05 kernel (bf16, fp32 accumulate).

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn_major``); ``b`` is ``[N,K]`` (or ``[K,N]`` when
    ``b_mn_major``).  Row strides must be multiples of 8 elements, inner stride 1.
    ``symmetric``: the caller knows the result equals its transpose (M == N, a multiple of 128); only the
    tiles on or above the diagonal are computed and the rest is mirrored (about half the tensor-core work).
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_mn_major:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn_major:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"reduce dims differ: {K} vs {Kb}"
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype == torch.bfloat16
    if cin is not None:
        assert cin.shape == (M, N) and cin.stride(1) == 1 and cin.dtype == torch.bfloat16
    if symmetric:
        assert M == N and N % 128 == 0, "symmetric outputs must be square with a multiple of 128 rows"
    rc = (_L().mfsdp_gemm_bf16_sym if symmetric else _L().mfsdp_gemm_bf16)(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), cin.data_ptr() if cin is not None else None,
        M, N, K, a.stride(0), b.stride(0), out.stride(0), cin.stride(0) if cin is not None else 0,
        int(a_mn_major), int(b_mn_major), float(alpha), float(beta), 0, None, None, 0, 0,
        status_word(a.device).data_ptr(), sm_count(a.device), force_bn, _stream())
    _lib.check(rc, "mfsdp_gemm_bf16")
    if symmetric:
        mirror_upper_(out, 1)
    return out


def mirror_upper_(d: torch.Tensor, mats: int = 1) -> torch.Tensor:
    """``d``: ``mats`` square matrices stacked along dim 0 (``[mats * n, n]``); copies each matrix's upper
    triangle onto its lower one in 64 x 64 blocks (diagonal blocks are left as they are)."""
    n = d.shape[-1]
    assert d.dtype == torch.bfloat16 and d.stride(-1) == 1 and d.numel() == mats * n * n and d.is_contiguous()
    _lib.check(_L().mfsdp_mirror_upper(d.data_ptr(), n, n, mats, _stream()), "mfsdp_mirror_upper")
    return d


def gemm_ag(a: torch.Tensor, b: torch.Tensor, plan, *, out: torch.Tensor | None = None,
            cin: torch.Tensor | None = None, alpha: float = 1.0, beta: float = 0.0) -> torch.Tensor:
    """``out = alpha * a·bᵀ + beta * cin`` where rows of ``b`` ([N, K], contiguous) are still on peer GPUs.

    ``plan`` (see ``parallel.peer.DeferredGather``) lists the copy jobs that bring them into ``b``'s
    local storage; the kernel runs them on eight extra warps per CTA while tiles whose rows have
    arrived are multiplied.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and b.is_contiguous() and a.stride(1) == 1
    M, Kd = a.shape
    N = b.shape[0]
    assert b.shape[1] == Kd and b.data_ptr() == plan.b_ptr and plan.bn in (128, 256)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    plan.flags.zero_()
    rc = _L().mfsdp_gemm_bf16_ag(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), cin.data_ptr() if cin is not None else None, M, N, Kd,
        a.stride(0), out.stride(0), cin.stride(0) if cin is not None else 0, alpha, beta,
        plan.src.data_ptr(), plan.dst.data_ptr(), plan.nbytes.data_ptr(), plan.flag_idx.data_ptr(), plan.njobs,
        plan.flags.data_ptr(), plan.need.data_ptr(), plan.first.data_ptr(), int(plan.rotate), plan.bn,
        int(plan.budget_ns),
        status_word(a.device).data_ptr(), sm_count(a.device), _stream())
    _lib.check(rc, "mfsdp_gemm_bf16_ag")
    return out


def grouped_gemm_m(a: torch.Tensor, b: torch.Tensor, tile_group: torch.Tensor, *,
                   b_mn_major: bool = False, out: torch.Tensor | None = None, cin: torch.Tensor | None = None,
                   alpha: float = 1.0, beta: float = 0.0, symmetric: bool = False,
                   groups_of_256_rows: bool = False) -> torch.Tensor:
    """M-grouped GEMM: rows of ``a`` come in 128-row tiles, tile ``t`` uses ``b[tile_group[t]]``;
    ``out = alpha * a·b[g]ᵀ + beta * cin`` (``cin``: ``[Mtot, N]``).

    ``a``: ``[Mtot, K]``; ``b``: ``[G, N, K]`` (or ``[G, K, N]`` when ``b_mn_major``); tiles whose
    group id is negative are skipped (their output rows are left untouched).  ``symmetric``: ``a`` stacks
    ``Mtot / N`` blocks of ``N`` rows whose outputs are symmetric ``N x N`` matrices (``N`` a multiple of 128);
    tiles below the diagonal are mirrored instead of computed.  ``groups_of_256_rows``: the caller's promise that
    every group has a multiple of 256 rows, which lets the two-CTA kernel (256 x 256 tiles) run.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and b.dim() == 3
    assert b.is_contiguous() and a.stride(1) == 1 and tile_group.dtype == torch.int32
    Mtot, K = a.shape
    G = b.shape[0]
    if b_mn_major:
        assert b.shape[1] == K
        N = b.shape[2]
        ldb = N
    else:
        assert b.shape[2] == K
        N = b.shape[1]
        ldb = K
    assert tile_group.numel() >= (Mtot + 127) // 128
    if out is None:
        out = torch.empty((Mtot, N), dtype=torch.bfloat16, device=a.device)
    if cin is not None:
        assert cin.shape == (Mtot, N) and cin.stride(1) == 1 and cin.dtype == torch.bfloat16
    if symmetric:
        assert N % 128 == 0 and Mtot % N == 0 and out.is_contiguous()
    rc = (_L().mfsdp_gemm_bf16_sym if symmetric else _L().mfsdp_gemm_bf16)(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), cin.data_ptr() if cin is not None else None, Mtot, N, K,
        a.stride(0), ldb, out.stride(0), cin.stride(0) if cin is not None else 0, 0, int(b_mn_major),
        float(alpha), float(beta), 1, tile_group.data_ptr(), None, G, 0,
        status_word(a.device).data_ptr(), sm_count(a.device), 2 if groups_of_256_rows and Mtot % 256 == 0 else 0, _stream())
    _lib.check(rc, "mfsdp_gemm_bf16[m-grouped]")
    if symmetric:
        mirror_upper_(out, Mtot // N)
    return out


def grouped_gemm_k(a: torch.Tensor, b: torch.Tensor, group_offsets: torch.Tensor, num_groups: int,
                   out: torch.Tensor | None = None, symmetric: bool = False) -> torch.Tensor:
    """K-grouped GEMM (expert wgrad): ``out[g] = a[rows_g]ᵀ · b[rows_g]``.

    ``a``: ``[Ktot, M]``, ``b``: ``[Ktot, N]``; ``group_offsets`` int32 ``[G+1]`` with offsets that
    are multiples of 64; ``M`` must be a multiple of 128.  Returns ``[G, M, N]``.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    Ktot, M = a.shape
    N = b.shape[1]
    assert b.shape[0] == Ktot and group_offsets.dtype == torch.int32
    if out is None:
        out = torch.empty((num_groups, M, N), dtype=torch.bfloat16, device=a.device)
    if symmetric:     # every out[g] equals its transpose (a is b): mirror instead of computing the lower tiles
        assert M == N and N % 128 == 0 and out.is_contiguous()
    rc = (_L().mfsdp_gemm_bf16_sym if symmetric else _L().mfsdp_gemm_bf16)(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), None, M, N, 0, a.stride(0), b.stride(0), N, 0,
        1, 1, 1.0, 0.0, 2, None, group_offsets.data_ptr(), num_groups, Ktot,
        status_word(a.device).data_ptr(), sm_count(a.device), 0, _stream())
    _lib.check(rc, "mfsdp_gemm_bf16[k-grouped]")
    if symmetric:
        mirror_upper_(out.view(num_groups * M, N), num_groups)
    return out


# ------------------------------------------------------------------ norm / rope / swiglu / CE
def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float):
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    assert x2.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    y = torch.empty_like(x2)
    rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    _lib.check(_L().mfsdp_rmsnorm_fwd(x2.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(),
                                      x2.shape[0], H, float(eps), _stream()), "rmsnorm_fwd")
    return y.view(x.shape), rstd


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor,
                dres: torch.Tensor | None = None, dw_out: torch.Tensor | None = None,
                accumulate_dw: bool = False):
    """Returns ``(dx, dw)``; ``dx`` already includes ``dres`` (the residual-stream gradient)."""
    H = x.shape[-1]
    x2, dy2 = x.reshape(-1, H), dy.reshape(-1, H)
    assert x2.is_contiguous() and dy2.is_contiguous()
    dx = torch.empty_like(x2)
    acc = _scratch_f32(min(x2.shape[0], 148 * 4) * H, x.device, "rms_dw")
    if dw_out is None:
        dw_out = torch.empty(H, dtype=torch.bfloat16, device=x.device)
        accumulate_dw = False
    dr = dres.reshape(-1, H) if dres is not None else None
    _lib.check(_L().mfsdp_rmsnorm_bwd(dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                      dr.data_ptr() if dr is not None else None, dx.data_ptr(),
                                      acc.data_ptr(), dw_out.data_ptr(), int(accumulate_dw),
                                      x2.shape[0], H, _stream()), "rmsnorm_bwd")
    return dx.view(x.shape), dw_out


def rope_(buf: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_len: int, col0: int,
          n_heads: int, head_dim: int, backward: bool = False) -> torch.Tensor:
    """In-place rotary embedding on ``n_heads`` heads starting at column ``col0`` of ``[T, ld]``."""
    assert buf.dim() == 2 and buf.stride(1) == 1 and buf.dtype == torch.bfloat16
    assert cos.dtype == torch.float32 and cos.is_contiguous() and cos.shape[-1] == head_dim // 2
    assert cos.shape[0] >= seq_len
    _lib.check(_L().mfsdp_rope(buf.data_ptr(), cos.data_ptr(), sin.data_ptr(), buf.shape[0], seq_len,
                               buf.stride(0), col0, n_heads, head_dim, -1.0 if backward else 1.0,
                               _stream()), "rope")
    return buf


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    T, F2 = gu.shape
    assert gu.is_contiguous() and gu.dtype == torch.bfloat16
    h = torch.empty((T, F2 // 2), dtype=torch.bfloat16, device=gu.device)
    _lib.check(_L().mfsdp_swiglu_fwd(gu.data_ptr(), h.data_ptr(), T, F2 // 2, _stream()), "swiglu_fwd")
    return h


def swiglu_bwd(dh: torch.Tensor, gu: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    T, F2 = gu.shape
    assert dh.is_contiguous() and gu.is_contiguous()
    dgu = out if out is not None else torch.empty_like(gu)
    _lib.check(_L().mfsdp_swiglu_bwd(dh.data_ptr(), gu.data_ptr(), dgu.data_ptr(), T, F2 // 2, _stream()),
               "swiglu_bwd")
    return dgu


_EMBED_WORK: dict[tuple, torch.Tensor] = {}


def embedding_bwd(dy: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """``out[v] (+)= sum of dy[t] over positions with ids[t] == v`` (bf16 rows, fp32 sums in position order).

    ``dy``: ``[T, H]`` bf16, ``ids``: ``[T]`` int64, ``out``: ``[V, H]`` bf16 with unit inner stride.  Without
    ``accumulate`` every row of ``out`` is written (zeros where an id does not occur)."""
    assert dy.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and ids.dtype == torch.int64
    assert dy.dim() == 2 and out.dim() == 2 and dy.stride(1) == 1 and out.stride(1) == 1 and ids.is_contiguous()
    T, H = dy.shape
    V = out.shape[0]
    assert out.shape[1] == H and ids.numel() == T
    key = (V, T, str(dy.device))
    work = _EMBED_WORK.get(key)
    if work is None:      # count | start | order; reused by every call of this size (calls are stream-ordered)
        work = _EMBED_WORK[key] = torch.empty(2 * V + T, dtype=torch.int32, device=dy.device)
    _lib.check(_L().mfsdp_embedding_bwd(dy.data_ptr(), dy.stride(0), ids.data_ptr(), out.data_ptr(), out.stride(0),
                                        T, V, H, int(accumulate), work.data_ptr(), _stream()), "embedding_bwd")
    return out


def cross_entropy_(logits: torch.Tensor, target: torch.Tensor, grad_scale: float | torch.Tensor,
                   ignore_index: int = -100) -> torch.Tensor:
    """Per-row loss (fp32); ``logits`` is overwritten with ``(softmax - onehot) * grad_scale``.
    ``grad_scale`` is a host float or a one-element fp32 device tensor (read by the kernel, no host sync)."""
    assert logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype == torch.bfloat16
    assert target.dtype == torch.int64 and target.is_contiguous()
    rows, V = logits.shape
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    if isinstance(grad_scale, torch.Tensor):
        assert grad_scale.dtype == torch.float32 and grad_scale.numel() == 1 and grad_scale.device == logits.device
        _lib.check(_L().mfsdp_cross_entropy_dev_scale(logits.data_ptr(), target.data_ptr(), loss.data_ptr(), rows, V,
                                                      logits.stride(0), grad_scale.data_ptr(), int(ignore_index),
                                                      _stream()), "cross_entropy")
        return loss
    _lib.check(_L().mfsdp_cross_entropy(logits.data_ptr(), target.data_ptr(), loss.data_ptr(), rows, V,
                                        logits.stride(0), float(grad_scale), int(ignore_index),
                                        _stream()), "cross_entropy")
    return loss


# ------------------------------------------------------------------ optimizers
def adamw_flat_(p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor, *, lr: float,
                beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
                grad_scale: float = 1.0, p_lp: torch.Tensor | None = None) -> None:
    assert p.dtype == torch.float32 and m.dtype == torch.float32 and v.dtype == torch.float32
    assert g.dtype in (torch.bfloat16, torch.float32) and g.numel() == p.numel()
    _lib.check(_L().mfsdp_adamw_flat(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(),
                                     int(g.dtype == torch.bfloat16),
                                     p_lp.data_ptr() if p_lp is not None else None, p.numel(),
                                     lr, beta1, beta2, eps, weight_decay, int(step), grad_scale,
                                     _stream()), "adamw_flat")


def sgd_flat_(p: torch.Tensor, mom: torch.Tensor | None, g: torch.Tensor, *, lr: float,
              momentum: float, weight_decay: float, first_step: bool, grad_scale: float = 1.0,
              p_lp: torch.Tensor | None = None) -> None:
    assert p.dtype == torch.float32
    _lib.check(_L().mfsdp_sgd_flat(p.data_ptr(), mom.data_ptr() if mom is not None else None,
                                   g.data_ptr(), int(g.dtype == torch.bfloat16),
                                   p_lp.data_ptr() if p_lp is not None else None, p.numel(), lr,
                                   momentum, weight_decay, grad_scale, int(first_step), _stream()),
               "sgd_flat")


def muon_momentum(buf: torch.Tensor, g: torch.Tensor, u_out: torch.Tensor, sumsq: torch.Tensor,
                  mu: float, grad_scale: float, nesterov: bool) -> None:
    _lib.check(_L().mfsdp_muon_momentum(buf.data_ptr(), g.data_ptr(), int(g.dtype == torch.bfloat16),
                                        u_out.data_ptr(), sumsq.data_ptr(), buf.numel(), mu,
                                        grad_scale, int(nesterov), _stream()), "muon_momentum")


def muon_normalize_(x: torch.Tensor, sumsq: torch.Tensor, eps: float = 1e-7) -> None:
    _lib.check(_L().mfsdp_muon_normalize(x.data_ptr(), sumsq.data_ptr(), x.numel(), eps, _stream()),
               "muon_normalize")


def muon_apply_(p: torch.Tensor, o: torch.Tensor, rows: int, cols: int, transposed: bool, lr: float,
                weight_decay: float, adjusted_lr: float, p_lp: torch.Tensor | None = None) -> None:
    _lib.check(_L().mfsdp_muon_apply(p.data_ptr(), o.data_ptr(),
                                     p_lp.data_ptr() if p_lp is not None else None, rows, cols,
                                     int(transposed), lr, weight_decay, adjusted_lr, _stream()),
               "muon_apply")


# ------------------------------------------------------------------ copies
def copy_segments(src: torch.Tensor, dst: torch.Tensor, src_off: torch.Tensor, dst_off: torch.Tensor,
                  lens: torch.Tensor, max_len: int) -> None:
    """``dst[dst_off[s] : +len[s]] = src[src_off[s] : +len[s]]`` for device int64 tables."""
    assert src.dtype == dst.dtype and src_off.dtype == torch.int64
    _lib.check(_L().mfsdp_copy_segments(src.data_ptr(), dst.data_ptr(), src_off.data_ptr(),
                                        dst_off.data_ptr(), lens.data_ptr(), src_off.numel(),
                                        int(max_len), src.element_size(), _stream()), "copy_segments")


def cast_f32_bf16(src: torch.Tensor, dst: torch.Tensor) -> None:
    assert src.dtype == torch.float32 and dst.dtype == torch.bfloat16 and src.numel() == dst.numel()
    _lib.check(_L().mfsdp_cast_f32_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), _stream()),
               "cast_f32_bf16")
