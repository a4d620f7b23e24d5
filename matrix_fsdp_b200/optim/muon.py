"""Muon for whole-matrix owners: momentum + Nesterov, quintic Newton-Schulz, decoupled decay.

Update rule (identical to ``torch.optim.Muon``, ``torch/optim/_muon.py:276-310``)::

    buf  <- lerp(buf, g, 1 - mu);  u <- nesterov ? lerp(g, buf, mu) : buf
    X    <- bf16(u) (transposed if rows > cols);  X <- X / max(||X||_F, eps)
    k times:  A = X Xᵀ;  B = b A + c A A;  X = a X + B X
    p    <- p (1 - lr wd) - adjust(lr, shape) * X

On CUDA each Newton-Schulz product runs on the tcgen05 GEMM with the polynomial folded into
the epilogue (``alpha * acc + beta * C``), so an iteration is three kernels with no separate
axpy, and tall matrices are handled by switching operand majors instead of transposing.  The Gram
matrix and its polynomial are symmetric: their GEMMs compute only the tiles that reach the diagonal
or lie above it and a small block-transpose kernel mirrors the rest (two of the three products of an
iteration do about half the tensor-core work).  The
element-wise stages (momentum/Nesterov + Frobenius norm, scaling, parameter update + bf16 emit)
are single fused kernels.  The reference delegates all of this to ``torch.optim.Muon``
(``matrix_fsdp/optim/wrapper.py:416-429``), i.e. 15 cuBLAS ``addmm`` calls per matrix.
"""
from __future__ import annotations

import math
import os
from collections.abc import Iterable

import torch
from torch.optim import Optimizer

DEFAULT_NS_COEFFICIENTS = (3.4445, -4.7750, 2.0315)
DEFAULT_MUON_ADJUST_LR_FN = "match_rms_adamw"
EPS = 1e-7
MAX_BATCH_ELEMENTS = 1 << 28      # elements of one stacked Newton-Schulz operand (512 MB of bf16)
SHARE_WINDOW_ELEMENTS = 1 << 29   # elements exchanged per all-reduce when replicas share Newton-Schulz (1 GB of bf16)
# X Xᵀ and b A + c A A are symmetric: compute the tiles on or above the diagonal, mirror the rest
SYMMETRIC_PRODUCTS = os.environ.get("MFSDP_MUON_SYMMETRIC", "1") != "0"


def adjust_lr(lr: float, adjust_lr_fn: str | None, shape) -> float:
    a, b = int(shape[0]), int(shape[1])
    if adjust_lr_fn is None or adjust_lr_fn == "original":
        return lr * math.sqrt(max(1.0, a / b))
    if adjust_lr_fn == "match_rms_adamw":
        return lr * 0.2 * math.sqrt(max(a, b))
    raise ValueError(f"Unknown adjust_lr_fn={adjust_lr_fn!r}; expected 'original' or 'match_rms_adamw'.")


def newton_schulz_reference(u: torch.Tensor, coefficients=DEFAULT_NS_COEFFICIENTS, steps: int = 5,
                            eps: float = EPS) -> torch.Tensor:
    """Plain torch implementation (CPU path and test oracle)."""
    a, b, c = coefficients
    x = u.bfloat16()
    tall = x.size(0) > x.size(1)
    if tall:
        x = x.T
    x = x / x.norm().clamp(min=eps)
    for _ in range(steps):
        g = x @ x.T
        bm = torch.addmm(g, g, g, beta=b, alpha=c)
        x = torch.addmm(x, bm, x, beta=a)
    return x.T if tall else x


def _symmetric_pays(n: int, matrices: int) -> bool:
    """Skipping the tiles below the diagonal only shortens a product that has more than one wave of 256 x 256
    tiles to begin with (74 CTA pairs); below that the extra mirror launch costs more than it saves (measured:
    2048 x 2048 slower, 4096 x 4096 1.35x faster than the full products)."""
    return SYMMETRIC_PRODUCTS and matrices * (n // 256) ** 2 >= 148


def newton_schulz_sm100(x: torch.Tensor, coefficients=DEFAULT_NS_COEFFICIENTS, steps: int = 5) -> torch.Tensor:
    """Newton-Schulz on an already normalised bf16 ``[rows, cols]`` matrix with tcgen05 GEMMs.

    Works in the matrix's own orientation: for tall matrices the Gram matrix is ``XᵀX`` and the
    update is ``X <- a X + X B`` (``B`` is symmetric), so nothing is ever transposed in memory.
    """
    from ..ops import kernels as K

    a, b, c = coefficients
    rows, cols = x.shape
    tall = rows > cols
    n = cols if tall else rows
    gram = torch.empty((n, n), dtype=torch.bfloat16, device=x.device)
    poly = torch.empty_like(gram)
    nxt = torch.empty_like(x)
    sym = n % 128 == 0 and _symmetric_pays(n, 1)  # Gram matrix and its polynomial equal their transposes
    for _ in range(steps):
        if tall:
            K.gemm(x, x, a_mn_major=True, b_mn_major=True, out=gram, symmetric=sym)            # XᵀX
            K.gemm(gram, gram, out=poly, cin=gram, alpha=c, beta=b, symmetric=sym)             # bA + cAA
            K.gemm(x, poly, out=nxt, cin=x, alpha=1.0, beta=a)                  # aX + X B
        else:
            K.gemm(x, x, out=gram, symmetric=sym)                                              # XXᵀ
            K.gemm(gram, gram, out=poly, cin=gram, alpha=c, beta=b, symmetric=sym)
            K.gemm(poly, x, b_mn_major=True, out=nxt, cin=x, alpha=1.0, beta=a)  # aX + B X
        x, nxt = nxt, x
    return x


_TILE_GROUPS: dict[tuple, torch.Tensor] = {}


def _tile_groups(groups: int, rows_per_group: int, device) -> torch.Tensor:
    """int32 group id of every 128-row tile of ``groups`` stacked matrices of ``rows_per_group`` rows."""
    key = (groups, rows_per_group, str(device))
    t = _TILE_GROUPS.get(key)
    if t is None:
        t = torch.arange(groups, dtype=torch.int32, device=device).repeat_interleave(rows_per_group // 128)
        _TILE_GROUPS[key] = t
    return t


def newton_schulz_sm100_batched(x: torch.Tensor, coefficients=DEFAULT_NS_COEFFICIENTS, steps: int = 5) -> torch.Tensor:
    """Newton-Schulz on ``G`` normalised bf16 matrices of one shape, stacked as ``[G, rows, cols]``: every
    product of an iteration is ONE grouped tcgen05 launch over all matrices (three launches per iteration
    whatever G is), so the tiles of several matrices fill the 148 SMs' waves together — a single
    4096 x 4096 product is 3.5 waves of 128 x 256 tiles, i.e. the last wave runs half empty.

    Needs ``min(rows, cols)`` and, for tall matrices, ``rows`` to be multiples of 128 (tiles must not
    straddle two matrices); callers fall back to :func:`newton_schulz_sm100` otherwise.
    """
    from ..ops import kernels as K

    a, b, c = coefficients
    G, rows, cols = x.shape
    tall = rows > cols
    n = cols if tall else rows
    dev = x.device
    gram = torch.empty((G * n, n), dtype=torch.bfloat16, device=dev)
    poly = torch.empty_like(gram)
    x2 = x.reshape(G * rows, cols)
    nxt = torch.empty_like(x2)
    tg_n = _tile_groups(G, n, dev)
    sym = _symmetric_pays(n, G)       # n is a multiple of 128 here
    p_n, p_rows = n % 256 == 0, rows % 256 == 0      # whole 256-row tiles per matrix: the two-CTA kernel may run
    if tall:
        offsets = torch.arange(G + 1, dtype=torch.int32, device=dev) * rows
        tg_rows = _tile_groups(G, rows, dev)
    for _ in range(steps):
        if tall:
            K.grouped_gemm_k(x2, x2, offsets, G, out=gram.view(G, n, n), symmetric=sym)                   # XᵀX
            K.grouped_gemm_m(gram, gram.view(G, n, n), tg_n, out=poly, cin=gram, alpha=c, beta=b, symmetric=sym,
                             groups_of_256_rows=p_n)                                                      # bA + cAA
            K.grouped_gemm_m(x2, poly.view(G, n, n), tg_rows, out=nxt, cin=x2, alpha=1.0, beta=a,
                             groups_of_256_rows=p_rows)                                                   # aX + X B
        else:
            K.grouped_gemm_m(x2, x2.view(G, n, cols), tg_n, out=gram, symmetric=sym, groups_of_256_rows=p_n)   # XXᵀ
            K.grouped_gemm_m(gram, gram.view(G, n, n), tg_n, out=poly, cin=gram, alpha=c, beta=b, symmetric=sym,
                             groups_of_256_rows=p_n)
            K.grouped_gemm_m(poly, x2.view(G, n, cols), tg_n, b_mn_major=True, out=nxt, cin=x2, alpha=1.0, beta=a,
                             groups_of_256_rows=p_n)
        x2, nxt = nxt, x2
    return x2.view(G, rows, cols)


def can_batch_newton_schulz(shape) -> bool:
    rows, cols = int(shape[0]), int(shape[1])
    n = min(rows, cols)
    return n % 128 == 0 and (rows <= cols or rows % 128 == 0) and cols % 8 == 0


def _use_kernels(t: torch.Tensor) -> bool:
    if t.device.type != "cuda":
        return False
    from ..ops import lib

    if lib.disabled_by_env():
        return False
    lib.load(required=True)
    rows, cols = t.shape
    return rows % 8 == 0 and cols % 8 == 0


def ns_flops(shape, steps: int) -> int:
    """Multiply-add count of ``steps`` Newton-Schulz iterations on a ``shape`` matrix (used to balance work)."""
    m, n = min(shape), max(shape)
    return steps * (2 * m * m * n * 2 + 2 * m * m * m)


def assign_to_replicas(shapes: list, replicas: int, steps: int) -> list[int]:
    """Replica index per matrix: largest first onto the least loaded replica (ties: lowest index).  Depends only on
    the shapes and their order, so every replica computes the same table without talking."""
    load = [0] * replicas
    out = [0] * len(shapes)
    for j in sorted(range(len(shapes)), key=lambda j: (-ns_flops(shapes[j], steps), j)):
        r = min(range(replicas), key=lambda r: (load[r], r))
        out[j] = r
        load[r] += ns_flops(shapes[j], steps)
    return out


class MatrixMuon(Optimizer):
    """Muon over 2-D parameters that this rank owns whole (matrix-owner layouts).

    A step has three stages per matrix: *prepare* (momentum, Nesterov, Frobenius scaling -> the normalised
    operand), *orthogonalise* (Newton-Schulz) and *apply* (decay, update, low-precision copy).  Under hybrid
    sharding every replica owns the same matrices and holds the same reduced gradients, so
    :meth:`share_newton_schulz_over` splits the orthogonalisation -- by far the most expensive stage -- across
    the replicate group: each replica orthogonalises only its share (balanced by FLOPs), the results are
    exchanged with one all-reduce of a buffer that is zero where a replica did no work (``x + 0`` is exact), and
    every replica applies all of them.  The element-wise stages stay redundant so that the momentum buffers and
    parameters of the replicas remain bit-identical.
    """

    def __init__(self, params: Iterable, *, lr: float = 1e-3, weight_decay: float = 0.1, momentum: float = 0.95,
                 nesterov: bool = True, ns_coefficients=DEFAULT_NS_COEFFICIENTS, eps: float = EPS, ns_steps: int = 5,
                 adjust_lr_fn: str | None = None, low_precision_of=None) -> None:
        if lr < 0 or momentum < 0 or weight_decay < 0:
            raise ValueError("invalid Muon hyper-parameters")
        if adjust_lr_fn not in (None, "original", "match_rms_adamw"):
            raise ValueError(f"Unknown adjust_lr_fn={adjust_lr_fn!r}.")
        super().__init__(params, dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov,
                                      ns_coefficients=tuple(ns_coefficients), eps=eps, ns_steps=ns_steps,
                                      adjust_lr_fn=adjust_lr_fn))
        # optional callable param -> bf16 tensor to refresh after the update (all-gather source)
        self._low_precision_of = low_precision_of
        self.grad_scale = 1.0
        self.ns_share_group = None
        self.ns_matrices_done = 0        # matrices this rank orthogonalised in the last step (diagnostic)

    def share_newton_schulz_over(self, group) -> None:
        """Split Newton-Schulz over the ranks of ``group`` (the replicate group of a hybrid-sharded mesh); every
        rank of it must own the same matrices with the same gradients.  ``None`` switches sharing off."""
        self.ns_share_group = group

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self.ns_matrices_done = 0
        for group in self.param_groups:
            todo = []
            for p in group["params"]:
                if (p.grad is None and getattr(p, "_grad_override", None) is None) or p.numel() == 0:
                    continue
                if p.ndim != 2:
                    raise ValueError("Muon only supports 2D parameters; route the rest to AdamW.")
                todo.append(p)
            if not todo:
                continue
            if self.ns_share_group is not None:
                self._step_shared(todo, group)
                continue
            by_shape: dict[tuple, list] = {}
            for p in todo:
                if self._kernel_path(p) and can_batch_newton_schulz(p.shape):
                    by_shape.setdefault(tuple(p.shape), []).append(p)
                else:
                    self._apply(p, self._orthogonalize([self._prepare(p, group)], group)[0], group)
            # matrices of one shape go through Newton-Schulz together (one grouped launch per product)
            for shape, ps in by_shape.items():
                per_chunk = max(1, MAX_BATCH_ELEMENTS // (shape[0] * shape[1]))
                for i in range(0, len(ps), per_chunk):
                    chunk = ps[i:i + per_chunk]
                    for p, o in zip(chunk, self._orthogonalize([self._prepare(p, group) for p in chunk], group)):
                        self._apply(p, o, group)
        return loss

    def _grad_of(self, p):
        g = getattr(p, "_grad_override", None)   # a gradient kept in another dtype (expert-parallel slices)
        return p.grad if g is None else g

    def _kernel_path(self, p) -> bool:
        g = self._grad_of(p)
        buf = self.state.get(p, {}).get("momentum_buffer")
        return _use_kernels(p) and p.dtype == torch.float32 and (buf is None or buf.dtype == torch.float32) \
            and g is not None and g.is_contiguous()

    # ------------------------------------------------------------------ the three stages
    def _prepare(self, p: torch.Tensor, group: dict) -> torch.Tensor:
        """Momentum + Nesterov; returns the Newton-Schulz operand (kernel path: bf16, already divided by its
        Frobenius norm; otherwise the raw update, normalised inside the reference iteration)."""
        st = self.state[p]
        kernels = self._kernel_path(p)
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32 if p.dtype == torch.float32 else p.dtype)
        buf, mu, g = st["momentum_buffer"], group["momentum"], self._grad_of(p)
        if kernels:
            from ..ops import kernels as K

            u = torch.empty(p.shape, dtype=torch.bfloat16, device=p.device)
            ss = torch.zeros(1, dtype=torch.float32, device=p.device)
            K.muon_momentum(buf.view(-1), g.reshape(-1), u.view(-1), ss, mu, float(self.grad_scale), group["nesterov"])
            K.muon_normalize_(u.view(-1), ss, group["eps"])
            return u
        gf = g.to(buf.dtype)
        if self.grad_scale != 1.0:
            gf = gf * self.grad_scale
        buf.lerp_(gf, 1 - mu)
        return gf.lerp(buf, mu) if group["nesterov"] else buf

    def _orthogonalize(self, us: list, group: dict) -> list:
        """Newton-Schulz on each operand; same-shape bf16 CUDA operands go through the grouped kernels together."""
        self.ns_matrices_done += len(us)
        coef, steps = group["ns_coefficients"], group["ns_steps"]
        native = [u.is_cuda and u.dtype == torch.bfloat16 and _use_kernels(u) for u in us]
        if len(us) > 1 and all(native) and len({tuple(u.shape) for u in us}) == 1 and can_batch_newton_schulz(us[0].shape):
            return list(newton_schulz_sm100_batched(torch.stack(us), coef, steps).unbind(0))
        return [newton_schulz_sm100(u, coef, steps) if nat else newton_schulz_reference(u, coef, steps, group["eps"])
                for u, nat in zip(us, native)]

    def _apply(self, p: torch.Tensor, o: torch.Tensor, group: dict) -> None:
        lr, wd = float(group["lr"]), group["weight_decay"]
        alr = adjust_lr(lr, group["adjust_lr_fn"], p.shape)
        lp = self._low_precision_of(p) if self._low_precision_of is not None else None
        if self._kernel_path(p) and o.dtype == torch.bfloat16:
            from ..ops import kernels as K

            K.muon_apply_(p.data.view(-1), o.reshape(-1), p.shape[0], p.shape[1], False, lr, wd, alr,
                          p_lp=lp.view(-1) if lp is not None and lp.dtype == torch.bfloat16 else None)
            if lp is not None and lp.dtype != torch.bfloat16:
                lp.copy_(p.data)
            return
        p.data.mul_(1 - lr * wd)
        p.data.add_(o.to(p.dtype), alpha=-alr)
        if lp is not None:
            lp.copy_(p.data)

    # ------------------------------------------------------------------ shared across replicas
    def _step_shared(self, ps: list, group: dict) -> None:
        import torch.distributed as dist

        pg = self.ns_share_group
        replicas, me = dist.get_world_size(pg), dist.get_rank(pg)
        owner = assign_to_replicas([tuple(p.shape) for p in ps], replicas, group["ns_steps"])
        # Work through the matrices in windows of at most SHARE_WINDOW_ELEMENTS: the normalised operands and the
        # exchange buffer of a window are temporaries (2 x 2 bytes per element), and a model's worth of them at
        # once would cost as much memory as the bf16 parameters themselves.
        window: list[int] = []
        size = 0
        for j, p in enumerate(ps):
            n = (p.numel() + 7) // 8 * 8
            if window and size + n > SHARE_WINDOW_ELEMENTS:
                self._share_window(ps, window, owner, me, replicas, pg, group)
                window, size = [], 0
            window.append(j)
            size += n
        if window:
            self._share_window(ps, window, owner, me, replicas, pg, group)

    def _share_window(self, ps: list, window: list[int], owner: list[int], me: int, replicas: int, pg, group: dict) -> None:
        import torch.distributed as dist

        us = {j: self._prepare(ps[j], group) for j in window}          # every replica: keeps momentum in sync
        offsets, total = {}, 0
        for j in window:
            offsets[j] = total
            total += (ps[j].numel() + 7) // 8 * 8
        flat = torch.zeros(total, dtype=torch.bfloat16, device=ps[window[0]].device)
        mine_by_shape: dict[tuple, list[int]] = {}
        for j in window:
            if owner[j] == me:
                mine_by_shape.setdefault(tuple(ps[j].shape), []).append(j)
        for shape, idx in mine_by_shape.items():
            per_chunk = max(1, MAX_BATCH_ELEMENTS // (shape[0] * shape[1]))
            for i in range(0, len(idx), per_chunk):
                chunk = idx[i:i + per_chunk]
                for j, o in zip(chunk, self._orthogonalize([us[j] for j in chunk], group)):
                    flat[offsets[j]:offsets[j] + ps[j].numel()].copy_(o.reshape(-1))
        del us
        if replicas > 1:
            dist.all_reduce(flat, group=pg)
        for j in window:
            self._apply(ps[j], flat[offsets[j]:offsets[j] + ps[j].numel()].view(ps[j].shape), group)
