"""Tensor-level wrappers of the MoE routing / expert-parallel kernels in ``csrc/moe.cu``.

The reference ships no MoE kernels; the dispatcher these replace is the PyTorch fixture of its EP test
(``test/fsdp/test_deepseek_v3_ep_train.py:472-563``: four ``all_to_all_single`` calls, argsort, index_select,
scatter_add and a Python loop over local experts).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import lib as _lib

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float

_lib.register_signatures({
    "mfsdp_moe_router_topk": [_vp, _ll, _i, _i, _i, _vp, _vp, _vp, _vp, _vp],
    "mfsdp_moe_router_bwd": [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _ll, _vp],
    "mfsdp_moe_assign_slots": [_vp, _i, _i, _vp, _vp, _vp],
    "mfsdp_moe_push_counts": [_vp, _i, _i, _vp, _i, _vp],
    "mfsdp_moe_plan": [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "mfsdp_moe_zero_pad": [_vp, _i, _i, _vp, _vp, _vp],
    "mfsdp_moe_dispatch_push": [_vp, _ll, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _i, _vp],
    "mfsdp_moe_combine_pull": [_vp, _ll, _i, _i, _i, _vp, _vp, _vp, _vp, _ll, _i, _vp, _vp, _vp, _i, _vp],
    "mfsdp_moe_swiglu_bwd_dot": [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp],
})

_u64 = C.c_ulonglong


def _L():
    return _lib.load(required=True)


def _st() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def addr_array(addrs) -> C.Array:
    return (_u64 * len(addrs))(*[int(a) for a in addrs])


def router_topk(logits: torch.Tensor, top_k: int, prob_sum: torch.Tensor | None = None):
    """``logits`` [T, E] bf16 -> ``(probs [T, E] f32, idx [T, K] i32, weight [T, K] f32)``."""
    T, E = logits.shape
    probs = torch.empty(T, E, dtype=torch.float32, device=logits.device)
    idx = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    _lib.check(_L().mfsdp_moe_router_topk(logits.data_ptr(), logits.stride(0), T, E, top_k, probs.data_ptr(),
                                          idx.data_ptr(), w.data_ptr(), _p(prob_sum), _st()), "moe_router_topk")
    return probs, idx, w


def router_bwd(probs: torch.Tensor, idx: torch.Tensor, dw: torch.Tensor, aux_grad: torch.Tensor | None) -> torch.Tensor:
    T, E = probs.shape
    dlogits = torch.empty(T, E, dtype=torch.bfloat16, device=probs.device)
    _lib.check(_L().mfsdp_moe_router_bwd(probs.data_ptr(), idx.data_ptr(), dw.data_ptr(), _p(aux_grad), T, E,
                                         idx.shape[1], dlogits.data_ptr(), dlogits.stride(0), _st()), "moe_router_bwd")
    return dlogits


def assign_slots(idx: torch.Tensor, n_experts: int):
    """Deterministic queue position of every (token, k) entry and the per-expert counts."""
    n = idx.numel()
    slot = torch.empty(n, dtype=torch.int32, device=idx.device)
    counts = torch.empty(n_experts, dtype=torch.int32, device=idx.device)
    _lib.check(_L().mfsdp_moe_assign_slots(idx.data_ptr(), n, n_experts, slot.data_ptr(), counts.data_ptr(), _st()),
               "moe_assign_slots")
    return slot, counts


def push_counts(table_addrs, world: int, rank: int, counts: torch.Tensor) -> None:
    _lib.check(_L().mfsdp_moe_push_counts(addr_array(table_addrs), world, rank, counts.data_ptr(), counts.numel(),
                                          _st()), "moe_push_counts")


def plan(counts_all: torch.Tensor, world: int, rank: int, n_experts: int, cap_rows: int):
    dev = counts_all.device
    el = n_experts // world
    dest_base = torch.empty(n_experts, dtype=torch.int32, device=dev)
    group_offsets = torch.empty(el + 1, dtype=torch.int32, device=dev)
    group_rows = torch.empty(el, dtype=torch.int32, device=dev)
    tile_group = torch.empty(max(cap_rows // 128, 1), dtype=torch.int32, device=dev)
    stats = torch.zeros(2, dtype=torch.int32, device=dev)
    _lib.check(_L().mfsdp_moe_plan(counts_all.data_ptr(), world, rank, n_experts, cap_rows, dest_base.data_ptr(),
                                   group_offsets.data_ptr(), group_rows.data_ptr(), tile_group.data_ptr(),
                                   stats.data_ptr(), _st()), "moe_plan")
    return dest_base, group_offsets, group_rows, tile_group, stats


def zero_pad(buf: torch.Tensor, hidden: int, group_offsets: torch.Tensor, group_rows: torch.Tensor) -> None:
    _lib.check(_L().mfsdp_moe_zero_pad(buf.data_ptr(), hidden, group_rows.numel(), group_offsets.data_ptr(),
                                       group_rows.data_ptr(), _st()), "moe_zero_pad")


def dispatch_push(x: torch.Tensor, idx: torch.Tensor, recv_addrs, experts_per_rank: int, cap_rows: int, *,
                  slot: torch.Tensor | None = None, dest_base: torch.Tensor | None = None,
                  route: torch.Tensor | None = None, scale: torch.Tensor | None = None) -> torch.Tensor:
    """Store every (token, k) row of ``x`` into its expert owner's buffer; returns the route table."""
    T, H = x.shape
    K = idx.shape[1]
    route_out = None
    if route is None:
        route_out = torch.empty(T * K, dtype=torch.int32, device=x.device)
    _lib.check(_L().mfsdp_moe_dispatch_push(x.data_ptr(), x.stride(0), H, T * K, K, idx.data_ptr(), _p(slot),
                                            _p(dest_base), _p(route), _p(route_out), _p(scale), experts_per_rank,
                                            cap_rows, addr_array(recv_addrs), len(recv_addrs), _st()),
               "moe_dispatch_push")
    return route if route is not None else route_out


def combine_pull(src_addrs, idx: torch.Tensor, route: torch.Tensor, hidden: int, experts_per_rank: int, *,
                 weight: torch.Tensor | None = None, res: torch.Tensor | None = None, scalar_addrs=None):
    """Pull and sum each token's K expert rows; optionally also the per-row scalars."""
    T, K = idx.shape
    out = torch.empty(T, hidden, dtype=torch.bfloat16, device=idx.device)
    scal = torch.empty(T, K, dtype=torch.float32, device=idx.device) if scalar_addrs is not None else None
    _lib.check(_L().mfsdp_moe_combine_pull(out.data_ptr(), out.stride(0), hidden, T, K, idx.data_ptr(), route.data_ptr(),
                                           _p(weight), _p(res), res.stride(0) if res is not None else 0,
                                           experts_per_rank, addr_array(src_addrs),
                                           addr_array(scalar_addrs) if scalar_addrs is not None else None, _p(scal),
                                           len(src_addrs), _st()), "moe_combine_pull")
    return out, scal


def swiglu_bwd_dot(dh: torch.Tensor, gu: torch.Tensor, rowdot: torch.Tensor, row_limit: torch.Tensor | None = None):
    """Returns ``(dgu, h)`` and fills ``rowdot[row] = <h[row], dh[row]>``."""
    R, F2 = gu.shape
    dgu = torch.empty_like(gu)
    h = torch.empty(R, F2 // 2, dtype=gu.dtype, device=gu.device)
    _lib.check(_L().mfsdp_moe_swiglu_bwd_dot(dh.data_ptr(), gu.data_ptr(), dgu.data_ptr(), h.data_ptr(),
                                             rowdot.data_ptr(), R, F2 // 2, _p(row_limit), _st()),
               "moe_swiglu_bwd_dot")
    return dgu, h
