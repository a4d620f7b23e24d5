"""Causal attention kernels (head_dim 128) for sm_100a: Python entry points.

``fwd_available()`` / ``bwd_available()`` report whether the tcgen05 attention kernels are present in
the loaded kernel library; ``available()`` (both) is what the training path checks before it leaves
the library SDPA kernel.  The op matches ``F.scaled_dot_product_attention(q, k, v, is_causal=True)``
as used by the reference's bench models (test/fsdp/bench_fsdp2_compare.py:419,480).
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import lib as _lib

HEAD_DIM = 128

_lib.register_signatures({
    "mfsdp_attention_fwd": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_longlong,
                            C.c_longlong, C.c_float, C.c_void_p, C.c_void_p],
    "mfsdp_attention_bwd": [C.c_void_p] * 6 + [C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_longlong,
                                               C.c_longlong, C.c_float, C.c_void_p, C.c_void_p],
})


def _has(name: str) -> bool:
    lib = _lib.load()
    if lib is None or _lib.disabled_by_env():
        return False
    return hasattr(lib, name)


def fwd_available() -> bool:
    return _has("mfsdp_attention_fwd")


def bwd_available() -> bool:
    return _has("mfsdp_attention_bwd")


def available() -> bool:
    """Both kernels present (``MFSDP_ATTENTION=sdpa`` selects the library kernel, for A/B timing)."""
    import os

    if os.environ.get("MFSDP_ATTENTION", "native") == "sdpa":
        return False
    return fwd_available() and bwd_available()


def supports(seq: int) -> bool:
    """Sequence lengths the training path hands to these kernels (forward + backward): any positive length;
    partial tiles are masked inside the kernels."""
    return seq > 0


def _check_qkv(qkv: torch.Tensor, batch: int, seq: int, n_heads: int, head_dim: int) -> None:
    if head_dim != HEAD_DIM:
        raise ValueError(f"attention kernels are built for head_dim {HEAD_DIM}, got {head_dim}")
    if qkv.dtype != torch.bfloat16 or qkv.dim() != 2 or qkv.stride(1) != 1:
        raise ValueError("qkv must be a row-major bf16 matrix [batch*seq, 3*n_heads*head_dim]")
    if qkv.shape != (batch * seq, 3 * n_heads * head_dim):
        raise ValueError(f"qkv shape {tuple(qkv.shape)} does not match batch/seq/heads")
    if qkv.data_ptr() % 16 or qkv.stride(0) % 8:
        raise ValueError("qkv must be 16-byte aligned with a row stride that is a multiple of 8 elements")


def attention_fwd(qkv: torch.Tensor, batch: int, seq: int, n_heads: int, head_dim: int,
                  softmax_scale: float | None = None):
    """Causal attention over the fused projection buffer; returns ``(out [T, H] bf16, lse [B, nH, S] fp32)``."""
    from . import kernels as K

    _check_qkv(qkv, batch, seq, n_heads, head_dim)
    scale = 1.0 / math.sqrt(head_dim) if softmax_scale is None else float(softmax_scale)
    out = torch.empty(batch * seq, n_heads * head_dim, dtype=torch.bfloat16, device=qkv.device)
    lse = torch.empty(batch, n_heads, seq, dtype=torch.float32, device=qkv.device)
    status = K.status_word(qkv.device)
    lib = _lib.load()
    _lib.check(lib.mfsdp_attention_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), batch, seq, n_heads,
                                       qkv.stride(0), out.stride(0), scale, status.data_ptr(),
                                       torch.cuda.current_stream(qkv.device).cuda_stream),
               "mfsdp_attention_fwd")
    return out, lse


def attention_bwd(dout: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, lse: torch.Tensor, batch: int, seq: int,
                  n_heads: int, head_dim: int, softmax_scale: float | None = None) -> torch.Tensor:
    """Gradient of :func:`attention_fwd` with respect to ``qkv``; returns ``dqkv [T, 3H]`` bf16."""
    from . import kernels as K

    _check_qkv(qkv, batch, seq, n_heads, head_dim)
    if not supports(seq):
        raise ValueError(f"attention backward needs a positive sequence length, got {seq}")
    scale = 1.0 / math.sqrt(head_dim) if softmax_scale is None else float(softmax_scale)
    dout = dout.contiguous()
    out = out if out.stride(0) == dout.stride(0) else out.contiguous()
    dqkv = torch.empty_like(qkv, memory_format=torch.contiguous_format)
    scratch = torch.empty(2 * batch * n_heads * seq, dtype=torch.float32, device=qkv.device)
    status = K.status_word(qkv.device)
    lib = _lib.load()
    _lib.check(lib.mfsdp_attention_bwd(dout.data_ptr(), qkv.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                       dqkv.data_ptr(), scratch.data_ptr(), batch, seq, n_heads, qkv.stride(0), dout.stride(0),
                                       dqkv.stride(0), scale, status.data_ptr(),
                                       torch.cuda.current_stream(qkv.device).cuda_stream),
               "mfsdp_attention_bwd")
    return dqkv
