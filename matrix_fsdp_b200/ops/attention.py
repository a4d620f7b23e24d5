"""Causal attention kernels (head_dim 128) for sm_100a: Python entry points.

``available()`` reports whether the attention kernels are present in the loaded kernel library;
callers fall back to the library SDPA kernel otherwise.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import lib as _lib

_lib.register_signatures({
    "mfsdp_attention_fwd": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float,
                            C.c_void_p, C.c_void_p],
    "mfsdp_attention_bwd": [C.c_void_p] * 7 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p],
})


def available() -> bool:
    lib = _lib.load()
    if lib is None or _lib.disabled_by_env():
        return False
    return hasattr(lib, "mfsdp_attention_fwd") and hasattr(lib, "mfsdp_attention_bwd")


def attention_fwd(qkv: torch.Tensor, batch: int, seq: int, n_heads: int, head_dim: int):
    raise NotImplementedError


def attention_bwd(dout, qkv, out, lse, batch: int, seq: int, n_heads: int, head_dim: int):
    raise NotImplementedError
