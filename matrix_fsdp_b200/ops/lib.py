"""ctypes binding of ``libmfsdp_kernels.so`` (the sm_100a kernel library).

Launchers take raw device pointers plus the CUDA stream handle, so the same symbols are
callable from Python, from C and from a process that never imports torch.  On a machine
with a GPU the library must be present: ops fail loudly instead of falling back.

Counterpart of the reference's lazy extension loader (``matrix_fsdp/kernels/native.py:17-115``, pybind module
``matrix_fsdp._matrix_fsdp_cuda``); ``MFSDP_DISABLE_NATIVE_KERNELS`` plays the role of
``MATRIX_FSDP_DISABLE_NATIVE_KERNELS`` there.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB = None
_LIB_ERR: Exception | None = None

vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float

_SIGNATURES: dict[str, list] = {
    "mfsdp_gemm_bf16": [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i32, i32, f32, f32,
                        i32, vp, vp, i32, i64, vp, i32, i32, vp],
    "mfsdp_gemm_bf16_sym": [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i32, i32, f32, f32,
                            i32, vp, vp, i32, i64, vp, i32, i32, vp],
    "mfsdp_mirror_upper": [vp, i32, i64, i32, vp],
    "mfsdp_gemm_bf16_ag": [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, f32, f32, vp, vp, vp, vp, i32, vp, vp, vp, i32,
                           i32, C.c_ulonglong, vp, i32, vp],
    "mfsdp_rmsnorm_fwd": [vp, vp, vp, vp, i64, i32, f32, vp],
    "mfsdp_rmsnorm_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, i32, i64, i32, vp],
    "mfsdp_rope": [vp, vp, vp, i64, i32, i32, i32, i32, i32, f32, vp],
    "mfsdp_swiglu_fwd": [vp, vp, i64, i32, vp],
    "mfsdp_swiglu_bwd": [vp, vp, vp, i64, i32, vp],
    "mfsdp_embedding_bwd": [vp, i64, vp, vp, i64, i32, i32, i32, i32, vp, vp],
    "mfsdp_cross_entropy": [vp, vp, vp, i64, i32, i64, f32, i64, vp],
    "mfsdp_cross_entropy_dev_scale": [vp, vp, vp, i64, i32, i64, vp, i64, vp],
    "mfsdp_adamw_flat": [vp, vp, vp, vp, i32, vp, i64, f32, f32, f32, f32, f32, i64, f32, vp],
    "mfsdp_sgd_flat": [vp, vp, vp, i32, vp, i64, f32, f32, f32, f32, i32, vp],
    "mfsdp_muon_momentum": [vp, vp, i32, vp, vp, i64, f32, f32, i32, vp],
    "mfsdp_muon_normalize": [vp, vp, i64, f32, vp],
    "mfsdp_muon_apply": [vp, vp, vp, i32, i32, i32, f32, f32, f32, vp],
    "mfsdp_copy_segments": [vp, vp, vp, vp, vp, i32, i64, i32, vp],
    "mfsdp_cast_f32_bf16": [vp, vp, i64, vp],
}


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "libmfsdp_kernels.so"


def register_signatures(sigs: dict[str, list]) -> None:
    """Let sibling modules (attention, comm) declare their launchers before first load."""
    _SIGNATURES.update(sigs)
    if _LIB is not None:
        _bind(_LIB, sigs)


def _bind(lib, sigs) -> None:
    for name, args in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = args
        fn.restype = C.c_int


def load(required: bool = False):
    """Return the loaded library or ``None`` (raise when ``required``)."""
    global _LIB, _LIB_ERR
    if _LIB is not None:
        return _LIB
    if _LIB_ERR is None:
        path = lib_path()
        try:
            if not path.exists():
                raise FileNotFoundError(
                    f"{path} is missing: run `python -m matrix_fsdp_b200.ops.build`")
            lib = C.CDLL(str(path))
            _bind(lib, _SIGNATURES)
            _LIB = lib
            return _LIB
        except Exception as exc:  # noqa: BLE001 - reported below
            _LIB_ERR = exc
    if required:
        raise RuntimeError(f"sm_100a kernel library unavailable: {_LIB_ERR}")
    return None


def available() -> bool:
    return load() is not None


# kernels launched per launcher call (default 1); the counter feeds the benchmark's launch report
_KERNELS_PER_CALL = {"rmsnorm_bwd": 2, "mfsdp_attention_bwd": 3}
_LAUNCH_COUNT = [0]


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
    _LAUNCH_COUNT[0] += _KERNELS_PER_CALL.get(what, 1)


def launch_count() -> int:
    """Number of kernels of this library launched so far in this process."""
    return _LAUNCH_COUNT[0]


def disabled_by_env() -> bool:
    return os.environ.get("MFSDP_DISABLE_NATIVE_KERNELS", "0") not in ("", "0", "false", "False")
