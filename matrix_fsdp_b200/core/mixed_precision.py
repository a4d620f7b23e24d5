"""Validation and casting helpers for ``MixedPrecisionPolicy`` / ``OffloadPolicy``.

Parity: ``matrix_fsdp/core/mixed_precision.py:11-99``.
"""
from __future__ import annotations

from typing import Any

import torch
from torch.distributed.fsdp import CPUOffloadPolicy, MixedPrecisionPolicy, OffloadPolicy


def _dtype_name(dtype: torch.dtype | None) -> str | None:
    return None if dtype is None else str(dtype).replace("torch.", "")


def mixed_precision_policy_metadata(policy: MixedPrecisionPolicy | None) -> dict[str, object]:
    policy = policy or MixedPrecisionPolicy()
    return {
        "param_dtype": _dtype_name(policy.param_dtype),
        "reduce_dtype": _dtype_name(policy.reduce_dtype),
        "output_dtype": _dtype_name(policy.output_dtype),
        "cast_forward_inputs": bool(policy.cast_forward_inputs),
    }


def offload_policy_metadata(policy: OffloadPolicy | None) -> dict[str, object]:
    if isinstance(policy, CPUOffloadPolicy):
        return {"kind": "cpu", "pin_memory": bool(policy.pin_memory)}
    return {"kind": "none"}


def validate_mixed_precision_policy(policy: MixedPrecisionPolicy) -> None:
    if not isinstance(policy, MixedPrecisionPolicy):
        raise TypeError(f"mp_policy must be a MixedPrecisionPolicy, got {type(policy).__name__}.")
    for name in ("param_dtype", "reduce_dtype", "output_dtype"):
        dt = getattr(policy, name)
        if dt is not None and not (isinstance(dt, torch.dtype) and dt.is_floating_point):
            raise ValueError(f"mp_policy.{name} must be a floating point dtype or None, got {dt}.")


def validate_offload_policy(policy: OffloadPolicy) -> None:
    if not isinstance(policy, OffloadPolicy):
        raise TypeError(f"offload_policy must be an OffloadPolicy, got {type(policy).__name__}.")


def validate_offload_policy_for_device(policy: OffloadPolicy, device: torch.device) -> None:
    if isinstance(policy, CPUOffloadPolicy) and device.type != "cpu":
        raise NotImplementedError(
            "CPUOffloadPolicy is only supported for CPU-resident models; move the model to CPU or drop the policy.")


def cast_managed_parameter_dtype(tensor: torch.Tensor, dtype: torch.dtype | None) -> torch.Tensor:
    if dtype is None or tensor.dtype == dtype or not tensor.is_floating_point():
        return tensor
    return tensor.to(dtype)


def cast_floating_tensors(value: Any, dtype: torch.dtype | None) -> Any:
    """Recursively cast floating tensors inside tuples / lists / dicts."""
    if dtype is None:
        return value
    if isinstance(value, torch.Tensor):
        return value.to(dtype) if value.is_floating_point() and value.dtype != dtype else value
    if isinstance(value, tuple):
        items = [cast_floating_tensors(v, dtype) for v in value]
        return type(value)(*items) if hasattr(value, "_fields") else tuple(items)
    if isinstance(value, list):
        return [cast_floating_tensors(v, dtype) for v in value]
    if isinstance(value, dict):
        return {k: cast_floating_tensors(v, dtype) for k, v in value.items()}
    return value
