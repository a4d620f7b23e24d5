"""Wrap policies: predicates that select which sub-modules become FSDP units.

Parity: ``matrix_fsdp/policy/wrap.py:1-68``.
"""
from __future__ import annotations

from collections.abc import Callable, Iterable

from torch import nn

WrapPolicy = Callable[[nn.Module], bool]


def module_type_policy(module_types: type | Iterable[type]) -> WrapPolicy:
    types = (module_types,) if isinstance(module_types, type) else tuple(module_types)
    if not types:
        raise ValueError("module_type_policy needs at least one module type.")
    return lambda m: isinstance(m, types)


def size_based_policy(min_num_params: int, *, recurse: bool = True) -> WrapPolicy:
    if min_num_params < 0:
        raise ValueError("min_num_params must be non-negative.")
    return lambda m: sum(p.numel() for p in m.parameters(recurse=recurse)) >= min_num_params


def or_policy(*policies: WrapPolicy) -> WrapPolicy:
    return lambda m: any(p(m) for p in policies)


def and_policy(*policies: WrapPolicy) -> WrapPolicy:
    return lambda m: all(p(m) for p in policies)


def not_policy(policy: WrapPolicy) -> WrapPolicy:
    return lambda m: not policy(m)
