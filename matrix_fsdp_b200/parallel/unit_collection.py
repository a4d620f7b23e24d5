"""Find the FSDP units attached to a module tree.

Parity: ``matrix_fsdp/runtime/unit_collection.py:1-45``.
"""
from __future__ import annotations

from collections.abc import Iterable

from torch import nn


def collect_param_groups(module_or_units) -> list:
    """Units under ``module_or_units`` (a module, a unit, or an iterable of either), in id order."""
    from .fsdp_unit import MatrixFSDPParamGroup

    found: dict[int, MatrixFSDPParamGroup] = {}

    def visit(obj) -> None:
        if isinstance(obj, MatrixFSDPParamGroup):
            found[id(obj)] = obj
        elif isinstance(obj, nn.Module):
            for m in obj.modules():
                u = getattr(m, "_matrix_fsdp_param_group", None)
                if isinstance(u, MatrixFSDPParamGroup):     # another package may use the same attribute name
                    found[id(u)] = u
        elif isinstance(obj, Iterable):
            for item in obj:
                visit(item)
        else:
            raise TypeError(f"Cannot collect FSDP units from {type(obj).__name__}.")

    visit(module_or_units)
    return sorted(found.values(), key=lambda u: u.metadata.runtime_param_group_id)
