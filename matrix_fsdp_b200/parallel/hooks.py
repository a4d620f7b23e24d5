"""Autograd hook helpers: fire a pre-backward callback once however many outputs a module has.

Parity: ``matrix_fsdp/runtime/hooks.py:1-76``.
"""
from __future__ import annotations

from collections.abc import Callable, Mapping
from typing import Any

import torch


class ForwardBackwardContext:
    """One forward invocation of a unit; ``pre_backward`` runs at most once per backward pass."""

    def __init__(self, callback: Callable[[], None]) -> None:
        self._callback = callback
        self.fired = False
        self.num_hooks = 0

    def pre_backward(self, grad: torch.Tensor | None = None):
        if not self.fired:
            self.fired = True
            self._callback()
        return grad

    def reset(self) -> None:
        self.fired = False


def iter_tensors(value: Any):
    if isinstance(value, torch.Tensor):
        yield value
    elif isinstance(value, Mapping):
        for v in value.values():
            yield from iter_tensors(v)
    elif isinstance(value, (tuple, list)):
        for v in value:
            yield from iter_tensors(v)
    elif hasattr(value, "__dataclass_fields__"):
        for name in value.__dataclass_fields__:
            yield from iter_tensors(getattr(value, name))


def register_pre_backward_hooks(outputs: Any, ctx: ForwardBackwardContext) -> int:
    """Attach ``ctx.pre_backward`` to every output tensor that takes part in autograd."""
    n = 0
    for t in iter_tensors(outputs):
        if t.requires_grad:
            t.register_hook(ctx.pre_backward)
            n += 1
    ctx.num_hooks += n
    return n
