"""Small user-facing training helpers.

``train_step`` is the whole per-step call a user makes: copy the step's token batch from pinned
host memory, forward, backward, optimizer step, and read the loss back to the host.
"""
from __future__ import annotations

import torch


def pin(t: torch.Tensor) -> torch.Tensor:
    return t.pin_memory() if torch.cuda.is_available() and not t.is_pinned() else t


def train_step(model: torch.nn.Module, optimizer, host_tokens: torch.Tensor, host_targets: torch.Tensor,
               device: torch.device | str) -> float:
    """One optimisation step from host data; returns the loss as a Python float (device→host read)."""
    tokens = host_tokens.to(device, non_blocking=True)
    targets = host_targets.to(device, non_blocking=True)
    loss = model(tokens, targets)
    loss.backward()
    optimizer.step()
    optimizer.zero_grad(set_to_none=True)
    return float(loss.item())


def device_train_step(model: torch.nn.Module, optimizer, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Same step with inputs already on the device and the loss left on the device."""
    loss = model(tokens, targets)
    loss.backward()
    optimizer.step()
    optimizer.zero_grad(set_to_none=True)
    return loss.detach()
