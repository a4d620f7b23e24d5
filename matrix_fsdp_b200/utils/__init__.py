"""User-facing helpers: one-call training steps, sharded gradient clipping, gathered gradients, rank health."""
from .training import (clip_grad_norm_, device_train_step, gather_full_grads, pin, raise_on_device_error, train_step)

__all__ = ["clip_grad_norm_", "device_train_step", "gather_full_grads", "pin", "raise_on_device_error", "train_step"]
