"""User-facing helpers: one-call training steps, sharded gradient clipping, rank health."""
from .training import clip_grad_norm_, device_train_step, pin, train_step

__all__ = ["clip_grad_norm_", "device_train_step", "pin", "train_step"]
