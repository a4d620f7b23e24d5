"""Alias module kept for import compatibility (``matrix_fsdp/runtime/param_group.py:1-6``)."""
from .fsdp_unit import FSDPLifecycleState, FSDPRuntimeState, MatrixFSDPNoSync, MatrixFSDPParamGroup  # noqa: F401
