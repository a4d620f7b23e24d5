"""Default per-parameter shard hints derived from module structure.

Rules are tried in priority order and the first match wins: MoE expert owner → router/gate →
LM head (vocabulary projection) → linear weight (Muon, whole-matrix owner) → embedding →
norms → bias → anything ≤1-D.

Parity: ``matrix_fsdp/planning/shard_hint.py:20-185``.  Added rule: an output projection onto
the vocabulary (module named ``lm_head``/``output``/``unembed`` or carrying
``is_lm_head = True``) is AdamW + whole-parameter instead of Muon, which the reference's
defaults would otherwise assign to any ``nn.Linear`` weight.
"""
from __future__ import annotations

from collections.abc import Callable, Mapping, Sequence
from dataclasses import dataclass

from torch import nn

from ..core.managed_param import ParamRuntimeKind, ParamShardHint

ShardHintRuleFn = Callable[[str, nn.Module, str, nn.Parameter], "ParamShardHint | None"]


@dataclass(frozen=True)
class ShardHintRule:
    name: str
    apply: ShardHintRuleFn


def _split_param_fqn(fqn: str) -> tuple[str, str]:
    return tuple(fqn.rsplit(".", 1)) if "." in fqn else ("", fqn)  # type: ignore[return-value]


def _parse_expert_fqn(fqn: str, *, expert_module_names: Sequence[str]) -> tuple[int, str] | None:
    parts = fqn.split(".")
    for i, part in enumerate(parts[:-2]):
        if part in expert_module_names and parts[i + 1].isdigit():
            return int(parts[i + 1]), ".".join(parts[: i + 2])
    return None


def _is_linear_like(module: nn.Module) -> bool:
    return isinstance(module, nn.Linear) or bool(getattr(module, "is_linear_like", False))


def _is_norm_like(module: nn.Module) -> bool:
    norm_types = (nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d, nn.GroupNorm, nn.InstanceNorm1d,
                  nn.InstanceNorm2d, nn.InstanceNorm3d, nn.LayerNorm)
    rms = getattr(nn, "RMSNorm", None)
    if rms is not None:
        norm_types = norm_types + (rms,)
    return isinstance(module, norm_types) or bool(getattr(module, "is_norm_like", False))


def moe_expert_owner_rule(*, expert_module_names: Sequence[str] = ("experts",)) -> ShardHintRule:
    names = tuple(expert_module_names)

    def apply(fqn, owning_module, local_name, param):
        meta = _parse_expert_fqn(fqn, expert_module_names=names)
        if meta is None:
            return None
        expert_id, group_id = meta
        two_d = param.ndim == 2
        return ParamShardHint(optimizer_type="muon" if two_d else "adamw",
                              split_granularity="matrix_owner" if two_d else "parameter",
                              runtime_kind=ParamRuntimeKind.EXPERT_OWNER, parallel_role="routed_expert",
                              expert_id=expert_id, expert_group_id=group_id)

    return ShardHintRule("moe_expert_owner", apply)


def router_rule(*, module_names: Sequence[str] = ("gate", "router")) -> ShardHintRule:
    names = tuple(module_names)

    def apply(fqn, owning_module, local_name, param):
        if any(part in names for part in _split_param_fqn(fqn)[0].split(".")):
            return ParamShardHint(optimizer_type="adamw", split_granularity="parameter",
                                  runtime_kind=ParamRuntimeKind.FSDP_GATHER, parallel_role="router")
        return None

    return ShardHintRule("router", apply)


def lm_head_rule(*, module_names: Sequence[str] = ("lm_head", "output", "unembed")) -> ShardHintRule:
    names = tuple(module_names)

    def apply(fqn, owning_module, local_name, param):
        last = _split_param_fqn(fqn)[0].split(".")[-1]
        if getattr(owning_module, "is_lm_head", False) or (_is_linear_like(owning_module) and last in names):
            return ParamShardHint(optimizer_type="adamw", split_granularity="parameter", parallel_role="embedding")
        return None

    return ShardHintRule("lm_head", apply)


def muon_linear_weight_rule() -> ShardHintRule:
    def apply(fqn, owning_module, local_name, param):
        if _is_linear_like(owning_module) and local_name == "weight" and param.ndim == 2:
            return ParamShardHint(optimizer_type="muon", split_granularity="matrix_owner")
        return None

    return ShardHintRule("muon_linear_weight", apply)


def no_split_embedding_rule() -> ShardHintRule:
    def apply(fqn, owning_module, local_name, param):
        if isinstance(owning_module, nn.Embedding) and local_name == "weight":
            return ParamShardHint(optimizer_type="adamw", split_granularity="parameter")
        return None

    return ShardHintRule("no_split_embedding", apply)


def no_split_norm_rule() -> ShardHintRule:
    def apply(fqn, owning_module, local_name, param):
        if _is_norm_like(owning_module):
            return ParamShardHint(optimizer_type="adamw", split_granularity="parameter")
        return None

    return ShardHintRule("no_split_norm", apply)


def no_split_bias_rule() -> ShardHintRule:
    def apply(fqn, owning_module, local_name, param):
        if local_name == "bias":
            return ParamShardHint(optimizer_type="adamw", split_granularity="parameter")
        return None

    return ShardHintRule("no_split_bias", apply)


def no_split_1d_rule() -> ShardHintRule:
    def apply(fqn, owning_module, local_name, param):
        if param.ndim <= 1:
            return ParamShardHint(optimizer_type="adamw", split_granularity="parameter")
        return None

    return ShardHintRule("no_split_1d", apply)


def default_shard_hint_rules() -> tuple[ShardHintRule, ...]:
    return (moe_expert_owner_rule(), router_rule(), lm_head_rule(), muon_linear_weight_rule(),
            no_split_embedding_rule(), no_split_norm_rule(), no_split_bias_rule(), no_split_1d_rule())


def build_shard_hints(module: nn.Module, *, rules: Sequence[ShardHintRule] | None = None,
                      overrides: Mapping[str, ParamShardHint] | None = None) -> dict[str, ParamShardHint]:
    chosen = tuple(rules or default_shard_hint_rules())
    modules = dict(module.named_modules())
    hints: dict[str, ParamShardHint] = {}
    fqns = set()
    for fqn, param in module.named_parameters(recurse=True, remove_duplicate=True):
        fqns.add(fqn)
        mod_fqn, local = _split_param_fqn(fqn)
        owner = modules[mod_fqn]
        for rule in chosen:
            hint = rule.apply(fqn, owner, local, param)
            if hint is not None:
                hints[fqn] = hint
                break
    if overrides:
        unknown = set(overrides) - fqns
        if unknown:
            raise ValueError(f"Shard hint overrides refer to unknown parameters: {', '.join(sorted(unknown))}.")
        hints.update(overrides)
    return hints
