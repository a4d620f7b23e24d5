"""Mixture-of-experts decoder (softmax top-k router with load-balance loss, SwiGLU experts).

Dense parameters (attention, norms, router, embeddings, LM head) are sharded by ``fully_shard``; the
experts are expert-parallel: every rank of the EP group owns ``n_experts / ep_size`` experts whole and
they are passed to ``fully_shard`` as ``ignored_params``, which is how the reference composes FSDP with
an upper-stack EP owner (test/fsdp/test_deepseek_v3_ep_train.py:566-640, docs/introduction.md:238-271).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from ..ops import functional as OF
from ..ops import moe_functional as MF
from .llama import LMHead, Matrix, RMSNorm, TokenEmbedding


@dataclass
class MoEConfig:
    vocab_size: int = 32000
    hidden: int = 2048
    n_layers: int = 16
    n_heads: int = 16
    head_dim: int = 128
    n_experts: int = 64
    expert_ffn: int = 1408
    top_k: int = 6
    aux_loss_coef: float = 0.01
    rope_theta: float = 10000.0
    eps: float = 1e-5
    init_std: float = 0.02
    capacity_factor: float = 0.0          # <= 0: receive buffers sized for the worst case, no row is ever dropped
    max_seq_len: int = 4096
    seed: int = 0
    loss_ignore_index: int | None = None

    @staticmethod
    def config5() -> "MoEConfig":
        return MoEConfig()

    @staticmethod
    def tiny(**kw) -> "MoEConfig":
        base = dict(vocab_size=512, hidden=256, n_layers=2, n_heads=2, head_dim=128, n_experts=8, expert_ffn=128,
                    top_k=2, max_seq_len=256)
        base.update(kw)
        return MoEConfig(**base)


class Experts(nn.Module):
    """This rank's experts: ``w_gate_up`` [El, 2F, H] (gate rows then up rows) and ``w_down`` [El, H, F].

    Expert ``e`` is initialised from a generator seeded by (seed, layer, e), so the weights do not
    depend on how many ranks share the experts.
    """

    is_expert_parallel = True

    def __init__(self, cfg: MoEConfig, layer: int, first_expert: int, n_local: int, device=None, dtype=None) -> None:
        super().__init__()
        h, f = cfg.hidden, cfg.expert_ffn
        self.first_expert, self.n_local = first_expert, n_local
        gen_dev = torch.device(device) if device is not None and torch.device(device).type == "cuda" else torch.device("cpu")
        dt = dtype or torch.float32
        gu = torch.empty(n_local, 2 * f, h, dtype=dt, device=gen_dev)
        dn = torch.empty(n_local, h, f, dtype=dt, device=gen_dev)
        g = torch.Generator(device=gen_dev)
        for el in range(n_local):
            g.manual_seed(cfg.seed * 1_000_003 + layer * 4099 + first_expert + el + 17)
            gu[el].copy_(torch.empty(2 * f, h, dtype=torch.float32, device=gen_dev).normal_(0.0, cfg.init_std, generator=g))
            dn[el].copy_(torch.empty(h, f, dtype=torch.float32, device=gen_dev).normal_(0.0, cfg.init_std, generator=g))
        self.w_gate_up = nn.Parameter(gu.to(device=device))
        self.w_down = nn.Parameter(dn.to(device=device))


class MoEBlock(nn.Module):
    def __init__(self, cfg: MoEConfig, layer: int, ep_group=None, device=None, dtype=None) -> None:
        super().__init__()
        self.cfg, self.layer, self.ep_group = cfg, layer, ep_group
        h, std = cfg.hidden, cfg.init_std
        assert cfg.n_heads * cfg.head_dim == h
        self.attn_norm = RMSNorm(h, cfg.eps)
        self.wq = Matrix(h, h, std)
        self.wk = Matrix(h, h, std)
        self.wv = Matrix(h, h, std)
        self.wo = Matrix(h, h, std)
        self.mlp_norm = RMSNorm(h, cfg.eps)
        self.router = Matrix(h, cfg.n_experts, std)
        self.router.is_router = True
        world = dist.get_world_size(ep_group) if (dist.is_initialized() and ep_group is not False) else 1
        rank = dist.get_rank(ep_group) if world > 1 else 0
        if cfg.n_experts % world:
            raise ValueError(f"{cfg.n_experts} experts do not divide over {world} ranks")
        n_local = cfg.n_experts // world
        self.ep_world, self.ep_rank = world, rank
        self.experts = Experts(cfg, layer, rank * n_local, n_local, device=device, dtype=dtype)
        self.last_aux: torch.Tensor | None = None

    def _shape(self, batch: int, seq: int) -> OF.BlockShape:
        c = self.cfg
        return OF.BlockShape(batch, seq, c.hidden, c.n_heads, c.head_dim, c.expert_ffn, c.eps, c.rope_theta)

    def _group(self):
        if self.ep_world <= 1:
            return None
        return self.ep_group if self.ep_group is not None else dist.group.WORLD

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, s, h = x.shape
        c = self.cfg
        cos, sin = OF.rope_tables(max(s, 1), c.head_dim, c.rope_theta, x.device)
        native = (OF.use_native(x) and self.wq.weight.dtype == torch.bfloat16 and c.head_dim == 128
                  and self.experts.w_gate_up.dtype == torch.bfloat16 and h % 128 == 0 and c.expert_ffn % 64 == 0)
        if native:
            from ..parallel.expert_parallel import ExpertParallelContext

            x2 = x.reshape(b * s, h)
            x1 = MF.attention_half(x2, self, self._shape(b, s), cos, sin)
            xn = OF.rms_norm(x1, self.mlp_norm.weight, c.eps)
            ep = ExpertParallelContext.get(self._group(), x.device, h, c.n_experts, c.top_k, b * s, c.capacity_factor)
            y, aux = MF.moe_ffn(xn, x1, self.router.weight, self.experts.w_gate_up, self.experts.w_down, ep, c.top_k,
                                c.aux_loss_coef, router_param=self.router.weight)
            self.last_aux = aux
            return y.view(b, s, h)
        xn = self.attn_norm(x)
        q = F.linear(xn, self.wq.weight).view(b, s, c.n_heads, c.head_dim)
        k = F.linear(xn, self.wk.weight).view(b, s, c.n_heads, c.head_dim)
        v = F.linear(xn, self.wv.weight).view(b, s, c.n_heads, c.head_dim)
        q, k = OF.apply_rope_reference(q, cos, sin), OF.apply_rope_reference(k, cos, sin)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x1 = x + F.linear(o.transpose(1, 2).reshape(b, s, h), self.wo.weight)
        xn = self.mlp_norm(x1).reshape(b * s, h)
        y, aux = MF.moe_ffn_reference(xn, x1.reshape(b * s, h), self.router.weight, self.experts.w_gate_up,
                                      self.experts.w_down, c.top_k, c.aux_loss_coef, group=self._group())
        self.last_aux = aux
        return y.view(b, s, h)


class MoEModel(nn.Module):
    """Decoder-only MoE LM; ``forward(tokens, targets)`` returns mean CE + the layers' balance losses."""

    def __init__(self, cfg: MoEConfig, ep_group=None, device=None, dtype=None) -> None:
        super().__init__()
        self.cfg = cfg
        self.embed = TokenEmbedding(cfg.vocab_size, cfg.hidden)
        nn.init.normal_(self.embed.weight, mean=0.0, std=cfg.init_std)
        self.layers = nn.ModuleList([MoEBlock(cfg, i, ep_group, device=device, dtype=dtype) for i in range(cfg.n_layers)])
        self.head = LMHead(cfg.hidden, cfg.vocab_size, cfg.eps, cfg.init_std)

    @property
    def final_norm(self) -> RMSNorm:
        return self.head.final_norm

    @property
    def lm_head(self) -> Matrix:
        return self.head.lm_head

    def expert_parameters(self) -> list[nn.Parameter]:
        return [p for layer in self.layers for p in layer.experts.parameters()]

    def forward(self, tokens: torch.Tensor, targets: torch.Tensor | None = None) -> torch.Tensor:
        x = self.embed(tokens)
        for layer in self.layers:
            x = layer(x)
        logits = self.head(x)
        if targets is None:
            return logits
        n_valid = targets.numel() if self.cfg.loss_ignore_index is None else None
        ignore = -100 if self.cfg.loss_ignore_index is None else self.cfg.loss_ignore_index
        loss = OF.fused_cross_entropy(logits, targets, ignore_index=ignore, n_valid=n_valid)
        for layer in self.layers:
            if layer.last_aux is not None:
                loss = loss + layer.last_aux.to(loss.dtype)
        return loss

    def active_params_per_token(self) -> int:
        c = self.cfg
        per_layer = 4 * c.hidden * c.hidden + c.hidden * c.n_experts + c.top_k * 3 * c.hidden * c.expert_ffn
        return c.n_layers * per_layer + c.hidden * c.vocab_size

    def flops_per_token(self, seq_len: int) -> float:
        c = self.cfg
        attn = 2 * 2 * seq_len * c.hidden * 0.5
        return 3.0 * (2 * self.active_params_per_token() + c.n_layers * attn)


def shard_moe(model: MoEModel, *, mesh=None, dp_mesh_dims=None, mp_policy=None, optimizer_policy=None,
              reshard_after_forward=None) -> MoEModel:
    """``fully_shard`` the dense parameters of every block (experts ignored), then embedding and head."""
    from torch.distributed.fsdp import MixedPrecisionPolicy

    from ..api import fully_shard

    mp = mp_policy or MixedPrecisionPolicy()
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, dp_mesh_dims=dp_mesh_dims, mp_policy=mp, optimizer_policy=optimizer_policy,
                    reshard_after_forward=reshard_after_forward, ignored_params=set(layer.experts.parameters()))
    # embedding and head (final norm + LM head) are units of their own, like the dense model's
    for part in (model.embed, model.head):
        fully_shard(part, mesh=mesh, dp_mesh_dims=dp_mesh_dims, mp_policy=mp, optimizer_policy=optimizer_policy,
                    reshard_after_forward=reshard_after_forward)
    from .llama import _attach_model_no_sync

    _attach_model_no_sync(model)
    return model


def configure_moe_optimizer(model: MoEModel, optimizer: str = "mixed_muon_adamw", *, lr: float = 3e-4,
                            muon_lr: float = 0.02, weight_decay: float = 0.0, **kw):
    """Dense parameters: ``configure_optimizer``; experts: the same kind of optimizer (Muon, AdamW or SGD) on the
    owning rank."""
    from ..optim.expert import CombinedOptimizer, ExpertParallelOptimizer
    from ..optim.wrapper import configure_optimizer

    mixed = optimizer in ("mixed_muon_adamw", "muon_adamw", "mixed", "muon")
    if mixed:
        dense = configure_optimizer(model, optimizer, lr=lr, muon_lr=muon_lr, weight_decay=weight_decay, **kw)
        experts = ExpertParallelOptimizer(model.expert_parameters(), "muon", lr=muon_lr, weight_decay=weight_decay,
                                          momentum=kw.get("muon_momentum", 0.95), ns_steps=kw.get("muon_ns_steps", 5),
                                          adjust_lr_fn=kw.get("muon_adjust_lr_fn"))
    elif optimizer == "sgd":
        dense = configure_optimizer(model, optimizer, lr=lr, weight_decay=weight_decay, **kw)
        experts = ExpertParallelOptimizer(model.expert_parameters(), "sgd", lr=lr, weight_decay=weight_decay,
                                          sgd_momentum=kw.get("momentum", 0.0))
    else:
        dense = configure_optimizer(model, optimizer, lr=lr, weight_decay=weight_decay, **kw)
        experts = ExpertParallelOptimizer(model.expert_parameters(), "adamw", lr=lr, weight_decay=weight_decay,
                                          betas=kw.get("betas", (0.9, 0.999)), eps=kw.get("eps", 1e-8))
    return CombinedOptimizer(dense, experts)


def clip_moe_grad_norm_(model: MoEModel, max_norm: float, norm_type: float = 2.0, *, expert_scale: float = 1.0,
                        error_if_nonfinite: bool = False) -> torch.Tensor:
    """Clip the global gradient norm of an MoE model: the sharded dense gradients plus the expert gradients, of
    which every rank of the expert-parallel group holds its own experts'.  ``expert_scale`` is the factor the
    expert optimizer applies to its gradients (``1 / world`` when they are to be means over the ranks' tokens; the
    expert backward leaves sums).  Returns the norm before clipping; call it between ``backward()`` and ``step()``."""
    from ..utils.training import clip_grad_norm_

    group = model.layers[0]._group() if len(model.layers) else None
    return clip_grad_norm_(model, max_norm, norm_type, error_if_nonfinite,
                           extra_grads=[p.grad for p in model.expert_parameters()], extra_group=group,
                           extra_scale=expert_scale)


def save_moe_checkpoint(model: MoEModel, directory: str, optimizer=None) -> None:
    """Dense parameters (and their optimizer state) through ``save_matrix_dcp``; every EP rank adds one file
    with the experts it owns (weights, fp32 masters and optimizer state), keyed by global expert id."""
    import os

    from ..checkpoint import save_matrix_dcp

    dense_opt = getattr(optimizer, "dense", optimizer)
    save_matrix_dcp(model, directory, optimizer=dense_opt)
    rank = dist.get_rank() if dist.is_initialized() else 0
    payload = {"experts": {}, "optimizer": None}
    for li, layer in enumerate(model.layers):
        ex = layer.experts
        payload["experts"][li] = {"first_expert": ex.first_expert, "w_gate_up": ex.w_gate_up.detach().cpu(),
                                  "w_down": ex.w_down.detach().cpu()}
    expert_opt = getattr(optimizer, "experts", None)
    if expert_opt is not None:
        payload["optimizer"] = _to_cpu(expert_opt.state_dict())
    torch.save(payload, os.path.join(directory, f"experts_rank{rank}.pt"))
    if dist.is_initialized():
        dist.barrier()


def load_moe_checkpoint(model: MoEModel, directory: str, optimizer=None, allow_reshard: bool = False) -> None:
    """Inverse of :func:`save_moe_checkpoint`.  With ``allow_reshard`` the expert-parallel size may differ from the
    one that wrote the files: experts are addressed by their global id, every rank reads the files that hold the
    experts it owns now and cuts their rows (weights, masters and optimizer state) out of them."""
    import glob
    import os

    from ..checkpoint import load_matrix_dcp

    dense_opt = getattr(optimizer, "dense", optimizer)
    load_matrix_dcp(model, directory, optimizer=dense_opt, allow_reshard=allow_reshard)
    rank = dist.get_rank() if dist.is_initialized() else 0
    expert_opt = getattr(optimizer, "experts", None)
    mine = os.path.join(directory, f"experts_rank{rank}.pt")
    payload = torch.load(mine, map_location="cpu", weights_only=False) if os.path.exists(mine) else None
    same = payload is not None and all(
        payload["experts"][li]["first_expert"] == layer.experts.first_expert
        and payload["experts"][li]["w_down"].shape == layer.experts.w_down.shape
        for li, layer in enumerate(model.layers))
    if same:
        for li, layer in enumerate(model.layers):
            rec, ex = payload["experts"][li], layer.experts
            with torch.no_grad():
                ex.w_gate_up.copy_(rec["w_gate_up"])
                ex.w_down.copy_(rec["w_down"])
        if expert_opt is not None and payload.get("optimizer") is not None:
            expert_opt.load_state_dict(payload["optimizer"])
        return
    if not allow_reshard:
        raise ValueError("expert checkpoint was written with a different expert-parallel layout")
    files = sorted(glob.glob(os.path.join(directory, "experts_rank*.pt")))
    sources = [torch.load(f, map_location="cpu", weights_only=False) for f in files]
    for li, layer in enumerate(model.layers):
        ex = layer.experts
        with torch.no_grad():
            for name in ("w_gate_up", "w_down"):
                rows = _expert_rows([(src["experts"][li]["first_expert"], src["experts"][li][name]) for src in sources],
                                    ex.first_expert, ex.n_local)
                getattr(ex, name).copy_(rows)
    if expert_opt is not None and all(src.get("optimizer") is not None for src in sources):
        # optimizer entries are per expert parameter, in ``model.expert_parameters()`` order: two per layer
        firsts = [[src["experts"][li]["first_expert"] for li in range(len(model.layers)) for _ in range(2)]
                  for src in sources]
        my = [(layer.experts.first_expert, layer.experts.n_local) for layer in model.layers for _ in range(2)]
        expert_opt.load_state_dict(_reshard_expert_optimizer_state([s["optimizer"] for s in sources], firsts, my))


def _expert_rows(sources, first: int, count: int):
    """Rows ``[first, first + count)`` by global expert id out of ``[(first id, tensor or list), ...]``."""
    picked = []
    for e in range(first, first + count):
        for src_first, rows in sources:
            if src_first <= e < src_first + len(rows):
                picked.append(rows[e - src_first])
                break
        else:
            raise ValueError(f"no checkpoint file holds expert {e}")
    return picked if not isinstance(picked[0], torch.Tensor) else torch.stack(picked)


def _reshard_expert_optimizer_state(states: list, firsts: list, mine: list) -> dict:
    """One expert-optimizer state dict for the experts this rank owns, cut from the writers' state dicts."""
    kinds = {s["kind"] for s in states}
    if len(kinds) != 1:
        raise ValueError(f"expert optimizer kinds differ between files: {sorted(kinds)}")
    out = {"kind": states[0]["kind"], "step": max(int(s["step"]) for s in states)}
    per_param = {"masters": True, "exp_avg": True, "exp_avg_sq": True, "momentum_buffer": True, "momentum": True}
    for key in states[0]:
        if key not in per_param:
            continue
        if any(len(s[key]) == 0 for s in states):            # SGD without momentum keeps an empty list
            out[key] = []
            continue
        out[key] = []
        for i, (first, count) in enumerate(mine):
            rows = _expert_rows([(firsts[k][i], s[key][i]) for k, s in enumerate(states)], first, count)
            out[key].append(rows)
    return out


def _to_cpu(obj):
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj
