"""Optimizer for expert-parallel parameters (each rank owns its experts whole, no FSDP unit).

Expert weights are bf16 ``[El, rows, cols]`` parameters; this optimizer keeps the fp32 master copy and
the optimizer state, runs Muon (Newton-Schulz on the tcgen05 GEMM, one expert matrix at a time),
AdamW or SGD on the master, and writes the bf16 weights back in the same kernels.  The reference leaves
EP-owned parameters to the caller's own optimizer (``ignored_params``,
test/fsdp/test_deepseek_v3_ep_train.py:600-640).
"""
from __future__ import annotations

import torch
from torch import nn

from .muon import MatrixMuon


class ExpertParallelOptimizer:
    def __init__(self, params, kind: str = "muon", *, lr: float = 0.02, weight_decay: float = 0.0,
                 momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 5, adjust_lr_fn: str | None = None,
                 betas=(0.9, 0.95), eps: float = 1e-8, sgd_momentum: float = 0.0) -> None:
        if kind not in ("muon", "adamw", "sgd"):
            raise ValueError(f"unknown expert optimizer {kind!r}")
        self.kind = kind
        self.params = [p for p in params]
        for p in self.params:
            if p.dim() != 3:
                raise ValueError("expert parameters are [experts, rows, cols]")
        self.defaults = dict(lr=lr, weight_decay=weight_decay, betas=tuple(betas), eps=eps, momentum=sgd_momentum)
        self.param_groups = [dict(params=self.params, **self.defaults)]
        self.masters = [p.detach().float().clone() for p in self.params]
        self.step_count = 0
        self.grad_scale = 1.0
        self._lp: dict[int, torch.Tensor] = {}
        if kind == "muon":
            self._slices: list[list[nn.Parameter]] = []
            flat: list[nn.Parameter] = []
            for p, m in zip(self.params, self.masters):
                row = []
                for e in range(p.shape[0]):
                    s = nn.Parameter(m[e], requires_grad=False)
                    self._lp[id(s)] = p.data[e]
                    row.append(s)
                    flat.append(s)
                self._slices.append(row)
            self.muon = MatrixMuon(flat, lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov,
                                   ns_steps=ns_steps, adjust_lr_fn=adjust_lr_fn,
                                   low_precision_of=lambda s: self._lp[id(s)])
        elif kind == "sgd":
            self.momentum_buffer = [torch.zeros_like(m) for m in self.masters] if sgd_momentum else []
        else:
            self.exp_avg = [torch.zeros_like(m) for m in self.masters]
            self.exp_avg_sq = [torch.zeros_like(m) for m in self.masters]

    @torch.no_grad()
    def step(self) -> None:
        self.step_count += 1
        if self.kind == "muon":
            self.muon.grad_scale = self.grad_scale
            for g in self.muon.param_groups:
                g["lr"] = self.param_groups[0]["lr"]
            for p, row in zip(self.params, self._slices):
                for e, s in enumerate(row):
                    s._grad_override = None if p.grad is None else p.grad[e]
            self.muon.step()
            for row in self._slices:
                for s in row:
                    s._grad_override = None
            return
        g0 = self.param_groups[0]
        if self.kind == "sgd":
            # plain tensor ops on the fp32 masters (no Newton-Schulz, no moments worth a kernel of their own)
            for i, (p, m) in enumerate(zip(self.params, self.masters)):
                if p.grad is None:
                    continue
                g = p.grad.float() * float(self.grad_scale)
                if g0["weight_decay"]:
                    g = g.add(m, alpha=g0["weight_decay"])
                if g0["momentum"]:
                    buf = self.momentum_buffer[i]
                    buf.copy_(g) if self.step_count == 1 else buf.mul_(g0["momentum"]).add_(g)
                    g = buf
                m.add_(g, alpha=-float(g0["lr"]))
                p.data.copy_(m)
            return
        from .flat import _adamw_reference_, _native

        for p, m, a, b in zip(self.params, self.masters, self.exp_avg, self.exp_avg_sq):
            if p.grad is None:
                continue
            kw = dict(lr=float(g0["lr"]), beta1=g0["betas"][0], beta2=g0["betas"][1], eps=g0["eps"],
                      weight_decay=g0["weight_decay"], step=self.step_count, grad_scale=self.grad_scale)
            if _native(p.device) and p.dtype == torch.bfloat16 and p.grad.is_contiguous():
                from ..ops import kernels as K

                K.adamw_flat_(m.view(-1), a.view(-1), b.view(-1), p.grad.view(-1), p_lp=p.data.view(-1), **kw)
            else:
                _adamw_reference_(m.view(-1), a.view(-1), b.view(-1), p.grad.reshape(-1).float(), p_lp=None, **kw)
                p.data.copy_(m)

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    def state_dict(self) -> dict:
        sd = {"kind": self.kind, "step": self.step_count, "masters": self.masters}
        if self.kind == "muon":
            sd["momentum"] = [[self.muon.state[s].get("momentum_buffer") for s in row] for row in self._slices]
        elif self.kind == "sgd":
            sd["momentum_buffer"] = self.momentum_buffer
        else:
            sd["exp_avg"], sd["exp_avg_sq"] = self.exp_avg, self.exp_avg_sq
        return sd

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        for m, src, p in zip(self.masters, sd["masters"], self.params):
            m.copy_(src)
            p.data.copy_(m)
        if self.kind == "muon":
            for row, bufs in zip(self._slices, sd["momentum"]):
                for s, b in zip(row, bufs):
                    if b is not None:
                        self.muon.state[s]["momentum_buffer"] = b.clone()
        elif self.kind == "sgd":
            for dst, src in zip(self.momentum_buffer, sd.get("momentum_buffer", [])):
                dst.copy_(src)
        else:
            for dst, src in zip(self.exp_avg, sd["exp_avg"]):
                dst.copy_(src)
            for dst, src in zip(self.exp_avg_sq, sd["exp_avg_sq"]):
                dst.copy_(src)


class CombinedOptimizer:
    """Steps the optimizer of the FSDP-managed dense parameters and the expert optimizer together."""

    def __init__(self, dense, experts: ExpertParallelOptimizer | None) -> None:
        self.dense, self.experts = dense, experts

    @property
    def param_groups(self):
        return list(self.dense.param_groups) + (self.experts.param_groups if self.experts else [])

    def step(self, closure=None):
        out = self.dense.step(closure) if closure is not None else self.dense.step()
        if self.experts is not None:
            self.experts.step()
        return out

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.dense.zero_grad(set_to_none=set_to_none)
        if self.experts is not None:
            self.experts.zero_grad(set_to_none=set_to_none)

    def state_dict(self) -> dict:
        return {"dense": self.dense.state_dict(), "experts": self.experts.state_dict() if self.experts else None}

    def load_state_dict(self, sd: dict) -> None:
        self.dense.load_state_dict(sd["dense"])
        if self.experts is not None and sd.get("experts") is not None:
            self.experts.load_state_dict(sd["experts"])
