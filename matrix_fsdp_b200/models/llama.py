"""Llama-style decoder (RMSNorm, RoPE, causal attention, SwiGLU) on the sm_100a ops.

Parameters are kept as separate matrices (``wq, wk, wv, wo, w_gate, w_up, w_down``) so that a
matrix-owner layout / Muon sees seven 2-D matrices per block; because an FSDP unit lays its
parameters out back to back in one flat buffer, ``wq|wk|wv`` and ``w_gate|w_up`` are adjacent in
memory and the block node multiplies them as one fused matrix.

On CUDA/bf16 each block is a single autograd node (:class:`DecoderBlockFunction`); elsewhere the
same math runs as plain PyTorch ops, which is also the reference the tests compare against.

The reference has no model library; its benches use a LayerNorm/GELU toy transformer
(``test/fsdp/bench_fsdp2_compare.py:456-514``) and a DeepSeek-style fixture
(``test/fsdp/test_deepseek_v3_ep_train.py:354-563``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import functional as OF


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden: int = 2048
    n_layers: int = 8
    n_heads: int = 16
    head_dim: int = 128
    ffn: int = 5504
    rope_theta: float = 10000.0
    eps: float = 1e-5
    tie_embeddings: bool = False
    init_std: float = 0.02
    activation_checkpointing: bool = False
    max_seq_len: int = 4096
    loss_ignore_index: int | None = None   # None: every target counts (lets the loss skip a host sync)

    @staticmethod
    def config1() -> "LlamaConfig":
        return LlamaConfig(vocab_size=1024, hidden=256, n_layers=2, n_heads=4, head_dim=64, ffn=688,
                           tie_embeddings=True, max_seq_len=128)

    @staticmethod
    def config2() -> "LlamaConfig":
        return LlamaConfig(vocab_size=32000, hidden=2048, n_layers=8, n_heads=16, head_dim=128, ffn=5504)

    @staticmethod
    def config3() -> "LlamaConfig":
        return LlamaConfig(vocab_size=32000, hidden=4096, n_layers=32, n_heads=32, head_dim=128, ffn=11008,
                           activation_checkpointing=True)

    @staticmethod
    def config4() -> "LlamaConfig":
        return LlamaConfig(vocab_size=32000, hidden=5120, n_layers=40, n_heads=40, head_dim=128, ffn=13824,
                           activation_checkpointing=True)


class RMSNorm(nn.Module):
    is_norm_like = True

    def __init__(self, dim: int, eps: float = 1e-5) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return OF.rms_norm(x, self.weight, self.eps)


class Matrix(nn.Module):
    """A bias-free linear map holding ``weight`` [out, in]; flagged so shard-hint rules treat it as Linear."""

    is_linear_like = True

    def __init__(self, in_features: int, out_features: int, std: float = 0.02, is_lm_head: bool = False) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.is_lm_head = is_lm_head
        nn.init.normal_(self.weight, mean=0.0, std=std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return OF.linear(x, self.weight, self.weight)


class TokenEmbedding(nn.Embedding):
    """``nn.Embedding`` (same parameter name and shape) whose backward writes the owning unit's gradient bucket."""

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if self.padding_idx is not None or self.max_norm is not None or self.scale_grad_by_freq or self.sparse:
            return super().forward(ids)           # options the kernel path does not implement
        return OF.embedding(ids, self.weight, self.weight)


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig) -> None:
        super().__init__()
        self.cfg = cfg
        h, f, std = cfg.hidden, cfg.ffn, cfg.init_std
        assert cfg.n_heads * cfg.head_dim == h
        # registration order is the flat-buffer order: keep q|k|v and gate|up adjacent
        self.attn_norm = RMSNorm(h, cfg.eps)
        self.wq = Matrix(h, h, std)
        self.wk = Matrix(h, h, std)
        self.wv = Matrix(h, h, std)
        self.wo = Matrix(h, h, std)
        self.mlp_norm = RMSNorm(h, cfg.eps)
        self.w_gate = Matrix(h, f, std)
        self.w_up = Matrix(h, f, std)
        self.w_down = Matrix(f, h, std)

    def _shape(self, batch: int, seq: int) -> OF.BlockShape:
        c = self.cfg
        return OF.BlockShape(batch, seq, c.hidden, c.n_heads, c.head_dim, c.ffn, c.eps, c.rope_theta)

    def mfsdp_fuses_first_gemm(self, x: torch.Tensor, *a, **k) -> bool:
        """Asked by the FSDP unit before forward: will this call run the QKV GEMM that can take the
        q|k|v rows of the all-gather?  (The unit's parameters are bf16 once unsharded.)"""
        return x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 3 and self.cfg.hidden % 8 == 0 \
            and self.cfg.ffn % 8 == 0 and not OF._lib.disabled_by_env()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """``x``: [B, S, H]."""
        b, s, h = x.shape
        c = self.cfg
        cos, sin = OF.rope_tables(max(s, 1), c.head_dim, c.rope_theta, x.device)
        if OF.use_native(x) and self.wq.weight.dtype == torch.bfloat16 and h % 8 == 0 and c.ffn % 8 == 0:
            y = OF.decoder_block(x.reshape(b * s, h), self, self._shape(b, s), cos, sin,
                                 recompute=c.activation_checkpointing and torch.is_grad_enabled())
            return y.view(b, s, h)
        if c.activation_checkpointing and torch.is_grad_enabled():
            from torch.utils.checkpoint import checkpoint

            return checkpoint(self._forward_reference, x, cos, sin, use_reentrant=False)
        return self._forward_reference(x, cos, sin)

    def _forward_reference(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        b, s, h = x.shape
        xn = self.attn_norm(x)
        q = F.linear(xn, self.wq.weight).view(b, s, c.n_heads, c.head_dim)
        k = F.linear(xn, self.wk.weight).view(b, s, c.n_heads, c.head_dim)
        v = F.linear(xn, self.wv.weight).view(b, s, c.n_heads, c.head_dim)
        q, k = OF.apply_rope_reference(q, cos, sin), OF.apply_rope_reference(k, cos, sin)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + F.linear(o.transpose(1, 2).reshape(b, s, h), self.wo.weight)
        xn = self.mlp_norm(x)
        hidden = F.silu(F.linear(xn, self.w_gate.weight)) * F.linear(xn, self.w_up.weight)
        return x + F.linear(hidden, self.w_down.weight)


class LMHead(nn.Module):
    """Final norm + vocabulary projection as one module, so they can be one FSDP unit of their own:
    its all-gather is then prefetched behind the last block instead of riding with the embedding."""

    def __init__(self, hidden: int, vocab_size: int, eps: float, std: float) -> None:
        super().__init__()
        self.final_norm = RMSNorm(hidden, eps)
        self.lm_head = Matrix(hidden, vocab_size, std, is_lm_head=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.lm_head(self.final_norm(x))


class LlamaModel(nn.Module):
    """Decoder-only LM.  ``forward(tokens, targets=None)`` returns logits or the mean CE loss."""

    def __init__(self, cfg: LlamaConfig) -> None:
        super().__init__()
        self.cfg = cfg
        self.embed = TokenEmbedding(cfg.vocab_size, cfg.hidden)
        nn.init.normal_(self.embed.weight, mean=0.0, std=cfg.init_std)
        self.layers = nn.ModuleList([LlamaBlock(cfg) for _ in range(cfg.n_layers)])
        self.head = LMHead(cfg.hidden, cfg.vocab_size, cfg.eps, cfg.init_std)
        if cfg.tie_embeddings:
            self.head.lm_head.weight = self.embed.weight

    @property
    def final_norm(self) -> RMSNorm:
        return self.head.final_norm

    @property
    def lm_head(self) -> Matrix:
        return self.head.lm_head

    def forward(self, tokens: torch.Tensor, targets: torch.Tensor | None = None) -> torch.Tensor:
        x = self.embed(tokens)
        for layer in self.layers:
            x = layer(x)
        logits = self.head(x)
        if targets is None:
            return logits
        n_valid = targets.numel() if self.cfg.loss_ignore_index is None else None
        ignore = -100 if self.cfg.loss_ignore_index is None else self.cfg.loss_ignore_index
        return OF.fused_cross_entropy(logits, targets, ignore_index=ignore, n_valid=n_valid,
                                      unit_upstream_grad=getattr(self, "loss_is_final", False))

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token (fwd+bwd = 3× forward), causal attention counted at half density."""
        c = self.cfg
        per_layer = 2 * (4 * c.hidden * c.hidden + 3 * c.hidden * c.ffn)
        attn = 2 * 2 * seq_len * c.hidden * 0.5
        head = 2 * c.hidden * c.vocab_size
        return 3.0 * (c.n_layers * (per_layer + attn) + head)


def _mark_fused_first_gemm(layer: LlamaBlock) -> None:
    """Tell the layer's FSDP unit which rows of its flat buffer (q|k|v, when adjacent) the block's first
    GEMM reads, so a transport that can may deliver them inside that GEMM (``MFSDP_FUSED_AG_GEMM=0`` disables)."""
    import os

    unit = getattr(layer, "_matrix_fsdp_param_group", None)
    if unit is None or os.environ.get("MFSDP_FUSED_AG_GEMM", "1") == "0":
        return
    by_fqn = {mp.fqn: mp for mp in unit.registry}
    try:
        q, k, v = (by_fqn[n] for n in ("wq.weight", "wk.weight", "wv.weight"))
    except KeyError:
        return
    if q.offset + q.numel == k.offset and k.offset + k.numel == v.offset and q.offset % 8 == 0:
        unit.fused_first_gemm_range = (q.offset, v.offset + v.numel, layer.cfg.hidden)


def shard_llama(model: LlamaModel, *, mesh=None, dp_mesh_dims=None, mp_policy=None, optimizer_policy=None,
                reshard_after_forward=None, shard_root: bool = True, **kw) -> LlamaModel:
    """``fully_shard`` every block, then the embedding and the head (final norm + LM head) as two units of
    their own; with tied embeddings (one shared parameter) or an optimizer policy that plans the root as a
    whole they stay one root unit."""
    from torch.distributed.fsdp import MixedPrecisionPolicy

    from ..api import fully_shard, matrix_fully_shard

    mp = mp_policy or MixedPrecisionPolicy()
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, dp_mesh_dims=dp_mesh_dims, mp_policy=mp, optimizer_policy=optimizer_policy,
                    reshard_after_forward=reshard_after_forward, **kw)
        _mark_fused_first_gemm(layer)
    if shard_root:
        if model.cfg.tie_embeddings:
            # one parameter serves as embedding and LM head: a single root unit that admits the alias
            hints = None
            if optimizer_policy is not None:
                from ..planning.shard_hint import build_shard_hints

                hints = {k: v for k, v in build_shard_hints(model).items() if not k.startswith("layers.")}
            matrix_fully_shard(model, mesh, dp_mesh_dims=dp_mesh_dims, mp_policy=mp, shard_hints=hints,
                               auto_planner_policy="muon_shard_aware" if optimizer_policy else None,
                               owner_assignment="role_greedy" if optimizer_policy else "rotate",
                               reshard_after_forward=True if reshard_after_forward is None else reshard_after_forward,
                               allow_shared_params=True)
        else:
            # two units: the head's gather is prefetched behind the last block and the embedding's behind
            # the optimizer step; each reduce-scatter is half the bytes of a combined root
            for part in (model.embed, model.head):
                fully_shard(part, mesh=mesh, dp_mesh_dims=dp_mesh_dims, mp_policy=mp,
                            optimizer_policy=optimizer_policy, reshard_after_forward=reshard_after_forward, **kw)
    _attach_model_no_sync(model)
    return model


def _attach_model_no_sync(model: nn.Module) -> None:
    """``model.no_sync()`` over every unit below the model, also when the model itself is no unit (blocks,
    embedding and head are units of their own, so no ``fully_shard`` call ever saw the root)."""
    from ..api import _attach_no_sync
    from ..parallel.unit_collection import collect_param_groups

    _attach_no_sync(model, collect_param_groups(model))
