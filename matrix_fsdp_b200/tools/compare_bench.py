"""Compare this runtime with PyTorch FSDP2 and with an eager data-parallel oracle on the reference's toy model.

    python -m matrix_fsdp_b200.tools.compare_bench --world-size 2 --device cpu \
        --modes matrix_default matrix_owner_muon fsdp2 --hidden 256 --layers 2 --seq 64 --steps 5 --correctness

Model ``transformer_split_qkv``: per block separate q / k / v / proj / up0 / up1 / down ``nn.Linear`` (no bias),
two LayerNorms, GELU, non-causal SDPA; input is a random hidden state ``[B, S, H]`` and the loss is the MSE
against a random target (no embedding, no LM head), as in the reference's bench
(test/fsdp/bench_fsdp2_compare.py:456-483,2951-2957,3022-3023).

Modes
  ``matrix_default``      ``fully_shard`` per block, AdamW
  ``matrix_row``          row sharding (``shard_placement_fn=Shard(0)``), AdamW
  ``matrix_owner_muon``   ``optimizer_policy="mixed_muon_adamw"`` (whole-matrix owners) + mixed Muon / AdamW
  ``fsdp2``               ``torch.distributed.fsdp.fully_shard`` per block, AdamW
  ``fsdp2_muon``          FSDP2 + ``torch.optim.Muon`` on the DTensor shards (every Newton-Schulz product redistributes
                          the sharded matrices) + AdamW for the rest: the baseline of the reference's Muon rows
Per mode it reports the step time (host clock around synchronised steps, max over ranks), phase times
(zero_grad / forward / backward / step), peak memory, and with ``--correctness`` the loss difference and the
largest full-parameter difference against an eager model whose gradients the tool all-reduces itself.
Ranks are spawned with ``torch.multiprocessing`` and rendezvous through a ``file://`` store.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F
from torch import nn

MODES = ("matrix_default", "matrix_row", "matrix_owner_muon", "fsdp2", "fsdp2_muon")


class SplitQKVBlock(nn.Module):
    def __init__(self, hidden: int, heads: int, inter: int) -> None:
        super().__init__()
        self.heads = heads
        self.norm1, self.norm2 = nn.LayerNorm(hidden), nn.LayerNorm(hidden)
        self.q, self.k, self.v, self.proj = (nn.Linear(hidden, hidden, bias=False) for _ in range(4))
        self.up0, self.up1 = nn.Linear(hidden, inter, bias=False), nn.Linear(hidden, inter, bias=False)
        self.down = nn.Linear(inter, hidden, bias=False)

    def forward(self, x):
        b, s, h = x.shape
        y = self.norm1(x)
        q, k, v = (m(y).view(b, s, self.heads, h // self.heads).transpose(1, 2) for m in (self.q, self.k, self.v))
        a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, s, h)
        x = x + self.proj(a)
        y = self.norm2(x)
        return x + self.down(F.gelu(self.up0(y)) * self.up1(y))


def build_model(hidden: int, layers: int, heads: int, inter: int) -> nn.Sequential:
    torch.manual_seed(0)
    return nn.Sequential(*[SplitQKVBlock(hidden, heads, inter) for _ in range(layers)])


def _sync(cuda: bool) -> None:
    if cuda:
        torch.cuda.synchronize()


def _setup_mode(mode: str, model: nn.Module, args):
    """Returns (optimizer, gather_full) where gather_full() -> {name: full tensor}."""
    if mode.startswith("matrix"):
        from torch.distributed.tensor.placement_types import Shard

        from matrix_fsdp_b200 import configure_optimizer, fully_shard
        from matrix_fsdp_b200.api import reset_shared_owner_planners
        from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions, get_model_state_dict

        reset_shared_owner_planners()
        kw = {}
        if mode == "matrix_row":
            kw["shard_placement_fn"] = lambda p: Shard(0)
        if mode == "matrix_owner_muon":
            kw["optimizer_policy"] = "mixed_muon_adamw"
        for blk in model:
            fully_shard(blk, **kw)
        if mode == "matrix_owner_muon":
            opt = configure_optimizer(model, "mixed_muon_adamw", muon_lr=args.muon_lr, adamw_lr=args.lr,
                                      muon_momentum=0.95, muon_ns_steps=5, muon_adjust_lr_fn="original",
                                      weight_decay=0.0)
        else:
            opt = configure_optimizer(model, "adamw", lr=args.lr, weight_decay=0.0)
        return opt, lambda: get_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True))
    from torch.distributed.fsdp import fully_shard as fsdp2_fully_shard

    for blk in model:
        fsdp2_fully_shard(blk)
    if mode == "fsdp2_muon":
        # torch.optim.Muon on DTensor shards: every Newton-Schulz matmul redistributes the sharded matrix
        mats = [p for p in model.parameters() if p.dim() == 2]
        rest = [p for p in model.parameters() if p.dim() != 2]
        opt = _Both(torch.optim.Muon(mats, lr=args.muon_lr, momentum=0.95, nesterov=True, ns_steps=5, weight_decay=0.0),
                    torch.optim.AdamW(rest, lr=args.lr, weight_decay=0.0))
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=args.lr, weight_decay=0.0)

    def gather_full():
        out = {}
        for n, p in model.named_parameters():
            t = p.detach()
            out[n] = t.full_tensor() if hasattr(t, "full_tensor") else t
        return out

    return opt, gather_full


class _Both:
    """Two optimizers stepped together (Muon for the matrices, AdamW for the rest)."""

    def __init__(self, *opts) -> None:
        self.opts = opts

    def step(self) -> None:
        for o in self.opts:
            o.step()

    def zero_grad(self) -> None:
        for o in self.opts:
            o.zero_grad()


def _eager_reference(args, device, world: int, rank: int, mode: str):
    """Eager model + the same optimizer family; gradients are averaged over ranks by hand."""
    ref = build_model(args.hidden, args.layers, args.heads, args.inter).to(device)
    if mode in ("matrix_owner_muon", "fsdp2_muon") and hasattr(torch.optim, "Muon"):
        mats = [p for p in ref.parameters() if p.dim() == 2]
        rest = [p for p in ref.parameters() if p.dim() != 2]
        opts = [torch.optim.Muon(mats, lr=args.muon_lr, momentum=0.95, nesterov=True, ns_steps=5, weight_decay=0.0),
                torch.optim.AdamW(rest, lr=args.lr, weight_decay=0.0)]
    else:
        opts = [torch.optim.AdamW(ref.parameters(), lr=args.lr, weight_decay=0.0)]
    return ref, opts


def _run_mode(mode: str, args, device, world: int, rank: int) -> dict:
    cuda = device.type == "cuda"
    model = build_model(args.hidden, args.layers, args.heads, args.inter).to(device)
    try:
        opt, gather_full = _setup_mode(mode, model, args)
    except Exception as exc:                                   # a mode this torch build cannot run
        return {"mode": mode, "unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    ref, ropts = _eager_reference(args, device, world, rank, mode) if args.correctness else (None, [])
    gen = torch.Generator().manual_seed(1234 + rank)
    phases = {"zero_grad": 0.0, "forward": 0.0, "backward": 0.0, "step": 0.0}
    total, loss_diff = 0.0, 0.0
    if cuda:
        torch.cuda.reset_peak_memory_stats()
    for step in range(args.warmup + args.steps):
        x = torch.randn(args.batch, args.seq, args.hidden, generator=gen).to(device)
        y = torch.randn(args.batch, args.seq, args.hidden, generator=gen).to(device)
        timed = step >= args.warmup
        _sync(cuda)
        t0 = time.perf_counter()
        opt.zero_grad()
        _sync(cuda)
        t1 = time.perf_counter()
        loss = F.mse_loss(model(x), y)
        _sync(cuda)
        t2 = time.perf_counter()
        loss.backward()
        _sync(cuda)
        t3 = time.perf_counter()
        opt.step()
        _sync(cuda)
        t4 = time.perf_counter()
        if timed:
            for name, dt in zip(phases, (t1 - t0, t2 - t1, t3 - t2, t4 - t3)):
                phases[name] += dt * 1e3
            total += (t4 - t0) * 1e3
        if ref is not None:
            rl = F.mse_loss(ref(x), y)
            rl.backward()
            if world > 1:
                for p in ref.parameters():
                    dist.all_reduce(p.grad)
                    p.grad.div_(world)
            for o in ropts:
                o.step()
                o.zero_grad()
            loss_diff = max(loss_diff, abs(float(loss.detach()) - float(rl.detach())))
    row = {"mode": mode, "step_ms": total / args.steps, "phase_ms": {k: v / args.steps for k, v in phases.items()},
           "peak_mb": torch.cuda.max_memory_allocated() / 2 ** 20 if cuda else 0.0}
    if ref is not None:
        full = gather_full()
        diff = 0.0
        for n, p in ref.named_parameters():
            diff = max(diff, float((full[n].to(p.device).float() - p.detach().float()).abs().max()))
        row["max_loss_diff_vs_eager"], row["max_param_diff_vs_eager"] = loss_diff, diff
    stats = torch.tensor([row["step_ms"], row["peak_mb"]], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    row["step_ms"], row["peak_mb"] = float(stats[0]), float(stats[1])
    return row


def _worker(rank: int, world: int, args, init_file: str, out_file: str) -> None:
    os.environ["GLOO_SOCKET_IFNAME"] = "lo"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    cuda = args.device == "cuda"
    if cuda:
        torch.cuda.set_device(rank)
    device = torch.device("cuda", rank) if cuda else torch.device("cpu")
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", init_method=f"file://{init_file}", rank=rank,
                                world_size=world)
    rows = [_run_mode(m, args, device, world, rank) for m in args.modes]
    for r in rows:
        base_mode = "fsdp2_muon" if r["mode"] == "matrix_owner_muon" else "fsdp2"
        base = next((b for b in rows if b["mode"] == base_mode and "step_ms" in b), None)
        if base and "step_ms" in r and r is not base and not r["mode"].startswith("fsdp2"):
            r[f"speedup_vs_{base_mode}"] = base["step_ms"] / r["step_ms"]
    if rank == 0:
        with open(out_file, "w") as f:
            json.dump(rows, f)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--modes", nargs="+", default=["matrix_default", "fsdp2"], choices=MODES)
    ap.add_argument("--world-size", type=int, default=2)
    ap.add_argument("--device", choices=("cpu", "cuda"), default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--inter", type=int, default=None)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--muon-lr", type=float, default=0.02)
    ap.add_argument("--correctness", action="store_true")
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    args.inter = args.inter or 4 * args.hidden
    with tempfile.TemporaryDirectory() as tmp:
        out_file = os.path.join(tmp, "rows.json")
        if args.world_size == 1:
            _worker(0, 1, args, os.path.join(tmp, "rdzv"), out_file)
        else:
            mp.spawn(_worker, args=(args.world_size, args, os.path.join(tmp, "rdzv"), out_file), nprocs=args.world_size,
                     join=True)
        rows = json.load(open(out_file))
    for r in rows:
        print(json.dumps(r))
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
