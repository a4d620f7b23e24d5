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
  ... and one mode per runtime option that selects another code path (see ``MATRIX_MODES``).
Per mode it reports the step time (host clock around synchronised steps, max over ranks), phase times
(zero_grad / forward / backward / step), peak memory, and with ``--correctness`` the loss difference, the
largest full-parameter difference and the per-parameter difference of the gathered full gradients of the first
step (worst parameter named) against an eager model whose gradients the tool all-reduces itself.
``--memory-trace`` adds allocated / peak / reserved bytes after every phase of the last step and the bytes the
runtime's own buffers hold; ``--microbench copy_in`` and ``--microbench materialize`` time the gradient-bucket
copy-in variants and the parameter view swap in isolation (bench_fsdp2_compare.py:967-1175,1865-1932).
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

# mode -> (sharding keyword arguments, optimizer kind, optimizer keyword arguments).  Every runtime option of
# this package that selects a different code path has a mode, so their cost and their results can be compared
# side by side (the reference's bench lists its variants the same way, bench_fsdp2_compare.py:50-111).
_OWNER = dict(auto_shard_hints=True, auto_planner_policy="muon_shard_aware", owner_assignment="role_greedy")
MATRIX_MODES: dict[str, tuple[dict, str, dict]] = {
    "matrix_default": ({}, "adamw", {}),
    "matrix_row": ({"row": True}, "adamw", {}),
    "matrix_owner_muon": ({"policy": "mixed_muon_adamw"}, "mixed_muon_adamw", {}),
    "matrix_owner_adamw": ({"expert": _OWNER}, "adamw", {}),
    "matrix_no_reshard": ({"reshard_after_forward": False}, "adamw", {}),
    "matrix_zero_copy_grads": ({"expert": dict(use_zero_copy_grad_bucket=True)}, "adamw", {}),
    "matrix_saved_tensor_hooks": ({"expert": dict(use_saved_tensor_hooks=True)}, "adamw", {}),
    "matrix_keep_storage": ({"expert": dict(shrink_full_param_storage_after_backward=False)}, "adamw", {}),
    "matrix_flat_reduce": ({"expert": dict(backward_reduce_strategy="flat")}, "adamw", {}),
    "matrix_per_param_reduce": ({"expert": dict(backward_reduce_strategy="per_param")}, "adamw", {}),
    "matrix_per_param_allreduce": ({"expert": dict(backward_reduce_strategy="per_param_allreduce")}, "adamw", {}),
    "matrix_padded_all_gather": ({"expert": dict(param_gather_strategy="matrix_all_gather")}, "adamw", {}),
    "matrix_uneven_all_gather": ({"expert": dict(param_gather_strategy="uneven_all_gather")}, "adamw", {}),
    "matrix_all_reduce_gather": ({"expert": dict(param_gather_strategy="all_reduce")}, "adamw", {}),
    "matrix_owner_broadcast": ({"expert": dict(_OWNER, param_gather_strategy="owner_broadcast")}, "adamw", {}),
    "matrix_library_collectives": ({"expert": dict(matrix_collective_backend="torch")}, "adamw", {}),
    "matrix_owner_muon_library": ({"expert": dict(_OWNER, matrix_collective_backend="torch")}, "mixed_muon_adamw", {}),
    "matrix_no_prefetch": ({}, "adamw", dict(max_unsharded_prefetch_units=0)),
    "matrix_prefetch2": ({}, "adamw", dict(max_unsharded_prefetch_units=2)),
    "matrix_adaptive_prefetch": ({}, "adamw", dict(prefetch_policy="adaptive")),
    "matrix_profile_guided_prefetch": ({}, "adamw", dict(prefetch_policy="profile_guided")),
    "matrix_two_pending_reduces": ({}, "adamw", dict(max_pending_backward_reduces=2)),
    "matrix_fused_reduce_update": ({}, "adamw", dict(fused_reduce_update=True)),
    "matrix_sgd": ({}, "sgd", {}),
}
MODES = tuple(MATRIX_MODES) + ("fsdp2", "fsdp2_no_reshard", "fsdp2_muon")


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

        from matrix_fsdp_b200 import configure_optimizer, fully_shard, matrix_fully_shard
        from matrix_fsdp_b200.api import reset_shared_owner_planners
        from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions, get_model_state_dict

        reset_shared_owner_planners()
        shard_kw, opt_kind, opt_kw = MATRIX_MODES[mode]
        for blk in model:
            if "expert" in shard_kw:
                matrix_fully_shard(blk, **shard_kw["expert"])
            else:
                kw = {}
                if shard_kw.get("row"):
                    kw["shard_placement_fn"] = lambda p: Shard(0)
                if shard_kw.get("policy"):
                    kw["optimizer_policy"] = shard_kw["policy"]
                if "reshard_after_forward" in shard_kw:
                    kw["reshard_after_forward"] = shard_kw["reshard_after_forward"]
                fully_shard(blk, **kw)
        if opt_kind == "mixed_muon_adamw":
            opt = configure_optimizer(model, "mixed_muon_adamw", muon_lr=args.muon_lr, adamw_lr=args.lr,
                                      muon_momentum=0.95, muon_ns_steps=5, muon_adjust_lr_fn="original",
                                      weight_decay=0.0, **opt_kw)
        elif opt_kind == "sgd":
            opt = configure_optimizer(model, "sgd", lr=args.lr, **opt_kw)
        else:
            opt = configure_optimizer(model, "adamw", lr=args.lr, weight_decay=0.0, **opt_kw)
        return opt, lambda: get_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True))
    from torch.distributed.fsdp import fully_shard as fsdp2_fully_shard

    for blk in model:
        fsdp2_fully_shard(blk, reshard_after_forward=mode != "fsdp2_no_reshard")
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
    muon = mode == "fsdp2_muon" or (mode in MATRIX_MODES and MATRIX_MODES[mode][1] == "mixed_muon_adamw")
    if mode in MATRIX_MODES and MATRIX_MODES[mode][1] == "sgd":
        return ref, [torch.optim.SGD(ref.parameters(), lr=args.lr)]
    if muon and hasattr(torch.optim, "Muon"):
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
    grad_check = None
    mem_trace: dict[str, dict] = {}

    def mem(tag: str) -> None:
        if args.memory_trace and cuda:
            mem_trace[tag] = {"allocated_mb": torch.cuda.memory_allocated() / 2 ** 20,
                              "max_allocated_mb": torch.cuda.max_memory_allocated() / 2 ** 20,
                              "reserved_mb": torch.cuda.memory_reserved() / 2 ** 20}

    for step in range(args.warmup + args.steps):
        x = torch.randn(args.batch, args.seq, args.hidden, generator=gen).to(device)
        y = torch.randn(args.batch, args.seq, args.hidden, generator=gen).to(device)
        timed = step >= args.warmup
        last = step == args.warmup + args.steps - 1
        _sync(cuda)
        t0 = time.perf_counter()
        opt.zero_grad()
        _sync(cuda)
        t1 = time.perf_counter()
        loss = F.mse_loss(model(x), y)
        _sync(cuda)
        t2 = time.perf_counter()
        if last:
            mem("after_forward")
        loss.backward()
        _sync(cuda)
        t3 = time.perf_counter()
        if last:
            mem("after_backward")
        if ref is not None and step == 0:
            grad_check = _full_grads(mode, model)
        opt.step()
        _sync(cuda)
        t4 = time.perf_counter()
        if last:
            mem("after_step")
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
            if grad_check is not None and step == 0:
                grad_check = _compare_grads(grad_check, ref)
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
        if isinstance(grad_check, dict) and "worst_param" in grad_check:
            row["full_grad_check"] = grad_check
    if args.memory_trace:
        row["memory_trace"] = mem_trace
        if mode.startswith("matrix"):
            from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

            acct: dict[str, int] = {}
            for u in collect_param_groups(model):
                for k, v in u.flat_buffer.memory_snapshot().items():
                    if k.endswith("_bytes"):
                        acct[k] = acct.get(k, 0) + int(v)
            row["runtime_buffer_bytes"] = acct
    stats = torch.tensor([row["step_ms"], row["peak_mb"]], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    row["step_ms"], row["peak_mb"] = float(stats[0]), float(stats[1])
    return row


def _full_grads(mode: str, model: nn.Module) -> dict[str, torch.Tensor]:
    """Gathered full gradients by parameter name, after backward and before the optimizer step."""
    if mode.startswith("matrix"):
        from matrix_fsdp_b200.utils import gather_full_grads

        return gather_full_grads(model)
    out = {}
    for n, p in model.named_parameters():
        g = p.grad
        if g is not None:
            out[n] = (g.full_tensor() if hasattr(g, "full_tensor") else g).detach().float().clone()
    return out


def _compare_grads(full: dict[str, torch.Tensor], ref: nn.Module) -> dict:
    worst, worst_abs, worst_rel = None, 0.0, 0.0
    for n, p in ref.named_parameters():
        if n not in full or p.grad is None:
            continue
        d = (full[n].to(p.device).float().reshape(p.shape) - p.grad.float()).abs().max().item()
        rel = d / max(p.grad.float().abs().max().item(), 1e-12)
        if d >= worst_abs:
            worst, worst_abs = n, d
        worst_rel = max(worst_rel, rel)
    return {"params_compared": len(full), "worst_param": worst, "max_abs_diff": worst_abs, "max_rel_diff": worst_rel}


def _microbench(kind: str, args, device) -> list[dict]:
    """Host + device time of two per-step runtime chores, without any model around them."""
    from matrix_fsdp_b200.parallel.collectives import SegmentTables
    from matrix_fsdp_b200.core.layout import LayoutSegment
    from matrix_fsdp_b200.parallel.grad_bucket import BucketParam, MatrixGradBucket

    cuda = device.type == "cuda"
    h, inter = args.hidden, args.inter
    shapes = [(h,), (h, h), (h, h), (h, h), (h, h), (h,), (inter, h), (inter, h), (h, inter)]
    numels = [int(torch.Size(s).numel()) for s in shapes]
    total = sum(numels)
    world = max(args.world_size, 2)
    rows = []

    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        _sync(cuda)
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        _sync(cuda)
        return (time.perf_counter() - t0) * 1e3 / reps

    if kind == "copy_in":
        grads = [torch.randn(n, device=device) for n in numels]
        offs = [sum(numels[:i]) for i in range(len(numels))]
        layouts = {
            "flat_contiguous": [[LayoutSegment(r * (total // world), (r + 1) * (total // world) if r < world - 1 else total, 0)]
                                for r in range(world)],
            "whole_param_owners": None,
        }
        owners: list[list] = [[] for _ in range(world)]
        cur = [0] * world
        for i, (o, n) in enumerate(zip(offs, numels)):
            r = i % world
            owners[r].append(LayoutSegment(o, o + n, cur[r]))
            cur[r] += n
        layouts["whole_param_owners"] = owners
        for name, segs in layouts.items():
            tables = SegmentTables.build(total, segs, 0)
            bucket = MatrixGradBucket(tables, [BucketParam(f"p{i}", o, n) for i, (o, n) in enumerate(zip(offs, numels))],
                                      grads[0].dtype, device)
            bucket.attach(torch.empty(total, device=device))
            ms = timed(lambda: bucket.copy_in(grads))
            rows.append({"microbench": "copy_in", "layout": name, "numel": total, "ms": ms,
                         "gb_per_s": 2 * total * 4 / ms / 1e6, "path": bucket.copy_in(grads)})
        return rows
    # materialize: swapping param.data between local and full views (a host loop over the parameters)
    from matrix_fsdp_b200 import fully_shard
    from matrix_fsdp_b200.api import reset_shared_owner_planners

    reset_shared_owner_planners()
    blk = SplitQKVBlock(args.hidden, args.heads, args.inter).to(device)
    fully_shard(blk)
    unit = blk._matrix_fsdp_param_group
    fb = unit.flat_buffer

    def swap():
        fb._materialize_full()
        fb.use_full_param_buffer()
        fb.use_local_shards()

    rows.append({"microbench": "materialize", "params": len(unit.registry), "numel": fb.total_numel,
                 "view_swap_ms": timed(swap), "full_buffer_mode": "alias" if fb.full_aliases_shard else "storage_resize"})
    return rows


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
    if args.microbench:
        rows = _microbench(args.microbench, args, device)
        if rank == 0:
            with open(out_file, "w") as f:
                json.dump(rows, f)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
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
    ap.add_argument("--memory-trace", action="store_true")
    ap.add_argument("--microbench", choices=("copy_in", "materialize"), default=None)
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
