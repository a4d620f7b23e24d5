"""Run a small sharded model for a few steps and dump timing, memory and the runtime event log.

    python -m matrix_fsdp_b200.tools.runtime_profile --mode prefetch --world-size 2 --device cpu

Modes (``MODES`` below): dense AdamW with forward+backward prefetch (``prefetch``), without
(``no_prefetch``), two units ahead (``prefetch2``), with the measuring policies (``adaptive``,
``profile_guided``), post-reshard backward prefetch (``prefetch_post_reshard``), row sharding (``row``),
zero-copy gradient bucket (``zero_copy``), saved-tensor hooks with pooled buffers (``saved_hooks``),
HSDP (``hsdp``, needs world >= 4), and the whole-matrix-owner Muon runs ``matrix_owner_muon``,
``matrix_owner_muon_library`` (library collectives only) and ``matrix_owner_muon_hsdp``.
The workload is chosen with ``--model mlp|transformer|transformer_split_qkv`` (``--seq-len``, ``--heads``), the
unit granularity with ``--unit block|linear``, and the run with ``--optimizer`` (overrides the mode's),
``--dtype``, ``--activation-checkpoint`` (``--checkpoint-use-reentrant``), the scheduler caps
``--max-active-full-param-buffers / -numel / -memory-mb`` and ``--profile-memory-limit-mb`` (profile-guided
prefetch); ``--format json`` and ``--output FILE`` pick the form and the destination of the report.
Ranks are spawned with ``torch.multiprocessing`` and rendezvous through a ``file://`` store (Gloo
on CPU, NCCL on CUDA).  Reports step ms and peak MB as the max over ranks, the aggregated event
summary (per name / category / phase / collective, with device time and exposed wait per collective
when ``--device-timeline`` is given on CUDA), the scheduler table, and with ``--dump-events`` every
recorded event in order, as text or JSON.

Parity: ``matrix_fsdp/tools/runtime_profile.py:1-698``.
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
from torch import nn

# mode -> (fully_shard / matrix_fully_shard keyword arguments, optimizer kind, scheduler keyword arguments)
MODE_TABLE: dict[str, tuple[dict, str, dict]] = {
    "prefetch": ({}, "adamw", dict(max_unsharded_prefetch_units=1)),
    "no_prefetch": ({}, "adamw", dict(max_unsharded_prefetch_units=0)),
    "prefetch2": ({}, "adamw", dict(max_unsharded_prefetch_units=2)),
    "adaptive": ({}, "adamw", dict(prefetch_policy="adaptive")),
    "profile_guided": ({}, "adamw", dict(prefetch_policy="profile_guided", profile_iterations=1)),
    "prefetch_post_reshard": ({}, "adamw", dict(backward_prefetch_timing="post_reshard")),
    "row": ({"row": True}, "adamw", {}),
    "zero_copy": ({"expert": dict(use_zero_copy_grad_bucket=True)}, "adamw", {}),
    "saved_hooks": ({"expert": dict(use_saved_tensor_hooks=True)}, "adamw", {}),
    "hsdp": ({"hsdp": True}, "adamw", {}),
    "matrix_owner_muon": ({"policy": "mixed_muon_adamw"}, "mixed_muon_adamw", {}),
    "matrix_owner_muon_library": ({"expert": dict(auto_shard_hints=True, auto_planner_policy="muon_shard_aware",
                                                  owner_assignment="role_greedy", matrix_collective_backend="torch")},
                                  "mixed_muon_adamw", {}),
    "matrix_owner_muon_hsdp": ({"policy": "mixed_muon_adamw", "hsdp": True}, "mixed_muon_adamw", {}),
}
MODES = tuple(MODE_TABLE)


class _Block(nn.Module):
    def __init__(self, d: int) -> None:
        super().__init__()
        self.norm = nn.LayerNorm(d)
        self.up = nn.Linear(d, 4 * d, bias=False)
        self.down = nn.Linear(4 * d, d, bias=False)

    def forward(self, x):
        return x + self.down(torch.nn.functional.gelu(self.up(self.norm(x))))


class _AttnBlock(nn.Module):
    """Pre-norm attention + MLP block; ``split`` keeps q, k, v (and nothing else) as separate matrices."""

    def __init__(self, d: int, heads: int, inter: int, split: bool) -> None:
        super().__init__()
        self.heads, self.split = heads, split
        self.norm1, self.norm2 = nn.LayerNorm(d), nn.LayerNorm(d)
        if split:
            self.q, self.k, self.v = (nn.Linear(d, d, bias=False) for _ in range(3))
        else:
            self.qkv = nn.Linear(d, 3 * d, bias=False)
        self.proj = nn.Linear(d, d, bias=False)
        self.up, self.down = nn.Linear(d, inter, bias=False), nn.Linear(inter, d, bias=False)

    def forward(self, x):
        b, t, d = x.shape
        h = self.norm1(x)
        q, k, v = (self.q(h), self.k(h), self.v(h)) if self.split else self.qkv(h).chunk(3, dim=-1)
        q, k, v = (z.view(b, t, self.heads, d // self.heads).transpose(1, 2) for z in (q, k, v))
        a = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, t, d)
        x = x + self.proj(a)
        return x + self.down(torch.nn.functional.gelu(self.up(self.norm2(x))))


class _Checkpointed(nn.Module):
    def __init__(self, inner: nn.Module, reentrant: bool) -> None:
        super().__init__()
        self.inner, self.reentrant = inner, reentrant

    def forward(self, x):
        from torch.utils.checkpoint import checkpoint

        return checkpoint(self.inner, x, use_reentrant=self.reentrant)


def _make_model(args) -> nn.Module:
    if args.model == "mlp":
        blocks = [_Block(args.hidden) for _ in range(args.layers)]
    else:
        blocks = [_AttnBlock(args.hidden, args.heads, args.intermediate or 4 * args.hidden,
                             args.model == "transformer_split_qkv") for _ in range(args.layers)]
    return nn.Sequential(*blocks)


def _units_of(model: nn.Module, unit: str) -> list[nn.Module]:
    """Modules to shard, innermost first; with ``linear`` every ``nn.Linear`` is a unit and each block becomes a
    root unit for what is left in it (its norms)."""
    if unit == "block":
        return list(model)
    out: list[nn.Module] = []
    for blk in model:
        out += [m for m in blk.modules() if isinstance(m, nn.Linear)]
        out.append(blk)
    return out


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
    from torch.distributed.tensor.placement_types import Shard

    from matrix_fsdp_b200 import (DataParallelMeshDims, configure_optimizer, format_runtime_events, fully_shard,
                                  matrix_fully_shard, summarize_param_groups, summarize_runtime_events,
                                  summarize_scheduler)
    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.parallel import device_timeline

    reset_shared_owner_planners()
    if args.device_timeline and cuda:
        device_timeline.enable(True)
    torch.manual_seed(0)
    model = _make_model(args).to(device)
    shard_kw, opt_kind, sched_kw = MODE_TABLE[args.mode]
    sched_kw = dict(sched_kw)
    if args.optimizer:
        opt_kind = args.optimizer
    for key in ("max_active_full_param_buffers", "max_active_full_param_numel"):
        if getattr(args, key) is not None:
            sched_kw[key] = getattr(args, key)
    if args.max_active_full_param_memory_mb > 0:
        sched_kw["max_active_full_param_memory_mb"] = args.max_active_full_param_memory_mb
    if args.profile_memory_limit_mb > 0 and sched_kw.get("prefetch_policy") == "profile_guided":
        sched_kw["max_active_full_param_memory_mb"] = args.profile_memory_limit_mb
    mp_kw = {}
    if args.dtype != "float32":
        from torch.distributed.fsdp import MixedPrecisionPolicy

        mp_kw["mp_policy"] = MixedPrecisionPolicy(param_dtype=getattr(torch, args.dtype))
    mesh, dims = None, None
    if shard_kw.get("hsdp"):
        from torch.distributed.device_mesh import init_device_mesh

        mesh = init_device_mesh(args.device, (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
        dims = DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate")
    for blk in _units_of(model, args.unit):
        if "expert" in shard_kw:
            matrix_fully_shard(blk, mesh, dp_mesh_dims=dims, **shard_kw["expert"], **mp_kw)
        else:
            kw = {"shard_placement_fn": (lambda p: Shard(0))} if shard_kw.get("row") else {}
            fully_shard(blk, mesh=mesh, dp_mesh_dims=dims, optimizer_policy=shard_kw.get("policy"), **kw, **mp_kw)
    run_model = model
    if args.activation_checkpoint:
        run_model = nn.Sequential(*[_Checkpointed(b, args.checkpoint_use_reentrant) for b in model])
    opt = configure_optimizer(model, opt_kind, lr=1e-3, **sched_kw)
    in_dtype = getattr(torch, args.dtype)
    shape = (args.batch, args.hidden) if args.model == "mlp" else (args.batch, args.seq_len, args.hidden)
    gen = torch.Generator().manual_seed(rank)
    times = []
    for step in range(args.steps + args.warmup):
        x = torch.randn(*shape, generator=gen).to(device=device, dtype=in_dtype)
        if args.activation_checkpoint and args.checkpoint_use_reentrant:
            x.requires_grad_(True)
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        run_model(x).float().pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
        if cuda:
            torch.cuda.synchronize()
        if step >= args.warmup:
            times.append((time.perf_counter() - t0) * 1e3)
    step_ms = sum(times) / max(len(times), 1)
    peak_mb = torch.cuda.max_memory_allocated() / 2 ** 20 if cuda else 0.0
    stats = torch.tensor([step_ms, peak_mb], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    if rank == 0:
        summary = summarize_runtime_events(model)
        units = summarize_param_groups(model)
        payload = {"mode": args.mode, "world_size": world, "device": args.device, "model": args.model, "unit": args.unit,
                   "optimizer": opt_kind, "dtype": args.dtype, "activation_checkpoint": bool(args.activation_checkpoint),
                   "step_ms": float(stats[0]), "step_ms_each": times,
                   "peak_mb": float(stats[1]), "events": summary, "scheduler": summarize_scheduler(model),
                   "units": [{k: v for k, v in u.items() if k not in ("scheduler",)} for u in units]}
        if args.dump_events:
            from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

            evs = sorted((e for u in collect_param_groups(model) for e in u.runtime_events), key=lambda e: e.sequence)
            payload["event_log"] = [{k: v for k, v in e.as_dict().items() if k != "extra" and v not in (None, 0, False, (), "")}
                                    for e in evs]
        lines = [f"mode={args.mode} model={args.model} unit={args.unit} optimizer={opt_kind} world={world} "
                 f"step_ms={payload['step_ms']:.3f} peak_mb={payload['peak_mb']:.1f}",
                 format_runtime_events(model, limit=12)]
        sc = payload["scheduler"]
        if sc:
            lines.append(f"scheduler: policy={sc['prefetch_policy']} fwd_depth={sc['forward_prefetch_depth']} "
                         f"bwd_depth={sc['backward_prefetch_depth']} counters={sc['counters']}")
        lines.append("units:")
        for u in payload["units"]:
            lines.append(f"  {u.get('name')}: params={u.get('num_params')} numel={u.get('total_numel')} "
                         f"local={u.get('local_numel')} planner={u.get('planner_name')} mode={u.get('runtime_mode')}")
        lines += [f"   {row}" for row in payload.get("event_log", [])]
        payload["text"] = "\n".join(lines)
        with open(out_file, "w") as f:
            json.dump(payload, f, default=str)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_profile(args) -> dict:
    with tempfile.TemporaryDirectory() as tmp:
        out_file = os.path.join(tmp, "out.json")
        init_file = os.path.join(tmp, "rdzv")
        if args.world_size == 1:
            _worker(0, 1, args, init_file, out_file)
        else:
            mp.spawn(_worker, args=(args.world_size, args, init_file, out_file), nprocs=args.world_size, join=True)
        with open(out_file) as f:
            return json.load(f)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=MODES, default="prefetch")
    ap.add_argument("--world-size", type=int, default=2)
    ap.add_argument("--device", choices=("cpu", "cuda"), default="cpu")
    ap.add_argument("--hidden", type=int, default=32)
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--model", choices=("mlp", "transformer", "transformer_split_qkv"), default="mlp")
    ap.add_argument("--unit", choices=("block", "linear"), default="block")
    ap.add_argument("--intermediate", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=16)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--optimizer", choices=("sgd", "adamw", "muon", "mixed_muon_adamw"), default=None,
                    help="override the optimizer the mode names")
    ap.add_argument("--dtype", choices=("float32", "bfloat16", "float16"), default="float32")
    ap.add_argument("--activation-checkpoint", action="store_true")
    ap.add_argument("--checkpoint-use-reentrant", action="store_true")
    ap.add_argument("--max-active-full-param-buffers", type=int, default=None)
    ap.add_argument("--max-active-full-param-numel", type=int, default=None)
    ap.add_argument("--max-active-full-param-memory-mb", type=float, default=0.0)
    ap.add_argument("--profile-memory-limit-mb", type=float, default=0.0)
    ap.add_argument("--format", choices=("text", "json"), default="text", dest="output_format")
    ap.add_argument("--output", default="", help="write the report to this file instead of stdout")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--dump-events", action="store_true", help="every recorded runtime event, in order")
    ap.add_argument("--device-timeline", action="store_true",
                    help="CUDA: record CUDA-event spans so the collective table carries device and exposed time")
    args = ap.parse_args(argv)
    if MODE_TABLE[args.mode][0].get("hsdp") and (args.world_size < 4 or args.world_size % 2):
        ap.error(f"{args.mode} needs an even world size >= 4")
    if args.model != "mlp" and args.hidden % args.heads:
        ap.error("--hidden must be a multiple of --heads")
    payload = run_profile(args)
    text = payload.pop("text", "")
    as_json = args.json or args.output_format == "json"
    report = json.dumps(payload) if as_json else text
    if args.output:
        with open(args.output, "w") as f:
            f.write(report + "\n")
    else:
        print(report)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
