"""Headline benchmark: sharded training step of a Llama-style decoder, tokens/s per box.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference] [--config 2|3|tiny]

Default config is BASELINE config 2: AdamW, dp_shard = N, bf16 parameters and compute with fp32
master weights and optimizer state, 8 layers, hidden 2048, 16 heads x 128, SwiGLU 5504, vocab
32000, micro-batch 4 x seq 1024 per GPU (weak scaling), synthetic uniform token ids, random
N(0, 0.02) weights.  For N > 1 launch under ``torch.distributed.run``.

Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events around exactly K steps,
barrier + synchronize on both sides, max over ranks) with the step inputs already on the device.
``e2e`` is the same metric through the user-facing ``train_step`` call, whose timed region
includes the host→device copy of every step's batch from pinned memory and the device→host read
of the loss.

``--impl reference`` runs the unmodified reference package (installed under ``baseline/_ref``)
through its public ``fully_shard`` / ``configure_optimizer`` on a stock-PyTorch model of the same
architecture (``baseline/ref_llama.py``).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONFIGS = {
    "2": dict(model="llama-8L-h2048-ffn5504-v32000", vocab_size=32000, hidden=2048, n_layers=8, n_heads=16,
              head_dim=128, ffn=5504, micro_batch=4, seq_len=1024, optimizer="adamw", ac=False,
              lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1),
    "3": dict(model="llama-32L-h4096-ffn11008-v32000", vocab_size=32000, hidden=4096, n_layers=32, n_heads=32,
              head_dim=128, ffn=11008, micro_batch=1, seq_len=4096, optimizer="mixed_muon_adamw", ac=True,
              lr=0.02, betas=(0.9, 0.95), weight_decay=0.1),
    "4": dict(model="llama-40L-h5120-ffn13824-v32000", vocab_size=32000, hidden=5120, n_layers=40, n_heads=40,
              head_dim=128, ffn=13824, micro_batch=1, seq_len=4096, optimizer="mixed_muon_adamw", ac=True,
              lr=0.02, betas=(0.9, 0.95), weight_decay=0.1, hsdp_replicate=2),
    "5": dict(model="moe-16L-h2048-e64x1408-top6-v32000", kind="moe", vocab_size=32000, hidden=2048, n_layers=16,
              n_heads=16, head_dim=128, n_experts=64, expert_ffn=1408, top_k=6, micro_batch=2, seq_len=4096,
              optimizer="mixed_muon_adamw", ac=False, lr=0.02, betas=(0.9, 0.95), weight_decay=0.1),
    "5s": dict(model="moe-4L-h1024-e16x512-top2-v8192", kind="moe", vocab_size=8192, hidden=1024, n_layers=4,
               n_heads=8, head_dim=128, n_experts=16, expert_ffn=512, top_k=2, micro_batch=2, seq_len=1024,
               optimizer="mixed_muon_adamw", ac=False, lr=0.02, betas=(0.9, 0.95), weight_decay=0.1),
    "5t": dict(model="moe-2L-h256-e8x128-top2-v512", kind="moe", vocab_size=512, hidden=256, n_layers=2, n_heads=2,
               head_dim=128, n_experts=8, expert_ffn=128, top_k=2, micro_batch=2, seq_len=64, optimizer="mixed_muon_adamw",
               ac=False, lr=0.02, betas=(0.9, 0.95), weight_decay=0.1),
    "4t": dict(model="llama-2L-h256-ffn688-v1024-hsdp", vocab_size=1024, hidden=256, n_layers=2, n_heads=2, head_dim=128,
               ffn=688, micro_batch=2, seq_len=128, optimizer="mixed_muon_adamw", ac=True, lr=0.02, betas=(0.9, 0.95),
               weight_decay=0.1, hsdp_replicate=2),
    "tiny": dict(model="llama-2L-h256-ffn688-v1024", vocab_size=1024, hidden=256, n_layers=2, n_heads=2,
                 head_dim=128, ffn=688, micro_batch=2, seq_len=128, optimizer="adamw", ac=False,
                 lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1),
}


# ------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self._thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------ builders
def build_ours_moe(cfg: dict, device, mesh, world: int):
    from torch.distributed.fsdp import MixedPrecisionPolicy

    from matrix_fsdp_b200.models.moe import MoEConfig, MoEModel, configure_moe_optimizer, shard_moe

    mcfg = MoEConfig(vocab_size=cfg["vocab_size"], hidden=cfg["hidden"], n_layers=cfg["n_layers"],
                     n_heads=cfg["n_heads"], head_dim=cfg["head_dim"], n_experts=cfg["n_experts"],
                     expert_ffn=cfg["expert_ffn"], top_k=cfg["top_k"], max_seq_len=cfg["seq_len"],
                     # 0 (default): receive buffers sized for the worst case, nothing is ever dropped; a positive
                     # factor caps them at that multiple of the average load and the line reports what was lost
                     capacity_factor=float(os.environ.get("MFSDP_MOE_CAPACITY_FACTOR", "0")))
    torch.manual_seed(0)
    model = MoEModel(mcfg, ep_group=None if world > 1 else False, device=device, dtype=torch.bfloat16).to(device)
    shard_moe(model, mesh=mesh, mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16),
              optimizer_policy="mixed_muon_adamw")
    opt = configure_moe_optimizer(model, "mixed_muon_adamw", muon_lr=cfg["lr"], adamw_lr=3e-4,
                                  adamw_betas=cfg["betas"], weight_decay=cfg["weight_decay"], muon_momentum=0.95,
                                  muon_ns_steps=5, muon_adjust_lr_fn="original", **_sched_overrides())
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    for u in collect_param_groups(model):
        u.runtime_trace_enabled = False
    return model, opt


_SCHED_OVERRIDES: dict = {}


def _sched_overrides() -> dict:
    """Scheduler options given as ``--sched KEY=VALUE`` (experiments; the headline run passes none)."""
    return dict(_SCHED_OVERRIDES)


def build_ours(cfg: dict, device, mesh, world: int):
    from torch.distributed.fsdp import MixedPrecisionPolicy

    if cfg.get("kind") == "moe":
        return build_ours_moe(cfg, device, mesh, world)

    from matrix_fsdp_b200.models.llama import LlamaConfig, LlamaModel, shard_llama
    from matrix_fsdp_b200.optim import configure_optimizer

    mcfg = LlamaConfig(vocab_size=cfg["vocab_size"], hidden=cfg["hidden"], n_layers=cfg["n_layers"],
                       n_heads=cfg["n_heads"], head_dim=cfg["head_dim"], ffn=cfg["ffn"],
                       activation_checkpointing=cfg["ac"], max_seq_len=cfg["seq_len"])
    torch.manual_seed(0)
    with torch.device(device):
        model = LlamaModel(mcfg)
    model.loss_is_final = True
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16)
    policy = "mixed_muon_adamw" if cfg["optimizer"] == "mixed_muon_adamw" else None
    shard_llama(model, mesh=mesh, mp_policy=mp, optimizer_policy=policy)
    if cfg["optimizer"] == "adamw":
        # the sharded AdamW update runs inside the gradient reduce-scatter kernel (peer transport, N > 1) or, on one
        # GPU, right after each unit's backward on a side stream (beside the next unit's backward GEMMs)
        fused = os.environ.get("MFSDP_FUSED_REDUCE_UPDATE", "1") != "0"
        opt = configure_optimizer(model, "adamw", lr=cfg["lr"], betas=cfg["betas"], weight_decay=cfg["weight_decay"],
                                  fused_reduce_update=fused, **_sched_overrides())
    else:
        opt = configure_optimizer(model, "mixed_muon_adamw", muon_lr=cfg["lr"], adamw_lr=3e-4,
                                  adamw_betas=cfg["betas"], weight_decay=cfg["weight_decay"], muon_momentum=0.95,
                                  muon_ns_steps=5, muon_adjust_lr_fn="original", **_sched_overrides())
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    for u in collect_param_groups(model):
        u.runtime_trace_enabled = False
    return model, opt


def build_reference(cfg: dict, device, mesh, world: int):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "matrix_fsdp")):
        raise FileNotFoundError("reference package is not installed under baseline/_ref")
    sys.path.insert(0, ref_dir)
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import matrix_fsdp as R
    from ref_llama import RefLlama
    from torch.distributed.fsdp import MixedPrecisionPolicy

    if cfg.get("kind") == "moe":
        from ref_moe import RefCombinedOptimizer, RefMoE

        torch.manual_seed(0)
        with torch.device(device):
            model = RefMoE(cfg["vocab_size"], cfg["hidden"], cfg["n_layers"], cfg["n_heads"], cfg["head_dim"],
                           cfg["n_experts"], cfg["expert_ffn"], cfg["top_k"], world=world,
                           ep_group=dist.new_group(list(range(world))) if world > 1 else None)
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16)
        for layer in model.layers:
            R.fully_shard(layer, mesh=mesh, mp_policy=mp, optimizer_policy="mixed_muon_adamw",
                          ignored_params=set(layer.experts.parameters()))
        # the reference's root call does not skip parameters that nested units already manage: name them
        R.fully_shard(model, mesh=mesh, mp_policy=mp,
                      ignored_params={p for layer in model.layers for p in layer.parameters()})
        dense = R.configure_optimizer(model, "mixed_muon_adamw", muon_lr=cfg["lr"], adamw_lr=3e-4,
                                      adamw_betas=cfg["betas"], weight_decay=cfg["weight_decay"], muon_momentum=0.95,
                                      muon_ns_steps=5, muon_adjust_lr_fn="original")
        experts = torch.optim.Muon(model.expert_parameters(), lr=cfg["lr"], momentum=0.95, nesterov=True, ns_steps=5,
                                   weight_decay=cfg["weight_decay"])
        for u in R.collect_param_groups(model):
            u.runtime_trace_enabled = False
        return model, RefCombinedOptimizer(dense, experts)
    torch.manual_seed(0)
    with torch.device(device):
        model = RefLlama(cfg["vocab_size"], cfg["hidden"], cfg["n_layers"], cfg["n_heads"], cfg["head_dim"], cfg["ffn"],
                         activation_checkpointing=cfg["ac"])
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16)
    policy = "mixed_muon_adamw" if cfg["optimizer"] == "mixed_muon_adamw" else None
    for layer in model.layers:
        R.fully_shard(layer, mesh=mesh, mp_policy=mp, optimizer_policy=policy)
    # the reference's root call does not skip parameters that nested units already manage (it would register
    # their local shard views a second time): pass them as ignored_params, which is its documented way
    R.fully_shard(model, mesh=mesh, mp_policy=mp,
                  ignored_params={p for layer in model.layers for p in layer.parameters()})
    if cfg["optimizer"] == "adamw":
        opt = R.configure_optimizer(model, "adamw", lr=cfg["lr"], betas=cfg["betas"], weight_decay=cfg["weight_decay"])
    else:
        opt = R.configure_optimizer(model, "mixed_muon_adamw", muon_lr=cfg["lr"], adamw_lr=3e-4,
                                    adamw_betas=cfg["betas"], weight_decay=cfg["weight_decay"], muon_momentum=0.95,
                                    muon_ns_steps=5, muon_adjust_lr_fn="original")
    for u in R.collect_param_groups(model):
        u.runtime_trace_enabled = False
    return model, opt


# ------------------------------------------------------------------------------------ checkpoint reshard check
def _state_checksums(model, opt) -> dict[str, int]:
    """Layout-independent checksums: for every parameter and optimizer state tensor the sum of its elements' bit
    patterns (as integers) over all ranks of the shard group.  Equal tensors give equal sums on any sharding."""
    from matrix_fsdp_b200.checkpoint.state_dict import iter_optimizer_components
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    def bits(t: torch.Tensor) -> torch.Tensor:
        t = t.detach().contiguous().reshape(-1)
        view = t.view(torch.int32) if t.element_size() == 4 else t.view(torch.int16)
        return view.to(torch.int64).sum().reshape(1)

    sums: dict[str, torch.Tensor] = {}
    units = collect_param_groups(model)
    for ui, u in enumerate(units):
        fb = u.flat_buffer
        for mp in u.registry:
            piece = fb.pieces.get(mp.fqn)
            zero = torch.zeros(1, dtype=torch.int64, device=fb.device)
            sums[f"u{ui}.{mp.fqn}.param"] = bits(fb.local_shard[piece.local_start:piece.local_end]) if piece else zero
            for comp, o in iter_optimizer_components(opt):
                for name, v in sorted(o.state.get(mp.param, {}).items()):
                    if isinstance(v, torch.Tensor) and v.dim() > 0 and piece is not None and v.numel() == piece.numel:
                        sums[f"u{ui}.{mp.fqn}.{comp}.{name}"] = bits(v)
    keys: list = [None] * (dist.get_world_size() if dist.is_initialized() else 1)
    if dist.is_initialized():
        dist.all_gather_object(keys, sorted(sums))
    else:
        keys = [sorted(sums)]
    all_keys = sorted({k for ks in keys for k in ks})
    dev = units[0].flat_buffer.device
    vec = torch.cat([sums.get(k, torch.zeros(1, dtype=torch.int64, device=dev)).to(dev) for k in all_keys])
    if dist.is_initialized():
        dist.all_reduce(vec)                      # replicas count the same pieces: divide that factor out below
    rep = max(units[0].replicate_world_size, 1)
    return {k: int(v) // rep for k, v in zip(all_keys, vec.tolist())}


def verify_reshard(cfg: dict, model, opt, device, world: int, rank: int) -> dict:
    """save_matrix_dcp from the benchmarked (possibly HSDP) model, load_matrix_dcp(allow_reshard=True) into the same
    model on a flat dp_shard = world mesh, and compare parameter / optimizer-state checksums."""
    import shutil
    import tempfile

    from matrix_fsdp_b200 import load_matrix_dcp, save_matrix_dcp
    from matrix_fsdp_b200.api import reset_shared_owner_planners

    path = [tempfile.mkdtemp(prefix="mfsdp_reshard_") if rank == 0 else None]
    if world > 1:
        dist.broadcast_object_list(path, src=0)
    t0 = time.perf_counter()
    save_matrix_dcp(model, path[0], optimizer=opt)
    before = _state_checksums(model, opt)
    flat_cfg = {k: v for k, v in cfg.items() if k != "hsdp_replicate"}
    mesh = None
    if world > 1:
        from torch.distributed.device_mesh import init_device_mesh

        mesh = init_device_mesh(device.type, (world,), mesh_dim_names=("dp_shard",))
    reset_shared_owner_planners()
    model_b, opt_b = build_ours(flat_cfg, device, mesh, world)
    load_matrix_dcp(model_b, path[0], optimizer=opt_b, allow_reshard=True)
    after = _state_checksums(model_b, opt_b)
    common = sorted(set(before) & set(after))
    bad = [k for k in common if before[k] != after[k]]
    if world > 1:
        dist.barrier()
    if rank == 0:
        shutil.rmtree(path[0], ignore_errors=True)
    return {"tensors_compared": len(common), "mismatched": bad[:5], "checksums_equal": not bad and bool(common),
            "seconds": time.perf_counter() - t0, "target_parallelism": f"dp_shard{world}"}


# ------------------------------------------------------------------------------------ diagnostics
def _transport_description(model) -> str:
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    kinds = set()
    for u in collect_param_groups(model):
        t = u.flat_buffer.transport
        kinds.add(t.describe() if hasattr(t, "describe") else t.kind)
    return ",".join(sorted(kinds))


def _moe_drop_report(model, device, world: int) -> dict:
    """Rows the expert-parallel dispatch could not place (0 on a dropless run), summed over ranks and layers
    for every step since the model was built."""
    from matrix_fsdp_b200.parallel.expert_parallel import live_contexts

    lost = torch.zeros(1, dtype=torch.int64, device=device)
    routed = torch.zeros(1, dtype=torch.int64, device=device)
    dropless = True
    for ctx in live_contexts():
        lost += ctx.rows_lost_total()
        routed += ctx.rows_routed_total()
        dropless = dropless and ctx.dropless
    if world > 1:
        dist.all_reduce(lost)
        dist.all_reduce(routed)
    return {"rows_lost": int(lost.item()), "rows_routed": int(routed.item()), "sized_for_worst_case": dropless,
            "capacity_factor": float(os.environ.get("MFSDP_MOE_CAPACITY_FACTOR", "0"))}


def write_timeline(path: str, device_step, sync, rank: int, world: int, device, bench_line: dict) -> dict:
    """Three extra steps with CUDA-event spans around every collective; per-row max over ranks."""
    from matrix_fsdp_b200.parallel import device_timeline as TL

    TL.enable(True)
    device_step(0)                       # first step with recording on is not reported
    sync()
    TL.clear()
    TL.mark_origin()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    n = 3
    for i in range(n):
        device_step(i + 1)
    ev1.record()
    torch.cuda.synchronize()
    spans = TL.resolve()
    step_ms = ev0.elapsed_time(ev1) / n
    TL.enable(False)
    rows = [s.as_row() for s in spans if s.device_ms is not None]
    gathered: list = [None] * world
    if world > 1:
        dist.all_gather_object(gathered, (step_ms, rows))
    else:
        gathered = [(step_ms, rows)]
    totals = {"step_ms": max(g[0] for g in gathered)}
    if rank != 0:
        return totals
    # same collectives in the same order on every rank: merge row by row
    base = gathered[0][1]
    lines = [f"# Step timeline: {bench_line['config']['model']}, {bench_line['config']['parallelism']}, "
             f"transport {bench_line.get('transport')}", "",
             f"Command: `python -m torch.distributed.run --nnodes=1 --nproc-per-node {world} bench.py --gpus {world} "
             f"--steps {bench_line['steps']} --warmup {bench_line['warmup']} --timeline {path}` (for 1 GPU: plain "
             "`python bench.py ...`).", "",
             f"Spans are CUDA events on the communication streams, {n} steps after the timed region "
             f"(device step {totals['step_ms']:.3f} ms with recording on; bench line: "
             f"{bench_line['ms_per_step']:.3f} ms).  `exposed` is the time the compute stream stood still at the "
             "wait for that collective; every figure is the max over ranks, per step-local row.", ""]
    per_kind: dict[str, dict] = {}
    table = ["| # | unit | collective | impl | MB | issued for | start ms | device ms (max) | device ms (min) | exposed ms (max) |",
             "|---|---|---|---|---|---|---|---|---|---|"]
    for i, r in enumerate(base):
        peers = [g[1][i] for g in gathered if i < len(g[1])]
        dmax = max(p["device_ms"] for p in peers)
        dmin = min(p["device_ms"] for p in peers)
        emax = max((p["exposed_ms"] or 0.0) for p in peers)
        k = per_kind.setdefault(r["kind"], {"count": 0, "device_ms": 0.0, "exposed_ms": 0.0, "bytes": 0})
        k["count"] += 1
        k["device_ms"] += dmax
        k["exposed_ms"] += emax
        k["bytes"] += r["bytes"]
        table.append(f"| {i} | {r['unit']} | {r['kind']} | {r['impl']} | {r['bytes'] / 2 ** 20:.1f} | {r['reason']} | "
                     f"{(r['start_ms'] or 0.0):.3f} | {dmax:.3f} | {dmin:.3f} | {emax:.3f} |")
    lines.append("| collective | count / step | device ms / step | exposed ms / step | MB / step |")
    lines.append("|---|---|---|---|---|")
    for kind, k in per_kind.items():
        lines.append(f"| {kind} | {k['count'] / n:.1f} | {k['device_ms'] / n:.3f} | {k['exposed_ms'] / n:.3f} | "
                     f"{k['bytes'] / n / 2 ** 20:.1f} |")
        totals[kind] = {"device_ms_per_step": k["device_ms"] / n, "exposed_ms_per_step": k["exposed_ms"] / n}
    lines += ["", "Rows (all recorded steps, in issue order on rank 0):", ""] + table
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
    return totals


# ------------------------------------------------------------------------------------ main
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--config", default="2", choices=sorted(CONFIGS))
    ap.add_argument("--device", default=None)
    ap.add_argument("--verify-reshard", action="store_true",
                    help="after timing: save_matrix_dcp, load resharded onto a flat dp_shard mesh, compare checksums")
    ap.add_argument("--sched", nargs="*", default=[], metavar="KEY=VALUE",
                    help="scheduler options for the repo's arm, e.g. next_step_prefetch_units=1")
    ap.add_argument("--timeline", default=None, metavar="FILE.md",
                    help="after timing: run 3 more steps with CUDA-event spans around every collective and write "
                         "the per-unit table (start, device time, exposed wait; max over ranks) to FILE.md")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    for kv in args.sched:
        k, _, v = kv.partition("=")
        _SCHED_OVERRIDES[k] = {"true": True, "false": False, "none": None}.get(v.lower(), None) if v.lower() in (
            "true", "false", "none") else (int(v) if v.lstrip("-").isdigit() else (float(v) if v.replace(".", "", 1).isdigit() else v))
    dump_after = float(os.environ.get("MFSDP_BENCH_DUMP_STACKS_AFTER_S", "0"))
    if dump_after > 0:           # diagnose a run that stops making progress: print every thread's stack
        import faulthandler

        faulthandler.dump_traceback_later(dump_after, exit=False, file=sys.stderr)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available() and args.device != "cpu"
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "matrix_fsdp")):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "reference package not installed under baseline/_ref"}))
        return
    device = torch.device("cuda", local_rank) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    mesh = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if cuda else "gloo", device_id=device if cuda else None)
        from torch.distributed.device_mesh import init_device_mesh

        rep = cfg.get("hsdp_replicate", 1)
        if rep > 1 and world % rep == 0 and world > rep:
            mesh = init_device_mesh("cuda" if cuda else "cpu", (rep, world // rep),
                                    mesh_dim_names=("dp_replicate", "dp_shard"))
        else:
            mesh = init_device_mesh("cuda" if cuda else "cpu", (world,), mesh_dim_names=("dp_shard",))
    if args.gpus != world and rank == 0 and world > 1:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)

    build = build_ours if args.impl == "ours" else build_reference
    model, opt = build(cfg, device, mesh, world)

    B, S, V = cfg["micro_batch"], cfg["seq_len"], cfg["vocab_size"]
    total_steps = args.warmup + args.steps
    gen = torch.Generator().manual_seed(1234 + rank)
    e2e_warm = min(3, args.steps)
    host = torch.randint(0, V, (total_steps + e2e_warm + args.steps, B, S + 1), generator=gen, dtype=torch.int64)
    if cuda:
        host = host.pin_memory()
    dev_batches = host[: total_steps].to(device)

    def sync():
        if cuda:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    def device_step(i: int):
        batch = dev_batches[i]
        loss = model(batch[:, :-1], batch[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def e2e_step(i: int) -> float:
        # pinned host batch -> device, forward, backward, optimizer step, loss back to the host
        # (every call gets a batch no earlier step has seen)
        hb = host[total_steps + i]
        if args.impl == "ours":
            from matrix_fsdp_b200.utils import train_step        # the user-facing call of this package

            return train_step(model, opt, hb[:, :-1], hb[:, 1:], device)
        tokens = hb[:, :-1].to(device, non_blocking=True)        # same steps spelled out: nothing of this package
        targets = hb[:, 1:].to(device, non_blocking=True)        # runs in the reference arm
        loss = model(tokens, targets)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return float(loss.item())

    launches_before = 0
    counter = None
    if args.impl == "ours":
        from matrix_fsdp_b200.ops import kernels as _K

        counter = _K

    # ---- warm-up (the last warm-up step is issued on an idle device: its host time is the pure cost of
    # enqueueing one step, which tells a launch-bound run from a device-bound one)
    host_issue_ms = None
    for i in range(args.warmup):
        if i == args.warmup - 1 and i > 0:
            sync()
            t_issue = time.perf_counter()
            last = device_step(i)
            host_issue_ms = (time.perf_counter() - t_issue) * 1e3
        else:
            last = device_step(i)
    sync()
    if cuda:
        torch.cuda.reset_peak_memory_stats()
    if counter is not None:
        launches_before = counter.launch_count()

    # ---- device-timed region
    sampler = ClockSampler(local_rank) if (cuda and rank == 0) else None
    if sampler:
        sampler.start()
    if cuda:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    t0 = time.perf_counter()
    for i in range(args.warmup, total_steps):
        last = device_step(i)
    if cuda:
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
    else:
        ms = (time.perf_counter() - t0) * 1e3
    launches = (counter.launch_count() - launches_before) if counter is not None else 0
    clocks = sampler.stop() if sampler else {}
    sync()
    final_loss = float(last.item())
    peak_mb = torch.cuda.max_memory_allocated() / 2 ** 20 if cuda else 0.0
    symmetric_mb = 0.0
    if args.impl == "ours" and world > 1 and cuda:
        from matrix_fsdp_b200.parallel.peer import PeerContext

        symmetric_mb = PeerContext.symmetric_bytes / 2 ** 20   # cudaMalloc'd outside torch's allocator
        peak_mb += symmetric_mb

    # ---- end-to-end region (public train_step semantics: H2D each step, D2H loss read each step)
    for i in range(e2e_warm):
        e2e_step(i)
    sync()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_loss = e2e_step(e2e_warm + i)
    if cuda:
        torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3

    stats = torch.tensor([ms, e2e_ms, peak_mb], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms, e2e_ms, peak_mb = (float(x) for x in stats.tolist())

    tokens_per_step = B * S * world
    parallelism = f"dp_shard{world}"
    if mesh is not None and mesh.ndim == 2:
        parallelism = f"dp_replicate{mesh.shape[0]}xdp_shard{mesh.shape[1]}"
    if cfg.get("kind") == "moe":
        parallelism += f"+ep{world}"
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms / 1e3)
    out = {
        "metric": "tokens_per_s_per_box", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids; random-init N(0,0.02) weights",
        "impl": args.impl, "peak_mb": peak_mb, "symmetric_mb": symmetric_mb, "final_loss": final_loss,
        "config": {"model": cfg["model"], "global_batch": B * world, "micro_batch_per_gpu": B, "seq_len": S,
                   "parallelism": parallelism, "optimizer": cfg["optimizer"],
                   "precision": "bf16 params+compute, fp32 master weights and optimizer state",
                   "activation_checkpointing": cfg["ac"],
                   "l2": "no explicit flush: each step streams >1 GB of weights/activations (L2 is 126 MB)"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": 2 * B * S * 8, "d2h_bytes_per_step": 4 + (4 if args.impl == "ours" and cuda else 0),
                "last_loss": e2e_loss},
        "gpu_launches": launches, "host_issue_ms_per_step": host_issue_ms,
    }
    if args.impl == "ours":
        out["transport"] = _transport_description(model)
        if cfg.get("kind") == "moe":
            out["moe"] = _moe_drop_report(model, device, world)
    if args.timeline and args.impl == "ours" and cuda:
        out["timeline"] = write_timeline(args.timeline, device_step, sync, rank, world, device, out)
    if args.verify_reshard and args.impl == "ours":
        out["reshard"] = verify_reshard(cfg, model, opt, device, world, rank)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        if args.impl == "ours" and cuda:
            from matrix_fsdp_b200.parallel.peer import PeerTransport

            PeerTransport.close_all()       # nobody exits while a peer may still touch its symmetric memory
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
