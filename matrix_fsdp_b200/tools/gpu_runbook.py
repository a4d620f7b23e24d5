"""Named GPU regression batches, a no-GPU preflight that writes the runbook, and the log -> table summariser.

    python -m matrix_fsdp_b200.tools.regression batch <name> [--dry-run] [--report-dir DIR] [--world-size 8 ...]
    python -m matrix_fsdp_b200.tools.regression plan  [--out-dir DIR] [--no-local-checks]
    python -m matrix_fsdp_b200.tools.regression summarize DIR [--json]

A *batch* is an ordered list of steps; a step is one child process (its command line, extra environment
and the log file its output goes to).  ``--dry-run`` prints the steps as a shell script instead of
running them, which is also what ``plan`` writes to ``commands.sh`` after its CPU sanity checks, so the
GPU time of a machine is spent on commands that already parsed and imported on a CPU box.

Every step writes ``<report-dir>/<step>.log``.  The tools of this package print one JSON object per
line for their results; ``summarize`` collects those lines from every log of a report directory and
prints the phase table (per mode, with the ratio against the library FSDP row of the same log), the
memory table, the collective-bandwidth table and the device-timeline table.

Parity: ``scripts/run_gpu_test_batch.sh``, ``scripts/run_gpu_regression.sh``, ``scripts/run_gpu_comm_report.sh``,
``scripts/prepare_gpu_benchmark.sh`` and ``scripts/summarize_gpu_comm_report.py`` of the reference.
"""
from __future__ import annotations

import json
import os
import shlex
import subprocess
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
PY = sys.executable


@dataclass
class Settings:
    """Shape of the workload the batches run; every field has a command-line override."""
    world_size: int = 4
    planner_world_sizes: tuple[int, ...] = (4, 8)
    large_world_sizes: tuple[int, ...] = (4, 8)
    layers: int = 16
    large_layers: tuple[int, ...] = (16, 24, 32)
    hidden: int = 1024
    inter: int = 4096
    heads: int = 8
    seq: int = 4096
    batch: int = 1
    warmup: int = 3
    steps: int = 8
    trials: int = 3
    correctness_layers: int = 4
    correctness_seq: int = 512

    def model_args(self, *, layers: int | None = None, seq: int | None = None) -> list[str]:
        return ["--device", "cuda", "--world-size", str(self.world_size), "--layers", str(layers or self.layers),
                "--hidden", str(self.hidden), "--inter", str(self.inter), "--heads", str(self.heads),
                "--seq", str(seq or self.seq), "--batch", str(self.batch), "--warmup", str(self.warmup),
                "--steps", str(self.steps)]


@dataclass
class Step:
    name: str
    argv: list[str]
    env: dict[str, str] = field(default_factory=dict)
    timeout: float = 1800.0

    def shell(self, report_dir: str) -> str:
        envs = " ".join(f"{k}={shlex.quote(v)}" for k, v in self.env.items())
        cmd = " ".join(shlex.quote(a) for a in self.argv)
        return f"{envs + ' ' if envs else ''}timeout {int(self.timeout)} {cmd} > {shlex.quote(report_dir)}/{self.name}.log 2>&1"


def _tool(name: str, *args: str) -> list[str]:
    return [PY, "-m", f"matrix_fsdp_b200.tools.{name}", *args]


def _torchrun(n: int, port: int, *tail: str) -> list[str]:
    return [PY, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
            "--master-port", str(port), *tail]


_SMOKE_TESTS = ("sharded_training_peer_vs_nccl or nvls_collectives or training_without_nvls or owner_muon or "
                "gather_gemm or hsdp or expert_parallel or checkpoint")


def _cuda_smoke(s: Settings) -> list[Step]:
    return [Step("cuda_smoke", [PY, "-m", "pytest", "tests/test_gpu_multi.py", "-m", "gpu", "-x", "-q", "-k", _SMOKE_TESTS],
                 timeout=1200)]


def _cuda_full(s: Settings) -> list[Step]:
    return [Step("cuda_full", [PY, "-m", "pytest", "tests", "-m", "gpu", "-x", "-q"], timeout=2400)]


def _planner(s: Settings) -> list[Step]:
    return [Step(f"planner_ws{ws}", _tool("planner_report", "--model", "transformer", "--layers", str(s.layers), "--hidden",
                                         str(s.hidden), "--ffn", str(s.inter), "--world-size", str(ws), "--json"))
            for ws in s.planner_world_sizes]


def _compare(name: str, modes: list[str], s: Settings, *extra: str, layers=None, seq=None) -> Step:
    return Step(name, _tool("compare_bench", "--modes", *modes, *s.model_args(layers=layers, seq=seq), *extra))


def _compare_adamw(s: Settings) -> list[Step]:
    return [_compare("compare_adamw", ["fsdp2", "matrix_default", "matrix_row", "matrix_no_reshard", "fsdp2_no_reshard"], s),
            _compare("compare_adamw_correctness", ["fsdp2", "matrix_default"], s, "--correctness",
                     layers=s.correctness_layers, seq=s.correctness_seq)]


def _compare_muon(s: Settings) -> list[Step]:
    return [_compare("compare_muon", ["fsdp2_muon", "matrix_owner_muon", "matrix_owner_muon_library"], s),
            _compare("compare_muon_correctness", ["fsdp2_muon", "matrix_owner_muon"], s, "--correctness",
                     layers=s.correctness_layers, seq=s.correctness_seq)]


def _compare_adamw_vs_muon(s: Settings) -> list[Step]:
    return [_compare("compare_adamw_vs_muon", ["fsdp2", "matrix_owner_muon"], s)]


def _fully_shard_api(s: Settings) -> list[Step]:
    return [_compare("fully_shard_api", ["fsdp2", "matrix_default", "matrix_sgd"], s, "--correctness",
                     layers=s.correctness_layers, seq=s.correctness_seq)]


def _runtime_profile(s: Settings) -> list[Step]:
    modes = ("prefetch", "no_prefetch", "adaptive", "zero_copy", "saved_hooks", "matrix_owner_muon")
    return [Step(f"runtime_profile_{m}", _tool("runtime_profile", "--mode", m, "--device", "cuda", "--world-size",
                                               str(s.world_size), "--hidden", str(s.hidden), "--layers", str(min(s.layers, 8)),
                                               "--batch", str(max(s.batch, 2)), "--json", "--device-timeline"))
            for m in modes]


def _reserved_trace(s: Settings) -> list[Step]:
    return [_compare("reserved_trace", ["fsdp2", "matrix_default", "matrix_keep_storage"], s, "--memory-trace",
                     layers=max(s.large_layers))]


def _checkpoint_large(s: Settings) -> list[Step]:
    return [Step("checkpoint_large", _torchrun(s.world_size, 29531, "bench.py", "--gpus", str(s.world_size), "--config", "4",
                                               "--steps", str(s.steps), "--warmup", str(s.warmup), "--verify-reshard"))]


def _copyin(s: Settings) -> list[Step]:
    return [Step(f"microbench_{k}", _tool("compare_bench", "--microbench", k, "--device", "cuda", "--world-size", "1",
                                          "--hidden", str(s.hidden), "--layers", "1"))
            for k in ("copy_in", "materialize")]


def _comm(s: Settings) -> list[Step]:
    n = s.world_size
    return [Step("comm_bench_even", _torchrun(n, 29532, "-m", "matrix_fsdp_b200.tools.comm_bench", "--fused")),
            Step("comm_bench_owner", _torchrun(n, 29533, "-m", "matrix_fsdp_b200.tools.comm_bench", "--layout", "owner")),
            Step("comm_bench_without_multicast", _torchrun(n, 29534, "-m", "matrix_fsdp_b200.tools.comm_bench"),
                 env={"MFSDP_NVLS": "0"})]


def _group_sweep(s: Settings) -> list[Step]:
    out = []
    for depth in (0, 1, 2):
        mode = {0: "matrix_no_prefetch", 1: "matrix_default", 2: "matrix_prefetch2"}[depth]
        for t in range(s.trials):
            out.append(_compare(f"group_sweep_depth{depth}_trial{t}", [mode], s))
    return out


def _large(s: Settings) -> list[Step]:
    out = []
    for ws in s.large_world_sizes:
        for cfg in ("3", "4"):
            out.append(Step(f"large_cfg{cfg}_ws{ws}", _torchrun(ws, 29540 + ws, "bench.py", "--gpus", str(ws), "--config", cfg,
                                                               "--steps", str(s.steps), "--warmup", str(s.warmup))))
    return out


def _bench_arms(s: Settings) -> list[Step]:
    out = []
    for impl in ("reference", "ours"):
        for n in (1, 2, 4, 8):
            if n > max(s.world_size, 1):
                continue
            tail = ["bench.py", "--impl", impl, "--gpus", str(n), "--steps", "20", "--warmup", "5"]
            out.append(Step(f"bench_{impl}_n{n}", [PY, *tail] if n == 1 else _torchrun(n, 29550 + n, *tail)))
    return out


def _trace_report(s: Settings) -> list[Step]:
    n = s.world_size
    return (_comm(s) + [_compare("phase_adamw", ["fsdp2", "matrix_default"], s, "--memory-trace"),
                        _compare("phase_muon", ["fsdp2_muon", "matrix_owner_muon"], s, "--memory-trace")]
            + [Step("step_timeline", _torchrun(n, 29535, "bench.py", "--gpus", str(n), "--steps", "10", "--warmup", "3",
                                               "--timeline", "{report_dir}/step_timeline.md"))]
            + _runtime_profile(s)[:2])


def _all(s: Settings) -> list[Step]:
    return (_cuda_smoke(s) + _planner(s) + _compare_adamw(s) + _fully_shard_api(s) + _compare_muon(s)
            + _runtime_profile(s) + _reserved_trace(s) + _copyin(s))


BATCHES = {
    "cuda-smoke": (_cuda_smoke, "selected multi-GPU correctness tests"),
    "cuda-full": (_cuda_full, "every GPU test"),
    "planner": (_planner, "planner reports for the planner world sizes"),
    "compare-adamw": (_compare_adamw, "library FSDP vs this framework, AdamW, timing and correctness"),
    "compare-adamw-vs-muon": (_compare_adamw_vs_muon, "library FSDP AdamW vs the owner-layout Muon path"),
    "fully-shard-api": (_fully_shard_api, "public fully_shard API with plain torch optimizers"),
    "compare-muon": (_compare_muon, "library FSDP + Muon vs owner-layout Muon"),
    "trace-report": (_trace_report, "communication / phase / memory / timeline report into one directory"),
    "runtime-profile": (_runtime_profile, "event-level runtime profiles, one per runtime mode"),
    "reserved-trace": (_reserved_trace, "per-rank allocated / reserved memory on the large model"),
    "checkpoint-large": (_checkpoint_large, "largest config with the save -> reshard -> load check"),
    "copyin": (_copyin, "gradient copy-in and materialisation microbenchmarks"),
    "comm": (_comm, "collective and fused compute+collective bandwidth"),
    "group-sweep": (_group_sweep, "isolated trials over prefetch depths"),
    "large": (_large, "opt-in large-model sweeps over world sizes"),
    "bench-arms": (_bench_arms, "bench.py for both arms at N = 1, 2, 4, 8"),
    "all": (_all, "cuda-smoke, planner, compare-adamw, fully-shard-api, compare-muon, runtime-profile, reserved-trace, copyin"),
}


def steps_of(batch: str, settings: Settings, report_dir: str) -> list[Step]:
    if batch not in BATCHES:
        raise KeyError(f"unknown batch {batch!r}; known: {', '.join(BATCHES)}")
    steps = BATCHES[batch][0](settings)
    for st in steps:
        st.argv = [a.replace("{report_dir}", report_dir) for a in st.argv]
    return steps


def render_script(batch: str, settings: Settings, report_dir: str) -> str:
    lines = ["#!/usr/bin/env bash", f"# batch: {batch} -- {BATCHES[batch][1]}", "set -uo pipefail",
             f"cd {shlex.quote(str(ROOT))}", f"mkdir -p {shlex.quote(report_dir)}", "failed=0"]
    for st in steps_of(batch, settings, report_dir):
        lines.append(f"echo '+ {st.name}'; {st.shell(report_dir)} || {{ echo '  failed: {st.name}'; failed=$((failed+1)); }}")
    lines.append(f"{shlex.quote(PY)} -m matrix_fsdp_b200.tools.regression summarize {shlex.quote(report_dir)} "
                 f"> {shlex.quote(report_dir)}/summary.txt")
    lines.append('exit $failed')
    return "\n".join(lines) + "\n"


def run_batch(batch: str, settings: Settings, report_dir: str) -> int:
    os.makedirs(report_dir, exist_ok=True)
    failed = 0
    for st in steps_of(batch, settings, report_dir):
        t0 = time.perf_counter()
        log = os.path.join(report_dir, f"{st.name}.log")
        with open(log, "w") as f:
            try:
                rc = subprocess.run(st.argv, cwd=ROOT, stdout=f, stderr=subprocess.STDOUT, timeout=st.timeout,
                                    env={**os.environ, **st.env}).returncode
            except subprocess.TimeoutExpired:
                rc = 124
        failed += rc != 0
        print(f"{st.name:40s} rc={rc:<4d} {time.perf_counter() - t0:7.1f}s  {log}")
    text = format_summary(summarize_report(Path(report_dir)))
    Path(report_dir, "summary.txt").write_text(text)
    print(text)
    return 1 if failed else 0


# ----------------------------------------------------------------------------------------------
# preflight
# ----------------------------------------------------------------------------------------------
def _local_checks() -> list[tuple[str, list[str]]]:
    tools = sorted(str(p.relative_to(ROOT)) for p in (ROOT / "matrix_fsdp_b200" / "tools").glob("*.py"))
    return [("python_compile", [PY, "-m", "py_compile", "bench.py", *tools]),
            ("cpu_summary_tests", [PY, "-m", "pytest", "tests/test_summary_and_facade.py", "tests/test_tools.py", "-q", "-m",
                                   "not gpu"]),
            ("kernel_library", [PY, "-m", "matrix_fsdp_b200.tools.regression", "package"])]


def prepare(out_dir: str, settings: Settings, *, local_checks: bool = True,
            batches: tuple[str, ...] = ("bench-arms", "compare-adamw", "compare-muon", "trace-report", "runtime-profile",
                                        "copyin")) -> dict:
    """Write ``commands.sh`` (every step of ``batches``, in order, then the summary) and
    ``preflight_summary.txt`` (settings, policy, outcome of the CPU checks) into ``out_dir``."""
    os.makedirs(out_dir, exist_ok=True)
    summary = [f"{k}={v}" for k, v in vars(settings).items()]
    summary += ["", "policy:", "- AdamW: library FSDP vs matrix_default", "- Muon: library FSDP + Muon vs owner layouts",
                "- collectives: peer-memory kernels (NVSwitch multicast when present), library collectives as the named modes",
                ""]
    results = {}
    if local_checks:
        for name, cmd in _local_checks():
            try:
                p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=1800)
                rc, tail = p.returncode, (p.stdout + p.stderr).strip().splitlines()[-1:] or [""]
            except subprocess.TimeoutExpired:
                rc, tail = 124, ["timeout"]
            results[name] = rc
            summary.append(f"== {name} == rc={rc} {tail[0][:120]}")
    report_dir = os.path.join(out_dir, "report")
    script = ["#!/usr/bin/env bash", "set -uo pipefail", f"cd {shlex.quote(str(ROOT))}",
              f"mkdir -p {shlex.quote(report_dir)}"]
    n_steps = 0
    for b in batches:
        script.append(f"# ---- {b}: {BATCHES[b][1]}")
        for st in steps_of(b, settings, report_dir):
            script.append(st.shell(report_dir) + f" || echo 'failed: {st.name}'")
            n_steps += 1
    script.append(f"{shlex.quote(PY)} -m matrix_fsdp_b200.tools.regression summarize {shlex.quote(report_dir)} "
                  f"| tee {shlex.quote(report_dir)}/summary.txt")
    cmd_file = os.path.join(out_dir, "commands.sh")
    Path(cmd_file).write_text("\n".join(script) + "\n")
    os.chmod(cmd_file, 0o755)
    summary.append(f"commands={cmd_file} steps={n_steps}")
    Path(out_dir, "preflight_summary.txt").write_text("\n".join(summary) + "\n")
    return {"commands": cmd_file, "steps": n_steps, "local_checks": results}


# ----------------------------------------------------------------------------------------------
# log -> tables
# ----------------------------------------------------------------------------------------------
def _json_lines(path: Path) -> list[dict]:
    out = []
    for ln in path.read_text(errors="replace").splitlines():
        ln = ln.strip()
        if ln.startswith("{") and ln.endswith("}"):
            try:
                obj = json.loads(ln)
            except json.JSONDecodeError:
                continue
            if isinstance(obj, dict):
                out.append(obj)
    return out


_LIBRARY_ROW = {"matrix_owner_muon": "fsdp2_muon", "matrix_owner_muon_library": "fsdp2_muon"}


def summarize_report(report_dir: Path) -> dict:
    """Collect the result lines of every ``*.log`` under ``report_dir`` into four row lists."""
    phase, memory, comm, timeline, bench, failures = [], [], [], [], [], []
    for log in sorted(report_dir.glob("*.log")):
        rows = _json_lines(log)
        by_mode = {r["mode"]: r for r in rows if "mode" in r and "step_ms" in r}
        for r in rows:
            if "mode" in r and "unavailable" in r:
                failures.append({"log": log.name, "mode": r["mode"], "why": r["unavailable"]})
            elif "mode" in r and "step_ms" in r:
                ph = r.get("phase_ms", {})
                base = by_mode.get(_LIBRARY_ROW.get(r["mode"], "fsdp2"))
                row = {"log": log.name, "mode": r["mode"], "step_ms": r["step_ms"], "fwd_ms": ph.get("forward"),
                       "bwd_ms": ph.get("backward"), "opt_ms": ph.get("step", ph.get("optimizer")), "peak_mb": r.get("peak_mb"),
                       "vs_library": (base["step_ms"] / r["step_ms"]) if base and base is not r and r["step_ms"] else None,
                       "max_param_diff": r.get("max_param_diff_vs_eager")}
                phase.append(row)
                for tag, snap in (r.get("memory_trace") or {}).items():
                    memory.append({"log": log.name, "mode": r["mode"], "phase": tag, **snap})
                for kind, d in ((r.get("events") or {}).get("by_collective") or {}).items():
                    if isinstance(d, dict):
                        timeline.append({"log": log.name, "mode": r["mode"], "collective": kind, **d})
            elif "transport" in r and "op" in r:
                comm.append({"log": log.name, **r})
            elif "op" in r and "fused_ms" in r:
                comm.append({"log": log.name, "transport": "fused", "ms": r["fused_ms"], **r})
            elif "metric" in r and "value" in r:
                bench.append({"log": log.name, "impl": r.get("impl", "ours"), "n_gpus": r.get("n_gpus"),
                              "config": (r.get("config") or {}).get("model"), "value": r["value"], "unit": r.get("unit"),
                              "ms_per_step": r.get("ms_per_step"), "e2e": (r.get("e2e") or {}).get("value"),
                              "peak_mb": r.get("peak_mem_mb")})
        lines = log.read_text(errors="replace").splitlines()
        if any(ln.startswith("Traceback (most recent call last)") for ln in lines):
            failures.append({"log": log.name, "mode": "", "why": "traceback in log"})
        elif lines and " failed" in lines[-1]:
            failures.append({"log": log.name, "mode": "", "why": lines[-1].strip("= ")[:100]})
    # both arms side by side
    arms = []
    ours = {(b["config"], b["n_gpus"]): b for b in bench if b["impl"] != "reference"}
    for b in bench:
        if b["impl"] == "reference" and (b["config"], b["n_gpus"]) in ours:
            o = ours[(b["config"], b["n_gpus"])]
            arms.append({"config": b["config"], "n_gpus": b["n_gpus"], "reference": b["value"], "ours": o["value"],
                         "ratio": o["value"] / b["value"] if b["value"] else None})
    return {"report_dir": str(report_dir), "phase": phase, "memory": memory, "comm": comm, "timeline": timeline,
            "bench": bench, "arms": arms, "failures": failures}


def _fmt(v) -> str:
    if v is None:
        return "-"
    if isinstance(v, float):
        return f"{v:.3f}" if abs(v) < 1000 else f"{v:.0f}"
    return str(v)


def _table(headers: tuple[str, ...], rows: list[dict]) -> list[str]:
    cells = [[_fmt(r.get(h)) for h in headers] for r in rows]
    widths = [max(len(h), *(len(c[i]) for c in cells)) if cells else len(h) for i, h in enumerate(headers)]
    line = lambda vals: "  ".join(v.ljust(w) for v, w in zip(vals, widths)).rstrip()   # noqa: E731
    return [line(headers), line(tuple("-" * w for w in widths)), *(line(c) for c in cells)]


def format_summary(summary: dict) -> str:
    out = [f"report: {summary['report_dir']}"]
    sections = (("step time by mode", ("log", "mode", "step_ms", "fwd_ms", "bwd_ms", "opt_ms", "peak_mb", "vs_library",
                                       "max_param_diff"), "phase"),
                ("bench.py", ("log", "impl", "config", "n_gpus", "value", "unit", "ms_per_step", "e2e", "peak_mb"), "bench"),
                ("both arms", ("config", "n_gpus", "reference", "ours", "ratio"), "arms"),
                ("collectives", ("log", "transport", "op", "ms", "recv_gb_per_s", "frac_of_measured_nvlink_770",
                                 "unfused_ms", "frac_of_roofline"), "comm"),
                ("device time of collectives", ("log", "mode", "collective", "count", "device_ms", "exposed_ms",
                                                "gbytes_per_s"), "timeline"),
                ("memory", ("log", "mode", "phase", "allocated_mb", "max_allocated_mb", "reserved_mb"), "memory"),
                ("failures", ("log", "mode", "why"), "failures"))
    for title, headers, key in sections:
        rows = summary.get(key) or []
        if rows:
            out += ["", f"== {title} ==", *_table(headers, rows)]
    return "\n".join(out) + "\n"
