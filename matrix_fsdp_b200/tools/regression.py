"""Runbooks as one CLI: isolated test runs, isolated benchmark runs and the package / kernel-library check.

    python -m matrix_fsdp_b200.tools.regression tests [--gpu] [--timeout 900]
    python -m matrix_fsdp_b200.tools.regression bench --configs 2 5s --gpus 1 2 --trials 2 [--impl ours reference]
    python -m matrix_fsdp_b200.tools.regression package
    python -m matrix_fsdp_b200.tools.regression batch <name> [--dry-run] [--report-dir DIR]   (named GPU batches)
    python -m matrix_fsdp_b200.tools.regression plan [--out-dir DIR]                          (no-GPU preflight + commands.sh)
    python -m matrix_fsdp_b200.tools.regression summarize DIR [--json]                        (logs -> tables)

``tests`` runs every test file in its own interpreter (a crash or a hang in one file cannot take the
others with it) and prints one line per file; ``bench`` runs ``bench.py`` once per (config, N, trial) in
a fresh process, collects the JSON lines and prints a median table; ``package`` builds the kernel
library for sm_100a, checks that every exported entry point the Python side binds is present, and
imports the public API; ``batch`` / ``plan`` / ``summarize`` are described in ``gpu_runbook.py``.  Child processes are ended by their own timeout only (never by name).

Parity: scripts/run_test.sh, scripts/run_isolated_gpu_benchmark.py, scripts/summarize_gpu_comm_report.py,
scripts/check_package.sh and scripts/build_cuda_kernels.sh of the reference.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _run(cmd: list[str], timeout: float, env: dict | None = None) -> tuple[int, str, float]:
    t0 = time.perf_counter()
    try:
        p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=timeout, env=env)
        return p.returncode, p.stdout + p.stderr, time.perf_counter() - t0
    except subprocess.TimeoutExpired as exc:
        out = (exc.stdout or b"").decode(errors="replace") if isinstance(exc.stdout, bytes) else (exc.stdout or "")
        return 124, out + "\n[timeout]", time.perf_counter() - t0


def cmd_tests(args) -> int:
    files = sorted(glob.glob(os.path.join(ROOT, "tests", "test_*.py")))
    marker = "gpu" if args.gpu else "not gpu"
    failed = 0
    for f in files:
        rc, out, dt = _run([sys.executable, "-m", "pytest", f, "-x", "-q", "-m", marker], args.timeout)
        tail = [ln for ln in out.strip().splitlines() if ln.strip()][-1:] or [""]
        status = "ok" if rc in (0, 5) else ("timeout" if rc == 124 else f"rc={rc}")   # 5: nothing selected
        failed += status not in ("ok",)
        print(f"{os.path.basename(f):40s} {status:8s} {dt:7.1f}s  {tail[0][:90]}")
    print(f"{len(files) - failed}/{len(files)} files passed")
    return 1 if failed else 0


def _bench_cmd(config: str, n: int, impl: str, steps: int, warmup: int, port: int) -> list[str]:
    tail = ["bench.py", "--gpus", str(n), "--config", config, "--impl", impl, "--steps", str(steps), "--warmup", str(warmup)]
    if n == 1:
        return [sys.executable] + tail
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
            "127.0.0.1", "--master-port", str(port)] + tail


def cmd_bench(args) -> int:
    rows = []
    for impl in args.impl:
        for config in args.configs:
            for n in args.gpus:
                vals, ms = [], []
                for trial in range(args.trials):
                    rc, out, _ = _run(_bench_cmd(config, n, impl, args.steps, args.warmup, 29500 + trial), args.timeout)
                    line = next((ln for ln in reversed(out.splitlines()) if ln.startswith("{")), None)
                    if rc != 0 or line is None:
                        print(f"[{impl} cfg{config} N={n} trial {trial}] failed rc={rc}", file=sys.stderr)
                        continue
                    rec = json.loads(line)
                    if "value" in rec:
                        vals.append(rec["value"])
                        ms.append(rec["ms_per_step"])
                if vals:
                    rows.append({"impl": impl, "config": config, "n_gpus": n, "trials": len(vals),
                                 "tokens_per_s_median": statistics.median(vals), "ms_per_step_median": statistics.median(ms)})
    for r in rows:
        print(json.dumps(r))
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


def cmd_package(args) -> int:
    from ..ops import build, lib

    so = str(build.build(verbose=False))
    import matrix_fsdp_b200 as pkg
    from ..ops import attention, moe_kernels  # noqa: F401  (register their entry points)
    from ..parallel import peer  # noqa: F401

    handle = lib.load(required=True)
    missing = [name for name in lib._SIGNATURES if not hasattr(handle, name)]

    exported = [n for n in getattr(pkg, "__all__", []) if not hasattr(pkg, n)]
    print(json.dumps({"library": so, "entry_points": len(lib._SIGNATURES),
                      "missing_entry_points": missing, "public_names": len(getattr(pkg, "__all__", [])),
                      "unresolved_public_names": exported}))
    return 1 if (missing or exported) else 0


def _settings(args):
    from .gpu_runbook import Settings

    base = Settings()
    kw = {}
    for name, default in vars(base).items():
        v = getattr(args, name, None)
        if v is not None:
            kw[name] = tuple(v) if isinstance(default, tuple) else v
    return Settings(**kw)


def _add_settings(p) -> None:
    from .gpu_runbook import Settings

    for name, default in vars(Settings()).items():
        flag = "--" + name.replace("_", "-")
        if isinstance(default, tuple):
            p.add_argument(flag, type=int, nargs="+", default=None)
        else:
            p.add_argument(flag, type=int, default=None)


def cmd_batch(args) -> int:
    from . import gpu_runbook as rb

    report_dir = args.report_dir or os.path.join(ROOT, "benchmark_results", f"{args.name}_{time.strftime('%Y%m%d_%H%M%S')}")
    if args.dry_run:
        print(rb.render_script(args.name, _settings(args), report_dir), end="")
        return 0
    return rb.run_batch(args.name, _settings(args), report_dir)


def cmd_plan(args) -> int:
    from . import gpu_runbook as rb

    out_dir = args.out_dir or os.path.join(ROOT, "benchmark_results", f"gpu_preflight_{time.strftime('%Y%m%d_%H%M%S')}")
    res = rb.prepare(out_dir, _settings(args), local_checks=not args.no_local_checks)
    print(json.dumps(res))
    return 1 if any(res["local_checks"].values()) else 0


def cmd_summarize(args) -> int:
    from pathlib import Path

    from . import gpu_runbook as rb

    summary = rb.summarize_report(Path(args.report_dir))
    print(json.dumps(summary) if args.json else rb.format_summary(summary), end="" if not args.json else "\n")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    t = sub.add_parser("tests")
    t.add_argument("--gpu", action="store_true")
    t.add_argument("--timeout", type=float, default=900.0)
    b = sub.add_parser("bench")
    b.add_argument("--configs", nargs="+", default=["2"])
    b.add_argument("--gpus", type=int, nargs="+", default=[1])
    b.add_argument("--impl", nargs="+", default=["ours"], choices=["ours", "reference"])
    b.add_argument("--trials", type=int, default=1)
    b.add_argument("--steps", type=int, default=10)
    b.add_argument("--warmup", type=int, default=3)
    b.add_argument("--timeout", type=float, default=900.0)
    b.add_argument("--out", default=None)
    sub.add_parser("package")
    from .gpu_runbook import BATCHES

    bt = sub.add_parser("batch", description="\n".join(f"{k:24s}{v[1]}" for k, v in BATCHES.items()),
                        formatter_class=argparse.RawDescriptionHelpFormatter)
    bt.add_argument("name", choices=sorted(BATCHES))
    bt.add_argument("--dry-run", action="store_true", help="print the batch as a shell script")
    bt.add_argument("--report-dir", default=None)
    _add_settings(bt)
    pl = sub.add_parser("plan")
    pl.add_argument("--out-dir", default=None)
    pl.add_argument("--no-local-checks", action="store_true")
    _add_settings(pl)
    sm = sub.add_parser("summarize")
    sm.add_argument("report_dir")
    sm.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    return {"tests": cmd_tests, "bench": cmd_bench, "package": cmd_package, "batch": cmd_batch, "plan": cmd_plan,
            "summarize": cmd_summarize}[args.cmd](args)


if __name__ == "__main__":
    raise SystemExit(main())
