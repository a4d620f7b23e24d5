"""CLI tools run on tiny CPU configs and produce parseable output."""
import json

from matrix_fsdp_b200.tools import device_api_probe, planner_report, runtime_profile


def test_planner_report_cli(capsys):
    assert planner_report.main(["--layers", "2", "--world-size", "4", "--json"]) == 0
    out = capsys.readouterr().out
    payload = json.loads(out.strip().splitlines()[-1])
    assert len(payload["units"]) == 2 and len(payload["rank_units"]) == 4
    assert planner_report.main(["--model", "mlp", "--policy", "balanced", "--world-size", "2", "--layers", "1"]) == 0
    assert "candidate" in capsys.readouterr().out


def test_runtime_profile_single_and_two_ranks(capsys):
    assert runtime_profile.main(["--world-size", "1", "--json", "--layers", "2"]) == 0
    one = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert one["step_ms"] > 0 and one["events"]["num_events"] > 0
    assert runtime_profile.main(["--world-size", "2", "--mode", "matrix_owner_muon", "--json"]) == 0
    two = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert two["world_size"] == 2 and two["units"][0]["planner_name"] == "matrix_owner_tail_role_greedy"
    assert any(k.startswith("all_gather") for k in two["events"]["by_collective"])


def test_device_probe():
    p = device_api_probe.probe()
    assert "kernel_library_present" in p and "nccl_version" in p


def test_planner_bench_reports_balance(capsys):
    import json

    from matrix_fsdp_b200.tools import planner_bench

    assert planner_bench.main(["--hidden", "256", "--layers", "3", "--world", "2", "4", "--repeat", "1"]) == 0
    rows = [json.loads(ln) for ln in capsys.readouterr().out.strip().splitlines()]
    assert {r["strategy"] for r in rows} == set(planner_bench.STRATEGIES)
    for r in rows:
        assert r["owned_imbalance"] >= 1.0 and r["ms_per_block"] > 0
    best = min(r["owned_imbalance"] for r in rows if r["world"] == 4)
    assert best < 1.6


def test_regression_package_check(capsys):
    import json

    from matrix_fsdp_b200.tools import regression

    assert regression.main(["package"]) == 0
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec["missing_entry_points"] == [] and rec["unresolved_public_names"] == []


def test_bench_reshard_verification_on_four_cpu_ranks():
    """bench.py --verify-reshard: HSDP 2 x 2 run, save, load resharded onto dp_shard = 4, equal checksums."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", "29541", "bench.py", "--gpus", "4", "--config", "4t", "--device", "cpu",
           "--steps", "1", "--warmup", "1", "--verify-reshard"]
    env = dict(os.environ, GLOO_SOCKET_IFNAME="lo", OMP_NUM_THREADS="1")
    p = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stderr[-2000:]
    line = next(ln for ln in reversed(p.stdout.splitlines()) if ln.startswith("{"))
    rec = json.loads(line)
    assert rec["config"]["parallelism"] == "dp_replicate2xdp_shard2" and rec["n_gpus"] == 4
    assert rec["reshard"]["checksums_equal"] and rec["reshard"]["tensors_compared"] > 20
    assert rec["reshard"]["target_parallelism"] == "dp_shard4"


def test_compare_bench_against_fsdp2_and_eager(capsys):
    import json

    from matrix_fsdp_b200.tools import compare_bench

    rc = compare_bench.main(["--world-size", "2", "--device", "cpu", "--modes", "matrix_default", "matrix_owner_muon",
                             "fsdp2", "--hidden", "32", "--layers", "2", "--heads", "2", "--seq", "8", "--steps", "2",
                             "--warmup", "1", "--correctness"])
    assert rc == 0
    rows = {r["mode"]: r for r in map(json.loads, capsys.readouterr().out.strip().splitlines())}
    assert set(rows) == {"matrix_default", "matrix_owner_muon", "fsdp2"}
    for mode, r in rows.items():
        if "unavailable" in r:
            assert mode == "fsdp2"                       # only the library mode may be missing in a torch build
            continue
        assert r["step_ms"] > 0 and set(r["phase_ms"]) == {"zero_grad", "forward", "backward", "step"}
        assert r["max_loss_diff_vs_eager"] < 1e-5 and r["max_param_diff_vs_eager"] < 1e-4, (mode, r)


def test_nccl_feature_probe_with_fabricated_headers(tmp_path, monkeypatch):
    """Header / version logic of the NCCL probe, on header files written by the test."""
    import torch

    from matrix_fsdp_b200.tools.device_api_probe import probe_nccl_features

    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(device_api_probe, "_include_dirs", lambda extra: [__import__("pathlib").Path(p) for p in extra])
    old, new = tmp_path / "old", tmp_path / "new"
    old.mkdir(), new.mkdir()
    (old / "nccl.h").write_text("typedef struct ncclDevComm ncclDevComm;\n")
    (new / "nccl.h").write_text("typedef struct ncclDevComm ncclDevComm;\nncclResult_t ncclDevCommCreate();\n")
    (new / "nccl_device").mkdir()
    (new / "nccl_device" / "gin.h").write_text("struct ncclGin {};\n#define NCCL_GIN_SIGNAL_INC 1\n")

    # a runtime older than the device API: the headers declare it, yet it is not ready, and the reason says why
    monkeypatch.setattr(torch.cuda.nccl, "version", lambda: (2, 27, 5))
    p = probe_nccl_features(extra_include_dirs=(str(old),), library="")
    f = p["features"]["device_api"]
    assert p["nccl_version"] == (2, 27, 5) and f["declared_in_headers"] and not f["runtime_new_enough"] and not f["ready"]
    assert "older" in p["reason"]

    # new runtime, headers without GIN: device API ready, GIN not
    monkeypatch.setattr(torch.cuda.nccl, "version", lambda: 22809)     # packed integer form
    p = probe_nccl_features(extra_include_dirs=(str(old),), library="")
    assert p["nccl_version"] == (2, 28, 9)
    assert p["features"]["device_api"]["ready"] and not p["features"]["gin"]["ready"] and "gin" in p["reason"]

    # new runtime and GIN headers in the nccl_device/ subtree: everything visible
    monkeypatch.setattr(torch.cuda.nccl, "version", lambda: "2.30.4")
    p = probe_nccl_features(extra_include_dirs=(str(new),), library="")
    assert all(v["ready"] for v in p["features"].values()) and "visible" in p["reason"]
    assert any(h.endswith("gin.h") for h in p["headers"])

    # no headers at all
    p = probe_nccl_features(extra_include_dirs=(str(tmp_path / "nowhere"),), library="")
    assert not p["features"]["device_api"]["ready"] and "No NCCL headers" in p["reason"]


def test_runbook_batches_render_and_plan(tmp_path, capsys):
    from matrix_fsdp_b200.tools import gpu_runbook as rb
    from matrix_fsdp_b200.tools import regression

    s = rb.Settings(world_size=8, layers=4)
    for name in rb.BATCHES:
        steps = rb.steps_of(name, s, str(tmp_path / "rep"))
        assert steps and len({st.name for st in steps}) == len(steps), name
        script = rb.render_script(name, s, str(tmp_path / "rep"))
        assert script.count("timeout ") == len(steps) and "summarize" in script
    assert regression.main(["batch", "trace-report", "--dry-run", "--world-size", "2", "--report-dir", str(tmp_path / "r")]) == 0
    out = capsys.readouterr().out
    assert "--nproc-per-node=2" in out and f"--timeline {tmp_path / 'r'}/step_timeline.md" in out
    assert regression.main(["plan", "--out-dir", str(tmp_path / "pre"), "--no-local-checks", "--world-size", "4"]) == 0
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    text = open(res["commands"]).read()
    assert res["steps"] == text.count(" || echo 'failed:") and "bench.py --impl reference --gpus 4" in text
    assert "world_size=4" in (tmp_path / "pre" / "preflight_summary.txt").read_text()


def test_runbook_summariser_builds_tables_from_logs(tmp_path, capsys):
    from matrix_fsdp_b200.tools import gpu_runbook as rb
    from matrix_fsdp_b200.tools import regression

    rep = tmp_path / "rep"
    rep.mkdir()
    (rep / "compare_adamw.log").write_text("\n".join([
        "NCCL version 2.28.9+cuda12.9",
        json.dumps({"mode": "fsdp2", "step_ms": 20.0, "phase_ms": {"forward": 6.0, "backward": 12.0, "step": 2.0},
                    "peak_mb": 900.0}),
        json.dumps({"mode": "matrix_default", "step_ms": 16.0, "phase_ms": {"forward": 5.0, "backward": 10.0, "step": 1.0},
                    "peak_mb": 800.0, "max_param_diff_vs_eager": 1e-3,
                    "memory_trace": {"after_backward": {"allocated_mb": 1.0, "max_allocated_mb": 2.0, "reserved_mb": 3.0}}}),
        json.dumps({"mode": "matrix_row", "unavailable": "ValueError: nope"})]))
    (rep / "comm_bench_even.log").write_text("\n".join([
        json.dumps({"transport": "peer", "op": "all_gather", "ms": 0.2, "recv_gb_per_s": 600.0,
                    "frac_of_measured_nvlink_770": 0.78}),
        json.dumps({"op": "rs+adamw", "unfused_ms": 0.5, "fused_ms": 0.3, "frac_of_roofline": 0.8})]))
    (rep / "bench_reference_n2.log").write_text(json.dumps(
        {"metric": "tokens_per_s", "value": 100.0, "unit": "tok/s", "impl": "reference", "n_gpus": 2, "ms_per_step": 10.0,
         "config": {"model": "m"}}))
    (rep / "bench_ours_n2.log").write_text(json.dumps(
        {"metric": "tokens_per_s", "value": 150.0, "unit": "tok/s", "n_gpus": 2, "ms_per_step": 6.6, "config": {"model": "m"},
         "e2e": {"value": 140.0}}))
    (rep / "runtime_profile_prefetch.log").write_text(json.dumps(
        {"mode": "prefetch", "step_ms": 3.0, "peak_mb": 10.0,
         "events": {"by_collective": {"all_gather/ag_pull": {"count": 4, "device_ms": 0.4, "exposed_ms": 0.1}}}}))
    (rep / "broken.log").write_text("Traceback (most recent call last):\n  boom\n")
    s = rb.summarize_report(rep)
    by_mode = {r["mode"]: r for r in s["phase"]}
    assert abs(by_mode["matrix_default"]["vs_library"] - 1.25) < 1e-9 and by_mode["fsdp2"]["vs_library"] is None
    assert by_mode["matrix_default"]["opt_ms"] == 1.0 and by_mode["fsdp2"]["fwd_ms"] == 6.0
    assert s["arms"] == [{"config": "m", "n_gpus": 2, "reference": 100.0, "ours": 150.0, "ratio": 1.5}]
    assert {c["op"] for c in s["comm"]} == {"all_gather", "rs+adamw"}
    assert s["memory"][0]["phase"] == "after_backward" and s["timeline"][0]["collective"] == "all_gather/ag_pull"
    assert {f["log"] for f in s["failures"]} == {"broken.log", "compare_adamw.log"}
    assert regression.main(["summarize", str(rep)]) == 0
    text = capsys.readouterr().out
    for title in ("step time by mode", "both arms", "collectives", "device time of collectives", "memory", "failures"):
        assert f"== {title} ==" in text
    assert "1.250" in text and "1.500" in text


def test_planner_report_units_models_and_json(capsys):
    """Every model kind and unit granularity plans; the JSON form carries the per-unit candidate rows and the
    per-rank totals, and the totals are the sums of the selected rows."""
    for model in planner_report.MODELS:
        assert planner_report.main(["--model", model, "--layers", "2", "--hidden", "128", "--heads", "2", "--experts", "4",
                                    "--world-size", "4", "--selected-only"]) == 0
        assert "== rank load ==" in capsys.readouterr().out
    assert planner_report.main(["--model", "transformer", "--unit", "linear", "--policy", "balanced", "--layers", "1",
                                "--hidden", "128", "--world-size", "2", "--format", "json"]) == 0
    d = json.loads(capsys.readouterr().out)
    assert len(d["units"]) == 5                      # qkv, proj, fc1, fc2 and the two norms as <root>
    assert d["units"][-1]["unit"] == "<root>" and all(len(u["rows"]) > 1 for u in d["units"][:-1])
    for key, field in (("rank_units", "rank_units"), ("rank_memory_bytes", "rank_memory_bytes"),
                       ("rank_comm_bytes", "rank_comm_bytes")):
        sums = [sum(u["rows"][0][field][r] for u in d["units"]) for r in range(2)]
        assert list(d[key]) == sums
    # a stateful owner planner sees the units in order: its running load is monotone and ends at the totals
    assert planner_report.main(["--unit", "block", "--layers", "3", "--hidden", "128", "--world-size", "4",
                                "--owner-assignment", "rotate", "--rotation-strategy", "round_robin", "--format", "json"]) == 0
    d = json.loads(capsys.readouterr().out)
    loads = [u["cumulative_rank_units"] for u in d["units"]]
    assert list(loads[-1]) == list(d["rank_units"]) and all(a <= b for x, y in zip(loads, loads[1:]) for a, b in zip(x, y))
    assert d["imbalance"]["units"] >= 1.0 and sum(d["rank_ns_flops"]) > 0
    # the whole model as one unit under the model-wide assignment
    assert planner_report.main(["--unit", "model", "--owner-assignment", "model_wide", "--layers", "2", "--hidden", "128",
                                "--world-size", "4", "--selected-only"]) == 0
    assert "<model>" in capsys.readouterr().out


def test_runtime_profile_models_units_and_output_file(tmp_path, capsys):
    out = tmp_path / "profile.json"
    assert runtime_profile.main(["--world-size", "2", "--model", "transformer", "--hidden", "32", "--heads", "4",
                                 "--activation-checkpoint", "--dtype", "bfloat16", "--mode", "no_prefetch",
                                 "--format", "json", "--output", str(out)]) == 0
    assert capsys.readouterr().out.strip() == ""
    d = json.loads(out.read_text())
    assert d["model"] == "transformer" and d["dtype"] == "bfloat16" and d["activation_checkpoint"] and len(d["step_ms_each"]) == 2
    assert d["scheduler"]["counters"]["forward_prefetch_issued"] == 0
    # one unit per Linear plus one root unit per block for the norms; optimizer override; text form
    assert runtime_profile.main(["--world-size", "1", "--model", "transformer_split_qkv", "--unit", "linear", "--layers", "2",
                                 "--hidden", "32", "--heads", "4", "--optimizer", "sgd",
                                 "--max-active-full-param-buffers", "3"]) == 0
    text = capsys.readouterr().out
    assert "optimizer=sgd" in text and text.count("param_group_") >= 2 * 7


def test_runbook_runs_a_batch_and_writes_the_summary(tmp_path, monkeypatch, capsys):
    """``run_batch`` executes every step in its own process, keeps one log per step and ends with the tables."""
    import sys

    from matrix_fsdp_b200.tools import gpu_runbook as rb

    row = {"mode": "matrix_default", "step_ms": 2.0, "phase_ms": {"forward": 1.0, "backward": 0.8, "step": 0.2}, "peak_mb": 1.0}
    ok = rb.Step("fake_compare", [sys.executable, "-c", f"import json; print(json.dumps({row!r}))"])
    bad = rb.Step("fake_failure", [sys.executable, "-c", "raise SystemExit(3)"])
    monkeypatch.setitem(rb.BATCHES, "fake", (lambda s: [ok, bad], "two fabricated steps"))
    rc = rb.run_batch("fake", rb.Settings(), str(tmp_path / "rep"))
    out = capsys.readouterr().out
    assert rc == 1 and "fake_compare" in out and "rc=3" in out
    assert (tmp_path / "rep" / "fake_compare.log").read_text().startswith("{")
    summary = (tmp_path / "rep" / "summary.txt").read_text()
    assert "== step time by mode ==" in summary and "matrix_default" in summary


def test_compare_bench_modes_run_and_match_eager_on_two_cpu_ranks(capsys):
    """A cross-section of the comparison bench's runtime modes on 2 Gloo ranks: every mode reports a step time,
    none is unavailable, parameters after the steps equal the eager model's, and the full gradients gathered
    by parameter name were checked."""
    from matrix_fsdp_b200.tools import compare_bench

    modes = ["matrix_default", "matrix_row", "matrix_owner_muon", "matrix_zero_copy_grads", "matrix_saved_tensor_hooks",
             "matrix_per_param_reduce", "matrix_all_reduce_gather", "matrix_adaptive_prefetch", "matrix_fused_reduce_update",
             "fsdp2"]
    assert compare_bench.main(["--device", "cpu", "--world-size", "2", "--hidden", "32", "--heads", "2", "--layers", "2",
                               "--seq", "8", "--steps", "1", "--warmup", "1", "--correctness", "--modes", *modes]) == 0
    rows = [json.loads(ln) for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
    assert [r["mode"] for r in rows] == modes
    for r in rows:
        assert "unavailable" not in r and r["step_ms"] > 0, r
        assert r["max_param_diff_vs_eager"] < 1e-4 and r["max_loss_diff_vs_eager"] < 1e-4, r
    checked = [r for r in rows if "full_grad_check" in r]
    assert len(checked) >= 5 and all(c["full_grad_check"]["max_abs_diff"] < 1e-4 and c["full_grad_check"]["params_compared"] > 0 for c in checked)
    assert all(set(r["phase_ms"]) >= {"forward", "backward", "step"} for r in rows)


def test_selfcheck_runs_its_checks_on_two_ranks(capsys):
    import json

    from matrix_fsdp_b200.tools import selfcheck

    assert selfcheck.main(["--ranks", "2", "--steps", "2", "--json"]) == 0
    result = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert result["ok"] and result["ranks"] == 2 and len(result["reports"]) == 2
    names = [c["name"] for c in result["reports"][0]["checks"]]
    assert "re-sharded checkpoint restores the parameters bit for bit" in names and all(
        c["ok"] for rep in result["reports"] for c in rep["checks"])
    text = selfcheck.format_result(result)
    assert "RESULT: all checks held" in text and "param_group_0" in text
    broken = dict(result, ok=False, reports=[dict(result["reports"][0], error="Traceback: boom"), result["reports"][1]])
    assert "FAILED" in selfcheck.format_result(broken) and "boom" in selfcheck.format_result(broken)
