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
