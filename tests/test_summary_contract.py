"""Summaries of units, schedulers and event logs, one property per test: synthetic event lists pin the
aggregation rules, short real runs pin what the runtime actually records.  The reference's counterpart is
test/fsdp/test_summary.py (13 tests)."""
import pytest
import torch
from torch import nn

from matrix_fsdp_b200 import configure_optimizer, fully_shard
from matrix_fsdp_b200.api import reset_shared_owner_planners
from matrix_fsdp_b200.parallel.runtime_event import RuntimeEvent
from matrix_fsdp_b200.parallel.summary import (format_param_group_summary, format_runtime_events, summarize_param_groups,
                                               summarize_runtime_events, summarize_scheduler)


def _ev(name, seq, ms=1.0, unit="param_group_0", **kw):
    return RuntimeEvent(name=name, unit=unit, sequence=seq, lifecycle_state="sharded", duration_ms=ms, **kw)


def _trained(n=3, steps=1, **opt_kw):
    reset_shared_owner_planners()
    torch.manual_seed(0)
    model = nn.Sequential(*[nn.Linear(8, 8) for _ in range(n)])
    for blk in model:
        fully_shard(blk)
    opt = configure_optimizer(model, "adamw", lr=1e-2, **opt_kw)
    for _ in range(steps):
        model(torch.randn(2, 8)).sum().backward()
        opt.step()
        opt.zero_grad()
    return model, opt


# ------------------------------------------------------------------------------------------ synthetic logs
def test_events_are_ordered_by_sequence_before_they_are_aggregated():
    events = [_ev("post_forward", 2), _ev("pre_forward", 1), _ev("init", 0)]
    s = summarize_runtime_events(events)
    assert s["num_events"] == 3 and set(s["by_name"]) == {"init", "pre_forward", "post_forward"}


def test_stats_carry_count_total_mean_and_max():
    s = summarize_runtime_events([_ev("reshard", 0, 1.0), _ev("reshard", 1, 3.0), _ev("reshard", 2, 2.0)])
    st = s["by_name"]["reshard"]
    assert st == {"count": 3, "total_ms": 6.0, "mean_ms": 2.0, "max_ms": 3.0}


def test_categories_group_names_by_prefix_and_unknown_names_fall_into_other():
    s = summarize_runtime_events([_ev("start_unshard:pre_forward", 0), _ev("wait_unshard:pre_forward", 1),
                                  _ev("start_reduce_scatter", 2), _ev("something_new", 3)])
    assert s["by_category"]["unshard"]["count"] == 2 and s["by_category"]["reduce"]["count"] == 1
    assert s["by_category"]["other"]["count"] == 1


def test_phase_of_an_unshard_follows_its_reason():
    s = summarize_runtime_events([_ev("unshard", 0, reason="pre_forward"), _ev("unshard", 1, reason="pre_backward"),
                                  _ev("unshard", 2, reason="backward_prefetch")])
    assert s["by_phase"]["forward"]["count"] == 1 and s["by_phase"]["backward"]["count"] == 2


def test_phases_split_forward_backward_optimizer_and_init():
    names = ["init", "pre_forward", "start_unshard:forward_prefetch", "post_forward", "pre_backward",
             "finalize_backward", "start_reduce_scatter", "wait_reduce_scatter", "reshard_before_optimizer"]
    s = summarize_runtime_events([_ev(n, i) for i, n in enumerate(names)])
    assert {k: v["count"] for k, v in s["by_phase"].items()} == {"init": 1, "forward": 3, "backward": 4, "optimizer": 1}


def test_collective_rows_are_keyed_by_kind_backend_and_impl():
    kw = dict(collective_kind="all_gather", collective_backend="torch_dist", collective_bytes=100, collective_count=1)
    events = [_ev("start_unshard:pre_forward", 0, collective_impl="padded_all_gather", **kw),
              _ev("start_unshard:pre_forward", 1, collective_impl="all_gather_into_tensor", **kw),
              _ev("start_unshard:pre_forward", 2, collective_impl="padded_all_gather", **kw)]
    rows = summarize_runtime_events(events)["by_collective"]
    assert rows["all_gather/torch_dist/padded_all_gather"]["count"] == 2
    assert rows["all_gather/torch_dist/padded_all_gather"]["bytes"] == 200
    assert rows["all_gather/torch_dist/all_gather_into_tensor"]["count"] == 1


def test_issue_and_wait_host_time_are_kept_apart():
    kw = dict(collective_kind="reduce_scatter", collective_backend="torch_dist", collective_impl="padded_reduce_scatter",
              collective_bytes=64, collective_count=1)
    row = summarize_runtime_events([_ev("start_reduce_scatter", 0, 0.5, **kw), _ev("wait_reduce_scatter", 1, 2.0, **kw)]
                                   )["by_collective"]["reduce_scatter/torch_dist/padded_reduce_scatter"]
    assert row["issue_host_ms"] == 0.5 and row["wait_host_ms"] == 2.0 and row["host_ms"] == 2.5
    assert row["count"] == 1 and row["bytes"] == 64                   # the wait is not a second launch


def test_device_time_and_bandwidth_come_from_events_that_were_timed_on_the_device():
    kw = dict(collective_kind="all_gather", collective_backend="peer", collective_impl="push", collective_bytes=2_000_000,
              collective_count=1)
    rows = summarize_runtime_events([_ev("start_unshard:pre_forward", 0, device_ms=1.0, **kw),
                                     _ev("start_unshard:pre_forward", 1, device_ms=None, **kw)])["by_collective"]
    row = rows["all_gather/peer/push"]
    assert row["device_timed"] == 1 and row["device_ms"] == 1.0
    assert row["device_gbytes_per_s"] == pytest.approx(2.0)          # 2 MB in 1 ms, the untimed launch left out


def test_untimed_collectives_report_no_bandwidth():
    kw = dict(collective_kind="all_gather", collective_backend="torch_dist", collective_impl="x", collective_bytes=10,
              collective_count=1)
    row = summarize_runtime_events([_ev("start_unshard:pre_forward", 0, **kw)])["by_collective"]["all_gather/torch_dist/x"]
    assert row["device_gbytes_per_s"] is None and row["device_timed"] == 0


def test_prefetch_and_workspace_reuse_are_counted_per_collective():
    kw = dict(collective_kind="all_gather", collective_backend="torch_dist", collective_impl="x", collective_bytes=10,
              collective_count=1)
    row = summarize_runtime_events([_ev("start_unshard:forward_prefetch", 0, prefetched=True, workspace_reused=True, **kw),
                                    _ev("start_unshard:pre_forward", 1, **kw)])["by_collective"]["all_gather/torch_dist/x"]
    assert row["prefetched"] == 1 and row["workspace_reused"] == 1 and row["max_bytes"] == 10


def test_high_water_marks_are_maxima_over_the_log():
    s = summarize_runtime_events([_ev("unshard", 0, active_full_param_buffers=1, grad_bucket_bytes=10),
                                  _ev("unshard", 1, active_full_param_buffers=3, pending_reduce_scatter_count=2),
                                  _ev("reshard", 2, active_full_param_buffers=2, grad_bucket_bytes=40)])
    assert s["max_active_full_param_buffers"] == 3 and s["max_pending_reduce_scatter"] == 2
    assert s["max_grad_bucket_bytes"] == 40


def test_prefetched_unshards_and_recompute_skips_are_counted():
    s = summarize_runtime_events([_ev("unshard", 0, prefetched=True), _ev("unshard", 1), _ev("start_unshard:x", 2, prefetched=True),
                                  _ev("pre_forward_recompute_skip", 3, recompute=True)])
    assert s["prefetched_unshards"] == 1 and s["recompute_skips"] == 1


def test_per_unit_table_separates_the_units():
    s = summarize_runtime_events([_ev("init", 0, unit="param_group_0"), _ev("init", 1, unit="param_group_1"),
                                  _ev("reshard", 2, unit="param_group_1")])
    assert s["by_unit"]["param_group_0"]["count"] == 1 and s["by_unit"]["param_group_1"]["count"] == 2


def test_an_empty_log_summarises_to_zeroes():
    s = summarize_runtime_events([])
    assert s["num_events"] == 0 and s["by_name"] == {} and s["max_active_full_param_buffers"] == 0
    assert "runtime events: 0" in format_runtime_events([])


# ------------------------------------------------------------------------------------------ real runs
def test_a_real_step_records_every_phase_for_every_unit():
    model, _ = _trained()
    s = summarize_runtime_events(model)
    assert set(s["by_phase"]) >= {"init", "forward", "backward"}
    assert len(s["by_unit"]) == 3
    for name in ("pre_forward", "post_forward", "pre_backward_unshard", "finalize_backward", "start_reduce_scatter"):
        assert s["by_name"][name]["count"] == 3, name


def test_a_list_of_units_and_the_module_give_the_same_summary():
    model, _ = _trained()
    units = [b._matrix_fsdp_param_group for b in model]
    assert summarize_runtime_events(units)["num_events"] == summarize_runtime_events(model)["num_events"]
    events = [e for u in units for e in u.runtime_events]
    assert summarize_runtime_events(events)["by_name"].keys() == summarize_runtime_events(model)["by_name"].keys()


def test_tracing_can_be_switched_off_per_unit():
    from matrix_fsdp_b200 import matrix_fully_shard

    reset_shared_owner_planners()
    m = nn.Linear(4, 4)
    matrix_fully_shard(m, runtime_trace_enabled=False)
    opt = configure_optimizer(m, "sgd", lr=0.1)
    m(torch.randn(2, 4)).sum().backward()
    opt.step()
    assert m._matrix_fsdp_param_group.runtime_events == []
    assert summarize_runtime_events(m)["num_events"] == 0


def test_param_group_summary_reports_layout_options_and_memory():
    model, _ = _trained()
    rows = summarize_param_groups(model)
    assert [r["name"] for r in rows] == [b._matrix_fsdp_param_group.name for b in model]
    r = rows[0]
    assert r["world_size"] == 1 and r["state"] == "sharded" and r["num_params"] == 2 and r["total_numel"] == 72
    assert r["shard_sizes"] == (72,) and r["transport"] == "local" and r["full_buffer_mode"] == "alias"
    assert r["backward_reduce_strategy"] == "bucket_reduce_scatter" and r["param_gather_strategy"] == "auto"
    assert r["memory"]["local_shard_bytes"] == 72 * 4 and r["num_events"] > 0 and r["scheduler"] is not None


def test_formatted_summaries_name_every_unit_and_the_tables():
    model, _ = _trained()
    text = format_param_group_summary(model)
    for b in model:
        assert b._matrix_fsdp_param_group.name in text
    log = format_runtime_events(model, limit=3)
    assert "by category:" in log and "by name:" in log and "by phase:" in log
    assert len([line for line in log.split("by name:")[1].split("by phase:")[0].splitlines() if line.strip()]) == 3


def test_scheduler_summary_hit_ratio_counts_prefetched_gathers():
    model, _ = _trained(n=4, steps=2)
    s = summarize_scheduler(model)
    assert s["num_units"] == 4 and 0.0 < s["prefetch_hit_ratio"] <= 1.0
    assert s["pending_reduces"] == 0 and s["active_full_param_buffers"] == 0
    model, _ = _trained(n=4, steps=2, max_unsharded_prefetch_units=0)
    assert summarize_scheduler(model)["prefetch_hit_ratio"] == 0.0


def test_scheduler_summary_is_none_without_a_scheduler():
    reset_shared_owner_planners()
    m = nn.Linear(4, 4)
    fully_shard(m)
    assert summarize_scheduler(m) is None or summarize_scheduler(m)["num_units"] == 1
