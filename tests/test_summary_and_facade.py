"""Observability (unit summaries, runtime event aggregation), the optimizer state manager and the FSDP2-shaped
state-dict facade, all at world size 1."""
import copy

import torch
from torch import nn

from matrix_fsdp_b200 import configure_optimizer, fully_shard
from matrix_fsdp_b200.api import reset_shared_owner_planners
from matrix_fsdp_b200.parallel.summary import (format_param_group_summary, format_runtime_events,
                                               summarize_param_groups, summarize_runtime_events)
from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups


def _model(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Sequential(nn.Linear(6, 8), nn.GELU()), nn.Sequential(nn.Linear(8, 4)))


def _trained(policy=None, optimizer="adamw"):
    reset_shared_owner_planners()
    model = _model()
    for block in model:
        fully_shard(block, optimizer_policy=policy)
    opt = configure_optimizer(model, optimizer, lr=1e-2)
    for s in range(2):
        x = torch.randn(3, 6, generator=torch.Generator().manual_seed(s))
        model(x).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
    return model, opt


def test_param_group_summary_fields():
    model, _ = _trained()
    rows = summarize_param_groups(model)
    assert len(rows) == 2
    r = rows[0]
    assert r["state"] == "sharded" and r["world_size"] == 1 and r["num_params"] == 2
    assert r["total_numel"] == 6 * 8 + 8 == r["local_numel"] and r["transport"] == "local"
    comm = r["communication"]
    assert comm["param_buffer_type"] in ("static", "elastic") and "effective_param_gather_backend" in comm
    assert r["scheduler"] is not None and r["num_events"] > 0
    text = format_param_group_summary(model)
    assert rows[0]["name"] in text and "planner=" in text


def test_runtime_event_aggregation():
    model, _ = _trained()
    summary = summarize_runtime_events(model)
    names = summary["by_name"] if "by_name" in summary else summary
    flat = str(summary)
    for expected in ("pre_forward", "unshard", "reshard_after_forward", "pre_backward_unshard"):
        assert expected in flat, expected
    assert summary.get("num_events", 1) > 0
    unit = collect_param_groups(model)[0]
    ev = unit.runtime_events[0]
    assert ev.sequence >= 0 and ev.name and ev.unit == unit.name and ev.lifecycle_state
    seqs = [e.sequence for u in collect_param_groups(model) for e in u.runtime_events]
    assert len(set(seqs)) == len(seqs)                                # one global sequence across units
    text = format_runtime_events(model, limit=5)
    assert text.startswith("runtime events:") and "by category:" in text
    assert len(text.splitlines()) < len(format_runtime_events(model).splitlines())
    assert "pre_forward" in format_runtime_events(model)
    quiet = collect_param_groups(model)[1]
    quiet.runtime_trace_enabled = False
    before = len(quiet.runtime_events)
    model(torch.randn(2, 6)).sum().backward()
    assert len(quiet.runtime_events) == before


def test_optimizer_state_manager_lists_local_state():
    model, opt = _trained()
    st = opt.local_state_summary()
    infos = [info for _, info in opt.state_manager.iter_param_infos()]
    assert {i.fqn for i in infos} >= {"0.weight", "0.bias"} and all(i.component == "optimizer" for i in infos)
    assert all(i.local_numel == i.param_numel for i in infos)               # one rank: every parameter is local and whole
    tensors = list(opt.state_manager.iter_state_tensors())
    assert len(tensors) >= 2 * len(infos)                             # exp_avg and exp_avg_sq per parameter
    assert st is not None


def test_fsdp2_shaped_state_dict_facade_round_trip():
    from matrix_fsdp_b200 import (get_model_state_dict, get_optimizer_state_dict, get_state_dict, set_model_state_dict,
                                  set_optimizer_state_dict)
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions

    model, opt = _trained()
    full = get_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True))
    eager = _model()
    assert set(full) == set(eager.state_dict())
    assert all(full[k].shape == v.shape for k, v in eager.state_dict().items())
    msd, osd = get_state_dict(model, opt)
    reset_shared_owner_planners()
    other = _model(seed=4)
    for block in other:
        fully_shard(block)
    opt2 = configure_optimizer(other, "adamw", lr=1e-2)
    set_model_state_dict(other, msd)
    set_optimizer_state_dict(other, opt2, osd)
    for a, b in zip(collect_param_groups(model), collect_param_groups(other)):
        assert torch.equal(a.flat_buffer.local_shard, b.flat_buffer.local_shard)
    x = torch.randn(3, 6, generator=torch.Generator().manual_seed(7))
    for m, o in ((model, opt), (other, opt2)):
        m(x).pow(2).mean().backward()
        o.step()
        o.zero_grad()
    for a, b in zip(collect_param_groups(model), collect_param_groups(other)):
        assert torch.equal(a.flat_buffer.local_shard, b.flat_buffer.local_shard)
    assert get_optimizer_state_dict(model, opt).keys() == get_optimizer_state_dict(other, opt2).keys()
    # loading the gathered full tensors into an eager copy reproduces the sharded model's forward
    eager.load_state_dict(get_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True)))
    assert torch.allclose(eager(x), model(x), atol=1e-6)


def test_unit_debug_accessors():
    model, _ = _trained(policy="mixed_muon_adamw", optimizer="mixed_muon_adamw")
    unit = collect_param_groups(model)[0]
    assert unit.owner_ranks("0.weight") == (0,)
    assert set(unit.params_for_rank(0)) == {"0.weight", "0.bias"}
    segs = unit.rank_segments_for_param("0.bias", 0)
    assert len(segs) == 1 and segs[0].numel == 8
    sd = unit.state_dict()
    assert sd["total_numel"] == 56 and sd["param_fqns"] == ("0.weight", "0.bias") or "param_shard" in sd
    unit.unshard()
    assert unit.state.value == "unsharded" and model[0][0].weight.shape == (8, 6)
    unit.reshard()
    assert unit.state.value == "sharded"


def test_full_optimizer_state_dict_is_keyed_by_parameter_name():
    from matrix_fsdp_b200 import get_optimizer_state_dict
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions

    model, opt = _trained()
    full = get_optimizer_state_dict(model, opt, options=MatrixStateDictOptions(full_state_dict=True, cpu_offload=True))
    comp = full["optimizer"]
    names = dict(model.named_parameters()).keys()
    assert set(comp["state"]) == set(names)
    entry = comp["state"]["0.0.weight"]
    assert entry["exp_avg"].shape == (8, 6) and entry["exp_avg_sq"].shape == (8, 6) and entry["step"] == 2.0
    assert entry["exp_avg"].device.type == "cpu" and comp["param_groups"][0]["lr"] == 1e-2
    mixed_model, mixed = _trained(policy="mixed_muon_adamw", optimizer="mixed_muon_adamw")
    full2 = get_optimizer_state_dict(mixed_model, mixed, options=MatrixStateDictOptions(full_state_dict=True))
    assert set(full2) == {"muon", "adamw"}
    assert "momentum_buffer" in full2["muon"]["state"]["0.0.weight"]
    assert "exp_avg" in full2["adamw"]["state"]["0.0.bias"]


def test_event_summary_has_phase_collective_and_scheduler_tables():
    import torch.nn as nn

    from matrix_fsdp_b200 import (configure_optimizer, format_runtime_events, fully_shard, summarize_param_groups,
                                  summarize_runtime_events, summarize_scheduler)
    from matrix_fsdp_b200.api import reset_shared_owner_planners

    reset_shared_owner_planners()
    torch.manual_seed(0)
    model = nn.Sequential(nn.Sequential(nn.Linear(6, 6), nn.Tanh()), nn.Sequential(nn.Linear(6, 3)))
    for blk in model:
        fully_shard(blk)
    opt = configure_optimizer(model, "adamw", lr=1e-2)
    for _ in range(2):
        model(torch.randn(4, 6)).sum().backward()
        opt.step()
        opt.zero_grad()
    s = summarize_runtime_events(model)
    assert {"forward", "backward"} <= set(s["by_phase"])
    assert s["by_phase"]["backward"]["collectives"] >= 2 and s["by_phase"]["forward"]["count"] > 0
    coll = next(v for k, v in s["by_collective"].items() if k.startswith("reduce_scatter"))
    assert {"issue_host_ms", "wait_host_ms", "device_ms", "exposed_ms", "prefetched", "max_bytes"} <= set(coll)
    sched = summarize_scheduler(model)
    assert sched["num_units"] == 2 and sched["forward_prefetch_depth"] == 1
    assert sched["counters"]["iterations"] == 2 and "pool" in sched
    text = format_runtime_events(model)
    assert "by phase:" in text and "collectives:" in text
    row = summarize_param_groups(model)[0]
    assert row["full_buffer_mode"] in ("alias", "storage_resize") and "transport_detail" in row
    assert len(row["communication"]) >= 20
