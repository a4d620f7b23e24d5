"""Expert parallelism on gloo ranks, one (experts, top-k, optimizer) per case: three steps of the EP model (experts
split over the ranks, dense parts sharded) equal the single-process model that keeps every expert local and sees
the ranks' sequences as data-parallel micro-batches; plus checkpoint resume with experts split over the ranks,
with AdamW, SGD and Muon on the experts.  All cases of a world size share one spawn.  The reference trains its
EP model in test/fsdp/test_deepseek_v3_ep_train.py:472-563 (3 tests, GPU only)."""
import json
import os
import tempfile
import traceback

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_ranks

# experts, top-k, optimizer
TRAIN_CASES = ["E4-K1-adamw", "E4-K2-adamw", "E4-K3-adamw", "E8-K2-adamw", "E8-K4-adamw", "E4-K2-sgd", "E8-K3-sgd",
               "E4-K2-sgdm", "E2-K1-adamw", "E2-K2-adamw", "E4-K2-adamw-skewed", "E8-K2-sgd-skewed"]
CLIP_CASES = ["clip-2", "clip-1", "clip-inf"]
RESUME_CASES = ["resume-E4-K2-adamw", "resume-E4-K2-sgd", "resume-E4-K2-mixed_muon_adamw", "resume-E8-K3-adamw"]
TRAIN4_CASES = ["E4-K2-adamw", "E8-K2-adamw", "E8-K3-sgd", "E8-K2-adamw-skewed"]
RESUME4_CASES = ["resume-E8-K2-mixed_muon_adamw"]


def _cfg(n_experts, top_k):
    from matrix_fsdp_b200.models.moe import MoEConfig

    return MoEConfig(vocab_size=96, hidden=32, n_layers=2, n_heads=2, head_dim=16, n_experts=n_experts, expert_ffn=24,
                     top_k=top_k, max_seq_len=32)


def _tokens(world):
    return torch.randint(0, 96, (world, 13), generator=torch.Generator().manual_seed(0))


def _parse(name):
    e, k, opt = name.removeprefix("resume-").split("-")
    return int(e[1:]), int(k[1:]), opt


def _train_case(rank, world, name):
    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.models.moe import MoEModel, configure_moe_optimizer, shard_moe
    from matrix_fsdp_b200.parallel.expert_parallel import reset_contexts

    skewed = name.endswith("-skewed")
    n_experts, top_k, opt_kind = _parse(name.removesuffix("-skewed"))
    reset_shared_owner_planners()
    reset_contexts()
    cfg = _cfg(n_experts, top_k)
    torch.manual_seed(0)
    model = MoEModel(cfg)
    torch.manual_seed(0)
    ref = MoEModel(cfg, ep_group=False)
    el = n_experts // world
    assert model.layers[0].experts.w_down.shape[0] == el
    if skewed:
        # tokens whose features sum to a positive number go to the first top_k experts, the others to the next
        # top_k, nobody to the rest (no ties anywhere): ranks that own only the rest receive no token at all
        with torch.no_grad():
            for m in (model, ref):
                for layer in m.layers:
                    layer.router.weight.zero_()
                    layer.router.weight[:top_k] = 50.0
                    layer.router.weight[top_k:2 * top_k] = -50.0
    shard_moe(model)
    momentum = 0.9 if opt_kind == "sgdm" else 0.0
    hyper = dict(lr=1e-2, betas=(0.9, 0.95)) if opt_kind == "adamw" else dict(lr=0.05, momentum=momentum)
    opt = configure_moe_optimizer(model, "adamw" if opt_kind == "adamw" else "sgd", **hyper)
    ref_params = [p for n, p in ref.named_parameters() if ".experts." not in n] + ref.expert_parameters()
    ropt = torch.optim.AdamW(ref_params, lr=1e-2, weight_decay=0.0, betas=(0.9, 0.95)) if opt_kind == "adamw" \
        else torch.optim.SGD(ref_params, lr=0.05, momentum=momentum)
    toks = _tokens(world)
    for step in range(3):
        mine = toks[rank:rank + 1]
        loss = model(mine[:, :-1], mine[:, 1:])
        loss.backward()
        losses = []
        for r in range(world):
            l_r = ref(toks[r:r + 1, :-1], toks[r:r + 1, 1:])
            (l_r / world).backward()
            losses.append(l_r.detach())
        assert torch.allclose(loss.detach(), losses[rank], atol=2e-5), (step, float(loss), float(losses[rank]))
        for p in model.expert_parameters():                # EP sums all ranks' tokens; the DP mean needs 1 / world
            p.grad.div_(world)
        opt.step()
        opt.zero_grad()
        ropt.step()
        ropt.zero_grad()
    for a, b in zip(model.layers, ref.layers):
        lo, hi = rank * el, (rank + 1) * el
        assert torch.allclose(a.experts.w_down, b.experts.w_down[lo:hi], atol=3e-5)
        assert torch.allclose(a.experts.w_gate_up, b.experts.w_gate_up[lo:hi], atol=3e-5)


def _clip_case(rank, world, name):
    """Global-norm clipping over dense shards plus expert gradients equals clipping the all-local model."""
    import math

    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.models.moe import MoEModel, clip_moe_grad_norm_, configure_moe_optimizer, shard_moe
    from matrix_fsdp_b200.parallel.expert_parallel import reset_contexts

    norm_type = math.inf if name.endswith("inf") else float(name.rsplit("-", 1)[1])
    reset_shared_owner_planners()
    reset_contexts()
    cfg = _cfg(4, 2)
    torch.manual_seed(0)
    model = MoEModel(cfg)
    torch.manual_seed(0)
    ref = MoEModel(cfg, ep_group=False)
    shard_moe(model)
    opt = configure_moe_optimizer(model, "sgd", lr=0.05)
    ref_params = [p for n, p in ref.named_parameters() if ".experts." not in n] + ref.expert_parameters()
    ropt = torch.optim.SGD(ref_params, lr=0.05)
    toks = _tokens(world)
    el = cfg.n_experts // world
    for max_norm_factor in (0.3, 10.0):                       # one step that clips, one that does not
        mine = toks[rank:rank + 1]
        model(mine[:, :-1], mine[:, 1:]).backward()
        for r in range(world):
            (ref(toks[r:r + 1, :-1], toks[r:r + 1, 1:]) / world).backward()
        rtotal = torch.nn.utils.get_total_norm([p.grad for p in ref_params], norm_type)
        max_norm = float(rtotal) * max_norm_factor
        total = clip_moe_grad_norm_(model, max_norm, norm_type, expert_scale=1.0 / world)
        assert torch.allclose(total, rtotal, rtol=1e-4), (float(total), float(rtotal))
        torch.nn.utils.clip_grad_norm_(ref_params, max_norm, norm_type)
        for p in model.expert_parameters():                   # what expert_scale stood for
            p.grad.div_(world)
        opt.step()
        opt.zero_grad()
        ropt.step()
        ropt.zero_grad()
    for a, b in zip(model.layers, ref.layers):
        lo, hi = rank * el, (rank + 1) * el
        assert torch.allclose(a.experts.w_down, b.experts.w_down[lo:hi], atol=3e-5)
        assert torch.allclose(a.experts.w_gate_up, b.experts.w_gate_up[lo:hi], atol=3e-5)
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions, get_model_state_dict

    full = get_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True))
    for n, p in ref.named_parameters():
        if ".experts." not in n:
            assert torch.allclose(full[n], p.detach(), atol=3e-5), n


def _resume_case(rank, world, name, base_dir):
    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.models.moe import (MoEModel, configure_moe_optimizer, load_moe_checkpoint, save_moe_checkpoint,
                                             shard_moe)
    from matrix_fsdp_b200.parallel.expert_parallel import reset_contexts

    n_experts, top_k, opt_kind = _parse(name)
    cfg = _cfg(n_experts, top_k)
    toks = _tokens(world)[rank:rank + 1]
    mixed = opt_kind == "mixed_muon_adamw"

    def make(seed):
        reset_shared_owner_planners()
        torch.manual_seed(seed)
        m = MoEModel(cfg)
        shard_moe(m, optimizer_policy="mixed_muon_adamw" if mixed else None)
        kw = dict(lr=1e-2, muon_lr=0.02) if mixed else (dict(lr=0.05, momentum=0.9) if opt_kind == "sgd" else dict(lr=1e-2))
        return m, configure_moe_optimizer(m, opt_kind, **kw)

    def step(m, o):
        m(toks[:, :-1], toks[:, 1:]).backward()
        o.step()
        o.zero_grad()

    reset_contexts()
    model, opt = make(0)
    for _ in range(2):
        step(model, opt)
    directory = os.path.join(base_dir, name)
    if rank == 0:
        os.makedirs(directory, exist_ok=True)
    dist.barrier()
    save_moe_checkpoint(model, directory, optimizer=opt)
    step(model, opt)
    expect = model(toks[:, :-1], toks[:, 1:]).detach()
    twin, topt = make(3)                                      # other weights: everything has to come from the files
    load_moe_checkpoint(twin, directory, optimizer=topt)
    step(twin, topt)
    got = twin(toks[:, :-1], toks[:, 1:]).detach()
    assert torch.allclose(got, expect, atol=1e-5), (float(got), float(expect))
    for a, b in zip(model.layers, twin.layers):
        assert torch.allclose(a.experts.w_down, b.experts.w_down, atol=1e-6)


def _reshard_model(opt_kind, seed):
    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.models.moe import MoEModel, configure_moe_optimizer, shard_moe
    from matrix_fsdp_b200.parallel.expert_parallel import reset_contexts

    reset_shared_owner_planners()
    reset_contexts()
    mixed = opt_kind == "mixed_muon_adamw"
    torch.manual_seed(seed)
    m = MoEModel(_cfg(8, 2))
    shard_moe(m, optimizer_policy="mixed_muon_adamw" if mixed else None)
    kw = {"adamw": dict(lr=1e-2), "sgd": dict(lr=0.05, momentum=0.9), "mixed_muon_adamw": dict(lr=1e-2, muon_lr=0.02)}
    return m, configure_moe_optimizer(m, opt_kind, **kw[opt_kind])


def _expert_state_rows(model, opt):
    """{name: [n_local, ...] tensor} of everything the expert optimizer and the experts hold, per expert row."""
    ex_opt = opt.experts
    out = {}
    for i, p in enumerate(model.expert_parameters()):
        out[f"w{i}"] = p.detach().clone()
        out[f"master{i}"] = ex_opt.masters[i].clone()
        if ex_opt.kind == "adamw":
            out[f"exp_avg{i}"], out[f"exp_avg_sq{i}"] = ex_opt.exp_avg[i].clone(), ex_opt.exp_avg_sq[i].clone()
        elif ex_opt.kind == "sgd":
            out[f"momentum{i}"] = ex_opt.momentum_buffer[i].clone()
        else:
            out[f"momentum{i}"] = torch.stack([ex_opt.muon.state[s]["momentum_buffer"] for s in ex_opt._slices[i]])
    return out


def _reshard_write_case(rank, world, name, base_dir):
    """Two ranks train, save, and leave every expert's state gathered by global id for the readers to check."""
    from matrix_fsdp_b200.models.moe import save_moe_checkpoint

    opt_kind = name.split("-", 1)[1]
    model, opt = _reshard_model(opt_kind, 0)
    toks = _tokens(world)[rank:rank + 1]
    for _ in range(2):
        model(toks[:, :-1], toks[:, 1:]).backward()
        opt.step()
        opt.zero_grad()
    directory = os.path.join(base_dir, f"reshard-{opt_kind}")
    if rank == 0:
        os.makedirs(directory, exist_ok=True)
    dist.barrier()
    save_moe_checkpoint(model, directory, optimizer=opt)
    rows = _expert_state_rows(model, opt)
    gathered = [None] * world
    dist.all_gather_object(gathered, rows)
    if rank == 0:
        torch.save({k: torch.cat([g[k] for g in gathered]) for k in rows}, os.path.join(directory, "all_experts.pt"))
    dist.barrier()


def _reshard_read_case(rank, world, name, base_dir):
    """Another expert-parallel size reads the files: every rank finds its experts' rows, and trains on."""
    from matrix_fsdp_b200.models.moe import load_moe_checkpoint

    opt_kind = name.split("-", 1)[1]
    directory = os.path.join(base_dir, f"reshard-{opt_kind}")
    model, opt = _reshard_model(opt_kind, 5)
    with pytest.raises(ValueError):
        load_moe_checkpoint(model, directory, optimizer=opt)              # another layout: has to be asked for
    model, opt = _reshard_model(opt_kind, 5)
    load_moe_checkpoint(model, directory, optimizer=opt, allow_reshard=True)
    want = torch.load(os.path.join(directory, "all_experts.pt"))
    el = 8 // world
    for k, v in _expert_state_rows(model, opt).items():
        assert torch.equal(v, want[k][rank * el:(rank + 1) * el]), k
    toks = _tokens(world)[rank:rank + 1]
    before = model.layers[0].experts.w_down.detach().clone()
    loss = model(toks[:, :-1], toks[:, 1:])
    loss.backward()
    opt.step()
    opt.zero_grad()
    assert torch.isfinite(loss) and not torch.equal(model.layers[0].experts.w_down, before)


def _worker(rank, world, out_path, names, base_dir):
    results = {}
    for name in names:
        try:
            if name.startswith("resume-"):
                _resume_case(rank, world, name, base_dir)
            elif name.startswith("clip-"):
                _clip_case(rank, world, name)
            elif name.startswith("reshardwrite-"):
                _reshard_write_case(rank, world, name, base_dir)
            elif name.startswith("reshardread-"):
                _reshard_read_case(rank, world, name, base_dir)
            else:
                _train_case(rank, world, name)
            mine = ""
        except Exception:
            mine = traceback.format_exc()
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        results[name] = "\n".join(f"--- rank {r} ---\n{t}" for r, t in enumerate(gathered) if t)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(results, f)


def _spawn(world, names, base_dir):
    path = os.path.join(base_dir, f"outcomes-{world}.json")
    run_ranks(_worker, world, path, names, base_dir, timeout=600.0)
    with open(path) as f:
        return json.load(f)


RESHARD_KINDS = ("adamw", "sgd", "mixed_muon_adamw")
RESHARD_WRITE = [f"reshardwrite-{k}" for k in RESHARD_KINDS]
RESHARD_READ = [f"reshardread-{k}" for k in RESHARD_KINDS]


@pytest.fixture(scope="module")
def shared_dir():
    with tempfile.TemporaryDirectory() as tmp:
        yield tmp


@pytest.fixture(scope="module")
def outcomes(shared_dir):
    return _spawn(2, TRAIN_CASES + RESUME_CASES + CLIP_CASES + RESHARD_WRITE, shared_dir)


@pytest.fixture(scope="module")
def outcomes4(shared_dir, outcomes):                  # after the two-rank job: it reads what that one wrote
    return _spawn(4, TRAIN4_CASES + RESUME4_CASES + RESHARD_READ, shared_dir)


@pytest.mark.parametrize("case", TRAIN_CASES + RESUME_CASES + CLIP_CASES)
def test_two_rank_expert_parallel(outcomes, case):
    assert case in outcomes, "the worker did not reach this case"
    assert not outcomes[case], outcomes[case]


@pytest.mark.parametrize("case", TRAIN4_CASES + RESUME4_CASES)
def test_four_rank_expert_parallel(outcomes4, case):
    assert case in outcomes4, "the worker did not reach this case"
    assert not outcomes4[case], outcomes4[case]


@pytest.mark.parametrize("kind", RESHARD_KINDS)
def test_expert_checkpoint_moves_from_two_ranks_to_four(outcomes, outcomes4, kind):
    assert not outcomes[f"reshardwrite-{kind}"], outcomes[f"reshardwrite-{kind}"]
    assert not outcomes4[f"reshardread-{kind}"], outcomes4[f"reshardread-{kind}"]
