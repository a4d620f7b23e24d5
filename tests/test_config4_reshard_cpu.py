"""BASELINE config 4 in miniature on 4 gloo ranks: a Llama decoder trained with mixed Muon / AdamW on an HSDP
2 x 2 mesh is saved with ``save_matrix_dcp`` and loaded, resharded, onto a flat dp_shard = 4 mesh; parameters and
optimizer state must come across bitwise, and both runs must continue identically."""
import os
import tempfile

import torch
import torch.distributed as dist

from dist_utils import run_ranks


def _build(mesh_kind: str):
    from torch.distributed.device_mesh import init_device_mesh

    from matrix_fsdp_b200 import DataParallelMeshDims
    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.models.llama import LlamaConfig, LlamaModel, shard_llama
    from matrix_fsdp_b200.optim import configure_optimizer

    reset_shared_owner_planners()
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=96, hidden=32, n_layers=2, n_heads=2, head_dim=16, ffn=48, activation_checkpointing=True,
                      max_seq_len=16)
    model = LlamaModel(cfg)
    if mesh_kind == "hsdp":
        mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("dp_replicate", "dp_shard"))
        dims = DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate")
    else:
        mesh = init_device_mesh("cpu", (4,), mesh_dim_names=("dp_shard",))
        dims = None
    shard_llama(model, mesh=mesh, dp_mesh_dims=dims, optimizer_policy="mixed_muon_adamw")
    opt = configure_optimizer(model, "mixed_muon_adamw", muon_lr=0.02, adamw_lr=3e-3, muon_momentum=0.95,
                              muon_ns_steps=5, muon_adjust_lr_fn="original", weight_decay=0.1)
    return model, opt


def _step(model, opt, step: int):
    # every rank sees the same batch, so the HSDP run and the flat run average identical gradients
    g = torch.Generator().manual_seed(1000 + step)
    tok = torch.randint(0, 96, (2, 9), generator=g)
    loss = model(tok[:, :-1], tok[:, 1:])
    loss.backward()
    opt.step()
    opt.zero_grad()
    return loss.detach()


def _full_state(model, opt):
    """Full (unsharded) parameters and optimizer tensors keyed by FQN, assembled on every rank."""
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions, get_model_state_dict, get_optimizer_state_dict

    o = MatrixStateDictOptions(full_state_dict=True)
    return get_model_state_dict(model, options=o), get_optimizer_state_dict(model, opt, options=o)


def _flatten(d, prefix=""):
    out = {}
    for k, v in d.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict):
            out.update(_flatten(v, key + "/"))
        elif isinstance(v, torch.Tensor):
            out[key] = v
    return out


def _worker(rank, world, directory):
    from matrix_fsdp_b200 import load_matrix_dcp, save_matrix_dcp

    model, opt = _build("hsdp")
    for s in range(3):
        _step(model, opt, s)
    save_matrix_dcp(model, directory, optimizer=opt)
    params_a, optim_a = _full_state(model, opt)
    loss_a = _step(model, opt, 3)

    model_b, opt_b = _build("flat")
    load_matrix_dcp(model_b, directory, optimizer=opt_b, allow_reshard=True)
    params_b, optim_b = _full_state(model_b, opt_b)
    assert set(params_a) == set(params_b)
    for k in params_a:
        assert torch.equal(params_a[k], params_b[k]), k                      # bitwise
    fa, fb = _flatten(optim_a), _flatten(optim_b)
    tensors = [k for k in fa if fa[k].dim() > 0]
    assert tensors and set(tensors) <= set(fb)
    for k in tensors:
        assert torch.equal(fa[k], fb[k]), k                                  # bitwise optimizer state
    loss_b = _step(model_b, opt_b, 3)
    assert torch.allclose(loss_a, loss_b, atol=1e-6), (loss_a, loss_b)
    dist.barrier()


def test_hsdp_2x2_checkpoint_reshards_onto_dp_shard_4():
    with tempfile.TemporaryDirectory() as d:
        run_ranks(_worker, 4, d, timeout=600.0)
        assert os.path.exists(os.path.join(d, "matrix_metadata.pt"))


def _shared_ns_worker(rank, world):
    """Splitting Newton-Schulz over the two replicas changes who computes, not what: parameters and momentum
    are bitwise those of the run where every replica orthogonalises every matrix."""
    from matrix_fsdp_b200.optim import muon as muon_mod
    from matrix_fsdp_b200.optim.muon import MatrixMuon

    muon_mod.SHARE_WINDOW_ELEMENTS = 2048        # several exchange windows per step (the matrices have 1536-3072 elements)
    results = {}
    for share in (True, False):
        model, opt = _build("hsdp")
        muon = opt.muon
        if isinstance(muon, MatrixMuon):
            assert muon.ns_share_group is not None                   # hybrid mesh: sharing is on by default
            if not share:
                muon.share_newton_schulz_over(None)
        done = 0
        for s in range(3):
            _step(model, opt, s)
            done += getattr(muon, "ns_matrices_done", 0)
        params, optim = _full_state(model, opt)
        results[share] = (params, _flatten(optim), done)
    (pa, oa, done_shared), (pb, ob, done_all) = results[True], results[False]
    for k in pa:
        assert torch.equal(pa[k], pb[k]), k
    for k in oa:
        if oa[k].dim() > 0:
            assert torch.equal(oa[k], ob[k]), k
    counts = torch.tensor([done_shared, done_all])
    dist.all_reduce(counts)
    assert counts[1] == 2 * counts[0] and counts[0] > 0              # each matrix orthogonalised once, not twice
    dist.barrier()


def test_hsdp_replicas_share_newton_schulz():
    run_ranks(_shared_ns_worker, 4)
