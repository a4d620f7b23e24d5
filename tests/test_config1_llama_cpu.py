"""BASELINE config 1: CPU/gloo world_size 2, fp32 Llama (2L, h256, 4x64 heads, SwiGLU 688, vocab 1024,
tied embeddings), row sharding per block, AdamW(3e-4, 0.9/0.95, wd 0.1), batch 2 x seq 128 from seed 0:
5 steps must reproduce the single-process loss curve and parameters."""
import copy

import torch
import torch.distributed as dist
from torch.distributed.tensor.placement_types import Shard

from dist_utils import run_ranks


def _data():
    g = torch.Generator().manual_seed(0)
    return [torch.randint(0, 1024, (2, 129), generator=g) for _ in range(5)]


def _worker(rank, world):
    from matrix_fsdp_b200 import configure_optimizer, fully_shard, matrix_fully_shard
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions, get_model_state_dict
    from matrix_fsdp_b200.models.llama import LlamaConfig, LlamaModel

    torch.manual_seed(0)
    cfg = LlamaConfig.config1()
    model = LlamaModel(cfg)
    ref = copy.deepcopy(model)
    for layer in model.layers:
        fully_shard(layer, shard_placement_fn=lambda p: Shard(0))
    matrix_fully_shard(model, allow_shared_params=True)      # embedding (tied with the LM head) + final norm
    opt = configure_optimizer(model, "adamw", lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    ropt = torch.optim.AdamW(ref.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    for batch in _data():
        mine = batch[rank:rank + 1]                            # each rank takes one of the two sequences
        loss = model(mine[:, :-1], mine[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad()
        rl = ref(batch[:, :-1], batch[:, 1:])                  # single-process model sees the global batch
        rl.backward()
        ropt.step()
        ropt.zero_grad()
        gl = loss.detach().clone()
        dist.all_reduce(gl)
        assert abs(gl.item() / world - rl.item()) < 1e-4, (gl.item() / world, rl.item())
    full = get_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True))
    for k, v in ref.state_dict().items():
        assert torch.allclose(full[k], v, atol=2e-5, rtol=1e-4), k
    assert full["head.lm_head.weight"].data_ptr() != 0 and torch.equal(full["head.lm_head.weight"], full["embed.weight"])


def test_config1_two_rank_gloo_matches_single_process():
    run_ranks(_worker, 2)
