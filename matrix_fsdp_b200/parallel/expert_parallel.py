"""Expert-parallel (EP) runtime: symmetric receive / output buffers and the epoch flags that order
dispatch and combine between the ranks of one node.

The reference has no EP runtime (docs/introduction.md:238-271); its test fixture moves tokens with four
``all_to_all_single`` calls per layer (test/fsdp/test_deepseek_v3_ep_train.py:501-548).  Here every
rank owns two row buffers in peer-mapped memory:

* ``recv`` — rows that other ranks *push* into (tokens in forward, output gradients in backward),
  grouped by local expert on 256-row boundaries so the grouped GEMM consumes them in place;
* ``out``  — rows this rank's experts produced, which the token owners *pull* and reduce.

One context is shared by all MoE layers of a model: a rank can only start pushing layer ``l+1`` after
it pulled layer ``l`` from every owner, and an owner only raises its "ready" flag after its GEMMs read
``recv``, so reuse of both buffers is ordered by the flags themselves.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

KIND_COUNTS, KIND_PUSHED, KIND_READY = 0, 1, 2

_CONTEXTS: dict[tuple, "ExpertParallelContext"] = {}


class ExpertParallelContext:
    def __init__(self, group, device: torch.device, hidden: int, n_experts: int, top_k: int, max_tokens: int,
                 capacity_factor: float = 0.0) -> None:
        self.group, self.device = group, device
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        if n_experts % self.world:
            raise ValueError(f"{n_experts} experts do not divide over {self.world} expert-parallel ranks")
        self.hidden, self.n_experts, self.top_k = hidden, n_experts, top_k
        self.experts_per_rank = n_experts // self.world
        # Receive capacity.  ``capacity_factor`` <= 0 (or None) sizes for the worst case, every routed row of
        # every rank landing here: nothing can ever be dropped.  A positive factor sizes for that multiple of
        # the average load; rows beyond it are dropped on the owner, counted in ``lost_rows`` (never silently:
        # ``rows_lost_total()`` is what benches and training loops report).
        rows = max_tokens * top_k
        self.dropless = not capacity_factor or capacity_factor <= 0
        if self.world > 1:
            rows = rows * self.world if self.dropless else min(int(rows * capacity_factor), rows * self.world)
        self.lost_rows = torch.zeros(1, dtype=torch.int64, device=device)
        self.routed_rows = 0
        # every expert group is padded to whole 256-row tiles (the grouped GEMMs run on CTA pairs)
        self.cap_rows = (rows + self.experts_per_rank * 256 + 255) // 256 * 256
        self.max_tokens = max_tokens
        self._epoch = {KIND_COUNTS: 0, KIND_PUSHED: 0, KIND_READY: 0}
        nbytes = self.cap_rows * hidden * 2
        if self.world == 1:
            self.peer = None
            self.recv = torch.empty(self.cap_rows, hidden, dtype=torch.bfloat16, device=device)
            self.out = torch.empty(self.cap_rows, hidden, dtype=torch.bfloat16, device=device)
            self.out_scalar = torch.zeros(self.cap_rows, dtype=torch.float32, device=device)
            self.counts_all = torch.zeros(self.world, n_experts, dtype=torch.int32, device=device)
            self.recv_addrs = [self.recv.data_ptr()]
            self.out_addrs = [self.out.data_ptr()]
            self.scalar_addrs = [self.out_scalar.data_ptr()]
            self.counts_addrs = [self.counts_all.data_ptr()]
            return
        from .peer import MAX_UNITS, PeerTransport

        transport = PeerTransport.create(group, device)
        if transport is None:
            raise RuntimeError("expert parallelism over peer memory needs CUDA IPC and peer access between all ranks")
        self.peer = transport.ctx
        self._flag_unit = MAX_UNITS - 1
        recv = self.peer.alloc(nbytes)
        out = self.peer.alloc(nbytes)
        scal = self.peer.alloc(self.cap_rows * 4, zero=True)
        cnt = self.peer.alloc(self.world * n_experts * 4, zero=True)
        self.recv = recv.tensor.view(torch.bfloat16).view(self.cap_rows, hidden)
        self.out = out.tensor.view(torch.bfloat16).view(self.cap_rows, hidden)
        self.out_scalar = scal.tensor.view(torch.float32)
        self.counts_all = cnt.tensor.view(torch.int32).view(self.world, n_experts)
        self.recv_addrs, self.out_addrs = list(recv.peer_addr), list(out.peer_addr)
        self.scalar_addrs, self.counts_addrs = list(scal.peer_addr), list(cnt.peer_addr)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    @classmethod
    def get(cls, group, device: torch.device, hidden: int, n_experts: int, top_k: int, max_tokens: int,
            capacity_factor: float = 0.0) -> "ExpertParallelContext":
        key = (id(group) if group is not None else 0, device.index, hidden, n_experts, top_k)
        ctx = _CONTEXTS.get(key)
        if ctx is None or ctx.max_tokens < max_tokens:
            ctx = cls(group, device, hidden, n_experts, top_k, max_tokens, capacity_factor)
            _CONTEXTS[key] = ctx
        return ctx

    # ------------------------------------------------------------------ ordering
    def fence(self, kind: int) -> None:
        """Raise my flag of ``kind`` on every rank, then wait until every rank raised theirs."""
        if self.world == 1:
            return
        self._epoch[kind] += 1
        stream = torch.cuda.current_stream(self.device)
        self.peer.signal_wait(self._flag_unit, kind, self._epoch[kind], stream)

    def exchange_counts(self, counts: torch.Tensor) -> torch.Tensor:
        """All ranks learn every rank's per-expert counts; returns the local ``[W, E]`` table."""
        from ..ops import moe_kernels as MK

        MK.push_counts(self.counts_addrs, self.world, self.rank, counts)
        self.fence(KIND_COUNTS)
        return self.counts_all

    # ------------------------------------------------------------------ drop accounting
    def note_plan(self, stats: torch.Tensor, routed: int) -> None:
        """After every dispatch plan: ``stats[1]`` = rows this rank (as owner) could not place."""
        self.lost_rows += stats[1:2].to(torch.int64)
        self.routed_rows += int(routed)

    def rows_lost_total(self) -> int:
        return int(self.lost_rows.item())

    def rows_routed_total(self) -> int:
        return int(self.routed_rows)


def live_contexts() -> list[ExpertParallelContext]:
    return list(_CONTEXTS.values())


def reset_contexts() -> None:
    _CONTEXTS.clear()
