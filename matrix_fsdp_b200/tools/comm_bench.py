"""Micro-benchmark of the all-gather / reduce-scatter transports.

    python -m torch.distributed.run --nproc-per-node N -m matrix_fsdp_b200.tools.comm_bench \
        --numel 50000000 --layout even|owner --iters 20

Times each transport (peer kernels, NCCL equal/padded, owner broadcast) with CUDA events on the
launching stream after warm-up, takes the max over ranks and reports logical bus bandwidth
(bytes every rank must receive ÷ time) and the fraction of the measured NVLink peer-copy rate.

Parity: ``matrix_fsdp/tools/comm_bench.py:1-224``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..core.layout import LayoutSegment
from ..parallel.collectives import SegmentTables
from ..parallel.transport import TorchDistTransport

NVLINK_PEER_GBS = 770.0   # measured per-direction peer copy on this pool


def make_tables(total: int, world: int, rank: int, layout: str) -> SegmentTables:
    if layout == "even":
        per = (total // world) // 8 * 8
        sizes = [per] * world
        sizes[-1] += total - per * world
    else:  # owner-like: alternating big / small chunks
        weights = [3 if r % 2 == 0 else 1 for r in range(world)]
        unit = total // sum(weights) // 8 * 8
        sizes = [w * unit for w in weights]
        sizes[-1] += total - sum(sizes)
    segs, cur = [], 0
    for s in sizes:
        segs.append((LayoutSegment(cur, cur + s, 0),))
        cur += s
    return SegmentTables.build(total, segs, rank)


def time_op(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def fused_paths(peer, tables: SegmentTables, args, world: int, dev) -> list[dict]:
    """Fused kernels against their unfused sequences, with roofline fractions.

    AG+GEMM: the q|k|v rows ([3H, H] at element offset H of the block) arrive inside the QKV GEMM of a
    ``tokens x H`` activation.  Roofline = max(GEMM FLOPs / sustained GEMM rate, remote bytes / link rate).
    RS+AdamW: reduce-scatter with the sharded AdamW update applied in the same kernel.  Roofline =
    bytes pulled over NVLink / link rate (the optimizer traffic is local HBM, an order of magnitude faster).
    """
    from ..ops import kernels as K

    rank = dist.get_rank()
    h, t = args.hidden, args.tokens
    lo, hi = h, h + 3 * h * h
    n_local = tables.shard_sizes[rank]
    key = "bench_fused"
    shard = peer.alloc_persistent(n_local, torch.bfloat16, dev, "shard", symmetric_numel=tables.max_shard)
    shard.normal_(0, 0.02)
    full = torch.empty(args.numel, dtype=torch.bfloat16, device=dev)
    x = (torch.randn(t, h, device=dev) * 0.1).bfloat16()
    out = torch.empty(t, 3 * h, dtype=torch.bfloat16, device=dev)
    w = full[lo:hi].view(3 * h, h)
    res = []

    def unfused():
        peer.gather(shard, full, tables, unit_key=key).wait()
        K.gemm(x, w, out=out)

    def fused():
        hd = peer.gather(shard, full, tables, unit_key=key, defer=(lo, hi, h))
        hd.wait()
        K.gemm_ag(x, w, hd.deferred, out=out)

    def gather_rest_only():
        peer.gather(shard, full, tables, unit_key=key, defer=(lo, hi, h)).wait()

    def gemm_only():
        K.gemm(x, w, out=out)

    ms_u, ms_f = time_op(unfused, args.iters), time_op(fused, args.iters)
    ms_rest, ms_gemm = time_op(gather_rest_only, args.iters), time_op(gemm_only, args.iters)
    flops = 2.0 * t * 3 * h * h
    remote = sum(max(0, min(s.global_start + s.numel, hi) - max(s.global_start, lo))
                 for r, segs in enumerate(tables.rank_segments) if r != rank for s in segs) * 2
    rt = torch.tensor([float(remote)], device=dev)
    dist.all_reduce(rt, op=dist.ReduceOp.MAX)          # the slowest rank is the one that pulls the most
    remote = float(rt.item())
    roof_ms = max(flops / (args.gemm_tflops * 1e12), remote / (NVLINK_PEER_GBS * 1e9)) * 1e3
    fused_part = ms_f - ms_rest
    res.append({"op": "ag+gemm", "unfused_ms": ms_u, "fused_ms": ms_f, "gather_of_other_rows_ms": ms_rest,
                "gemm_alone_ms": ms_gemm, "fused_gemm_part_ms": fused_part, "roofline_ms": roof_ms,
                "frac_of_roofline": roof_ms / fused_part if fused_part > 0 else None,
                "remote_mb": remote / 2 ** 20, "gflop": flops / 1e9})

    grad = peer.acquire_grad_buffer(key, args.numel, torch.bfloat16, dev)
    grad.normal_(0, 1e-3)
    p = torch.zeros(n_local, dtype=torch.float32, device=dev)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    lp = torch.zeros(n_local, dtype=torch.bfloat16, device=dev)
    g = torch.empty(n_local, dtype=torch.float32, device=dev)
    hp = dict(lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
    step = [0]

    def rs_then_adamw():
        step[0] += 1
        peer.reduce(grad, g, tables, scale=1.0 / world, unit_key=key).wait()
        K.adamw_flat_(p, m, v, g, step=step[0], p_lp=lp, **hp)

    def rs_adamw_fused():
        step[0] += 1
        peer.reduce_update(grad, tables, dict(p=p, m=m, v=v, p_lp=lp, step=step[0], **hp), scale=1.0 / world,
                           unit_key=key).wait()

    ms_u, ms_f = time_op(rs_then_adamw, args.iters), time_op(rs_adamw_fused, args.iters)
    pulled = (world - 1) * n_local * 2
    roof_ms = pulled / (NVLINK_PEER_GBS * 1e9) * 1e3
    res.append({"op": "rs+adamw", "unfused_ms": ms_u, "fused_ms": ms_f, "roofline_ms": roof_ms,
                "frac_of_roofline": roof_ms / ms_f, "pulled_mb": pulled / 2 ** 20})
    return res


def moe_paths(args, world: int, dev) -> list[dict]:
    """Expert-parallel dispatch (permute + all-to-all in one push kernel) and combine (all-to-all + unpermute +
    weighted sum in one pull kernel) for ``--tokens`` tokens of width ``--hidden`` routed top-``--top-k`` over
    ``--experts`` experts, against ``all_to_all_single`` moving the same rows there and back (which still needs the
    permutation and the weighted sum around it).  Roofline = remote bytes / measured NVLink rate."""
    from ..ops import moe_kernels as MK
    from ..parallel.expert_parallel import KIND_PUSHED, KIND_READY, ExpertParallelContext

    T, H, E, k = args.tokens, args.hidden, args.experts, args.top_k
    ep = ExpertParallelContext.get(dist.group.WORLD, dev, H, E, k, T, capacity_factor=0.0)
    El = ep.experts_per_rank
    x = torch.randn(T, H, device=dev).bfloat16()
    logits = torch.randn(T, E, device=dev).bfloat16()
    _, idx, w = MK.router_topk(logits, k, torch.zeros(E, dtype=torch.float32, device=dev))
    state = {}

    def dispatch():
        slot, counts = MK.assign_slots(idx, E)
        counts_all = ep.exchange_counts(counts)
        dest_base, group_offsets, group_rows, tile_group, stats = MK.plan(counts_all, ep.world, ep.rank, E, ep.cap_rows)
        state["route"] = MK.dispatch_push(x, idx, ep.recv_addrs, El, ep.cap_rows, slot=slot, dest_base=dest_base)
        ep.fence(KIND_PUSHED)

    def combine():
        ep.fence(KIND_READY)
        MK.combine_pull(ep.recv_addrs, idx, state["route"], H, El, weight=w)      # pull the rows back, weighted sum

    dispatch()
    d_ms = time_op(dispatch, args.iters)
    c_ms = time_op(combine, args.iters)
    rows = T * k
    remote = rows * H * 2 * (world - 1) / world
    # library baseline: equal-split all-to-all of the same number of rows in both directions
    per_peer = (rows + world - 1) // world
    send = torch.randn(world * per_peer, H, device=dev).bfloat16()
    recv = torch.empty_like(send)
    a2a_ms = time_op(lambda: dist.all_to_all_single(recv, send), args.iters)
    out = []
    for op, ms in (("moe_dispatch_push", d_ms), ("moe_combine_pull", c_ms), ("nccl_all_to_all_single", a2a_ms)):
        out.append({"op": op, "ms": ms, "rows": rows, "remote_mb": remote / 2 ** 20,
                    "remote_gb_per_s": remote / (ms * 1e-3) / 1e9,
                    "frac_of_measured_nvlink_770": remote / (ms * 1e-3) / 1e9 / NVLINK_PEER_GBS,
                    "rows_lost": ep.rows_lost_total()})
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--numel", type=int, default=50_593_792)   # one Llama-2048 block
    ap.add_argument("--layout", choices=("even", "owner"), default="even")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default=None)
    ap.add_argument("--fused", action="store_true", help="also time the fused compute+collective kernels")
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--gemm-tflops", type=float, default=1400.0, help="sustained bf16 GEMM rate used as roofline")
    ap.add_argument("--moe", action="store_true", help="also time the expert-parallel dispatch / combine kernels")
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=6)
    args = ap.parse_args(argv)
    rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    world, dev = dist.get_world_size(), torch.device("cuda", rank)
    tables = make_tables(args.numel, world, dist.get_rank(), args.layout)
    n_local = tables.shard_sizes[dist.get_rank()]
    results = []
    transports = {"nccl_auto": TorchDistTransport(dist.group.WORLD),
                  "nccl_owner_broadcast": TorchDistTransport(dist.group.WORLD, gather_impl="owner_broadcast",
                                                             reduce_impl="owner_reduce")}
    from ..parallel.peer import PeerTransport

    peer = PeerTransport.create(dist.group.WORLD, dev)
    if peer is not None:
        transports = {"peer": peer, **transports}
    full = torch.empty(args.numel, dtype=torch.bfloat16, device=dev)
    for name, tr in transports.items():
        shard = tr.alloc_persistent(n_local, torch.bfloat16, dev, "shard", symmetric_numel=tables.max_shard)
        shard.normal_()
        grad = tr.acquire_grad_buffer(f"bench_{name}", args.numel, torch.bfloat16, dev)
        grad.normal_()
        out = torch.empty(n_local, dtype=torch.float32 if name == "peer" else torch.bfloat16, device=dev)
        key = f"bench_{name}"
        dst = full
        if name == "peer":
            # with NVSwitch multicast the gather pushes into a persistent symmetric full-parameter slot
            slot = tr.alloc_full_buffer(key, args.numel, torch.bfloat16, tables, exclusive=True)
            dst = slot if slot is not None else full
        impls = {}

        def run_ag():
            h = tr.gather(shard, dst, tables, unit_key=key)
            impls["all_gather"] = h.info.get("impl", "")
            h.wait()

        def run_rs():
            h = tr.reduce(grad, out, tables, scale=1.0 / world, unit_key=key)
            impls["reduce_scatter"] = h.info.get("impl", "")
            h.wait()

        ag = time_op(run_ag, args.iters)
        rs = time_op(run_rs, args.iters)
        recv_bytes = (args.numel - n_local) * 2
        for op, ms in (("all_gather", ag), ("reduce_scatter", rs)):
            gbs = recv_bytes / (ms * 1e-3) / 1e9
            results.append({"transport": name, "op": op, "impl": impls.get(op, ""), "ms": ms, "recv_gb_per_s": gbs,
                            "frac_of_measured_nvlink_770": gbs / NVLINK_PEER_GBS})
    if peer is not None and args.fused:
        results += fused_paths(peer, tables, args, world, dev)
    if args.moe:
        results += moe_paths(args, world, dev)
    if dist.get_rank() == 0:
        for r in results:
            print(json.dumps(r))
        if args.out:
            with open(args.out, "w") as f:
                json.dump({"world": world, "numel": args.numel, "layout": args.layout, "results": results}, f, indent=1)
    PeerTransport.close_all()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
