"""Spawn helpers for multi-rank CPU tests (gloo over loopback, file:// rendezvous)."""
import os
import tempfile
import time
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank, world, fn, init_file, args, err_dir):
    os.environ["GLOO_SOCKET_IFNAME"] = "lo"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    torch.set_num_threads(1)
    try:
        dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
    except Exception:
        with open(os.path.join(err_dir, f"rank{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world: int, *args, timeout: float = 240.0):
    """Run ``fn(rank, world, *args)`` on ``world`` gloo ranks; re-raise the first rank's traceback."""
    with tempfile.TemporaryDirectory() as tmp:
        init_file = os.path.join(tmp, "rdzv")
        ctx = mp.spawn(_entry, args=(world, fn, init_file, args, tmp), nprocs=world, join=False)
        try:
            # ``join`` returns each time one rank ends, so wait against a deadline; ranks still running after it
            # are stuck (one left a collective the others are still in) and are ended here, by the handles this
            # call started
            deadline = time.monotonic() + 3 * timeout
            ok = ctx.join(timeout=timeout)
            while not ok and time.monotonic() < deadline:
                ok = ctx.join(timeout=max(1.0, deadline - time.monotonic()))
            if not ok:
                for proc in ctx.processes:
                    if proc.is_alive():
                        proc.terminate()
                for proc in ctx.processes:
                    proc.join(10)
                raise TimeoutError(f"ranks still running after {3 * timeout:.0f} s")
        except Exception as exc:
            msgs = []
            for r in range(world):
                p = os.path.join(tmp, f"rank{r}.err")
                if os.path.exists(p):
                    msgs.append(f"--- rank {r} ---\n" + open(p).read())
            raise AssertionError("\n".join(msgs) or str(exc)) from None


def _cases_worker(rank, world, cases, out_path):
    import json

    results = {}
    for name, fn, args in cases:
        try:
            fn(rank, world, *args)
            mine = ""
        except Exception:
            mine = traceback.format_exc()
        # a case fails if it failed on any rank; ranks stay in step because every case ends with this exchange
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        results[name] = "\n".join(f"--- rank {r} ---\n{t}" for r, t in enumerate(gathered) if t)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(results, f)


def run_cases(world: int, cases, *, timeout: float = 600.0) -> dict:
    """Run ``[(name, fn, args), ...]`` as ``fn(rank, world, *args)`` one after the other inside ONE spawn of
    ``world`` gloo ranks (starting the ranks costs more than most cases) and return ``{name: "" or the ranks'
    tracebacks}``.  Use it from a module-scoped fixture and give every case a test of its own."""
    import json

    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "outcomes.json")
        run_ranks(_cases_worker, world, list(cases), path, timeout=timeout)
        with open(path) as f:
            return json.load(f)


def check_case(outcomes: dict, name: str) -> None:
    assert name in outcomes, "the ranks did not reach this case"
    assert not outcomes[name], outcomes[name]
