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
