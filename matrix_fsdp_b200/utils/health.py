"""Host-side failure detection: rank heartbeats in a key-value store plus the device status word.

The data plane of this framework never blocks forever (every device wait is bounded and reports a
status code), so a lost peer shows up either as a ``peer flag wait timed out`` status or — earlier and
cheaper — as a missing heartbeat on the host.  :class:`RankHealth` gives the second: every rank
publishes ``(step, wall time)`` between steps, and ``assert_alive()`` before launching the next step
raises :class:`RankFailure` naming the ranks that left or went silent, so the survivors stop between
steps with no kernel or collective in flight and can resume from the last checkpoint on a different
world size (``load_matrix_dcp(..., allow_reshard=True)``).

The reference has no failure detection at all (its failures surface as NCCL errors,
``matrix_fsdp/kernels/native/matrix_nccl.cpp:23-27``).
"""
from __future__ import annotations

import time


class RankFailure(RuntimeError):
    def __init__(self, missing: list[int], reason: str) -> None:
        super().__init__(f"ranks {missing} {reason}")
        self.missing = missing
        self.reason = reason


class RankHealth:
    """Heartbeats over any ``torch.distributed`` store (``TCPStore`` / ``FileStore`` / ``HashStore``)."""

    def __init__(self, store, rank: int, world_size: int, *, timeout_s: float = 30.0, prefix: str = "mfsdp_hb") -> None:
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world_size, timeout_s, prefix
        self.beat(-1)

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}:alive")

    def leave(self, reason: str = "left") -> None:
        """Announce an orderly exit (called between steps, with nothing in flight)."""
        self.store.set(self._key(self.rank), f"-1:{time.time():.3f}:{reason}")

    def _read(self, rank: int):
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(rank)]):
                return None
            raw = self.store.get(self._key(rank)).decode()
        except Exception:  # noqa: BLE001
            return None
        step, ts, state = raw.split(":", 2)
        return int(step), float(ts), state

    def peers(self) -> dict[int, tuple | None]:
        return {r: self._read(r) for r in range(self.world)}

    def assert_alive(self, *, min_step: int | None = None) -> None:
        now = time.time()
        gone, silent = [], []
        for r, rec in self.peers().items():
            if r == self.rank:
                continue
            if rec is None:
                silent.append(r)
            elif rec[2] != "alive":
                gone.append(r)
            elif now - rec[1] > self.timeout_s or (min_step is not None and rec[0] < min_step
                                                   and now - rec[1] > self.timeout_s):
                silent.append(r)
        if gone:
            raise RankFailure(gone, "left the job")
        if silent:
            raise RankFailure(silent, f"sent no heartbeat for more than {self.timeout_s:.1f}s")


def check_device_status(device=None) -> None:
    """Raise if any bounded device wait on ``device`` ran out since the last check (device→host read)."""
    from ..ops import kernels

    kernels.check_status(device)
