"""Device-side timeline of the collectives of a training step, from CUDA events.

The runtime event log carries *host* durations (how long a call took to enqueue).  What decides the
step time is what happened on the device: when a collective really started on its stream, how long
it ran, and for how long the compute stream then stood still waiting for it (the *exposed* time).
While the timeline is enabled every collective handle records

``start``       on the communication stream, right after it has waited for the issuing stream;
``end``         on the communication stream, after the last kernel of the collective;
``wait_begin``  on the consuming stream, just before it is made to wait for ``end``;
``wait_end``    on the consuming stream, just after.

``wait_end - wait_begin`` is the stall the consumer saw; a fully hidden collective shows ~0 there.
Events are only read after :func:`resolve` synchronised the device, so enabling the timeline adds
a few event records per collective and no host sync to the step itself.

The reference measures host enqueue/wait times only (``matrix_fsdp/runtime/runtime_event.py:14-50``,
``runtime/summary.py:40-271``).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

_ENABLED = False
_COLLECT = True       # keep every span in the module-level list (False: spans live on their handles only)
_SPANS: list["CollectiveSpan"] = []
_ORIGIN = None


@dataclass
class CollectiveSpan:
    unit: str
    kind: str                      # all_gather | reduce_scatter | all_reduce
    impl: str = ""
    nbytes: int = 0
    reason: str = ""
    start: object = None
    end: object = None
    wait_begin: object = None
    wait_end: object = None
    # filled by resolve()
    start_ms: float | None = None
    device_ms: float | None = None
    wait_at_ms: float | None = None
    exposed_ms: float | None = None
    extra: dict = field(default_factory=dict)

    def as_row(self) -> dict:
        return {"unit": self.unit, "kind": self.kind, "impl": self.impl, "bytes": self.nbytes, "reason": self.reason,
                "start_ms": self.start_ms, "device_ms": self.device_ms, "wait_at_ms": self.wait_at_ms,
                "exposed_ms": self.exposed_ms}


def enabled() -> bool:
    return _ENABLED


def enable(on: bool = True, *, collect: bool = True) -> None:
    """Switch span recording on or off (CUDA only; a no-op elsewhere).  ``collect=False`` records the
    events on the handles without keeping a global list (what the adaptive prefetch policies use)."""
    global _ENABLED, _COLLECT
    _ENABLED = bool(on) and torch.cuda.is_available()
    if on:
        _COLLECT = bool(collect)


def clear() -> None:
    global _ORIGIN
    _SPANS.clear()
    _ORIGIN = None


def mark_origin(stream=None) -> None:
    """Record the time origin of the step on ``stream`` (default: the current stream)."""
    global _ORIGIN
    if _ENABLED:
        _ORIGIN = torch.cuda.Event(enable_timing=True)
        _ORIGIN.record(stream if stream is not None else torch.cuda.current_stream())


def open_span(unit: str, kind: str, stream, *, impl: str = "", nbytes: int = 0, reason: str = "") -> CollectiveSpan | None:
    """Call on the host right after ``stream`` was ordered behind the issuing stream."""
    if not _ENABLED:
        return None
    sp = CollectiveSpan(unit=unit, kind=kind, impl=impl, nbytes=int(nbytes), reason=reason)
    sp.start = torch.cuda.Event(enable_timing=True)
    sp.start.record(stream if stream is not None else torch.cuda.current_stream())
    if _COLLECT:
        _SPANS.append(sp)
    return sp


def close_span(sp: CollectiveSpan | None, stream, *, impl: str | None = None) -> None:
    if sp is None:
        return
    sp.end = torch.cuda.Event(enable_timing=True)
    sp.end.record(stream if stream is not None else torch.cuda.current_stream())
    if impl is not None:
        sp.impl = impl


def begin_wait(sp: CollectiveSpan | None) -> None:
    if sp is None or sp.wait_begin is not None:
        return
    sp.wait_begin = torch.cuda.Event(enable_timing=True)
    sp.wait_begin.record(torch.cuda.current_stream())


def end_wait(sp: CollectiveSpan | None) -> None:
    if sp is None or sp.wait_end is not None or sp.wait_begin is None:
        return
    sp.wait_end = torch.cuda.Event(enable_timing=True)
    sp.wait_end.record(torch.cuda.current_stream())


def try_resolve_span(sp: CollectiveSpan) -> bool:
    """Fill ``device_ms`` / ``exposed_ms`` of one span without synchronising; False while its events are
    still pending."""
    if sp.device_ms is not None:
        return True
    if sp.start is None or sp.end is None or not sp.end.query():
        return False
    try:
        sp.device_ms = sp.start.elapsed_time(sp.end)
        if sp.wait_begin is not None and sp.wait_end is not None and sp.wait_end.query():
            sp.exposed_ms = max(sp.wait_begin.elapsed_time(sp.wait_end), 0.0)
    except RuntimeError:
        return False
    return True


def resolve() -> list[CollectiveSpan]:
    """Synchronise and turn the recorded events into milliseconds relative to the origin."""
    if not _SPANS:
        return []
    torch.cuda.synchronize()
    origin = _ORIGIN
    for sp in _SPANS:
        if sp.start is None or sp.end is None:
            continue
        try:
            sp.device_ms = sp.start.elapsed_time(sp.end)
            if origin is not None:
                sp.start_ms = origin.elapsed_time(sp.start)
            if sp.wait_begin is not None and sp.wait_end is not None:
                sp.exposed_ms = max(sp.wait_begin.elapsed_time(sp.wait_end), 0.0)
                if origin is not None:
                    sp.wait_at_ms = origin.elapsed_time(sp.wait_begin)
        except RuntimeError:
            continue       # an event that was never reached (e.g. a discarded prefetch)
    return list(_SPANS)


def summarize(spans: list[CollectiveSpan] | None = None) -> dict:
    """Totals per collective kind: device time, exposed time, bytes, achieved GB/s."""
    spans = resolve() if spans is None else spans
    out: dict[str, dict] = {}
    for sp in spans:
        if sp.device_ms is None:
            continue
        d = out.setdefault(sp.kind, {"count": 0, "device_ms": 0.0, "exposed_ms": 0.0, "bytes": 0})
        d["count"] += 1
        d["device_ms"] += sp.device_ms
        d["exposed_ms"] += sp.exposed_ms or 0.0
        d["bytes"] += sp.nbytes
    for d in out.values():
        d["gbytes_per_s"] = d["bytes"] / d["device_ms"] / 1e6 if d["device_ms"] > 0 else 0.0
    return out


def format_rows(spans: list[CollectiveSpan] | None = None) -> str:
    """Markdown table, one row per collective in start order."""
    spans = resolve() if spans is None else spans
    rows = sorted((s for s in spans if s.device_ms is not None), key=lambda s: (s.start_ms or 0.0))
    lines = ["| unit | collective | impl | MB | issued for | start ms | device ms | waited at ms | exposed ms |",
             "|---|---|---|---|---|---|---|---|---|"]
    f = lambda v: "" if v is None else f"{v:.3f}"   # noqa: E731
    for s in rows:
        lines.append(f"| {s.unit} | {s.kind} | {s.impl} | {s.nbytes / 2 ** 20:.1f} | {s.reason} | {f(s.start_ms)} | "
                     f"{f(s.device_ms)} | {f(s.wait_at_ms)} | {f(s.exposed_ms)} |")
    return "\n".join(lines)
