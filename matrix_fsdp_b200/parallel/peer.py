"""Peer-memory transport: FSDP collectives as hand-written kernels over symmetric peer buffers.

One :class:`PeerContext` per (process group, device) owns *symmetric* memory: every rank performs
the same sequence of allocations and learns every peer's address of each segment once -- through
``torch.distributed._symmetric_memory`` (which also yields the NVSwitch multicast address), or through
``cudaMalloc`` + CUDA IPC handles where that is not available.  :class:`PeerTransport` then implements the transport interface on top of it:

``gather``   publish "my shard for this unit is ready (epoch e)" → wait for every peer's flag →
             ``ag_pull`` copies each peer's segments from its shard buffer straight into the local
             full-parameter buffer (no padding, no staging, any layout);
``reduce``   publish "my gradients for this unit are complete" → wait for peers →
             ``rs_pull_reduce`` sums the owned segments across all ranks' gradient buffers in fp32,
             applies the 1/world scale and writes the local gradient shard → publish "pulled" so
             owners may reuse their gradient buffers.

With NVLS (``MFSDP_NVLS``, default on when the symmetric segments could be bound to an NVSwitch
multicast object) the same two operations go through the switch instead: ``gather`` *pushes* only
this rank's shard with ``multimem.st`` into a persistent, symmetric full-parameter slot (every
rank's copy is written by the switch), ``reduce`` reads each owned element once with
``multimem.ld_reduce`` (the switch sums the ranks' gradient buffers).  Slots are shared by units
that are never unsharded together; a "free" flag published at reshard keeps a pusher from
overwriting a slot a peer still reads.  The plain peer-load kernels stay as the fallback and are
the only path when ``MFSDP_NVLS=0`` (failure tests: a rank must never exit while its memory is
bound to a multicast object that others still use).

Gradient buffers come from a small ring of symmetric slots per size class; a slot is handed to the
next unit only after every peer has published "pulled" for its previous user.  All waits are
bounded (``MFSDP_PEER_WAIT_TIMEOUT_S``) and report through the device status word.

The reference's closest analogue is its optional NCCL send/recv + per-call window registration
path (``matrix_fsdp/kernels/native/matrix_nccl.cpp:176-395``, ``kernels/gin/native/rma_nccl.cpp:
104-195``), which its own gap analysis lists as lacking persistent symmetric buffers
(``docs/deepep_v2_gap_analysis.md:59-236``).
"""
from __future__ import annotations

import ctypes as C
import os
import time
import socket

import torch
import torch.distributed as dist

from ..ops import lib as _lib
from . import device_timeline as _tl
from .collectives import MatrixCollectiveHandle, SegmentTables
from .transport import LocalTransport

_u64, _vp, _i32, _i64 = C.c_ulonglong, C.c_void_p, C.c_int, C.c_longlong
_lib.register_signatures({
    "mfsdp_dev_malloc": [_u64, C.POINTER(C.c_void_p)],
    "mfsdp_dev_free": [_vp],
    "mfsdp_ipc_get_handle": [_vp, C.c_char_p],
    "mfsdp_ipc_open_handle": [C.c_char_p, C.POINTER(C.c_void_p)],
    "mfsdp_ipc_close_handle": [_vp],
    "mfsdp_can_access_peer": [_i32, _i32],
    "mfsdp_peer_signal": [C.POINTER(_u64), _i32, _u64, _vp],
    "mfsdp_peer_wait": [_vp, _i32, _i32, _u64, _u64, _vp, _vp],
    "mfsdp_peer_signal_wait": [C.POINTER(_u64), _vp, _i32, _i32, _u64, _u64, _vp, _vp],
    "mfsdp_validate_pull_table": [_vp, _vp, _vp, _i32, _i64, _i32, C.POINTER(_u64), C.POINTER(_u64), _i32, _vp, _vp],
    "mfsdp_validate_reduce_table": [_vp, _vp, _vp, _i32, _i64, _i64, _vp, _vp],
    "mfsdp_ag_pull": [_vp, _vp, _vp, _vp, _i32, _i64, _i32, _vp, _vp],
    "mfsdp_rs_pull_reduce": [C.POINTER(_u64), _i32, _i32, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i32, _i32,
                             C.c_float, _vp, _vp],
    "mfsdp_rs_pull_adamw": [C.POINTER(_u64), _i32, _i32, _vp, _vp, _vp, _i32, _i64, _i32, C.c_float, _vp, _vp, _vp,
                            _vp, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, _i32, _vp, _vp],
    "mfsdp_ag_push_mc": [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _vp, _vp],
    "mfsdp_rs_mc_reduce": [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i32, _i32, C.c_float, _vp, _vp],
    "mfsdp_rs_mc_adamw": [_vp, _vp, _vp, _vp, _i32, _i64, _i32, C.c_float, _vp, _vp, _vp, _vp, C.c_float, C.c_float,
                          C.c_float, C.c_float, C.c_float, _i32, _vp, _vp],
    "mfsdp_ar_mc": [_vp, _i64, _i32, _i32, _i32, C.c_float, _vp, _vp],
})

KIND_SHARD, KIND_GRAD, KIND_PULLED, KIND_FREE = 0, 1, 2, 3
N_KINDS = 4
MAX_UNITS = 2048
SEGMENT_ENV = "MFSDP_PEER_SEGMENT_MB"
NVLS_ENV = "MFSDP_NVLS"                    # auto (default) | 0 | 1
FULL_SLOTS_ENV = "MFSDP_PEER_FULL_SLOTS"   # full-parameter slots per size class (NVLS all-gather)
BOUNDS_ENV = "MFSDP_DEBUG_BOUNDS"          # 1: validate every pull / reduce table on the device
TIMEOUT_ENV = "MFSDP_PEER_WAIT_TIMEOUT_S"
RING_ENV = "MFSDP_PEER_GRAD_SLOTS"


def _stream_handle(stream) -> int:
    return (stream if stream is not None else torch.cuda.current_stream()).cuda_stream


class SymBuffer:
    """A symmetric allocation: the local tensor, the address of the same bytes on every peer, and (when
    the segment is bound to an NVSwitch multicast object) the multicast address of those bytes."""

    __slots__ = ("tensor", "peer_addr", "nbytes", "mc_addr")

    def __init__(self, tensor: torch.Tensor, peer_addr: list[int], nbytes: int, mc_addr: int = 0) -> None:
        self.tensor, self.peer_addr, self.nbytes, self.mc_addr = tensor, peer_addr, nbytes, mc_addr


class _RawDeviceMemory:
    """Adapter exposing a raw device allocation through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _nvls_requested() -> str:
    v = os.environ.get(NVLS_ENV, "auto").strip().lower()
    return {"": "auto", "true": "1", "on": "1", "false": "0", "off": "0"}.get(v, v)


class PeerContext:
    symmetric_bytes = 0   # bytes of symmetric segments this process allocated (outside torch's allocator)

    def __init__(self, group, device: torch.device) -> None:
        self.group, self.device = group, device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.lib = _lib.load(required=True)
        # small allocations share segments of this size; large ones get a segment of their own size
        self.segment_bytes = int(float(os.environ.get(SEGMENT_ENV, "64")) * 2 ** 20)
        self._segments: list[dict] = []
        self._opened: dict[bytes, int] = {}
        self._by_ptr: dict[int, SymBuffer] = {}
        self.timeout_ns = int(float(os.environ.get(TIMEOUT_ENV, "120")) * 1e9)
        self.debug_bounds = os.environ.get(BOUNDS_ENV, "0") not in ("", "0")
        self.nvls = self._decide_nvls()
        from ..ops import kernels

        self.status = kernels.status_word(device)
        flags = self.alloc(MAX_UNITS * N_KINDS * self.world * 8, zero=True)
        self.flags = flags
        self.flags_u64 = flags.tensor.view(torch.int64)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    # ------------------------------------------------------------------ symmetric allocation
    def _decide_nvls(self) -> bool:
        """Collective: all ranks agree whether segments come from torch's symmetric-memory allocator
        (``cuMemCreate`` + multicast binding, which gives every segment a multicast address)."""
        want = _nvls_requested()
        ok = False
        # Sub-groups of the world (the shard and replicate groups of a hybrid mesh) keep CUDA-IPC segments: with
        # symmetric-memory segments a 2 x 2 mesh stopped in the rendezvous of a gradient buffer allocated during the
        # first backward (all four ranks inside ``rendezvous``, ended by the run's time limit; cause not found).
        whole_world = dist.get_world_size(self.group) == dist.get_world_size()
        if want != "0" and (whole_world or want == "1"):
            try:
                import torch.distributed._symmetric_memory as symm_mem   # noqa: F401
                from torch._C._autograd import DeviceType
                from torch._C._distributed_c10d import _SymmetricMemory

                ok = bool(_SymmetricMemory.has_multicast_support(DeviceType.CUDA, self.device.index or 0))
            except Exception:  # noqa: BLE001  (an old torch, no fabric support, ...)
                ok = False
        votes: list = [None] * self.world
        dist.all_gather_object(votes, ok, group=self.group)
        ok = all(votes)
        if want == "1" and not ok:
            raise RuntimeError("MFSDP_NVLS=1 but NVSwitch multicast is not available on every rank")
        return ok

    def _new_segment(self, nbytes: int) -> dict:
        nbytes = (nbytes + (2 << 20) - 1) // (2 << 20) * (2 << 20)
        if self.nvls:
            import torch.distributed._symmetric_memory as symm_mem

            t = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            hdl = symm_mem.rendezvous(t, self.group)
            bases = [int(a) for a in hdl.buffer_ptrs]
            mc = int(hdl.multicast_ptr or 0)
            if bases[self.rank] != t.data_ptr():
                raise RuntimeError("symmetric-memory handle does not describe the local tensor")
            PeerContext.symmetric_bytes += nbytes
            seg = {"tensor": t, "bases": bases, "used": 0, "nbytes": nbytes, "mc": mc, "handle": hdl}
            self._segments.append(seg)
            return seg
        raw = C.c_void_p()
        rc = self.lib.mfsdp_dev_malloc(nbytes, C.byref(raw))
        if rc != 0:
            raise RuntimeError(f"cudaMalloc of a {nbytes >> 20} MiB symmetric segment failed with code {rc}")
        t = torch.as_tensor(_RawDeviceMemory(int(raw.value), nbytes), device=self.device)
        hbuf = C.create_string_buffer(64)
        rc = self.lib.mfsdp_ipc_get_handle(raw, hbuf)
        if rc != 0:
            raise RuntimeError(f"cudaIpcGetMemHandle failed with code {rc}")
        handle, offset = hbuf.raw, 0
        PeerContext.symmetric_bytes += nbytes
        gathered: list = [None] * self.world
        dist.all_gather_object(gathered, (handle, offset, nbytes), group=self.group)
        bases = []
        for r, (h, off, nb) in enumerate(gathered):
            if nb != nbytes:
                raise RuntimeError("symmetric allocation sizes differ across ranks")
            if r == self.rank:
                bases.append(t.data_ptr())
                continue
            base = self._opened.get(h)
            if base is None:
                out = C.c_void_p()
                rc = self.lib.mfsdp_ipc_open_handle(h, C.byref(out))
                if rc != 0:
                    raise RuntimeError(f"cudaIpcOpenMemHandle failed with code {rc}")
                base = int(out.value)
                self._opened[h] = base
            bases.append(base + off)
        seg = {"tensor": t, "bases": bases, "used": 0, "nbytes": nbytes, "mc": 0, "handle": None}
        self._segments.append(seg)
        return seg

    def alloc(self, nbytes: int, *, zero: bool = False, align: int = 256) -> SymBuffer:
        """Collective: every rank must call with the same ``nbytes`` in the same order."""
        nbytes = max(int(nbytes), 16)
        seg = None
        if nbytes * 4 >= self.segment_bytes:
            seg = self._new_segment(nbytes)           # large buffers: a segment of exactly their size
        else:
            for s in self._segments:
                start = (s["used"] + align - 1) // align * align
                if start + nbytes <= s["nbytes"]:
                    seg = s
                    break
            if seg is None:
                seg = self._new_segment(self.segment_bytes)
        start = (seg["used"] + align - 1) // align * align
        seg["used"] = start + nbytes
        view = seg["tensor"][start:start + nbytes]
        if zero:
            view.zero_()
        buf = SymBuffer(view, [b + start for b in seg["bases"]], nbytes, seg["mc"] + start if seg["mc"] else 0)
        self._by_ptr[view.data_ptr()] = buf
        return buf

    def lookup(self, tensor: torch.Tensor) -> SymBuffer | None:
        return self._by_ptr.get(tensor.data_ptr())

    # ------------------------------------------------------------------ flags
    def slot(self, unit_index: int, kind: int, src: int) -> int:
        return (unit_index * N_KINDS + kind) * self.world + src

    def _slot_addrs(self, unit_index: int, kind: int):
        idx = self.slot(unit_index, kind, self.rank)
        return (_u64 * self.world)(*[self.flags.peer_addr[r] + idx * 8 for r in range(self.world)])

    def signal(self, unit_index: int, kind: int, value: int, stream) -> None:
        """Write ``value`` into my slot of every rank's flag page (including my own)."""
        _lib.check(self.lib.mfsdp_peer_signal(self._slot_addrs(unit_index, kind), self.world, value,
                                              _stream_handle(stream)), "peer_signal")

    def wait(self, unit_index: int, kind: int, value: int, stream) -> None:
        """Wait until every rank's slot in my page reached ``value``."""
        first = self.slot(unit_index, kind, 0)
        _lib.check(self.lib.mfsdp_peer_wait(self.flags.tensor.data_ptr(), first, self.world, value, self.timeout_ns,
                                            self.status.data_ptr(), _stream_handle(stream)), "peer_wait")

    def signal_wait(self, unit_index: int, kind: int, value: int, stream) -> None:
        """``signal`` then ``wait`` on the same slot row, as one launch."""
        first = self.slot(unit_index, kind, 0)
        _lib.check(self.lib.mfsdp_peer_signal_wait(self._slot_addrs(unit_index, kind), self.flags.tensor.data_ptr(),
                                                   first, self.world, value, self.timeout_ns, self.status.data_ptr(),
                                                   _stream_handle(stream)), "peer_signal_wait")


class DeferredGather:
    """The part of a unit's all-gather that is left to the GEMM which first reads it.

    ``[lo, hi)`` (elements of the full buffer) holds a row-major ``[N, K]`` weight.  The copy jobs are
    grouped by the GEMM's ``bn``-row blocks of that weight; ``need[b]`` is the number of jobs of block b.
    ``complete()`` performs the same copies with the plain pull kernel instead.
    """

    MAX_JOB_BYTES = 48 * 1024   # small jobs: every CTA's gather warps get work and each row block completes early

    def __init__(self, transport: "PeerTransport", shard_buf: SymBuffer, tables: SegmentTables, full: torch.Tensor,
                 lo: int, hi: int, k: int) -> None:
        es = full.element_size()
        assert es == 2 and (hi - lo) % k == 0 and lo % 8 == 0 and k % 8 == 0
        n = (hi - lo) // k
        self.lo, self.hi, self.k, self.n = lo, hi, k, n
        self.bn = 256 if n > 128 else 128
        self.b_ptr = full.data_ptr() + lo * es
        self.full_ptr = full.data_ptr()
        self.budget_ns = transport.ctx.timeout_ns
        self.lib = transport.ctx.lib
        self.status_ptr = transport.ctx.status.data_ptr()
        block = self.bn * k
        nblocks = (n + self.bn - 1) // self.bn
        src, dst, nbytes, flag = [], [], [], []
        psrc, pdst, plen = [], [], []
        need = [0] * nblocks
        max_elems = self.MAX_JOB_BYTES // es
        for r, segs in enumerate(tables.rank_segments):
            for sg in segs:
                g0, g1 = max(sg.global_start, lo), min(sg.global_start + sg.numel, hi)
                if g0 >= g1:
                    continue
                psrc.append(shard_buf.peer_addr[r] + (sg.local_start + g0 - sg.global_start) * es)
                pdst.append(g0)
                plen.append(g1 - g0)
                cur = g0
                while cur < g1:
                    b = (cur - lo) // block
                    end = min(g1, lo + (b + 1) * block, cur + max_elems)
                    src.append(shard_buf.peer_addr[r] + (sg.local_start + cur - sg.global_start) * es)
                    dst.append(full.data_ptr() + cur * es)
                    nbytes.append((end - cur) * es)
                    flag.append(b)
                    need[b] += 1
                    cur = end
        if any(x % 16 for x in src + dst + nbytes):
            raise ValueError("deferred gather pieces are not 16-byte aligned")
        # jobs in block order, so the tiles scheduled first find their rows first
        order = sorted(range(len(src)), key=lambda i: flag[i])
        dev = full.device
        i64 = lambda xs: torch.tensor(xs, dtype=torch.int64, device=dev)          # noqa: E731
        i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=dev)          # noqa: E731
        self.src, self.dst = i64([src[i] for i in order]), i64([dst[i] for i in order])
        self.nbytes, self.flag_idx = i32([nbytes[i] for i in order]), i32([flag[i] for i in order])
        self.njobs = len(order)
        self.need = i32(need)
        first, acc = [], 0
        for c in need:
            first.append(acc)
            acc += c
        self.first = i32(first)                       # jobs are sorted by block: block b owns [first[b], first[b] + need[b])
        # finished jobs per block, then claimed jobs per block (zeroed before every launch)
        self.flags = torch.zeros(2 * nblocks, dtype=torch.int32, device=dev)
        # the schedule starts at the block that holds this rank's own rows: they need no NVLink traffic
        mine = [(max(sg.global_start, lo) - lo) // block for sg in tables.my_segments
                if max(sg.global_start, lo) < min(sg.global_start + sg.numel, hi)]
        self.rotate = min(mine) if mine else 0
        self._plain = {"src": i64(psrc), "dst": i64(pdst), "len": i64(plen), "n": len(psrc), "max": max(plen, default=0)}

    def complete(self, stream=None) -> None:
        """Copy the deferred rows with the plain pull kernel (nobody fused them into a GEMM)."""
        t = self._plain
        run = stream if stream is not None else torch.cuda.current_stream()
        _lib.check(self.lib.mfsdp_ag_pull(self.full_ptr, t["src"].data_ptr(), t["dst"].data_ptr(), t["len"].data_ptr(),
                                          t["n"], t["max"], 2, self.status_ptr, run.cuda_stream), "ag_pull")


class _Slot:
    __slots__ = ("buf", "held", "last_unit", "last_epoch", "event")

    def __init__(self, buf: SymBuffer) -> None:
        self.buf, self.held, self.last_unit, self.last_epoch, self.event = buf, False, None, 0, None


class _FullSlot:
    """A persistent symmetric full-parameter buffer shared by units that are never unsharded together."""

    __slots__ = ("buf", "units", "holder", "last_unit", "last_epoch", "exclusive")

    def __init__(self, buf: SymBuffer, exclusive: bool = False) -> None:
        self.buf = buf
        self.exclusive = exclusive
        self.units: list[str] = []
        self.holder: str | None = None      # unit whose parameters the slot holds right now
        self.last_unit: str | None = None   # previous occupant and the gather epoch it was filled in
        self.last_epoch = 0


def _aligned16(tables: SegmentTables, es: int) -> bool:
    return all((sg.global_start * es) % 16 == 0 and (sg.local_start * es) % 16 == 0 and (sg.numel * es) % 16 == 0
               for segs in tables.rank_segments for sg in segs)


class PeerTransport(LocalTransport):
    kind = "peer"
    needs_symmetric_buffers = True
    accumulates_fp32 = True

    _transports: dict[tuple, "PeerTransport"] = {}

    def __init__(self, ctx: PeerContext) -> None:
        super().__init__()
        self.ctx = ctx
        self.group = ctx.group
        self._unit_index: dict[str, int] = {}
        self._epochs: dict[str, dict[str, int]] = {}
        self._tables: dict[tuple, dict] = {}
        self._rings: dict[int, list[_Slot]] = {}
        self._slot_of_ptr: dict[int, _Slot] = {}
        self.max_slots = int(os.environ.get(RING_ENV, "3"))
        self.launches = 0
        self._ar_state: dict[tuple, dict] = {}
        # NVLS: persistent full-parameter slots (all-gather by multimem.st push)
        self.nvls = ctx.nvls
        # The multicast push delivers every shard to ALL copies of the slot, the sender's own included, so a GPU
        # ingests the whole buffer instead of (W-1)/W of it.  On 2 GPUs that doubles the inbound traffic and the
        # pull gather wins by 0.75 ms per config-2 step (measured back to back); "auto" therefore pushes only
        # from 4 ranks up.  MFSDP_NVLS_GATHER=1 / 0 forces either.
        mode = os.environ.get("MFSDP_NVLS_GATHER", "auto")
        self.nvls_gather = ctx.nvls and (mode == "1" or (mode not in ("0", "1") and ctx.world >= 4))
        self.nvls_reduce = ctx.nvls and os.environ.get("MFSDP_NVLS_REDUCE", "1") != "0"
        self.full_slots_per_class = max(int(os.environ.get(FULL_SLOTS_ENV, "2")), 1)
        self._full_rings: dict[int, list[_FullSlot]] = {}
        self._full_slot_of_unit: dict[str, _FullSlot] = {}

    # ------------------------------------------------------------------ construction
    @classmethod
    def create(cls, group, device: torch.device) -> "PeerTransport | None":
        if device.type != "cuda" or not _lib.available() or _lib.disabled_by_env():
            return None
        # one transport per (group, device): units index one shared flag page, so they must share the
        # unit numbering, the epoch counters and the gradient-slot ring
        key = (id(group), device.index)
        if key in cls._transports:
            return cls._transports[key]
        world = dist.get_world_size(group)
        if world > 16:
            return None
        hosts: list = [None] * world
        dist.all_gather_object(hosts, (socket.gethostname(), torch.cuda.current_device()), group=group)
        if len({h for h, _ in hosts}) != 1:
            return None
        lib = _lib.load(required=True)
        me = torch.cuda.current_device()
        ok = all(d == me or lib.mfsdp_can_access_peer(me, d) for _, d in hosts)
        flags: list = [None] * world
        dist.all_gather_object(flags, bool(ok), group=group)
        if not all(flags):
            return None
        ctx = PeerContext(group, device)
        transport = cls(ctx)
        cls._transports[key] = transport
        return transport

    @classmethod
    def close_all(cls) -> None:
        """Collective, at the end of a program: every rank finishes its own GPU work, then waits for all others,
        before any of them exits and its symmetric (possibly multicast-bound) memory goes away under a peer."""
        for transport in list(cls._transports.values()):
            ctx = transport.ctx
            try:
                torch.cuda.synchronize(ctx.device)
                dist.barrier(group=ctx.group)
            except Exception:  # noqa: BLE001  (the process group may already be gone)
                pass

    def _unit(self, unit_key: str) -> int:
        idx = self._unit_index.get(unit_key)
        if idx is None:
            idx = len(self._unit_index)
            if idx >= MAX_UNITS - 1:        # the last index belongs to the expert-parallel runtime
                raise RuntimeError("too many FSDP units for the peer flag page")
            self._unit_index[unit_key] = idx
            self._epochs[unit_key] = {"shard": 0, "grad": 0}
        return idx

    def describe(self) -> str:
        if not self.nvls:
            return "peer"
        return "peer+nvls(" + "+".join(n for n, on in (("gather", self.nvls_gather), ("reduce", self.nvls_reduce)) if on) + ")"

    # ------------------------------------------------------------------ allocation hooks
    def alloc_persistent(self, numel: int, dtype: torch.dtype, device: torch.device, tag: str = "",
                         symmetric_numel: int | None = None) -> torch.Tensor:
        es = torch.empty((), dtype=dtype).element_size()
        buf = self.ctx.alloc(max(symmetric_numel or numel, 1) * es)
        t = buf.tensor.view(dtype)[:numel]
        self.ctx._by_ptr[t.data_ptr()] = buf
        return t

    def alloc_full_buffer(self, unit_key: str, numel: int, dtype: torch.dtype, tables: SegmentTables,
                          *, exclusive: bool = False) -> torch.Tensor | None:
        """A persistent symmetric full-parameter buffer for the NVLS all-gather, or None when this unit
        keeps the allocator-backed buffer (no multicast, or a layout whose pieces are not 16-byte aligned).

        Collective: units are created in the same order on every rank, so the k-th unit of a size class
        lands in slot ``k % slots`` everywhere.  ``exclusive`` units (never resharded between uses) get
        a slot of their own."""
        es = torch.empty((), dtype=dtype).element_size()
        if not self.nvls_gather or es not in (2, 4) or numel * es < 16 or not _aligned16(tables, es):
            return None
        nbytes = (numel * es + 15) // 16 * 16
        ring = self._full_rings.setdefault(nbytes, [])
        shared = [s for s in ring if not s.exclusive]
        k = sum(len(s.units) for s in shared)       # units of this class placed in shared slots so far
        if exclusive or len(shared) < self.full_slots_per_class:
            buf = self.ctx.alloc(nbytes)
            if not buf.mc_addr:
                return None
            slot = _FullSlot(buf, exclusive)
            ring.append(slot)
        else:
            slot = shared[k % len(shared)]
        slot.units.append(unit_key)
        self._full_slot_of_unit[unit_key] = slot
        self._unit(unit_key)
        return slot.buf.tensor.view(dtype)[:numel]

    def full_slot_available(self, unit_key: str) -> bool:
        slot = self._full_slot_of_unit.get(unit_key)
        return slot is None or slot.holder in (None, unit_key)

    def release_full_buffer(self, unit_key: str) -> None:
        """The unit resharded: once the kernels already enqueued on the current stream are done, peers may
        overwrite its slot (only published when another unit shares the slot)."""
        slot = self._full_slot_of_unit.get(unit_key)
        if slot is None or slot.holder != unit_key:
            return
        slot.holder = None
        # always published: a unit built later (another model in this process) may come to share the slot
        self.ctx.signal(self._unit(unit_key), KIND_FREE, slot.last_epoch, None)
        self.launches += 1

    def acquire_grad_buffer(self, unit_key, numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        es = torch.empty((), dtype=dtype).element_size()
        nbytes = numel * es
        ring = self._rings.setdefault(nbytes, [])
        slot = next((s for s in ring if not s.held and s.last_unit == unit_key), None)
        if slot is None and len(ring) < self.max_slots:
            slot = _Slot(self.ctx.alloc(nbytes))
            ring.append(slot)
        if slot is None:
            free = [s for s in ring if not s.held]
            slot = min(free, key=lambda s: s.last_epoch) if free else None
        if slot is None:
            slot = _Slot(self.ctx.alloc(nbytes))
            ring.append(slot)
        if slot.last_unit is not None and slot.last_epoch > 0:
            # every peer must have finished pulling the previous user's gradients out of this slot;
            # this GPU's own pull is ordered by a stream event, so the spin only ever waits on other GPUs
            if slot.event is not None:
                torch.cuda.current_stream().wait_event(slot.event)
            self.ctx.wait(self._unit(slot.last_unit), KIND_PULLED, slot.last_epoch, None)
            self.launches += 1
        slot.held = True
        slot.last_unit = unit_key
        t = slot.buf.tensor.view(dtype)[:numel]
        self._slot_of_ptr[t.data_ptr()] = slot
        return t

    def release_grad_buffer(self, unit_key, buf: torch.Tensor) -> None:
        slot = self._slot_of_ptr.get(buf.data_ptr())
        if slot is not None:
            slot.held = False

    # ------------------------------------------------------------------ gather
    def _gather_tables(self, unit_key, shard_buf: SymBuffer, tables: SegmentTables, es: int, device) -> dict:
        key = ("ag", unit_key, shard_buf.tensor.data_ptr())
        t = self._tables.get(key)
        if t is None:
            src, dst, ln = [], [], []
            for r, local_off, global_off, numel in tables.pull_rows():    # merged runs of the layout's plan
                src.append(shard_buf.peer_addr[r] + local_off * es)
                dst.append(global_off)
                ln.append(numel)
            t = {"src": torch.tensor(src, dtype=torch.int64, device=device),
                 "dst": torch.tensor(dst, dtype=torch.int64, device=device),
                 "len": torch.tensor(ln, dtype=torch.int64, device=device), "n": len(src), "max": max(ln, default=0)}
            self._tables[key] = t
        return t

    def _push_tables(self, unit_key, tables: SegmentTables, es: int, device) -> dict:
        key = ("push", unit_key)
        t = self._tables.get(key)
        if t is None:
            segs = tables.my_segments
            t = {"src": torch.tensor([s.local_start * es for s in segs], dtype=torch.int64, device=device),
                 "dst": torch.tensor([s.global_start * es for s in segs], dtype=torch.int64, device=device),
                 "len": torch.tensor([s.numel * es for s in segs], dtype=torch.int64, device=device), "n": len(segs),
                 "max": max((s.numel * es for s in segs), default=0)}
            self._tables[key] = t
        return t

    supports_deferred_gather = True

    def _deferred_tables(self, unit_key, shard_buf: SymBuffer, tables: SegmentTables, full, defer) -> tuple:
        """(plan for the deferred range, pull tables for everything else), cached per unit."""
        lo, hi, k = defer
        key = ("ag_defer", unit_key, shard_buf.tensor.data_ptr(), full.data_ptr(), lo, hi, k)
        hit = self._tables.get(key)
        if hit is None:
            es = full.element_size()
            plan = DeferredGather(self, shard_buf, tables, full, lo, hi, k)
            src, dst, ln = [], [], []
            for r, segs in enumerate(tables.rank_segments):
                for sg in segs:
                    g0, g1 = sg.global_start, sg.global_start + sg.numel
                    for a, b in ((g0, min(g1, lo)), (max(g0, hi), g1)):
                        if a < b:
                            src.append(shard_buf.peer_addr[r] + (sg.local_start + a - g0) * es)
                            dst.append(a)
                            ln.append(b - a)
            dev = full.device
            rest = {"src": torch.tensor(src, dtype=torch.int64, device=dev),
                    "dst": torch.tensor(dst, dtype=torch.int64, device=dev),
                    "len": torch.tensor(ln, dtype=torch.int64, device=dev), "n": len(src), "max": max(ln, default=0)}
            hit = (plan, rest)
            self._tables[key] = hit
        return hit

    def _validate_pull(self, t: dict, full: torch.Tensor, shard_buf: SymBuffer, run) -> None:
        ctx = self.ctx
        lo = (_u64 * ctx.world)(*shard_buf.peer_addr)
        hi = (_u64 * ctx.world)(*[a + shard_buf.nbytes for a in shard_buf.peer_addr])
        _lib.check(ctx.lib.mfsdp_validate_pull_table(t["src"].data_ptr(), t["dst"].data_ptr(), t["len"].data_ptr(),
                                                     t["n"], full.numel(), full.element_size(), lo, hi, ctx.world,
                                                     ctx.status.data_ptr(), run.cuda_stream), "validate_pull_table")
        self.launches += 1

    def gather(self, shard, full, tables: SegmentTables, *, stream=None, unit_key=None,
               defer: tuple | None = None, wait_current: bool = True) -> MatrixCollectiveHandle:
        """``wait_current=False``: the caller has already ordered ``stream`` behind everything the gather
        depends on (the event of the unit's fused update); it is then not made to wait for the current stream."""
        buf = self.ctx.lookup(shard)
        if buf is None:
            raise RuntimeError("peer gather needs a shard that lives in symmetric memory")
        t_host = time.perf_counter()
        ui = self._unit(unit_key)
        ep = self._epochs[unit_key]
        ep["shard"] += 1
        e = ep["shard"]
        es = full.element_size()
        ctx = self.ctx
        cur = torch.cuda.current_stream()
        run = stream if stream is not None else cur
        if stream is not None and wait_current:
            stream.wait_stream(cur)
        span = _tl.open_span(unit_key or "", "all_gather", run, nbytes=full.numel() * es)
        fslot = self._full_slot_of_unit.get(unit_key)
        plan = None
        if fslot is not None and fslot.buf.tensor.data_ptr() == full.data_ptr():
            # ---- NVLS: push my shard into every rank's copy of the slot through the switch
            if fslot.holder not in (None, unit_key):
                raise RuntimeError(
                    f"full-parameter slot of {unit_key} still holds {fslot.holder}: more units are unsharded at once "
                    f"than there are slots per size class; raise {FULL_SLOTS_ENV} or lower the prefetch depth")
            if fslot.last_unit is not None and fslot.last_unit != unit_key and fslot.last_epoch > 0:
                # every rank (this one included) has stopped reading the previous occupant
                ctx.wait(self._unit(fslot.last_unit), KIND_FREE, fslot.last_epoch, run)
                self.launches += 1
            fslot.holder, fslot.last_unit, fslot.last_epoch = unit_key, unit_key, e
            t = self._push_tables(unit_key, tables, es, full.device)
            t_tables = time.perf_counter()
            _lib.check(ctx.lib.mfsdp_ag_push_mc(shard.data_ptr(), fslot.buf.mc_addr, t["src"].data_ptr(),
                                                t["dst"].data_ptr(), t["len"].data_ptr(), t["n"], t["max"],
                                                ctx.status.data_ptr(), run.cuda_stream), "ag_push_mc")
            # "my shard has landed everywhere" / "everybody's shard has landed here"
            ctx.signal_wait(ui, KIND_SHARD, e, run)
            self.launches += 2
            impl = "ag_push_mc"
        else:
            if defer is not None and es == 2:
                plan, t = self._deferred_tables(unit_key, buf, tables, full, defer)
            else:
                t = self._gather_tables(unit_key, buf, tables, es, full.device)
            t_tables = time.perf_counter()
            ctx.signal_wait(ui, KIND_SHARD, e, run)
            if ctx.debug_bounds:
                self._validate_pull(t, full, buf, run)
            _lib.check(ctx.lib.mfsdp_ag_pull(full.data_ptr(), t["src"].data_ptr(), t["dst"].data_ptr(),
                                             t["len"].data_ptr(), t["n"], t["max"], es, ctx.status.data_ptr(),
                                             run.cuda_stream), "ag_pull")
            self.launches += 2
            impl = "ag_pull+gemm" if plan is not None else "ag_pull"
        _tl.close_span(span, run, impl=impl)
        ev = None
        if stream is not None:
            ev = torch.cuda.Event()
            ev.record(stream)
        t_end = time.perf_counter()
        h = MatrixCollectiveHandle(event=ev, info={
            "kind": "all_gather", "impl": impl, "backend": self.kind,
            "bytes": full.numel() * es, "count": 1,
            "sync_mode": "stream_event" if stream is not None else "stream_order",
            # host time inside the call: table lookup / slot handshake, then flag and kernel launches
            "host_phases_ms": {"tables": (t_tables - t_host) * 1e3, "launch": (t_end - t_tables) * 1e3}})
        h.deferred = plan
        h.span = span
        return h

    # ------------------------------------------------------------------ all-reduce (HSDP replicate group)
    def all_reduce(self, tensor, group, *, scale=None):
        """Sum ``tensor`` over ``group`` with the same kernels as the reduce-scatter: every rank publishes
        its values in a symmetric staging buffer, waits for the others and either reads all of them
        (fixed rank order, fp32 sum) or, with NVLS, sums its slice through the switch and stores the
        result to every copy (``multimem.ld_reduce`` + ``multimem.st``).

        Used for the dp_replicate step of HSDP after the dp_shard reduce-scatter (the reference runs
        ``dist.all_reduce`` + ``div_`` synchronously there, matrix_fsdp/runtime/flat_buffer.py:1472-1480).
        """
        rep = PeerTransport.create(group, tensor.device) if tensor.is_cuda else None
        if rep is None or tensor.dtype not in (torch.float32, torch.bfloat16) or not tensor.is_contiguous() \
                or dist.get_world_size(group) == 1:
            return super().all_reduce(tensor, group, scale=scale)
        return rep._all_reduce_own_group(tensor, scale)

    def _all_reduce_own_group(self, tensor: torch.Tensor, scale) -> None:
        ctx = self.ctx
        key = ("ar", tensor.numel(), tensor.dtype)   # one staging buffer per size: successive exchanges are ordered by the flags
        st = self._ar_state.get(key)
        if st is None:
            buf = ctx.alloc((tensor.numel() * tensor.element_size() + 15) // 16 * 16)
            dev = tensor.device
            st = {"buf": buf, "view": buf.tensor.view(tensor.dtype)[:tensor.numel()], "epoch": 0,
                  "unit": self._unit(key),
                  "g": torch.zeros(1, dtype=torch.int64, device=dev), "l": torch.zeros(1, dtype=torch.int64, device=dev),
                  "len": torch.tensor([tensor.numel()], dtype=torch.int64, device=dev)}
            self._ar_state[key] = st
        run = torch.cuda.current_stream()
        ui = st["unit"]
        is_bf16 = int(tensor.dtype == torch.bfloat16)
        use_mc = bool(self.nvls_reduce and st["buf"].mc_addr and tensor.numel() % 8 == 0)
        if st["epoch"] > 0 and not use_mc:
            ctx.wait(ui, KIND_PULLED, st["epoch"], run)          # everyone has read the previous exchange
        st["epoch"] += 1
        e = st["epoch"]
        st["view"].copy_(tensor.view(-1))
        ctx.signal_wait(ui, KIND_GRAD, e, run)
        if use_mc:
            _lib.check(ctx.lib.mfsdp_ar_mc(st["buf"].mc_addr, tensor.numel(), is_bf16, ctx.rank, ctx.world,
                                           float(1.0 if scale is None else scale), ctx.status.data_ptr(),
                                           run.cuda_stream), "ar_mc")
            ctx.signal_wait(ui, KIND_PULLED, e, run)             # every slice has been stored everywhere
            tensor.view(-1).copy_(st["view"])
            self.launches += 5
            return
        ptrs = (_u64 * ctx.world)(*st["buf"].peer_addr)
        _lib.check(ctx.lib.mfsdp_rs_pull_reduce(
            ptrs, ctx.world, ctx.rank, tensor.data_ptr(), st["g"].data_ptr(), st["l"].data_ptr(), st["len"].data_ptr(),
            1, tensor.numel(), is_bf16, is_bf16, 0, float(1.0 if scale is None else scale), ctx.status.data_ptr(),
            run.cuda_stream), "rs_pull_reduce")
        ctx.signal(ui, KIND_PULLED, e, run)
        self.launches += 5

    # ------------------------------------------------------------------ reduce
    def _reduce_tables(self, unit_key, tables: SegmentTables, device) -> dict:
        key = ("rs", unit_key)
        t = self._tables.get(key)
        if t is None:
            segs = tables.my_segments
            t = {"g": torch.tensor([s.global_start for s in segs], dtype=torch.int64, device=device),
                 "l": torch.tensor([s.local_start for s in segs], dtype=torch.int64, device=device),
                 "len": torch.tensor([s.numel for s in segs], dtype=torch.int64, device=device), "n": len(segs),
                 "max": max((s.numel for s in segs), default=0),
                 "vec8": all(s.global_start % 8 == 0 and s.local_start % 8 == 0 and s.numel % 8 == 0 for s in segs)}
            self._tables[key] = t
        return t

    def reduce_update(self, full_grad, tables: SegmentTables, update: dict, *, scale=None, stream=None,
                      unit_key=None) -> MatrixCollectiveHandle:
        """Reduce-scatter fused with the sharded AdamW update (``update``: p, m, v, p_lp tensors and
        lr, beta1, beta2, eps, weight_decay, step); the reduced gradient is never written."""
        return self.reduce(full_grad, None, tables, scale=scale, stream=stream, unit_key=unit_key, update=update)

    def reduce(self, full_grad, out_shard, tables: SegmentTables, *, scale=None, stream=None, unit_key=None,
               accumulate: bool = False, update: dict | None = None) -> MatrixCollectiveHandle:
        buf = self.ctx.lookup(full_grad)
        if buf is None:
            raise RuntimeError("peer reduce needs a gradient buffer from acquire_grad_buffer()")
        if full_grad.dtype not in (torch.bfloat16, torch.float32) or \
                (update is None and out_shard.dtype not in (torch.bfloat16, torch.float32)):
            raise TypeError("peer reduce supports bf16 / fp32 gradients")
        t_host = time.perf_counter()
        ui = self._unit(unit_key)
        ep = self._epochs[unit_key]
        ep["grad"] += 1
        e = ep["grad"]
        slot = self._slot_of_ptr.get(full_grad.data_ptr())
        if slot is not None:
            slot.last_epoch = e
        t = self._reduce_tables(unit_key, tables, full_grad.device)
        t_tables = time.perf_counter()
        cur = torch.cuda.current_stream()
        run = stream if stream is not None else cur
        if stream is not None:
            stream.wait_stream(cur)
        ctx = self.ctx
        span = _tl.open_span(unit_key or "", "reduce_scatter", run,
                             nbytes=full_grad.numel() * full_grad.element_size())
        ctx.signal_wait(ui, KIND_GRAD, e, run)
        in_bf16 = int(full_grad.dtype == torch.bfloat16)
        sc = float(1.0 if scale is None else scale)
        use_mc = bool(self.nvls_reduce and buf.mc_addr and t["vec8"]
                      and (out_shard is None or out_shard.data_ptr() % 16 == 0))
        if ctx.debug_bounds:
            shard_numel = update["p"].numel() if update is not None else out_shard.numel()
            _lib.check(ctx.lib.mfsdp_validate_reduce_table(t["g"].data_ptr(), t["l"].data_ptr(), t["len"].data_ptr(),
                                                           t["n"], full_grad.numel(), shard_numel,
                                                           ctx.status.data_ptr(), run.cuda_stream),
                       "validate_reduce_table")
            self.launches += 1
        if update is not None:
            u = update
            tail = (u["p"].data_ptr(), u["m"].data_ptr(), u["v"].data_ptr(),
                    u["p_lp"].data_ptr() if u.get("p_lp") is not None else None,
                    float(u["lr"]), float(u["beta1"]), float(u["beta2"]), float(u["eps"]), float(u["weight_decay"]),
                    int(u["step"]), ctx.status.data_ptr(), run.cuda_stream)
            if use_mc:
                _lib.check(ctx.lib.mfsdp_rs_mc_adamw(buf.mc_addr, t["g"].data_ptr(), t["l"].data_ptr(),
                                                     t["len"].data_ptr(), t["n"], t["max"], in_bf16, sc, *tail),
                           "rs_mc_adamw")
            else:
                ptrs = (_u64 * ctx.world)(*buf.peer_addr)
                _lib.check(ctx.lib.mfsdp_rs_pull_adamw(ptrs, ctx.world, ctx.rank, t["g"].data_ptr(), t["l"].data_ptr(),
                                                       t["len"].data_ptr(), t["n"], t["max"], in_bf16, sc, *tail),
                           "rs_pull_adamw")
            impl = "rs_mc_adamw" if use_mc else "rs_pull_adamw"
        else:
            out_bf16 = int(out_shard.dtype == torch.bfloat16)
            if use_mc:
                _lib.check(ctx.lib.mfsdp_rs_mc_reduce(buf.mc_addr, out_shard.data_ptr(), t["g"].data_ptr(),
                                                      t["l"].data_ptr(), t["len"].data_ptr(), t["n"], t["max"],
                                                      in_bf16, out_bf16, int(accumulate), sc, ctx.status.data_ptr(),
                                                      run.cuda_stream), "rs_mc_reduce")
            else:
                ptrs = (_u64 * ctx.world)(*buf.peer_addr)
                _lib.check(ctx.lib.mfsdp_rs_pull_reduce(
                    ptrs, ctx.world, ctx.rank, out_shard.data_ptr(), t["g"].data_ptr(), t["l"].data_ptr(),
                    t["len"].data_ptr(), t["n"], t["max"], in_bf16, out_bf16, int(accumulate), sc,
                    ctx.status.data_ptr(), run.cuda_stream), "rs_pull_reduce")
            impl = "rs_mc_reduce" if use_mc else "rs_pull_reduce"
        ctx.signal(ui, KIND_PULLED, e, run)
        self.launches += 3
        _tl.close_span(span, run, impl=impl)
        ev = torch.cuda.Event()
        ev.record(run)
        if slot is not None:
            slot.event = ev
        if stream is None:
            ev = None
        t_end = time.perf_counter()
        h = MatrixCollectiveHandle(event=ev, info={
            "kind": "reduce_scatter", "impl": impl, "backend": self.kind,
            "bytes": full_grad.numel() * full_grad.element_size(), "count": 1,
            "sync_mode": "stream_event" if stream is not None else "stream_order",
            "host_phases_ms": {"tables": (t_tables - t_host) * 1e3, "launch": (t_end - t_tables) * 1e3}})
        h.span = span
        return h

    def check_health(self) -> None:
        """Raise if any bounded wait on this device ran out (reads the status word: a device sync)."""
        from ..ops import kernels

        kernels.check_status(self.ctx.device)
