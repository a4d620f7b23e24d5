"""Report what the peer-memory data plane can use on this machine.

    python -m matrix_fsdp_b200.tools.device_api_probe

Prints a JSON object: kernel library present / loadable, GPUs and their pairwise peer access, NCCL
version bundled with torch and whether it is new enough for NCCL's device API (2.28.0) and GIN
(2.28.7), and -- from :func:`probe_nccl_features` -- whether the NCCL *headers* found on this machine
declare those interfaces and whether the NCCL *library* loaded into this process exports their host
entry points.  This framework's own one-sided kernels need only peer access and symmetric memory.

Parity: ``matrix_fsdp/tools/nccl_device_api_probe.py:1-61`` and ``kernels/gin/probe.py:1-192``.
"""
from __future__ import annotations

import ctypes
import json
import os
import sysconfig
from pathlib import Path

import torch

from ..ops import lib

# feature -> (oldest NCCL runtime that has it, tokens one of which its headers declare, host entry points
# the shared library exports when it was built with it)
NCCL_FEATURES: dict[str, tuple[tuple[int, int, int], tuple[str, ...], tuple[str, ...]]] = {
    "device_api": ((2, 28, 0), ("ncclDevComm", "ncclDevCommCreate", "ncclCommWindowRegister"),
                   ("ncclDevCommCreate", "ncclCommWindowRegister")),
    "gin": ((2, 28, 7), ("ncclGin", "NCCL_GIN", "ncclLsa"), ()),
}
_FEATURE_ORDER = ("device_api", "gin")       # a later feature needs every earlier one


def nccl_runtime_version() -> tuple[int, ...] | None:
    """NCCL version torch reports, as a tuple, whatever form (tuple, packed int, dotted string) it comes in."""
    try:
        v = torch.cuda.nccl.version()
    except Exception:  # noqa: BLE001
        return None
    if isinstance(v, int):
        return (v // 1000, v % 1000 // 100, v % 100) if v < 20000 else (v // 10000, v % 10000 // 100, v % 100)
    if isinstance(v, str):
        nums = tuple(int(x) for x in v.split(".") if x.isdigit())
        return nums or None
    try:
        return tuple(int(x) for x in v)
    except TypeError:
        return None


def _include_dirs(extra: tuple[str, ...]) -> list[Path]:
    env = os.environ
    wanted = [Path(p) for p in extra]
    wanted += [Path(env[k]) / sub for k, sub in (("NCCL_INCLUDE_DIR", ""), ("NCCL_ROOT", "include"), ("CUDA_HOME", "include"))
               if env.get(k)]
    wanted += [Path(sysconfig.get_paths()["purelib"]) / "nvidia" / "nccl" / "include", Path("/usr/local/cuda/include"),
               Path("/usr/include"), Path("/usr/local/include")]
    out: list[Path] = []
    for p in wanted:
        try:
            r = p.expanduser().resolve()
        except OSError:
            continue
        if r.is_dir() and r not in out:
            out.append(r)
    return out


def _loaded_nccl_library() -> str | None:
    """Path of the NCCL shared object mapped into this process (torch loads it with CUDA builds)."""
    try:
        with open("/proc/self/maps") as f:
            for line in f:
                path = line.rsplit(" ", 1)[-1].strip()
                if "libnccl" in os.path.basename(path):
                    return path
    except OSError:
        pass
    return None


def probe_nccl_features(*, extra_include_dirs: tuple[str, ...] = (), library: str | None = None) -> dict:
    """Which NCCL interfaces are usable here: runtime version, header declarations, exported entry points.

    A feature is *ready* when CUDA is available, the runtime is new enough, some ``nccl*.h`` in the include
    directories declares one of its tokens and every earlier feature is ready.  ``reason`` names the first
    thing that is missing (or says that everything is visible).  ``extra_include_dirs`` are searched first;
    ``library`` overrides the shared object whose exports are checked."""
    version = nccl_runtime_version()
    dirs = _include_dirs(tuple(extra_include_dirs))
    headers = [h for d in dirs for h in (*sorted(d.glob("nccl*.h")), *sorted(d.glob("nccl*/**/*.h")))]
    text = ""
    for h in headers:
        try:
            text += h.read_text(errors="ignore") + "\n"
        except OSError:
            pass
    lib_path = library or _loaded_nccl_library()
    handle = None
    if lib_path:
        try:
            handle = ctypes.CDLL(lib_path)
        except OSError:
            handle = None
    cuda = torch.cuda.is_available()
    out: dict = {"cuda_available": cuda, "nccl_version": version, "include_dirs": [str(d) for d in dirs],
                 "headers": [str(h) for h in headers], "library": lib_path, "features": {}}
    reason, earlier_ready = None, True
    if not cuda:
        reason = "CUDA is not available in this Python environment."
    elif version is None:
        reason = "torch did not report an NCCL runtime version."
    for name in _FEATURE_ORDER:
        need, tokens, symbols = NCCL_FEATURES[name]
        padded = tuple(version or ()) + (0,) * 3
        new_enough = version is not None and padded[:3] >= need
        declared = any(t in text for t in tokens)
        exported = None if handle is None or not symbols else all(hasattr(handle, s) for s in symbols)
        ready = bool(cuda and earlier_ready and new_enough and declared)
        out["features"][name] = {"runtime_new_enough": new_enough, "declared_in_headers": declared,
                                 "exported_by_library": exported, "ready": ready}
        if reason is None and not ready:
            if not new_enough:
                reason = f"NCCL runtime {version} is older than {need}, which {name} needs."
            elif not headers:
                reason = "No NCCL headers were found."
            else:
                reason = f"The NCCL headers declare none of {', '.join(tokens)} ({name})."
        earlier_ready = ready
    out["reason"] = reason or "The NCCL device API and GIN declarations are visible."
    return out


def probe() -> dict:
    out: dict = {"kernel_library": str(lib.lib_path()), "kernel_library_present": lib.lib_path().exists(),
                 "kernel_library_loadable": lib.available(), "cuda_available": torch.cuda.is_available()}
    try:
        v = torch.cuda.nccl.version()
        out["nccl_version"] = ".".join(str(x) for x in v)
        out["nccl_device_api"] = tuple(v) >= (2, 28, 0)
        out["nccl_gin"] = tuple(v) >= (2, 28, 7)
    except Exception as exc:  # noqa: BLE001
        out["nccl_version"] = f"unavailable: {exc}"
    out["nccl_features"] = probe_nccl_features()
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        out["gpus"] = [torch.cuda.get_device_name(i) for i in range(n)]
        L = lib.load()
        if L is not None:
            import matrix_fsdp_b200.parallel.peer  # noqa: F401

            out["peer_access"] = [[bool(i == j or L.mfsdp_can_access_peer(i, j)) for j in range(n)] for i in range(n)]
        out["peer_transport_usable"] = bool(L is not None and n >= 1)
    return out


def main() -> int:
    print(json.dumps(probe(), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
