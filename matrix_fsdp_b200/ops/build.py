"""In-tree build of the sm_100a kernel library (``libmfsdp_kernels.so``).

The kernels are plain CUDA C++ with ``extern "C"`` launchers (no torch headers), so a
full rebuild is a handful of nvcc invocations that cross-compile without a GPU.  The
shared object is written next to this file; Python reaches it through ctypes
(:mod:`matrix_fsdp_b200.ops.lib`).

The reference builds its two optional torch extensions from ``setup.py:17-96`` with no
``-gencode`` at all; here every translation unit is compiled for ``sm_100a`` only.

Run ``python -m matrix_fsdp_b200.ops.build`` to (re)build; ``--force`` ignores
timestamps, ``--verbose`` adds ``-Xptxas -v``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
OUT_DIR = Path(__file__).resolve().parent
LIB_NAME = "libmfsdp_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def lib_path() -> Path:
    return OUT_DIR / LIB_NAME


def is_stale() -> bool:
    lib = lib_path()
    if not lib.exists():
        return True
    t = lib.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link the shared library."""
    if not force and not is_stale():
        return lib_path()
    nvcc = _nvcc()
    obj_dir = OUT_DIR / "build"
    obj_dir.mkdir(exist_ok=True)
    common = [
        nvcc, *ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo", "--use_fast_math",
        "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
    ]
    if verbose:
        common += ["-Xptxas", "-v"]

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        hdr_time = max([p.stat().st_mtime for p in list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))] or [0])
        if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_time):
            return obj
        cmd = common + ["-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose and res.stderr:
            sys.stderr.write(res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(compile_one, sources()))
    # Shared cudart: inside a torch process the loader binds to the libcudart.so.12 torch already
    # loaded, so both sides see one runtime (same per-thread current device, same primary context).
    link = [nvcc, *ARCH_FLAGS, "-shared", "-cudart", "shared", "-o", str(lib_path()), *map(str, objs)]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib_path()


if __name__ == "__main__":
    out = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(out)
