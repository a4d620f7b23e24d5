"""Report what the peer-memory data plane can use on this machine.

    python -m matrix_fsdp_b200.tools.device_api_probe

Prints a JSON object: kernel library present / loadable, GPUs and their pairwise peer access, NCCL
version bundled with torch and whether it is new enough for NCCL's device API (2.28.0) and GIN
(2.28.7).  This framework's own one-sided kernels need only peer access and CUDA IPC.

Parity: ``matrix_fsdp/tools/nccl_device_api_probe.py:1-61`` and ``kernels/gin/probe.py:1-192``.
"""
from __future__ import annotations

import json

import torch

from ..ops import lib


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
