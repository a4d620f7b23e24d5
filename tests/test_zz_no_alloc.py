"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the point where they need this op
(no allocator of their own, or one that must not be entered there), so ``mfsdp_rmsnorm_bwd_noalloc``
keeps its fp32 scratch inside the library.  The test drives it with ctypes exactly as a C caller
would, twice in a row (every call reuses the same built-in scratch), and checks both results against
the regular entry point, which takes its scratch from the caller, and against the same math written
in fp32 PyTorch.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    from matrix_fsdp_b200.ops import kernels as K
    from matrix_fsdp_b200.ops import lib

    L = lib.load(required=True)
    fn = L.mfsdp_rmsnorm_bwd_noalloc
    vp = C.c_void_p
    fn.argtypes = [vp, vp, vp, vp, vp, vp, vp, C.c_int, C.c_longlong, C.c_int, vp]
    fn.restype = C.c_int
    stream = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(0)
    for call, (rows, H) in enumerate([(777, 2048), (300, 4096)]):
        x = torch.randn(rows, H, device="cuda").bfloat16()
        dy = torch.randn(rows, H, device="cuda").bfloat16()
        dres = torch.randn(rows, H, device="cuda").bfloat16()
        w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
        _, rstd = K.rmsnorm_fwd(x, w, 1e-5)
        ref_dx, ref_dw = K.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
        dx = torch.empty_like(x)
        dw = torch.empty(H, device="cuda", dtype=torch.bfloat16)
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(),
                dw.data_ptr(), 0, rows, H, stream)
        assert rc == 0, f"call {call} returned {rc}"
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        assert _rel(dx, ref_dx) < 1e-2
        assert _rel(dw, ref_dw) < 1e-2
        # the op itself in fp32: dx = rstd (g - xhat mean(g xhat)) + dres with g = dy w, dw = sum_rows dy xhat
        xhat = x.float() * rstd[:, None]
        g = dy.float() * w.float()
        fp32_dx = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True)) + dres.float()
        fp32_dw = (dy.float() * xhat).sum(0)
        assert _rel(dx, fp32_dx) < 1e-2
        assert _rel(dw, fp32_dw) < 1e-2
    # sizes beyond the built-in scratch are refused with the documented code
    assert fn(None, None, None, None, None, None, None, 0, 16, 8192 + 8, stream) == -2
    assert fn(None, None, None, None, None, None, None, 0, 16, 100, stream) == -2
