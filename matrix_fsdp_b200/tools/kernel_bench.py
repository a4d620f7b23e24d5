"""Time single kernels of the library against their rooflines (one GPU).

    python -m matrix_fsdp_b200.tools.kernel_bench --what gemm|elementwise|muon|attention [--small]

Every number is CUDA-event timed after warm-up; between iterations the inputs rotate through enough
distinct buffers to exceed L2.  Fractions are of the measured peaks in ``MEASURED_PEAKS.json``
(fallback 6650 GB/s, 1590 TFLOP/s).  ``--small`` runs one tiny case, sized for profiler captures.

The reference has no single-kernel benchmark; its closest tools are the copy-in and parameter-materialisation
micro-benchmarks inside ``test/fsdp/bench_fsdp2_compare.py:2686-2770``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks() -> tuple[float, float, str]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def _time(fns, iters: int = 20, warmup: int = 3) -> float:
    for i in range(warmup):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fns[i % len(fns)]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_gemm(small: bool, shape=None):
    from ..ops import kernels as K

    hbm, tf, src = _peaks()
    shapes = [tuple(shape)] if shape else [(1024, 1024, 1024)] if small else [
        (4096, 6144, 2048), (4096, 2048, 2048), (4096, 11008, 2048), (4096, 2048, 5504), (4096, 32000, 2048),
        (8192, 8192, 8192), (4096, 12288, 4096), (4096, 4096, 11008)]
    rows = []
    for M, N, Kd in shapes:
        nbuf = max(2, int(160e6 // ((M * Kd + N * Kd + M * N) * 2)) + 1) if not small else 2
        a = [torch.randn(M, Kd, device="cuda").bfloat16() for _ in range(nbuf)]
        b = [torch.randn(N, Kd, device="cuda").bfloat16() for _ in range(nbuf)]
        o = [torch.empty(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(nbuf)]
        bt = [x.t().contiguous() for x in b]
        at = [x.t().contiguous() for x in a]
        fl = 2.0 * M * N * Kd / 1e9
        t_nt = _time([lambda i=i: K.gemm(a[i], b[i], out=o[i]) for i in range(nbuf)])
        t_nn = _time([lambda i=i: K.gemm(a[i], bt[i], b_mn_major=True, out=o[i]) for i in range(nbuf)])
        t_tn = _time([lambda i=i: K.gemm(at[i], bt[i], a_mn_major=True, b_mn_major=True, out=o[i]) for i in range(nbuf)])
        t_lib = _time([lambda i=i: torch.matmul(a[i], b[i].t(), out=o[i]) for i in range(nbuf)])
        # the same three products on the single-CTA kernel (128 x 256 tiles); the default above is the two-CTA
        # cta_group::2 kernel with 256 x 256 tiles
        s_nt = _time([lambda i=i: K.gemm(a[i], b[i], out=o[i], force_bn=256) for i in range(nbuf)])
        s_nn = _time([lambda i=i: K.gemm(a[i], bt[i], b_mn_major=True, out=o[i], force_bn=256) for i in range(nbuf)])
        s_tn = _time([lambda i=i: K.gemm(at[i], bt[i], a_mn_major=True, b_mn_major=True, out=o[i], force_bn=256)
                      for i in range(nbuf)])
        rows.append({"shape": [M, N, Kd], "fwd_tflops": fl / t_nt, "dgrad_tflops": fl / t_nn, "wgrad_tflops": fl / t_tn,
                     "single_cta_fwd_tflops": fl / s_nt, "single_cta_dgrad_tflops": fl / s_nn,
                     "single_cta_wgrad_tflops": fl / s_tn, "cublas_tflops": fl / t_lib,
                     "fwd_frac_of_%s_peak" % src: fl / t_nt / tf, "fwd_vs_cublas": t_lib / t_nt,
                     "single_cta_fwd_vs_cublas": t_lib / s_nt})
        print(json.dumps(rows[-1]), flush=True)
    K.check_status()
    return rows


def bench_elementwise(small: bool):
    from ..ops import kernels as K

    hbm, tf, src = _peaks()
    T, H, F, V = (512, 2048, 5504, 32000) if small else (16384, 2048, 5504, 32000)
    rows = []
    x = torch.randn(T, H, device="cuda").bfloat16()
    w = torch.ones(H, device="cuda").bfloat16()
    dy = torch.randn_like(x)
    y, rstd = K.rmsnorm_fwd(x, w, 1e-5)
    gu = torch.randn(T, 2 * F, device="cuda").bfloat16()
    dh = torch.randn(T, F, device="cuda").bfloat16()
    n = 100_000_000 if not small else 4_000_000
    p = torch.randn(n, device="cuda")
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    g = torch.randn(n, device="cuda").bfloat16()
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    rowsV = 4096 if not small else 256
    logits = torch.randn(rowsV, V, device="cuda").bfloat16()
    tgt = torch.randint(0, V, (rowsV,), device="cuda")
    cases = [
        ("rmsnorm_fwd", lambda: K.rmsnorm_fwd(x, w, 1e-5), 2 * T * H * 2),
        ("rmsnorm_bwd", lambda: K.rmsnorm_bwd(dy, x, w, rstd, dres=dy), 4 * T * H * 2),
        ("swiglu_fwd", lambda: K.swiglu_fwd(gu), 3 * T * F * 2),
        ("swiglu_bwd", lambda: K.swiglu_bwd(dh, gu), 5 * T * F * 2),
        ("adamw_flat", lambda: K.adamw_flat_(p, m, v, g, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                                             step=3, p_lp=lp), n * 28),
        ("cross_entropy", lambda: K.cross_entropy_(logits, tgt, 1.0 / rowsV), 2 * rowsV * V * 2),
    ]
    for name, fn, nbytes in cases:
        ms = _time([fn])
        gbs = nbytes / (ms * 1e-3) / 1e9
        rows.append({"kernel": name, "ms": ms, "gb_per_s": gbs, "frac_of_%s_hbm" % src: gbs / hbm})
        print(json.dumps(rows[-1]), flush=True)
    return rows


def bench_muon(small: bool):
    from ..optim.muon import newton_schulz_reference, newton_schulz_sm100
    from ..planning.planner_eval import newton_schulz_flops

    hbm, tf, src = _peaks()
    shapes = [(512, 512)] if small else [(2048, 2048), (5504, 2048), (4096, 4096), (11008, 4096)]
    rows = []
    for r, c in shapes:
        g = torch.randn(r, c, device="cuda")
        x = (g / g.norm()).bfloat16()
        ms = _time([lambda: newton_schulz_sm100(x, steps=5)], iters=5)
        ms_ref = _time([lambda: newton_schulz_reference(g, steps=5)], iters=5)
        fl = newton_schulz_flops(r, c, 5) / 1e9
        rows.append({"shape": [r, c], "ours_ms": ms, "torch_ms": ms_ref, "ours_tflops": fl / ms,
                     "frac_of_%s_peak" % src: fl / ms / tf, "speedup_vs_torch": ms_ref / ms})
        print(json.dumps(rows[-1]), flush=True)
    return rows


def bench_attention(small: bool):
    """Causal attention forward/backward (head_dim 128) against the library SDPA kernel.

    FLOPs: forward 4*B*nH*S^2*128/2 (two GEMMs, causal half); backward counted as 2.5x forward.
    """
    import torch.nn.functional as F

    from ..ops import attention as A
    from ..ops import kernels as K

    _, tf, src = _peaks()
    cases = [(1, 2048, 16)] if small else [(4, 1024, 16), (2, 4096, 32), (1, 8192, 32)]
    rows = []
    for B, S, nH in cases:
        hd, H = 128, nH * 128
        qkv = torch.randn(B * S, 3 * H, device="cuda", dtype=torch.bfloat16)
        fl = 4.0 * B * nH * S * S * hd / 2 / 1e9
        t_f = _time([lambda: A.attention_fwd(qkv, B, S, nH, hd)])
        out, lse = A.attention_fwd(qkv, B, S, nH, hd)
        do = torch.randn_like(out)
        t_b = _time([lambda: A.attention_bwd(do, qkv, out, lse, B, S, nH, hd)])
        q, k, v = (qkv[:, i * H:(i + 1) * H].view(B, S, nH, hd).transpose(1, 2) for i in range(3))
        t_lib = _time([lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True)])
        rows.append({"B": B, "S": S, "heads": nH, "fwd_ms": t_f, "fwd_tflops": fl / t_f, "bwd_ms": t_b,
                     "bwd_tflops": 2.5 * fl / t_b, "sdpa_fwd_ms": t_lib, "sdpa_fwd_tflops": fl / t_lib,
                     "fwd_frac_of_%s_peak" % src: fl / t_f / tf})
        print(json.dumps(rows[-1]), flush=True)
    K.check_status()
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", choices=("gemm", "elementwise", "muon", "attention"), default="gemm")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--out", default=None)
    ap.add_argument("--shape", type=int, nargs=3, default=None, metavar=("M", "N", "K"))
    args = ap.parse_args(argv)
    if args.what == "gemm":
        rows = bench_gemm(args.small, args.shape)
    else:
        rows = {"elementwise": bench_elementwise, "muon": bench_muon, "attention": bench_attention}[args.what](args.small)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
