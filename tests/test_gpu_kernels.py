"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from matrix_fsdp_b200.ops import kernels
    return kernels


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(dtype)


def _rel_err(got, ref):
    got, ref = got.float(), ref.float()
    return ((got - ref).norm() / ref.norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(256, 512, 128), (384, 640, 320), (4096, 2048, 2048), (200, 72, 136)])
def test_gemm_majors(K, a_mn, b_mn, shape):
    M, N, Kd = shape
    torch.manual_seed(0)
    a = _rand(M, Kd)
    b = _rand(N, Kd)
    ref = a.float() @ b.float().t()
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    out = K.gemm(a_in, b_in, a_mn_major=a_mn, b_mn_major=b_mn)
    K.check_status()
    assert _rel_err(out, ref) < 1e-2
    # forcing the narrow tile must agree too
    out2 = K.gemm(a_in, b_in, a_mn_major=a_mn, b_mn_major=b_mn, force_bn=128)
    K.check_status()
    assert _rel_err(out2, ref) < 1e-2


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("shape", [(512, 512, 256), (384, 320, 200), (1024, 2304, 512), (4096, 2048, 2048), (136, 72, 64)])
def test_gemm_cta_pair_kernel(K, a_mn, b_mn, shape):
    """The two-CTA (cta_group::2) kernel: 256 x 256 tiles over a cluster of two, every operand-major form, ragged
    edges (rows / columns / reduce length that do not fill a tile), and the scale / add epilogue."""
    M, N, Kd = shape
    torch.manual_seed(M + N)
    a, b, c = _rand(M, Kd), _rand(N, Kd), _rand(M, N)
    ref = a.float() @ b.float().t()
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    K.gemm(a_in, b_in, a_mn_major=a_mn, b_mn_major=b_mn, out=out, force_bn=2)
    K.check_status()
    assert torch.isfinite(out.float()).all()
    assert _rel_err(out, ref) < 1e-2
    out2 = K.gemm(a_in, b_in, a_mn_major=a_mn, b_mn_major=b_mn, cin=c, alpha=0.5, beta=2.0, force_bn=2)
    K.check_status()
    assert _rel_err(out2, 0.5 * ref + 2.0 * c.float()) < 1e-2
    # repeated launches (barrier phases, tensor-memory alloc / free across launches) stay correct
    for _ in range(3):
        out3 = K.gemm(a_in, b_in, a_mn_major=a_mn, b_mn_major=b_mn, force_bn=2)
    assert torch.equal(out3, out)


def test_gemm_alpha_beta_cin(K):
    torch.manual_seed(1)
    a, b, c = _rand(512, 256), _rand(384, 256), _rand(512, 384)
    ref = 0.5 * (a.float() @ b.float().t()) + 2.0 * c.float()
    out = K.gemm(a, b, cin=c, alpha=0.5, beta=2.0)
    K.check_status()
    assert _rel_err(out, ref) < 1e-2


def test_gemm_strided_views(K):
    torch.manual_seed(2)
    big = _rand(512, 1024)
    a = big[:, 256:512]            # row stride 1024, K = 256
    b = _rand(128, 256)
    out_big = torch.zeros(512, 512, device="cuda", dtype=torch.bfloat16)
    out = out_big[:, 128:256]
    K.gemm(a, b, out=out)
    K.check_status()
    assert _rel_err(out, a.float() @ b.float().t()) < 1e-2
    assert out_big[:, :128].abs().sum() == 0 and out_big[:, 256:].abs().sum() == 0


def test_grouped_gemm_m_and_k(K):
    torch.manual_seed(3)
    G, N, Kd = 4, 256, 192
    rows = [128, 0, 256, 128]
    tile_group = []
    for g, r in enumerate(rows):
        tile_group += [g] * (r // 128)
    tile_group.append(-1)  # a padding tile that is skipped
    Mtot = 128 * len(tile_group)
    a = _rand(Mtot, Kd)
    w = _rand(G, N, Kd)
    tg = torch.tensor(tile_group, dtype=torch.int32, device="cuda")
    out = torch.zeros(Mtot, N, device="cuda", dtype=torch.bfloat16)
    K.grouped_gemm_m(a, w, tg, out=out)
    K.check_status()
    for t, g in enumerate(tile_group):
        sl = slice(t * 128, (t + 1) * 128)
        if g < 0:
            assert out[sl].abs().sum() == 0
        else:
            assert _rel_err(out[sl], a[sl].float() @ w[g].float().t()) < 1e-2
    # dgrad form: B stored [G, K(reduce), N]
    dy = _rand(Mtot, N)
    dx = torch.zeros(Mtot, Kd, device="cuda", dtype=torch.bfloat16)
    K.grouped_gemm_m(dy, w, tg, b_mn_major=True, out=dx)
    K.check_status()
    for t, g in enumerate(tile_group):
        if g >= 0:
            sl = slice(t * 128, (t + 1) * 128)
            assert _rel_err(dx[sl], dy[sl].float() @ w[g].float()) < 1e-2
    # wgrad form
    offs = [0]
    for r in rows:
        offs.append(offs[-1] + r)
    go = torch.tensor(offs, dtype=torch.int32, device="cuda")
    dw = K.grouped_gemm_k(dy[: offs[-1]], a[: offs[-1]], go, G)
    K.check_status()
    for g in range(G):
        ref = dy[offs[g]:offs[g + 1]].float().t() @ a[offs[g]:offs[g + 1]].float()
        if rows[g] == 0:
            assert dw[g].abs().sum() == 0
        else:
            assert _rel_err(dw[g], ref) < 1e-2


@pytest.mark.parametrize("H", [256, 2048, 4096, 5120])
def test_rmsnorm(K, H):
    torch.manual_seed(4)
    x, w = _rand(300, H), (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    y, rstd = K.rmsnorm_fwd(x, w, 1e-5)
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    assert _rel_err(y, ref) < 1e-2
    dy, dres = _rand(300, H), _rand(300, H)
    ref.backward(dy.float())
    dx, dw = K.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
    assert _rel_err(dx, xf.grad + dres.float()) < 1e-2
    assert _rel_err(dw, wf.grad) < 1e-2


def test_rope_roundtrip_and_reference(K):
    torch.manual_seed(5)
    B, S, nH, D = 2, 64, 4, 128
    ld = 3 * nH * D
    buf = _rand(B * S, ld)
    orig = buf.clone()
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(S, device="cuda").float()[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    K.rope_(buf, cos, sin, S, 0, 2 * nH, D)  # q and k heads
    q = orig[:, : 2 * nH * D].float().view(B, S, 2 * nH, D)
    x1, x2 = q[..., : D // 2], q[..., D // 2:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    ref = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).view(B * S, -1)
    assert _rel_err(buf[:, : 2 * nH * D], ref) < 1e-2
    assert torch.equal(buf[:, 2 * nH * D:], orig[:, 2 * nH * D:])
    K.rope_(buf, cos, sin, S, 0, 2 * nH, D, backward=True)
    assert _rel_err(buf, orig) < 2e-2


def test_swiglu(K):
    torch.manual_seed(6)
    T, F = 257, 688
    gu = _rand(T, 2 * F)
    guf = gu.float().requires_grad_(True)
    ref = torch.nn.functional.silu(guf[:, :F]) * guf[:, F:]
    h = K.swiglu_fwd(gu)
    assert _rel_err(h, ref) < 1e-2
    dh = _rand(T, F)
    ref.backward(dh.float())
    dgu = K.swiglu_bwd(dh, gu)
    assert _rel_err(dgu, guf.grad) < 1e-2


@pytest.mark.parametrize("V", [1024, 32000])
def test_cross_entropy(K, V):
    torch.manual_seed(7)
    rows = 130
    logits = _rand(rows, V, scale=2.0)
    tgt = torch.randint(0, V, (rows,), device="cuda")
    tgt[3] = -100
    lf = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, tgt, ignore_index=-100, reduction="none")
    n_valid = (tgt != -100).sum().item()
    (ref.sum() / n_valid).backward()
    work = logits.clone()
    loss = K.cross_entropy_(work, tgt, 1.0 / n_valid)
    assert torch.allclose(loss, ref, atol=2e-2, rtol=1e-2)
    assert _rel_err(work, lf.grad) < 2e-2
    # the same with the scale read from device memory, and through the masked-target functional path
    work2 = logits.clone()
    scale_dev = torch.full((1,), 1.0 / n_valid, device="cuda")
    loss2 = K.cross_entropy_(work2, tgt, scale_dev)
    assert torch.equal(loss2, loss) and torch.equal(work2, work)
    from matrix_fsdp_b200.ops import functional as OF

    lg = logits.clone().requires_grad_(True)
    out = OF.fused_cross_entropy(lg * 1.0, tgt, ignore_index=-100)
    assert abs(float(out) - float(ref.sum() / n_valid)) < 2e-2
    out.backward()
    assert _rel_err(lg.grad, lf.grad) < 2e-2


@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_adamw_flat_matches_torch(K, gdtype):
    torch.manual_seed(8)
    n = 100003
    p0 = torch.randn(n, device="cuda")
    p = p0.clone()
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ref_p = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([ref_p], lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda").to(gdtype)
        ref_p.grad = g.float() * 0.5
        opt.step()
        K.adamw_flat_(p, m, v, g, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                      step=step, grad_scale=0.5, p_lp=lp)
    assert torch.allclose(p, ref_p.detach(), atol=1e-6, rtol=1e-5)
    assert torch.equal(lp, p.bfloat16())


def test_sgd_and_muon_elementwise(K):
    torch.manual_seed(9)
    n = 5000
    p0, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    p, mom = p0.clone(), torch.zeros(n, device="cuda")
    ref = torch.nn.Parameter(p0.clone())
    opt = torch.optim.SGD([ref], lr=0.1, momentum=0.9, weight_decay=0.01)
    for i in range(2):
        ref.grad = g.clone()
        opt.step()
        K.sgd_flat_(p, mom, g, lr=0.1, momentum=0.9, weight_decay=0.01, first_step=(i == 0))
    assert torch.allclose(p, ref.detach(), atol=1e-6, rtol=1e-5)
    # Muon stage 1: lerp momentum + Nesterov + norm
    rows, cols = 96, 160
    buf = torch.randn(rows * cols, device="cuda")
    gm = torch.randn(rows * cols, device="cuda")
    ref_buf = buf.clone().lerp_(gm, 1 - 0.95)
    ref_u = gm.lerp(ref_buf, 0.95)
    u = torch.empty(rows * cols, device="cuda", dtype=torch.bfloat16)
    ss = torch.zeros(1, device="cuda")
    K.muon_momentum(buf, gm, u, ss, 0.95, 1.0, True)
    assert torch.allclose(buf, ref_buf, atol=1e-6)
    assert _rel_err(u, ref_u) < 1e-2
    assert abs(ss.item() - u.float().pow(2).sum().item()) / ss.item() < 1e-3
    K.muon_normalize_(u, ss)
    assert abs(u.float().norm().item() - 1.0) < 1e-2
    pm = torch.randn(rows, cols, device="cuda")
    pm0 = pm.clone()
    o_t = _rand(cols, rows)
    K.muon_apply_(pm, o_t, rows, cols, True, 0.02, 0.1, 0.03)
    assert torch.allclose(pm, pm0 * (1 - 0.02 * 0.1) - 0.03 * o_t.float().t(), atol=1e-5)


def test_copy_segments_and_cast(K):
    torch.manual_seed(10)
    src = torch.arange(10000, device="cuda", dtype=torch.float32).bfloat16()
    dst = torch.zeros(12000, device="cuda", dtype=torch.bfloat16)
    so = torch.tensor([0, 1001, 5000], device="cuda", dtype=torch.int64)
    do = torch.tensor([8, 3003, 9001], device="cuda", dtype=torch.int64)
    ln = torch.tensor([1000, 777, 2999], device="cuda", dtype=torch.int64)
    K.copy_segments(src, dst, so, do, ln, 2999)
    ref = torch.zeros_like(dst)
    for s, d, l in zip(so.tolist(), do.tolist(), ln.tolist()):
        ref[d:d + l] = src[s:s + l]
    assert torch.equal(dst, ref)
    f = torch.randn(4099, device="cuda")
    b = torch.empty(4099, device="cuda", dtype=torch.bfloat16)
    K.cast_f32_bf16(f, b)
    assert torch.equal(b, f.bfloat16())


def test_gemm_with_fused_gather_single_gpu():
    """The all-gather-fused GEMM with its copy jobs reading from a second local buffer: rows of B
    arrive through the kernel's gather warps while tiles are computed."""
    from types import SimpleNamespace

    from matrix_fsdp_b200.ops import kernels as K

    torch.manual_seed(0)
    M, N, Kd, bn = 1024, 1536, 512, 256
    a = (torch.randn(M, Kd, device="cuda") * 0.1).bfloat16()
    src = (torch.randn(N, Kd, device="cuda") * 0.1).bfloat16()       # stands in for the peers' shards
    b = torch.zeros(N, Kd, device="cuda", dtype=torch.bfloat16)
    b[:300] = src[:300]                                              # some rows are already local
    nblocks = (N + bn - 1) // bn
    jobs, need = [], [0] * nblocks
    row = 300
    while row < N:
        blk = row // bn
        end = min(N, (blk + 1) * bn, row + 100)
        jobs.append((src.data_ptr() + row * Kd * 2, b.data_ptr() + row * Kd * 2, (end - row) * Kd * 2, blk))
        need[blk] += 1
        row = end
    dev = "cuda"
    first = [sum(need[:i]) for i in range(nblocks)]                  # jobs above are generated in block order
    plan = SimpleNamespace(
        b_ptr=b.data_ptr(), bn=bn, njobs=len(jobs), budget_ns=int(2e9), rotate=2,
        first=torch.tensor(first, dtype=torch.int32, device=dev),
        src=torch.tensor([j[0] for j in jobs], dtype=torch.int64, device=dev),
        dst=torch.tensor([j[1] for j in jobs], dtype=torch.int64, device=dev),
        nbytes=torch.tensor([j[2] for j in jobs], dtype=torch.int32, device=dev),
        flag_idx=torch.tensor([j[3] for j in jobs], dtype=torch.int32, device=dev),
        need=torch.tensor(need, dtype=torch.int32, device=dev),
        flags=torch.zeros(2 * nblocks, dtype=torch.int32, device=dev))
    out = K.gemm_ag(a, b, plan)
    torch.cuda.synchronize()
    K.check_status()
    assert torch.equal(b, src)
    ref = a.float() @ src.float().t()
    assert (out.float() - ref).abs().max().item() < 2e-2
    # a second call with the rows in place and no jobs is a plain GEMM
    plan.njobs, plan.need = 0, torch.zeros(nblocks, dtype=torch.int32, device=dev)
    out2 = K.gemm_ag(a, b, plan)
    torch.cuda.synchronize()
    assert torch.equal(out2, out)


@pytest.mark.parametrize("T,V,H", [(1000, 517, 256), (8192, 32000, 2048), (300, 40, 1024)])
def test_embedding_backward_matches_fp32(K, T, V, H):
    """Sum of the output-gradient rows of equal ids: against an fp32 index_add, with heavy duplicates, ids outside
    the vocabulary, accumulation into an existing gradient, and run-to-run bitwise equality."""
    torch.manual_seed(T + V)
    dy = _rand(T, H)
    ids = torch.randint(0, V, (T,), device="cuda")
    ids[: T // 4] = ids[0]                      # one id that occurs T/4 times
    ids[-1] = -1                                # an id that is not in the vocabulary contributes nothing
    valid = ids >= 0
    ref = torch.zeros(V, H, device="cuda").index_add_(0, ids[valid], dy[valid].float())
    out = torch.full((V, H), float("nan"), device="cuda", dtype=torch.bfloat16)
    K.embedding_bwd(dy, ids, out)
    assert torch.isfinite(out.float()).all()
    assert _rel_err(out, ref) < 5e-3
    again = torch.empty_like(out)
    K.embedding_bwd(dy, ids, again)
    assert torch.equal(out, again)
    prev = _rand(V, H)
    acc = prev.clone()
    K.embedding_bwd(dy, ids, acc, accumulate=True)
    assert _rel_err(acc, ref + prev.float()) < 5e-3
    untouched = torch.ones(V, dtype=torch.bool, device="cuda")
    untouched[ids[valid]] = False
    assert torch.equal(acc[untouched], prev[untouched])


def test_embedding_function_gradient_matches_torch(K):
    from matrix_fsdp_b200.ops import functional as OF

    torch.manual_seed(3)
    w = torch.nn.Parameter(_rand(1024, 512))
    w_ref = torch.nn.Parameter(w.detach().clone())
    ids = torch.randint(0, 1024, (4, 96), device="cuda")
    up = _rand(4, 96, 512)
    OF.embedding(ids, w, w).backward(up)
    torch.nn.functional.embedding(ids, w_ref).backward(up)
    assert w.grad is not None and w.grad.shape == w_ref.grad.shape
    assert _rel_err(w.grad, w_ref.grad.float()) < 5e-3


def test_grouped_gemms_on_cta_pairs(K):
    """M-grouped GEMM with the caller's promise of 256-row groups, and K-grouped GEMM with 256-row outputs: both
    run the two-CTA kernel and must match fp32."""
    torch.manual_seed(11)
    G, N, Kd = 3, 384, 320
    rows = [256, 512, 256]
    tile_group = torch.tensor(sum(([g] * (r // 128) for g, r in enumerate(rows)), []), dtype=torch.int32, device="cuda")
    a, w, c = _rand(sum(rows), Kd), _rand(G, N, Kd), _rand(sum(rows), N)
    out = torch.full((sum(rows), N), float("nan"), device="cuda", dtype=torch.bfloat16)
    K.grouped_gemm_m(a, w, tile_group, out=out, cin=c, alpha=1.0, beta=0.5, groups_of_256_rows=True)
    K.check_status()
    r0 = 0
    for g, r in enumerate(rows):
        ref = a[r0:r0 + r].float() @ w[g].float().t() + 0.5 * c[r0:r0 + r].float()
        assert _rel_err(out[r0:r0 + r], ref) < 1e-2, g
        r0 += r
    # MN-major B (the aX + BX product of Newton-Schulz)
    wt = w.transpose(1, 2).contiguous()
    out2 = K.grouped_gemm_m(a, wt, tile_group, b_mn_major=True, groups_of_256_rows=True)
    K.check_status()
    r0 = 0
    for g, r in enumerate(rows):
        assert _rel_err(out2[r0:r0 + r], a[r0:r0 + r].float() @ w[g].float().t()) < 1e-2, g
        r0 += r
    # K-grouped, 512-row outputs
    kk, M2, N2 = 192, 512, 320
    a2, b2 = _rand(G * kk, M2), _rand(G * kk, N2)
    offsets = torch.arange(G + 1, dtype=torch.int32, device="cuda") * kk
    o3 = K.grouped_gemm_k(a2, b2, offsets, G)
    K.check_status()
    ref3 = torch.bmm(a2.view(G, kk, M2).float().transpose(1, 2), b2.view(G, kk, N2).float())
    assert _rel_err(o3, ref3) < 1e-2
