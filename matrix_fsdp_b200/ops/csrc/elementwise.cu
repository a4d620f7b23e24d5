// Bandwidth-bound kernels of the model and optimizer path: RMSNorm, RoPE, SwiGLU,
// fused softmax-cross-entropy, flat sharded AdamW/SGD, Muon element-wise stages and the
// segment copy kernels of the flat-buffer runtime.  All use 16-byte vector accesses
// and one pass over HBM per tensor; reductions stay in registers/shared memory.
//
// Counterparts in the reference: the segment copies replace
// matrix_fsdp/kernels/native/matrix_copy_cuda.cu:8-87 (one element per thread there);
// everything else runs as stock PyTorch ops in the reference (torch.optim.AdamW,
// F.layer_norm, ... see test/fsdp/bench_fsdp2_compare.py:305-514).
#include "common.cuh"

namespace mfsdp {

// ============================================================== RMSNorm
// One CTA per row; H <= 8 * 8 * blockDim (each thread keeps up to 8 vectors of 8 bf16).
template <int VPT>
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                                   int H, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * H);
  const int nvec = H >> 3;
  uint4 xv[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      xv[i] = xr[v];
      const uint32_t u[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(u[e]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      const uint4 wv = wr[v];
      const uint32_t u[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(u[e]);
        const float2 g = unpack_bf16x2(ww[e]);
        o[e] = pack_bf16x2(f.x * rstd * g.x, f.y * rstd * g.y);
      }
      yr[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// Sum R values over the block at once (one round of barriers for R rows); `red` holds R * 32 floats.
template <int R>
__device__ __forceinline__ void block_sum_rows(float (&v)[R], float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int r = 0; r < R; ++r) v[r] = warp_sum(v[r]);
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) red[r * 32 + warp] = v[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) v[r] = warp_sum(lane < nwarps ? red[r * 32 + lane] : 0.f);
  __syncthreads();
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres);  dw += sum_rows dy * xhat.
// Persistent over rows so each CTA folds its dw partial into the fp32 accumulator once.  A CTA works
// on ROWS rows per trip: all their loads are issued before the first use and one pair of barriers
// serves the ROWS row-dots, which is what the kernel's time goes to at hidden sizes of a few thousand.
template <int VPT, int ROWS>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_acc, long long rows, int H) {
  __shared__ float red[ROWS * 32];
  const int nvec = H >> 3;
  float dwp[VPT][8];
  float wf[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int e = 0; e < 8; ++e) { dwp[i][e] = 0.f; wf[i][e] = 0.f; }
    if (v < nvec) {
      const uint4 wv = reinterpret_cast<const uint4*>(w)[v];
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 g = unpack_bf16x2(ww[e]);
        wf[i][2 * e] = g.x; wf[i][2 * e + 1] = g.y;
      }
    }
  }
  for (long long row0 = (long long)blockIdx.x * ROWS; row0 < rows; row0 += (long long)gridDim.x * ROWS) {
    uint4 xv[ROWS][VPT], dv[ROWS][VPT];
    float rstd[ROWS], dot[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const long long row = row0 + r;
      const bool live = row < rows;
      rstd[r] = live ? rstd_in[row] : 0.f;
      dot[r] = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (live && v < nvec) {
          xv[r][i] = reinterpret_cast<const uint4*>(x + row * H)[v];
          dv[r][i] = reinterpret_cast<const uint4*>(dy + row * H)[v];
        } else {
          xv[r][i] = make_uint4(0, 0, 0, 0);
          dv[r][i] = make_uint4(0, 0, 0, 0);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const uint32_t xu[4] = {xv[r][i].x, xv[r][i].y, xv[r][i].z, xv[r][i].w};
        const uint32_t du[4] = {dv[r][i].x, dv[r][i].y, dv[r][i].z, dv[r][i].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 xf = unpack_bf16x2(xu[e]);
          const float2 df = unpack_bf16x2(du[e]);
          const float xh0 = xf.x * rstd[r], xh1 = xf.y * rstd[r];
          dwp[i][2 * e] += df.x * xh0;
          dwp[i][2 * e + 1] += df.y * xh1;
          dot[r] += df.x * wf[i][2 * e] * xh0 + df.y * wf[i][2 * e + 1] * xh1;
        }
      }
    }
    block_sum_rows<ROWS>(dot, red);
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const long long row = row0 + r;
      if (row >= rows) break;
      const float mean_dot = dot[r] / (float)H;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
          const uint32_t xu[4] = {xv[r][i].x, xv[r][i].y, xv[r][i].z, xv[r][i].w};
          const uint32_t du[4] = {dv[r][i].x, dv[r][i].y, dv[r][i].z, dv[r][i].w};
          float o[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 xf = unpack_bf16x2(xu[e]);
            const float2 df = unpack_bf16x2(du[e]);
            o[2 * e] = rstd[r] * (df.x * wf[i][2 * e] - xf.x * rstd[r] * mean_dot);
            o[2 * e + 1] = rstd[r] * (df.y * wf[i][2 * e + 1] - xf.y * rstd[r] * mean_dot);
          }
          if (dres) {
            const uint4 rv = reinterpret_cast<const uint4*>(dres + row * H)[v];
            const uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 rf = unpack_bf16x2(ru[e]);
              o[2 * e] += rf.x; o[2 * e + 1] += rf.y;
            }
          }
          reinterpret_cast<uint4*>(dx + row * H)[v] =
              make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]),
                         pack_bf16x2(o[6], o[7]));
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      // one partial row per CTA in the scratch matrix [gridDim.x, H]; no atomics
      float* dst = dw_acc + (long long)blockIdx.x * H + v * 8;
      reinterpret_cast<float4*>(dst)[0] = make_float4(dwp[i][0], dwp[i][1], dwp[i][2], dwp[i][3]);
      reinterpret_cast<float4*>(dst)[1] = make_float4(dwp[i][4], dwp[i][5], dwp[i][6], dwp[i][7]);
    }
  }
}

// out[c] (bf16) = (accumulate ? out[c] : 0) + sum_r partial[r, c]; one thread per column, rows
// strided over blockIdx.y-less 2-D thread blocks (32 columns x 8 row lanes).
__global__ void colsum_f32_to_bf16_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                          int rows, int H, int accumulate) {
  __shared__ float tile[8][33];
  const int col = blockIdx.x * 32 + threadIdx.x;
  float acc = 0.f;
  if (col < H)
    for (int r = threadIdx.y; r < rows; r += 8) acc += partial[(long long)r * H + col];
  tile[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && col < H) {
    float v = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) v += tile[j][threadIdx.x];
    if (accumulate) v += __bfloat162float(out[col]);
    out[col] = __float2bfloat16_rn(v);
  }
}

// ============================================================== RoPE
// In-place rotary embedding ("rotate-half" pairing i <-> i + D/2) on `n_heads` heads that
// start at column `col0` of a [T, ld] matrix; cos/sin tables are [S, D/2] fp32, position of
// row t is t % S.  sign = +1 forward, -1 backward (the transpose of a rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, long long T, int S, int ld, int col0,
                            int n_heads, int D, float sign) {
  const int half = D >> 1;
  const int vec_per_head = half >> 3;  // 8 bf16 per vector
  const long long total = T * (long long)n_heads * vec_per_head;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vec_per_head);
    const int h = (int)((idx / vec_per_head) % n_heads);
    const long long t = idx / ((long long)vec_per_head * n_heads);
    const int pos = (int)(t % S);
    __nv_bfloat16* base = qkv + t * ld + col0 + h * D + v * 8;
    uint4 a = *reinterpret_cast<uint4*>(base);
    uint4 b = *reinterpret_cast<uint4*>(base + half);
    const float4 c0 = *reinterpret_cast<const float4*>(cos_t + (long long)pos * half + v * 8);
    const float4 c1 = *reinterpret_cast<const float4*>(cos_t + (long long)pos * half + v * 8 + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sin_t + (long long)pos * half + v * 8);
    const float4 s1 = *reinterpret_cast<const float4*>(sin_t + (long long)pos * half + v * 8 + 4);
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint32_t au[4] = {a.x, a.y, a.z, a.w}, bu[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x1 = unpack_bf16x2(au[e]);
      const float2 x2 = unpack_bf16x2(bu[e]);
      const float s_lo = sign * sn[2 * e], s_hi = sign * sn[2 * e + 1];
      const float o1x = x1.x * cs[2 * e] - x2.x * s_lo;
      const float o1y = x1.y * cs[2 * e + 1] - x2.y * s_hi;
      const float o2x = x2.x * cs[2 * e] + x1.x * s_lo;
      const float o2y = x2.y * cs[2 * e + 1] + x1.y * s_hi;
      au[e] = pack_bf16x2(o1x, o1y);
      bu[e] = pack_bf16x2(o2x, o2y);
    }
    *reinterpret_cast<uint4*>(base) = make_uint4(au[0], au[1], au[2], au[3]);
    *reinterpret_cast<uint4*>(base + half) = make_uint4(bu[0], bu[1], bu[2], bu[3]);
  }
}

// ============================================================== SwiGLU
// gu is [T, 2F]: gate in columns [0,F), up in [F,2F).  h = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h,
                                  long long T, int F) {
  const int vpr = F >> 3;
  const long long total = T * vpr;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / vpr;
    const int v = (int)(idx % vpr);
    const uint4 g = *reinterpret_cast<const uint4*>(gu + t * 2 * F + v * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + t * 2 * F + F + v * 8);
    const uint32_t gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = unpack_bf16x2(gg[e]);
      const float2 b = unpack_bf16x2(uu[e]);
      const float sx = a.x / (1.f + __expf(-a.x)), sy = a.y / (1.f + __expf(-a.y));
      o[e] = pack_bf16x2(sx * b.x, sy * b.y);
    }
    *reinterpret_cast<uint4*>(h + t * F + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// dgu[:, :F] = dh * up * dsilu(gate);  dgu[:, F:] = dh * silu(gate).
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dh,
                                  const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  const int vpr = F >> 3;
  const long long total = T * vpr;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / vpr;
    const int v = (int)(idx % vpr);
    const uint4 g = *reinterpret_cast<const uint4*>(gu + t * 2 * F + v * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + t * 2 * F + F + v * 8);
    const uint4 d = *reinterpret_cast<const uint4*>(dh + t * F + v * 8);
    const uint32_t gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w},
                   dd[4] = {d.x, d.y, d.z, d.w};
    uint32_t og[4], ou[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = unpack_bf16x2(gg[e]);
      const float2 b = unpack_bf16x2(uu[e]);
      const float2 c = unpack_bf16x2(dd[e]);
      const float sgx = 1.f / (1.f + __expf(-a.x)), sgy = 1.f / (1.f + __expf(-a.y));
      const float silx = a.x * sgx, sily = a.y * sgy;
      const float dsx = sgx * (1.f + a.x * (1.f - sgx)), dsy = sgy * (1.f + a.y * (1.f - sgy));
      og[e] = pack_bf16x2(c.x * b.x * dsx, c.y * b.y * dsy);
      ou[e] = pack_bf16x2(c.x * silx, c.y * sily);
    }
    *reinterpret_cast<uint4*>(dgu + t * 2 * F + v * 8) = make_uint4(og[0], og[1], og[2], og[3]);
    *reinterpret_cast<uint4*>(dgu + t * 2 * F + F + v * 8) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}

// ============================================================== cross-entropy
// One CTA (1024 threads) per row keeps the whole row in registers (V <= 1024*8*VPT):
// loss[row] = logsumexp - logit[target]; logits are overwritten with
// (softmax - onehot) * grad_scale, i.e. the gradient of the mean loss.  When `grad_scale_dev` is
// given the scale is read from device memory (1 / number of counted targets, computed on the device),
// so a caller that masks targets needs no device-to-host read to launch this.
template <int VPT>
__global__ void __launch_bounds__(1024)
cross_entropy_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
                             float* __restrict__ loss, int V, long long ld, float grad_scale,
                             const float* __restrict__ grad_scale_dev, long long ignore_index) {
  __shared__ float red[32];
  if (grad_scale_dev != nullptr) grad_scale = *grad_scale_dev;
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int nvec = V >> 3;
  float f[VPT][8];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      const uint4 u = reinterpret_cast<const uint4*>(lr)[v];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = unpack_bf16x2(w[e]);
        f[i][2 * e] = a.x; f[i][2 * e + 1] = a.y;
        mx = fmaxf(mx, fmaxf(a.x, a.y));
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[i][e] = -INFINITY;
    }
  }
  mx = block_max(mx, red);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      f[i][e] = __expf(f[i][e] - mx);
      sum += f[i][e];
    }
  sum = block_sum(sum, red);
  const long long tgt = target[row];
  const bool valid = (tgt != ignore_index) && tgt >= 0 && tgt < V;
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (valid) l = logf(sum) + mx - __bfloat162float(lr[tgt]);
    loss[row] = l;
  }
  __syncthreads();  // the target logit is read above before any thread overwrites the row
  const float inv = valid ? grad_scale / sum : 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        o[e] = f[i][e] * inv;
        if (valid && (long long)(v * 8 + e) == tgt) o[e] -= grad_scale;
      }
      reinterpret_cast<uint4*>(lr)[v] = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]),
                                                   pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
    }
  }
}

// ============================================================== flat optimizers
// Sharded AdamW over one contiguous flat range.  Master weights and both moments are fp32;
// the gradient arrives as bf16 or fp32 and is scaled by `grad_scale` (1/world, clipping)
// on the fly; the kernel also emits the low-precision copy that the next all-gather
// ships, so no separate cast kernel runs.  Matches torch.optim.AdamW (decoupled decay,
// bias correction, eps outside the sqrt of the corrected second moment).
template <typename GradT>
__global__ void adamw_flat_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                  const GradT* __restrict__ g, __nv_bfloat16* __restrict__ p_lp,
                                  long long n, float lr, float beta1, float beta2, float eps,
                                  float weight_decay, float bias1, float bias2_sqrt, float grad_scale) {
  const long long nv = n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += stride) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float gg[4];
    if constexpr (sizeof(GradT) == 2) {
      const uint2 u = reinterpret_cast<const uint2*>(g)[i];
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
      gg[0] = a.x; gg[1] = a.y; gg[2] = b.x; gg[3] = b.y;
    } else {
      const float4 a = reinterpret_cast<const float4*>(g)[i];
      gg[0] = a.x; gg[1] = a.y; gg[2] = a.z; gg[3] = a.w;
    }
    float* pa = reinterpret_cast<float*>(&pp);
    float* ma = reinterpret_cast<float*>(&mm);
    float* va = reinterpret_cast<float*>(&vv);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float gr = gg[e] * grad_scale;
      pa[e] *= (1.f - lr * weight_decay);
      ma[e] = beta1 * ma[e] + (1.f - beta1) * gr;
      va[e] = beta2 * va[e] + (1.f - beta2) * gr * gr;
      const float denom = sqrtf(va[e]) / bias2_sqrt + eps;
      pa[e] -= (lr / bias1) * (ma[e] / denom);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (p_lp)
      reinterpret_cast<uint2*>(p_lp)[i] = make_uint2(pack_bf16x2(pa[0], pa[1]), pack_bf16x2(pa[2], pa[3]));
  }
  // scalar tail
  for (long long i = (nv << 2) + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    float gr;
    if constexpr (sizeof(GradT) == 2) gr = __bfloat162float(g[i]) * grad_scale;
    else gr = (float)g[i] * grad_scale;
    float pv = p[i] * (1.f - lr * weight_decay);
    const float mv = beta1 * m[i] + (1.f - beta1) * gr;
    const float vv2 = beta2 * v[i] + (1.f - beta2) * gr * gr;
    pv -= (lr / bias1) * (mv / (sqrtf(vv2) / bias2_sqrt + eps));
    p[i] = pv; m[i] = mv; v[i] = vv2;
    if (p_lp) p_lp[i] = __float2bfloat16_rn(pv);
  }
}

// SGD with optional momentum over a flat fp32 range (same fused low-precision emit).
template <typename GradT>
__global__ void sgd_flat_kernel(float* __restrict__ p, float* __restrict__ mom,
                                const GradT* __restrict__ g, __nv_bfloat16* __restrict__ p_lp,
                                long long n, float lr, float momentum, float weight_decay,
                                float grad_scale, int first_step) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    float gr;
    if constexpr (sizeof(GradT) == 2) gr = __bfloat162float(g[i]) * grad_scale;
    else gr = (float)g[i] * grad_scale;
    float pv = p[i];
    gr += weight_decay * pv;
    if (mom) {
      const float b = first_step ? gr : momentum * mom[i] + gr;
      mom[i] = b;
      gr = b;
    }
    pv -= lr * gr;
    p[i] = pv;
    if (p_lp) p_lp[i] = __float2bfloat16_rn(pv);
  }
}

// ============================================================== Muon element-wise stages
// Stage 1 (per matrix): buf = mu*buf + (1-mu)*g*scale  (torch's lerp form),
// u = nesterov ? lerp(g*scale, buf, mu) : buf; emits u as bf16 and accumulates sum(u^2).
template <typename GradT>
__global__ void muon_momentum_kernel(float* __restrict__ buf, const GradT* __restrict__ g,
                                     __nv_bfloat16* __restrict__ u_out, float* __restrict__ sumsq,
                                     long long n, float mu, float grad_scale, int nesterov) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    float gr;
    if constexpr (sizeof(GradT) == 2) gr = __bfloat162float(g[i]) * grad_scale;
    else gr = (float)g[i] * grad_scale;
    const float b = buf[i] + (1.f - mu) * (gr - buf[i]);
    buf[i] = b;
    const float u = nesterov ? gr + mu * (b - gr) : b;
    const __nv_bfloat16 ub = __float2bfloat16_rn(u);
    u_out[i] = ub;
    const float uf = __bfloat162float(ub);
    acc += uf * uf;
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(sumsq, acc);
}

// x *= 1 / max(sqrt(sumsq), eps)   (bf16 in place)
__global__ void muon_normalize_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ sumsq,
                                      long long n, float eps) {
  const float inv = 1.f / fmaxf(sqrtf(*sumsq), eps);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride)
    x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) * inv);
}

// p = p*(1 - lr*wd) - adjusted_lr * o ; o is the orthogonalised update, stored either as
// [rows, cols] (transposed = 0) or as [cols, rows] (transposed = 1).
__global__ void muon_apply_kernel(float* __restrict__ p, const __nv_bfloat16* __restrict__ o,
                                  __nv_bfloat16* __restrict__ p_lp, int rows, int cols,
                                  int transposed, float lr, float weight_decay, float adjusted_lr) {
  const long long n = (long long)rows * cols;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    long long j = i;
    if (transposed) {
      const long long r = i / cols, c = i % cols;
      j = c * rows + r;
    }
    float pv = p[i] * (1.f - lr * weight_decay);
    pv -= adjusted_lr * __bfloat162float(o[j]);
    p[i] = pv;
    if (p_lp) p_lp[i] = __float2bfloat16_rn(pv);
  }
}

// ============================================================== segment copies
struct SegTable {  // device arrays of length nseg
  const long long* src_off;
  const long long* dst_off;
  const long long* len;
};

// Copies nseg (src_off, dst_off, len) element ranges; blockIdx.y walks segments.
// 16-byte vectors when both sides are 16-byte aligned, scalar head/tail otherwise.
template <typename T>
__global__ void copy_segments_kernel(const T* __restrict__ src, T* __restrict__ dst, SegTable tab,
                                     int nseg) {
  for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
    const T* sp = src + tab.src_off[s];
    T* dp = dst + tab.dst_off[s];
    const long long n = tab.len[s];
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    constexpr int kPer = 16 / sizeof(T);
    const uintptr_t sa = reinterpret_cast<uintptr_t>(sp), da = reinterpret_cast<uintptr_t>(dp);
    if ((sa & 15) == (da & 15)) {
      long long head = ((16 - (sa & 15)) & 15) / sizeof(T);
      if (head > n) head = n;
      const long long nvec = (n - head) / kPer;
      for (long long i = tid; i < head; i += stride) dp[i] = sp[i];
      const uint4* sv = reinterpret_cast<const uint4*>(sp + head);
      uint4* dv = reinterpret_cast<uint4*>(dp + head);
      for (long long i = tid; i < nvec; i += stride) dv[i] = sv[i];
      for (long long i = head + nvec * kPer + tid; i < n; i += stride) dp[i] = sp[i];
    } else {
      for (long long i = tid; i < n; i += stride) dp[i] = sp[i];
    }
  }
}

// fp32 -> bf16 cast over segments (mixed-precision shard -> gather staging).
__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                     long long n) {
  const long long nv = n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
                       ((reinterpret_cast<uintptr_t>(dst) & 7) == 0);
  if (aligned) {
    for (long long i = tid; i < nv; i += stride) {
      const float4 a = reinterpret_cast<const float4*>(src)[i];
      reinterpret_cast<uint2*>(dst)[i] = make_uint2(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w));
    }
    for (long long i = (nv << 2) + tid; i < n; i += stride) dst[i] = __float2bfloat16_rn(src[i]);
  } else {
    for (long long i = tid; i < n; i += stride) dst[i] = __float2bfloat16_rn(src[i]);
  }
}

static inline int grid_for(long long work, int threads, int max_blocks = 148 * 8) {
  long long b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return (int)b;
}

// ============================================================== embedding backward
// dW[v, :] = sum over the positions t with ids[t] == v of dy[t, :], written (or accumulated) straight into
// the gradient bucket.  A stable counting sort of the T token ids (count per id, exclusive scan over the
// vocabulary, rank of each position among the earlier equal ids) gives every vocabulary row the list of its
// positions in their original order, so the fp32 sum of a row is the same in every run; one CTA per
// vocabulary row then sums its list and writes the row once, zeros where an id does not occur -- no separate
// fill of the V x H gradient, no atomics on values, and five short launches instead of a 64-bit radix sort.
__global__ void embed_count_kernel(const long long* __restrict__ ids, int T, int V, int* __restrict__ count) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const long long v = ids[t];
  if (v >= 0 && v < V) atomicAdd(&count[v], 1);
}

__global__ void __launch_bounds__(1024) embed_scan_kernel(const int* __restrict__ count, int* __restrict__ start, int V) {
  __shared__ int part[1024];
  const int per = (V + 1023) / 1024;
  const int lo = min(threadIdx.x * per, V), hi = min(lo + per, V);
  int s = 0;
  for (int i = lo; i < hi; ++i) s += count[i];
  part[threadIdx.x] = s;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {      // inclusive scan of the 1024 partial sums
    const int add = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
    __syncthreads();
    part[threadIdx.x] += add;
    __syncthreads();
  }
  int run = part[threadIdx.x] - s;
  for (int i = lo; i < hi; ++i) {
    start[i] = run;
    run += count[i];
  }
}

__global__ void __launch_bounds__(256) embed_place_kernel(const long long* __restrict__ ids, int T, int V,
                                                          const int* __restrict__ start, int* __restrict__ order) {
  __shared__ int tile[2048];
  const int t = blockIdx.x * 256 + threadIdx.x;
  const long long mine64 = t < T ? ids[t] : -1;
  const bool valid = mine64 >= 0 && mine64 < V;
  const int mine = valid ? (int)mine64 : -1;
  const int limit = min((blockIdx.x + 1) * 256, T);   // positions before the end of this block
  int rank = 0;
  for (int base = 0; base < limit; base += 2048) {
    const int n = min(2048, limit - base);
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += 256) {
      const long long v = ids[base + i];
      tile[i] = (v >= 0 && v < V) ? (int)v : -2;
    }
    __syncthreads();
    if (valid) {
      const int upto = min(n, t - base);             // only earlier positions count
      for (int i = 0; i < upto; ++i) rank += (tile[i] == mine);
    }
  }
  if (valid) order[start[mine] + rank] = t;
}

__global__ void __launch_bounds__(256) embed_sum_kernel(const __nv_bfloat16* __restrict__ dy, long long lddy,
                                                        __nv_bfloat16* __restrict__ dw, long long lddw, int H,
                                                        const int* __restrict__ count, const int* __restrict__ start,
                                                        const int* __restrict__ order, int accumulate) {
  const int v = blockIdx.x;
  const int n = count[v];
  if (n == 0 && accumulate) return;
  const int first = start[v];
  __nv_bfloat16* out = dw + (long long)v * lddw;
  for (int c = threadIdx.x * 8; c < H; c += 256 * 8) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (accumulate) {
      const uint4 u = *reinterpret_cast<const uint4*>(out + c);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 a = unpack_bf16x2(w[e]); acc[2 * e] = a.x; acc[2 * e + 1] = a.y; }
    }
    for (int j = 0; j < n; ++j) {
      const int t = order[first + j];
      const uint4 u = *reinterpret_cast<const uint4*>(dy + (long long)t * lddy + c);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 a = unpack_bf16x2(w[e]); acc[2 * e] += a.x; acc[2 * e + 1] += a.y; }
    }
    *reinterpret_cast<uint4*>(out + c) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                    pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

}  // namespace mfsdp

using namespace mfsdp;

MFSDP_API int mfsdp_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows,
                                int H, float eps, cudaStream_t st) {
  if (H % 8 || H > 8 * 8 * 1024) return -2;
  const int nvec = H / 8;
  int threads = 256;
  if (nvec <= 128) threads = 128;
  const int vpt = (nvec + threads - 1) / threads;
  auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w; auto Y = (__nv_bfloat16*)y;
  if (vpt <= 1) rmsnorm_fwd_kernel<1><<<(unsigned)rows, threads, 0, st>>>(X, W, Y, rstd, H, eps);
  else if (vpt <= 2) rmsnorm_fwd_kernel<2><<<(unsigned)rows, threads, 0, st>>>(X, W, Y, rstd, H, eps);
  else if (vpt <= 4) rmsnorm_fwd_kernel<4><<<(unsigned)rows, threads, 0, st>>>(X, W, Y, rstd, H, eps);
  else if (vpt <= 8) rmsnorm_fwd_kernel<8><<<(unsigned)rows, threads, 0, st>>>(X, W, Y, rstd, H, eps);
  else return -2;
  return (int)cudaGetLastError();
}

// Rows of CTAs used by the backward kernel (= rows of the dw scratch matrix).
MFSDP_API int mfsdp_rmsnorm_bwd_scratch_rows(long long rows) { return (int)(rows < 148 * 4 ? rows : 148 * 4); }

// CTAs for `rows` rows taken `rows_per_trip` at a time with at most `cap` CTAs: every CTA makes the same
// number of trips (up to rounding), so none idles while the others finish.
static int rmsnorm_bwd_grid(long long rows, int rows_per_trip, int cap) {
  const long long groups = (rows + rows_per_trip - 1) / rows_per_trip;
  if (groups <= cap) return (int)(groups < 1 ? 1 : groups);
  const long long trips = (groups + cap - 1) / cap;
  return (int)((groups + trips - 1) / trips);
}

// dw_acc: fp32 scratch of mfsdp_rmsnorm_bwd_scratch_rows(rows) x H floats (fully overwritten, needs no
// initialisation); dw (bf16) = (accumulate ? dw : 0) + column sums of the scratch.
MFSDP_API int mfsdp_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                                const void* dres, void* dx, float* dw_acc, void* dw,
                                int accumulate_dw, long long rows, int H, cudaStream_t st) {
  if (H % 8 || H > 8 * 4 * 256) return -2;
  const int nvec = H / 8;
  const int threads = 256;
  const int vpt = (nvec + threads - 1) / threads;
  const int grid = rmsnorm_bwd_grid(rows, vpt <= 1 ? 4 : (vpt <= 2 ? 2 : 1), mfsdp_rmsnorm_bwd_scratch_rows(rows));
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  auto DR = (const __nv_bfloat16*)dres; auto DX = (__nv_bfloat16*)dx;
  if (vpt <= 1) rmsnorm_bwd_kernel<1, 4><<<grid, threads, 0, st>>>(DY, X, W, rstd, DR, DX, dw_acc, rows, H);
  else if (vpt <= 2) rmsnorm_bwd_kernel<2, 2><<<grid, threads, 0, st>>>(DY, X, W, rstd, DR, DX, dw_acc, rows, H);
  else if (vpt <= 4) rmsnorm_bwd_kernel<4, 1><<<grid, threads, 0, st>>>(DY, X, W, rstd, DR, DX, dw_acc, rows, H);
  else return -2;
  if (dw) colsum_f32_to_bf16_kernel<<<(H + 31) / 32, dim3(32, 8), 0, st>>>(dw_acc, (__nv_bfloat16*)dw, grid, H, accumulate_dw);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_rope(void* qkv, const float* cos_t, const float* sin_t, long long T, int S, int ld,
                         int col0, int n_heads, int D, float sign, cudaStream_t st) {
  if (D % 16 || ld % 8 || col0 % 8) return -2;
  const long long work = T * (long long)n_heads * (D / 16);
  rope_kernel<<<grid_for(work, 256, 148 * 16), 256, 0, st>>>((__nv_bfloat16*)qkv, cos_t, sin_t, T, S, ld, col0,
                                                   n_heads, D, sign);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_swiglu_fwd(const void* gu, void* h, long long T, int F, cudaStream_t st) {
  if (F % 8) return -2;
  swiglu_fwd_kernel<<<grid_for(T * (F / 8), 256, 148 * 16), 256, 0, st>>>((const __nv_bfloat16*)gu,
                                                                 (__nv_bfloat16*)h, T, F);
  return (int)cudaGetLastError();
}

// dW[V, H] (row pitch lddw) from dy[T, H] (row pitch lddy) and ids[T]; `work` holds 2 * V + T ints.  Ids outside
// [0, V) contribute nothing.  accumulate != 0 adds to what dW holds (rows whose id does not occur stay as they are).
MFSDP_API int mfsdp_embedding_bwd(const void* dy, long long lddy, const long long* ids, void* dw, long long lddw,
                                  int T, int V, int H, int accumulate, int* work, cudaStream_t st) {
  if (T <= 0 || V <= 0 || H <= 0 || (H % 8) || (lddy % 8) || (lddw % 8)) return -2;
  if (((uintptr_t)dy & 15) || ((uintptr_t)dw & 15)) return -2;
  int* count = work;
  int* start = work + V;
  int* order = work + 2 * (long long)V;
  cudaError_t e = cudaMemsetAsync(count, 0, sizeof(int) * (size_t)V, st);
  if (e != cudaSuccess) return (int)e;
  embed_count_kernel<<<(T + 255) / 256, 256, 0, st>>>(ids, T, V, count);
  embed_scan_kernel<<<1, 1024, 0, st>>>(count, start, V);
  embed_place_kernel<<<(T + 255) / 256, 256, 0, st>>>(ids, T, V, start, order);
  embed_sum_kernel<<<V, 256, 0, st>>>((const __nv_bfloat16*)dy, lddy, (__nv_bfloat16*)dw, lddw, H, count, start, order,
                                       accumulate);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_swiglu_bwd(const void* dh, const void* gu, void* dgu, long long T, int F,
                               cudaStream_t st) {
  if (F % 8) return -2;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256, 148 * 16), 256, 0, st>>>(
      (const __nv_bfloat16*)dh, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, T, F);
  return (int)cudaGetLastError();
}

static int launch_cross_entropy(void* logits, const long long* target, float* loss, long long rows, int V,
                                long long ld, float grad_scale, const float* grad_scale_dev,
                                long long ignore_index, cudaStream_t st) {
  if (V % 8 || ld % 8) return -2;
  const int nvec = V / 8;
  const int vpt = (nvec + 1023) / 1024;
  auto L = (__nv_bfloat16*)logits;
  const unsigned g = (unsigned)rows;
  if (vpt <= 1) cross_entropy_fwd_bwd_kernel<1><<<g, 1024, 0, st>>>(L, target, loss, V, ld, grad_scale, grad_scale_dev, ignore_index);
  else if (vpt <= 2) cross_entropy_fwd_bwd_kernel<2><<<g, 1024, 0, st>>>(L, target, loss, V, ld, grad_scale, grad_scale_dev, ignore_index);
  else if (vpt <= 4) cross_entropy_fwd_bwd_kernel<4><<<g, 1024, 0, st>>>(L, target, loss, V, ld, grad_scale, grad_scale_dev, ignore_index);
  else if (vpt <= 6) cross_entropy_fwd_bwd_kernel<6><<<g, 1024, 0, st>>>(L, target, loss, V, ld, grad_scale, grad_scale_dev, ignore_index);
  else return -2;
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_cross_entropy(void* logits, const long long* target, float* loss, long long rows,
                                  int V, long long ld, float grad_scale, long long ignore_index,
                                  cudaStream_t st) {
  return launch_cross_entropy(logits, target, loss, rows, V, ld, grad_scale, nullptr, ignore_index, st);
}

// Same, with the gradient scale read from device memory at `grad_scale_dev` (one float).
MFSDP_API int mfsdp_cross_entropy_dev_scale(void* logits, const long long* target, float* loss, long long rows,
                                            int V, long long ld, const float* grad_scale_dev,
                                            long long ignore_index, cudaStream_t st) {
  if (grad_scale_dev == nullptr) return -2;
  return launch_cross_entropy(logits, target, loss, rows, V, ld, 0.f, grad_scale_dev, ignore_index, st);
}

MFSDP_API int mfsdp_adamw_flat(float* p, float* m, float* v, const void* g, int grad_is_bf16, void* p_lp,
                               long long n, float lr, float beta1, float beta2, float eps,
                               float weight_decay, long long step, float grad_scale, cudaStream_t st) {
  if (n <= 0) return 0;
  if (((uintptr_t)p & 15) || ((uintptr_t)m & 15) || ((uintptr_t)v & 15) ||
      ((uintptr_t)g & (grad_is_bf16 ? 7 : 15)) || ((uintptr_t)p_lp & 7))
    return -2;
  const float bias1 = 1.f - powf(beta1, (float)step);
  const float bias2_sqrt = sqrtf(1.f - powf(beta2, (float)step));
  const int grid = grid_for(n / 4 + 1, 256, 148 * 8);
  if (grad_is_bf16)
    adamw_flat_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, m, v, (const __nv_bfloat16*)g, (__nv_bfloat16*)p_lp, n, lr,
                                                           beta1, beta2, eps, weight_decay, bias1, bias2_sqrt, grad_scale);
  else
    adamw_flat_kernel<float><<<grid, 256, 0, st>>>(p, m, v, (const float*)g, (__nv_bfloat16*)p_lp, n, lr, beta1, beta2,
                                                   eps, weight_decay, bias1, bias2_sqrt, grad_scale);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_sgd_flat(float* p, float* mom, const void* g, int grad_is_bf16, void* p_lp, long long n,
                             float lr, float momentum, float weight_decay, float grad_scale,
                             int first_step, cudaStream_t st) {
  if (n <= 0) return 0;
  const int grid = grid_for(n, 256, 148 * 8);
  if (grad_is_bf16)
    sgd_flat_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, mom, (const __nv_bfloat16*)g, (__nv_bfloat16*)p_lp, n, lr,
                                                         momentum, weight_decay, grad_scale, first_step);
  else
    sgd_flat_kernel<float><<<grid, 256, 0, st>>>(p, mom, (const float*)g, (__nv_bfloat16*)p_lp, n, lr, momentum,
                                                 weight_decay, grad_scale, first_step);
  return (int)cudaGetLastError();
}

// sumsq must be zero on entry.
MFSDP_API int mfsdp_muon_momentum(float* buf, const void* g, int grad_is_bf16, void* u_out, float* sumsq,
                                  long long n, float mu, float grad_scale, int nesterov, cudaStream_t st) {
  if (n <= 0) return 0;
  const int grid = grid_for(n, 256, 148 * 4);
  if (grad_is_bf16)
    muon_momentum_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(buf, (const __nv_bfloat16*)g, (__nv_bfloat16*)u_out,
                                                              sumsq, n, mu, grad_scale, nesterov);
  else
    muon_momentum_kernel<float><<<grid, 256, 0, st>>>(buf, (const float*)g, (__nv_bfloat16*)u_out, sumsq, n, mu,
                                                      grad_scale, nesterov);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_muon_normalize(void* x, const float* sumsq, long long n, float eps, cudaStream_t st) {
  if (n <= 0) return 0;
  muon_normalize_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, st>>>((__nv_bfloat16*)x, sumsq, n, eps);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_muon_apply(float* p, const void* o, void* p_lp, int rows, int cols, int transposed,
                               float lr, float weight_decay, float adjusted_lr, cudaStream_t st) {
  const long long n = (long long)rows * cols;
  if (n <= 0) return 0;
  muon_apply_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, st>>>(p, (const __nv_bfloat16*)o, (__nv_bfloat16*)p_lp, rows,
                                                              cols, transposed, lr, weight_decay, adjusted_lr);
  return (int)cudaGetLastError();
}

// elem_size in {1,2,4,8}; offsets/lengths are in elements and live in device memory.
MFSDP_API int mfsdp_copy_segments(const void* src, void* dst, const long long* src_off,
                                  const long long* dst_off, const long long* len, int nseg,
                                  long long max_len, int elem_size, cudaStream_t st) {
  if (nseg <= 0) return 0;
  SegTable tab{src_off, dst_off, len};
  const int per16 = 16 / elem_size;
  int gx = grid_for(max_len / per16 + 1, 256, 148 * 4);
  int gy = nseg < 65535 ? nseg : 65535;
  if ((long long)gx * gy > 148 * 16) gx = (148 * 16 + gy - 1) / gy;
  dim3 grid(gx, gy);
  switch (elem_size) {
    case 1: copy_segments_kernel<uint8_t><<<grid, 256, 0, st>>>((const uint8_t*)src, (uint8_t*)dst, tab, nseg); break;
    case 2: copy_segments_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t*)src, (uint16_t*)dst, tab, nseg); break;
    case 4: copy_segments_kernel<uint32_t><<<grid, 256, 0, st>>>((const uint32_t*)src, (uint32_t*)dst, tab, nseg); break;
    case 8: copy_segments_kernel<uint64_t><<<grid, 256, 0, st>>>((const uint64_t*)src, (uint64_t*)dst, tab, nseg); break;
    default: return -2;
  }
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  cast_f32_bf16_kernel<<<grid_for(n / 4 + 1, 256, 148 * 8), 256, 0, st>>>(src, (__nv_bfloat16*)dst, n);
  return (int)cudaGetLastError();
}

// ============================================================== allocation-free RMSNorm backward
// Declared and documented in mfsdp_noalloc.h.  The weight-gradient partial sums go to a device
// array that is part of the library image instead of a caller-provided buffer.  In host code the
// array's name is only a handle for the runtime, so its device address is looked up once per device
// with cudaGetSymbolAddress and that pointer is what the kernels receive.
#include "mfsdp_noalloc.h"

namespace mfsdp {
static __device__ __align__(256) float g_noalloc_dw_scratch[MFSDP_NOALLOC_SCRATCH_ROWS * MFSDP_NOALLOC_MAX_HIDDEN];
constexpr int kNoAllocMaxDevices = 64;
static float* g_noalloc_scratch_addr[kNoAllocMaxDevices] = {nullptr};
}  // namespace mfsdp

MFSDP_API int mfsdp_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                        const void* dres, void* dx, void* dw, int accumulate_dw, long long rows,
                                        int H, cudaStream_t st) {
  if (rows <= 0 || H <= 0 || H % 8 || H > MFSDP_NOALLOC_MAX_HIDDEN) return -2;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoAllocMaxDevices) return -2;
  float* scratch = g_noalloc_scratch_addr[dev];
  if (scratch == nullptr) {
    // set-up, once per device, with that device current
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_dw_scratch);
    if (e != cudaSuccess) return (int)e;
    scratch = static_cast<float*>(p);
    g_noalloc_scratch_addr[dev] = scratch;
  }
  const int nvec = H / 8;
  const int threads = 256;
  const int vpt = (nvec + threads - 1) / threads;
  const int grid = rmsnorm_bwd_grid(rows, vpt <= 1 ? 4 : (vpt <= 2 ? 2 : 1), MFSDP_NOALLOC_SCRATCH_ROWS);
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  auto DR = (const __nv_bfloat16*)dres; auto DX = (__nv_bfloat16*)dx;
  if (vpt <= 1) rmsnorm_bwd_kernel<1, 4><<<grid, threads, 0, st>>>(DY, X, W, rstd, DR, DX, scratch, rows, H);
  else if (vpt <= 2) rmsnorm_bwd_kernel<2, 2><<<grid, threads, 0, st>>>(DY, X, W, rstd, DR, DX, scratch, rows, H);
  else if (vpt <= 4) rmsnorm_bwd_kernel<4, 1><<<grid, threads, 0, st>>>(DY, X, W, rstd, DR, DX, scratch, rows, H);
  else return -2;
  if (dw) colsum_f32_to_bf16_kernel<<<(H + 31) / 32, dim3(32, 8), 0, st>>>(scratch, (__nv_bfloat16*)dw, grid, H, accumulate_dw);
  return (int)cudaGetLastError();
}
