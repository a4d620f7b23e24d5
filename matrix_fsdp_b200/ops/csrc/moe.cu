// Mixture-of-experts routing and expert-parallel dispatch / combine kernels for sm_100a.
//
// Data flow of one MoE layer (W expert-parallel ranks, E experts, E/W per rank, top-K routing):
//   router_topk      softmax over expert logits, top-K ids and weights per token
//   assign_slots     deterministic position of every (token, k) entry inside its expert's queue
//   push_counts      every rank writes its per-expert counts into every peer's table
//   plan             from the W x E table: where my rows for expert e start in the owner's buffer,
//                    256-row aligned expert groups on the owner, tile->expert map for the grouped GEMM
//   dispatch_push    permute + all-to-all in one step: each entry's hidden row is stored straight
//                    into the owner's receive buffer over mapped peer memory
//   (grouped GEMMs on the owner: gemm_sm100.cu)
//   combine_pull     unpermute + all-to-all + weighted sum in one step: each token pulls its K expert
//                    rows from the owners' output buffers and reduces them in registers
// The reference has no expert-parallel runtime; its test fixture dispatches with four
// all_to_all_single calls plus argsort / index_select / scatter_add
// (test/fsdp/test_deepseek_v3_ep_train.py:472-563).  Cross-rank ordering uses the epoch flags of
// peer.cu (bounded waits); these kernels only move data.
#include "common.cuh"

namespace mfsdp {

constexpr int kMaxEpRanks = 16;
constexpr int kMaxTopK = 8;

struct EpPtrs {
  void* p[kMaxEpRanks];
};

// ------------------------------------------------------------------ router
// One warp per token.  logits: [T, E] bf16 (row stride ld).  E <= 256 (lanes past E hold -inf / 0).
template <int VPL>
__global__ void moe_router_topk_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int T, int E, int K,
                                       float* __restrict__ probs, int* __restrict__ topk_idx,
                                       float* __restrict__ topk_w, float* __restrict__ prob_sum) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float v[VPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    v[i] = (i * 32 + lane < E) ? __bfloat162float(logits[(long long)t * ld + i * 32 + lane]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    v[i] = __expf(v[i] - mx);
    sum += v[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    v[i] *= inv;
    if (i * 32 + lane < E) {
      probs[(long long)t * E + i * 32 + lane] = v[i];
      if (prob_sum) atomicAdd(&prob_sum[i * 32 + lane], v[i]);
    } else {
      v[i] = -2.f;   // never selected
    }
  }
  unsigned taken = 0;
  for (int k = 0; k < K; ++k) {
    float best = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (!((taken >> i) & 1u) && v[i] > best) {
        best = v[i];
        bi = i * 32 + lane;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
    if (lane == 0) {
      topk_idx[(long long)t * K + k] = bi;
      topk_w[(long long)t * K + k] = best;
    }
  }
}

// dlogits = p * (dprobs - <p, dprobs>), dprobs[e] = aux_grad[e] + sum_k [idx_k == e] dw_k.
template <int VPL>
__global__ void moe_router_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ topk_idx,
                                      const float* __restrict__ dw, const float* __restrict__ aux_grad, int T, int E,
                                      int K, __nv_bfloat16* __restrict__ dlogits, long long ld) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float p[VPL], d[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const bool in = i * 32 + lane < E;
    p[i] = in ? probs[(long long)t * E + i * 32 + lane] : 0.f;
    d[i] = (in && aux_grad) ? aux_grad[i * 32 + lane] : 0.f;
  }
  for (int k = 0; k < K; ++k) {
    const int e = topk_idx[(long long)t * K + k];
    const float g = dw[(long long)t * K + k];
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (e == i * 32 + lane) d[i] += g;
  }
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) dot += p[i] * d[i];
  dot = warp_sum(dot);
#pragma unroll
  for (int i = 0; i < VPL; ++i)
    if (i * 32 + lane < E) dlogits[(long long)t * ld + i * 32 + lane] = __float2bfloat16(p[i] * (d[i] - dot));
}

// ------------------------------------------------------------------ slots
// Block e walks all N = T*K entries in order and numbers the ones routed to expert e, so slot order
// is token order (deterministic).  counts[e] = number of entries of expert e.
__global__ void moe_assign_slots_kernel(const int* __restrict__ topk_idx, int N, int* __restrict__ slot,
                                        int* __restrict__ counts) {
  __shared__ int warp_tot[8];
  __shared__ int running;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  for (int base = 0; base < N; base += 256 * 4) {
    const int i0 = base + threadIdx.x * 4;
    int f[4], c = 0;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      f[u] = (i0 + u < N) && (topk_idx[i0 + u] == e);
      c += f[u];
    }
    int incl = c;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += o;
    }
    if (lane == 31) warp_tot[wid] = incl;
    __syncthreads();
    int pre = running;
    for (int w = 0; w < wid; ++w) pre += warp_tot[w];
    int pos = pre + incl - c;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (f[u]) slot[i0 + u] = pos++;
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < 8; ++w) tot += warp_tot[w];
      running += tot;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = running;
}

// Write my counts row into every rank's [W, E] table.
__global__ void moe_push_counts_kernel(EpPtrs tables, int W, int rank, const int* __restrict__ counts, int E) {
  for (int i = threadIdx.x; i < W * E; i += blockDim.x) {
    const int r = i / E, e = i % E;
    reinterpret_cast<int*>(tables.p[r])[rank * E + e] = counts[e];
  }
}

// ------------------------------------------------------------------ plan
// counts_all: [W, E] (row = source rank).  Expert e lives on rank e / El; on its owner the rows of
// expert e form one group that starts on a 256-row boundary, ordered by source rank.
//   dest_base[e]       row in the owner's buffer where this rank's rows for expert e start
//   group_offsets[El+1] padded group starts of my experts (clamped to the capacity)
//   group_rows[El]     real rows of each of my groups (clamped)
//   tile_group[tiles]  expert of every 128-row tile of my buffer, -1 for unused tiles
//   stats[0] = padded rows in use on this rank, stats[1] = rows lost to the capacity limit (this rank as owner)
// Expert groups start on multiples of this many rows: whole 256-row tiles per group let the grouped GEMMs run on
// CTA pairs (a pair's two CTAs share one B operand, so a 256-row tile must belong to one expert).
constexpr int kGroupAlign = 256;

__global__ void moe_plan_kernel(const int* __restrict__ counts_all, int W, int rank, int E, int cap_rows,
                                int* __restrict__ dest_base, int* __restrict__ group_offsets,
                                int* __restrict__ group_rows, int* __restrict__ tile_group, int* __restrict__ stats) {
  __shared__ int total[256], before[256], start[256];
  const int El = E / W;
  const int cap = cap_rows / kGroupAlign * kGroupAlign;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, bef = 0;
    for (int s = 0; s < W; ++s) {
      const int c = counts_all[s * E + e];
      if (s < rank) bef += c;
      tot += c;
    }
    total[e] = tot;
    before[e] = bef;
  }
  __syncthreads();
  if (threadIdx.x < W) {
    const int r = threadIdx.x;
    int acc = 0;
    for (int el = 0; el < El; ++el) {
      const int e = r * El + el;
      start[e] = acc;
      acc += (total[e] + kGroupAlign - 1) / kGroupAlign * kGroupAlign;
    }
    if (r == rank) {
      int lost = 0;
      for (int el = 0; el < El; ++el) {
        const int e = r * El + el;
        const int st = min(start[e], cap);
        const int rows = max(0, min(total[e], cap - st));
        group_offsets[el] = st;
        group_rows[el] = rows;
        lost += total[e] - rows;
      }
      group_offsets[El] = min(acc, cap);
      stats[0] = min(acc, cap);
      stats[1] = lost;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) dest_base[e] = start[e] + before[e];
  const int tiles = cap / 128;
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    const int row = t * 128;
    int g = -1;
    for (int el = 0; el < El; ++el) {
      const int e = rank * El + el;
      if (row >= start[e] && row < start[e] + (total[e] + kGroupAlign - 1) / kGroupAlign * kGroupAlign) g = el;
    }
    tile_group[t] = g;
  }
}

// Zero the alignment rows at the end of each of my expert groups (so they contribute nothing to
// the grouped GEMMs, whatever an earlier layer left in the buffer).
__global__ void moe_zero_pad_kernel(__nv_bfloat16* __restrict__ buf, int H, const int* __restrict__ group_offsets,
                                    const int* __restrict__ group_rows) {
  const int el = blockIdx.x;
  const int r0 = group_offsets[el] + group_rows[el];
  const int r1 = min(group_offsets[el + 1], (r0 + kGroupAlign - 1) / kGroupAlign * kGroupAlign);
  const int vpr = H >> 3;
  const long long n = (long long)max(0, r1 - r0) * vpr;
  uint4* base = reinterpret_cast<uint4*>(buf + (long long)r0 * H);
  for (long long i = threadIdx.x; i < n; i += blockDim.x) base[i] = make_uint4(0, 0, 0, 0);
}

// ------------------------------------------------------------------ dispatch (permute + all-to-all)
// One warp per (token, k) entry.  With route_in == nullptr the destination row is
// dest_base[e] + slot and is recorded in route_out (-1 when it falls outside the capacity); with
// route_in the recorded rows are reused (backward re-dispatch of gradients).
__global__ void moe_dispatch_push_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int H, int N, int K,
                                         const int* __restrict__ topk_idx, const int* __restrict__ slot,
                                         const int* __restrict__ dest_base, const int* __restrict__ route_in,
                                         int* __restrict__ route_out, const float* __restrict__ scale, int El,
                                         int cap_rows, EpPtrs recv) {
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (i >= N) return;
  const int e = topk_idx[i];
  int row;
  if (route_in) {
    row = route_in[i];
  } else {
    row = dest_base[e] + slot[i];
    if (row >= cap_rows / 256 * 256) row = -1;
    if (lane == 0) route_out[i] = row;
  }
  if (row < 0) return;
  const int t = i / K;
  const float s = scale ? scale[i] : 1.f;
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * ldx);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(recv.p[e / El]) + (long long)row * H);
  for (int v = lane; v < (H >> 3); v += 32) {
    uint4 a = src[v];
    if (scale) {
      uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16x2(w[q]);
        w[q] = pack_bf16x2(f.x * s, f.y * s);
      }
      a = make_uint4(w[0], w[1], w[2], w[3]);
    }
    dst[v] = a;
  }
}

// ------------------------------------------------------------------ combine (all-to-all + unpermute + weighted sum)
// One warp per token: out[t] = res[t] + sum_k w[t,k] * src_{rank(t,k)}[route[t,k]].  With row_scalar
// tables given, scal_out[t,k] = row_scalar_{rank}[route] / max(w, tiny) is pulled as well
// (the router-weight gradient that the owner computed per row).
__global__ void moe_combine_pull_kernel(__nv_bfloat16* __restrict__ out, long long ldo, int H, int T, int K,
                                        const int* __restrict__ topk_idx, const int* __restrict__ route,
                                        const float* __restrict__ weight, const __nv_bfloat16* __restrict__ res,
                                        long long ldres, int El, EpPtrs src, EpPtrs row_scalar,
                                        float* __restrict__ scal_out, int has_scalar) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const uint4* rows[kMaxTopK];
  float w[kMaxTopK];
#pragma unroll
  for (int k = 0; k < kMaxTopK; ++k) {
    rows[k] = nullptr;
    w[k] = 0.f;
    if (k < K) {
      const long long i = (long long)t * K + k;
      const int row = route[i];
      const int r = topk_idx[i] / El;
      w[k] = weight ? weight[i] : 1.f;
      if (row >= 0) rows[k] = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src.p[r]) + (long long)row * H);
      if (has_scalar && lane == k) {
        const float wv = weight ? weight[i] : 1.f;
        scal_out[i] = (row >= 0) ? reinterpret_cast<const float*>(row_scalar.p[r])[row] / fmaxf(wv, 1e-20f) : 0.f;
      }
    }
  }
  for (int v = lane; v < (H >> 3); v += 32) {
    float acc[8];
    if (res) {
      const uint4 a = *reinterpret_cast<const uint4*>(res + (long long)t * ldres + v * 8);
      const float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      acc[0] = f0.x; acc[1] = f0.y; acc[2] = f1.x; acc[3] = f1.y; acc[4] = f2.x; acc[5] = f2.y; acc[6] = f3.x; acc[7] = f3.y;
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
    }
    uint4 a[kMaxTopK];
#pragma unroll
    for (int k = 0; k < kMaxTopK; ++k)
      if (k < K && rows[k]) a[k] = rows[k][v];
#pragma unroll
    for (int k = 0; k < kMaxTopK; ++k) {
      if (k < K && rows[k]) {
        const float2 f0 = unpack_bf16x2(a[k].x), f1 = unpack_bf16x2(a[k].y), f2 = unpack_bf16x2(a[k].z), f3 = unpack_bf16x2(a[k].w);
        acc[0] += w[k] * f0.x; acc[1] += w[k] * f0.y; acc[2] += w[k] * f1.x; acc[3] += w[k] * f1.y;
        acc[4] += w[k] * f2.x; acc[5] += w[k] * f2.y; acc[6] += w[k] * f3.x; acc[7] += w[k] * f3.y;
      }
    }
    *reinterpret_cast<uint4*>(out + (long long)t * ldo + v * 8) =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

// ------------------------------------------------------------------ expert SwiGLU backward with row dot
// One warp per row (rows >= *row_limit are skipped):
//   h = silu(gate) * up (recomputed and written for the down-projection wgrad),
//   dgu = swiglu'(gu) * dh,  rowdot[row] = <h, dh>.
__global__ void moe_swiglu_bwd_dot_kernel(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ gu,
                                          __nv_bfloat16* __restrict__ dgu, __nv_bfloat16* __restrict__ h,
                                          float* __restrict__ rowdot, int R, int F, const int* __restrict__ row_limit) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= R || (row_limit && row >= *row_limit)) return;
  float dot = 0.f;
  for (int v = lane; v < (F >> 3); v += 32) {
    const uint4 g = *reinterpret_cast<const uint4*>(gu + (long long)row * 2 * F + v * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + (long long)row * 2 * F + F + v * 8);
    const uint4 d = *reinterpret_cast<const uint4*>(dh + (long long)row * F + v * 8);
    const uint32_t gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w}, dd[4] = {d.x, d.y, d.z, d.w};
    uint32_t og[4], ou[4], oh[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = unpack_bf16x2(gg[e]), b = unpack_bf16x2(uu[e]), c = unpack_bf16x2(dd[e]);
      const float sgx = 1.f / (1.f + __expf(-a.x)), sgy = 1.f / (1.f + __expf(-a.y));
      const float silx = a.x * sgx, sily = a.y * sgy;
      const float dsx = sgx * (1.f + a.x * (1.f - sgx)), dsy = sgy * (1.f + a.y * (1.f - sgy));
      const float hx = silx * b.x, hy = sily * b.y;
      dot += hx * c.x + hy * c.y;
      og[e] = pack_bf16x2(c.x * b.x * dsx, c.y * b.y * dsy);
      ou[e] = pack_bf16x2(c.x * silx, c.y * sily);
      oh[e] = pack_bf16x2(hx, hy);
    }
    *reinterpret_cast<uint4*>(dgu + (long long)row * 2 * F + v * 8) = make_uint4(og[0], og[1], og[2], og[3]);
    *reinterpret_cast<uint4*>(dgu + (long long)row * 2 * F + F + v * 8) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
    *reinterpret_cast<uint4*>(h + (long long)row * F + v * 8) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
  }
  dot = warp_sum(dot);
  if (lane == 0) rowdot[row] = dot;
}

}  // namespace mfsdp

using namespace mfsdp;

static EpPtrs make_ptrs(const unsigned long long* addrs, int n) {
  EpPtrs p{};
  for (int i = 0; i < n && i < kMaxEpRanks; ++i) p.p[i] = reinterpret_cast<void*>(addrs[i]);
  return p;
}

MFSDP_API int mfsdp_moe_router_topk(const void* logits, long long ld, int T, int E, int K, float* probs, int* topk_idx,
                                    float* topk_w, float* prob_sum, cudaStream_t st) {
  if (E < 1 || E > 256 || K < 1 || K > kMaxTopK || K > E) return -2;
  const int grid = (T + 7) / 8;
  auto lg = (const __nv_bfloat16*)logits;
  const int vpl = (E + 31) / 32;
  switch (vpl <= 1 ? 1 : vpl <= 2 ? 2 : vpl <= 4 ? 4 : 8) {
    case 1: moe_router_topk_kernel<1><<<grid, 256, 0, st>>>(lg, ld, T, E, K, probs, topk_idx, topk_w, prob_sum); break;
    case 2: moe_router_topk_kernel<2><<<grid, 256, 0, st>>>(lg, ld, T, E, K, probs, topk_idx, topk_w, prob_sum); break;
    case 4: moe_router_topk_kernel<4><<<grid, 256, 0, st>>>(lg, ld, T, E, K, probs, topk_idx, topk_w, prob_sum); break;
    case 8: moe_router_topk_kernel<8><<<grid, 256, 0, st>>>(lg, ld, T, E, K, probs, topk_idx, topk_w, prob_sum); break;
    default: return -2;
  }
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_moe_router_bwd(const float* probs, const int* topk_idx, const float* dw, const float* aux_grad, int T,
                                   int E, int K, void* dlogits, long long ld, cudaStream_t st) {
  if (E < 1 || E > 256 || K < 1 || K > kMaxTopK) return -2;
  const int grid = (T + 7) / 8;
  auto dl = (__nv_bfloat16*)dlogits;
  const int vpl = (E + 31) / 32;
  switch (vpl <= 1 ? 1 : vpl <= 2 ? 2 : vpl <= 4 ? 4 : 8) {
    case 1: moe_router_bwd_kernel<1><<<grid, 256, 0, st>>>(probs, topk_idx, dw, aux_grad, T, E, K, dl, ld); break;
    case 2: moe_router_bwd_kernel<2><<<grid, 256, 0, st>>>(probs, topk_idx, dw, aux_grad, T, E, K, dl, ld); break;
    case 4: moe_router_bwd_kernel<4><<<grid, 256, 0, st>>>(probs, topk_idx, dw, aux_grad, T, E, K, dl, ld); break;
    case 8: moe_router_bwd_kernel<8><<<grid, 256, 0, st>>>(probs, topk_idx, dw, aux_grad, T, E, K, dl, ld); break;
    default: return -2;
  }
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_moe_assign_slots(const int* topk_idx, int N, int E, int* slot, int* counts, cudaStream_t st) {
  moe_assign_slots_kernel<<<E, 256, 0, st>>>(topk_idx, N, slot, counts);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_moe_push_counts(const unsigned long long* tables, int W, int rank, const int* counts, int E,
                                    cudaStream_t st) {
  if (W < 1 || W > kMaxEpRanks) return -2;
  moe_push_counts_kernel<<<1, 256, 0, st>>>(make_ptrs(tables, W), W, rank, counts, E);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_moe_plan(const int* counts_all, int W, int rank, int E, int cap_rows, int* dest_base,
                             int* group_offsets, int* group_rows, int* tile_group, int* stats, cudaStream_t st) {
  if (W < 1 || W > kMaxEpRanks || E > 256 || E % W) return -2;
  moe_plan_kernel<<<1, 256, 0, st>>>(counts_all, W, rank, E, cap_rows, dest_base, group_offsets, group_rows, tile_group, stats);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_moe_zero_pad(void* buf, int H, int El, const int* group_offsets, const int* group_rows,
                                 cudaStream_t st) {
  moe_zero_pad_kernel<<<El, 256, 0, st>>>((__nv_bfloat16*)buf, H, group_offsets, group_rows);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_moe_dispatch_push(const void* x, long long ldx, int H, int N, int K, const int* topk_idx,
                                      const int* slot, const int* dest_base, const int* route_in, int* route_out,
                                      const float* scale, int El, int cap_rows, const unsigned long long* recv, int W,
                                      cudaStream_t st) {
  if (H % 8 || W < 1 || W > kMaxEpRanks || (!route_in && !route_out)) return -2;
  moe_dispatch_push_kernel<<<(N + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, H, N, K, topk_idx, slot, dest_base,
                                                       route_in, route_out, scale, El, cap_rows, make_ptrs(recv, W));
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_moe_combine_pull(void* out, long long ldo, int H, int T, int K, const int* topk_idx, const int* route,
                                     const float* weight, const void* res, long long ldres, int El,
                                     const unsigned long long* src, const unsigned long long* row_scalar,
                                     float* scal_out, int W, cudaStream_t st) {
  if (H % 8 || W < 1 || W > kMaxEpRanks || K > kMaxTopK) return -2;
  EpPtrs sc = row_scalar ? make_ptrs(row_scalar, W) : EpPtrs{};
  moe_combine_pull_kernel<<<(T + 7) / 8, 256, 0, st>>>((__nv_bfloat16*)out, ldo, H, T, K, topk_idx, route, weight,
                                                      (const __nv_bfloat16*)res, ldres, El, make_ptrs(src, W), sc,
                                                      scal_out, row_scalar ? 1 : 0);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_moe_swiglu_bwd_dot(const void* dh, const void* gu, void* dgu, void* h, float* rowdot, int R, int F,
                                       const int* row_limit, cudaStream_t st) {
  if (F % 8) return -2;
  moe_swiglu_bwd_dot_kernel<<<(R + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)dh, (const __nv_bfloat16*)gu,
                                                        (__nv_bfloat16*)dgu, (__nv_bfloat16*)h, rowdot, R, F, row_limit);
  return (int)cudaGetLastError();
}
