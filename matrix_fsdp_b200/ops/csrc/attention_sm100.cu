// Causal self-attention (head_dim 128) for sm_100a on tcgen05 / TMEM, forward and backward.
//
// Input is the fused projection buffer qkv [T, 3H] (row = b*S + s; q heads, then k heads, then v heads,
// RoPE already applied); output is [T, H] plus the per-row log-sum-exp the backward needs.
//
// Forward, one CTA per (batch, head, 128-query tile), 192 threads:
//   warp 0   : TMA producer (Q once, then K/V tiles of 128 keys through a 2-stage ring)
//   warp 1   : tcgen05.mma issuer.  S_j = Q K_j^T goes to one of two TMEM buffers so that S_{j+1} is
//              computed while the softmax of tile j runs; O += P_j V_j accumulates in TMEM.
//   warps 2-5: softmax.  Thread r owns query row r (the 32x32b TMEM load shape gives one row per lane,
//              so row max / row sum need no shuffles), writes P as bf16 into a 128B-swizzled shared
//              tile (the A operand of the second MMA) and rescales O in TMEM only when the running
//              maximum moved by more than 2^8 (lazy rescaling).
// Every wait is bounded; on a timeout the kernel records a status code and leaves through the normal
// teardown.
//
// The reference calls F.scaled_dot_product_attention in its bench models
// (test/fsdp/bench_fsdp2_compare.py:419,480); this file is that op written for Blackwell.
#include "common.cuh"
#include <cuda.h>

namespace mfsdp {

int make_tmap_bf16_2d(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld,
                      int box_rows, int box_cols);   // defined in gemm_sm100.cu

constexpr int kHd = 128;            // head dim
constexpr int kBq = 128;            // queries per CTA
constexpr int kBk = 128;            // keys per iteration
constexpr int kTileBytes = 128 * 128 * 2;   // one [128 x 128] bf16 tile = two 64-column chunks of 16 KB
constexpr int kHalfTile = kTileBytes / 2;
constexpr int kAttnThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnFwdArgs {
  int B, S, nH;
  float scale_log2;          // softmax scale * log2(e)
  __nv_bfloat16* out;        // [T, H]
  long long ld_out;
  float* lse;                // [B, nH, S]  natural-log log-sum-exp of the scaled scores
  int* status;
};

struct AttnFwdSmem {
  // offsets from the 1024-aligned base
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;            // 2 stages
  static constexpr int kV = kK + 2 * kTileBytes;        // 2 stages
  static constexpr int kP = kV + 2 * kTileBytes;
  static constexpr int kBars = kP + kTileBytes;
  static constexpr int kBytes = kBars + 256 + 1024;
};

__device__ __forceinline__ void softmax_bar_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// Issue the 8 k-steps of a 128x128x128 MMA whose operands are [128 x 128] bf16 tiles stored as two
// 64-column swizzled chunks.  A K-major operand advances 32 B per k-step inside a chunk and one chunk
// per 64 k; an MN-major operand advances 16 rows (2048 B) per k-step.
__device__ __forceinline__ void mma_tile_128(uint32_t tmem_d, uint32_t a_base, bool a_mn, uint32_t b_base, bool b_mn,
                                             uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint64_t ad = a_mn ? make_smem_desc_sw128(a_base + k * 2048, kHalfTile, 1024)
                             : make_smem_desc_sw128(a_base + (k >> 2) * kHalfTile + (k & 3) * 32, 16, 1024);
    const uint64_t bd = b_mn ? make_smem_desc_sw128(b_base + k * 2048, kHalfTile, 1024)
                             : make_smem_desc_sw128(b_base + (k >> 2) * kHalfTile + (k & 3) * 32, 16, 1024);
    umma_f16_ss(tmem_d, ad, bd, idesc, (accumulate || k > 0) ? 1u : 0u);
  }
}

// Load a [128 rows x 128 cols] bf16 tile whose top-left corner is (row0, col0) as two 64-column boxes.
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar, int col0, int row0) {
  tma_load_2d(dst, map, bar, col0, row0);
  tma_load_2d(dst + kHalfTile, map, bar, col0 + 64, row0);
}

__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tma_qkv, const AttnFwdArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttnFwdSmem::kBars);
  uint64_t* q_full = bars;             // [1]
  uint64_t* k_full = bars + 1;         // [2]
  uint64_t* k_empty = bars + 3;        // [2]
  uint64_t* v_full = bars + 5;         // [2]
  uint64_t* v_empty = bars + 7;        // [2]
  uint64_t* s_full = bars + 9;         // [2]
  uint64_t* p_full = bars + 11;        // [1]
  uint64_t* pv_done = bars + 12;       // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;     // heavy (late) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int H = p.nH * kHd;
  const int q0 = qt * kBq;
  const int row_base = b * p.S;
  int nkv = (q0 + kBq + kBk - 1) / kBk;
  const int max_kv = (p.S + kBk - 1) / kBk;
  if (nkv > max_kv) nkv = max_kv;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 13; ++i) mbar_init(smem_u32(&bars[i]), (i == 11) ? 128 : 1);
    mbar_fence_init();
    tma_prefetch_desc(&tma_qkv);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;
  const uint32_t sQ = smem_u32(smem + AttnFwdSmem::kQ), sK = smem_u32(smem + AttnFwdSmem::kK),
                 sV = smem_u32(smem + AttnFwdSmem::kV), sP = smem_u32(smem + AttnFwdSmem::kP);

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(smem_u32(q_full), kTileBytes);
      tma_load_tile(sQ, &tma_qkv, smem_u32(q_full), h * kHd, row_base + q0);
      for (int j = 0; j < nkv; ++j) {
        const uint32_t s = j & 1, ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&k_empty[s]), ph ^ 1, p.status, abort_flag)) break;
        mbar_arrive_expect_tx(smem_u32(&k_full[s]), kTileBytes);
        tma_load_tile(sK + s * kTileBytes, &tma_qkv, smem_u32(&k_full[s]), H + h * kHd, row_base + j * kBk);
        if (!mbar_wait(smem_u32(&v_empty[s]), ph ^ 1, p.status, abort_flag)) break;
        mbar_arrive_expect_tx(smem_u32(&v_full[s]), kTileBytes);
        tma_load_tile(sV + s * kTileBytes, &tma_qkv, smem_u32(&v_full[s]), 2 * H + h * kHd, row_base + j * kBk);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);
      bool ok = mbar_wait(smem_u32(q_full), 0, p.status, abort_flag) &&
                mbar_wait(smem_u32(&k_full[0]), 0, p.status, abort_flag);
      if (ok) {
        tc_fence_after();
        mma_tile_128(tmem_base, sQ, false, sK, false, idesc_s, false);
        umma_commit(smem_u32(&k_empty[0]));
        umma_commit(smem_u32(&s_full[0]));
      }
      for (int j = 0; j < nkv && ok; ++j) {
        if (j + 1 < nkv) {
          const uint32_t s1 = (j + 1) & 1, ph1 = ((j + 1) >> 1) & 1;
          if (!mbar_wait(smem_u32(&k_full[s1]), ph1, p.status, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_tile_128(tmem_base + s1 * 128, sQ, false, sK + s1 * kTileBytes, false, idesc_s, false);
          umma_commit(smem_u32(&k_empty[s1]));
          umma_commit(smem_u32(&s_full[s1]));
        }
        const uint32_t s = j & 1, ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(p_full), j & 1, p.status, abort_flag)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&v_full[s]), ph, p.status, abort_flag)) { ok = false; break; }
        tc_fence_after();
        mma_tile_128(tmem_o, sP, false, sV + s * kTileBytes, true, idesc_o, j > 0);
        umma_commit(smem_u32(&v_empty[s]));
        umma_commit(smem_u32(pv_done));
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue (128 threads)
    const int q = warp & 3;
    const int r = q * 32 + lane;                 // query row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const int qi = q0 + r;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      mbar_wait(smem_u32(&s_full[j & 1]), (j >> 1) & 1, p.status, abort_flag);
      softmax_bar_sync();
      if (*abort_flag) { ok = false; break; }
      tc_fence_after();
      float s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(tmem_base + (j & 1) * 128 + lane_off + c * 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) s[c * 32 + e] = __uint_as_float(t[e]);
      }
      if (j == nkv - 1) {
        const int kv0 = j * kBk;
#pragma unroll
        for (int e = 0; e < 128; ++e)
          if (kv0 + e > qi) s[e] = -INFINITY;
      }
      float mx = s[0];
#pragma unroll
      for (int e = 1; e < 128; ++e) mx = fmaxf(mx, s[e]);
      mx *= p.scale_log2;
      if (mx == -INFINITY) mx = 0.f;
      float m_new = fmaxf(m_used, mx);
      const bool need = (j > 0) && (m_new - m_used > 8.f);
      const bool any_need = __any_sync(0xffffffffu, need);
      const float m_next = (j == 0 || any_need) ? m_new : m_used;
      const float factor = (j == 0) ? 0.f : exp2f(m_used - m_next);
      float sum = 0.f;
      uint32_t pk[64];
#pragma unroll
      for (int e = 0; e < 64; ++e) {
        const float p0 = exp2f(s[2 * e] * p.scale_log2 - m_next);
        const float p1 = exp2f(s[2 * e + 1] * p.scale_log2 - m_next);
        sum += p0 + p1;
        pk[e] = pack_bf16x2(p0, p1);
      }
      l = l * factor + sum;
      m_used = m_next;
      if (j > 0) {
        mbar_wait(smem_u32(pv_done), (j - 1) & 1, p.status, abort_flag);
        softmax_bar_sync();
        if (*abort_flag) { ok = false; break; }
        tc_fence_after();
        if (any_need) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t t[32];
            tmem_ld_32x32b_x32(tmem_o + lane_off + c * 32, t);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) t[e] = __float_as_uint(__uint_as_float(t[e]) * factor);
            tmem_st_32x32b_x32(tmem_o + lane_off + c * 32, t);
          }
          tmem_st_wait();
        }
      }
      uint8_t* prow = smem + AttnFwdSmem::kP + r * 128;
#pragma unroll
      for (int kc = 0; kc < 16; ++kc) {
        const int phys = (kc & 7) ^ (r & 7);
        *reinterpret_cast<uint4*>(prow + (kc >> 3) * kHalfTile + phys * 16) =
            make_uint4(pk[kc * 4], pk[kc * 4 + 1], pk[kc * 4 + 2], pk[kc * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(p_full));
    }
    if (ok) {
      mbar_wait(smem_u32(pv_done), (nkv - 1) & 1, p.status, abort_flag);
      softmax_bar_sync();
      ok = !*abort_flag;
    }
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l;
      const bool row_ok = qi < p.S;
      __nv_bfloat16* orow = p.out + (long long)(row_base + qi) * p.ld_out + h * kHd;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(tmem_o + lane_off + c * 32, t);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(t[g * 8 + 0]) * inv, __uint_as_float(t[g * 8 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(t[g * 8 + 2]) * inv, __uint_as_float(t[g * 8 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(t[g * 8 + 4]) * inv, __uint_as_float(t[g * 8 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(t[g * 8 + 6]) * inv, __uint_as_float(t[g * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = o;
          }
        }
      }
      if (row_ok && p.lse) p.lse[((long long)b * p.nH + h) * p.S + qi] = (m_used + log2f(l)) * 0.6931471805599453f;
    }
  }
  if (*abort_flag) __nanosleep(1000000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace mfsdp

using namespace mfsdp;

// qkv: [B*S, 3*nH*128] bf16 (row stride ld_qkv elements); out: [B*S, nH*128]; lse: [B, nH, S] fp32.
MFSDP_API int mfsdp_attention_fwd(const void* qkv, void* out, float* lse, int B, int S, int nH, long long ld_qkv,
                                  long long ld_out, float softmax_scale, int* status, cudaStream_t st) {
  if (B <= 0 || S <= 0 || nH <= 0 || (ld_qkv % 8) || (ld_out % 8)) return -2;
  cudaFree(nullptr);   // tensor-map encoding needs a current context on this thread
  CUtensorMap map;
  int rc = make_tmap_bf16_2d(&map, qkv, (long long)B * S, 3LL * nH * kHd, ld_qkv, 128, 64);
  if (rc) return rc;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnFwdSmem::kBytes);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  AttnFwdArgs a{};
  a.B = B; a.S = S; a.nH = nH;
  a.scale_log2 = softmax_scale * kLog2e;
  a.out = (__nv_bfloat16*)out; a.ld_out = ld_out; a.lse = lse; a.status = status;
  dim3 grid((S + kBq - 1) / kBq, nH, B);
  attn_fwd_kernel<<<grid, kAttnThreads, AttnFwdSmem::kBytes, st>>>(map, a);
  return (int)cudaGetLastError();
}
