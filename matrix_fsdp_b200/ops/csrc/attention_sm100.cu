// Causal self-attention (head_dim 128) for sm_100a on tcgen05 / TMEM, forward and backward.
//
// Input is the fused projection buffer qkv [T, 3H] (row = b*S + s; q heads, then k heads, then v heads,
// RoPE already applied); output is [T, H] plus the per-row log-sum-exp the backward needs.
//
// Forward, one CTA per (batch, head, 128-query tile), 192 threads:
//   warp 0   : TMA producer (Q once, then K/V tiles of 128 keys through a 2-stage ring)
//   warp 1   : tcgen05.mma issuer.  S_j = Q K_j^T goes to one of two TMEM buffers so that S_{j+1} is
//              computed while the softmax of tile j runs; O += P_j V_j accumulates in TMEM.
//   warps 2-9: softmax.  Two threads own query row r (the 32x32b TMEM load shape gives one row per
//              lane), one per 64-key half; they exchange the half-row maximum through shared memory,
//              write P as bf16 into a 128B-swizzled shared tile (the A operand of the second MMA) and
//              rescale O in TMEM only when the running maximum moved by more than 2^8 (lazy rescaling).
// Every wait is bounded; on a timeout the kernel records a status code and leaves through the normal
// teardown.
//
// The reference calls F.scaled_dot_product_attention in its bench models
// (test/fsdp/bench_fsdp2_compare.py:419,480); this file is that op written for Blackwell.
#include "common.cuh"
#include <cuda.h>
#include <cstdlib>

namespace mfsdp {

int make_tmap_bf16_2d(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld,
                      int box_rows, int box_cols);   // defined in gemm_sm100.cu (cached)
void ensure_context_on_this_thread();                // likewise

constexpr int kHd = 128;            // head dim
constexpr int kBq = 128;            // queries per CTA
constexpr int kBk = 128;            // keys per iteration
constexpr int kTileBytes = 128 * 128 * 2;   // one [128 x 128] bf16 tile = two 64-column chunks of 16 KB
constexpr int kHalfTile = kTileBytes / 2;
constexpr int kAttnThreads = 320;          // warp 0 TMA, warp 1 MMA, warps 2-9 softmax (two per TMEM lane quadrant)
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
  static constexpr int kXchg = kP + kTileBytes;          // row max [2 parities][2 halves][128] + row sum [2][128]
  static constexpr int kBars = kXchg + 3 * 1024;
  static constexpr int kBytes = kBars + 256 + 1024;
};

__device__ __forceinline__ void softmax_bar_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }
// Barrier over the 256 softmax threads that also ORs a predicate, so that every thread takes the
// same decision about leaving the loop after a wait ran out.
__device__ __forceinline__ bool softmax_bar_or(bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, 2, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out) : "r"((uint32_t)pred) : "memory");
  return out != 0;
}

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
    for (int i = 0; i < 13; ++i) mbar_init(smem_u32(&bars[i]), (i == 11) ? 256 : 1);
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
    // ------------------------------------------------------------ softmax / epilogue (256 threads)
    const int q = warp & 3;                      // TMEM lane quadrant this warp may access
    const int half = (warp - 2) >> 2;            // which 64 keys of the tile / which 64 columns of O
    const int r = q * 32 + lane;                 // query row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const int qi = q0 + r;
    float* xmax = reinterpret_cast<float*>(smem + AttnFwdSmem::kXchg);     // [parity][half][128]
    float* xsum = xmax + 512;                                              // [half][128]
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      mbar_wait(smem_u32(&s_full[j & 1]), (j >> 1) & 1, p.status, abort_flag);
      tc_fence_after();
      float s[64];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(tmem_base + (j & 1) * 128 + lane_off + half * 64 + c * 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) s[c * 32 + e] = __uint_as_float(t[e]);
      }
      if (j == nkv - 1) {
        const int kv0 = j * kBk + half * 64;
#pragma unroll
        for (int e = 0; e < 64; ++e)
          if (kv0 + e > qi) s[e] = -INFINITY;
      }
      float mx = s[0];
#pragma unroll
      for (int e = 1; e < 64; ++e) mx = fmaxf(mx, s[e]);
      xmax[(j & 1) * 256 + half * 128 + r] = mx;
      if (softmax_bar_or(*abort_flag != 0)) { ok = false; break; }
      mx = fmaxf(mx, xmax[(j & 1) * 256 + (half ^ 1) * 128 + r]) * p.scale_log2;
      if (mx == -INFINITY) mx = 0.f;
      const float m_new = fmaxf(m_used, mx);
      const bool need = (j > 0) && (m_new - m_used > 8.f);
      const bool any_need = __any_sync(0xffffffffu, need);
      const float m_next = (j == 0 || any_need) ? m_new : m_used;
      const float factor = (j == 0) ? 0.f : exp2f(m_used - m_next);
      float sum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float p0 = exp2f(s[2 * e] * p.scale_log2 - m_next);
        const float p1 = exp2f(s[2 * e + 1] * p.scale_log2 - m_next);
        sum += p0 + p1;
        pk[e] = pack_bf16x2(p0, p1);
      }
      l = l * factor + sum;
      m_used = m_next;
      if (j > 0) {
        mbar_wait(smem_u32(pv_done), (j - 1) & 1, p.status, abort_flag);
        tc_fence_after();
        if (any_need) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t t[32];
            tmem_ld_32x32b_x32(tmem_o + lane_off + half * 64 + c * 32, t);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) t[e] = __float_as_uint(__uint_as_float(t[e]) * factor);
            tmem_st_32x32b_x32(tmem_o + lane_off + half * 64 + c * 32, t);
          }
          tmem_st_wait();
        }
      }
      uint8_t* prow = smem + AttnFwdSmem::kP + half * kHalfTile + r * 128;
#pragma unroll
      for (int kc = 0; kc < 8; ++kc) {
        const int phys = kc ^ (r & 7);
        *reinterpret_cast<uint4*>(prow + phys * 16) = make_uint4(pk[kc * 4], pk[kc * 4 + 1], pk[kc * 4 + 2], pk[kc * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(p_full));
    }
    if (ok) {
      mbar_wait(smem_u32(pv_done), (nkv - 1) & 1, p.status, abort_flag);
      xsum[half * 128 + r] = l;
      ok = !softmax_bar_or(*abort_flag != 0);
    }
    if (ok) {
      tc_fence_after();
      l += xsum[(half ^ 1) * 128 + r];
      const float inv = 1.f / l;
      const bool row_ok = qi < p.S;
      __nv_bfloat16* orow = p.out + (long long)(row_base + qi) * p.ld_out + h * kHd + half * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(tmem_o + lane_off + half * 64 + c * 32, t);
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
      if (half == 0 && row_ok && p.lse) p.lse[((long long)b * p.nH + h) * p.S + qi] = (m_used + log2f(l)) * 0.6931471805599453f;
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


// =============================================================================== backward
// Two kernels without atomics, sharing one body:
//   DQ = false: one CTA per (batch, head, 128-key tile).  K_j and V_j stay in shared memory; the
//               query axis streams in tiles of 64 rows (Q_t, dO_t).  S^T = K_j Q_t^T and
//               dP^T = V_j dO_t^T land in TMEM (thread = key row), P^T and dS^T go to swizzled shared
//               tiles, dV += P^T dO_t and dK += dS^T Q_t accumulate in TMEM.
//   DQ = true : one CTA per (batch, head, 128-query tile).  Q_i and dO_i stay; keys stream in tiles
//               of 64 (K_t, V_t).  S = Q_i K_t^T, dP = dO_i V_t^T, dS to shared, dQ += dS K_t.
// The 64-wide streamed tiles leave room for two TMEM buffers of S/dP (2 x 128 columns) beside the
// two 128-column accumulators, and for two stages of every streamed shared tile, so the tensor pipe
// works on tile t+1 while the softmax threads turn tile t into P / dS.
constexpr int kBt = 64;                       // streamed rows per iteration
constexpr int kStreamBytes = kBt * 128 * 2;   // one streamed [64 x 128] tile = two 8 KB chunks
constexpr int kPBytes = 128 * kBt * 2;        // one [128 x 64] P or dS tile (single 64-column chunk)

struct AttnBwdArgs {
  int B, S, nH;
  float scale, scale_log2;
  const float* lse2;         // [B, nH, S] log-sum-exp in log2 units
  const float* delta;        // [B, nH, S] rowsum(dO * O)
  __nv_bfloat16* dqkv;       // [T, 3H]
  long long ld_dqkv;
  int* status;
};

constexpr int kBwdStages = 3;   // streamed-tile ring: deep enough to hide the TMA latency behind two tiles of work

struct AttnBwdSmem {
  static constexpr int kA0 = 0;
  static constexpr int kA1 = kA0 + kTileBytes;
  static constexpr int kB = kA1 + kTileBytes;             // kBwdStages stages x (B0, B1)
  static constexpr int kP = kB + kBwdStages * 2 * kStreamBytes;   // 2 stages x (P, dS)
  static constexpr int kRow = kP + 4 * kPBytes;           // 2 stages x 128 floats (lse2 | delta of the streamed rows)
  static constexpr int kBars = kRow + 2 * 128 * 4;
  static constexpr int kBytes = kBars + 256 + 1024;
};

// [128 x 128] stationary tile through a [64 rows x 64 cols] box map: four boxes.
__device__ __forceinline__ void tma_load_tile_4(uint32_t dst, const CUtensorMap* map, uint32_t bar, int col0, int row0) {
  tma_load_2d(dst, map, bar, col0, row0);
  tma_load_2d(dst + 8192, map, bar, col0, row0 + 64);
  tma_load_2d(dst + kHalfTile, map, bar, col0 + 64, row0);
  tma_load_2d(dst + kHalfTile + 8192, map, bar, col0 + 64, row0 + 64);
}
// [64 x 128] streamed tile: two boxes.
__device__ __forceinline__ void tma_load_stream(uint32_t dst, const CUtensorMap* map, uint32_t bar, int col0, int row0) {
  tma_load_2d(dst, map, bar, col0, row0);
  tma_load_2d(dst + 8192, map, bar, col0 + 64, row0);
}

// D[128 x 64] = A[128 x 128 (K-major)] * B[64 x 128 (K-major)]^T
__device__ __forceinline__ void mma_sdp(uint32_t tmem_d, uint32_t a_base, uint32_t b_base) {
  constexpr uint32_t idesc = make_idesc_bf16(128, kBt, false, false);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint64_t ad = make_smem_desc_sw128(a_base + (k >> 2) * kHalfTile + (k & 3) * 32, 16, 1024);
    const uint64_t bd = make_smem_desc_sw128(b_base + (k >> 2) * 8192 + (k & 3) * 32, 16, 1024);
    umma_f16_ss(tmem_d, ad, bd, idesc, k > 0 ? 1u : 0u);
  }
}
// Same product with the A operand (P or dS as packed bf16 pairs) read from tensor memory: the thread that
// owns row r stored elements [32h, 32h+32) of its row as 16 packed columns at column offset 32h, so
// k-step kk (16 elements) starts at column (kk >> 1) * 32 + (kk & 1) * 8.
__device__ __forceinline__ void mma_acc_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(128, 128, false, true);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint64_t bd = make_smem_desc_sw128(b_base + k * 2048, 8192, 1024);
    umma_f16_ts(tmem_d, tmem_a + (k >> 1) * 32 + (k & 1) * 8, bd, idesc, (accumulate || k > 0) ? 1u : 0u);
  }
}
// D[128 x 128] (+)= P[128 x 64 (K-major)] * B[64 x 128 (rows along K, N contiguous)]
__device__ __forceinline__ void mma_acc(uint32_t tmem_d, uint32_t p_base, uint32_t b_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(128, 128, false, true);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint64_t ad = make_smem_desc_sw128(p_base + k * 32, 16, 1024);
    const uint64_t bd = make_smem_desc_sw128(b_base + k * 2048, 8192, 1024);
    umma_f16_ss(tmem_d, ad, bd, idesc, (accumulate || k > 0) ? 1u : 0u);
  }
}

// PT: P and dS stay in tensor memory (written over the S / dP columns their thread just read) and feed
// the accumulation MMAs from there; otherwise they go through swizzled shared tiles.
template <bool DQ, bool PT>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tma_qkv, const __grid_constant__ CUtensorMap tma_do,
                const AttnBwdArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttnBwdSmem::kBars);
  uint64_t* stat_full = bars;          // [1]
  uint64_t* b_full = bars + 1;         // [3]
  uint64_t* b_empty = bars + 4;        // [3] streamed tiles of a stage consumed by both of their MMAs
  uint64_t* sdp_full = bars + 7;       // [2]
  uint64_t* p_full = bars + 9;         // [2] count 256
  uint64_t* p_free = bars + 11;        // [2] P / dS tiles of a stage consumed
  uint64_t* acc_done = bars + 13;      // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* row_vals = reinterpret_cast<float*>(smem + AttnBwdSmem::kRow);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int H = p.nH * kHd;
  const int row_base = b * p.S;
  // DQ: stationary tile = queries [r0, r0+128), streamed = keys.  Otherwise stationary = keys.
  const int tile = DQ ? ((int)gridDim.x - 1 - (int)blockIdx.x) : (int)blockIdx.x;
  const int r0 = tile * 128;
  const int t_begin = DQ ? 0 : (r0 / kBt);
  const int t_end = DQ ? ((min(r0 + 128, p.S) + kBt - 1) / kBt) : ((p.S + kBt - 1) / kBt);
  const int T = t_end - t_begin;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 14; ++i) mbar_init(smem_u32(&bars[i]), (i == 9 || i == 10) ? 256 : 1);
    mbar_fence_init();
    tma_prefetch_desc(&tma_qkv);
    tma_prefetch_desc(&tma_do);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_acc0 = tmem_base + 256, tmem_acc1 = tmem_base + 384;
  const uint32_t sA0 = smem_u32(smem + AttnBwdSmem::kA0), sA1 = smem_u32(smem + AttnBwdSmem::kA1),
                 sB = smem_u32(smem + AttnBwdSmem::kB), sP = smem_u32(smem + AttnBwdSmem::kP);

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(smem_u32(stat_full), 2 * kTileBytes);
      if (DQ) {
        tma_load_tile_4(sA0, &tma_qkv, smem_u32(stat_full), h * kHd, row_base + r0);          // Q_i
        tma_load_tile_4(sA1, &tma_do, smem_u32(stat_full), h * kHd, row_base + r0);           // dO_i
      } else {
        tma_load_tile_4(sA0, &tma_qkv, smem_u32(stat_full), H + h * kHd, row_base + r0);      // K_j
        tma_load_tile_4(sA1, &tma_qkv, smem_u32(stat_full), 2 * H + h * kHd, row_base + r0);  // V_j
      }
      for (int i = 0; i < T; ++i) {
        const uint32_t s = i % kBwdStages, ph = (i / kBwdStages) & 1;
        if (!mbar_wait(smem_u32(&b_empty[s]), ph ^ 1, p.status, abort_flag)) break;
        mbar_arrive_expect_tx(smem_u32(&b_full[s]), 2 * kStreamBytes);
        const int row = row_base + (t_begin + i) * kBt;
        const uint32_t dst = sB + s * 2 * kStreamBytes;
        if (DQ) {
          tma_load_stream(dst, &tma_qkv, smem_u32(&b_full[s]), H + h * kHd, row);                     // K_t
          tma_load_stream(dst + kStreamBytes, &tma_qkv, smem_u32(&b_full[s]), 2 * H + h * kHd, row);  // V_t
        } else {
          tma_load_stream(dst, &tma_qkv, smem_u32(&b_full[s]), h * kHd, row);                         // Q_t
          tma_load_stream(dst + kStreamBytes, &tma_do, smem_u32(&b_full[s]), h * kHd, row);           // dO_t
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(smem_u32(stat_full), 0, p.status, abort_flag) &&
                mbar_wait(smem_u32(&b_full[0]), 0, p.status, abort_flag);
      if (ok) {
        tc_fence_after();
        mma_sdp(tmem_base, sA0, sB);
        mma_sdp(tmem_base + kBt, sA1, sB + kStreamBytes);
        umma_commit(smem_u32(&sdp_full[0]));
      }
      for (int i = 0; i < T && ok; ++i) {
        if (i + 1 < T) {
          const uint32_t b1 = (i + 1) % kBwdStages, bph1 = ((i + 1) / kBwdStages) & 1, t1 = (i + 1) & 1;
          if (!mbar_wait(smem_u32(&b_full[b1]), bph1, p.status, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_sdp(tmem_base + t1 * 128, sA0, sB + b1 * 2 * kStreamBytes);
          mma_sdp(tmem_base + t1 * 128 + kBt, sA1, sB + b1 * 2 * kStreamBytes + kStreamBytes);
          umma_commit(smem_u32(&sdp_full[t1]));
        }
        const uint32_t s = i & 1, ph = (i >> 1) & 1, bsi = i % kBwdStages;
        if (!mbar_wait(smem_u32(&p_full[s]), ph, p.status, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t bs = sB + bsi * 2 * kStreamBytes, ps = sP + s * 2 * kPBytes;
        if (PT) {
          if (!DQ) mma_acc_ts(tmem_acc0, tmem_base + s * 128, bs + kStreamBytes, i > 0);
          mma_acc_ts(tmem_acc1, tmem_base + s * 128 + kBt, bs, i > 0);
        } else {
          if (!DQ) mma_acc(tmem_acc0, ps, bs + kStreamBytes, i > 0);     // dV += P^T dO_t
          mma_acc(tmem_acc1, ps + kPBytes, bs, i > 0);                   // dK += dS^T Q_t   |   dQ += dS K_t
        }
        umma_commit(smem_u32(&b_empty[bsi]));
        umma_commit(smem_u32(&p_free[s]));
      }
      if (ok) umma_commit(smem_u32(acc_done));
    }
  } else {
    const int q = warp & 3;                      // TMEM lane quadrant this warp may access
    const int half = (warp - 2) >> 2;            // which 32 of the 64 streamed columns this thread handles
    const int r = q * 32 + lane;                 // stationary row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const int stat_idx = r0 + r;
    const long long vec_base = ((long long)b * p.nH + h) * p.S;
    // DQ: this thread's own row statistics.  Otherwise the streamed rows' statistics go through
    // shared memory: thread r of the first half fetches lse2 (r < 64) or delta (r >= 64) of streamed row (r & 63).
    float own_lse = 0.f, own_delta = 0.f;
    if (DQ && stat_idx < p.S) {
      own_lse = p.lse2[vec_base + stat_idx];
      own_delta = p.delta[vec_base + stat_idx];
    }
    auto fetch = [&](int t) -> float {
      const int idx = t * kBt + (r & 63);
      if (DQ || half != 0 || idx >= p.S) return 0.f;
      return (r < 64) ? p.lse2[vec_base + idx] : p.delta[vec_base + idx];
    };
    float next_val = fetch(t_begin);
    if (!DQ && half == 0) row_vals[r] = next_val;
    bool ok = true;
    for (int i = 0; i < T; ++i) {
      const int t = t_begin + i;
      const uint32_t s = i & 1, ph = (i >> 1) & 1;
      if (i + 1 < T) next_val = fetch(t + 1);
      mbar_wait(smem_u32(&sdp_full[s]), ph, p.status, abort_flag);
      if (!PT && i >= 2) mbar_wait(smem_u32(&p_free[s]), ph ^ 1, p.status, abort_flag);
      if (softmax_bar_or(*abort_flag != 0)) { ok = false; break; }
      tc_fence_after();
      const int c0 = t * kBt;                    // first streamed index of this tile
      // mask needed when the tile touches the diagonal or the end of the sequence
      const bool need_mask = DQ ? (c0 + kBt - 1 > r0) : (c0 < r0 + 128 || c0 + kBt > p.S);
      const float* rv = row_vals + s * 128;
      uint8_t* prow = smem + AttnBwdSmem::kP + s * 2 * kPBytes + r * 128;
      {
        const int c = half;
        uint32_t sv[32], dv[32];
        tmem_ld_32x32b_x32(tmem_base + s * 128 + lane_off + c * 32, sv);
        tmem_ld_32x32b_x32(tmem_base + s * 128 + kBt + lane_off + c * 32, dv);
        tmem_ld_wait();
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          float l4[4], d4[4];
          if (DQ) {
#pragma unroll
            for (int u = 0; u < 4; ++u) { l4[u] = own_lse; d4[u] = own_delta; }
          } else {
            const float4 a = *reinterpret_cast<const float4*>(rv + c * 32 + e);
            const float4 bq = *reinterpret_cast<const float4*>(rv + 64 + c * 32 + e);
            l4[0] = a.x; l4[1] = a.y; l4[2] = a.z; l4[3] = a.w;
            d4[0] = bq.x; d4[1] = bq.y; d4[2] = bq.z; d4[3] = bq.w;
          }
          float pv[4], dsv[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float pe = exp2f(__uint_as_float(sv[e + u]) * p.scale_log2 - l4[u]);
            float de = pe * (__uint_as_float(dv[e + u]) - d4[u]) * p.scale;
            if (need_mask) {
              const int sidx = c0 + c * 32 + e + u;
              const bool valid = DQ ? (sidx <= stat_idx) : (sidx >= stat_idx && sidx < p.S);
              if (!valid) { pe = 0.f; de = 0.f; }
            }
            pv[u] = pe; dsv[u] = de;
          }
          pp[e >> 1] = pack_bf16x2(pv[0], pv[1]);
          pp[(e >> 1) + 1] = pack_bf16x2(pv[2], pv[3]);
          dd[e >> 1] = pack_bf16x2(dsv[0], dsv[1]);
          dd[(e >> 1) + 1] = pack_bf16x2(dsv[2], dsv[3]);
        }
        if (PT) {
          // over the columns this thread just read: P at the start of its 32 S columns, dS likewise in dP
          if (!DQ) tmem_st_32x32b_x16(tmem_base + s * 128 + lane_off + c * 32, pp);
          tmem_st_32x32b_x16(tmem_base + s * 128 + kBt + lane_off + c * 32, dd);
          tmem_st_wait();
        } else {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int phys = ((c * 4 + g) ^ (r & 7)) * 16;
            if (!DQ) *reinterpret_cast<uint4*>(prow + phys) = make_uint4(pp[g * 4], pp[g * 4 + 1], pp[g * 4 + 2], pp[g * 4 + 3]);
            *reinterpret_cast<uint4*>(prow + kPBytes + phys) = make_uint4(dd[g * 4], dd[g * 4 + 1], dd[g * 4 + 2], dd[g * 4 + 3]);
          }
        }
      }
      if (!DQ && half == 0 && i + 1 < T) row_vals[(s ^ 1) * 128 + r] = next_val;
      if (!PT) fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(&p_full[s]));
    }
    if (ok) {
      mbar_wait(smem_u32(acc_done), 0, p.status, abort_flag);
      ok = !softmax_bar_or(*abort_flag != 0);
    }
    if (ok) {
      // tcgen05.ld is warp-collective: every lane takes part, only the stores depend on the row being valid
      const bool row_ok = stat_idx < p.S;
      tc_fence_after();
      __nv_bfloat16* grow = p.dqkv + (long long)(row_base + stat_idx) * p.ld_dqkv + h * kHd;
#pragma unroll
      for (int a = (DQ ? 1 : 0); a < 2; ++a) {
        // acc0 = dV (columns 2H..), acc1 = dK (columns H..) or dQ (columns 0..); each half stores 64 columns
        __nv_bfloat16* dst = grow + (DQ ? 0 : (a == 0 ? 2 * H : H)) + half * 64;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t t4[32];
          tmem_ld_32x32b_x32((a == 0 ? tmem_acc0 : tmem_acc1) + lane_off + half * 64 + c * 32, t4);
          tmem_ld_wait();
          if (!row_ok) continue;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(t4[g * 8 + 0]), __uint_as_float(t4[g * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(t4[g * 8 + 2]), __uint_as_float(t4[g * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(t4[g * 8 + 4]), __uint_as_float(t4[g * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(t4[g * 8 + 6]), __uint_as_float(t4[g * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = o;
          }
        }
      }
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

// lse2 = lse * log2(e); delta = rowsum(dO * O).  One warp per (row, head).
__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ dout, long long ld_do,
                                     const __nv_bfloat16* __restrict__ out, long long ld_o,
                                     const float* __restrict__ lse, float* __restrict__ lse2,
                                     float* __restrict__ delta, int B, int S, int nH) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * nH;
  if (w >= total) return;
  const int hh = (int)(w % nH);
  const long long row = w / nH;
  const int bb = (int)(row / S), ss = (int)(row % S);
  const uint2 a = *reinterpret_cast<const uint2*>(dout + row * ld_do + hh * kHd + lane * 4);
  const uint2 o = *reinterpret_cast<const uint2*>(out + row * ld_o + hh * kHd + lane * 4);
  const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), o0 = unpack_bf16x2(o.x), o1 = unpack_bf16x2(o.y);
  float acc = a0.x * o0.x + a0.y * o0.y + a1.x * o1.x + a1.y * o1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const long long idx = ((long long)bb * nH + hh) * S + ss;
    delta[idx] = acc;
    lse2[idx] = lse[idx] * kLog2e;
  }
}
}  // namespace mfsdp

using namespace mfsdp;

// qkv: [B*S, 3*nH*128] bf16 (row stride ld_qkv elements); out: [B*S, nH*128]; lse: [B, nH, S] fp32.
MFSDP_API int mfsdp_attention_fwd(const void* qkv, void* out, float* lse, int B, int S, int nH, long long ld_qkv,
                                  long long ld_out, float softmax_scale, int* status, cudaStream_t st) {
  if (B <= 0 || S <= 0 || nH <= 0 || (ld_qkv % 8) || (ld_out % 8)) return -2;
  ensure_context_on_this_thread();
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

// dout, out: [B*S, nH*128] bf16; lse: [B, nH, S]; dqkv: [B*S, 3*nH*128] bf16 (written in full);
// scratch: 2 * B * nH * S floats.
MFSDP_API int mfsdp_attention_bwd(const void* dout, const void* qkv, const void* out, const float* lse, void* dqkv,
                                  float* scratch, int B, int S, int nH, long long ld_qkv, long long ld_o,
                                  long long ld_dqkv, float softmax_scale, int* status, cudaStream_t st) {
  if (B <= 0 || S <= 0 || nH <= 0 || (ld_qkv % 8) || (ld_o % 8) || (ld_dqkv % 8) || !scratch) return -2;
  ensure_context_on_this_thread();
  CUtensorMap map_qkv, map_do;
  int rc = make_tmap_bf16_2d(&map_qkv, qkv, (long long)B * S, 3LL * nH * kHd, ld_qkv, kBt, 64);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&map_do, dout, (long long)B * S, (long long)nH * kHd, ld_o, kBt, 64);
  if (rc) return rc;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaSuccess;
    const void* kerns[4] = {(const void*)attn_bwd_kernel<false, false>, (const void*)attn_bwd_kernel<true, false>,
                            (const void*)attn_bwd_kernel<false, true>, (const void*)attn_bwd_kernel<true, true>};
    for (int i = 0; i < 4 && e == cudaSuccess; ++i)
      e = cudaFuncSetAttribute(kerns[i], cudaFuncAttributeMaxDynamicSharedMemorySize, AttnBwdSmem::kBytes);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  const long long n = (long long)B * nH * S;
  float* lse2 = scratch;
  float* delta = scratch + n;
  attn_bwd_prep_kernel<<<(unsigned)((n + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)dout, ld_o, (const __nv_bfloat16*)out,
                                                                ld_o, lse, lse2, delta, B, S, nH);
  AttnBwdArgs a{};
  a.B = B; a.S = S; a.nH = nH;
  a.scale = softmax_scale; a.scale_log2 = softmax_scale * kLog2e;
  a.lse2 = lse2; a.delta = delta;
  a.dqkv = (__nv_bfloat16*)dqkv; a.ld_dqkv = ld_dqkv; a.status = status;
  dim3 grid((S + 127) / 128, nH, B);
  static const bool p_in_tmem = [] {
    const char* e = getenv("MFSDP_ATTN_P_TMEM");
    return e ? atoi(e) != 0 : true;
  }();
  if (p_in_tmem) {
    attn_bwd_kernel<false, true><<<grid, kAttnThreads, AttnBwdSmem::kBytes, st>>>(map_qkv, map_do, a);
    attn_bwd_kernel<true, true><<<grid, kAttnThreads, AttnBwdSmem::kBytes, st>>>(map_qkv, map_do, a);
  } else {
    attn_bwd_kernel<false, false><<<grid, kAttnThreads, AttnBwdSmem::kBytes, st>>>(map_qkv, map_do, a);
    attn_bwd_kernel<true, false><<<grid, kAttnThreads, AttnBwdSmem::kBytes, st>>>(map_qkv, map_do, a);
  }
  return (int)cudaGetLastError();
}
