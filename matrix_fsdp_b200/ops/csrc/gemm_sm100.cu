// Persistent, warp-specialised bf16 GEMM for sm_100a built on tcgen05.mma with TMEM
// accumulators and TMA-fed shared-memory operand rings.
//
//   D[M,N] = alpha * (A · B^T) + beta * Cin        (bf16 in, fp32 accumulate, bf16 out)
//
// Either operand may be K-major ([rows, K], the nn.Linear forward form) or MN-major
// ([K, rows], which is what dgrad and wgrad see), so forward, dgrad and wgrad all run
// on the same kernel without a transpose pass.  Two grouped forms serve the MoE
// experts: "M-grouped" (each 128-row tile of A multiplies its own expert's B) and
// "K-grouped" (each expert's output is reduced over its own token range).
//
// CTA layout (192 threads, one CTA per SM):
//   warp 0   : TMA producer (one lane)        -> full[stage]
//   warp 1   : tcgen05.mma issuer (one lane)  -> empty[stage], tmem_full[acc]; owns TMEM alloc
//   warps 2-5: epilogue: tcgen05.ld -> scale/add -> swizzled smem staging -> TMA store
// Two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1.
//
// CTA-pair form (TWO_SM): clusters of two CTAs compute 256 x 256 tiles with tcgen05.mma.cta_group::2.
// Each CTA loads its 128 rows of A and its 128 of the 256 rows of B (half the B traffic per SM of the
// single-CTA form), the leader CTA's lane issues the MMAs for both, commits are multicast to both CTAs'
// barriers, and each CTA's epilogue drains its own 128 accumulator rows.
//
// The role the reference gives to cuBLAS through torch.nn.functional.linear
// (test/fsdp/bench_fsdp2_compare.py:456-483 builds its blocks from nn.Linear) is what
// this kernel takes over.
#include "common.cuh"
#include <cuda.h>
#include <cstdio>
#include <mutex>

namespace mfsdp {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kChunkBytes = 8192;      // one 64-wide MN chunk x 64 k-rows of bf16
constexpr int kEpiBufBytes = BM * 128; // 128 rows x 64 bf16

struct GemmArgs {
  int M, N, K;
  int tiles_m, tiles_n;
  float alpha, beta;
  const __nv_bfloat16* cin;
  long long ldcin;
  int* status;
  int group_mode;            // 0 dense, 1 M-grouped, 2 K-grouped
  const int* tile_group;     // mode 1: group id per M tile (-1 = tile has no rows)
  const int* group_offsets;  // mode 2: [G+1] offsets along the reduce dimension
  int b_group_stride;        // mode 1: rows added to B's row coordinate per group
  int tiles_m_per_group;     // mode 2
  int m_per_group;           // mode 2
  int raster_group_m;        // M-tiles per rasterisation group
  int total_tiles;           // work items walked by the persistent CTAs
  int tile_m;                // rows of one work item: 128, or 256 for CTA pairs
  // Symmetric output (sym_rows > 0): every output matrix is sym_rows*128 square and equal to its own
  // transpose (X Xᵀ, polynomials of it), so only tiles that reach the diagonal or lie above it are
  // computed; the caller mirrors the rest.  Work items enumerate exactly those tiles, row by row.
  int sym_rows;              // tile rows (of tile_m rows) per symmetric matrix (0 = off)
  int sym_q;                 // tile width / tile_m (1 or 2)
  int sym_tiles_per_matrix;
  // Fused all-gather (GATHER kernels only): B's rows are still on peer GPUs when the kernel starts.
  // Eight extra warps per CTA copy them into B's local buffer job by job (16-byte peer loads, local
  // stores) and count finished jobs per B tile row-block; the TMA producer waits (bounded) until
  // the row-block of its tile is complete before loading it.
  const unsigned long long* ag_src;   // [njobs] peer (or local) source address
  const unsigned long long* ag_dst;   // [njobs] destination address inside B's local buffer
  const int* ag_bytes;                // [njobs] multiple of 16
  const int* ag_flag;                 // [njobs] B row-block (tile column) the job belongs to
  int ag_njobs;
  unsigned* ag_flags;                 // [2 * tiles_n] zero at launch: finished jobs per row-block, then claimed jobs
  const int* ag_need;                 // [tiles_n] jobs per row-block
  const int* ag_first;                // [tiles_n] index of the first job of each row-block (jobs are sorted by block)
  int ag_rotate;                      // tile columns are walked starting here (the local rank's rows come first)
  unsigned long long ag_budget_ns;
};

constexpr int kGatherThreads = 256;

template <int BN, bool TWO_SM = false>
struct GemmCfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBRows = TWO_SM ? BN / 2 : BN;          // rows of B this CTA stages
  static constexpr int kBBytes = kBRows * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (kBRows == 256) ? 4 : 6;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 2 * kEpiBufBytes + 1024 + 256;
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier of the four epilogue warps that also ORs a flag, so that all of them take the same way out.
__device__ __forceinline__ bool epi_bar_any(int flag) {
  uint32_t any;
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, 1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
               : "=r"(any) : "r"(flag) : "memory");
  return any != 0;
}

struct TileCoord {
  int m0, n0;        // element offsets into the (per-group) output
  int out_row0;      // row of D this tile starts at
  int a_row_k0;      // first reduce index
  int nkb;           // number of 64-wide reduce blocks
  int b_row_off;     // mode 1: offset added to B's row coordinate
  bool skip;
};

// Tiles of tile-row i of a symmetric matrix that lie entirely below the diagonal: floor(i / q); the
// number of kept tiles in rows [0, i) is therefore i * tiles_n - S(i), S(i) = sum_{j<i} floor(j / q).
__host__ __device__ __forceinline__ int sym_kept_before(int i, int tiles_n, int q) {
  const int m = i / q;
  return i * tiles_n - (q * (m * (m - 1) / 2) + (i - m * q) * m);
}

__device__ __forceinline__ TileCoord decode_tile(const GemmArgs& p, int tile) {
  int tm, tn;
  if (p.sym_rows > 0) {
    const int mat = tile / p.sym_tiles_per_matrix;
    const int rem = tile - mat * p.sym_tiles_per_matrix;
    int lo = 0, hi = p.sym_rows - 1;      // last row i with sym_kept_before(i) <= rem
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (sym_kept_before(mid, p.tiles_n, p.sym_q) <= rem) lo = mid; else hi = mid - 1;
    }
    tm = mat * p.sym_rows + lo;
    tn = lo / p.sym_q + (rem - sym_kept_before(lo, p.tiles_n, p.sym_q));
  } else {
    // Grouped rasterisation: 8 M-tiles share each sweep over N so that the CTAs running
    // at the same time reuse A and B tiles out of L2.
    const int kGroupM = p.raster_group_m;
    const int per_group = kGroupM * p.tiles_n;
    const int gid = tile / per_group;
    const int first_m = gid * kGroupM;
    const int gsz = min(p.tiles_m - first_m, kGroupM);
    tm = first_m + (tile % per_group) % gsz;
    tn = (tile % per_group) / gsz;
    if (p.ag_rotate) tn = (tn + p.ag_rotate) % p.tiles_n;
  }
  TileCoord c;
  c.skip = false;
  c.n0 = tn;  // scaled by the caller's BN
  c.b_row_off = 0;
  c.a_row_k0 = 0;
  c.nkb = (p.K + BK - 1) / BK;
  if (p.group_mode == 0) {
    c.m0 = tm * p.tile_m;
    c.out_row0 = c.m0;
  } else if (p.group_mode == 1) {
    c.m0 = tm * p.tile_m;
    c.out_row0 = c.m0;
    const int g = p.tile_group[c.m0 / BM];     // groups are named per 128-row tile
    if (g < 0) c.skip = true;
    c.b_row_off = (g < 0 ? 0 : g) * p.b_group_stride;
  } else {
    const int g = tm / p.tiles_m_per_group;
    c.m0 = (tm % p.tiles_m_per_group) * p.tile_m;
    c.out_row0 = g * p.m_per_group + c.m0;
    const int k_lo = p.group_offsets[g], k_hi = p.group_offsets[g + 1];
    c.a_row_k0 = k_lo;
    c.nkb = (k_hi - k_lo + BK - 1) / BK;
  }
  return c;
}

template <int BN, bool A_MN, bool B_MN, bool GATHER = false, bool TWO_SM = false>
__global__ void __launch_bounds__(GATHER ? kGemmThreads + kGatherThreads : kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a,
                         const __grid_constant__ CUtensorMap tma_b,
                         const __grid_constant__ CUtensorMap tma_d, const GemmArgs p) {
  static_assert(!(TWO_SM && GATHER) && (!TWO_SM || BN == 256), "CTA pairs: dense 256 x 256 tiles only");
  using Cfg = GemmCfg<BN, TWO_SM>;
  // CTA pairs: `worker` indexes the pair, `cta_rank` the CTA inside it (0 = leader, issues the MMAs)
  const uint32_t cta_rank = TWO_SM ? cluster_ctarank() : 0u;
  const int worker = TWO_SM ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int nworkers = TWO_SM ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int pair_row = TWO_SM ? (int)cta_rank * BM : 0;              // this CTA's rows inside the 256-row tile
  const int pair_col = TWO_SM ? (int)cta_rank * (BN / 2) : 0;        // this CTA's rows of B inside the 256
  constexpr uint32_t kStageTx = TWO_SM ? 2u * Cfg::kStageBytes : (uint32_t)Cfg::kStageBytes;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_base = smem + kStages * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_base + 2 * kEpiBufBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tfull_bar = bars + 2 * kStages;
  uint64_t* tempty_bar = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tfull_bar[b]), 1);
      mbar_init(smem_u32(&tempty_bar[b]), TWO_SM ? 2 : kEpiThreads);   // pairs: one arrival per CTA's epilogue
    }
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    tma_prefetch_desc(&tma_d);
  }
  if (warp == 1) {
    if (TWO_SM) {
      tmem_alloc_pair(smem_u32(tmem_slot), Cfg::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if (TWO_SM) cluster_sync_all();      // the peer's barriers must be initialised before anything signals them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.total_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = worker; tile < total_tiles && ok; tile += nworkers) {
        TileCoord c = decode_tile(p, tile);
        if (c.skip) continue;
        const int n0 = c.n0 * BN;
        if (GATHER) {
          // rows [n0, n0 + BN) of B must have landed in local memory (written by gather warps of
          // any CTA through the generic proxy) before the async proxy reads them
          const unsigned need = (unsigned)p.ag_need[c.n0];
          const unsigned* flag = p.ag_flags + c.n0;
          const uint64_t t0 = globaltimer_ns();
          uint32_t spins = 0;
          while (ld_acquire_gpu_u32(flag) < need) {
            if ((++spins & 0xff) == 0) {
              if (*abort_flag || globaltimer_ns() - t0 > p.ag_budget_ns) {
                *abort_flag = 1;
                if (p.status) atomicCAS(p.status, 0, (int)kErrPeerFlagTimeout);
                ok = false;
                break;
              }
            }
          }
          if (!ok) break;
          fence_proxy_async_all();
        }
        for (int kb = 0; kb < c.nkb; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, p.status, abort_flag)) { ok = false; break; }
          const uint32_t fb = smem_u32(&full_bar[s]);
          // pairs: the leader's barrier counts the bytes of both CTAs; only the leader arms it
          if (!TWO_SM || cta_rank == 0) mbar_arrive_expect_tx(fb, kStageTx);
          const uint32_t a_dst = smem_u32(smem + s * Cfg::kStageBytes);
          const uint32_t b_dst = a_dst + Cfg::kABytes;
          const int k0 = c.a_row_k0 + kb * BK;
          const int am0 = c.m0 + pair_row, bn0 = n0 + pair_col;
          auto load = [&](uint32_t dst, const CUtensorMap* map, int c0, int c1) {
            if (TWO_SM) tma_load_2d_pair(dst, map, fb, c0, c1);
            else tma_load_2d(dst, map, fb, c0, c1);
          };
          if (!A_MN) {
            load(a_dst, &tma_a, k0, am0);
          } else {
            load(a_dst, &tma_a, am0, k0);
            load(a_dst + kChunkBytes, &tma_a, am0 + 64, k0);
          }
          if (!B_MN) {
            load(b_dst, &tma_b, k0, bn0 + c.b_row_off);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::kBRows / 64; ++j)
              load(b_dst + j * kChunkBytes, &tma_b, bn0 + 64 * j, k0 + c.b_row_off);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TWO_SM ? 2 * BM : BM, BN, A_MN, B_MN);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int tile = worker; tile < total_tiles && ok; tile += nworkers) {
        TileCoord c = decode_tile(p, tile);
        if (c.skip) continue;
        const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), aph ^ 1, p.status, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < c.nkb; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, p.status, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + s * Cfg::kStageBytes);
          const uint32_t b_base = a_base + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(a_base + k * 2048, kChunkBytes, 1024)
                                        : make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(b_base + k * 2048, kChunkBytes, 1024)
                                        : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            if (TWO_SM) umma_f16_ss_pair(tmem_d, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else umma_f16_ss(tmem_d, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          if (TWO_SM) umma_commit_pair(smem_u32(&empty_bar[s]));
          else umma_commit(smem_u32(&empty_bar[s]));
        }
        if (!ok) break;
        if (TWO_SM) umma_commit_pair(smem_u32(&tfull_bar[acc]));
        else umma_commit(smem_u32(&tfull_bar[acc]));
        ++lt;
      }
    }
  } else if (GATHER && warp >= 6) {
    // ------------------------------------------------------------ gather warps
    // Jobs are claimed, not assigned: a CTA first claims the jobs of the row-blocks its own tiles read (in
    // the order it will read them), then whatever is left.  Every job is therefore executed by a CTA that
    // is running, and a producer that waits for a row-block only ever waits for CTAs that are resident:
    // the kernel makes progress with any number of co-resident CTAs, also when other streams hold SMs.
    const int gt = threadIdx.x - kGemmThreads;
    __shared__ int claimed_job;
    unsigned* claims = p.ag_flags + p.tiles_n;
    auto drain_block = [&](int b) {
      const int need = p.ag_need[b];
      while (true) {
        if (gt == 0) claimed_job = (int)atomicAdd(claims + b, 1u);
        asm volatile("bar.sync 3, 256;" ::: "memory");
        const int k = claimed_job;
        asm volatile("bar.sync 3, 256;" ::: "memory");
        if (k >= need) break;
        const int j = p.ag_first[b] + k;
        const uint4* src = reinterpret_cast<const uint4*>(p.ag_src[j]);
        uint4* dst = reinterpret_cast<uint4*>(p.ag_dst[j]);
        const int nvec = p.ag_bytes[j] >> 4;
        int i = gt;
        // 8 independent 16-byte peer loads in flight per thread to cover the NVLink latency
        for (; i + 7 * kGatherThreads < nvec; i += 8 * kGatherThreads) {
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = src[i + u * kGatherThreads];
#pragma unroll
          for (int u = 0; u < 8; ++u) dst[i + u * kGatherThreads] = v[u];
        }
        for (; i < nvec; i += kGatherThreads) dst[i] = src[i];
        __threadfence();
        asm volatile("bar.sync 3, 256;" ::: "memory");
        if (gt == 0) red_release_gpu_add_u32(p.ag_flags + b, 1u);
      }
    };
    for (int tile = worker; tile < total_tiles; tile += nworkers) {
      const TileCoord c = decode_tile(p, tile);
      if (!c.skip) drain_block(c.n0);
    }
    for (int b = 0; b < p.tiles_n; ++b) drain_block((b + p.ag_rotate) % p.tiles_n);
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;                // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    uint32_t lt = 0, store_cnt = 0;
    for (int tile = worker; tile < total_tiles; tile += nworkers) {
      TileCoord c = decode_tile(p, tile);
      if (c.skip) continue;
      const int n0 = c.n0 * BN;
      const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
      mbar_wait(smem_u32(&tfull_bar[acc]), aph, p.status, abort_flag);
      if (epi_bar_any(*abort_flag)) break;     // a uniform decision: nobody is left behind at a later barrier
      tc_fence_after();
      const long long grow = (long long)c.out_row0 + pair_row + row_in_tile;
      const bool row_ok = (p.group_mode == 2) ? (c.m0 + pair_row + row_in_tile < p.m_per_group)
                                              : (c.m0 + pair_row + row_in_tile < p.M);
#pragma unroll 1
      for (int ch = 0; ch < BN / 64; ++ch) {
        const int ncol0 = n0 + ch * 64;
        if (ncol0 >= p.N) break;
        const uint32_t buf = store_cnt & 1;
        uint8_t* ebuf = epi_base + buf * kEpiBufBytes;
        if (epi_tid == 0) tma_store_wait_read<1>();
        epi_bar_sync();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          if (c.nkb > 0) {
            tmem_ld_32x32b_x32(tmem_base + acc * BN + ((uint32_t)(q * 32) << 16) + ch * 64 + h * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = p.alpha * __uint_as_float(r[j]);
          if (p.cin != nullptr && p.beta != 0.f && row_ok) {
            const __nv_bfloat16* crow = p.cin + grow * p.ldcin + ncol0 + h * 32;
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              const int col = ncol0 + h * 32 + g8 * 8;
              if (col + 8 <= p.N && ((reinterpret_cast<uintptr_t>(crow + g8 * 8) & 15) == 0)) {
                const uint4 u = *reinterpret_cast<const uint4*>(crow + g8 * 8);
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 f = unpack_bf16x2(w[e]);
                  v[g8 * 8 + 2 * e] += p.beta * f.x;
                  v[g8 * 8 + 2 * e + 1] += p.beta * f.y;
                }
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  if (col + e < p.N) v[g8 * 8 + e] += p.beta * __bfloat162float(crow[g8 * 8 + e]);
              }
            }
          }
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            uint4 o;
            o.x = pack_bf16x2(v[g8 * 8 + 0], v[g8 * 8 + 1]);
            o.y = pack_bf16x2(v[g8 * 8 + 2], v[g8 * 8 + 3]);
            o.z = pack_bf16x2(v[g8 * 8 + 4], v[g8 * 8 + 5]);
            o.w = pack_bf16x2(v[g8 * 8 + 6], v[g8 * 8 + 7]);
            const int chunk = h * 4 + g8;
            const int phys = chunk ^ (row_in_tile & 7);
            *reinterpret_cast<uint4*>(ebuf + row_in_tile * 128 + phys * 16) = o;
          }
        }
        fence_proxy_async_smem();
        epi_bar_sync();
        // (a pair's second CTA may own no rows at all at the bottom edge: nothing to store then)
        if (epi_tid == 0 && (!TWO_SM || c.m0 + pair_row < p.M)) {
          tma_store_2d(&tma_d, smem_u32(ebuf), ncol0, c.out_row0 + pair_row);
          tma_store_commit();
        }
        ++store_cnt;
      }
      tc_fence_before();
      if (TWO_SM) {
        epi_bar_sync();                  // all four warps of this CTA have read their accumulator rows
        if (epi_tid == 0) mbar_arrive_leader(smem_u32(&tempty_bar[acc]));
      } else {
        mbar_arrive(smem_u32(&tempty_bar[acc]));
      }
      ++lt;
    }
    if (epi_tid == 0) tma_store_wait_all<0>();
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) __nanosleep(1000000);  // let TMA copies in flight land before the CTA exits
  tc_fence_before();
  if (TWO_SM) cluster_sync_all();      // neither CTA frees tensor memory while the pair's MMAs may touch it
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (TWO_SM) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    else tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// Encoding a tensor map is a driver call; a training step asks for the same few hundred
// (base, shape, stride, box) combinations over and over (persistent parameter, gradient and
// activation buffers), so encoded maps are kept in a small per-process table.
struct TmapKey {
  const void* base;
  long long rows, cols, ld;
  int box_rows, box_cols;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           box_cols == o.box_cols;
  }
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kTmapSlots = 4096;   // direct-mapped; a collision simply re-encodes
static TmapSlot g_tmap_cache[kTmapSlots];
static std::mutex g_tmap_mutex;

static inline size_t tmap_hash(const TmapKey& k) {
  size_t h = reinterpret_cast<size_t>(k.base) >> 4;
  h ^= (size_t)k.rows * 0x9E3779B97F4A7C15ull;
  h ^= ((size_t)k.cols << 21) ^ ((size_t)k.ld << 7) ^ ((size_t)k.box_rows << 3) ^ (size_t)k.box_cols;
  h ^= h >> 29;
  return h % kTmapSlots;
}

// The driver needs a current context on the calling thread before it can encode a map; a thread that
// has not made a runtime call yet (an autograd worker) has none until a runtime call binds it.
void ensure_context_on_this_thread() {
  thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

// rows x cols row-major bf16 tensor (row stride `ld` elements); box = box_rows x box_cols.
int make_tmap_bf16_2d(CUtensorMap* map, const void* base, long long rows, long long cols,
                      long long ld, int box_rows, int box_cols) {
  const TmapKey key{base, rows, cols, ld, box_rows, box_cols};
  TmapSlot& slot = g_tmap_cache[tmap_hash(key)];
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    if (slot.used && slot.key == key) {
      *map = slot.map;
      return 0;
    }
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  ensure_context_on_this_thread();
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return (int)r;
  std::lock_guard<std::mutex> lock(g_tmap_mutex);
  slot.key = key;
  slot.map = *map;
  slot.used = true;
  return 0;
}

template <int BN, bool A_MN, bool B_MN, bool GATHER = false>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                       const GemmArgs& args, int grid, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static bool attr_set = false;
  auto kern = gemm_bf16_tcgen05_kernel<BN, A_MN, B_MN, GATHER>;
  if (!attr_set) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  kern<<<grid, GATHER ? kGemmThreads + kGatherThreads : kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, td, args);
  return (int)cudaGetLastError();
}

// CTA-pair kernels are launched as clusters of two; the persistent grid is as many pairs as can be
// resident at once (a GPC with an odd number of free SMs leaves one without a partner).
template <bool A_MN, bool B_MN>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                            const GemmArgs& args, int num_sms, cudaStream_t stream) {
  using Cfg = GemmCfg<256, true>;
  auto kern = gemm_bf16_tcgen05_kernel<256, A_MN, B_MN, false, true>;
  static int max_pairs = -1;
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_pairs < 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    cfg.gridDim = dim3((unsigned)(num_sms & ~1));
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess) return (int)e;
    if (n <= 0) return -3;
    max_pairs = n;
  }
  int pairs = args.total_tiles < max_pairs ? args.total_tiles : max_pairs;
  if (pairs > num_sms / 2) pairs = num_sms / 2;
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  return (int)cudaLaunchKernelEx(&cfg, kern, ta, tb, td, args);
}

// MFSDP_GEMM_2SM = 1 (default): CTA pairs whenever the problem is eligible (measured 3-14 % faster than the
// single-CTA kernel on every dense shape of the models), 0: only on request, 2: only when the pair schedule
// fills its waves at least as well as the single-CTA one.
static int pair_mode() {
  static int v = [] {
    const char* e = getenv("MFSDP_GEMM_2SM");
    return e ? atoi(e) : 1;
  }();
  return v;
}

static int pairs_resident(int num_sms) {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("MFSDP_GEMM_2SM_PAIRS");   // assumed resident pairs for the schedule estimate
    v = e ? atoi(e) : num_sms / 2;
  }
  return v;
}

}  // namespace mfsdp

using namespace mfsdp;

// Returns 0 on success, a CUDA / driver error code otherwise, or -2 for a bad argument.
// Layout contract (all bf16, strides in elements, 16-byte aligned bases and row pitches):
//   a_mn_major = 0: A is [M, K];   1: A is [K, M]
//   b_mn_major = 0: B is [N, K];   1: B is [K, N]
//   D, Cin are [M, N].
// group_mode 1 (M-grouped): A/D rows are grouped in 128-row tiles, tile_group[t] names the
//   group of M-tile t; B holds num_groups matrices stacked along its row dimension.
// group_mode 2 (K-grouped): both operands are MN-major and stacked along the reduce
//   dimension; group g reduces rows [group_offsets[g], group_offsets[g+1]) and writes
//   D rows [g*M, (g+1)*M).  M must be a multiple of 128 and offsets multiples of 64.
static int gemm_bf16_impl(const void* A, const void* B, void* D, const void* Cin, int M, int N,
                          int K, long long lda, long long ldb, long long ldd, long long ldcin,
                          int a_mn_major, int b_mn_major, float alpha, float beta,
                          int group_mode, const int* tile_group, const int* group_offsets,
                          int num_groups, long long k_total, int* status, int num_sms,
                          int force_bn, int symmetric, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K < 0) return -2;
  // symmetric outputs: square matrices of N rows (stacked along M in the grouped modes), whole tiles
  if (symmetric && ((N % BM) != 0 || (group_mode == 1 ? (M % N) != 0 : M != N))) return -2;
  ensure_context_on_this_thread();
  if ((lda % 8) || (ldb % 8) || (ldd % 8)) return -2;
  if (((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)D & 15)) return -2;
  if (group_mode == 2 && (!a_mn_major || !b_mn_major || (M % BM) != 0)) return -2;
  if (group_mode != 0 && num_groups <= 0) return -2;

  GemmArgs args{};
  args.M = M; args.N = N; args.K = K;
  args.alpha = alpha; args.beta = beta;
  args.cin = reinterpret_cast<const __nv_bfloat16*>(Cin);
  args.ldcin = ldcin;
  args.status = status;
  args.group_mode = group_mode;
  args.raster_group_m = 8;
  args.tile_m = BM;
  args.tile_group = tile_group;
  args.group_offsets = group_offsets;
  args.m_per_group = M;
  args.tiles_m_per_group = (M + BM - 1) / BM;

  const int tiles_m_base = (M + BM - 1) / BM;
  args.tiles_m = (group_mode == 2) ? tiles_m_base * num_groups : tiles_m_base;

  // Tile width: 256 keeps the tensor pipe fed per shared-memory byte; 128 wins when it
  // fills the last wave better.
  int bn = 256;
  if (force_bn == 128 || force_bn == 256) {
    bn = force_bn;
  } else if (N <= 128) {
    bn = 128;
  } else {
    auto eff = [&](int b) {
      long long t = (long long)args.tiles_m * ((N + b - 1) / b);
      if (symmetric) t = (long long)(args.tiles_m / (N / BM)) * sym_kept_before(N / BM, (N + b - 1) / b, b / BM);
      const long long waves = (t + num_sms - 1) / num_sms;
      const double padded_n = (double)((N + b - 1) / b) * b;
      return ((double)t / (double)(waves * num_sms)) * ((double)N / padded_n) *
             (b == 256 ? 1.0 : 0.72);
    };
    bn = eff(256) >= eff(128) ? 256 : 128;
  }
  // CTA pairs (256 x 256 tiles over two SMs).  force_bn == 2 asks for them whatever the environment says, and
  // in the M-grouped mode it is also the caller's promise that every group has a multiple of 256 rows (a pair's
  // two CTAs share one B operand, so a tile must not straddle two groups).
  bool pair = false;
  const bool pair_req = force_bn == 2;
  const bool pair_auto = force_bn == 0 && pair_mode() != 0;
  if (pair_req || pair_auto) {
    const bool sym_ok = !symmetric || (N % 256) == 0;
    if (group_mode == 0) {
      if (pair_req || symmetric) {
        pair = sym_ok && K > 0;
      } else if (M > BM && N > 128 && K > 0) {
        const int np = pairs_resident(num_sms);
        const long long t2 = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
        const double fill2 = (double)t2 / (double)(((t2 + np - 1) / np) * np) *
                             ((double)M / (double)(((M + 255) / 256) * 256)) * ((double)N / (double)(((N + 255) / 256) * 256));
        const long long t1 = (long long)args.tiles_m * ((N + bn - 1) / bn);
        const double fill1 = (double)t1 / (double)(((t1 + num_sms - 1) / num_sms) * num_sms) *
                             ((double)N / (double)(((N + bn - 1) / bn) * bn)) * (bn == 256 ? 1.0 : 0.72);
        pair = pair_mode() == 1 || fill2 * 1.05 >= fill1;
      }
    } else if (group_mode == 1) {
      pair = pair_req && (M % 256) == 0 && sym_ok && K > 0;
    } else {
      pair = (M % 256) == 0 && sym_ok;          // K-grouped: whole 256-row tiles per group
    }
  }
  if (pair) {
    bn = 256;
    args.tile_m = 2 * BM;
    const int tiles_m_pair = (M + 2 * BM - 1) / (2 * BM);
    args.tiles_m_per_group = tiles_m_pair;
    args.tiles_m = (group_mode == 2) ? tiles_m_pair * num_groups : tiles_m_pair;
  }
  args.tiles_n = (N + bn - 1) / bn;
  args.b_group_stride = (group_mode == 1) ? (b_mn_major ? K : N) : 0;

  // Tensor maps.
  CUtensorMap ta, tb, td;
  int rc;
  const long long red = (group_mode == 2) ? k_total : K;
  if (!a_mn_major) rc = make_tmap_bf16_2d(&ta, A, M, red, lda, BM, 64);
  else             rc = make_tmap_bf16_2d(&ta, A, red, M, lda, BK, 64);
  if (rc) return rc;
  const long long b_groups = (group_mode == 1) ? num_groups : 1;
  if (!b_mn_major) rc = make_tmap_bf16_2d(&tb, B, (long long)N * b_groups, red, ldb, pair ? 128 : bn, 64);
  else             rc = make_tmap_bf16_2d(&tb, B, red * b_groups, N, ldb, BK, 64);
  if (rc) return rc;
  const long long d_rows = (group_mode == 2) ? (long long)M * num_groups : M;
  rc = make_tmap_bf16_2d(&td, D, d_rows, N, ldd, BM, 64);
  if (rc) return rc;

  int total = args.tiles_m * args.tiles_n;
  if (symmetric) {
    args.sym_rows = N / args.tile_m;
    args.sym_q = bn / args.tile_m;
    args.sym_tiles_per_matrix = sym_kept_before(args.sym_rows, args.tiles_n, args.sym_q);
    total = (args.tiles_m / args.sym_rows) * args.sym_tiles_per_matrix;
  }
  args.total_tiles = total;
  if (pair) {
    return a_mn_major ? (b_mn_major ? launch_gemm_pair<true, true>(ta, tb, td, args, num_sms, stream)
                                    : launch_gemm_pair<true, false>(ta, tb, td, args, num_sms, stream))
                      : (b_mn_major ? launch_gemm_pair<false, true>(ta, tb, td, args, num_sms, stream)
                                    : launch_gemm_pair<false, false>(ta, tb, td, args, num_sms, stream));
  }
  const int grid = total < num_sms ? total : num_sms;
#define MFSDP_LAUNCH(BN_)                                                                   \
  (a_mn_major ? (b_mn_major ? launch_gemm<BN_, true, true>(ta, tb, td, args, grid, stream)  \
                            : launch_gemm<BN_, true, false>(ta, tb, td, args, grid, stream)) \
              : (b_mn_major ? launch_gemm<BN_, false, true>(ta, tb, td, args, grid, stream) \
                            : launch_gemm<BN_, false, false>(ta, tb, td, args, grid, stream)))
  return bn == 256 ? MFSDP_LAUNCH(256) : MFSDP_LAUNCH(128);
#undef MFSDP_LAUNCH
}

MFSDP_API int mfsdp_gemm_bf16(const void* A, const void* B, void* D, const void* Cin, int M, int N,
                              int K, long long lda, long long ldb, long long ldd, long long ldcin,
                              int a_mn_major, int b_mn_major, float alpha, float beta,
                              int group_mode, const int* tile_group, const int* group_offsets,
                              int num_groups, long long k_total, int* status, int num_sms,
                              int force_bn, cudaStream_t stream) {
  return gemm_bf16_impl(A, B, D, Cin, M, N, K, lda, ldb, ldd, ldcin, a_mn_major, b_mn_major, alpha, beta, group_mode,
                        tile_group, group_offsets, num_groups, k_total, status, num_sms, force_bn, 0, stream);
}

// Same product for outputs known to be symmetric (every output matrix is N x N with N a multiple of 128:
// M == N, or M a multiple of N in the M-grouped mode).  Only the tiles on or above the diagonal are
// computed and written; entries below the diagonal that fall outside those tiles are left untouched, so
// the caller follows with mfsdp_mirror_upper.
MFSDP_API int mfsdp_gemm_bf16_sym(const void* A, const void* B, void* D, const void* Cin, int M, int N,
                                  int K, long long lda, long long ldb, long long ldd, long long ldcin,
                                  int a_mn_major, int b_mn_major, float alpha, float beta,
                                  int group_mode, const int* tile_group, const int* group_offsets,
                                  int num_groups, long long k_total, int* status, int num_sms,
                                  int force_bn, cudaStream_t stream) {
  return gemm_bf16_impl(A, B, D, Cin, M, N, K, lda, ldb, ldd, ldcin, a_mn_major, b_mn_major, alpha, beta, group_mode,
                        tile_group, group_offsets, num_groups, k_total, status, num_sms, force_bn, 1, stream);
}

// D[i][j] = D[j][i] for i > j, for `mats` stacked n x n matrices (n a multiple of 64), 64 x 64 blocks.
__global__ void __launch_bounds__(256) mirror_upper_kernel(__nv_bfloat16* __restrict__ d, int n, long long ldd) {
  __shared__ unsigned short tile[64][66];
  const int bj = blockIdx.x, bi = blockIdx.y;
  if (bi <= bj) return;                           // diagonal blocks were computed whole
  unsigned short* base = reinterpret_cast<unsigned short*>(d) + (long long)blockIdx.z * n * ldd;
  const int cp = threadIdx.x & 31, r0 = threadIdx.x >> 5;
  for (int r = r0; r < 64; r += 8) {              // source block (bj, bi): above the diagonal
    const unsigned v = *reinterpret_cast<const unsigned*>(base + (long long)(bj * 64 + r) * ldd + bi * 64 + 2 * cp);
    tile[r][2 * cp] = (unsigned short)(v & 0xffffu);
    tile[r][2 * cp + 1] = (unsigned short)(v >> 16);
  }
  __syncthreads();
  for (int r = r0; r < 64; r += 8) {              // destination block (bi, bj), row r = source column r
    const unsigned v = (unsigned)tile[2 * cp][r] | ((unsigned)tile[2 * cp + 1][r] << 16);
    *reinterpret_cast<unsigned*>(base + (long long)(bi * 64 + r) * ldd + bj * 64 + 2 * cp) = v;
  }
}

MFSDP_API int mfsdp_mirror_upper(void* D, int n, long long ldd, int mats, cudaStream_t stream) {
  if (n <= 0 || (n % 64) != 0 || (ldd % 2) != 0 || mats <= 0 || ((uintptr_t)D & 3)) return -2;
  if (n == 64) return 0;
  mirror_upper_kernel<<<dim3(n / 64, n / 64, mats), 256, 0, stream>>>((__nv_bfloat16*)D, n, ldd);
  return (int)cudaGetLastError();
}

// All-gather fused into the GEMM that first consumes the gathered weight:
//   D[M,N] = alpha * A[M,K] * B[N,K]^T + beta * Cin,  B row-major and contiguous (ldb == K),
// where (parts of) B are not in local memory yet.  `njobs` copy jobs (device tables) bring them in
// from peer memory with plain 16-byte loads while the tensor-core tiles whose B rows already
// arrived run; ag_flag[j] names the bn-row block of B that job j belongs to and ag_need[b] is the
// number of jobs of block b (0 for blocks that are already local), ag_first[b] the index of its first
// job (jobs are sorted by block).  `flags` (2 * tiles_n words: finished and claimed jobs per block) must
// be zero.  `rotate`: tile column the schedule starts at (the block holding the local rank's rows).  Returns the tile width used through *bn_out when called with njobs < 0 (planning call).
MFSDP_API int mfsdp_gemm_bf16_ag(const void* A, const void* B, void* D, const void* Cin, int M, int N, int K,
                                 long long lda, long long ldd, long long ldcin, float alpha, float beta,
                                 const unsigned long long* ag_src, const unsigned long long* ag_dst,
                                 const int* ag_bytes, const int* ag_flag, int njobs, unsigned* flags,
                                 const int* ag_need, const int* ag_first, int rotate, int bn,
                                 unsigned long long budget_ns, int* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (bn != 128 && bn != 256) || njobs < 0) return -2;
  ensure_context_on_this_thread();
  if ((lda % 8) || (K % 8) || (ldd % 8)) return -2;
  if (((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)D & 15)) return -2;
  GemmArgs args{};
  args.M = M; args.N = N; args.K = K;
  args.alpha = alpha; args.beta = beta;
  args.cin = (const __nv_bfloat16*)Cin; args.ldcin = ldcin;
  args.status = status;
  args.group_mode = 0;
  args.m_per_group = M;
  args.tiles_m = (M + BM - 1) / BM;
  args.tiles_m_per_group = args.tiles_m;
  args.tiles_n = (N + bn - 1) / bn;
  args.tile_m = BM;
  args.raster_group_m = 8;   // (walking a whole B row-block first measured slower: 0.193 vs 0.144 ms on 4 GPUs)
  args.ag_src = ag_src; args.ag_dst = ag_dst; args.ag_bytes = ag_bytes; args.ag_flag = ag_flag;
  args.ag_njobs = njobs; args.ag_flags = flags; args.ag_need = ag_need; args.ag_budget_ns = budget_ns;
  args.ag_first = ag_first;
  args.ag_rotate = (rotate > 0 && rotate < args.tiles_n) ? rotate : 0;
  CUtensorMap ta, tb, td;
  int rc = make_tmap_bf16_2d(&ta, A, M, K, lda, BM, 64);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tb, B, N, K, K, bn, 64);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&td, D, M, N, ldd, BM, 64);
  if (rc) return rc;
  const int total = args.tiles_m * args.tiles_n;
  args.total_tiles = total;
  const int grid = total < num_sms ? total : num_sms;
  return bn == 256 ? launch_gemm<256, false, false, true>(ta, tb, td, args, grid, stream)
                   : launch_gemm<128, false, false, true>(ta, tb, td, args, grid, stream);
}
