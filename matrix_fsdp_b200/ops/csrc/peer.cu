// Peer-memory collectives for one NVSwitch node: parameter all-gather as a *pull* of peer shards,
// gradient reduce-scatter as a *pull-and-sum* of peer gradient buffers, plus the cross-GPU flag
// protocol that orders them.  Every rank maps its peers' buffers once (CUDA IPC) and the kernels
// read them with plain 16-byte loads over NVLink; nothing is staged, padded or re-packed, so
// uneven / owner layouts cost exactly their bytes.
//
// Flags are 64-bit epoch counters living in each rank's own flag page; a peer publishes by
// writing its slot *in the waiter's page* (st.release.sys after a system fence), so waiters spin
// on local memory.  Every wait is bounded by a wall-clock budget and reports through a status word
// instead of hanging (code kErrPeerFlagTimeout).
//
// What these replace in the reference: NCCL all_gather_into_tensor / padded gather + unpad copies /
// grouped ncclBroadcast|Send/Recv (matrix_fsdp/runtime/collectives.py:208-492,
// kernels/native/matrix_nccl.cpp:111-335) and reduce_scatter_tensor + div_ / grouped ncclReduce
// (collectives.py:927-990, matrix_nccl.cpp:337-395).
#include "common.cuh"
#include <cstdlib>
#include <cstring>

namespace mfsdp {

constexpr int kMaxPeers = 16;

struct PeerPtrs {
  const void* p[kMaxPeers];
};
struct FlagPtrs {
  unsigned long long* p[kMaxPeers];
};

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// One thread per peer: flag_slots[t] (in the t-th peer's page, or our own) := value.
__global__ void peer_signal_kernel(FlagPtrs slots, int n, unsigned long long value) {
  const int t = threadIdx.x;
  if (t < n && slots.p[t] != nullptr) {
    __threadfence_system();
    st_release_sys(slots.p[t], value);
  }
}

// Spin until *slot >= value, the budget ends, or some kernel already reported an error: once the
// status word is set every later wait returns at once, so one lost peer costs one budget, not one
// budget per collective.
__device__ __forceinline__ void bounded_flag_wait(const unsigned long long* slot, unsigned long long value,
                                                  unsigned long long budget_ns, int* status) {
  if (ld_acquire_sys(slot) >= value) return;
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  const uint64_t t0 = globaltimer_ns();
  unsigned spins = 0;
  while (ld_acquire_sys(slot) < value) {
    if ((++spins & 0xff) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return;
      if (globaltimer_ns() - t0 > budget_ns) {
        atomicCAS(status, 0, (int)kErrPeerFlagTimeout);
        return;
      }
      __nanosleep(200);
    }
  }
}

// One thread per awaited slot (all in this rank's page).
__global__ void peer_wait_kernel(const unsigned long long* flags, int first, int n, unsigned long long value,
                                 unsigned long long budget_ns, int* status) {
  const int t = threadIdx.x;
  if (t >= n) return;
  bounded_flag_wait(flags + first + t, value, budget_ns, status);
}

// Publish and wait in one launch: thread t writes `value` into this rank's slot of peer t's page,
// then waits for peer t's slot in the local page.  The two halves touch different GPUs' pages, so
// the launch never waits on itself.
__global__ void peer_signal_wait_kernel(FlagPtrs slots, const unsigned long long* flags, int first, int n,
                                        unsigned long long value, unsigned long long budget_ns, int* status) {
  const int t = threadIdx.x;
  if (t >= n) return;
  if (slots.p[t] != nullptr) {
    __threadfence_system();
    st_release_sys(slots.p[t], value);
  }
  bounded_flag_wait(flags + first + t, value, budget_ns, status);
}

// Debug aid (MFSDP_DEBUG_BOUNDS=1): check a pull table against the destination extent and the
// windows of peer memory the sources may come from; a bad entry records kErrBounds and the data
// kernels behind it (which all return early on a set status word) touch nothing.
struct AddrWindows {
  unsigned long long lo[16];
  unsigned long long hi[16];
  int n;
};
__global__ void validate_pull_table_kernel(const unsigned long long* src_addr, const long long* dst_off,
                                           const long long* len, int nseg, long long dst_numel, int elem_size,
                                           AddrWindows win, int* status) {
  for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < nseg; s += gridDim.x * blockDim.x) {
    const long long n = len[s], d = dst_off[s];
    bool ok = n >= 0 && d >= 0 && d + n <= dst_numel;
    const unsigned long long a = src_addr[s], b = a + (unsigned long long)n * elem_size;
    bool inside = win.n == 0;
    for (int w = 0; w < win.n; ++w) inside = inside || (a >= win.lo[w] && b <= win.hi[w]);
    if (!(ok && inside)) atomicCAS(status, 0, (int)kErrBounds);
  }
}
__global__ void validate_reduce_table_kernel(const long long* global_off, const long long* local_off,
                                             const long long* len, int nseg, long long full_numel,
                                             long long shard_numel, int* status) {
  for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < nseg; s += gridDim.x * blockDim.x) {
    const long long n = len[s], g = global_off[s], l = local_off[s];
    if (!(n >= 0 && g >= 0 && l >= 0 && g + n <= full_numel && l + n <= shard_numel))
      atomicCAS(status, 0, (int)kErrBounds);
  }
}

// ------------------------------------------------------------------ all-gather (pull)
struct PullTable {           // device arrays of length nseg
  const unsigned long long* src_addr;   // absolute address of the segment in the owner's (mapped) memory
  const long long* dst_off;             // element offset in the local full buffer
  const long long* len;                 // elements
};

template <typename T>
__global__ void ag_pull_kernel(T* __restrict__ dst, PullTable tab, int nseg, const int* status) {
  if (status != nullptr && *status != 0) return;   // an earlier wait gave up: the peers' data is not there
  constexpr int kPer = 16 / sizeof(T);
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
    const T* sp = reinterpret_cast<const T*>(tab.src_addr[s]);
    T* dp = dst + tab.dst_off[s];
    const long long n = tab.len[s];
    const uintptr_t sa = reinterpret_cast<uintptr_t>(sp), da = reinterpret_cast<uintptr_t>(dp);
    if ((sa & 15) == (da & 15)) {
      long long head = ((16 - (sa & 15)) & 15) / sizeof(T);
      if (head > n) head = n;
      const long long nvec = (n - head) / kPer;
      for (long long i = tid; i < head; i += stride) dp[i] = sp[i];
      const uint4* sv = reinterpret_cast<const uint4*>(sp + head);
      uint4* dv = reinterpret_cast<uint4*>(dp + head);
      long long i = tid;
      // 4 independent 16-byte loads in flight per thread to cover NVLink latency
      for (; i + 3 * stride < nvec; i += 4 * stride) {
        const uint4 a = sv[i], b = sv[i + stride], c = sv[i + 2 * stride], d = sv[i + 3 * stride];
        dv[i] = a; dv[i + stride] = b; dv[i + 2 * stride] = c; dv[i + 3 * stride] = d;
      }
      for (; i < nvec; i += stride) dv[i] = sv[i];
      for (long long j = head + nvec * kPer + tid; j < n; j += stride) dp[j] = sp[j];
    } else {
      for (long long i = tid; i < n; i += stride) dp[i] = sp[i];
    }
  }
}

// ------------------------------------------------------------------ reduce-scatter (pull + sum)
struct ReduceTable {         // my segments
  const long long* global_off;   // element offset in every rank's full gradient buffer
  const long long* local_off;    // element offset in my output shard
  const long long* len;
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = unpack_bf16x2(w[e]);
    v[2 * e] = f.x; v[2 * e + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                            pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
}
__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ void from_f(float& d, float x) { d = x; }
__device__ __forceinline__ void from_f(__nv_bfloat16& d, float x) { d = __float2bfloat16_rn(x); }

// Raw 8-element vectors: all peers' loads are issued before the first conversion, so WORLD
// 16-byte (bf16) or 32-byte (fp32) requests are in flight per thread.
struct Raw8bf { uint4 u; };
struct Raw8f { float4 a, b; };
__device__ __forceinline__ Raw8bf load_raw8(const __nv_bfloat16* p) { return {*reinterpret_cast<const uint4*>(p)}; }
__device__ __forceinline__ Raw8f load_raw8(const float* p) {
  return {reinterpret_cast<const float4*>(p)[0], reinterpret_cast<const float4*>(p)[1]};
}
__device__ __forceinline__ void add_raw8(float (&acc)[8], const Raw8bf& r) {
  const uint32_t w[4] = {r.u.x, r.u.y, r.u.z, r.u.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = unpack_bf16x2(w[e]);
    acc[2 * e] += f.x; acc[2 * e + 1] += f.y;
  }
}
__device__ __forceinline__ void add_raw8(float (&acc)[8], const Raw8f& r) {
  acc[0] += r.a.x; acc[1] += r.a.y; acc[2] += r.a.z; acc[3] += r.a.w;
  acc[4] += r.b.x; acc[5] += r.b.y; acc[6] += r.b.z; acc[7] += r.b.w;
}

// acc[0..8) = sum over ranks of 8 consecutive elements at `off`, fp32, rank order (rank, rank+1, ...).
template <typename TIn, int WORLD>
__device__ __forceinline__ void sum_peers8(const PeerPtrs& grads, int world, int rank, long long off,
                                           float (&acc)[8]) {
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  if constexpr (WORLD > 0) {
    decltype(load_raw8((const TIn*)nullptr)) raw[WORLD];
#pragma unroll
    for (int k = 0; k < WORLD; ++k) {
      const int r = (rank + k) & (WORLD - 1);          // WORLD is a power of two here
      raw[k] = load_raw8(reinterpret_cast<const TIn*>(grads.p[r]) + off);
    }
#pragma unroll
    for (int k = 0; k < WORLD; ++k) add_raw8(acc, raw[k]);
  } else {
    for (int k = 0; k < world; ++k) {
      const int r = (rank + k) % world;
      add_raw8(acc, load_raw8(reinterpret_cast<const TIn*>(grads.p[r]) + off));
    }
  }
}

// out[local_off + i] = scale * sum_r grads_r[global_off + i], fp32 accumulation, rank order fixed
// (starting at the local rank's own buffer) so the result is deterministic.
// WORLD > 0 fixes the peer count at compile time so the peer loop unrolls into WORLD independent
// 16-byte loads in flight per thread (the NVLink round trip is the latency to cover).
template <typename TIn, typename TOut, bool ACCUM, int WORLD>
__global__ void rs_pull_reduce_kernel(PeerPtrs grads, int world_rt, int rank, TOut* __restrict__ out,
                                      ReduceTable tab, int nseg, float scale, const int* status) {
  if (status != nullptr && *status != 0) return;
  const int world = WORLD > 0 ? WORLD : world_rt;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
    const long long g0 = tab.global_off[s], l0 = tab.local_off[s], n = tab.len[s];
    const bool aligned = ((g0 * sizeof(TIn)) % 16 == 0) && ((l0 * sizeof(TOut)) % 16 == 0) &&
                         ((reinterpret_cast<uintptr_t>(out) % 16) == 0);
    const long long nvec = aligned ? n / 8 : 0;
    for (long long i = tid; i < nvec; i += stride) {
      float acc[8];
      sum_peers8<TIn, WORLD>(grads, world, rank, g0 + i * 8, acc);
      TOut* o = out + l0 + i * 8;
      if (ACCUM) {
        float prev[8];
        load8(o, prev);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = acc[e] * scale + prev[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] *= scale;
      }
      store8(o, acc);
    }
    for (long long i = nvec * 8 + tid; i < n; i += stride) {
      float acc = 0.f;
      for (int k = 0; k < world; ++k) {
        const int r = (rank + k) % world;
        acc += to_f(reinterpret_cast<const TIn*>(grads.p[r])[g0 + i]);
      }
      acc *= scale;
      if (ACCUM) acc += to_f(out[l0 + i]);
      from_f(out[l0 + i], acc);
    }
  }
}

// Reduce-scatter fused with the sharded AdamW update: the reduced gradient never touches memory.
//   g = scale * sum_r grads_r[global_off + i]   (bf16 or fp32 in, fp32 sum, fixed rank order)
//   p, m, v (fp32, this rank's shard) updated in place; p_lp = bf16 copy of p for the next all-gather.
struct AdamWArgs {
  float* p;
  float* m;
  float* v;
  __nv_bfloat16* p_lp;
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2_sqrt;
};

__device__ __forceinline__ void adamw_one(float& p, float& m, float& v, float g, const AdamWArgs& a) {
  p *= (1.f - a.lr * a.weight_decay);
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  p -= (a.lr / a.bias1) * (m / (sqrtf(v) / a.bias2_sqrt + a.eps));
}

template <typename TIn, int WORLD>
__global__ void rs_pull_adamw_kernel(PeerPtrs grads, int world_rt, int rank, ReduceTable tab, int nseg, float scale,
                                     AdamWArgs a, const int* status) {
  // p / m / v are updated in place: never run on gradients whose arrival a wait has given up on
  if (status != nullptr && *status != 0) return;
  const int world = WORLD > 0 ? WORLD : world_rt;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
    const long long g0 = tab.global_off[s], l0 = tab.local_off[s], n = tab.len[s];
    const bool aligned = ((g0 * sizeof(TIn)) % 16 == 0) && (l0 % 8 == 0);
    const long long nvec = aligned ? n / 8 : 0;
    for (long long i = tid; i < nvec; i += stride) {
      float acc[8];
      sum_peers8<TIn, WORLD>(grads, world, rank, g0 + i * 8, acc);
      const long long j = l0 + i * 8;
      float pp[8], mm[8], vv[8];
      load8(a.p + j, pp);
      load8(a.m + j, mm);
      load8(a.v + j, vv);
#pragma unroll
      for (int e = 0; e < 8; ++e) adamw_one(pp[e], mm[e], vv[e], acc[e] * scale, a);
      store8(a.p + j, pp);
      store8(a.m + j, mm);
      store8(a.v + j, vv);
      if (a.p_lp) store8(a.p_lp + j, pp);
    }
    for (long long i = nvec * 8 + tid; i < n; i += stride) {
      float acc = 0.f;
      for (int k = 0; k < world; ++k) {
        const int r = (rank + k) % world;
        acc += to_f(reinterpret_cast<const TIn*>(grads.p[r])[g0 + i]);
      }
      const long long j = l0 + i;
      float pp = a.p[j], mm = a.m[j], vv = a.v[j];
      adamw_one(pp, mm, vv, acc * scale, a);
      a.p[j] = pp; a.m[j] = mm; a.v[j] = vv;
      if (a.p_lp) a.p_lp[j] = __float2bfloat16_rn(pp);
    }
  }
}

// ------------------------------------------------------------------ NVLS (multimem through the NVSwitch)
// A buffer that every rank allocated symmetrically and bound to one multicast object has, beside its
// per-rank addresses, one *multicast* address.  A store to it lands in all ranks' copies (the switch
// replicates it), a `ld_reduce` from it returns the sum over all ranks' copies (the switch adds them).
// So the all-gather is a push of only this rank's own shard (1/W of the bytes leave the GPU, the SMs
// touch 1/W of the data), and the reduce-scatter reads each owned element once instead of W times.
// The in-switch sum of bf16 inputs is accumulated in fp32 (.acc::f32) and returned as bf16.
__device__ __forceinline__ void multimem_st16(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
template <typename T>
struct McUnroll {
  static constexpr int value = sizeof(T) == 2 ? 8 : 4;   // 16-byte requests: one per 8 bf16, two per 8 fp32
};

// Raw results of the in-switch reductions of one trip (converted to fp32 only when consumed, which keeps
// the registers per thread low enough for four CTAs per SM).
__device__ __forceinline__ Raw8bf mc_raw8(const __nv_bfloat16* mc, long long off) {
  return {multimem_ld_reduce_bf16x8(mc + off)};
}
__device__ __forceinline__ Raw8f mc_raw8(const float* mc, long long off) {
  return {multimem_ld_reduce_f32x4(mc + off), multimem_ld_reduce_f32x4(mc + off + 4)};
}
__device__ __forceinline__ void raw_to_f32(const Raw8bf& r, float (&acc)[8]) {
  const uint32_t w[4] = {r.u.x, r.u.y, r.u.z, r.u.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = unpack_bf16x2(w[e]);
    acc[2 * e] = f.x; acc[2 * e + 1] = f.y;
  }
}
__device__ __forceinline__ void raw_to_f32(const Raw8f& r, float (&acc)[8]) {
  acc[0] = r.a.x; acc[1] = r.a.y; acc[2] = r.a.z; acc[3] = r.a.w;
  acc[4] = r.b.x; acc[5] = r.b.y; acc[6] = r.b.z; acc[7] = r.b.w;
}

// All-gather as a push: copy this rank's segments (byte offsets, all multiples of 16) from its shard
// into the multicast address of the full-parameter buffer, i.e. into every rank's copy at once.
struct PushTable {
  const long long* src_byte;   // offset in the local shard
  const long long* dst_byte;   // offset in the full buffer
  const long long* nbytes;
};
__global__ void ag_push_mc_kernel(const char* __restrict__ shard, char* mc_full, PushTable tab, int nseg,
                                  const int* status) {
  if (status != nullptr && *status != 0) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
    const uint4* sv = reinterpret_cast<const uint4*>(shard + tab.src_byte[s]);
    char* dv = mc_full + tab.dst_byte[s];
    const long long nvec = tab.nbytes[s] / 16;
    long long i = tid;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      const uint4 a = sv[i], b = sv[i + stride], c = sv[i + 2 * stride], d = sv[i + 3 * stride];
      multimem_st16(dv + i * 16, a);
      multimem_st16(dv + (i + stride) * 16, b);
      multimem_st16(dv + (i + 2 * stride) * 16, c);
      multimem_st16(dv + (i + 3 * stride) * 16, d);
    }
    for (; i < nvec; i += stride) multimem_st16(dv + i * 16, sv[i]);
  }
  // make the multicast stores visible system-wide before the flag that follows in stream order
  __threadfence_system();
}

// Reduce-scatter through the switch: out[local_off + i] = scale * (sum over ranks)[global_off + i].
// Segment offsets and lengths are multiples of 8 elements (checked by the launcher's caller).
template <typename TIn, typename TOut, bool ACCUM>
__global__ void __launch_bounds__(256, 2) rs_mc_reduce_kernel(const TIn* mc_grad, TOut* __restrict__ out, ReduceTable tab, int nseg,
                                    float scale, const int* status) {
  constexpr int kMcUnroll = McUnroll<TIn>::value;
  if (status != nullptr && *status != 0) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
    const long long g0 = tab.global_off[s], l0 = tab.local_off[s], nvec = tab.len[s] / 8;
    // kMcUnroll in-switch reductions in flight per thread: the round trip through the switch is several
    // microseconds, so the loads of one trip are all issued before the first result is used
    for (long long i0 = tid; i0 < nvec; i0 += kMcUnroll * stride) {
      decltype(mc_raw8(mc_grad, 0)) raw[kMcUnroll];
#pragma unroll
      for (int u = 0; u < kMcUnroll; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec) raw[u] = mc_raw8(mc_grad, g0 + i * 8);
      }
#pragma unroll
      for (int u = 0; u < kMcUnroll; ++u) {
        const long long i = i0 + u * stride;
        if (i >= nvec) break;
        float acc[8];
        raw_to_f32(raw[u], acc);
        TOut* o = out + l0 + i * 8;
        if (ACCUM) {
          float prev[8];
          load8(o, prev);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = acc[e] * scale + prev[e];
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] *= scale;
        }
        store8(o, acc);
      }
    }
  }
}

// The same reduction feeding the sharded AdamW update directly (the reduced gradient is never stored).
template <typename TIn>
__global__ void __launch_bounds__(256, 2) rs_mc_adamw_kernel(const TIn* mc_grad, ReduceTable tab, int nseg, float scale, AdamWArgs a,
                                   const int* status) {
  constexpr int kMcUnroll = McUnroll<TIn>::value;
  if (status != nullptr && *status != 0) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
    const long long g0 = tab.global_off[s], l0 = tab.local_off[s], nvec = tab.len[s] / 8;
    for (long long i0 = tid; i0 < nvec; i0 += kMcUnroll * stride) {
      decltype(mc_raw8(mc_grad, 0)) raw[kMcUnroll];
#pragma unroll
      for (int u = 0; u < kMcUnroll; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec) raw[u] = mc_raw8(mc_grad, g0 + i * 8);
      }
#pragma unroll
      for (int u = 0; u < kMcUnroll; ++u) {
        const long long i = i0 + u * stride;
        if (i >= nvec) break;
        const long long j = l0 + i * 8;
        float acc[8], pp[8], mm[8], vv[8];
        raw_to_f32(raw[u], acc);
        load8(a.p + j, pp);
        load8(a.m + j, mm);
        load8(a.v + j, vv);
#pragma unroll
        for (int e = 0; e < 8; ++e) adamw_one(pp[e], mm[e], vv[e], acc[e] * scale, a);
        store8(a.p + j, pp);
        store8(a.m + j, mm);
        store8(a.v + j, vv);
        if (a.p_lp) store8(a.p_lp + j, pp);
      }
    }
  }
}

// One-shot all-reduce in place on a multicast buffer: rank r sums the r-th slice through the switch
// and stores the scaled result back through the multicast address, so every copy ends up equal.
template <typename T>
__global__ void __launch_bounds__(256, 2) ar_mc_kernel(T* mc_buf, long long nvec8, int rank, int world, float scale, const int* status) {
  constexpr int kMcUnroll = McUnroll<T>::value;
  if (status != nullptr && *status != 0) return;
  const long long lo = nvec8 * rank / world, hi = nvec8 * (rank + 1) / world;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = lo + blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < hi; i0 += kMcUnroll * stride) {
    decltype(mc_raw8(mc_buf, 0)) raw[kMcUnroll];
#pragma unroll
    for (int u = 0; u < kMcUnroll; ++u)
      if (i0 + u * stride < hi) raw[u] = mc_raw8(mc_buf, (i0 + u * stride) * 8);
#pragma unroll
    for (int u = 0; u < kMcUnroll; ++u) {
      const long long i = i0 + u * stride;
      if (i >= hi) break;
      float acc[8];
      raw_to_f32(raw[u], acc);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= scale;
      if (sizeof(T) == 2) {
        multimem_st16(mc_buf + i * 8, make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                 pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7])));
      } else {
        multimem_st16(mc_buf + i * 8, make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]),
                                                 __float_as_uint(acc[2]), __float_as_uint(acc[3])));
        multimem_st16(mc_buf + i * 8 + 4, make_uint4(__float_as_uint(acc[4]), __float_as_uint(acc[5]),
                                                     __float_as_uint(acc[6]), __float_as_uint(acc[7])));
      }
    }
  }
  __threadfence_system();
}

// Upper bound on the CTAs of one pull kernel (MFSDP_PEER_MAX_BLOCKS).  The pull kernels run beside the
// GEMMs of the neighbouring block; fewer, longer-lived CTAs leave more issue slots to the tensor kernels.
static long long peer_max_blocks() {
  static long long v = [] {
    const char* e = getenv("MFSDP_PEER_MAX_BLOCKS");
    long long x = e ? atoll(e) : 0;
    return x > 0 ? x : 148LL * 2;
  }();
  return v;
}

static inline dim3 seg_grid(long long max_len, int per_thread, int nseg) {
  long long bx = (max_len / per_thread + 255) / 256;
  if (bx < 1) bx = 1;
  int gy = nseg < 1024 ? nseg : 1024;
  const long long cap = peer_max_blocks();
  if (bx * gy > cap) bx = (cap + gy - 1) / gy;
  return dim3((unsigned)bx, (unsigned)gy);
}

}  // namespace mfsdp

using namespace mfsdp;

// ------------------------------------------------------------------ IPC plumbing (host)
// Symmetric segments are plain cudaMalloc allocations owned by this library (not by a framework
// caching allocator), so the IPC handle always names the segment's base address.
MFSDP_API int mfsdp_dev_malloc(unsigned long long bytes, void** out) { return (int)cudaMalloc(out, bytes); }
MFSDP_API int mfsdp_dev_free(void* p) { return (int)cudaFree(p); }

MFSDP_API int mfsdp_ipc_get_handle(const void* dev_ptr, void* handle_out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(dev_ptr));
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out64, &h, sizeof(h));
  return 0;
}
MFSDP_API int mfsdp_ipc_open_handle(const void* handle64, void** dev_ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
  return (int)e;
}
MFSDP_API int mfsdp_ipc_close_handle(void* dev_ptr) { return (int)cudaIpcCloseMemHandle(dev_ptr); }
MFSDP_API int mfsdp_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }
MFSDP_API int mfsdp_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) return 0;
  return ok;
}

// ------------------------------------------------------------------ launchers
// slots[i]: address (in peer i's flag page, mapped here) of the slot this rank publishes to.
MFSDP_API int mfsdp_peer_signal(const unsigned long long* slot_addrs_host, int n, unsigned long long value,
                                cudaStream_t st) {
  if (n <= 0 || n > kMaxPeers) return -2;
  FlagPtrs fp{};
  for (int i = 0; i < n; ++i) fp.p[i] = reinterpret_cast<unsigned long long*>(slot_addrs_host[i]);
  peer_signal_kernel<<<1, 32, 0, st>>>(fp, n, value);
  return (int)cudaGetLastError();
}

// Wait until flags[first .. first+n) (this rank's own page) are all >= value.
MFSDP_API int mfsdp_peer_wait(const void* flags, int first, int n, unsigned long long value,
                                unsigned long long budget_ns, int* status, cudaStream_t st) {
  if (n <= 0 || n > 1024) return -2;
  peer_wait_kernel<<<1, ((n + 31) / 32) * 32, 0, st>>>((const unsigned long long*)flags, first, n, value, budget_ns,
                                                        status);
  return (int)cudaGetLastError();
}

// Publish `value` to every peer (slot_addrs_host as in mfsdp_peer_signal) and wait for theirs, one launch.
MFSDP_API int mfsdp_peer_signal_wait(const unsigned long long* slot_addrs_host, const void* flags, int first, int n,
                                     unsigned long long value, unsigned long long budget_ns, int* status,
                                     cudaStream_t st) {
  if (n <= 0 || n > kMaxPeers) return -2;
  FlagPtrs fp{};
  for (int i = 0; i < n; ++i) fp.p[i] = reinterpret_cast<unsigned long long*>(slot_addrs_host[i]);
  peer_signal_wait_kernel<<<1, 32, 0, st>>>(fp, (const unsigned long long*)flags, first, n, value, budget_ns, status);
  return (int)cudaGetLastError();
}

// Debug checks of the tables the pull / reduce kernels trust (record kErrBounds in the status word).
// win_lo/win_hi: `nwin` address windows (peer shard buffers) every source segment has to lie in.
MFSDP_API int mfsdp_validate_pull_table(const unsigned long long* src_addr, const long long* dst_off,
                                        const long long* len, int nseg, long long dst_numel, int elem_size,
                                        const unsigned long long* win_lo, const unsigned long long* win_hi, int nwin,
                                        int* status, cudaStream_t st) {
  if (nseg <= 0) return 0;
  if (nwin < 0 || nwin > 16) return -2;
  AddrWindows w{};
  w.n = nwin;
  for (int i = 0; i < nwin; ++i) { w.lo[i] = win_lo[i]; w.hi[i] = win_hi[i]; }
  validate_pull_table_kernel<<<1, 256, 0, st>>>(src_addr, dst_off, len, nseg, dst_numel, elem_size, w, status);
  return (int)cudaGetLastError();
}
MFSDP_API int mfsdp_validate_reduce_table(const long long* global_off, const long long* local_off,
                                          const long long* len, int nseg, long long full_numel,
                                          long long shard_numel, int* status, cudaStream_t st) {
  if (nseg <= 0) return 0;
  validate_reduce_table_kernel<<<1, 256, 0, st>>>(global_off, local_off, len, nseg, full_numel, shard_numel, status);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_ag_pull(void* dst, const unsigned long long* src_addr, const long long* dst_off,
                            const long long* len, int nseg, long long max_len, int elem_size, const int* status,
                            cudaStream_t st) {
  if (nseg <= 0) return 0;
  PullTable tab{src_addr, dst_off, len};
  const dim3 grid = seg_grid(max_len, (16 / elem_size) * 4, nseg);
  switch (elem_size) {
    case 2: ag_pull_kernel<uint16_t><<<grid, 256, 0, st>>>((uint16_t*)dst, tab, nseg, status); break;
    case 4: ag_pull_kernel<uint32_t><<<grid, 256, 0, st>>>((uint32_t*)dst, tab, nseg, status); break;
    case 1: ag_pull_kernel<uint8_t><<<grid, 256, 0, st>>>((uint8_t*)dst, tab, nseg, status); break;
    case 8: ag_pull_kernel<uint64_t><<<grid, 256, 0, st>>>((uint64_t*)dst, tab, nseg, status); break;
    default: return -2;
  }
  return (int)cudaGetLastError();
}

// grad_ptrs_host[r]: base of rank r's full gradient buffer for this unit (mapped here; own buffer for r == rank).
MFSDP_API int mfsdp_rs_pull_reduce(const unsigned long long* grad_ptrs_host, int world, int rank, void* out,
                                   const long long* global_off, const long long* local_off, const long long* len,
                                   int nseg, long long max_len, int in_is_bf16, int out_is_bf16, int accumulate,
                                   float scale, const int* status, cudaStream_t st) {
  if (nseg <= 0) return 0;
  if (world <= 0 || world > kMaxPeers) return -2;
  PeerPtrs pp{};
  for (int r = 0; r < world; ++r) pp.p[r] = reinterpret_cast<const void*>(grad_ptrs_host[r]);
  ReduceTable tab{global_off, local_off, len};
  const dim3 grid = seg_grid(max_len, 8, nseg);
#define MFSDP_RS_W(TI, TO, ACC, W) \
  rs_pull_reduce_kernel<TI, TO, ACC, W><<<grid, 256, 0, st>>>(pp, world, rank, (TO*)out, tab, nseg, scale, status)
#define MFSDP_RS_A(TI, TO, ACC)                  \
  do {                                           \
    switch (world) {                             \
      case 2: MFSDP_RS_W(TI, TO, ACC, 2); break; \
      case 4: MFSDP_RS_W(TI, TO, ACC, 4); break; \
      case 8: MFSDP_RS_W(TI, TO, ACC, 8); break; \
      default: MFSDP_RS_W(TI, TO, ACC, 0);       \
    }                                            \
  } while (0)
#define MFSDP_RS(TI, TO)                    \
  do {                                      \
    if (accumulate) MFSDP_RS_A(TI, TO, true); \
    else MFSDP_RS_A(TI, TO, false);         \
  } while (0)
  if (in_is_bf16 && !out_is_bf16) MFSDP_RS(__nv_bfloat16, float);
  else if (in_is_bf16 && out_is_bf16) MFSDP_RS(__nv_bfloat16, __nv_bfloat16);
  else if (!in_is_bf16 && !out_is_bf16) MFSDP_RS(float, float);
  else return -2;
#undef MFSDP_RS
#undef MFSDP_RS_A
#undef MFSDP_RS_W
  return (int)cudaGetLastError();
}

static bool adamw_ptrs_ok(const float* p, const float* m, const float* v, const void* p_lp) {
  return !(((uintptr_t)p % 16) || ((uintptr_t)m % 16) || ((uintptr_t)v % 16) || ((uintptr_t)p_lp % 16));
}

MFSDP_API int mfsdp_rs_pull_adamw(const unsigned long long* grad_ptrs_host, int world, int rank,
                                  const long long* global_off, const long long* local_off, const long long* len,
                                  int nseg, long long max_len, int in_is_bf16, float scale, float* p, float* m,
                                  float* v, void* p_lp, float lr, float beta1, float beta2, float eps,
                                  float weight_decay, int step, const int* status, cudaStream_t st) {
  if (nseg <= 0) return 0;
  if (world <= 0 || world > kMaxPeers || step < 1) return -2;
  if (!adamw_ptrs_ok(p, m, v, p_lp)) return -2;
  PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = reinterpret_cast<const void*>(grad_ptrs_host[i]);
  ReduceTable tab{global_off, local_off, len};
  AdamWArgs a{p, m, v, (__nv_bfloat16*)p_lp, lr, beta1, beta2, eps, weight_decay,
              1.f - powf(beta1, (float)step), sqrtf(1.f - powf(beta2, (float)step))};
  const dim3 grid = seg_grid(max_len, 8, nseg);
#define MFSDP_RA(TI)                                                                                              \
  do {                                                                                                            \
    switch (world) {                                                                                              \
      case 2: rs_pull_adamw_kernel<TI, 2><<<grid, 256, 0, st>>>(pp, world, rank, tab, nseg, scale, a, status); break; \
      case 4: rs_pull_adamw_kernel<TI, 4><<<grid, 256, 0, st>>>(pp, world, rank, tab, nseg, scale, a, status); break; \
      case 8: rs_pull_adamw_kernel<TI, 8><<<grid, 256, 0, st>>>(pp, world, rank, tab, nseg, scale, a, status); break; \
      default: rs_pull_adamw_kernel<TI, 0><<<grid, 256, 0, st>>>(pp, world, rank, tab, nseg, scale, a, status);       \
    }                                                                                                             \
  } while (0)
  if (in_is_bf16) MFSDP_RA(__nv_bfloat16);
  else MFSDP_RA(float);
#undef MFSDP_RA
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ NVLS launchers
// Grid of the multimem kernels (MFSDP_NVLS_BLOCKS, default one CTA on every other SM).  These kernels run beside the
// GEMMs and attention kernels of the neighbouring block, which need one CTA on EVERY SM (persistent grids of
// 148): a communication kernel that fills an SM's register file keeps that CTA from starting and the whole
// GEMM waits for it.  So the footprint per SM is at most one CTA of 256 threads, and the bytes in flight that the
// several-microsecond round trip through the switch needs come from kMcUnroll requests per thread instead
// of from more CTAs.
static long long nvls_blocks() {
  static long long v = [] {
    const char* e = getenv("MFSDP_NVLS_BLOCKS");
    long long x = e ? atoll(e) : 0;
    return x > 0 ? x : 74LL;      // measured on 2 and 8 GPUs: 74 beats 148 / 296 inside a training step
  }();
  return v;
}
static inline dim3 nvls_grid(long long max_vecs, int nseg) {
  long long bx = (max_vecs + 255) / 256;
  if (bx < 1) bx = 1;
  int gy = nseg < 64 ? nseg : 64;
  const long long cap = nvls_blocks();
  if (bx * gy > cap) bx = (cap + gy - 1) / gy;
  return dim3((unsigned)bx, (unsigned)gy);
}

// shard: local shard base; mc_full: multicast address of the full-parameter buffer; tables in bytes (x16).
MFSDP_API int mfsdp_ag_push_mc(const void* shard, void* mc_full, const long long* src_byte, const long long* dst_byte,
                               const long long* nbytes, int nseg, long long max_bytes, const int* status,
                               cudaStream_t st) {
  if (nseg <= 0) return 0;
  if (((uintptr_t)shard % 16) || ((uintptr_t)mc_full % 16)) return -2;
  PushTable tab{src_byte, dst_byte, nbytes};
  const dim3 grid = nvls_grid(max_bytes / 64, nseg);
  ag_push_mc_kernel<<<grid, 256, 0, st>>>((const char*)shard, (char*)mc_full, tab, nseg, status);
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_rs_mc_reduce(const void* mc_grad, void* out, const long long* global_off,
                                 const long long* local_off, const long long* len, int nseg, long long max_len,
                                 int in_is_bf16, int out_is_bf16, int accumulate, float scale, const int* status,
                                 cudaStream_t st) {
  if (nseg <= 0) return 0;
  if (((uintptr_t)mc_grad % 16) || ((uintptr_t)out % 16)) return -2;
  ReduceTable tab{global_off, local_off, len};
  const dim3 grid = nvls_grid(max_len / 8, nseg);
#define MFSDP_MC(TI, TO)                                                                                    \
  do {                                                                                                      \
    if (accumulate) rs_mc_reduce_kernel<TI, TO, true><<<grid, 256, 0, st>>>((const TI*)mc_grad, (TO*)out, tab, nseg, scale, status); \
    else rs_mc_reduce_kernel<TI, TO, false><<<grid, 256, 0, st>>>((const TI*)mc_grad, (TO*)out, tab, nseg, scale, status);          \
  } while (0)
  if (in_is_bf16 && !out_is_bf16) MFSDP_MC(__nv_bfloat16, float);
  else if (in_is_bf16 && out_is_bf16) MFSDP_MC(__nv_bfloat16, __nv_bfloat16);
  else if (!in_is_bf16 && !out_is_bf16) MFSDP_MC(float, float);
  else return -2;
#undef MFSDP_MC
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_rs_mc_adamw(const void* mc_grad, const long long* global_off, const long long* local_off,
                                const long long* len, int nseg, long long max_len, int in_is_bf16, float scale,
                                float* p, float* m, float* v, void* p_lp, float lr, float beta1, float beta2, float eps,
                                float weight_decay, int step, const int* status, cudaStream_t st) {
  if (nseg <= 0) return 0;
  if (step < 1 || ((uintptr_t)mc_grad % 16) || !adamw_ptrs_ok(p, m, v, p_lp)) return -2;
  ReduceTable tab{global_off, local_off, len};
  AdamWArgs a{p, m, v, (__nv_bfloat16*)p_lp, lr, beta1, beta2, eps, weight_decay,
              1.f - powf(beta1, (float)step), sqrtf(1.f - powf(beta2, (float)step))};
  const dim3 grid = nvls_grid(max_len / 8, nseg);
  if (in_is_bf16) rs_mc_adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)mc_grad, tab, nseg, scale, a, status);
  else rs_mc_adamw_kernel<float><<<grid, 256, 0, st>>>((const float*)mc_grad, tab, nseg, scale, a, status);
  return (int)cudaGetLastError();
}

// In-place all-reduce of `numel` elements (a multiple of 8) at the multicast address mc_buf.
MFSDP_API int mfsdp_ar_mc(void* mc_buf, long long numel, int is_bf16, int rank, int world, float scale,
                          const int* status, cudaStream_t st) {
  if (numel <= 0) return 0;
  if (numel % 8 || world <= 0 || rank < 0 || rank >= world || ((uintptr_t)mc_buf % 16)) return -2;
  const long long nvec8 = numel / 8;
  const dim3 grid = nvls_grid((nvec8 + world - 1) / world, 1);
  if (is_bf16) ar_mc_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)mc_buf, nvec8, rank, world, scale, status);
  else ar_mc_kernel<float><<<grid, 256, 0, st>>>((float*)mc_buf, nvec8, rank, world, scale, status);
  return (int)cudaGetLastError();
}
