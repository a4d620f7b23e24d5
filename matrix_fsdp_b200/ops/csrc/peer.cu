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

// One thread per awaited slot (all in this rank's page): spin until slot >= value or the budget ends.
__global__ void peer_wait_kernel(const unsigned long long* flags, int first, int n, unsigned long long value,
                                 unsigned long long budget_ns, int* status) {
  const int t = threadIdx.x;
  if (t >= n) return;
  const unsigned long long* slot = flags + first + t;
  if (ld_acquire_sys(slot) >= value) return;
  const uint64_t t0 = globaltimer_ns();
  unsigned spins = 0;
  while (ld_acquire_sys(slot) < value) {
    if ((++spins & 0xff) == 0) {
      if (globaltimer_ns() - t0 > budget_ns) {
        atomicCAS(status, 0, (int)kErrPeerFlagTimeout);
        return;
      }
      __nanosleep(200);
    }
  }
}

// ------------------------------------------------------------------ all-gather (pull)
struct PullTable {           // device arrays of length nseg
  const unsigned long long* src_addr;   // absolute address of the segment in the owner's (mapped) memory
  const long long* dst_off;             // element offset in the local full buffer
  const long long* len;                 // elements
};

template <typename T>
__global__ void ag_pull_kernel(T* __restrict__ dst, PullTable tab, int nseg) {
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

// out[local_off + i] = scale * sum_r grads_r[global_off + i], fp32 accumulation, rank order fixed
// (starting at the local rank's own buffer) so the result is deterministic.
template <typename TIn, typename TOut, bool ACCUM>
__global__ void rs_pull_reduce_kernel(PeerPtrs grads, int world, int rank, TOut* __restrict__ out,
                                      ReduceTable tab, int nseg, float scale) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
    const long long g0 = tab.global_off[s], l0 = tab.local_off[s], n = tab.len[s];
    const bool aligned = ((g0 * sizeof(TIn)) % 16 == 0) && ((l0 * sizeof(TOut)) % 16 == 0) &&
                         ((reinterpret_cast<uintptr_t>(out) % 16) == 0);
    const long long nvec = aligned ? n / 8 : 0;
    for (long long i = tid; i < nvec; i += stride) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int k = 0; k < world; ++k) {
        const int r = (rank + k) % world;
        float v[8];
        load8(reinterpret_cast<const TIn*>(grads.p[r]) + g0 + i * 8, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += v[e];
      }
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

template <typename TIn>
__global__ void rs_pull_adamw_kernel(PeerPtrs grads, int world, int rank, ReduceTable tab, int nseg, float scale,
                                     AdamWArgs a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
    const long long g0 = tab.global_off[s], l0 = tab.local_off[s], n = tab.len[s];
    const bool aligned = ((g0 * sizeof(TIn)) % 16 == 0) && (l0 % 8 == 0);
    const long long nvec = aligned ? n / 8 : 0;
    for (long long i = tid; i < nvec; i += stride) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int k = 0; k < world; ++k) {
        const int r = (rank + k) % world;
        float v[8];
        load8(reinterpret_cast<const TIn*>(grads.p[r]) + g0 + i * 8, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += v[e];
      }
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

// Upper bound on the CTAs of one pull kernel (MFSDP_PEER_MAX_BLOCKS).  The pull kernels run beside the
// GEMMs of the neighbouring block; fewer, longer-lived CTAs leave more issue slots to the tensor kernels.
static long long peer_max_blocks() {
  static long long v = [] {
    const char* e = getenv("MFSDP_PEER_MAX_BLOCKS");
    long long x = e ? atoll(e) : 0;
    return x > 0 ? x : 148LL * 8;
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

MFSDP_API int mfsdp_ag_pull(void* dst, const unsigned long long* src_addr, const long long* dst_off,
                            const long long* len, int nseg, long long max_len, int elem_size, cudaStream_t st) {
  if (nseg <= 0) return 0;
  PullTable tab{src_addr, dst_off, len};
  const dim3 grid = seg_grid(max_len, (16 / elem_size) * 4, nseg);
  switch (elem_size) {
    case 2: ag_pull_kernel<uint16_t><<<grid, 256, 0, st>>>((uint16_t*)dst, tab, nseg); break;
    case 4: ag_pull_kernel<uint32_t><<<grid, 256, 0, st>>>((uint32_t*)dst, tab, nseg); break;
    case 1: ag_pull_kernel<uint8_t><<<grid, 256, 0, st>>>((uint8_t*)dst, tab, nseg); break;
    case 8: ag_pull_kernel<uint64_t><<<grid, 256, 0, st>>>((uint64_t*)dst, tab, nseg); break;
    default: return -2;
  }
  return (int)cudaGetLastError();
}

// grad_ptrs_host[r]: base of rank r's full gradient buffer for this unit (mapped here; own buffer for r == rank).
MFSDP_API int mfsdp_rs_pull_reduce(const unsigned long long* grad_ptrs_host, int world, int rank, void* out,
                                   const long long* global_off, const long long* local_off, const long long* len,
                                   int nseg, long long max_len, int in_is_bf16, int out_is_bf16, int accumulate,
                                   float scale, cudaStream_t st) {
  if (nseg <= 0) return 0;
  if (world <= 0 || world > kMaxPeers) return -2;
  PeerPtrs pp{};
  for (int r = 0; r < world; ++r) pp.p[r] = reinterpret_cast<const void*>(grad_ptrs_host[r]);
  ReduceTable tab{global_off, local_off, len};
  const dim3 grid = seg_grid(max_len, 8, nseg);
#define MFSDP_RS(TI, TO)                                                                                   \
  do {                                                                                                     \
    if (accumulate) rs_pull_reduce_kernel<TI, TO, true><<<grid, 256, 0, st>>>(pp, world, rank, (TO*)out, tab, nseg, scale); \
    else rs_pull_reduce_kernel<TI, TO, false><<<grid, 256, 0, st>>>(pp, world, rank, (TO*)out, tab, nseg, scale);          \
  } while (0)
  if (in_is_bf16 && !out_is_bf16) MFSDP_RS(__nv_bfloat16, float);
  else if (in_is_bf16 && out_is_bf16) MFSDP_RS(__nv_bfloat16, __nv_bfloat16);
  else if (!in_is_bf16 && !out_is_bf16) MFSDP_RS(float, float);
  else return -2;
#undef MFSDP_RS
  return (int)cudaGetLastError();
}

MFSDP_API int mfsdp_rs_pull_adamw(const unsigned long long* grad_ptrs_host, int world, int rank,
                                  const long long* global_off, const long long* local_off, const long long* len,
                                  int nseg, long long max_len, int in_is_bf16, float scale, float* p, float* m,
                                  float* v, void* p_lp, float lr, float beta1, float beta2, float eps,
                                  float weight_decay, int step, cudaStream_t st) {
  if (nseg <= 0) return 0;
  if (world <= 0 || world > kMaxPeers || step < 1) return -2;
  if (((uintptr_t)p % 16) || ((uintptr_t)m % 16) || ((uintptr_t)v % 16) || ((uintptr_t)p_lp % 16)) return -2;
  PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = reinterpret_cast<const void*>(grad_ptrs_host[i]);
  ReduceTable tab{global_off, local_off, len};
  AdamWArgs a{p, m, v, (__nv_bfloat16*)p_lp, lr, beta1, beta2, eps, weight_decay,
              1.f - powf(beta1, (float)step), sqrtf(1.f - powf(beta2, (float)step))};
  const dim3 grid = seg_grid(max_len, 8, nseg);
  if (in_is_bf16) rs_pull_adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(pp, world, rank, tab, nseg, scale, a);
  else rs_pull_adamw_kernel<float><<<grid, 256, 0, st>>>(pp, world, rank, tab, nseg, scale, a);
  return (int)cudaGetLastError();
}
