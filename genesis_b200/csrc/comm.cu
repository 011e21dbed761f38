// Peer-memory communication over NVLink / NVSwitch: symmetric allocations shared through CUDA IPC,
// and the fused gradient all-reduce.  No NCCL call, no cluster-broadcast loads, no switch reductions: plain 16-byte
// loads from / stores to peer-mapped addresses issued by the compute threads themselves.
//
// Fused all-reduce (in place over a symmetric buffer, two-shot):
//   barrier A   "my bucket is complete" to every peer, wait for theirs        (per-CTA flag channels)
//   reduce      rank r owns slice r: 16-byte loads of that slice from all W ranks, fp32 accumulation,
//               x prescale (1/world) x 1/loss_scale (AMP unscale), Inf/NaN check (AMP overflow flag)
//   broadcast   the finished vector is stored into slice r of every rank's buffer
//   barrier B   "my stores are out", wait for the peers' => the whole buffer is final everywhere
// Flags carry a monotonically increasing epoch, so a late peer can never satisfy a later barrier.
// Every wait is bounded (time budget); on expiry the kernel records {code, peer, phase, epoch} in
// `status` and returns, leaving the context usable.
// Reference counterpart: ncclAllReduce per parameter + a divide kernel, genesis/nn/parallel.py:108-117.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace gb {

constexpr int COMM_MAX_WORLD = 16;
constexpr int COMM_MAX_CTAS = 64;
// flag layout inside the symmetric flag page (uint32): [phase(2)][cta(64)][src rank(16)], then the overflow epoch
constexpr int COMM_FLAG_WORDS = 2 * COMM_MAX_CTAS * COMM_MAX_WORLD;
constexpr int COMM_FOUND_SLOT = COMM_FLAG_WORDS;

struct PeerTable { void* ptr[COMM_MAX_WORLD]; };

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Signal every peer and wait for every peer on this CTA's channel of `phase`. Returns false on expiry.
__device__ __forceinline__ bool peer_barrier(const PeerTable& flags, int rank, int world, int phase, uint32_t epoch,
                                             unsigned long long budget_ns, int* status, int* s_fail) {
  __syncthreads();
  if (threadIdx.x < world) {
    const int peer = threadIdx.x;
    const int slot = (phase * COMM_MAX_CTAS + blockIdx.x) * COMM_MAX_WORLD;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(flags.ptr[peer]) + slot + rank, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.ptr[rank]) + slot + peer;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > budget_ns) {
        *s_fail = 1;
        report_error(status, GB_ERR_FLAG_TIMEOUT, peer, phase);
        if (status != nullptr) status[3] = (int)epoch;
        break;
      }
    }
  }
  __syncthreads();
  return *s_fail == 0;
}

template <typename T>
__global__ void __launch_bounds__(512)
allreduce_fused_kernel(PeerTable bufs, PeerTable flags, long long offset_elems, long long n, int rank, int world,
                       uint32_t epoch, float prescale, const float* __restrict__ loss_scale, int scale_is_reciprocal,
                       float* __restrict__ found_inf, unsigned long long budget_ns, int* __restrict__ status) {
  __shared__ int s_fail;
  __shared__ int s_bad;
  constexpr int V = Vec16<T>::N;
  if (threadIdx.x == 0) { s_fail = 0; s_bad = 0; }
  if (!peer_barrier(flags, rank, world, 0, epoch, budget_ns, status, &s_fail)) return;

  float scale = prescale;
  if (loss_scale != nullptr) scale *= scale_is_reciprocal ? 1.f / *loss_scale : *loss_scale;
  const long long nvec = n / V;                       // n is padded by the caller to world * V
  const long long per = nvec / world;
  const long long v0 = (long long)rank * per, v1 = (rank == world - 1) ? nvec : v0 + per;
  bool bad = false;
  // NVLink round trips are microseconds: keep UNR x world 16-byte loads in flight per thread
  constexpr int UNR = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < v1; i0 += stride * UNR) {
    float acc[UNR][V];
#pragma unroll
    for (int u = 0; u < UNR; ++u)
#pragma unroll
      for (int j = 0; j < V; ++j) acc[u][j] = 0.f;
    for (int p = 0; p < world; ++p) {
      const int src = (rank + p) % world;              // stagger peers so links are loaded evenly
      const T* base = reinterpret_cast<const T*>(bufs.ptr[src]) + offset_elems;
      uint4 raw[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long i = i0 + u * stride;
        if (i < v1) raw[u] = ld_volatile_v4(base + i * V);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        if (i0 + u * stride < v1) {
          const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[u][j] += Cvt<T>::to_f(e[j]);
        }
      }
    }
    Vec16<T> o[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u)
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float r = acc[u][j] * scale;
        if (!isfinite(r) && (i0 + u * stride < v1)) bad = true;
        o[u].v[j] = Cvt<T>::from_f(r);
      }
    for (int p = 0; p < world; ++p) {
      const int dst = (rank + p) % world;
      T* base = reinterpret_cast<T*>(bufs.ptr[dst]) + offset_elems;
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long i = i0 + u * stride;
        if (i < v1) st16(base + i * V, o[u]);
      }
    }
  }
  if (bad) s_bad = 1;
  __syncthreads();
  if (s_bad && threadIdx.x < world && found_inf != nullptr) {
    // tell every rank: this epoch overflowed
    st_release_sys(reinterpret_cast<uint32_t*>(flags.ptr[threadIdx.x]) + COMM_FOUND_SLOT, epoch);
  }
  if (!peer_barrier(flags, rank, world, 1, epoch, budget_ns, status, &s_fail)) return;
  if (found_inf != nullptr && threadIdx.x == 0) {
    if (ld_acquire_sys(reinterpret_cast<const uint32_t*>(flags.ptr[rank]) + COMM_FOUND_SLOT) == epoch)
      *found_inf = 1.f;
  }
}

// A wait on a flag nobody sets: used to exercise the timeout path without any peer.
__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t expect, unsigned long long budget_ns, int* status) {
  const uint64_t t0 = globaltimer_ns();
  while ((int32_t)(ld_acquire_sys(flag) - expect) < 0) {
    if (globaltimer_ns() - t0 > budget_ns) { report_error(status, GB_ERR_FLAG_TIMEOUT, 0, 0); return; }
  }
}

}  // namespace gb

using namespace gb;

// ---- symmetric memory plumbing -------------------------------------------------------------------
extern "C" int gb_symm_alloc(size_t nbytes, void** out) {
  cudaError_t e = cudaMalloc(out, nbytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*out, 0, nbytes);
}
extern "C" int gb_symm_free(void* p) { return (int)cudaFree(p); }
extern "C" int gb_ipc_get_handle(void* p, char* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int gb_ipc_open_handle(const char* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int gb_ipc_close_handle(void* p) { return (int)cudaIpcCloseMemHandle(p); }

// ---- fused all-reduce ------------------------------------------------------------------------------
// bufs / flags: arrays of `world` device pointers (this rank's own pointer at index `rank`).
// n elements starting at element `offset_elems` of every rank's buffer; n must be a multiple of
// world * (16 / elem size) and the start 16-byte aligned.
extern "C" int gb_allreduce_fused(void* const* bufs, void* const* flags, long long offset_elems, long long n,
                                  int rank, int world, unsigned int epoch, float prescale, const float* loss_scale,
                                  int scale_is_reciprocal, float* found_inf, int dt, int ctas,
                                  unsigned long long budget_ns, int* status, cudaStream_t st) {
  if (world > COMM_MAX_WORLD || world < 1) return -2;
  if (ctas > COMM_MAX_CTAS) ctas = COMM_MAX_CTAS;
  if (ctas < 1) ctas = 1;
  PeerTable tb, tf;
  for (int i = 0; i < world; ++i) { tb.ptr[i] = bufs[i]; tf.ptr[i] = flags[i]; }
  GB_DISPATCH_FLOAT(dt, T, {
    if (n % (world * Vec16<T>::N) != 0) return -3;
    allreduce_fused_kernel<T><<<ctas, 512, 0, st>>>(tb, tf, offset_elems, n, rank, world, epoch, prescale,
                                                    loss_scale, scale_is_reciprocal, found_inf, budget_ns, status);
  });
  return (int)cudaGetLastError();
}

extern "C" int gb_wait_flag(const unsigned int* flag, unsigned int expect, unsigned long long budget_ns, int* status,
                            cudaStream_t st) {
  wait_flag_kernel<<<1, 1, 0, st>>>(flag, expect, budget_ns, status);
  return (int)cudaGetLastError();
}
