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
#include "comm_common.cuh"

namespace gb {

// 256 threads and at most 80 registers: 20 K registers per CTA, which fit beside a resident GEMM CTA (43.5 K of the
// 64 K), so the reduction runs on SMs that backward keeps busy instead of taking SMs away from it.
// Epoch kept on the device (`ctr[0]` last finished epoch, `ctr[1]` CTAs of the running launch that are done): every
// CTA of a launch reads the same value because ctr[0] only moves once all of them have passed through here, and
// launches on one stream are ordered.  With it the launch takes nothing step-dependent by value, so a CUDA graph
// that contains the all-reduce can be replayed; all ranks issue the same launches, so their counters agree.
__device__ __forceinline__ void epoch_publish(uint32_t* ctr, uint32_t epoch) {
  if (ctr == nullptr || threadIdx.x != 0) return;
  __threadfence();
  if (atomicAdd(ctr + 1, 1u) == gridDim.x - 1) {
    ctr[1] = 0;
    __threadfence();
    *reinterpret_cast<volatile uint32_t*>(ctr) = epoch;
  }
}

// Reduce phase shared by both all-reduce kernels: this rank's slice [v0, v1) of 16-byte vectors is summed over all
// ranks in fp32.  NVLink round trips take microseconds, so what matters is how many loads a thread keeps in flight:
// with the world size known at compile time the loads of ALL peers for a batch of vectors are issued before the
// first one is consumed (8 vectors in flight per thread for any world size: UNR = 8 / W batches), instead of
// peer after peer.  `emit(i, acc)` receives the fp32 sums of vector i.
template <typename T, int W, typename Emit>
__device__ __forceinline__ void reduce_slice_w(const PeerTable& bufs, long long offset_elems, int rank, long long v0,
                                               long long v1, Emit emit) {
  constexpr int V = Vec16<T>::N;
  constexpr int UNR = 8 / W;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const T* base[W];
#pragma unroll
  for (int p = 0; p < W; ++p) base[p] = reinterpret_cast<const T*>(bufs.ptr[(rank + p) % W]) + offset_elems;
  for (long long i0 = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < v1; i0 += stride * UNR) {
    uint4 raw[UNR][W];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long i = i0 + u * stride;
#pragma unroll
      for (int p = 0; p < W; ++p)
        if (i < v1) raw[u][p] = ld_volatile_v4(base[p] + i * V);
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long i = i0 + u * stride;
      if (i >= v1) continue;
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
#pragma unroll
      for (int p = 0; p < W; ++p) {
        const T* e = reinterpret_cast<const T*>(&raw[u][p]);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += Cvt<T>::to_f(e[j]);
      }
      emit(i, acc);
    }
  }
}

// any world size: peer after peer, four vectors in flight per peer
template <typename T, typename Emit>
__device__ __forceinline__ void reduce_slice_any(const PeerTable& bufs, long long offset_elems, int rank, int world,
                                                 long long v0, long long v1, Emit emit) {
  constexpr int V = Vec16<T>::N;
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
#pragma unroll
    for (int u = 0; u < UNR; ++u)
      if (i0 + u * stride < v1) emit(i0 + u * stride, acc[u]);
  }
}

template <typename T, typename Emit>
__device__ __forceinline__ void reduce_slice(const PeerTable& bufs, long long offset_elems, int rank, int world,
                                             long long v0, long long v1, Emit emit) {
  if (world == 8) reduce_slice_w<T, 8>(bufs, offset_elems, rank, v0, v1, emit);
  else if (world == 4) reduce_slice_w<T, 4>(bufs, offset_elems, rank, v0, v1, emit);
  else if (world == 2) reduce_slice_w<T, 2>(bufs, offset_elems, rank, v0, v1, emit);
  else reduce_slice_any<T>(bufs, offset_elems, rank, world, v0, v1, emit);
}

template <typename T>
__global__ void __launch_bounds__(256, 3)
allreduce_fused_kernel(PeerTable bufs, PeerTable flags, long long offset_elems, long long n, int rank, int world,
                       uint32_t epoch, float prescale, const float* __restrict__ loss_scale, int scale_is_reciprocal,
                       float* __restrict__ found_inf, unsigned long long budget_ns, int* __restrict__ status,
                       uint32_t* __restrict__ epoch_ctr) {
  __shared__ int s_fail;
  __shared__ int s_bad;
  constexpr int V = Vec16<T>::N;
  if (threadIdx.x == 0) { s_fail = 0; s_bad = 0; }
  if (epoch_ctr != nullptr) epoch = *reinterpret_cast<volatile uint32_t*>(epoch_ctr) + 1;
  if (!peer_barrier(flags, rank, world, 0, epoch, budget_ns, status, &s_fail)) {
    epoch_publish(epoch_ctr, epoch);
    return;
  }

  float scale = prescale;
  if (loss_scale != nullptr) scale *= scale_is_reciprocal ? 1.f / *loss_scale : *loss_scale;
  const long long nvec = n / V;                       // n is padded by the caller to world * V
  const long long per = nvec / world;
  const long long v0 = (long long)rank * per, v1 = (rank == world - 1) ? nvec : v0 + per;
  bool bad = false;
  reduce_slice<T>(bufs, offset_elems, rank, world, v0, v1, [&](long long i, const float* acc) {
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float r = acc[j] * scale;
      if (!isfinite(r)) bad = true;
      o.v[j] = Cvt<T>::from_f(r);
    }
    for (int p = 0; p < world; ++p) {
      const int dst = (rank + p) % world;
      st16(reinterpret_cast<T*>(bufs.ptr[dst]) + offset_elems + i * V, o);
    }
  });
  if (bad) s_bad = 1;
  __syncthreads();
  if (s_bad && threadIdx.x < world && found_inf != nullptr) {
    // tell every rank: this epoch overflowed
    st_release_sys(reinterpret_cast<uint32_t*>(flags.ptr[threadIdx.x]) + COMM_FOUND_SLOT, epoch);
  }
  if (!peer_barrier(flags, rank, world, 1, epoch, budget_ns, status, &s_fail)) {
    epoch_publish(epoch_ctr, epoch);
    return;
  }
  if (found_inf != nullptr && threadIdx.x == 0) {
    if (ld_acquire_sys(reinterpret_cast<const uint32_t*>(flags.ptr[rank]) + COMM_FOUND_SLOT) == epoch)
      *found_inf = 1.f;
  }
  epoch_publish(epoch_ctr, epoch);
}

// Low-precision wire format: the gradients cross NVLink as 16-bit values (half the bytes of the fp32 form) while the
// caller keeps float32 gradients; both casts are phases of this kernel:
//   pack        local float32 bucket `grad` -> this rank's 16-bit symmetric buffer (round to nearest)
//   barrier A   every rank's 16-bit buffer is complete
//   reduce      rank r pulls slice r of all W buffers (16-byte loads of 8 values), accumulates in fp32, multiplies by
//               prescale (1/world; NOT yet by 1/loss_scale, so fp16 values keep their scaled range), checks Inf/NaN,
//               rounds to 16 bits and stores the result into slice r of every rank's buffer
//   barrier B   all slices of the local buffer are final
//   cast        the whole local 16-bit buffer -> `grad` (float32, in place) times 1/loss_scale
template <typename T>
__global__ void __launch_bounds__(256, 3)
allreduce_wire_kernel(PeerTable bufs, PeerTable flags, long long n, float* __restrict__ grad, int rank, int world,
                      uint32_t epoch, float prescale, const float* __restrict__ loss_scale, int scale_is_reciprocal,
                      float* __restrict__ found_inf, unsigned long long budget_ns, int* __restrict__ status,
                      uint32_t* __restrict__ epoch_ctr) {
  __shared__ int s_fail;
  __shared__ int s_bad;
  constexpr int V = Vec16<T>::N;                       // 8 values per 16-byte vector
  if (threadIdx.x == 0) { s_fail = 0; s_bad = 0; }
  if (epoch_ctr != nullptr) epoch = *reinterpret_cast<volatile uint32_t*>(epoch_ctr) + 1;
  const long long nvec = n / V;                        // n is padded by the caller to world * V
  const long long stride = (long long)gridDim.x * blockDim.x;
  {
    // pack phase (the barrier's system-scope fence and release publish these stores to the peers)
    T* mine = reinterpret_cast<T*>(bufs.ptr[rank]);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
      const float4 lo = *reinterpret_cast<const float4*>(grad + i * V);
      const float4 hi = *reinterpret_cast<const float4*>(grad + i * V + 4);
      Vec16<T> o;
      o.v[0] = Cvt<T>::from_f(lo.x); o.v[1] = Cvt<T>::from_f(lo.y); o.v[2] = Cvt<T>::from_f(lo.z);
      o.v[3] = Cvt<T>::from_f(lo.w); o.v[4] = Cvt<T>::from_f(hi.x); o.v[5] = Cvt<T>::from_f(hi.y);
      o.v[6] = Cvt<T>::from_f(hi.z); o.v[7] = Cvt<T>::from_f(hi.w);
      st16(mine + i * V, o);
    }
  }
  if (!peer_barrier(flags, rank, world, 0, epoch, budget_ns, status, &s_fail)) {
    epoch_publish(epoch_ctr, epoch);
    return;
  }
  const long long per = nvec / world;
  const long long v0 = (long long)rank * per, v1 = (rank == world - 1) ? nvec : v0 + per;
  bool bad = false;
  reduce_slice<T>(bufs, 0, rank, world, v0, v1, [&](long long i, const float* acc) {
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float r = acc[j] * prescale;
      if (!isfinite(r)) bad = true;
      o.v[j] = Cvt<T>::from_f(r);
    }
    for (int p = 0; p < world; ++p) {
      const int dst = (rank + p) % world;
      st16(reinterpret_cast<T*>(bufs.ptr[dst]) + i * V, o);
    }
  });
  if (bad) s_bad = 1;
  __syncthreads();
  if (s_bad && threadIdx.x < world && found_inf != nullptr)
    st_release_sys(reinterpret_cast<uint32_t*>(flags.ptr[threadIdx.x]) + COMM_FOUND_SLOT, epoch);
  if (!peer_barrier(flags, rank, world, 1, epoch, budget_ns, status, &s_fail)) {
    epoch_publish(epoch_ctr, epoch);
    return;
  }
  if (found_inf != nullptr && threadIdx.x == 0) {
    if (ld_acquire_sys(reinterpret_cast<const uint32_t*>(flags.ptr[rank]) + COMM_FOUND_SLOT) == epoch)
      *found_inf = 1.f;
  }
  // cast phase: peers wrote their slices with plain stores that barrier B made visible; read them past L1
  float inv = 1.f;
  if (loss_scale != nullptr) inv = scale_is_reciprocal ? 1.f / *loss_scale : *loss_scale;
  const T* mine = reinterpret_cast<const T*>(bufs.ptr[rank]);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const uint4 raw = ld_volatile_v4(mine + i * V);
    const T* e = reinterpret_cast<const T*>(&raw);
    float4 lo, hi;
    lo.x = Cvt<T>::to_f(e[0]) * inv; lo.y = Cvt<T>::to_f(e[1]) * inv;
    lo.z = Cvt<T>::to_f(e[2]) * inv; lo.w = Cvt<T>::to_f(e[3]) * inv;
    hi.x = Cvt<T>::to_f(e[4]) * inv; hi.y = Cvt<T>::to_f(e[5]) * inv;
    hi.z = Cvt<T>::to_f(e[6]) * inv; hi.w = Cvt<T>::to_f(e[7]) * inv;
    *reinterpret_cast<float4*>(grad + i * V) = lo;
    *reinterpret_cast<float4*>(grad + i * V + 4) = hi;
  }
  epoch_publish(epoch_ctr, epoch);
}

// ------------------------------------------------------------------------------------------------
// Pull-style data movement: all-gather, broadcast and all-to-all are the same kernel.  Every rank has
// staged what it sends in its symmetric buffer and publishes, per destination rank, where that rank's
// part starts and how long it is (two tables in its flag page).  After barrier A each rank reads the
// entries addressed to it and copies the parts out of the peers' buffers into LOCAL memory with plain
// peer loads; barrier B tells the owners that their buffers may be reused.
// ------------------------------------------------------------------------------------------------
constexpr int COMM_META_WORD = COMM_FLAG_WORDS + 64;     // uint32 index of the tables inside the flag page

struct SendTable { long long off[COMM_MAX_WORLD]; long long len[COMM_MAX_WORLD]; };   // bytes, per destination
struct RecvTable { long long off[COMM_MAX_WORLD]; };                                   // bytes, per source

__device__ __forceinline__ long long ld_volatile_s64(const long long* p) {
  long long v;
  asm volatile("ld.volatile.global.s64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(512)
peer_pull_kernel(PeerTable bufs, PeerTable flags, SendTable send, RecvTable recv, uint8_t* __restrict__ out,
                 int rank, int world, uint32_t epoch, unsigned long long budget_ns, int* __restrict__ status) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  // every CTA publishes the same tables before its own signal: whichever channel a peer waits on, the
  // tables are visible once that channel's flag is
  long long* my_meta = reinterpret_cast<long long*>(reinterpret_cast<uint32_t*>(flags.ptr[rank]) + COMM_META_WORD);
  if (threadIdx.x < world) {
    my_meta[threadIdx.x] = send.off[threadIdx.x];
    my_meta[COMM_MAX_WORLD + threadIdx.x] = send.len[threadIdx.x];
  }
  if (!peer_barrier(flags, rank, world, 0, epoch, budget_ns, status, &s_fail)) return;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  for (int p = 0; p < world; ++p) {
    const int src = (rank + p) % world;
    const long long* meta = reinterpret_cast<const long long*>(reinterpret_cast<const uint32_t*>(flags.ptr[src]) + COMM_META_WORD);
    const long long off = ld_volatile_s64(meta + rank);
    const long long len = ld_volatile_s64(meta + COMM_MAX_WORLD + rank);
    if (len <= 0) continue;
    const uint8_t* from = reinterpret_cast<const uint8_t*>(bufs.ptr[src]) + off;
    uint8_t* to = out + recv.off[src];
    if (((reinterpret_cast<uintptr_t>(from) | reinterpret_cast<uintptr_t>(to) | (uintptr_t)len) & 15) == 0) {
      const long long nv = len >> 4;
      constexpr int UNR = 4;
      for (long long i0 = tid; i0 < nv; i0 += nthreads * UNR) {
        uint4 v[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u)
          if (i0 + u * nthreads < nv) v[u] = ld_volatile_v4(from + ((i0 + u * nthreads) << 4));
#pragma unroll
        for (int u = 0; u < UNR; ++u)
          if (i0 + u * nthreads < nv) *reinterpret_cast<uint4*>(to + ((i0 + u * nthreads) << 4)) = v[u];
      }
    } else {
      for (long long i = tid; i < len; i += nthreads) to[i] = *reinterpret_cast<const volatile uint8_t*>(from + i);
    }
  }
  peer_barrier(flags, rank, world, 1, epoch, budget_ns, status, &s_fail);
}

// Reduce-scatter: every rank staged world x n elements; rank r sums slice r of all peers into local `out`.
template <typename T>
__global__ void __launch_bounds__(512)
peer_reduce_scatter_kernel(PeerTable bufs, PeerTable flags, T* __restrict__ out, long long n, int rank, int world,
                           uint32_t epoch, float scale, unsigned long long budget_ns, int* __restrict__ status) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  if (!peer_barrier(flags, rank, world, 0, epoch, budget_ns, status, &s_fail)) return;
  constexpr int V = Vec16<T>::N;
  const long long nvec = n / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    for (int p = 0; p < world; ++p) {
      const int src = (rank + p) % world;
      const uint4 raw = ld_volatile_v4(reinterpret_cast<const T*>(bufs.ptr[src]) + (long long)rank * n + i * V);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += Cvt<T>::to_f(e[j]);
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(acc[j] * scale);
    st16(out + i * V, o);
  }
  peer_barrier(flags, rank, world, 1, epoch, budget_ns, status, &s_fail);
}

__global__ void peer_barrier_kernel(PeerTable flags, int rank, int world, uint32_t epoch,
                                    unsigned long long budget_ns, int* __restrict__ status) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  peer_barrier(flags, rank, world, 0, epoch, budget_ns, status, &s_fail);
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
                                  unsigned long long budget_ns, int* status, unsigned int* epoch_ctr,
                                  cudaStream_t st) {
  if (world > COMM_MAX_WORLD || world < 1) return -2;
  if (ctas > COMM_MAX_CTAS) ctas = COMM_MAX_CTAS;
  if (ctas < 1) ctas = 1;
  PeerTable tb, tf;
  for (int i = 0; i < world; ++i) { tb.ptr[i] = bufs[i]; tf.ptr[i] = flags[i]; }
  GB_DISPATCH_FLOAT(dt, T, {
    if (n % (world * Vec16<T>::N) != 0) return -3;
    allreduce_fused_kernel<T><<<ctas, 256, 0, st>>>(tb, tf, offset_elems, n, rank, world, epoch, prescale,
                                                    loss_scale, scale_is_reciprocal, found_inf, budget_ns, status,
                                                    epoch_ctr);
  });
  return (int)cudaGetLastError();
}

// 16-bit wire form: `out` is this rank's float32 gradient bucket (n elements, 16-byte aligned; reduced in place),
// `bufs` the ranks' 16-bit symmetric staging buffers of n elements (n a multiple of world * 8).  dt: DT_F16 / DT_BF16.
extern "C" int gb_allreduce_wire(void* const* bufs, void* const* flags, long long n, float* out, int rank, int world,
                                 unsigned int epoch, float prescale, const float* loss_scale,
                                 int scale_is_reciprocal, float* found_inf, int dt, int ctas,
                                 unsigned long long budget_ns, int* status, unsigned int* epoch_ctr,
                                 cudaStream_t st) {
  if (world > COMM_MAX_WORLD || world < 1) return -2;
  if (dt != DT_F16 && dt != DT_BF16) return -4;
  if (n % (world * 8) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0) return -3;
  if (ctas > COMM_MAX_CTAS) ctas = COMM_MAX_CTAS;
  if (ctas < 1) ctas = 1;
  PeerTable tb, tf;
  for (int i = 0; i < world; ++i) { tb.ptr[i] = bufs[i]; tf.ptr[i] = flags[i]; }
  if (dt == DT_BF16)
    allreduce_wire_kernel<__nv_bfloat16><<<ctas, 256, 0, st>>>(tb, tf, n, out, rank, world, epoch, prescale,
                                                               loss_scale, scale_is_reciprocal, found_inf, budget_ns,
                                                               status, epoch_ctr);
  else
    allreduce_wire_kernel<__half><<<ctas, 256, 0, st>>>(tb, tf, n, out, rank, world, epoch, prescale, loss_scale,
                                                        scale_is_reciprocal, found_inf, budget_ns, status, epoch_ctr);
  return (int)cudaGetLastError();
}

extern "C" int gb_wait_flag(const unsigned int* flag, unsigned int expect, unsigned long long budget_ns, int* status,
                            cudaStream_t st) {
  wait_flag_kernel<<<1, 1, 0, st>>>(flag, expect, budget_ns, status);
  return (int)cudaGetLastError();
}

// ---- pull collectives ------------------------------------------------------------------------------
// send_off / send_len: where in THIS rank's symmetric buffer the part for destination d starts and its length;
// recv_off: where in `out` (local memory) the part coming from source s goes.  All in bytes.
extern "C" int gb_peer_pull(void* const* bufs, void* const* flags, const long long* send_off,
                            const long long* send_len, const long long* recv_off, void* out, int rank, int world,
                            unsigned int epoch, int ctas, unsigned long long budget_ns, int* status,
                            cudaStream_t st) {
  if (world > COMM_MAX_WORLD || world < 1) return -2;
  if (ctas > COMM_MAX_CTAS) ctas = COMM_MAX_CTAS;
  if (ctas < 1) ctas = 1;
  PeerTable tb, tf;
  SendTable sd;
  RecvTable rv;
  for (int i = 0; i < world; ++i) {
    tb.ptr[i] = bufs[i]; tf.ptr[i] = flags[i];
    sd.off[i] = send_off[i]; sd.len[i] = send_len[i]; rv.off[i] = recv_off[i];
  }
  peer_pull_kernel<<<ctas, 512, 0, st>>>(tb, tf, sd, rv, reinterpret_cast<uint8_t*>(out), rank, world, epoch,
                                         budget_ns, status);
  return (int)cudaGetLastError();
}

// out[n] = scale * sum over ranks of (their buffer)[rank * n .. rank * n + n); n a multiple of 16 bytes.
extern "C" int gb_peer_reduce_scatter(void* const* bufs, void* const* flags, void* out, long long n, int rank,
                                      int world, unsigned int epoch, float scale, int dt, int ctas,
                                      unsigned long long budget_ns, int* status, cudaStream_t st) {
  if (world > COMM_MAX_WORLD || world < 1) return -2;
  if (ctas > COMM_MAX_CTAS) ctas = COMM_MAX_CTAS;
  if (ctas < 1) ctas = 1;
  PeerTable tb, tf;
  for (int i = 0; i < world; ++i) { tb.ptr[i] = bufs[i]; tf.ptr[i] = flags[i]; }
  GB_DISPATCH_FLOAT(dt, T, {
    if (n % Vec16<T>::N != 0) return -3;
    peer_reduce_scatter_kernel<T><<<ctas, 512, 0, st>>>(tb, tf, reinterpret_cast<T*>(out), n, rank, world, epoch,
                                                        scale, budget_ns, status);
  });
  return (int)cudaGetLastError();
}

extern "C" int gb_peer_barrier(void* const* flags, int rank, int world, unsigned int epoch,
                               unsigned long long budget_ns, int* status, cudaStream_t st) {
  if (world > COMM_MAX_WORLD || world < 1) return -2;
  PeerTable tf;
  for (int i = 0; i < world; ++i) tf.ptr[i] = flags[i];
  peer_barrier_kernel<<<1, 32, 0, st>>>(tf, rank, world, epoch, budget_ns, status);
  return (int)cudaGetLastError();
}
