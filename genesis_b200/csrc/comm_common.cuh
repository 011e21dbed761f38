// Shared pieces of the peer-memory communication kernels (comm.cu, moe_comm.cu): the table of peer pointers,
// system-scope flag accesses and the bounded flag barrier.
#pragma once
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace gb {

constexpr int COMM_MAX_WORLD = 16;
constexpr int COMM_MAX_CTAS = 128;
// flag layout inside the symmetric flag page (uint32): [phase(2)][cta(128)][src rank(16)], then the overflow epoch
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

}  // namespace gb
