// Shared helpers of the kernel library: dtype codes, 16-bit float conversions, vector access.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace gb {

// Opt a kernel in to more than 48 KB of dynamic shared memory.  The attribute belongs to the (kernel, device) pair,
// so `mask` (one static word per kernel instantiation) keeps a bit per device: a process that works on several
// GPUs configures each of them on its first launch there.
template <typename KernT>
static inline int smem_opt_in(KernT kern, int bytes, unsigned long long& mask) {
  int dev = 0;
  cudaGetDevice(&dev);
  const unsigned long long bit = 1ull << (dev & 63);
  if (mask & bit) return 0;
  const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return (int)e;
  mask |= bit;
  return 0;
}

// dtype codes of the C ABI (mirrored in genesis_b200/ops/native.py)
enum : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2, DT_F64 = 3, DT_I32 = 4, DT_I64 = 5, DT_U8 = 6, DT_BOOL = 7 };

__device__ __forceinline__ float half_bits_to_float(uint16_t b, int dt) {
  if (dt == DT_BF16) return __uint_as_float((uint32_t)b << 16);
  return __half2float(__ushort_as_half(b));
}
__device__ __forceinline__ uint16_t float_to_half_bits(float v, int dt) {
  if (dt == DT_BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  return __half_as_ushort(__float2half_rn(v));
}
// two floats -> one packed 16-bit pair (a in the low half) with the single packed convert instruction;
// the scalar converts run on the quarter-rate conversion pipe
template <bool BF16>
__device__ __forceinline__ uint32_t pack2c(float a, float b) {
  uint32_t r;
  if (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ uint32_t pack2(float a, float b, int dt) {
  return dt == DT_BF16 ? pack2c<true>(a, b) : pack2c<false>(a, b);
}
__device__ __forceinline__ float load_as_float(const void* p, int dt, size_t i) {
  if (dt == DT_F32) return reinterpret_cast<const float*>(p)[i];
  return half_bits_to_float(reinterpret_cast<const uint16_t*>(p)[i], dt);
}
__device__ __forceinline__ void store_from_float(void* p, int dt, size_t i, float v) {
  if (dt == DT_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<uint16_t*>(p)[i] = float_to_half_bits(v, dt);
}

// Typed traits for templated kernels.
template <typename T> struct Cvt;
template <> struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// 16-byte vector of T
template <typename T> struct alignas(16) Vec16 { T v[16 / sizeof(T)]; static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ Vec16<T> ld16(const T* p) { return *reinterpret_cast<const Vec16<T>*>(p); }
template <typename T>
__device__ __forceinline__ void st16(T* p, const Vec16<T>& v) { *reinterpret_cast<Vec16<T>*>(p) = v; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum / max over up to 1024 threads; `sh` must hold 32 floats. Result in every thread.
__device__ __forceinline__ float block_sum(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : -INFINITY;
  return warp_max(r);
}

#define GB_DISPATCH_FLOAT(dt, T, ...)                                     \
  do {                                                                    \
    if ((dt) == gb::DT_F32) { using T = float; __VA_ARGS__; }             \
    else if ((dt) == gb::DT_F16) { using T = __half; __VA_ARGS__; }       \
    else if ((dt) == gb::DT_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else return -2;                                                       \
  } while (0)

static inline int gb_grid(long long n, int block, int max_blocks = 148 * 16) {
  long long g = (n + block - 1) / block;
  if (g > max_blocks) g = max_blocks;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace gb
