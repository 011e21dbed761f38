// Reductions (sum / max / min, fp32 accumulation) over a tensor viewed as [outer, red, inner]:
//   inner == 1  -> row kernel (one warp or one block per row, 128-bit loads)
//   otherwise   -> column kernel (threads own inner positions, loop over red; split + second pass
//                  when red is long and outer*inner is small)
// Full reductions are two-stage and deterministic (no atomics).
// Reference counterpart: genesis/ops/cuda/reduction_ops.py:97-753.
#include "common.cuh"

namespace gb {

enum RedOp : int { R_SUM = 0, R_MAX = 1, R_MIN = 2 };

__device__ __forceinline__ float red_init(int op) { return op == R_SUM ? 0.f : (op == R_MAX ? -INFINITY : INFINITY); }
__device__ __forceinline__ float red_comb(int op, float a, float b) {
  return op == R_SUM ? a + b : (op == R_MAX ? fmaxf(a, b) : fminf(a, b));
}
__device__ __forceinline__ float warp_red(int op, float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = red_comb(op, v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// one block per row; out[row] = scale * reduce(x[row, :])
template <typename T, typename O>
__global__ void reduce_rows_kernel(const T* __restrict__ x, O* __restrict__ out, long long rows, long long cols,
                                   int op, float scale) {
  __shared__ float sh[32];
  constexpr int V = Vec16<T>::N;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* p = x + row * cols;
    float acc = red_init(op);
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(p) & 15) == 0);
    long long done = 0;
    if (vec_ok) {
      const long long nv = cols / V;
      for (long long i = threadIdx.x; i < nv; i += blockDim.x) {
        Vec16<T> a = ld16(p + i * V);
#pragma unroll
        for (int j = 0; j < V; ++j) acc = red_comb(op, acc, Cvt<T>::to_f(a.v[j]));
      }
      done = nv * V;
    }
    for (long long i = done + threadIdx.x; i < cols; i += blockDim.x) acc = red_comb(op, acc, Cvt<T>::to_f(p[i]));
    acc = warp_red(op, acc);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) sh[w] = acc;
    __syncthreads();
    if (w == 0) {
      float r = lane < nw ? sh[lane] : red_init(op);
      r = warp_red(op, r);
      if (lane == 0) out[row] = Cvt<O>::from_f(r * scale);
    }
  }
}

// x viewed as [outer, red, inner]; each thread owns one (outer, inner) position of a red-split
template <typename T, typename O>
__global__ void reduce_mid_kernel(const T* __restrict__ x, O* __restrict__ out, long long outer, long long red,
                                  long long inner, int splits, int op, float scale) {
  const long long col = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long o = blockIdx.y;
  const int sp = blockIdx.z;
  if (col >= inner) return;
  const long long chunk = (red + splits - 1) / splits;
  const long long r0 = sp * chunk, r1 = (r0 + chunk < red) ? r0 + chunk : red;
  const T* p = x + o * red * inner + col;
  float acc = red_init(op);
#pragma unroll 8
  for (long long r = r0; r < r1; ++r) acc = red_comb(op, acc, Cvt<T>::to_f(p[r * inner]));
  out[((long long)sp * outer + o) * inner + col] = Cvt<O>::from_f(splits == 1 ? acc * scale : acc);
}

// Vector form of the column reduction (inner a multiple of 16 bytes, 16-byte aligned base): a CTA is 8 row lanes x 32
// column lanes, a thread reads 16 bytes of a row (a warp reads 512 contiguous bytes), the row lanes stride over the
// reduced extent and are combined through shared memory at the end.
template <typename T, typename O>
__global__ void __launch_bounds__(256)
reduce_mid_vec_kernel(const T* __restrict__ x, O* __restrict__ out, long long outer, long long red, long long inner,
                      int splits, int op, float scale) {
  constexpr int V = Vec16<T>::N;
  __shared__ float sh[8][32 * V + 1];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long col = ((long long)blockIdx.x * 32 + tx) * V;
  const long long o = blockIdx.y;
  const int sp = blockIdx.z;
  const long long chunk = (red + splits - 1) / splits;
  const long long r0 = sp * chunk, r1 = (r0 + chunk < red) ? r0 + chunk : red;
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = red_init(op);
  if (col < inner) {
    const T* p = x + o * red * inner + col;
#pragma unroll 4
    for (long long r = r0 + ty; r < r1; r += 8) {
      const Vec16<T> a = ld16(p + r * inner);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = red_comb(op, acc[j], Cvt<T>::to_f(a.v[j]));
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) sh[ty][tx * V + j] = acc[j];
  __syncthreads();
  for (int c = threadIdx.x; c < 32 * V; c += 256) {
    const long long gc = (long long)blockIdx.x * 32 * V + c;
    if (gc >= inner) continue;
    float r = sh[0][c];
#pragma unroll
    for (int q = 1; q < 8; ++q) r = red_comb(op, r, sh[q][c]);
    out[((long long)sp * outer + o) * inner + gc] = Cvt<O>::from_f(splits == 1 ? r * scale : r);
  }
}

}  // namespace gb

using namespace gb;

template <typename T>
static int rows_out(const void* x, void* out, long long rows, long long cols, int op, float scale, int odt,
                    cudaStream_t st) {
  const int block = cols >= 4096 ? 512 : (cols >= 512 ? 256 : 64);
  const int grid = (int)(rows < 148 * 32 ? rows : 148 * 32);
  if (odt == DT_F32) reduce_rows_kernel<T, float><<<grid, block, 0, st>>>((const T*)x, (float*)out, rows, cols, op, scale);
  else if (odt == DT_F16) reduce_rows_kernel<T, __half><<<grid, block, 0, st>>>((const T*)x, (__half*)out, rows, cols, op, scale);
  else if (odt == DT_BF16) reduce_rows_kernel<T, __nv_bfloat16><<<grid, block, 0, st>>>((const T*)x, (__nv_bfloat16*)out, rows, cols, op, scale);
  else return -2;
  return (int)cudaGetLastError();
}

extern "C" int gb_reduce_rows(int op, const void* x, void* out, long long rows, long long cols, float scale,
                              int idt, int odt, cudaStream_t st) {
  if (rows == 0) return 0;
  GB_DISPATCH_FLOAT(idt, T, return rows_out<T>(x, out, rows, cols, op, scale, odt, st));
  return -2;
}

template <typename T>
static int mid_out(const void* x, void* out, long long outer, long long red, long long inner, int splits, int op,
                   float scale, int odt, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  if (inner % V == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && red >= 16) {
    dim3 vgrid((unsigned)((inner + 32 * V - 1) / (32 * V)), (unsigned)outer, (unsigned)splits);
    if (odt == DT_F32) reduce_mid_vec_kernel<T, float><<<vgrid, 256, 0, st>>>((const T*)x, (float*)out, outer, red, inner, splits, op, scale);
    else if (odt == DT_F16) reduce_mid_vec_kernel<T, __half><<<vgrid, 256, 0, st>>>((const T*)x, (__half*)out, outer, red, inner, splits, op, scale);
    else if (odt == DT_BF16) reduce_mid_vec_kernel<T, __nv_bfloat16><<<vgrid, 256, 0, st>>>((const T*)x, (__nv_bfloat16*)out, outer, red, inner, splits, op, scale);
    else return -2;
    return (int)cudaGetLastError();
  }
  dim3 grid((unsigned)((inner + 127) / 128), (unsigned)outer, (unsigned)splits);
  if (odt == DT_F32) reduce_mid_kernel<T, float><<<grid, 128, 0, st>>>((const T*)x, (float*)out, outer, red, inner, splits, op, scale);
  else if (odt == DT_F16) reduce_mid_kernel<T, __half><<<grid, 128, 0, st>>>((const T*)x, (__half*)out, outer, red, inner, splits, op, scale);
  else if (odt == DT_BF16) reduce_mid_kernel<T, __nv_bfloat16><<<grid, 128, 0, st>>>((const T*)x, (__nv_bfloat16*)out, outer, red, inner, splits, op, scale);
  else return -2;
  return (int)cudaGetLastError();
}

// out: [splits, outer, inner] when splits > 1 (fp32 partials; caller reduces them with a second call
// where red = splits), else [outer, inner].
extern "C" int gb_reduce_mid(int op, const void* x, void* out, long long outer, long long red, long long inner,
                             int splits, float scale, int idt, int odt, cudaStream_t st) {
  if (outer == 0 || inner == 0) return 0;
  if (outer > 65535 || splits > 65535) return -2;
  GB_DISPATCH_FLOAT(idt, T, return mid_out<T>(x, out, outer, red, inner, splits, op, scale, odt, st));
  return -2;
}
