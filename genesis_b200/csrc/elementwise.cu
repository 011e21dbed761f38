// Elementwise kernel family: binary (tensor-tensor with <=4-D broadcasting, tensor-scalar), unary
// forward/backward, compare, where, clamp, cast, fill, strided copy, axpy.  All math in fp32;
// storage fp32 / fp16 / bf16.  Contiguous same-shape inputs take the 128-bit vectorised path.
// Reference counterparts: genesis/ops/cuda/basic_ops.py, strided_ops.py, comparison_ops.py and the
// copy kernels of genesis/backends/cuda.py (about 80 Triton kernels).
#include "common.cuh"

namespace gb {

enum BinOp : int { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_MAX, B_MIN, B_RSUB, B_RDIV, B_POW, B_RPOW };
enum UnOp : int { U_NEG = 0, U_EXP, U_LOG, U_SQRT, U_RSQRT, U_SIN, U_COS, U_TANH, U_SIGMOID, U_RELU, U_ABS,
                  U_SIGN, U_SILU, U_GELU, U_RECIP };
enum CmpOp : int { C_EQ = 0, C_NE, C_LT, C_LE, C_GT, C_GE };

__device__ __forceinline__ float bin_apply(int op, float a, float b) {
  switch (op) {
    case B_ADD: return a + b;
    case B_SUB: return a - b;
    case B_MUL: return a * b;
    case B_DIV: return a / b;
    case B_MAX: return fmaxf(a, b);
    case B_MIN: return fminf(a, b);
    case B_RSUB: return b - a;
    case B_RDIV: return b / a;
    case B_POW: return powf(a, b);
    default: return powf(b, a);
  }
}

__device__ __forceinline__ float un_apply(int op, float x) {
  switch (op) {
    case U_NEG: return -x;
    case U_EXP: return expf(x);
    case U_LOG: return logf(x);
    case U_SQRT: return sqrtf(x);
    case U_RSQRT: return rsqrtf(x);
    case U_SIN: return sinf(x);
    case U_COS: return cosf(x);
    case U_TANH: return tanhf(x);
    case U_SIGMOID: return 1.f / (1.f + expf(-x));
    case U_RELU: return x > 0.f ? x : 0.f;
    case U_ABS: return fabsf(x);
    case U_SIGN: return (x > 0.f) - (x < 0.f);
    case U_SILU: return x / (1.f + expf(-x));
    case U_GELU: {
      const float c = 0.7978845608028654f;
      return 0.5f * x * (1.f + tanhf(c * (x + 0.044715f * x * x * x)));
    }
    default: return 1.f / x;
  }
}

// derivative times g; `t` is x for ops that differentiate through the input and y for those
// that are cheaper through the output (exp, sqrt, tanh, sigmoid)
__device__ __forceinline__ float un_bwd(int op, float g, float t) {
  switch (op) {
    case U_NEG: return -g;
    case U_EXP: return g * t;
    case U_LOG: return g / t;
    case U_SQRT: return g / (2.f * t);
    case U_SIN: return g * cosf(t);
    case U_COS: return -g * sinf(t);
    case U_TANH: return g * (1.f - t * t);
    case U_SIGMOID: return g * t * (1.f - t);
    case U_RELU: return t > 0.f ? g : 0.f;
    case U_ABS: return g * ((t > 0.f) - (t < 0.f));
    case U_SILU: { float s = 1.f / (1.f + expf(-t)); return g * s * (1.f + t * (1.f - s)); }
    case U_GELU: {
      const float c = 0.7978845608028654f;
      float in = c * (t + 0.044715f * t * t * t);
      float th = tanhf(in);
      return g * (0.5f * (1.f + th) + 0.5f * t * (1.f - th * th) * c * (1.f + 3.f * 0.044715f * t * t));
    }
    case U_RECIP: return -g / (t * t);
    default: return g;
  }
}

template <typename T, typename F>
__global__ void map1_kernel(const T* __restrict__ x, T* __restrict__ out, long long n, F f) {
  constexpr int V = Vec16<T>::N;
  const long long nv = n / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    Vec16<T> a = ld16(x + i * V), o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(f(Cvt<T>::to_f(a.v[j])));
    st16(out + i * V, o);
  }
  for (long long i = nv * V + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = Cvt<T>::from_f(f(Cvt<T>::to_f(x[i])));
}

template <typename T, typename F>
__global__ void map2_kernel(const T* __restrict__ x, const T* __restrict__ y, T* __restrict__ out, long long n, F f) {
  constexpr int V = Vec16<T>::N;
  const long long nv = n / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    Vec16<T> a = ld16(x + i * V), b = ld16(y + i * V), o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(f(Cvt<T>::to_f(a.v[j]), Cvt<T>::to_f(b.v[j])));
    st16(out + i * V, o);
  }
  for (long long i = nv * V + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = Cvt<T>::from_f(f(Cvt<T>::to_f(x[i]), Cvt<T>::to_f(y[i])));
}

struct Shape4 { long long d[4]; long long sa[4]; long long sb[4]; };

// <=4-D broadcast: out contiguous over shape d, inputs addressed through element strides (0 = broadcast)
template <typename T>
__global__ void binary_strided_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                      long long n, Shape4 s, int op) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    long long r = i;
    const long long i3 = r % s.d[3]; r /= s.d[3];
    const long long i2 = r % s.d[2]; r /= s.d[2];
    const long long i1 = r % s.d[1]; r /= s.d[1];
    const long long i0 = r;
    const float x = Cvt<T>::to_f(a[i0 * s.sa[0] + i1 * s.sa[1] + i2 * s.sa[2] + i3 * s.sa[3]]);
    const float y = Cvt<T>::to_f(b[i0 * s.sb[0] + i1 * s.sb[1] + i2 * s.sb[2] + i3 * s.sb[3]]);
    out[i] = Cvt<T>::from_f(bin_apply(op, x, y));
  }
}

template <typename T>
__global__ void compare_kernel(const T* __restrict__ a, const T* __restrict__ b, float scalar, int use_scalar,
                               uint8_t* __restrict__ out, long long n, int op) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float x = Cvt<T>::to_f(a[i]);
    const float y = use_scalar ? scalar : Cvt<T>::to_f(b[i]);
    bool r;
    switch (op) {
      case C_EQ: r = x == y; break;
      case C_NE: r = x != y; break;
      case C_LT: r = x < y; break;
      case C_LE: r = x <= y; break;
      case C_GT: r = x > y; break;
      default: r = x >= y; break;
    }
    out[i] = r ? 1 : 0;
  }
}

template <typename T>
__global__ void where_kernel(const uint8_t* __restrict__ c, const T* __restrict__ a, const T* __restrict__ b,
                             float sa, float sb, int a_scalar, int b_scalar, T* __restrict__ out, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float x = a_scalar ? sa : Cvt<T>::to_f(a[i]);
    const float y = b_scalar ? sb : Cvt<T>::to_f(b[i]);
    out[i] = Cvt<T>::from_f(c[i] ? x : y);
  }
}

template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ src, D* __restrict__ dst, long long n) {
  constexpr int V = 8;
  const long long nv = n / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    S a[V];
    D o[V];
    if constexpr (sizeof(S) == 2) { *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(src + i * V); }
    else { *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(src + i * V);
           *reinterpret_cast<uint4*>(a + 4) = *reinterpret_cast<const uint4*>(src + i * V + 4); }
#pragma unroll
    for (int j = 0; j < V; ++j) o[j] = Cvt<D>::from_f(Cvt<S>::to_f(a[j]));
    if constexpr (sizeof(D) == 2) { *reinterpret_cast<uint4*>(dst + i * V) = *reinterpret_cast<uint4*>(o); }
    else { *reinterpret_cast<uint4*>(dst + i * V) = *reinterpret_cast<uint4*>(o);
           *reinterpret_cast<uint4*>(dst + i * V + 4) = *reinterpret_cast<uint4*>(o + 4); }
  }
  for (long long i = nv * V + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = Cvt<D>::from_f(Cvt<S>::to_f(src[i]));
}

template <typename T>
__global__ void fill_kernel(T* __restrict__ p, long long n, float v) {
  const T tv = Cvt<T>::from_f(v);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = tv;
}

// a += alpha * b, b possibly of another float dtype
template <typename TA, typename TB>
__global__ void axpy_kernel(TA* __restrict__ a, const TB* __restrict__ b, float alpha, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    a[i] = Cvt<TA>::from_f(Cvt<TA>::to_f(a[i]) + alpha * Cvt<TB>::to_f(b[i]));
}

struct CopyDesc { int ndim; long long shape[6]; long long ss[6]; long long ds[6]; };

// generic strided copy of `ES`-byte elements (<= 6 dims)
template <typename E>
__global__ void copy_strided_kernel(const E* __restrict__ src, E* __restrict__ dst, long long n, CopyDesc d) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    long long r = i, so = 0, dof = 0;
#pragma unroll
    for (int k = 5; k >= 0; --k) {
      if (k < d.ndim) {
        const long long idx = r % d.shape[k];
        r /= d.shape[k];
        so += idx * d.ss[k];
        dof += idx * d.ds[k];
      }
    }
    dst[dof] = src[so];
  }
}

// batched 2-D transpose through shared memory: dst[b][c][r] = src[b][r][c] with arbitrary batch strides
template <typename E>
__global__ void transpose_kernel(const E* __restrict__ src, E* __restrict__ dst, int R, int C, long long s_r,
                                 long long s_c, long long s_b, long long d_b) {
  __shared__ E tile[32][33];
  const int b = blockIdx.z;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const E* s = src + (long long)b * s_b;
  E* d = dst + (long long)b * d_b;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < R && c < C) tile[j][threadIdx.x] = s[(long long)r * s_r + (long long)c * s_c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < R && c < C) d[(long long)c * R + r] = tile[threadIdx.x][j];
  }
}

}  // namespace gb

using namespace gb;

extern "C" int gb_binary(int op, const void* a, const void* b, void* out, long long n, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, map2_kernel<T><<<gb_grid(n / Vec16<T>::N + 1, 256), 256, 0, st>>>(
      (const T*)a, (const T*)b, (T*)out, n, [op] __device__(float x, float y) { return bin_apply(op, x, y); }));
  return (int)cudaGetLastError();
}

extern "C" int gb_binary_scalar(int op, const void* a, float s, void* out, long long n, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, map1_kernel<T><<<gb_grid(n / Vec16<T>::N + 1, 256), 256, 0, st>>>(
      (const T*)a, (T*)out, n, [op, s] __device__(float x) { return bin_apply(op, x, s); }));
  return (int)cudaGetLastError();
}

extern "C" int gb_binary_strided(int op, const void* a, const void* b, void* out, const long long* shape,
                                 const long long* sa, const long long* sb, int dt, cudaStream_t st) {
  Shape4 s;
  long long n = 1;
  for (int i = 0; i < 4; ++i) { s.d[i] = shape[i]; s.sa[i] = sa[i]; s.sb[i] = sb[i]; n *= shape[i]; }
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, binary_strided_kernel<T><<<gb_grid(n, 256), 256, 0, st>>>(
      (const T*)a, (const T*)b, (T*)out, n, s, op));
  return (int)cudaGetLastError();
}

extern "C" int gb_unary(int op, const void* x, void* out, long long n, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, map1_kernel<T><<<gb_grid(n / Vec16<T>::N + 1, 256), 256, 0, st>>>(
      (const T*)x, (T*)out, n, [op] __device__(float v) { return un_apply(op, v); }));
  return (int)cudaGetLastError();
}

extern "C" int gb_unary_bwd(int op, const void* g, const void* t, void* out, long long n, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, map2_kernel<T><<<gb_grid(n / Vec16<T>::N + 1, 256), 256, 0, st>>>(
      (const T*)g, (const T*)t, (T*)out, n, [op] __device__(float gg, float tt) { return un_bwd(op, gg, tt); }));
  return (int)cudaGetLastError();
}

extern "C" int gb_clamp(const void* x, void* out, float lo, float hi, long long n, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, map1_kernel<T><<<gb_grid(n / Vec16<T>::N + 1, 256), 256, 0, st>>>(
      (const T*)x, (T*)out, n, [lo, hi] __device__(float v) { return fminf(fmaxf(v, lo), hi); }));
  return (int)cudaGetLastError();
}

extern "C" int gb_compare(int op, const void* a, const void* b, float scalar, int use_scalar, void* out,
                          long long n, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, compare_kernel<T><<<gb_grid(n, 256), 256, 0, st>>>(
      (const T*)a, (const T*)b, scalar, use_scalar, (uint8_t*)out, n, op));
  return (int)cudaGetLastError();
}

extern "C" int gb_where(const void* c, const void* a, const void* b, float sa, float sb, int a_scalar,
                        int b_scalar, void* out, long long n, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, where_kernel<T><<<gb_grid(n, 256), 256, 0, st>>>(
      (const uint8_t*)c, (const T*)a, (const T*)b, sa, sb, a_scalar, b_scalar, (T*)out, n));
  return (int)cudaGetLastError();
}

template <typename S>
static int cast_from(const void* src, void* dst, long long n, int ddt, cudaStream_t st) {
  const int g = gb_grid(n / 8 + 1, 256);
  if (ddt == DT_F32) cast_kernel<S, float><<<g, 256, 0, st>>>((const S*)src, (float*)dst, n);
  else if (ddt == DT_F16) cast_kernel<S, __half><<<g, 256, 0, st>>>((const S*)src, (__half*)dst, n);
  else if (ddt == DT_BF16) cast_kernel<S, __nv_bfloat16><<<g, 256, 0, st>>>((const S*)src, (__nv_bfloat16*)dst, n);
  else return -2;
  return (int)cudaGetLastError();
}

extern "C" int gb_cast(const void* src, void* dst, long long n, int sdt, int ddt, cudaStream_t st) {
  if (n == 0) return 0;
  if (sdt == DT_F32) return cast_from<float>(src, dst, n, ddt, st);
  if (sdt == DT_F16) return cast_from<__half>(src, dst, n, ddt, st);
  if (sdt == DT_BF16) return cast_from<__nv_bfloat16>(src, dst, n, ddt, st);
  return -2;
}

extern "C" int gb_fill(void* p, long long n, float v, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, fill_kernel<T><<<gb_grid(n, 256), 256, 0, st>>>((T*)p, n, v));
  return (int)cudaGetLastError();
}

template <typename TA>
static int axpy_from(void* a, const void* b, float alpha, long long n, int dtb, cudaStream_t st) {
  const int g = gb_grid(n, 256);
  if (dtb == DT_F32) axpy_kernel<TA, float><<<g, 256, 0, st>>>((TA*)a, (const float*)b, alpha, n);
  else if (dtb == DT_F16) axpy_kernel<TA, __half><<<g, 256, 0, st>>>((TA*)a, (const __half*)b, alpha, n);
  else if (dtb == DT_BF16) axpy_kernel<TA, __nv_bfloat16><<<g, 256, 0, st>>>((TA*)a, (const __nv_bfloat16*)b, alpha, n);
  else return -2;
  return (int)cudaGetLastError();
}

extern "C" int gb_axpy(void* a, const void* b, float alpha, long long n, int dta, int dtb, cudaStream_t st) {
  if (n == 0) return 0;
  if (dta == DT_F32) return axpy_from<float>(a, b, alpha, n, dtb, st);
  if (dta == DT_F16) return axpy_from<__half>(a, b, alpha, n, dtb, st);
  if (dta == DT_BF16) return axpy_from<__nv_bfloat16>(a, b, alpha, n, dtb, st);
  return -2;
}

extern "C" int gb_copy_strided(const void* src, void* dst, int ndim, const long long* shape, const long long* ss,
                               const long long* ds, int esize, cudaStream_t st) {
  if (ndim > 6) return -2;
  CopyDesc d;
  d.ndim = ndim;
  long long n = 1;
  for (int i = 0; i < ndim; ++i) { d.shape[i] = shape[i]; d.ss[i] = ss[i]; d.ds[i] = ds[i]; n *= shape[i]; }
  if (n == 0) return 0;
  const int g = gb_grid(n, 256);
  if (esize == 1) copy_strided_kernel<uint8_t><<<g, 256, 0, st>>>((const uint8_t*)src, (uint8_t*)dst, n, d);
  else if (esize == 2) copy_strided_kernel<uint16_t><<<g, 256, 0, st>>>((const uint16_t*)src, (uint16_t*)dst, n, d);
  else if (esize == 4) copy_strided_kernel<uint32_t><<<g, 256, 0, st>>>((const uint32_t*)src, (uint32_t*)dst, n, d);
  else if (esize == 8) copy_strided_kernel<uint64_t><<<g, 256, 0, st>>>((const uint64_t*)src, (uint64_t*)dst, n, d);
  else return -2;
  return (int)cudaGetLastError();
}

// dst[b][c][r] (contiguous) = src[b][r][c] where src has strides (s_b, s_r, s_c)
extern "C" int gb_transpose(const void* src, void* dst, int batch, int R, int C, long long s_b, long long s_r,
                            long long s_c, int esize, cudaStream_t st) {
  if (batch == 0 || R == 0 || C == 0) return 0;
  dim3 grid((C + 31) / 32, (R + 31) / 32, batch), block(32, 8);
  const long long d_b = (long long)R * C;
  if (esize == 2) transpose_kernel<uint16_t><<<grid, block, 0, st>>>((const uint16_t*)src, (uint16_t*)dst, R, C, s_r, s_c, s_b, d_b);
  else if (esize == 4) transpose_kernel<uint32_t><<<grid, block, 0, st>>>((const uint32_t*)src, (uint32_t*)dst, R, C, s_r, s_c, s_b, d_b);
  else if (esize == 8) transpose_kernel<uint64_t><<<grid, block, 0, st>>>((const uint64_t*)src, (uint64_t*)dst, R, C, s_r, s_c, s_b, d_b);
  else return -2;
  return (int)cudaGetLastError();
}
