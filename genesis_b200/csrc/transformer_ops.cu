// Memory-bound transformer pieces, one launch each:
//   SwiGLU  silu(gate) * up, forward and backward        (reference: triton_ops/silu.py + a mul)
//   RoPE    rotate-half rotation on [B, S, H, D]          (reference: ~14 launches, components.py:121-179)
//   embedding gather and accumulating scatter (fp32 atomics, duplicates add up)
//   Philox-4x32-10 uniform / normal / randint / dropout   (reference: LCG kernels, ops/cuda/random_ops.py)
//   row gather / scatter-add for mixture-of-experts dispatch and combine
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace gb {

// ------------------------------------------------------------------------------------------
// SwiGLU
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out,
                                  long long n) {
  constexpr int V = Vec16<T>::N;
  const long long nv = n / V, stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    Vec16<T> a = ld16(gate + i * V), b = ld16(up + i * V), o;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float g = Cvt<T>::to_f(a.v[j]);
      o.v[j] = Cvt<T>::from_f(g / (1.f + __expf(-g)) * Cvt<T>::to_f(b.v[j]));
    }
    st16(out + i * V, o);
  }
  for (long long i = nv * V + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float g = Cvt<T>::to_f(gate[i]);
    out[i] = Cvt<T>::from_f(g / (1.f + __expf(-g)) * Cvt<T>::to_f(up[i]));
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ gate, const T* __restrict__ up,
                                  T* __restrict__ dgate, T* __restrict__ dup, long long n) {
  constexpr int V = Vec16<T>::N;
  const long long nv = n / V, stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    Vec16<T> d = ld16(dy + i * V), a = ld16(gate + i * V), b = ld16(up + i * V), og, ou;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float g = Cvt<T>::to_f(a.v[j]), u = Cvt<T>::to_f(b.v[j]), dd = Cvt<T>::to_f(d.v[j]);
      const float s = 1.f / (1.f + __expf(-g));
      og.v[j] = Cvt<T>::from_f(dd * u * s * (1.f + g * (1.f - s)));
      ou.v[j] = Cvt<T>::from_f(dd * g * s);
    }
    st16(dgate + i * V, og);
    st16(dup + i * V, ou);
  }
  for (long long i = nv * V + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float g = Cvt<T>::to_f(gate[i]), u = Cvt<T>::to_f(up[i]), dd = Cvt<T>::to_f(dy[i]);
    const float s = 1.f / (1.f + __expf(-g));
    dgate[i] = Cvt<T>::from_f(dd * u * s * (1.f + g * (1.f - s)));
    dup[i] = Cvt<T>::from_f(dd * g * s);
  }
}

// Row-strided forms: gate and up are the two column halves of one [rows, 2 * cols] matrix (a fused gate/up
// projection), out is [rows, cols]; backward writes dgate | dup into the halves of one [rows, 2 * cols] matrix.
template <typename T>
__global__ void swiglu_fwd2d_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int cols) {
  constexpr int V = Vec16<T>::N;
  const int cpv = cols / V;
  const long long total = rows * cpv, stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / cpv;
    const int c = (int)(i % cpv) * V;
    const T* g = gu + r * 2 * cols + c;
    Vec16<T> a = ld16(g), b = ld16(g + cols), o;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float x = Cvt<T>::to_f(a.v[j]);
      o.v[j] = Cvt<T>::from_f(x / (1.f + __expf(-x)) * Cvt<T>::to_f(b.v[j]));
    }
    st16(out + r * cols + c, o);
  }
}

template <typename T>
__global__ void swiglu_bwd2d_kernel(const T* __restrict__ dy, const T* __restrict__ gu, T* __restrict__ dgu,
                                    long long rows, int cols) {
  constexpr int V = Vec16<T>::N;
  const int cpv = cols / V;
  const long long total = rows * cpv, stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / cpv;
    const int c = (int)(i % cpv) * V;
    const T* g = gu + r * 2 * cols + c;
    Vec16<T> d = ld16(dy + r * cols + c), a = ld16(g), b = ld16(g + cols), og, ou;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float x = Cvt<T>::to_f(a.v[j]), u = Cvt<T>::to_f(b.v[j]), dd = Cvt<T>::to_f(d.v[j]);
      const float sg = 1.f / (1.f + __expf(-x));
      og.v[j] = Cvt<T>::from_f(dd * u * sg * (1.f + x * (1.f - sg)));
      ou.v[j] = Cvt<T>::from_f(dd * x * sg);
    }
    T* o = dgu + r * 2 * cols + c;
    st16(o, og);
    st16(o + cols, ou);
  }
}

// ------------------------------------------------------------------------------------------
// RoPE (rotate-half): out[..., i] = x[i]*cos[i] - x[i+D/2]*sin[i];  out[..., i+D/2] = x[i+D/2]*cos + x[i]*sin
// cos/sin: fp32 [max_pos, D] with duplicated halves; positions: optional int64 [B, S].
// inverse = 1 applies the transposed rotation (used for the gradient).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ cosb,
                            const float* __restrict__ sinb, const long long* __restrict__ positions, int B, int S,
                            int H, int D, int inverse, long long xrs, long long ors) {
  const int half = D / 2;
  const long long total = (long long)B * S * H * half;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int d = (int)(i % half);
    const long long r = i / half;            // (b, s, h)
    const long long bs = r / H;
    const int s = (int)(bs % S);
    const long long pos = positions ? positions[bs] : s;
    const float c = cosb[pos * D + d];
    float sn = sinb[pos * D + d];
    if (inverse) sn = -sn;
    const int hh = (int)(r % H);
    const long long xb = bs * xrs + (long long)hh * D, ob = bs * ors + (long long)hh * D;   // token row strides
    const float x1 = Cvt<T>::to_f(x[xb + d]), x2 = Cvt<T>::to_f(x[xb + d + half]);
    out[ob + d] = Cvt<T>::from_f(x1 * c - x2 * sn);
    out[ob + d + half] = Cvt<T>::from_f(x2 * c + x1 * sn);
  }
}

// Vector form: a thread rotates one 16-byte group of the first half against its partner group of the second
// half (half % (16 / sizeof(T)) == 0, 16-byte aligned rows).
template <typename T>
__global__ void rope_vec_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ cosb,
                                const float* __restrict__ sinb, const long long* __restrict__ positions, int B, int S,
                                int H, int D, int inverse, long long xrs, long long ors) {
  constexpr int V = Vec16<T>::N;
  const int half = D / 2;
  const int gpr = half / V;                                  // vector groups per half row
  const long long total = (long long)B * S * H * gpr;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int g = (int)(i % gpr);
    const long long r = i / gpr;                             // (b, s, h)
    const long long bs = r / H;
    const int s = (int)(bs % S);
    const long long pos = positions ? positions[bs] : s;
    const float* cp = cosb + pos * D + g * V;
    const float* sp = sinb + pos * D + g * V;
    const int hh = (int)(r % H);
    const long long xb = bs * xrs + (long long)hh * D + g * V, ob = bs * ors + (long long)hh * D + g * V;
    const Vec16<T> a = ld16(x + xb), b2 = ld16(x + xb + half);
    Vec16<T> oa, ob2;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float c = cp[j];
      const float sn = inverse ? -sp[j] : sp[j];
      const float x1 = Cvt<T>::to_f(a.v[j]), x2 = Cvt<T>::to_f(b2.v[j]);
      oa.v[j] = Cvt<T>::from_f(x1 * c - x2 * sn);
      ob2.v[j] = Cvt<T>::from_f(x2 * c + x1 * sn);
    }
    st16(out + ob, oa);
    st16(out + ob + half, ob2);
  }
}

// One launch for the three head groups of a fused q | k | v projection y [rows, (Hq + 2 Hkv) D]:
//   merge = 0:  q = rope(y_q), k = rope(y_k), v = y_v            (three contiguous [rows, H, D] outputs)
//   merge = 1:  y_q = rope^T(q), y_k = rope^T(k), y_v = v        (the gradients, back into one buffer)
// Same vector form as rope_vec_kernel: a thread handles one 16-byte group of the first half of a head and its partner
// group of the second half.
template <typename T>
__global__ void qkv_rope_kernel(T* __restrict__ y, T* __restrict__ q, T* __restrict__ k, T* __restrict__ v,
                                const float* __restrict__ cosb, const float* __restrict__ sinb,
                                const long long* __restrict__ positions, long long rows, int S, int Hq, int Hkv, int D,
                                int merge) {
  constexpr int V = Vec16<T>::N;
  const int half = D / 2;
  const int gpr = half / V;
  const int Ht = Hq + 2 * Hkv;
  const long long total = rows * Ht * gpr;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int g = (int)(i % gpr);
    const long long r = i / gpr;
    const int h = (int)(r % Ht);
    const long long bs = r / Ht;
    T* yp = y + (bs * Ht + h) * D + g * V;
    T* sp;
    bool rot = true;
    if (h < Hq) sp = q + (bs * Hq + h) * D + g * V;
    else if (h < Hq + Hkv) sp = k + (bs * Hkv + (h - Hq)) * D + g * V;
    else { sp = v + (bs * Hkv + (h - Hq - Hkv)) * D + g * V; rot = false; }
    const T* src = merge ? sp : yp;
    T* dst = merge ? yp : sp;
    const Vec16<T> a = ld16(src), b2 = ld16(src + half);
    if (!rot) {
      st16(dst, a);
      st16(dst + half, b2);
      continue;
    }
    const long long pos = positions ? positions[bs] : (bs % S);
    const float* cp = cosb + pos * D + g * V;
    const float* snp = sinb + pos * D + g * V;
    Vec16<T> oa, ob2;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float c = cp[j];
      const float sn = merge ? -snp[j] : snp[j];
      const float x1 = Cvt<T>::to_f(a.v[j]), x2 = Cvt<T>::to_f(b2.v[j]);
      oa.v[j] = Cvt<T>::from_f(x1 * c - x2 * sn);
      ob2.v[j] = Cvt<T>::from_f(x2 * c + x1 * sn);
    }
    st16(dst, oa);
    st16(dst + half, ob2);
  }
}

// ------------------------------------------------------------------------------------------
// row gather / scatter
// ------------------------------------------------------------------------------------------
// out[i, :] = src[idx[i], :] (zeros when idx[i] < 0); 16-byte vectors, one warp per row chunk.
// An index >= src_rows (a token id outside the table) is never dereferenced: the row reads as zeros and the
// status word records {GB_ERR_BAD_INDEX, site 1, block, index}.
template <typename E, typename TI>
__global__ void gather_rows_kernel(const E* __restrict__ src, const TI* __restrict__ idx, E* __restrict__ out,
                                   long long nrows, int vec_per_row, long long src_rows, int* __restrict__ status) {
  const long long total = nrows * vec_per_row;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / vec_per_row;
    const int c = (int)(i % vec_per_row);
    const long long s = (long long)idx[r];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (s >= src_rows) { if (c == 0) report_error(status, GB_ERR_BAD_INDEX, 1, (int)s); }
    else if (s >= 0) v = reinterpret_cast<const uint4*>(src)[s * vec_per_row + c];
    reinterpret_cast<uint4*>(out)[i] = v;
  }
}

// acc[idx[i], :] += src[i, :] with fp32 atomics (acc fp32)
template <typename T, typename TI>
__global__ void scatter_add_rows_kernel(const T* __restrict__ src, const TI* __restrict__ idx,
                                        float* __restrict__ acc, long long nrows, int cols, long long acc_rows,
                                        int* __restrict__ status) {
  const long long total = nrows * cols;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / cols;
    const int c = (int)(i % cols);
    const long long d = (long long)idx[r];
    if (d >= acc_rows) { if (c == 0) report_error(status, GB_ERR_BAD_INDEX, 2, (int)d); }
    else if (d >= 0) atomicAdd(acc + d * cols + c, Cvt<T>::to_f(src[i]));
  }
}

// ------------------------------------------------------------------------------------------
// Philox-4x32-10
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 philox4x32(uint2 key, uint4 ctr) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}
__device__ __forceinline__ float u01(uint32_t x) { return (x >> 8) * (1.0f / 16777216.0f); }   // [0, 1)

// kind 0: uniform in [a, b); 1: normal(mean a, std b); 2: integers in [a, b)
template <typename T>
__global__ void random_kernel(T* __restrict__ out, long long n, unsigned long long seed, unsigned long long offset,
                              int kind, float a, float b) {
  const long long groups = (n + 3) / 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  for (long long gi = (long long)blockIdx.x * blockDim.x + threadIdx.x; gi < groups; gi += stride) {
    const uint4 r = philox4x32(key, make_uint4((uint32_t)gi, (uint32_t)(gi >> 32), (uint32_t)offset,
                                                (uint32_t)(offset >> 32)));
    float v[4];
    if (kind == 1) {
      const float u1 = fmaxf(u01(r.x), 5.9604645e-8f), u2 = u01(r.y);
      const float u3 = fmaxf(u01(r.z), 5.9604645e-8f), u4 = u01(r.w);
      const float r1 = sqrtf(-2.f * logf(u1)), r2 = sqrtf(-2.f * logf(u3));
      v[0] = r1 * cospif(2.f * u2); v[1] = r1 * sinpif(2.f * u2);
      v[2] = r2 * cospif(2.f * u4); v[3] = r2 * sinpif(2.f * u4);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = a + b * v[j];
    } else {
      v[0] = a + (b - a) * u01(r.x); v[1] = a + (b - a) * u01(r.y);
      v[2] = a + (b - a) * u01(r.z); v[3] = a + (b - a) * u01(r.w);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (gi * 4 + j < n) out[gi * 4 + j] = Cvt<T>::from_f(v[j]);
  }
}

__global__ void randint_kernel(long long* __restrict__ out, long long n, unsigned long long seed,
                               unsigned long long offset, long long lo, long long hi) {
  const long long groups = (n + 3) / 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  const unsigned long long range = (unsigned long long)(hi - lo);
  for (long long gi = (long long)blockIdx.x * blockDim.x + threadIdx.x; gi < groups; gi += stride) {
    const uint4 r = philox4x32(key, make_uint4((uint32_t)gi, (uint32_t)(gi >> 32), (uint32_t)offset,
                                                (uint32_t)(offset >> 32)));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (gi * 4 + j < n) out[gi * 4 + j] = lo + (long long)(((unsigned long long)w[j] * range) >> 32);
  }
}

// y = x * keep / (1-p); mask[i] = keep
template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ y, uint8_t* __restrict__ mask, long long n,
                               float p, unsigned long long seed, unsigned long long offset) {
  const long long groups = (n + 3) / 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  const float scale = 1.f / (1.f - p);
  for (long long gi = (long long)blockIdx.x * blockDim.x + threadIdx.x; gi < groups; gi += stride) {
    const uint4 r = philox4x32(key, make_uint4((uint32_t)gi, (uint32_t)(gi >> 32), (uint32_t)offset,
                                                (uint32_t)(offset >> 32)));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long i = gi * 4 + j;
      if (i < n) {
        const bool keep = u01(w[j]) >= p;
        mask[i] = keep ? 1 : 0;
        y[i] = Cvt<T>::from_f(keep ? Cvt<T>::to_f(x[i]) * scale : 0.f);
      }
    }
  }
}

}  // namespace gb

using namespace gb;

extern "C" int gb_swiglu_fwd(const void* gate, const void* up, void* out, long long n, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, swiglu_fwd_kernel<T><<<gb_grid(n / Vec16<T>::N + 1, 256), 256, 0, st>>>(
      (const T*)gate, (const T*)up, (T*)out, n));
  return (int)cudaGetLastError();
}

extern "C" int gb_swiglu_bwd(const void* dy, const void* gate, const void* up, void* dgate, void* dup, long long n,
                             int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, swiglu_bwd_kernel<T><<<gb_grid(n / Vec16<T>::N + 1, 256), 256, 0, st>>>(
      (const T*)dy, (const T*)gate, (const T*)up, (T*)dgate, (T*)dup, n));
  return (int)cudaGetLastError();
}

// gu [rows, 2 * cols] = gate | up; out [rows, cols].  cols a multiple of 16 bytes, 16-byte aligned bases.
extern "C" int gb_swiglu_fwd2d(const void* gu, void* out, long long rows, int cols, int dt, cudaStream_t st) {
  if (rows == 0 || cols == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, {
    if (cols % Vec16<T>::N != 0) return -3;
    swiglu_fwd2d_kernel<T><<<gb_grid(rows * (cols / Vec16<T>::N), 256), 256, 0, st>>>((const T*)gu, (T*)out, rows, cols);
  });
  return (int)cudaGetLastError();
}

// dy [rows, cols], gu [rows, 2 * cols] -> dgu [rows, 2 * cols] = dgate | dup
extern "C" int gb_swiglu_bwd2d(const void* dy, const void* gu, void* dgu, long long rows, int cols, int dt,
                               cudaStream_t st) {
  if (rows == 0 || cols == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, {
    if (cols % Vec16<T>::N != 0) return -3;
    swiglu_bwd2d_kernel<T><<<gb_grid(rows * (cols / Vec16<T>::N), 256), 256, 0, st>>>((const T*)dy, (const T*)gu, (T*)dgu, rows, cols);
  });
  return (int)cudaGetLastError();
}

// x_row_stride / out_row_stride: elements between consecutive tokens (H * D when the tensor is contiguous; larger when
// the heads are a column slice of a wider matrix, e.g. a fused q/k/v projection).
extern "C" int gb_rope(const void* x, void* out, const float* cosb, const float* sinb, const long long* positions,
                       int B, int S, int H, int D, int inverse, int dt, long long x_row_stride,
                       long long out_row_stride, cudaStream_t st) {
  const long long total = (long long)B * S * H * (D / 2);
  if (total == 0) return 0;
  const int es = dt == DT_F32 ? 4 : 2;
  const bool vec = (D / 2) % (16 / es) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                   (x_row_stride * es) % 16 == 0 && (out_row_stride * es) % 16 == 0;
  if (vec) {
    GB_DISPATCH_FLOAT(dt, T, rope_vec_kernel<T><<<gb_grid(total / Vec16<T>::N, 256), 256, 0, st>>>(
        (const T*)x, (T*)out, cosb, sinb, positions, B, S, H, D, inverse, x_row_stride, out_row_stride));
  } else {
    GB_DISPATCH_FLOAT(dt, T, rope_kernel<T><<<gb_grid(total, 256), 256, 0, st>>>(
        (const T*)x, (T*)out, cosb, sinb, positions, B, S, H, D, inverse, x_row_stride, out_row_stride));
  }
  return (int)cudaGetLastError();
}

// y, q, k, v contiguous and 16-byte aligned, (D / 2) a multiple of the 16-byte vector; -9 otherwise (the caller then uses
// gb_rope per head group and a copy).
extern "C" int gb_qkv_rope(void* y, void* q, void* k, void* v, const float* cosb, const float* sinb,
                           const long long* positions, long long rows, int S, int Hq, int Hkv, int D, int merge, int dt,
                           cudaStream_t st) {
  if (rows == 0) return 0;
  const int es = dt == DT_F32 ? 4 : 2;
  if (D % 2 || (D / 2) % (16 / es) != 0 ||
      ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
        reinterpret_cast<uintptr_t>(v)) & 15) != 0)
    return -9;
  const long long total = rows * (Hq + 2 * Hkv) * (D / 2) / (16 / es);
  GB_DISPATCH_FLOAT(dt, T, qkv_rope_kernel<T><<<gb_grid(total, 256), 256, 0, st>>>(
      (T*)y, (T*)q, (T*)k, (T*)v, cosb, sinb, positions, rows, S, Hq, Hkv, D, merge));
  return (int)cudaGetLastError();
}

// rows of `row_bytes` bytes (multiple of 16, 16-byte aligned bases)
extern "C" int gb_gather_rows(const void* src, const void* idx, void* out, long long nrows, long long row_bytes,
                              int idx_is_i64, long long src_rows, int* status, cudaStream_t st) {
  if (nrows == 0) return 0;
  const int vpr = (int)(row_bytes / 16);
  const int g = gb_grid(nrows * vpr, 256);
  if (idx_is_i64) gather_rows_kernel<uint4, long long><<<g, 256, 0, st>>>((const uint4*)src, (const long long*)idx, (uint4*)out, nrows, vpr, src_rows, status);
  else gather_rows_kernel<uint4, int><<<g, 256, 0, st>>>((const uint4*)src, (const int*)idx, (uint4*)out, nrows, vpr, src_rows, status);
  return (int)cudaGetLastError();
}

extern "C" int gb_scatter_add_rows(const void* src, const void* idx, float* acc, long long nrows, int cols, int dt,
                                   int idx_is_i64, long long acc_rows, int* status, cudaStream_t st) {
  if (nrows == 0) return 0;
  const int g = gb_grid(nrows * cols, 256);
  if (idx_is_i64) {
    GB_DISPATCH_FLOAT(dt, T, scatter_add_rows_kernel<T, long long><<<g, 256, 0, st>>>((const T*)src, (const long long*)idx, acc, nrows, cols, acc_rows, status));
  } else {
    GB_DISPATCH_FLOAT(dt, T, scatter_add_rows_kernel<T, int><<<g, 256, 0, st>>>((const T*)src, (const int*)idx, acc, nrows, cols, acc_rows, status));
  }
  return (int)cudaGetLastError();
}

extern "C" int gb_random(void* out, long long n, unsigned long long seed, unsigned long long offset, int kind,
                         float a, float b, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, random_kernel<T><<<gb_grid((n + 3) / 4, 256), 256, 0, st>>>((T*)out, n, seed, offset, kind, a, b));
  return (int)cudaGetLastError();
}

extern "C" int gb_randint(long long* out, long long n, unsigned long long seed, unsigned long long offset,
                          long long lo, long long hi, cudaStream_t st) {
  if (n == 0) return 0;
  randint_kernel<<<gb_grid((n + 3) / 4, 256), 256, 0, st>>>(out, n, seed, offset, lo, hi);
  return (int)cudaGetLastError();
}

extern "C" int gb_dropout(const void* x, void* y, void* mask, long long n, float p, unsigned long long seed,
                          unsigned long long offset, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, dropout_kernel<T><<<gb_grid((n + 3) / 4, 256), 256, 0, st>>>(
      (const T*)x, (T*)y, (uint8_t*)mask, n, p, seed, offset));
  return (int)cudaGetLastError();
}
