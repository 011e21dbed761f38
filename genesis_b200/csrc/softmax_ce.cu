// Softmax / log-softmax over the last dimension (forward, backward) and fused softmax
// cross-entropy for large vocabularies (forward: loss + log-sum-exp per row; backward: (p - onehot)
// * row gradient, optionally written over the logits).  One CTA per row, online max/sum in fp32,
// 128-bit loads; rows that fit are kept in registers, longer rows are re-read (they stay in L2).
// Reference counterparts: genesis/nn/triton_ops/softmax.py:33-480 and the composed loss of
// genesis/nn/modules/loss.py:77-100 / genesis/nn/functional.py:2313-2506.
#include "common.cuh"
#include "row_stream.cuh"

namespace gb {

struct MaxSum { float m, s; };
__device__ __forceinline__ MaxSum ms_comb(MaxSum a, MaxSum b) {
  MaxSum r;
  r.m = fmaxf(a.m, b.m);
  if (r.m == -INFINITY) { r.s = 0.f; return r; }
  r.s = a.s * __expf(a.m - r.m) + b.s * __expf(b.m - r.m);
  return r;
}
__device__ __forceinline__ MaxSum block_maxsum(MaxSum v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum t; t.m = __shfl_xor_sync(0xffffffffu, v.m, o); t.s = __shfl_xor_sync(0xffffffffu, v.s, o);
    v = ms_comb(v, t);
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) { sh[w] = v.m; sh[32 + w] = v.s; }
  __syncthreads();
  MaxSum r; r.m = lane < nw ? sh[lane] : -INFINITY; r.s = lane < nw ? sh[32 + lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum t; t.m = __shfl_xor_sync(0xffffffffu, r.m, o); t.s = __shfl_xor_sync(0xffffffffu, r.s, o);
    r = ms_comb(r, t);
  }
  return r;
}

template <typename T>
__device__ __forceinline__ MaxSum row_maxsum(const T* p, long long cols, float* sh) {
  constexpr int V = Vec16<T>::N;
  MaxSum acc; acc.m = -INFINITY; acc.s = 0.f;
  long long done = 0;
  if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    const long long nv = cols / V;
    for (long long i = threadIdx.x; i < nv; i += blockDim.x) {
      Vec16<T> a = ld16(p + i * V);
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < V; ++j) mx = fmaxf(mx, Cvt<T>::to_f(a.v[j]));
      if (mx > acc.m) { acc.s *= __expf(acc.m - mx); acc.m = mx; }
      if (acc.m != -INFINITY) {
#pragma unroll
        for (int j = 0; j < V; ++j) acc.s += __expf(Cvt<T>::to_f(a.v[j]) - acc.m);
      }
    }
    done = nv * V;
  }
  for (long long i = done + threadIdx.x; i < cols; i += blockDim.x) {
    const float v = Cvt<T>::to_f(p[i]);
    if (v > acc.m) { acc.s *= __expf(acc.m - v); acc.m = v; }
    if (acc.m != -INFINITY) acc.s += __expf(v - acc.m);
  }
  return block_maxsum(acc, sh);
}

template <typename T>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, long long cols,
                                   int log_mode) {
  __shared__ float sh[64];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* p = x + row * cols;
    T* q = y + row * cols;
    const MaxSum ms = row_maxsum(p, cols, sh);
    const float lse = ms.m + __logf(ms.s);
    const float inv = ms.s > 0.f ? 1.f / ms.s : 0.f;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) {
      const float v = Cvt<T>::to_f(p[i]);
      q[i] = Cvt<T>::from_f(log_mode ? v - lse : __expf(v - ms.m) * inv);
    }
  }
}

// Register-resident rows: cols / V <= 256 * MV vectors, 16-byte aligned.  The row is read once (MV 16-byte loads per
// thread, all in flight together), max and sum are two block reductions over registers, the result is written with
// 16-byte stores.  HBM traffic = one read + one write of the tensor.
constexpr int SM_THREADS = 256;

template <typename T, int MV>
__global__ void __launch_bounds__(SM_THREADS)
softmax_fwd_reg_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int cols, int log_mode) {
  __shared__ float sh[32];
  constexpr int V = Vec16<T>::N;
  const int nv = cols / V;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* p = x + row * cols;
    Vec16<T> buf[MV];
#pragma unroll
    for (int k = 0; k < MV; ++k) {
      const int i = threadIdx.x + k * SM_THREADS;
      if (i < nv) buf[k] = ld16(p + (long long)i * V);
    }
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < MV; ++k)
      if (threadIdx.x + k * SM_THREADS < nv)
#pragma unroll
        for (int j = 0; j < V; ++j) mx = fmaxf(mx, Cvt<T>::to_f(buf[k].v[j]));
    mx = block_max(mx, sh);
    const float m = mx == -INFINITY ? 0.f : mx;            // a row of -inf gives zeros, not NaN
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < MV; ++k)
      if (threadIdx.x + k * SM_THREADS < nv)
#pragma unroll
        for (int j = 0; j < V; ++j) sum += __expf(Cvt<T>::to_f(buf[k].v[j]) - m);
    sum = block_sum(sum, sh);
    const float inv = sum > 0.f ? 1.f / sum : 0.f, lse = m + __logf(sum);   // all -inf: zeros
#pragma unroll
    for (int k = 0; k < MV; ++k) {
      const int i = threadIdx.x + k * SM_THREADS;
      if (i < nv) {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float v = Cvt<T>::to_f(buf[k].v[j]);
          o.v[j] = Cvt<T>::from_f(log_mode ? v - lse : __expf(v - m) * inv);
        }
        st16(y + row * cols + (long long)i * V, o);
      }
    }
  }
}

template <typename T, int MV>
__global__ void __launch_bounds__(SM_THREADS)
softmax_bwd_reg_kernel(const T* __restrict__ g, const T* __restrict__ y, T* __restrict__ dx, long long rows, int cols,
                       int log_mode) {
  __shared__ float sh[32];
  constexpr int V = Vec16<T>::N;
  const int nv = cols / V;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    Vec16<T> gb_[MV], yb[MV];
#pragma unroll
    for (int k = 0; k < MV; ++k) {
      const int i = threadIdx.x + k * SM_THREADS;
      if (i < nv) { gb_[k] = ld16(g + row * cols + (long long)i * V); yb[k] = ld16(y + row * cols + (long long)i * V); }
    }
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < MV; ++k)
      if (threadIdx.x + k * SM_THREADS < nv)
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float gg = Cvt<T>::to_f(gb_[k].v[j]);
          acc += log_mode ? gg : gg * Cvt<T>::to_f(yb[k].v[j]);
        }
    acc = block_sum(acc, sh);
#pragma unroll
    for (int k = 0; k < MV; ++k) {
      const int i = threadIdx.x + k * SM_THREADS;
      if (i < nv) {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float gg = Cvt<T>::to_f(gb_[k].v[j]), yy = Cvt<T>::to_f(yb[k].v[j]);
          o.v[j] = Cvt<T>::from_f(log_mode ? gg - __expf(yy) * acc : yy * (gg - acc));
        }
        st16(dx + row * cols + (long long)i * V, o);
      }
    }
  }
}

// softmax: dx = y * (g - sum(g*y));  log-softmax: dx = g - exp(y) * sum(g)
template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ g, const T* __restrict__ y, T* __restrict__ dx,
                                   long long rows, long long cols, int log_mode) {
  __shared__ float sh[32];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* gp = g + row * cols;
    const T* yp = y + row * cols;
    float acc = 0.f;
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) {
      const float gg = Cvt<T>::to_f(gp[i]);
      acc += log_mode ? gg : gg * Cvt<T>::to_f(yp[i]);
    }
    acc = block_sum(acc, sh);
    for (long long i = threadIdx.x; i < cols; i += blockDim.x) {
      const float gg = Cvt<T>::to_f(gp[i]), yy = Cvt<T>::to_f(yp[i]);
      dx[row * cols + i] = Cvt<T>::from_f(log_mode ? gg - __expf(yy) * acc : yy * (gg - acc));
    }
  }
}

template <typename T, typename TI>
__global__ void __launch_bounds__(1024)
ce_fwd_kernel(const T* __restrict__ logits, const TI* __restrict__ target, float* __restrict__ loss,
              float* __restrict__ lse_out, long long rows, long long cols, long long ignore_index) {
  __shared__ float sh[64];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* p = logits + row * cols;
    const MaxSum ms = row_maxsum(p, cols, sh);
    if (threadIdx.x == 0) {
      const float lse = ms.m + logf(ms.s);
      lse_out[row] = lse;
      const long long t = (long long)target[row];
      loss[row] = (t == ignore_index || t < 0 || t >= cols) ? 0.f : lse - Cvt<T>::to_f(p[t]);
    }
  }
}

template <typename T, typename TI>
__global__ void __launch_bounds__(1024)
ce_bwd_kernel(const T* __restrict__ logits, const TI* __restrict__ target, const float* __restrict__ lse,
              const float* __restrict__ grow, T* __restrict__ dlogits, long long rows, long long cols,
              long long ignore_index) {
  constexpr int V = Vec16<T>::N;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* p = logits + row * cols;
    T* q = dlogits + row * cols;
    const long long t = (long long)target[row];
    const bool ignored = (t == ignore_index || t < 0 || t >= cols);
    const float gr = ignored ? 0.f : grow[row];
    const float l = lse[row];
    long long done = 0;
    if (((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(q)) & 15) == 0) {
      const long long nv = cols / V;
      for (long long i = threadIdx.x; i < nv; i += blockDim.x) {
        Vec16<T> a = ld16(p + i * V), o;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float pr = __expf(Cvt<T>::to_f(a.v[j]) - l);
          if (i * V + j == t) pr -= 1.f;
          o.v[j] = Cvt<T>::from_f(pr * gr);
        }
        st16(q + i * V, o);
      }
      done = nv * V;
    }
    for (long long i = done + threadIdx.x; i < cols; i += blockDim.x) {
      float pr = __expf(Cvt<T>::to_f(p[i]) - l);
      if (i == t) pr -= 1.f;
      q[i] = Cvt<T>::from_f(pr * gr);
    }
  }
}

// Narrow rows (up to 128 16-byte vectors): one warp per row, eight rows in flight per CTA, shuffles instead of block
// barriers, the exponentials kept in registers between the sum and the output pass (one exp per element).
template <typename T, int MVW>
__global__ void __launch_bounds__(SM_THREADS)
softmax_fwd_warp_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int cols, int log_mode) {
  constexpr int V = Vec16<T>::N;
  constexpr float L2E = 1.4426950408889634f;
  const int nv = cols / V;
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (SM_THREADS / 32);
  for (long long row = (long long)blockIdx.x * (SM_THREADS / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    const T* p = x + row * cols;
    Vec16<T> buf[MVW];
#pragma unroll
    for (int k = 0; k < MVW; ++k)
      if (lane + 32 * k < nv) buf[k] = ld16(p + (long long)(lane + 32 * k) * V);
    float e[MVW][V];
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < MVW; ++k)
#pragma unroll
      for (int j = 0; j < V; ++j) {
        e[k][j] = (lane + 32 * k < nv) ? Cvt<T>::to_f(buf[k].v[j]) : -INFINITY;
        mx = fmaxf(mx, e[k][j]);
      }
    mx = warp_max(mx);
    const float m = mx == -INFINITY ? 0.f : mx;
    float sum = 0.f;
    if (log_mode) {
#pragma unroll
      for (int k = 0; k < MVW; ++k)
#pragma unroll
        for (int j = 0; j < V; ++j) sum += exp2f((e[k][j] - m) * L2E);
    } else {
#pragma unroll
      for (int k = 0; k < MVW; ++k)
#pragma unroll
        for (int j = 0; j < V; ++j) { e[k][j] = exp2f((e[k][j] - m) * L2E); sum += e[k][j]; }
    }
    sum = warp_sum(sum);
    const float inv = sum > 0.f ? 1.f / sum : 0.f, lse = m + __logf(sum);   // all -inf: zeros
#pragma unroll
    for (int k = 0; k < MVW; ++k) {
      if (lane + 32 * k < nv) {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(log_mode ? e[k][j] - lse : e[k][j] * inv);
        st16(y + row * cols + (long long)(lane + 32 * k) * V, o);
      }
    }
  }
}

}  // namespace gb

using namespace gb;

static inline int row_block(long long cols) { return cols >= 8192 ? 1024 : (cols >= 2048 ? 512 : (cols >= 256 ? 256 : 64)); }

extern "C" int gb_softmax_fwd(const void* x, void* y, long long rows, long long cols, int log_mode, int dt,
                              cudaStream_t st) {
  if (rows == 0) return 0;
  const int grid = (int)(rows < 148 * 16 ? rows : 148 * 16);
  const int vlen = dt == DT_F32 ? 4 : 8;
  const bool reg = cols % vlen == 0 && cols / vlen <= SM_THREADS * 8 && cols < (1ll << 30) &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (reg) {
    const long long nv = cols / vlen;
    if (nv <= 128 && rows >= 64) {
      const long long want = (rows + SM_THREADS / 32 - 1) / (SM_THREADS / 32);
      const int wgrid = (int)(want < 148 * 8 ? want : 148 * 8);
#define SM_WARP(MVV) GB_DISPATCH_FLOAT(dt, T, softmax_fwd_warp_kernel<T, MVV><<<wgrid, SM_THREADS, 0, st>>>((const T*)x, (T*)y, rows, (int)cols, log_mode))
      if (nv <= 32) SM_WARP(1);
      else if (nv <= 64) SM_WARP(2);
      else SM_WARP(4);
#undef SM_WARP
      return (int)cudaGetLastError();
    }
#define SM_FWD(MVV) GB_DISPATCH_FLOAT(dt, T, softmax_fwd_reg_kernel<T, MVV><<<grid, SM_THREADS, 0, st>>>((const T*)x, (T*)y, rows, (int)cols, log_mode))
    if (nv <= SM_THREADS) SM_FWD(1);
    else if (nv <= 2 * SM_THREADS) SM_FWD(2);
    else if (nv <= 4 * SM_THREADS) SM_FWD(4);
    else SM_FWD(8);
#undef SM_FWD
    return (int)cudaGetLastError();
  }
  GB_DISPATCH_FLOAT(dt, T, softmax_fwd_kernel<T><<<grid, row_block(cols), 0, st>>>((const T*)x, (T*)y, rows, cols, log_mode));
  return (int)cudaGetLastError();
}

// Softmax / log-softmax forward of rows of 8 KB and more through the streamed-row skeleton (csrc/row_stream.cuh)
namespace gb {
// NV = 16-byte vectors per thread kept in registers as floats (0: rows too long for that, three passes over the
// shared-memory copy instead).  With NV > 0 the row is read from shared memory once and every exponential is evaluated
// once.
template <typename T, int NV>
struct SoftmaxRowOp {
  T* y; int log_mode;
  struct State {};
  __device__ __forceinline__ void init(State&, int) const {}
  __device__ __forceinline__ void row(State&, const T* s, long long r, int cols, float* sh) const {
    constexpr int V = Vec16<T>::N;
    constexpr float L2E = 1.4426950408889634f;
    const int nv = cols / V;
    T* out = y + r * cols;
    if constexpr (NV > 0) {
      float e[NV][V];
      float mx = -INFINITY;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * RS_THREADS;
        if (i < nv) {
          const Vec16<T> a = *reinterpret_cast<const Vec16<T>*>(s + (size_t)i * V);
#pragma unroll
          for (int j = 0; j < V; ++j) { e[k][j] = Cvt<T>::to_f(a.v[j]); mx = fmaxf(mx, e[k][j]); }
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) e[k][j] = -INFINITY;
        }
      }
      mx = block_max(mx, sh);
      const float m = mx == -INFINITY ? 0.f : mx;          // a row of -inf gives zeros, not NaN
      const float m2 = m * L2E;
      float sum = 0.f;
      if (log_mode) {
#pragma unroll
        for (int k = 0; k < NV; ++k)
#pragma unroll
          for (int j = 0; j < V; ++j) sum += exp2f(fmaf(e[k][j], L2E, -m2));
      } else {
#pragma unroll
        for (int k = 0; k < NV; ++k)
#pragma unroll
          for (int j = 0; j < V; ++j) { e[k][j] = exp2f(fmaf(e[k][j], L2E, -m2)); sum += e[k][j]; }
      }
      sum = block_sum(sum, sh);
      const float inv = sum > 0.f ? 1.f / sum : 0.f, lse = m + __logf(sum);
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * RS_THREADS;
        if (i < nv) {
          Vec16<T> o;
#pragma unroll
          for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(log_mode ? e[k][j] - lse : e[k][j] * inv);
          st16(out + (size_t)i * V, o);
        }
      }
    } else {
      float mx = -INFINITY;
#pragma unroll 4
      for (int i = threadIdx.x; i < nv; i += RS_THREADS) {
        const Vec16<T> a = *reinterpret_cast<const Vec16<T>*>(s + (size_t)i * V);
#pragma unroll
        for (int j = 0; j < V; ++j) mx = fmaxf(mx, Cvt<T>::to_f(a.v[j]));
      }
      mx = block_max(mx, sh);
      const float m = mx == -INFINITY ? 0.f : mx;
      const float m2 = m * L2E;
      float sum = 0.f;
#pragma unroll 4
      for (int i = threadIdx.x; i < nv; i += RS_THREADS) {
        const Vec16<T> a = *reinterpret_cast<const Vec16<T>*>(s + (size_t)i * V);
#pragma unroll
        for (int j = 0; j < V; ++j) sum += exp2f(fmaf(Cvt<T>::to_f(a.v[j]), L2E, -m2));
      }
      sum = block_sum(sum, sh);
      const float inv = sum > 0.f ? 1.f / sum : 0.f, lse = m + __logf(sum);
#pragma unroll 4
      for (int i = threadIdx.x; i < nv; i += RS_THREADS) {
        const Vec16<T> a = *reinterpret_cast<const Vec16<T>*>(s + (size_t)i * V);
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float v = Cvt<T>::to_f(a.v[j]);
          o.v[j] = Cvt<T>::from_f(log_mode ? v - lse : exp2f(fmaf(v, L2E, -m2)) * inv);
        }
        st16(out + (size_t)i * V, o);
      }
    }
  }
};
}  // namespace gb

// Same contract as gb_softmax_fwd for rows of 8 to 64 KB; -9 when the shape does not qualify.
extern "C" int gb_softmax_fwd_stream(const void* x, void* y, long long rows, long long cols, int log_mode, int dt,
                                     int* status, cudaStream_t st) {
  if (rows == 0) return 0;
  const int es = dt == DT_F32 ? 4 : 2;
  if (cols >= (1ll << 30) || !rs_shape_ok(x, rows, cols, es) || (reinterpret_cast<uintptr_t>(y) & 15) != 0) return -9;
  const long long nvec = cols / (16 / es);
  const int per_thread = (int)((nvec + RS_THREADS - 1) / RS_THREADS);      // 16-byte vectors per thread
  static unsigned long long cfg[3][5] = {};
#define RS_SM(T, k, NVV, c) return rs_launch<T, SoftmaxRowOp<T, NVV>>((const T*)x, rows, (int)cols, SoftmaxRowOp<T, NVV>{(T*)y, log_mode}, status, cfg[k][c], st)
#define RS_SM_T(T, k, LIM)                                      \
  do {                                                          \
    if (per_thread <= 2) RS_SM(T, k, 2, 0);                     \
    if (per_thread <= 4) RS_SM(T, k, 4, 1);                     \
    if (per_thread <= 8 && 8 <= LIM) RS_SM(T, k, 8, 2);         \
    if (per_thread <= 16 && 16 <= LIM) RS_SM(T, k, 16, 3);      \
    RS_SM(T, k, 0, 4);                                          \
  } while (0)
  // at most 64 floats of the row per thread in registers: 16 vectors of 4 floats, 8 vectors of 8 halves
  if (dt == DT_F32) RS_SM_T(float, 0, 16);
  if (dt == DT_BF16) RS_SM_T(__nv_bfloat16, 1, 8);
  if (dt == DT_F16) RS_SM_T(__half, 2, 8);
#undef RS_SM_T
#undef RS_SM
  return -9;
}

extern "C" int gb_softmax_bwd(const void* g, const void* y, void* dx, long long rows, long long cols, int log_mode,
                              int dt, cudaStream_t st) {
  if (rows == 0) return 0;
  const int grid = (int)(rows < 148 * 16 ? rows : 148 * 16);
  const int vlen = dt == DT_F32 ? 4 : 8;
  const bool reg = cols % vlen == 0 && cols / vlen <= SM_THREADS * 4 && cols < (1ll << 30) &&
                   ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0;
  if (reg) {
    const long long nv = cols / vlen;
#define SM_BWD(MVV) GB_DISPATCH_FLOAT(dt, T, softmax_bwd_reg_kernel<T, MVV><<<grid, SM_THREADS, 0, st>>>((const T*)g, (const T*)y, (T*)dx, rows, (int)cols, log_mode))
    if (nv <= SM_THREADS) SM_BWD(1);
    else if (nv <= 2 * SM_THREADS) SM_BWD(2);
    else SM_BWD(4);
#undef SM_BWD
    return (int)cudaGetLastError();
  }
  GB_DISPATCH_FLOAT(dt, T, softmax_bwd_kernel<T><<<grid, row_block(cols), 0, st>>>((const T*)g, (const T*)y, (T*)dx, rows, cols, log_mode));
  return (int)cudaGetLastError();
}

extern "C" int gb_ce_fwd(const void* logits, const void* target, float* loss, float* lse, long long rows,
                         long long cols, long long ignore_index, int dt, int target_is_i64, cudaStream_t st) {
  if (rows == 0) return 0;
  const int grid = (int)(rows < 148 * 8 ? rows : 148 * 8);
  const int block = row_block(cols);
  if (target_is_i64) {
    GB_DISPATCH_FLOAT(dt, T, ce_fwd_kernel<T, long long><<<grid, block, 0, st>>>((const T*)logits, (const long long*)target, loss, lse, rows, cols, ignore_index));
  } else {
    GB_DISPATCH_FLOAT(dt, T, ce_fwd_kernel<T, int><<<grid, block, 0, st>>>((const T*)logits, (const int*)target, loss, lse, rows, cols, ignore_index));
  }
  return (int)cudaGetLastError();
}

extern "C" int gb_ce_bwd(const void* logits, const void* target, const float* lse, const float* grow, void* dlogits,
                         long long rows, long long cols, long long ignore_index, int dt, int target_is_i64,
                         cudaStream_t st) {
  if (rows == 0) return 0;
  const int grid = (int)(rows < 148 * 8 ? rows : 148 * 8);
  const int block = row_block(cols);
  if (target_is_i64) {
    GB_DISPATCH_FLOAT(dt, T, ce_bwd_kernel<T, long long><<<grid, block, 0, st>>>((const T*)logits, (const long long*)target, lse, grow, (T*)dlogits, rows, cols, ignore_index));
  } else {
    GB_DISPATCH_FLOAT(dt, T, ce_bwd_kernel<T, int><<<grid, block, 0, st>>>((const T*)logits, (const int*)target, lse, grow, (T*)dlogits, rows, cols, ignore_index));
  }
  return (int)cudaGetLastError();
}
