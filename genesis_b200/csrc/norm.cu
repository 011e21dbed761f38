// Fused RMSNorm and LayerNorm, forward and backward.  fp32 math, 128-bit loads, the row is read
// once and kept in registers between the statistics pass and the normalisation pass.  Weight/bias
// gradients are reduced deterministically: every CTA accumulates the rows it owns into a private
// fp32 partial row, and a second kernel sums the partials column-wise (no atomics, no spin locks).
// Reference counterparts: genesis/nn/triton_ops/rmsnorm.py:14-126, genesis/nn/layer_norm.py:15-213,
// genesis/nn/triton_ops/layer_norm.py:16-133.
#include "common.cuh"
#include "row_stream.cuh"

namespace gb {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV_LIMIT = 8;   // at most this many 16-byte vectors cached per thread

template <typename T, int NORM_MAXV>
__device__ __forceinline__ int load_row(const T* p, long long cols, Vec16<T> (&buf)[NORM_MAXV]) {
  constexpr int V = Vec16<T>::N;
  const int nv = (int)(cols / V);
  int cnt = 0;
#pragma unroll
  for (int k = 0; k < NORM_MAXV; ++k) {
    const int i = threadIdx.x + k * NORM_THREADS;
    if (i < nv) { buf[k] = ld16(p + (long long)i * V); cnt = k + 1; }
  }
  return cnt;
}

// V consecutive weights starting at element `base` (16-byte aligned: base is a multiple of V) as floats
template <typename TW, int V>
__device__ __forceinline__ void load_weights(const TW* __restrict__ w, int base, float (&out)[V]) {
  if constexpr (sizeof(TW) == 4) {
#pragma unroll
    for (int q = 0; q < V / 4; ++q) {
      const float4 f = *reinterpret_cast<const float4*>(w + base + 4 * q);
      out[4 * q] = f.x; out[4 * q + 1] = f.y; out[4 * q + 2] = f.z; out[4 * q + 3] = f.w;
    }
  } else {
    const Vec16<TW> f = ld16(w + base);
#pragma unroll
    for (int j = 0; j < V; ++j) out[j] = Cvt<TW>::to_f(f.v[j]);
  }
}

template <typename TW, int V>
__device__ __forceinline__ void load_weights_or(const TW* __restrict__ w, int base, float fill, float (&out)[V]) {
  if (w != nullptr) load_weights<TW, V>(w, base, out);
  else {
#pragma unroll
    for (int j = 0; j < V; ++j) out[j] = fill;
  }
}

// ------------------------------------------------------------------------------------------
// RMSNorm.  With `res` the forward kernels normalise s = x + res (rounded to T, as a separate addition would leave it)
// and also store s to `sum_out`: the residual addition of a pre-norm transformer block rides along with the
// normalisation that follows it.  With `gres` the backward kernels add the gradient that reaches s along the
// residual path to the one coming back through the normalisation.
// ------------------------------------------------------------------------------------------
template <typename T, int NORM_MAXV>
__device__ __forceinline__ void add_residual_row(const T* __restrict__ res, T* __restrict__ sum_out, int nv,
                                                 Vec16<T> (&buf)[NORM_MAXV]) {
  constexpr int V = Vec16<T>::N;
#pragma unroll
  for (int k = 0; k < NORM_MAXV; ++k) {
    const int i = threadIdx.x + k * NORM_THREADS;
    if (i < nv) {
      const Vec16<T> rb = ld16(res + (long long)i * V);
#pragma unroll
      for (int j = 0; j < V; ++j) buf[k].v[j] = Cvt<T>::from_f(Cvt<T>::to_f(buf[k].v[j]) + Cvt<T>::to_f(rb.v[j]));
      st16(sum_out + (long long)i * V, buf[k]);
    }
  }
}

template <typename T, typename TW, int NORM_MAXV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const T* __restrict__ x, const TW* __restrict__ w, T* __restrict__ y, float* __restrict__ rstd,
                   long long rows, int cols, float eps, const T* __restrict__ res = nullptr,
                   T* __restrict__ sum_out = nullptr) {
  __shared__ float sh[32];
  constexpr int V = Vec16<T>::N;
  const int nv = cols / V;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    Vec16<T> buf[NORM_MAXV];
    load_row<T, NORM_MAXV>(x + row * cols, cols, buf);
    if (res != nullptr) add_residual_row<T, NORM_MAXV>(res + row * cols, sum_out + row * cols, nv, buf);
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_MAXV; ++k)
      if (threadIdx.x + k * NORM_THREADS < nv)
#pragma unroll
        for (int j = 0; j < V; ++j) { float v = Cvt<T>::to_f(buf[k].v[j]); ss += v * v; }
    ss = block_sum(ss, sh);
    const float r = rsqrtf(ss / cols + eps);
    if (threadIdx.x == 0) rstd[row] = r;
#pragma unroll
    for (int k = 0; k < NORM_MAXV; ++k) {
      const int i = threadIdx.x + k * NORM_THREADS;
      if (i < nv) {
        Vec16<T> o;
        float wv[V];
        load_weights<TW, V>(w, i * V, wv);
#pragma unroll
        for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(Cvt<T>::to_f(buf[k].v[j]) * r * wv[j]);
        st16(y + row * cols + (long long)i * V, o);
      }
    }
  }
}

// dx = rstd * (g*w - xhat * mean(g*w*xhat));  dw partial[cta] += g * xhat
template <typename T, typename TW, int NORM_MAXV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const T* __restrict__ g, const T* __restrict__ x, const TW* __restrict__ w,
                   const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dw_partial,
                   long long rows, int cols, const T* __restrict__ gres = nullptr) {
  __shared__ float sh[32];
  constexpr int V = Vec16<T>::N;
  const int nv = cols / V;
  float dwacc[NORM_MAXV][V];
#pragma unroll
  for (int k = 0; k < NORM_MAXV; ++k)
#pragma unroll
    for (int j = 0; j < V; ++j) dwacc[k][j] = 0.f;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    Vec16<T> xb[NORM_MAXV], gb_[NORM_MAXV];
    load_row<T, NORM_MAXV>(x + row * cols, cols, xb);
    load_row<T, NORM_MAXV>(g + row * cols, cols, gb_);
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_MAXV; ++k) {
      const int i = threadIdx.x + k * NORM_THREADS;
      if (i < nv) {
        float wv[V];
        load_weights<TW, V>(w, i * V, wv);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = Cvt<T>::to_f(xb[k].v[j]) * r;
          const float gg = Cvt<T>::to_f(gb_[k].v[j]);
          dot += gg * wv[j] * xh;
          dwacc[k][j] += gg * xh;
        }
      }
    }
    dot = block_sum(dot, sh) / cols;
#pragma unroll
    for (int k = 0; k < NORM_MAXV; ++k) {
      const int i = threadIdx.x + k * NORM_THREADS;
      if (i < nv) {
        Vec16<T> o, gr;
        float wv[V];
        load_weights<TW, V>(w, i * V, wv);
        if (gres != nullptr) gr = ld16(gres + row * cols + (long long)i * V);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = Cvt<T>::to_f(xb[k].v[j]) * r;
          const float gw = Cvt<T>::to_f(gb_[k].v[j]) * wv[j];
          float d = r * (gw - xh * dot);
          if (gres != nullptr) d += Cvt<T>::to_f(gr.v[j]);
          o.v[j] = Cvt<T>::from_f(d);
        }
        st16(dx + row * cols + (long long)i * V, o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < NORM_MAXV; ++k) {
    const int i = threadIdx.x + k * NORM_THREADS;
    if (i < nv)
#pragma unroll
      for (int j = 0; j < V; ++j) dw_partial[(long long)blockIdx.x * cols + i * V + j] = dwacc[k][j];
  }
}

// ------------------------------------------------------------------------------------------
// RMSNorm for narrow rows (cols <= 32 lanes x MVW vectors): one WARP per row, eight rows in flight per CTA, warp
// shuffles instead of block barriers, the weight row held in registers for the whole kernel.  A row of 896 bf16
// values keeps only 112 of a CTA's 256 threads busy in the row-per-CTA kernels above and pays two barriers per row.
// ------------------------------------------------------------------------------------------
constexpr int NORM_WARPS = NORM_THREADS / 32;

template <typename T, typename TW, int MVW>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_warp_kernel(const T* __restrict__ x, const TW* __restrict__ w, T* __restrict__ y, float* __restrict__ rstd,
                        long long rows, int cols, float eps, const T* __restrict__ res = nullptr,
                        T* __restrict__ sum_out = nullptr) {
  constexpr int V = Vec16<T>::N;
  const int nv = cols / V;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float wv[MVW][V];
#pragma unroll
  for (int k = 0; k < MVW; ++k)
    if (lane + 32 * k < nv) load_weights<TW, V>(w, (lane + 32 * k) * V, wv[k]);
  for (long long row = (long long)blockIdx.x * NORM_WARPS + warp; row < rows; row += (long long)gridDim.x * NORM_WARPS) {
    Vec16<T> buf[MVW];
#pragma unroll
    for (int k = 0; k < MVW; ++k)
      if (lane + 32 * k < nv) buf[k] = ld16(x + row * cols + (long long)(lane + 32 * k) * V);
    if (res != nullptr) {
      Vec16<T> rb[MVW];                       // all loads of the row in flight before the first use
#pragma unroll
      for (int k = 0; k < MVW; ++k)
        if (lane + 32 * k < nv) rb[k] = ld16(res + row * cols + (long long)(lane + 32 * k) * V);
#pragma unroll
      for (int k = 0; k < MVW; ++k)
        if (lane + 32 * k < nv) {
#pragma unroll
          for (int j = 0; j < V; ++j)
            buf[k].v[j] = Cvt<T>::from_f(Cvt<T>::to_f(buf[k].v[j]) + Cvt<T>::to_f(rb[k].v[j]));
          st16(sum_out + row * cols + (long long)(lane + 32 * k) * V, buf[k]);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < MVW; ++k)
      if (lane + 32 * k < nv)
#pragma unroll
        for (int j = 0; j < V; ++j) { const float v = Cvt<T>::to_f(buf[k].v[j]); ss += v * v; }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / cols + eps);
    if (lane == 0) rstd[row] = r;
#pragma unroll
    for (int k = 0; k < MVW; ++k)
      if (lane + 32 * k < nv) {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(Cvt<T>::to_f(buf[k].v[j]) * r * wv[k][j]);
        st16(y + row * cols + (long long)(lane + 32 * k) * V, o);
      }
  }
}

// Backward for narrow rows.  A row's gradient needs the whole row twice (dot product, then the result), so a warp that
// loads, reduces and stores one row at a time leaves the memory system idle half of the time.  Here every lane runs a
// private ring of asynchronous 16-byte copies (cp.async, global -> shared, no registers held): the operands of the
// next RING-1 rows of its warp are in flight while the current row is reduced.  A lane reads back only the slots it
// copied itself, so the ring needs no barriers, and cp.async.wait_group is a dependency wait, not a spin.
// One CTA per SM (the ring takes up to 144 KB), grid = at most 148 CTAs, each writing one row of the dw partials.
constexpr int NORM_RING = 2;
constexpr int NORM_BWD_THREADS = 512;                      // 16 warps: enough rows in progress to hide the per-row chain
constexpr int NORM_BWD_WARPS = NORM_BWD_THREADS / 32;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
               "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T, typename TW, int MVW>
__global__ void __launch_bounds__(NORM_BWD_THREADS, 1)
rmsnorm_bwd_warp_kernel(const T* __restrict__ g, const T* __restrict__ x, const TW* __restrict__ w,
                        const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dw_partial,
                        long long rows, int cols, const T* __restrict__ gres = nullptr) {
  constexpr int V = Vec16<T>::N;
  extern __shared__ __align__(16) unsigned char norm_smem[];
  const int nv = cols / V;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t row_bytes = (size_t)cols * sizeof(T);                       // a multiple of 16
  unsigned char* ring = norm_smem + (size_t)warp * NORM_RING * 3 * row_bytes;   // [stage][x | g | gres][row]
  const long long stride = (long long)gridDim.x * NORM_BWD_WARPS;
  const long long first = (long long)blockIdx.x * NORM_BWD_WARPS + warp;

  auto issue = [&](long long row, int stage) {
    if (row < rows) {
      unsigned char* base = ring + (size_t)stage * 3 * row_bytes;
#pragma unroll
      for (int k = 0; k < MVW; ++k) {
        const int i = lane + 32 * k;
        if (i < nv) {
          const long long off = row * cols + (long long)i * V;
          cp_async16(base + (size_t)i * 16, x + off);
          cp_async16(base + row_bytes + (size_t)i * 16, g + off);
          if (gres != nullptr) cp_async16(base + 2 * row_bytes + (size_t)i * 16, gres + off);
        }
      }
    }
    cp_async_commit();                                   // an empty group keeps the count uniform past the last row
  };

  float dwacc[MVW][V];
#pragma unroll
  for (int k = 0; k < MVW; ++k)
#pragma unroll
    for (int j = 0; j < V; ++j) dwacc[k][j] = 0.f;
#pragma unroll
  for (int st = 0; st < NORM_RING - 1; ++st) issue(first + st * stride, st);
  int stage = 0;
  for (long long row = first; row < rows; row += stride) {
    // refill the stage that the previous iteration consumed, then wait for this row's group (the oldest)
    issue(row + (NORM_RING - 1) * stride, (stage + NORM_RING - 1) % NORM_RING);
    cp_async_wait<NORM_RING - 1>();
    const unsigned char* base = ring + (size_t)stage * 3 * row_bytes;
    // both passes read the operands from the ring (shared memory) instead of holding them in registers
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < MVW; ++k)
      if (lane + 32 * k < nv) {
        const Vec16<T> xb = *reinterpret_cast<const Vec16<T>*>(base + (size_t)(lane + 32 * k) * 16);
        const Vec16<T> gb_ = *reinterpret_cast<const Vec16<T>*>(base + row_bytes + (size_t)(lane + 32 * k) * 16);
        float wv[V];
        load_weights<TW, V>(w, (lane + 32 * k) * V, wv);   // 3.5 KB row, resident in L1
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = Cvt<T>::to_f(xb.v[j]) * r;
          const float gg = Cvt<T>::to_f(gb_.v[j]);
          dot += gg * wv[j] * xh;
          dwacc[k][j] += gg * xh;
        }
      }
    dot = warp_sum(dot) / cols;
#pragma unroll
    for (int k = 0; k < MVW; ++k)
      if (lane + 32 * k < nv) {
        const Vec16<T> xb = *reinterpret_cast<const Vec16<T>*>(base + (size_t)(lane + 32 * k) * 16);
        const Vec16<T> gb_ = *reinterpret_cast<const Vec16<T>*>(base + row_bytes + (size_t)(lane + 32 * k) * 16);
        Vec16<T> o, gr;
        float wv[V];
        load_weights<TW, V>(w, (lane + 32 * k) * V, wv);
        if (gres != nullptr) gr = *reinterpret_cast<const Vec16<T>*>(base + 2 * row_bytes + (size_t)(lane + 32 * k) * 16);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = Cvt<T>::to_f(xb.v[j]) * r;
          float d = r * (Cvt<T>::to_f(gb_.v[j]) * wv[j] - xh * dot);
          if (gres != nullptr) d += Cvt<T>::to_f(gr.v[j]);
          o.v[j] = Cvt<T>::from_f(d);
        }
        st16(dx + row * cols + (long long)(lane + 32 * k) * V, o);
      }
    stage = (stage + 1) % NORM_RING;
  }
  cp_async_wait<0>();
  __syncthreads();                                       // every warp is done with its ring: reuse it for the reduction
  // this CTA's partial weight gradient: sum over its warps in a fixed order, one row of the partial buffer
  constexpr int RED_LD = 32 * MVW * V + 1;
  float* red = reinterpret_cast<float*>(norm_smem);
#pragma unroll
  for (int k = 0; k < MVW; ++k)
#pragma unroll
    for (int j = 0; j < V; ++j) red[warp * RED_LD + (lane + 32 * k) * V + j] = dwacc[k][j];
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += NORM_BWD_THREADS) {
    float sacc = 0.f;
#pragma unroll
    for (int wq = 0; wq < NORM_BWD_WARPS; ++wq) sacc += red[wq * RED_LD + c];
    dw_partial[(long long)blockIdx.x * cols + c] = sacc;
  }
}

// dynamic shared memory of the kernel above: the per-warp rings, or the reduction buffer if that is larger
static inline size_t rmsnorm_bwd_warp_smem(int cols, int esize, int mvw) {
  const size_t ring = (size_t)NORM_BWD_WARPS * NORM_RING * 3 * cols * esize;
  const size_t red = (size_t)NORM_BWD_WARPS * (32 * mvw * (16 / esize) + 1) * sizeof(float);
  return ring > red ? ring : red;
}

// ------------------------------------------------------------------------------------------
// LayerNorm
// ------------------------------------------------------------------------------------------
template <typename T, typename TW, int NORM_MAXV>
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_fwd_kernel(const T* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b, T* __restrict__ y,
                     float* __restrict__ mean, float* __restrict__ rstd, long long rows, int cols, float eps) {
  __shared__ float sh[32];
  constexpr int V = Vec16<T>::N;
  const int nv = cols / V;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    Vec16<T> buf[NORM_MAXV];
    load_row<T, NORM_MAXV>(x + row * cols, cols, buf);
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_MAXV; ++k)
      if (threadIdx.x + k * NORM_THREADS < nv)
#pragma unroll
        for (int j = 0; j < V; ++j) s += Cvt<T>::to_f(buf[k].v[j]);
    const float mu = block_sum(s, sh) / cols;
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_MAXV; ++k)
      if (threadIdx.x + k * NORM_THREADS < nv)
#pragma unroll
        for (int j = 0; j < V; ++j) { float d = Cvt<T>::to_f(buf[k].v[j]) - mu; ss += d * d; }
    const float r = rsqrtf(block_sum(ss, sh) / cols + eps);
    if (threadIdx.x == 0) { mean[row] = mu; rstd[row] = r; }
#pragma unroll
    for (int k = 0; k < NORM_MAXV; ++k) {
      const int i = threadIdx.x + k * NORM_THREADS;
      if (i < nv) {
        Vec16<T> o;
        float wv[V], bv[V];
        load_weights_or<TW, V>(w, i * V, 1.f, wv);
        load_weights_or<TW, V>(b, i * V, 0.f, bv);
#pragma unroll
        for (int j = 0; j < V; ++j)
          o.v[j] = Cvt<T>::from_f((Cvt<T>::to_f(buf[k].v[j]) - mu) * r * wv[j] + bv[j]);
        st16(y + row * cols + (long long)i * V, o);
      }
    }
  }
}

template <typename T, typename TW, int NORM_MAXV>
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_bwd_kernel(const T* __restrict__ g, const T* __restrict__ x, const TW* __restrict__ w,
                     const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
                     float* __restrict__ dw_partial, float* __restrict__ db_partial, long long rows, int cols) {
  __shared__ float sh[32];
  constexpr int V = Vec16<T>::N;
  const int nv = cols / V;
  float dwacc[NORM_MAXV][V], dbacc[NORM_MAXV][V];
#pragma unroll
  for (int k = 0; k < NORM_MAXV; ++k)
#pragma unroll
    for (int j = 0; j < V; ++j) { dwacc[k][j] = 0.f; dbacc[k][j] = 0.f; }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    Vec16<T> xb[NORM_MAXV], gb_[NORM_MAXV];
    load_row<T, NORM_MAXV>(x + row * cols, cols, xb);
    load_row<T, NORM_MAXV>(g + row * cols, cols, gb_);
    const float mu = mean[row], r = rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_MAXV; ++k) {
      const int i = threadIdx.x + k * NORM_THREADS;
      if (i < nv) {
        float wv[V];
        load_weights_or<TW, V>(w, i * V, 1.f, wv);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = (Cvt<T>::to_f(xb[k].v[j]) - mu) * r;
          const float gg = Cvt<T>::to_f(gb_[k].v[j]);
          const float gw = gg * wv[j];
          s1 += gw;
          s2 += gw * xh;
          dwacc[k][j] += gg * xh;
          dbacc[k][j] += gg;
        }
      }
    }
    s1 = block_sum(s1, sh) / cols;
    s2 = block_sum(s2, sh) / cols;
#pragma unroll
    for (int k = 0; k < NORM_MAXV; ++k) {
      const int i = threadIdx.x + k * NORM_THREADS;
      if (i < nv) {
        Vec16<T> o;
        float wv[V];
        load_weights_or<TW, V>(w, i * V, 1.f, wv);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = (Cvt<T>::to_f(xb[k].v[j]) - mu) * r;
          const float gw = Cvt<T>::to_f(gb_[k].v[j]) * wv[j];
          o.v[j] = Cvt<T>::from_f(r * (gw - s1 - xh * s2));
        }
        st16(dx + row * cols + (long long)i * V, o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < NORM_MAXV; ++k) {
    const int i = threadIdx.x + k * NORM_THREADS;
    if (i < nv)
#pragma unroll
      for (int j = 0; j < V; ++j) {
        dw_partial[(long long)blockIdx.x * cols + i * V + j] = dwacc[k][j];
        db_partial[(long long)blockIdx.x * cols + i * V + j] = dbacc[k][j];
      }
  }
}

}  // namespace gb

using namespace gb;

#define NORM_DISPATCH_T(dt, wdt, ...)                                                            \
  do {                                                                                           \
    if (dt == DT_F32 && wdt == DT_F32) { using T = float; using TW = float; __VA_ARGS__; }       \
    else if (dt == DT_BF16 && wdt == DT_F32) { using T = __nv_bfloat16; using TW = float; __VA_ARGS__; } \
    else if (dt == DT_F16 && wdt == DT_F32) { using T = __half; using TW = float; __VA_ARGS__; } \
    else if (dt == DT_BF16 && wdt == DT_BF16) { using T = __nv_bfloat16; using TW = __nv_bfloat16; __VA_ARGS__; } \
    else if (dt == DT_F16 && wdt == DT_F16) { using T = __half; using TW = __half; __VA_ARGS__; } \
    else return -2;                                                                              \
  } while (0)

// MV = 16-byte vectors cached per thread, the smallest of {1, 2, 4, 8} that covers a row
#define NORM_DISPATCH(dt, wdt, cols, ...)                                                        \
  do {                                                                                           \
    const int nvec_ = (cols) / ((dt) == DT_F32 ? 4 : 8);                                         \
    if (nvec_ <= NORM_THREADS) { constexpr int MV = 1; NORM_DISPATCH_T(dt, wdt, __VA_ARGS__); }  \
    else if (nvec_ <= 2 * NORM_THREADS) { constexpr int MV = 2; NORM_DISPATCH_T(dt, wdt, __VA_ARGS__); } \
    else if (nvec_ <= 4 * NORM_THREADS) { constexpr int MV = 4; NORM_DISPATCH_T(dt, wdt, __VA_ARGS__); } \
    else { constexpr int MV = 8; NORM_DISPATCH_T(dt, wdt, __VA_ARGS__); }                        \
  } while (0)

static inline bool norm_cols_ok(int cols, int dt) {
  const int v = dt == DT_F32 ? 4 : 8;
  return cols % v == 0 && cols / v <= NORM_THREADS * NORM_MAXV_LIMIT;
}

// Number of CTAs the backward kernels use (= rows of the partial buffers).
extern "C" int gb_norm_bwd_ctas(long long rows) { return (int)(rows < 148 * 4 ? rows : 148 * 4); }

static int rmsnorm_fwd_impl(const void* x, const void* w, void* y, float* rstd, long long rows, int cols, float eps,
                            int dt, int wdt, const void* res, void* sum_out, cudaStream_t st);

extern "C" int gb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int cols,
                              float eps, int dt, int wdt, cudaStream_t st) {
  return rmsnorm_fwd_impl(x, w, y, rstd, rows, cols, eps, dt, wdt, nullptr, nullptr, st);
}

// sum_out = x + res, y = rmsnorm(sum_out) * w, one pass
extern "C" int gb_add_rmsnorm_fwd(const void* x, const void* res, void* sum_out, const void* w, void* y, float* rstd,
                                  long long rows, int cols, float eps, int dt, int wdt, cudaStream_t st) {
  if (res == nullptr || sum_out == nullptr) return -3;
  return rmsnorm_fwd_impl(x, w, y, rstd, rows, cols, eps, dt, wdt, res, sum_out, st);
}

static int rmsnorm_fwd_impl(const void* x, const void* w, void* y, float* rstd, long long rows, int cols, float eps,
                            int dt, int wdt, const void* res, void* sum_out, cudaStream_t st) {
  if (rows == 0) return 0;
  if (!norm_cols_ok(cols, dt)) return -2;
  const int grid = (int)(rows < 148 * 8 ? rows : 148 * 8);
  const int nvec = cols / (dt == DT_F32 ? 4 : 8);
  if (nvec <= 128 && rows >= 64) {
    // narrow rows: warp per row (MVW = 1, 2 or 4 vectors per lane)
    const long long want = (rows + NORM_WARPS - 1) / NORM_WARPS;
    const int wgrid = (int)(want < 148 * 8 ? want : 148 * 8);
    if (nvec <= 32) { NORM_DISPATCH_T(dt, wdt, rmsnorm_fwd_warp_kernel<T, TW, 1><<<wgrid, NORM_THREADS, 0, st>>>((const T*)x, (const TW*)w, (T*)y, rstd, rows, cols, eps, (const T*)res, (T*)sum_out)); }
    else if (nvec <= 64) { NORM_DISPATCH_T(dt, wdt, rmsnorm_fwd_warp_kernel<T, TW, 2><<<wgrid, NORM_THREADS, 0, st>>>((const T*)x, (const TW*)w, (T*)y, rstd, rows, cols, eps, (const T*)res, (T*)sum_out)); }
    else { NORM_DISPATCH_T(dt, wdt, rmsnorm_fwd_warp_kernel<T, TW, 4><<<wgrid, NORM_THREADS, 0, st>>>((const T*)x, (const TW*)w, (T*)y, rstd, rows, cols, eps, (const T*)res, (T*)sum_out)); }
    return (int)cudaGetLastError();
  }
  NORM_DISPATCH(dt, wdt, cols, rmsnorm_fwd_kernel<T, TW, MV><<<grid, NORM_THREADS, 0, st>>>(
      (const T*)x, (const TW*)w, (T*)y, rstd, rows, cols, eps, (const T*)res, (T*)sum_out));
  return (int)cudaGetLastError();
}

// RMSNorm forward of rows of 8 KB and more through the streamed-row skeleton (csrc/row_stream.cuh)
namespace gb {
// NV > 0: every thread owns at most NV 16-byte vectors of a row, always the same columns, so their weights are loaded
// once per CTA and stay in registers for all rows (re-reading 64 KB of weights per row through an L1 that the row
// buffers leave little room in was the largest stall of the first version); NV = 0: weights read per row.
template <typename T, typename TW, int NV>
struct RmsRowOp {
  const TW* w; T* y; float* rstd; float eps;
  static constexpr int V = Vec16<T>::N;
  struct State { float wv[NV > 0 ? NV : 1][V]; };
  __device__ __forceinline__ void init(State& st, int cols) const {
    if constexpr (NV > 0) {
      const int nv = cols / V;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * RS_THREADS;
        if (i < nv) load_weights<TW, V>(w, i * V, st.wv[k]);
      }
    }
  }
  __device__ __forceinline__ void row(State& st, const T* s, long long r, int cols, float* sh) const {
    const int nv = cols / V;
    T* out = y + r * cols;
    if constexpr (NV > 0) {
      Vec16<T> a[NV];
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * RS_THREADS;
        if (i < nv) {
          a[k] = *reinterpret_cast<const Vec16<T>*>(s + (size_t)i * V);
#pragma unroll
          for (int j = 0; j < V; ++j) { const float v = Cvt<T>::to_f(a[k].v[j]); ss += v * v; }
        }
      }
      ss = block_sum(ss, sh);
      const float rr = rsqrtf(ss / cols + eps);
      if (threadIdx.x == 0) rstd[r] = rr;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * RS_THREADS;
        if (i < nv) {
          Vec16<T> o;
#pragma unroll
          for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(Cvt<T>::to_f(a[k].v[j]) * rr * st.wv[k][j]);
          st16(out + (size_t)i * V, o);
        }
      }
    } else {
      float ss = 0.f;
#pragma unroll 4
      for (int i = threadIdx.x; i < nv; i += RS_THREADS) {
        const Vec16<T> a = *reinterpret_cast<const Vec16<T>*>(s + (size_t)i * V);
#pragma unroll
        for (int j = 0; j < V; ++j) { const float v = Cvt<T>::to_f(a.v[j]); ss += v * v; }
      }
      ss = block_sum(ss, sh);
      const float rr = rsqrtf(ss / cols + eps);
      if (threadIdx.x == 0) rstd[r] = rr;
#pragma unroll 4
      for (int i = threadIdx.x; i < nv; i += RS_THREADS) {
        const Vec16<T> a = *reinterpret_cast<const Vec16<T>*>(s + (size_t)i * V);
        float wv[V];
        load_weights<TW, V>(w, i * V, wv);
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(Cvt<T>::to_f(a.v[j]) * rr * wv[j]);
        st16(out + (size_t)i * V, o);
      }
    }
  }
};
}  // namespace gb

// Same contract as gb_rmsnorm_fwd for rows of 8 to 64 KB; returns -9 when the shape does not qualify (the caller then
// uses gb_rmsnorm_fwd).  `status`: the library's status word (a copy that never arrives is reported there).
extern "C" int gb_rmsnorm_fwd_stream(const void* x, const void* w, void* y, float* rstd, long long rows, int cols,
                                     float eps, int dt, int wdt, int* status, cudaStream_t st) {
  if (rows == 0) return 0;
  const int es = dt == DT_F32 ? 4 : 2;
  if (!rs_shape_ok(x, rows, cols, es) || (reinterpret_cast<uintptr_t>(y) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(w) & 15) != 0)
    return -9;
  const long long nvec = (long long)cols / (16 / es);
  const int per_thread = (int)((nvec + RS_THREADS - 1) / RS_THREADS);      // 16-byte vectors per thread
  static unsigned long long cfg[5][4] = {};
#define RS_RMS1(T, TW, k, NVV, c) return rs_launch<T, RmsRowOp<T, TW, NVV>>((const T*)x, rows, cols, RmsRowOp<T, TW, NVV>{(const TW*)w, (T*)y, rstd, eps}, status, cfg[k][c], st)
#define RS_RMS(T, TW, k)                         \
  do {                                           \
    if (per_thread <= 2) RS_RMS1(T, TW, k, 2, 0); \
    if (per_thread <= 4) RS_RMS1(T, TW, k, 4, 1); \
    if (per_thread <= 8) RS_RMS1(T, TW, k, 8, 2); \
    RS_RMS1(T, TW, k, 0, 3);                      \
  } while (0)
  if (dt == DT_F32 && wdt == DT_F32) RS_RMS(float, float, 0);
  if (dt == DT_BF16 && wdt == DT_F32) RS_RMS(__nv_bfloat16, float, 1);
  if (dt == DT_F16 && wdt == DT_F32) RS_RMS(__half, float, 2);
  if (dt == DT_BF16 && wdt == DT_BF16) RS_RMS(__nv_bfloat16, __nv_bfloat16, 3);
  if (dt == DT_F16 && wdt == DT_F16) RS_RMS(__half, __half, 4);
#undef RS_RMS
#undef RS_RMS1
  return -9;
}

static int rmsnorm_bwd_impl(const void* g, const void* x, const void* w, const float* rstd, void* dx,
                            float* dw_partial, long long rows, int cols, int dt, int wdt, const void* gres,
                            cudaStream_t st);

extern "C" int gb_rmsnorm_bwd(const void* g, const void* x, const void* w, const float* rstd, void* dx,
                              float* dw_partial, long long rows, int cols, int dt, int wdt, cudaStream_t st) {
  return rmsnorm_bwd_impl(g, x, w, rstd, dx, dw_partial, rows, cols, dt, wdt, nullptr, st);
}

// dx = rmsnorm_backward(g) + gres: the gradient of s = x + res with respect to either addend
extern "C" int gb_add_rmsnorm_bwd(const void* g, const void* gres, const void* x, const void* w, const float* rstd,
                                  void* dx, float* dw_partial, long long rows, int cols, int dt, int wdt,
                                  cudaStream_t st) {
  return rmsnorm_bwd_impl(g, x, w, rstd, dx, dw_partial, rows, cols, dt, wdt, gres, st);
}

template <typename T, typename TW, int MVW>
static int launch_rmsnorm_bwd_warp(const void* g, const void* x, const void* w, const float* rstd, void* dx,
                                   float* dw_partial, long long rows, int cols, const void* gres, int grid,
                                   cudaStream_t st) {
  const size_t smem = rmsnorm_bwd_warp_smem(cols, (int)sizeof(T), MVW);
  static unsigned long long configured = 0;              // per instantiation and device: opt in to > 48 KB
  if (int e = smem_opt_in(rmsnorm_bwd_warp_kernel<T, TW, MVW>, 200 * 1024, configured)) return e;
  rmsnorm_bwd_warp_kernel<T, TW, MVW><<<grid, NORM_BWD_THREADS, smem, st>>>(
      (const T*)g, (const T*)x, (const TW*)w, rstd, (T*)dx, dw_partial, rows, cols, (const T*)gres);
  return (int)cudaGetLastError();
}

static inline bool rmsnorm_bwd_uses_warp_kernel(long long rows, int cols, int dt) {
  return cols / (dt == DT_F32 ? 4 : 8) <= 128 && rows >= 64;
}

// Number of CTAs gb_rmsnorm_bwd / gb_add_rmsnorm_bwd launch (= rows of dw_partial they write)
extern "C" int gb_rmsnorm_bwd_ctas(long long rows, int cols, int dt) {
  if (rmsnorm_bwd_uses_warp_kernel(rows, cols, dt)) {
    const long long want = (rows + NORM_BWD_WARPS - 1) / NORM_BWD_WARPS;
    return (int)(want < 148 ? want : 148);
  }
  return gb_norm_bwd_ctas(rows);
}

static int rmsnorm_bwd_impl(const void* g, const void* x, const void* w, const float* rstd, void* dx,
                            float* dw_partial, long long rows, int cols, int dt, int wdt, const void* gres,
                            cudaStream_t st) {
  if (rows == 0) return 0;
  if (!norm_cols_ok(cols, dt)) return -2;
  const int grid = gb_rmsnorm_bwd_ctas(rows, cols, dt);
  const int nvec = cols / (dt == DT_F32 ? 4 : 8);
  if (rmsnorm_bwd_uses_warp_kernel(rows, cols, dt)) {
    // narrow rows: warp per row; every CTA of the grid writes its row of the partial buffer
    if (nvec <= 32) { NORM_DISPATCH_T(dt, wdt, return (launch_rmsnorm_bwd_warp<T, TW, 1>(g, x, w, rstd, dx, dw_partial, rows, cols, gres, grid, st))); }
    else if (nvec <= 64) { NORM_DISPATCH_T(dt, wdt, return (launch_rmsnorm_bwd_warp<T, TW, 2>(g, x, w, rstd, dx, dw_partial, rows, cols, gres, grid, st))); }
    else { NORM_DISPATCH_T(dt, wdt, return (launch_rmsnorm_bwd_warp<T, TW, 4>(g, x, w, rstd, dx, dw_partial, rows, cols, gres, grid, st))); }
  }
  NORM_DISPATCH(dt, wdt, cols, rmsnorm_bwd_kernel<T, TW, MV><<<grid, NORM_THREADS, 0, st>>>(
      (const T*)g, (const T*)x, (const TW*)w, rstd, (T*)dx, dw_partial, rows, cols, (const T*)gres));
  return (int)cudaGetLastError();
}

extern "C" int gb_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                                long long rows, int cols, float eps, int dt, int wdt, cudaStream_t st) {
  if (rows == 0) return 0;
  if (!norm_cols_ok(cols, dt)) return -2;
  const int grid = (int)(rows < 148 * 8 ? rows : 148 * 8);
  NORM_DISPATCH(dt, wdt, cols, layernorm_fwd_kernel<T, TW, MV><<<grid, NORM_THREADS, 0, st>>>(
      (const T*)x, (const TW*)w, (const TW*)b, (T*)y, mean, rstd, rows, cols, eps));
  return (int)cudaGetLastError();
}

extern "C" int gb_layernorm_bwd(const void* g, const void* x, const void* w, const float* mean, const float* rstd,
                                void* dx, float* dw_partial, float* db_partial, long long rows, int cols, int dt,
                                int wdt, cudaStream_t st) {
  if (rows == 0) return 0;
  if (!norm_cols_ok(cols, dt)) return -2;
  const int grid = gb_norm_bwd_ctas(rows);
  NORM_DISPATCH(dt, wdt, cols, layernorm_bwd_kernel<T, TW, MV><<<grid, NORM_THREADS, 0, st>>>(
      (const T*)g, (const T*)x, (const TW*)w, mean, rstd, (T*)dx, dw_partial, db_partial, rows, cols));
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// RMSNorm backward without any allocation (declared in noalloc.h; no counterpart in the reference)
// ------------------------------------------------------------------------------------------------
// The regular entry point takes its per-CTA partial sums of the weight gradient from a buffer the
// caller allocates.  Some callers cannot allocate at all at the point where they need this kernel:
// code that runs under somebody else's memory manager with a fixed budget (a serving process that
// pre-sized its pools, a plugin inside another runtime) and code in a latency-critical loop where
// cudaMalloc / cudaFree are off limits because they synchronise the whole device.  For them the
// scratch lives in the library image itself.
namespace gb {

constexpr int NOALLOC_MAX_CTAS = 296;    // two CTAs per SM on a 148-SM part
constexpr int NOALLOC_MAX_COLS = 4096;   // widest row this entry point accepts

// 296 x 4096 floats = 4.6 MiB, resident on every GPU that loads the library until the process exits.
static __device__ __align__(256) float g_rmsnorm_bwd_scratch[NOALLOC_MAX_CTAS * NOALLOC_MAX_COLS];

// dw[c] = sum over the nct partial rows; one thread per column, fixed order => deterministic
__global__ void noalloc_colsum_kernel(const float* __restrict__ partial, float* __restrict__ dw, int nct, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float acc = 0.f;
  for (int r = 0; r < nct; ++r) acc += partial[(long long)r * cols + c];
  dw[c] = acc;
}

}  // namespace gb

#include <mutex>

namespace {
constexpr int kNoallocMaxDevices = 64;
float* g_scratch_ptr[kNoallocMaxDevices] = {nullptr};
std::mutex g_scratch_mu;
}  // namespace

extern "C" const char* gb_rmsnorm_bwd_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -10: return "rmsnorm_bwd_noalloc: cols exceeds the built-in scratch (max 4096 columns)";
    case -11: return "rmsnorm_bwd_noalloc: cols must be a multiple of 8 (16-bit) or 4 (float32) elements";
    case -12: return "rmsnorm_bwd_noalloc: unsupported dtype combination";
    case -13: return "rmsnorm_bwd_noalloc: device index out of range";
    default: return "rmsnorm_bwd_noalloc: CUDA runtime error (code is the cudaError_t value)";
  }
}

extern "C" int gb_rmsnorm_bwd_noalloc_max_cols() { return gb::NOALLOC_MAX_COLS; }

extern "C" int gb_rmsnorm_bwd_noalloc(const void* g, const void* x, const void* w, const float* rstd, void* dx,
                                      float* dw, long long rows, int cols, int dt, int wdt, cudaStream_t st) {
  if (cols > gb::NOALLOC_MAX_COLS) return -10;
  if (cols % (dt == DT_F32 ? 4 : 8) != 0 || cols <= 0) return -11;
  // no rows: the sum over rows is zero, and `dw` is documented as overwritten
  if (rows <= 0) return (int)cudaMemsetAsync(dw, 0, (size_t)cols * sizeof(float), st);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoallocMaxDevices) return -13;
  float* scratch;
  {
    // Set-up, once per device, with that device current: inside host code the array's name is only a
    // stand-in, the address a kernel may use comes from cudaGetSymbolAddress.
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (g_scratch_ptr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, gb::g_rmsnorm_bwd_scratch);
      if (e != cudaSuccess) return (int)e;
      g_scratch_ptr[dev] = static_cast<float*>(p);
    }
    scratch = g_scratch_ptr[dev];
  }
  const int grid = (int)(rows < gb::NOALLOC_MAX_CTAS ? rows : gb::NOALLOC_MAX_CTAS);
  // every CTA overwrites its whole partial row, so nothing in the scratch has to be cleared first
  do {
    const int nvec_ = cols / (dt == DT_F32 ? 4 : 8);
    if (nvec_ <= NORM_THREADS) {
      constexpr int MV = 1;
      if (dt == DT_F32 && wdt == DT_F32) rmsnorm_bwd_kernel<float, float, MV><<<grid, NORM_THREADS, 0, st>>>((const float*)g, (const float*)x, (const float*)w, rstd, (float*)dx, scratch, rows, cols);
      else if (dt == DT_BF16 && wdt == DT_F32) rmsnorm_bwd_kernel<__nv_bfloat16, float, MV><<<grid, NORM_THREADS, 0, st>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)x, (const float*)w, rstd, (__nv_bfloat16*)dx, scratch, rows, cols);
      else if (dt == DT_F16 && wdt == DT_F32) rmsnorm_bwd_kernel<__half, float, MV><<<grid, NORM_THREADS, 0, st>>>((const __half*)g, (const __half*)x, (const float*)w, rstd, (__half*)dx, scratch, rows, cols);
      else if (dt == DT_BF16 && wdt == DT_BF16) rmsnorm_bwd_kernel<__nv_bfloat16, __nv_bfloat16, MV><<<grid, NORM_THREADS, 0, st>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, scratch, rows, cols);
      else if (dt == DT_F16 && wdt == DT_F16) rmsnorm_bwd_kernel<__half, __half, MV><<<grid, NORM_THREADS, 0, st>>>((const __half*)g, (const __half*)x, (const __half*)w, rstd, (__half*)dx, scratch, rows, cols);
      else return -12;
    } else {
      constexpr int MV = 4;   // up to 4 vectors per thread covers 4096 fp32 / 8192 16-bit columns
      if (dt == DT_F32 && wdt == DT_F32) rmsnorm_bwd_kernel<float, float, MV><<<grid, NORM_THREADS, 0, st>>>((const float*)g, (const float*)x, (const float*)w, rstd, (float*)dx, scratch, rows, cols);
      else if (dt == DT_BF16 && wdt == DT_F32) rmsnorm_bwd_kernel<__nv_bfloat16, float, MV><<<grid, NORM_THREADS, 0, st>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)x, (const float*)w, rstd, (__nv_bfloat16*)dx, scratch, rows, cols);
      else if (dt == DT_F16 && wdt == DT_F32) rmsnorm_bwd_kernel<__half, float, MV><<<grid, NORM_THREADS, 0, st>>>((const __half*)g, (const __half*)x, (const float*)w, rstd, (__half*)dx, scratch, rows, cols);
      else if (dt == DT_BF16 && wdt == DT_BF16) rmsnorm_bwd_kernel<__nv_bfloat16, __nv_bfloat16, MV><<<grid, NORM_THREADS, 0, st>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, scratch, rows, cols);
      else if (dt == DT_F16 && wdt == DT_F16) rmsnorm_bwd_kernel<__half, __half, MV><<<grid, NORM_THREADS, 0, st>>>((const __half*)g, (const __half*)x, (const __half*)w, rstd, (__half*)dx, scratch, rows, cols);
      else return -12;
    }
  } while (0);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  gb::noalloc_colsum_kernel<<<(cols + 127) / 128, 128, 0, st>>>(scratch, dw, grid, cols);
  return (int)cudaGetLastError();
}
