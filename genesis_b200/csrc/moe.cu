// Mixture-of-experts routing kernels.
//   router forward : softmax over experts + top-k + renormalisation + per-expert histogram, one warp
//                    per token, one launch (reference: softmax kernel + k sequential arg-max launches +
//                    bincount, genesis/ops/cuda/tensor_ops.py:429-623)
//   router backward: gradient of the above w.r.t. the logits
//   sort           : counting sort of the (token, slot) pairs by expert into segments padded to a
//                    multiple of `align` rows (what the grouped GEMM consumes); replaces the reference's
//                    argsort = N sequential launches (tensor_ops.py:236-322)
#include "common.cuh"

namespace gb {

constexpr int ROUTER_MAX_PER_LANE = 8;   // experts <= 256

template <typename T>
__global__ void router_fwd_kernel(const T* __restrict__ logits, float* __restrict__ weights,
                                  int* __restrict__ experts, float* __restrict__ probs, int* __restrict__ counts,
                                  long long tokens, int E, int k, int renorm) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int per = (E + 31) / 32;
  for (long long t = warp; t < tokens; t += nwarps) {
    float v[ROUTER_MAX_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
      const int e = j * 32 + lane;
      v[j] = (j < per && e < E) ? Cvt<T>::to_f(logits[t * E + e]) : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) { v[j] = (v[j] == -INFINITY) ? 0.f : __expf(v[j] - mx); s += v[j]; }
    s = warp_sum(s);
    const float inv = 1.f / s;
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
      v[j] *= inv;
      const int e = j * 32 + lane;
      if (j < per && e < E) probs[t * E + e] = v[j];
    }
    // top-k by repeated warp arg-max (ties -> lowest expert id)
    float wsum = 0.f;
    float myw = 0.f;
    int mye = 0;
    for (int r = 0; r < k; ++r) {
      float best = -1.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
        const int e = j * 32 + lane;
        if (j < per && e < E && v[j] > best) { best = v[j]; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if ((bi & 31) == lane) {                     // remove from further rounds
#pragma unroll
        for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) if (j == (bi >> 5)) v[j] = -2.f;
      }
      wsum += best;
      if (lane == r) { myw = best; mye = bi; }
    }
    if (lane < k) {
      weights[t * k + lane] = renorm ? myw / (wsum + 1e-20f) : myw;
      experts[t * k + lane] = mye;
      atomicAdd(counts + mye, 1);
    }
  }
}

// dlogits = p * (tot - sum(p * tot)), tot = dprobs + scatter(dw_raw)
template <typename TO>
__global__ void router_bwd_kernel(const float* __restrict__ dweights, const float* __restrict__ dprobs,
                                  const float* __restrict__ probs, const int* __restrict__ experts,
                                  const float* __restrict__ weights, TO* __restrict__ dlogits, long long tokens,
                                  int E, int k, int renorm) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int per = (E + 31) / 32;
  for (long long t = warp; t < tokens; t += nwarps) {
    float p[ROUTER_MAX_PER_LANE], tot[ROUTER_MAX_PER_LANE];
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
      const int e = j * 32 + lane;
      const bool ok = j < per && e < E;
      p[j] = ok ? probs[t * E + e] : 0.f;
      tot[j] = (ok && dprobs != nullptr) ? dprobs[t * E + e] : 0.f;
    }
    if (dweights != nullptr) {
      // slot `lane` of this token
      float dw = lane < k ? dweights[t * k + lane] : 0.f;
      const float w = lane < k ? weights[t * k + lane] : 0.f;
      const int ex = lane < k ? experts[t * k + lane] : -1;
      if (renorm) {
        const float raw = (ex >= 0) ? probs[t * E + ex] : 0.f;
        const float rs = warp_sum(raw) + 1e-20f;
        const float dot = warp_sum(dw * w);
        dw = (dw - dot) / rs;
      }
      for (int r = 0; r < k; ++r) {
        const float d = __shfl_sync(0xffffffffu, dw, r);
        const int e = __shfl_sync(0xffffffffu, ex, r);
        if ((e & 31) == lane) {
#pragma unroll
          for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) if (j == (e >> 5)) tot[j] += d;
        }
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) dot += p[j] * tot[j];
    dot = warp_sum(dot);
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
      const int e = j * 32 + lane;
      if (j < per && e < E) dlogits[t * E + e] = Cvt<TO>::from_f(p[j] * (tot[j] - dot));
    }
  }
}

// offsets[e] = sum of counts[<e] rounded up to `align` per expert; cursor[e] = 0. One block.
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ offsets,
                                   int* __restrict__ cursor, int E, int align) {
  __shared__ int sh[1024];
  const int e = threadIdx.x;
  int c = (e < E) ? (counts[e] + align - 1) / align * align : 0;
  sh[e] = c;
  __syncthreads();
  for (int o = 1; o < blockDim.x; o <<= 1) {
    const int v = (e >= o) ? sh[e - o] : 0;
    __syncthreads();
    sh[e] += v;
    __syncthreads();
  }
  if (e < E) { offsets[e + 1] = sh[e]; cursor[e] = 0; }
  if (e == 0) offsets[0] = 0;
}

// pos[pair] = offsets[expert] + running index within the expert; row_token[pos] = pair / k
__global__ void moe_scatter_kernel(const int* __restrict__ experts, const int* __restrict__ offsets,
                                   int* __restrict__ cursor, int* __restrict__ pos, int* __restrict__ row_token,
                                   long long pairs, int k) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += stride) {
    const int e = experts[i];
    const int slot = offsets[e] + atomicAdd(cursor + e, 1);
    pos[i] = slot;
    row_token[slot] = (int)(i / k);
  }
}

// out[t, :] = sum_j w[t, j] * y[pos[t, j], :]
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const float* __restrict__ w, const int* __restrict__ pos,
                                   T* __restrict__ out, long long tokens, int k, int cols) {
  constexpr int V = Vec16<T>::N;
  const int vpr = cols / V;
  const long long total = tokens * vpr;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long t = i / vpr;
    const int c = (int)(i % vpr);
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    for (int s = 0; s < k; ++s) {
      const float ws = w[t * k + s];
      const Vec16<T> a = ld16(y + (long long)pos[t * k + s] * cols + c * V);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += ws * Cvt<T>::to_f(a.v[j]);
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(acc[j]);
    st16(out + t * cols + c * V, o);
  }
}

// backward of combine: dy[pos[t,j], :] = w[t,j] * g[t, :];  dw[t,j] = <g[t,:], y[pos[t,j],:]>
template <typename T>
__global__ void moe_combine_bwd_kernel(const T* __restrict__ g, const T* __restrict__ y, const float* __restrict__ w,
                                       const int* __restrict__ pos, T* __restrict__ dy, float* __restrict__ dw,
                                       long long tokens, int k, int cols) {
  // one warp per (token, slot)
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long pr = warp; pr < tokens * k; pr += nwarps) {
    const long long t = pr / k;
    const long long row = pos[pr];
    const float ws = w[pr];
    float dot = 0.f;
    for (int c = lane; c < cols; c += 32) {
      const float gg = Cvt<T>::to_f(g[t * cols + c]);
      dot += gg * Cvt<T>::to_f(y[row * cols + c]);
      dy[row * cols + c] = Cvt<T>::from_f(ws * gg);
    }
    dot = warp_sum(dot);
    if (lane == 0) dw[pr] = dot;
  }
}

}  // namespace gb

using namespace gb;

extern "C" int gb_router_fwd(const void* logits, float* weights, int* experts, float* probs, int* counts,
                             long long tokens, int E, int k, int renorm, int dt, cudaStream_t st) {
  if (tokens == 0) return 0;
  if (E > 32 * ROUTER_MAX_PER_LANE || k > 32) return -2;
  cudaMemsetAsync(counts, 0, sizeof(int) * E, st);
  const int grid = gb_grid(tokens * 32, 256);
  GB_DISPATCH_FLOAT(dt, T, router_fwd_kernel<T><<<grid, 256, 0, st>>>((const T*)logits, weights, experts, probs, counts, tokens, E, k, renorm));
  return (int)cudaGetLastError();
}

extern "C" int gb_router_bwd(const float* dweights, const float* dprobs, const float* probs, const int* experts,
                             const float* weights, void* dlogits, long long tokens, int E, int k, int renorm,
                             int out_dt, cudaStream_t st) {
  if (tokens == 0) return 0;
  if (E > 32 * ROUTER_MAX_PER_LANE || k > 32) return -2;
  const int grid = gb_grid(tokens * 32, 256);
  GB_DISPATCH_FLOAT(out_dt, T, router_bwd_kernel<T><<<grid, 256, 0, st>>>(dweights, dprobs, probs, experts, weights, (T*)dlogits, tokens, E, k, renorm));
  return (int)cudaGetLastError();
}

// experts [pairs] int32, counts [E]; outputs offsets [E+1], pos [pairs], row_token [max_rows] (pre-filled with -1
// here), cursor [E] scratch.
extern "C" int gb_moe_sort(const int* experts, const int* counts, int* offsets, int* cursor, int* pos,
                           int* row_token, long long pairs, int k, int E, int align, long long max_rows,
                           cudaStream_t st) {
  if (E > 1024) return -2;
  cudaMemsetAsync(row_token, 0xff, sizeof(int) * max_rows, st);
  int threads = 32;
  while (threads < E) threads <<= 1;
  moe_offsets_kernel<<<1, threads, 0, st>>>(counts, offsets, cursor, E, align);
  if (pairs > 0) moe_scatter_kernel<<<gb_grid(pairs, 256), 256, 0, st>>>(experts, offsets, cursor, pos, row_token, pairs, k);
  return (int)cudaGetLastError();
}

extern "C" int gb_moe_combine(const void* y, const float* w, const int* pos, void* out, long long tokens, int k,
                              int cols, int dt, cudaStream_t st) {
  if (tokens == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, {
    if (cols % Vec16<T>::N != 0) return -2;
    moe_combine_kernel<T><<<gb_grid(tokens * (cols / Vec16<T>::N), 256), 256, 0, st>>>((const T*)y, w, pos, (T*)out, tokens, k, cols);
  });
  return (int)cudaGetLastError();
}

extern "C" int gb_moe_combine_bwd(const void* g, const void* y, const float* w, const int* pos, void* dy, float* dw,
                                  long long tokens, int k, int cols, int dt, cudaStream_t st) {
  if (tokens == 0) return 0;
  GB_DISPATCH_FLOAT(dt, T, moe_combine_bwd_kernel<T><<<gb_grid(tokens * k * 32, 256), 256, 0, st>>>(
      (const T*)g, (const T*)y, w, pos, (T*)dy, dw, tokens, k, cols));
  return (int)cudaGetLastError();
}
