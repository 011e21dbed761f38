// Sorting, selection and index-producing kernels: row sort / argsort / top-k, arg-max, bincount, nonzero,
// triu / tril, one-hot, arange, repeat_interleave.
//
// Sort family: every row becomes 64-bit composites (order-preserving 32-bit key << 32 | column), so a plain
// ascending sort of the composites is a STABLE sort of the row (ties keep column order) in either direction.
// Rows of up to 8192 columns are sorted by one CTA in shared memory (bitonic network); longer rows run the same
// network over a caller-provided workspace, one launch per compare-exchange distance.
//
// Reference counterparts: genesis/ops/cuda/tensor_ops.py:16-623 (triu/tril 32x32 tiles; top-k as k sequential
// arg-max launches with a mask buffer; argsort as N sequential launches; bincount with one program per
// element), genesis/ops/cuda/basic_ops.py (arange, one_hot, nonzero with a host count read-back),
// genesis/ops/cuda/shape_ops.py:62-182 (repeat_interleave launched from a Python double loop).
#include "common.cuh"

namespace gb {

constexpr int SORT_SMEM_MAX = 8192;     // composites a CTA sorts in shared memory (64 KB)

__device__ __forceinline__ uint32_t order_key(float v) {
  uint32_t u = __float_as_uint(v);
  if (v != v) u = 0x7fc00000u;                          // every NaN sorts as the largest value
  if (v == 0.f) u = 0u;                                 // -0 and +0 compare equal
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ uint32_t order_key_i32(int v) { return (uint32_t)v ^ 0x80000000u; }

__device__ __forceinline__ uint32_t load_key(const void* p, int dt, size_t i) {
  if (dt == DT_I32) return order_key_i32(reinterpret_cast<const int*>(p)[i]);
  return order_key(load_as_float(p, dt, i));
}

__device__ __forceinline__ void copy_elem(void* dst, size_t di, const void* src, size_t si, int dt) {
  if (dt == DT_F32 || dt == DT_I32) reinterpret_cast<uint32_t*>(dst)[di] = reinterpret_cast<const uint32_t*>(src)[si];
  else reinterpret_cast<uint16_t*>(dst)[di] = reinterpret_cast<const uint16_t*>(src)[si];
}

// One CTA sorts one row in shared memory and writes the first `k` results.
__global__ void sort_rows_smem_kernel(const void* __restrict__ in, void* __restrict__ vals,
                                      long long* __restrict__ idx, int cols, int npow2, int k, int descending,
                                      int dt) {
  extern __shared__ unsigned long long comp[];
  const size_t row = blockIdx.x;
  for (int i = threadIdx.x; i < npow2; i += blockDim.x) {
    unsigned long long c = ~0ull;                       // padding sorts last
    if (i < cols) {
      uint32_t key = load_key(in, dt, row * cols + i);
      if (descending) key = ~key;
      c = ((unsigned long long)key << 32) | (uint32_t)i;
    }
    comp[i] = c;
  }
  __syncthreads();
  for (int size = 2; size <= npow2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < (npow2 >> 1); t += blockDim.x) {
        const int lo = 2 * t - (t & (stride - 1));      // index whose bit `stride` is clear
        const int hi = lo + stride;
        const bool up = (lo & size) == 0;
        const unsigned long long a = comp[lo], b = comp[hi];
        if ((a > b) == up) { comp[lo] = b; comp[hi] = a; }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    const int col = (int)(comp[i] & 0xffffffffu);
    if (idx != nullptr) idx[row * k + i] = col;
    if (vals != nullptr) copy_elem(vals, row * k + i, in, row * cols + col, dt);
  }
}

// Small k: the row goes to shared memory once, then k rounds of "find the smallest composite, emit it, retire it".
// 8 rounds over 4096 values cost a twentieth of the compare-exchanges of the full sorting network.
__global__ void __launch_bounds__(256)
topk_select_kernel(const void* __restrict__ in, void* __restrict__ vals, long long* __restrict__ idx, int cols, int k,
                   int descending, int dt) {
  extern __shared__ unsigned long long comp[];
  __shared__ unsigned long long wbest[8];
  const size_t row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < cols; i += 256) {
    uint32_t key = load_key(in, dt, row * cols + i);
    if (descending) key = ~key;
    comp[i] = ((unsigned long long)key << 32) | (uint32_t)i;
  }
  __syncthreads();
  for (int round = 0; round < k; ++round) {
    unsigned long long best = ~0ull;
    for (int i = threadIdx.x; i < cols; i += 256) { const unsigned long long c = comp[i]; best = c < best ? c : best; }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
      const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, m);
      best = o < best ? o : best;
    }
    if (lane == 0) wbest[warp] = best;
    __syncthreads();
    best = wbest[0];
#pragma unroll
    for (int q = 1; q < 8; ++q) best = wbest[q] < best ? wbest[q] : best;
    const int col = (int)(best & 0xffffffffu);
    if (threadIdx.x == 0) {
      if (idx != nullptr) idx[row * k + round] = col;
      if (vals != nullptr) copy_elem(vals, row * k + round, in, row * cols + col, dt);
      comp[col] = ~0ull;                                  // retired
    }
    __syncthreads();
  }
}

// Long rows: composites in global memory, one launch per compare-exchange distance.
__global__ void sort_fill_kernel(const void* __restrict__ in, unsigned long long* __restrict__ comp, long long rows,
                                 int cols, int npow2, int descending, int dt) {
  const long long n = rows * npow2;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n; g += (long long)gridDim.x * blockDim.x) {
    const long long row = g / npow2;
    const int i = (int)(g % npow2);
    unsigned long long c = ~0ull;
    if (i < cols) {
      uint32_t key = load_key(in, dt, row * cols + i);
      if (descending) key = ~key;
      c = ((unsigned long long)key << 32) | (uint32_t)i;
    }
    comp[g] = c;
  }
}
__global__ void sort_step_kernel(unsigned long long* __restrict__ comp, long long rows, int npow2, int size,
                                 int stride) {
  const long long half = npow2 >> 1;
  const long long n = rows * half;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n; g += (long long)gridDim.x * blockDim.x) {
    const long long row = g / half;
    const int t = (int)(g % half);
    const int lo = 2 * t - (t & (stride - 1));
    const int hi = lo + stride;
    const bool up = (lo & size) == 0;
    unsigned long long* base = comp + row * npow2;
    const unsigned long long a = base[lo], b = base[hi];
    if ((a > b) == up) { base[lo] = b; base[hi] = a; }
  }
}
__global__ void sort_emit_kernel(const void* __restrict__ in, const unsigned long long* __restrict__ comp,
                                 void* __restrict__ vals, long long* __restrict__ idx, long long rows, int cols,
                                 int npow2, int k, int dt) {
  const long long n = rows * k;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n; g += (long long)gridDim.x * blockDim.x) {
    const long long row = g / k;
    const int i = (int)(g % k);
    const int col = (int)(comp[row * npow2 + i] & 0xffffffffu);
    if (idx != nullptr) idx[g] = col;
    if (vals != nullptr) copy_elem(vals, g, in, row * cols + col, dt);
  }
}

// arg-max / arg-min over the last dimension, one warp per row, first occurrence wins
__global__ void argmax_rows_kernel(const void* __restrict__ in, long long* __restrict__ out, long long rows, int cols,
                                   int is_min, int dt) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += nwarps) {
    unsigned long long best = ~0ull;
    int c_done = 0;
    if (dt != DT_I32) {
      // 16-byte loads where the row allows it
      const int es = dt == DT_F32 ? 4 : 2, V = 16 / es;
      const char* rowp = reinterpret_cast<const char*>(in) + (size_t)r * cols * es;
      if ((reinterpret_cast<uintptr_t>(rowp) & 15) == 0) {
        const int nv = cols / V;
        for (int i = lane; i < nv; i += 32) {
          const uint4 raw = *reinterpret_cast<const uint4*>(rowp + (size_t)i * 16);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (j >= V) break;
            float v;
            if (dt == DT_F32) v = __uint_as_float(reinterpret_cast<const uint32_t*>(&raw)[j]);
            else v = half_bits_to_float(reinterpret_cast<const uint16_t*>(&raw)[j], dt);
            uint32_t key = order_key(v);
            if (!is_min) key = ~key;
            const unsigned long long comp = ((unsigned long long)key << 32) | (uint32_t)(i * V + j);
            best = comp < best ? comp : best;
          }
        }
        c_done = nv * V;
      }
    }
    for (int c = c_done + lane; c < cols; c += 32) {
      uint32_t key = load_key(in, dt, r * cols + c);
      if (!is_min) key = ~key;
      const unsigned long long comp = ((unsigned long long)key << 32) | (uint32_t)c;
      best = comp < best ? comp : best;
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
      const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, m);
      best = o < best ? o : best;
    }
    if (lane == 0) out[r] = (long long)(best & 0xffffffffu);
  }
}

// ------------------------------------------------------------------------------------------------
// bincount: per-CTA shared histogram when the bins fit, global atomics otherwise
// ------------------------------------------------------------------------------------------------
template <typename I>
__global__ void bincount_kernel(const I* __restrict__ idx, const float* __restrict__ weights, float* __restrict__ outw,
                                long long* __restrict__ outc, long long n, int nbins, int use_smem) {
  extern __shared__ float hist[];
  if (use_smem) {
    for (int i = threadIdx.x; i < nbins; i += blockDim.x) hist[i] = 0.f;
    __syncthreads();
  }
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n; g += (long long)gridDim.x * blockDim.x) {
    const long long b = (long long)idx[g];
    if (b < 0 || b >= nbins) continue;
    const float w = weights != nullptr ? weights[g] : 1.f;
    if (use_smem) atomicAdd(&hist[b], w);
    else if (outw != nullptr) atomicAdd(&outw[b], w);
    else atomicAdd(reinterpret_cast<unsigned long long*>(&outc[b]), 1ull);
  }
  if (use_smem) {
    __syncthreads();
    for (int i = threadIdx.x; i < nbins; i += blockDim.x) {
      const float h = hist[i];
      if (h == 0.f) continue;
      if (outw != nullptr) atomicAdd(&outw[i], h);
      else atomicAdd(reinterpret_cast<unsigned long long*>(&outc[i]), (unsigned long long)(h + 0.5f));
    }
  }
}

// ------------------------------------------------------------------------------------------------
// nonzero: per-block counts -> exclusive scan (one CTA) -> ordered write of flat indices
// ------------------------------------------------------------------------------------------------
constexpr int NZ_BLOCK = 1024;       // elements per block of the count / write passes (4 per thread)

__device__ __forceinline__ bool is_nonzero(const void* p, int dt, size_t i) {
  if (dt == DT_I32) return reinterpret_cast<const int*>(p)[i] != 0;
  if (dt == DT_I64) return reinterpret_cast<const long long*>(p)[i] != 0;
  if (dt == DT_U8 || dt == DT_BOOL) return reinterpret_cast<const uint8_t*>(p)[i] != 0;
  return load_as_float(p, dt, i) != 0.f;
}

__global__ void nonzero_count_kernel(const void* __restrict__ in, int* __restrict__ counts, long long n, int dt) {
  __shared__ int warp_sums[8];
  const long long base = (long long)blockIdx.x * NZ_BLOCK;
  int c = 0;
  for (int j = 0; j < 4; ++j) {
    const long long i = base + threadIdx.x * 4 + j;
    if (i < n && is_nonzero(in, dt, i)) ++c;
  }
  c = (int)warp_sum((float)c);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < 8; ++w) s += warp_sums[w];
    counts[blockIdx.x] = s;
  }
}
// in place: counts[i] <- sum of counts[0..i), counts[nblocks] <- total
__global__ void nonzero_scan_kernel(int* __restrict__ counts, int nblocks) {
  __shared__ int carry;
  __shared__ int tmp[1024];
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < nblocks; base += 1024) {
    const int i = base + threadIdx.x;
    const int v = i < nblocks ? counts[i] : 0;
    tmp[threadIdx.x] = v;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const int add = threadIdx.x >= off ? tmp[threadIdx.x - off] : 0;
      __syncthreads();
      tmp[threadIdx.x] += add;
      __syncthreads();
    }
    if (i < nblocks) counts[i] = carry + tmp[threadIdx.x] - v;
    __syncthreads();
    if (threadIdx.x == 0) carry += tmp[1023];
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[nblocks] = carry;
}
__global__ void nonzero_write_kernel(const void* __restrict__ in, const int* __restrict__ offsets,
                                     long long* __restrict__ out, long long n, int dt) {
  __shared__ int warp_offs[9];
  const long long base = (long long)blockIdx.x * NZ_BLOCK;
  bool nz[4];
  int c = 0;
  for (int j = 0; j < 4; ++j) {
    const long long i = base + threadIdx.x * 4 + j;
    nz[j] = i < n && is_nonzero(in, dt, i);
    c += nz[j] ? 1 : 0;
  }
  // exclusive scan of c over the 256 threads
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = c;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += o;
  }
  if (lane == 31) warp_offs[warp + 1] = incl;
  if (threadIdx.x == 0) warp_offs[0] = 0;
  __syncthreads();
  if (threadIdx.x == 0)
    for (int w = 1; w <= 8; ++w) warp_offs[w] += warp_offs[w - 1];
  __syncthreads();
  long long pos = (long long)offsets[blockIdx.x] + warp_offs[warp] + incl - c;
  for (int j = 0; j < 4; ++j)
    if (nz[j]) out[pos++] = base + threadIdx.x * 4 + j;
}

// ------------------------------------------------------------------------------------------------
// triu / tril over the last two dimensions; one_hot; arange; repeat_interleave
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void triu_tril_kernel(const T* __restrict__ in, T* __restrict__ out, long long n, int rows, int cols,
                                 int diag, int upper) {
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n; g += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(g % cols);
    const int r = (int)((g / cols) % rows);
    const bool keep = upper ? (c - r >= diag) : (c - r <= diag);
    out[g] = keep ? in[g] : T(0);
  }
}

template <typename I>
__global__ void one_hot_kernel(const I* __restrict__ idx, void* __restrict__ out, long long n, int classes, int dt) {
  const long long total = n * classes;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (long long)gridDim.x * blockDim.x) {
    const float v = ((long long)idx[g / classes] == g % classes) ? 1.f : 0.f;
    if (dt == DT_I64) reinterpret_cast<long long*>(out)[g] = (long long)v;
    else if (dt == DT_I32) reinterpret_cast<int*>(out)[g] = (int)v;
    else store_from_float(out, dt, g, v);
  }
}

__global__ void arange_kernel(void* __restrict__ out, long long n, double start, double step, int dt) {
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n; g += (long long)gridDim.x * blockDim.x) {
    const double v = start + step * (double)g;
    if (dt == DT_I64) reinterpret_cast<long long*>(out)[g] = (long long)v;
    else if (dt == DT_I32) reinterpret_cast<int*>(out)[g] = (int)v;
    else store_from_float(out, dt, g, (float)v);
  }
}

// out[o, i * rep + r, s] = in[o, i, s] for a tensor viewed as [outer, dim, inner]; esize-byte elements
__global__ void repeat_interleave_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, long long outer,
                                         long long dim, long long inner, int rep, int esize) {
  const long long total = outer * dim * rep * inner;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (long long)gridDim.x * blockDim.x) {
    const long long s = g % inner;
    const long long j = (g / inner) % (dim * rep);
    const long long o = g / (inner * dim * rep);
    const long long src = (o * dim + j / rep) * inner + s;
    if (esize == 2) reinterpret_cast<uint16_t*>(out)[g] = reinterpret_cast<const uint16_t*>(in)[src];
    else if (esize == 4) reinterpret_cast<uint32_t*>(out)[g] = reinterpret_cast<const uint32_t*>(in)[src];
    else if (esize == 8) reinterpret_cast<unsigned long long*>(out)[g] = reinterpret_cast<const unsigned long long*>(in)[src];
    else out[g] = in[src];
  }
}

static int next_pow2(int v) { int p = 1; while (p < v) p <<= 1; return p; }

}  // namespace gb

using namespace gb;

// Bytes of workspace gb_sort_rows needs (0 when the rows are sorted in shared memory).
extern "C" long long gb_sort_workspace(long long rows, int cols) {
  if (cols <= SORT_SMEM_MAX) return 0;
  return rows * (long long)next_pow2(cols) * 8;
}

// Stable sort of every row of in[rows, cols] (fp32 / fp16 / bf16 / int32); writes the first k sorted values
// (may be null) and their column indices (int64, may be null).  k == cols gives sort / argsort, k < cols top-k.
extern "C" int gb_sort_rows(const void* in, void* vals, long long* idx, long long rows, int cols, int k,
                            int descending, int dt, void* workspace, cudaStream_t st) {
  if (rows <= 0 || cols <= 0 || k <= 0) return 0;
  if (k > cols) return -3;
  if (dt != DT_F32 && dt != DT_F16 && dt != DT_BF16 && dt != DT_I32) return -2;
  const int np2 = next_pow2(cols);
  if (cols <= SORT_SMEM_MAX && k <= 16 && k < cols) {
    static unsigned long long cfgk = 0;
    if (int e = smem_opt_in(topk_select_kernel, SORT_SMEM_MAX * 8, cfgk)) return e;
    topk_select_kernel<<<(unsigned)rows, 256, (size_t)cols * 8, st>>>(in, vals, idx, cols, k, descending, dt);
    return (int)cudaGetLastError();
  }
  if (cols <= SORT_SMEM_MAX) {
    static unsigned long long cfg = 0;
    if (int e = smem_opt_in(sort_rows_smem_kernel, SORT_SMEM_MAX * 8, cfg)) return e;
    int threads = np2 / 2 < 32 ? 32 : (np2 / 2 > 1024 ? 1024 : np2 / 2);
    sort_rows_smem_kernel<<<(unsigned)rows, threads, np2 * 8, st>>>(in, vals, idx, cols, np2, k, descending, dt);
    return (int)cudaGetLastError();
  }
  if (workspace == nullptr) return -4;
  unsigned long long* comp = reinterpret_cast<unsigned long long*>(workspace);
  sort_fill_kernel<<<gb_grid(rows * np2, 256), 256, 0, st>>>(in, comp, rows, cols, np2, descending, dt);
  for (int size = 2; size <= np2; size <<= 1)
    for (int stride = size >> 1; stride > 0; stride >>= 1)
      sort_step_kernel<<<gb_grid(rows * (np2 / 2), 256), 256, 0, st>>>(comp, rows, np2, size, stride);
  sort_emit_kernel<<<gb_grid(rows * k, 256), 256, 0, st>>>(in, comp, vals, idx, rows, cols, np2, k, dt);
  return (int)cudaGetLastError();
}

extern "C" int gb_argmax_rows(const void* in, long long* out, long long rows, int cols, int is_min, int dt,
                              cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  if (dt != DT_F32 && dt != DT_F16 && dt != DT_BF16 && dt != DT_I32) return -2;
  argmax_rows_kernel<<<gb_grid(rows * 32, 256), 256, 0, st>>>(in, out, rows, cols, is_min, dt);
  return (int)cudaGetLastError();
}

// out must be zero-filled: float [nbins] when weights are given (out_is_float), int64 [nbins] otherwise.
extern "C" int gb_bincount(const void* idx, int idx_is_i64, const float* weights, void* out, long long n, int nbins,
                           cudaStream_t st) {
  if (n <= 0 || nbins <= 0) return 0;
  const int use_smem = nbins <= 8192 && (weights != nullptr || n < (1ll << 24)) ? 1 : 0;
  float* outw = weights != nullptr ? reinterpret_cast<float*>(out) : nullptr;
  long long* outc = weights != nullptr ? nullptr : reinterpret_cast<long long*>(out);
  const int grid = gb_grid(n, 256, 148 * 4);
  const size_t smem = use_smem ? (size_t)nbins * 4 : 0;
  if (idx_is_i64) bincount_kernel<long long><<<grid, 256, smem, st>>>((const long long*)idx, weights, outw, outc, n, nbins, use_smem);
  else bincount_kernel<int><<<grid, 256, smem, st>>>((const int*)idx, weights, outw, outc, n, nbins, use_smem);
  return (int)cudaGetLastError();
}

// Pass 1 + scan: counts must hold ceil(n / 1024) + 1 ints; counts[last] receives the number of nonzeros.
extern "C" int gb_nonzero_count(const void* in, int* counts, long long n, int dt, cudaStream_t st) {
  const long long nb = (n + NZ_BLOCK - 1) / NZ_BLOCK;
  if (nb > 0x7fffffffll) return -3;
  if (nb > 0) nonzero_count_kernel<<<(unsigned)nb, 256, 0, st>>>(in, counts, n, dt);
  nonzero_scan_kernel<<<1, 1024, 0, st>>>(counts, (int)nb);
  return (int)cudaGetLastError();
}
// Pass 2: flat int64 indices of the nonzero elements, ascending.
extern "C" int gb_nonzero_write(const void* in, const int* counts, long long* out, long long n, int dt,
                                cudaStream_t st) {
  const long long nb = (n + NZ_BLOCK - 1) / NZ_BLOCK;
  if (nb > 0) nonzero_write_kernel<<<(unsigned)nb, 256, 0, st>>>(in, counts, out, n, dt);
  return (int)cudaGetLastError();
}

extern "C" int gb_triu_tril(const void* in, void* out, long long n, int rows, int cols, int diag, int upper,
                            int esize, cudaStream_t st) {
  if (n <= 0) return 0;
  const int grid = gb_grid(n, 256);
  // zero of every supported type is all-zero bits: dispatch on the element size only
  if (esize == 2) triu_tril_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t*)in, (uint16_t*)out, n, rows, cols, diag, upper);
  else if (esize == 4) triu_tril_kernel<uint32_t><<<grid, 256, 0, st>>>((const uint32_t*)in, (uint32_t*)out, n, rows, cols, diag, upper);
  else if (esize == 8) triu_tril_kernel<unsigned long long><<<grid, 256, 0, st>>>((const unsigned long long*)in, (unsigned long long*)out, n, rows, cols, diag, upper);
  else if (esize == 1) triu_tril_kernel<uint8_t><<<grid, 256, 0, st>>>((const uint8_t*)in, (uint8_t*)out, n, rows, cols, diag, upper);
  else return -2;
  return (int)cudaGetLastError();
}

extern "C" int gb_one_hot(const void* idx, int idx_is_i64, void* out, long long n, int classes, int dt,
                          cudaStream_t st) {
  if (n <= 0 || classes <= 0) return 0;
  const int grid = gb_grid(n * classes, 256);
  if (idx_is_i64) one_hot_kernel<long long><<<grid, 256, 0, st>>>((const long long*)idx, out, n, classes, dt);
  else one_hot_kernel<int><<<grid, 256, 0, st>>>((const int*)idx, out, n, classes, dt);
  return (int)cudaGetLastError();
}

extern "C" int gb_arange(void* out, long long n, double start, double step, int dt, cudaStream_t st) {
  if (n <= 0) return 0;
  arange_kernel<<<gb_grid(n, 256), 256, 0, st>>>(out, n, start, step, dt);
  return (int)cudaGetLastError();
}

extern "C" int gb_repeat_interleave(const void* in, void* out, long long outer, long long dim, long long inner,
                                    int rep, int esize, cudaStream_t st) {
  const long long total = outer * dim * rep * inner;
  if (total <= 0) return 0;
  repeat_interleave_kernel<<<gb_grid(total, 256), 256, 0, st>>>((const uint8_t*)in, (uint8_t*)out, outer, dim, inner,
                                                               rep, esize);
  return (int)cudaGetLastError();
}
