// Indexing engine: concatenation, gather / scatter along a dimension, general advanced indexing (read, write,
// accumulate) and masked fill.
//
//   cat           out[outer, sum(inner_i)] <- inputs [outer, inner_i]            (stack = cat of [outer, 1 * inner])
//   gather_dim    out[c] = src[c with c[dim] := index[c]]                         (torch.gather semantics)
//   scatter_dim   dst[c with c[dim] := index[c]] (=|+=) src[c] | scalar          (scatter / scatter_add)
//   index_get     out[pre, b, post] = src[pre + sum_k idx_k[b] * stride_k + post]   (a[i0, i1, ...] with tensor indices)
//   index_put     dst[pre + sum_k idx_k[b] * stride_k + post] (=|+=) val[pre, b, post] | scalar
//   masked_fill   a[m, :] = scalar where mask[m]
//
// Index tensors may be int32 or int64, are broadcast through their strides (no expanded copy), may be negative
// (wrapped once) and are bounds-checked always: an out-of-range index is skipped and recorded in the status word
// (GB_ERR_BAD_INDEX, site 3 gather / 4 scatter / 5 indexed read / 6 indexed write), never dereferenced.
// Plain copies move opaque elements of 1 / 2 / 4 / 8 / 16 bytes; accumulation is typed (atomic adds).
// Reference counterparts: genesis/backends/cuda_kernels.py:324-1206 (gather / scatter / mask / cat kernels),
// genesis/ops/cuda/indexing_ops.py:14-625, genesis/backends/cuda.py:1617-1643 (IndexPlan execution).
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace gb {

constexpr int IDX_MAX = 4;      // index tensors per operation
constexpr int IDX_BDIMS = 4;    // dims of the broadcast index shape
constexpr int IDX_SIDE = 3;     // dims before / after the indexed block
constexpr int DIM_MAX = 6;      // dims of gather / scatter along a dimension
constexpr int CAT_MAX = 8;      // inputs per cat launch

template <int B> struct Bytes;
template <> struct Bytes<1> { using T = uint8_t; };
template <> struct Bytes<2> { using T = uint16_t; };
template <> struct Bytes<4> { using T = uint32_t; };
template <> struct Bytes<8> { using T = uint2; };
template <> struct Bytes<16> { using T = uint4; };

// ------------------------------------------------------------------------------------------------
// cat
// ------------------------------------------------------------------------------------------------
struct CatArgs {
  const void* src[CAT_MAX];
  long long inner[CAT_MAX];     // elements per outer row of input i
  long long offset[CAT_MAX];    // element offset of input i inside an output row
  long long out_inner;
  long long outer;
  int n;
};

template <typename U>
__global__ void __launch_bounds__(256) cat_kernel(CatArgs a, U* __restrict__ out) {
  const int i = blockIdx.y;
  if (i >= a.n) return;
  const U* __restrict__ src = reinterpret_cast<const U*>(a.src[i]);
  const long long inner = a.inner[i], total = inner * a.outer;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const long long o = e / inner, c = e - o * inner;
    out[o * a.out_inner + a.offset[i] + c] = src[e];
  }
}

// ------------------------------------------------------------------------------------------------
// gather / scatter along one dimension
// ------------------------------------------------------------------------------------------------
struct DimArgs {
  long long shape[DIM_MAX];        // index shape (= out shape for gather, = iteration space for scatter)
  long long data_stride[DIM_MAX];  // strides of the gathered-from / scattered-into tensor
  long long other_stride[DIM_MAX]; // strides of src (scatter); unused for gather (out is contiguous)
  long long idx_stride[DIM_MAX];
  long long dim_size;
  long long n;
  int nd, dim, idx_i64;
};

__device__ __forceinline__ long long load_index(const void* p, int is_i64, long long off) {
  return is_i64 ? reinterpret_cast<const long long*>(p)[off] : (long long)reinterpret_cast<const int*>(p)[off];
}

template <typename U>
__global__ void __launch_bounds__(256)
gather_dim_kernel(DimArgs a, const U* __restrict__ src, const void* __restrict__ idx, U* __restrict__ out,
                  int* __restrict__ status) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < a.n; e += stride) {
    long long r = e, so = 0, io = 0;
#pragma unroll
    for (int d = DIM_MAX - 1; d >= 0; --d) {
      if (d < a.nd) {
        const long long c = r % a.shape[d];
        r /= a.shape[d];
        io += c * a.idx_stride[d];
        if (d != a.dim) so += c * a.data_stride[d];
      }
    }
    long long j = load_index(idx, a.idx_i64, io);
    if (j < 0) j += a.dim_size;
    if (j < 0 || j >= a.dim_size) {
      report_error(status, GB_ERR_BAD_INDEX, 3, (int)j);
      out[e] = U{};
      continue;
    }
    out[e] = src[so + j * a.data_stride[a.dim]];
  }
}

template <typename T> __device__ __forceinline__ void atomic_add_t(T* p, T v) { atomicAdd(p, v); }
template <> __device__ __forceinline__ void atomic_add_t<long long>(long long* p, long long v) {
  atomicAdd(reinterpret_cast<unsigned long long*>(p), (unsigned long long)v);
}
template <> __device__ __forceinline__ void atomic_add_t<uint8_t>(uint8_t*, uint8_t) {}   // byte types only assign

// mode 0: assign, 1: add.  T is the real element type (needed for add); scalar_src: use `value` instead of src.
template <typename T>
__global__ void __launch_bounds__(256)
scatter_dim_kernel(DimArgs a, T* __restrict__ dst, const void* __restrict__ idx, const T* __restrict__ src, T value,
                   int scalar_src, int mode, int* __restrict__ status) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < a.n; e += stride) {
    long long r = e, d_o = 0, s_o = 0, io = 0;
#pragma unroll
    for (int d = DIM_MAX - 1; d >= 0; --d) {
      if (d < a.nd) {
        const long long c = r % a.shape[d];
        r /= a.shape[d];
        io += c * a.idx_stride[d];
        s_o += c * a.other_stride[d];
        if (d != a.dim) d_o += c * a.data_stride[d];
      }
    }
    long long j = load_index(idx, a.idx_i64, io);
    if (j < 0) j += a.dim_size;
    if (j < 0 || j >= a.dim_size) {
      report_error(status, GB_ERR_BAD_INDEX, 4, (int)j);
      continue;
    }
    const T v = scalar_src ? value : src[s_o];
    T* p = dst + d_o + j * a.data_stride[a.dim];
    if (mode) atomic_add_t<T>(p, v); else *p = v;
  }
}

// ------------------------------------------------------------------------------------------------
// general advanced indexing
// ------------------------------------------------------------------------------------------------
struct IndexArgs {
  const void* idx[IDX_MAX];
  long long idx_bstride[IDX_MAX][IDX_BDIMS];  // stride of index tensor k along broadcast dim b (0 = broadcast)
  long long dim_size[IDX_MAX];                // extent of the indexed dim (bounds, negative wrap)
  long long data_stride[IDX_MAX];             // stride of the indexed dim in the data tensor
  long long bshape[IDX_BDIMS];
  long long pre_shape[IDX_SIDE], pre_stride[IDX_SIDE];
  long long post_shape[IDX_SIDE], post_stride[IDX_SIDE];
  long long n_pre, n_b, n_post;
  int idx_i64[IDX_MAX];
  int nidx, nb, npre, npost;
};

// offset inside the data tensor of packed element e of [pre, b, post]; false: an index was out of range
__device__ __forceinline__ bool index_offset(const IndexArgs& a, long long e, long long& off, int* status, int site) {
  long long post = e % a.n_post;
  long long t = e / a.n_post;
  long long b = t % a.n_b;
  long long pre = t / a.n_b;
  off = 0;
#pragma unroll
  for (int d = IDX_SIDE - 1; d >= 0; --d) {
    if (d < a.npost) { off += (post % a.post_shape[d]) * a.post_stride[d]; post /= a.post_shape[d]; }
  }
#pragma unroll
  for (int d = IDX_SIDE - 1; d >= 0; --d) {
    if (d < a.npre) { off += (pre % a.pre_shape[d]) * a.pre_stride[d]; pre /= a.pre_shape[d]; }
  }
  long long bc[IDX_BDIMS];
#pragma unroll
  for (int d = IDX_BDIMS - 1; d >= 0; --d) {
    bc[d] = 0;
    if (d < a.nb) { bc[d] = b % a.bshape[d]; b /= a.bshape[d]; }
  }
#pragma unroll
  for (int k = 0; k < IDX_MAX; ++k) {
    if (k < a.nidx) {
      long long io = 0;
#pragma unroll
      for (int d = 0; d < IDX_BDIMS; ++d) io += bc[d] * a.idx_bstride[k][d];
      long long j = load_index(a.idx[k], a.idx_i64[k], io);
      if (j < 0) j += a.dim_size[k];
      if (j < 0 || j >= a.dim_size[k]) {
        report_error(status, GB_ERR_BAD_INDEX, site, (int)j);
        return false;
      }
      off += j * a.data_stride[k];
    }
  }
  return true;
}

template <typename U>
__global__ void __launch_bounds__(256)
index_get_kernel(IndexArgs a, const U* __restrict__ src, U* __restrict__ out, int* __restrict__ status) {
  const long long n = a.n_pre * a.n_b * a.n_post;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    long long off;
    if (index_offset(a, e, off, status, 5)) out[e] = src[off];
    else out[e] = U{};
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
index_put_kernel(IndexArgs a, T* __restrict__ dst, const T* __restrict__ val, T value, int scalar_src, int mode,
                 int* __restrict__ status) {
  const long long n = a.n_pre * a.n_b * a.n_post;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    long long off;
    if (!index_offset(a, e, off, status, 6)) continue;
    const T v = scalar_src ? value : val[e];
    if (mode) atomic_add_t<T>(dst + off, v); else dst[off] = v;
  }
}

// a[m, 0:inner] = value where mask[m] (mask: one byte per row, a contiguous)
template <typename U>
__global__ void __launch_bounds__(256)
masked_fill_kernel(U* __restrict__ a, const uint8_t* __restrict__ mask, U value, long long rows, long long inner) {
  const long long n = rows * inner;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    if (mask[e / inner]) a[e] = value;
  }
}

template <typename U>
__global__ void __launch_bounds__(256) fill_elems_kernel(U* __restrict__ a, U value, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) a[e] = value;
}

template <typename T> __host__ __device__ inline T scalar_from_double(double v) { return (T)v; }
template <> __host__ __device__ inline __half scalar_from_double<__half>(double v) { return __float2half_rn((float)v); }
template <> __host__ __device__ inline __nv_bfloat16 scalar_from_double<__nv_bfloat16>(double v) {
  return __float2bfloat16_rn((float)v);
}

}  // namespace gb

using namespace gb;

#define GB_DISPATCH_BYTES(es, U, ...)                               \
  do {                                                              \
    if ((es) == 1) { using U = Bytes<1>::T; __VA_ARGS__; }          \
    else if ((es) == 2) { using U = Bytes<2>::T; __VA_ARGS__; }     \
    else if ((es) == 4) { using U = Bytes<4>::T; __VA_ARGS__; }     \
    else if ((es) == 8) { using U = Bytes<8>::T; __VA_ARGS__; }     \
    else if ((es) == 16) { using U = Bytes<16>::T; __VA_ARGS__; }   \
    else return -2;                                                 \
  } while (0)

// every dtype the accumulate / typed-scalar paths cover
#define GB_DISPATCH_ELEM(dt, T, ...)                                         \
  do {                                                                       \
    if ((dt) == DT_F32) { using T = float; __VA_ARGS__; }                    \
    else if ((dt) == DT_F16) { using T = __half; __VA_ARGS__; }              \
    else if ((dt) == DT_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }      \
    else if ((dt) == DT_F64) { using T = double; __VA_ARGS__; }              \
    else if ((dt) == DT_I32) { using T = int; __VA_ARGS__; }                 \
    else if ((dt) == DT_I64) { using T = long long; __VA_ARGS__; }           \
    else return -2;                                                          \
  } while (0)

// srcs: n pointers (n <= 8); inner / offset in units of `es` bytes (the caller widens es when alignment allows).
extern "C" int gb_cat(const void* const* srcs, const long long* inner, const long long* offset, int n, void* out,
                      long long outer, long long out_inner, int es, cudaStream_t st) {
  if (n <= 0 || outer <= 0) return 0;
  if (n > CAT_MAX) return -3;
  CatArgs a;
  long long biggest = 0;
  for (int i = 0; i < n; ++i) {
    a.src[i] = srcs[i]; a.inner[i] = inner[i]; a.offset[i] = offset[i];
    if (inner[i] * outer > biggest) biggest = inner[i] * outer;
  }
  a.out_inner = out_inner; a.outer = outer; a.n = n;
  if (biggest == 0) return 0;
  dim3 grid(gb_grid(biggest, 256, 148 * 8), n);
  GB_DISPATCH_BYTES(es, U, cat_kernel<U><<<grid, 256, 0, st>>>(a, reinterpret_cast<U*>(out)));
  return (int)cudaGetLastError();
}

static int fill_dim_args(DimArgs& a, int nd, int dim, const long long* shape, const long long* data_stride,
                         const long long* other_stride, const long long* idx_stride, long long dim_size,
                         int idx_i64) {
  if (nd < 1 || nd > DIM_MAX || dim < 0 || dim >= nd) return -3;
  a.n = 1;
  for (int d = 0; d < DIM_MAX; ++d) {
    a.shape[d] = d < nd ? shape[d] : 1;
    a.data_stride[d] = d < nd ? data_stride[d] : 0;
    a.other_stride[d] = (d < nd && other_stride != nullptr) ? other_stride[d] : 0;
    a.idx_stride[d] = d < nd ? idx_stride[d] : 0;
    a.n *= a.shape[d];
  }
  a.nd = nd; a.dim = dim; a.dim_size = dim_size; a.idx_i64 = idx_i64;
  return 0;
}

// out (contiguous, index shape) <- src gathered along `dim`.
extern "C" int gb_gather_dim(const void* src, const void* idx, void* out, int nd, int dim, const long long* shape,
                             const long long* src_stride, const long long* idx_stride, long long dim_size,
                             int idx_i64, int es, int* status, cudaStream_t st) {
  DimArgs a;
  if (int r = fill_dim_args(a, nd, dim, shape, src_stride, nullptr, idx_stride, dim_size, idx_i64)) return r;
  if (a.n == 0) return 0;
  GB_DISPATCH_BYTES(es, U, gather_dim_kernel<U><<<gb_grid(a.n, 256), 256, 0, st>>>(
      a, reinterpret_cast<const U*>(src), idx, reinterpret_cast<U*>(out), status));
  return (int)cudaGetLastError();
}

// dst scattered along `dim` from src (strided) or the scalar `value`; mode 0 assign, 1 add.
extern "C" int gb_scatter_dim(void* dst, const void* idx, const void* src, double value, int scalar_src, int mode,
                              int nd, int dim, const long long* shape, const long long* dst_stride,
                              const long long* src_stride, const long long* idx_stride, long long dim_size,
                              int idx_i64, int dt, int* status, cudaStream_t st) {
  DimArgs a;
  if (int r = fill_dim_args(a, nd, dim, shape, dst_stride, src_stride, idx_stride, dim_size, idx_i64)) return r;
  if (a.n == 0) return 0;
  GB_DISPATCH_ELEM(dt, T, scatter_dim_kernel<T><<<gb_grid(a.n, 256), 256, 0, st>>>(
      a, reinterpret_cast<T*>(dst), idx, reinterpret_cast<const T*>(src), scalar_from_double<T>(value), scalar_src,
      mode, status));
  return (int)cudaGetLastError();
}

// Flat argument block of the general indexed read / write (all arrays padded to their maxima by the caller):
//   meta[0] nidx, [1] nb, [2] npre, [3] npost, [4..8) idx_i64
//   dims: [0..4) dim_size, [4..8) data_stride, [8..12) bshape, [12..15) pre_shape, [15..18) pre_stride,
//         [18..21) post_shape, [21..24) post_stride, [24..40) idx_bstride[k][d]
static int fill_index_args(IndexArgs& a, const void* const* idx, const int* meta, const long long* dims) {
  a.nidx = meta[0]; a.nb = meta[1]; a.npre = meta[2]; a.npost = meta[3];
  if (a.nidx < 1 || a.nidx > IDX_MAX || a.nb < 0 || a.nb > IDX_BDIMS || a.npre < 0 || a.npre > IDX_SIDE ||
      a.npost < 0 || a.npost > IDX_SIDE)
    return -3;
  for (int k = 0; k < IDX_MAX; ++k) {
    a.idx[k] = k < a.nidx ? idx[k] : nullptr;
    a.idx_i64[k] = meta[4 + k];
    a.dim_size[k] = dims[k];
    a.data_stride[k] = dims[4 + k];
    for (int d = 0; d < IDX_BDIMS; ++d) a.idx_bstride[k][d] = dims[24 + k * IDX_BDIMS + d];
  }
  a.n_b = 1; a.n_pre = 1; a.n_post = 1;
  for (int d = 0; d < IDX_BDIMS; ++d) { a.bshape[d] = d < a.nb ? dims[8 + d] : 1; a.n_b *= a.bshape[d]; }
  for (int d = 0; d < IDX_SIDE; ++d) {
    a.pre_shape[d] = d < a.npre ? dims[12 + d] : 1; a.pre_stride[d] = dims[15 + d]; a.n_pre *= a.pre_shape[d];
    a.post_shape[d] = d < a.npost ? dims[18 + d] : 1; a.post_stride[d] = dims[21 + d]; a.n_post *= a.post_shape[d];
  }
  return 0;
}

// Copies move bytes, so a contiguous innermost run may travel in wider units: returns the widest unit (<= 16 bytes)
// that divides the innermost extent, every stride and both base addresses, after rescaling `a` to that unit.
static int widen_index_units(IndexArgs& a, int es, const void* p0, const void* p1) {
  if (a.npost < 1 || a.post_stride[a.npost - 1] != 1) return es;
  for (int v = 16; v > es; v >>= 1) {
    const int f = v / es;
    bool ok = a.post_shape[a.npost - 1] % f == 0 &&
              (reinterpret_cast<uintptr_t>(p0) | reinterpret_cast<uintptr_t>(p1)) % v == 0;
    for (int d = 0; ok && d < a.npost - 1; ++d) ok = a.post_stride[d] % f == 0;
    for (int d = 0; ok && d < a.npre; ++d) ok = a.pre_stride[d] % f == 0;
    for (int k = 0; ok && k < a.nidx; ++k) ok = a.data_stride[k] % f == 0;
    if (!ok) continue;
    a.post_shape[a.npost - 1] /= f;
    a.n_post /= f;
    for (int d = 0; d < a.npost - 1; ++d) a.post_stride[d] /= f;
    for (int d = 0; d < a.npre; ++d) a.pre_stride[d] /= f;
    for (int k = 0; k < a.nidx; ++k) a.data_stride[k] /= f;
    return v;
  }
  return es;
}

extern "C" int gb_index_get(const void* src, void* out, const void* const* idx, const int* meta,
                            const long long* dims, int es, int* status, cudaStream_t st) {
  IndexArgs a;
  if (int r = fill_index_args(a, idx, meta, dims)) return r;
  if (a.n_pre * a.n_b * a.n_post == 0) return 0;
  es = widen_index_units(a, es, src, out);
  const long long n = a.n_pre * a.n_b * a.n_post;
  GB_DISPATCH_BYTES(es, U, index_get_kernel<U><<<gb_grid(n, 256), 256, 0, st>>>(
      a, reinterpret_cast<const U*>(src), reinterpret_cast<U*>(out), status));
  return (int)cudaGetLastError();
}

extern "C" int gb_index_put(void* dst, const void* val, double value, int scalar_src, int mode,
                            const void* const* idx, const int* meta, const long long* dims, int dt, int* status,
                            cudaStream_t st) {
  IndexArgs a;
  if (int r = fill_index_args(a, idx, meta, dims)) return r;
  const long long n = a.n_pre * a.n_b * a.n_post;
  if (n == 0) return 0;
  if (dt == DT_U8 || dt == DT_BOOL) {
    if (mode) return -2;
    index_put_kernel<uint8_t><<<gb_grid(n, 256), 256, 0, st>>>(
        a, reinterpret_cast<uint8_t*>(dst), reinterpret_cast<const uint8_t*>(val),
        (uint8_t)(dt == DT_BOOL ? (value != 0.0) : value), scalar_src, 0, status);
    return (int)cudaGetLastError();
  }
  GB_DISPATCH_ELEM(dt, T, index_put_kernel<T><<<gb_grid(n, 256), 256, 0, st>>>(
      a, reinterpret_cast<T*>(dst), reinterpret_cast<const T*>(val), scalar_from_double<T>(value), scalar_src, mode,
      status));
  return (int)cudaGetLastError();
}

// a viewed as [rows, inner] contiguous; mask [rows] bytes.
extern "C" int gb_masked_fill(void* a, const void* mask, double value, long long rows, long long inner, int dt,
                              cudaStream_t st) {
  const long long n = rows * inner;
  if (n == 0) return 0;
  if (dt == DT_U8 || dt == DT_BOOL) {
    masked_fill_kernel<uint8_t><<<gb_grid(n, 256), 256, 0, st>>>(
        reinterpret_cast<uint8_t*>(a), reinterpret_cast<const uint8_t*>(mask),
        (uint8_t)(dt == DT_BOOL ? (value != 0.0) : value), rows, inner);
    return (int)cudaGetLastError();
  }
  GB_DISPATCH_ELEM(dt, T, masked_fill_kernel<T><<<gb_grid(n, 256), 256, 0, st>>>(
      reinterpret_cast<T*>(a), reinterpret_cast<const uint8_t*>(mask), scalar_from_double<T>(value), rows, inner));
  return (int)cudaGetLastError();
}

// Contiguous fill for every element type the float fill kernel does not cover (integers, bool, float64).
extern "C" int gb_fill_elems(void* a, long long n, double value, int dt, cudaStream_t st) {
  if (n == 0) return 0;
  if (dt == DT_U8 || dt == DT_BOOL) {
    fill_elems_kernel<uint8_t><<<gb_grid(n, 256), 256, 0, st>>>(
        reinterpret_cast<uint8_t*>(a), (uint8_t)(dt == DT_BOOL ? (value != 0.0) : value), n);
    return (int)cudaGetLastError();
  }
  GB_DISPATCH_ELEM(dt, T, fill_elems_kernel<T><<<gb_grid(n, 256), 256, 0, st>>>(
      reinterpret_cast<T*>(a), scalar_from_double<T>(value), n));
  return (int)cudaGetLastError();
}
