// Wide rows streamed through shared memory: one CTA owns a grid-strided set of rows and keeps the NEXT row of its set
// in flight (one bulk asynchronous copy per row, completion counted on an mbarrier) while the current row is reduced
// and written out from shared memory.  The register-resident row kernels load a row, reduce it, then store it, and
// with rows of 8 KB and more too few rows fit on an SM for the three phases of different rows to cover each other
// (measured: 46 % DRAM utilisation on [8192, 16384] bf16); here loads never wait for the arithmetic.
// `Op::row(state, srow, r, cols, sh)` is called by all threads of the CTA with the row in shared memory; `Op::State` is
// per-thread data that `Op::init` prepares once per CTA (column weights kept in registers across rows).
#pragma once
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace gb {

constexpr int RS_THREADS = 256;
constexpr int RS_MIN_ROW_BYTES = 8192;        // below this the register-resident kernels have enough rows in flight
constexpr int RS_MAX_ROW_BYTES = 65536;

// `bytes` from global to shared memory (both 16-byte aligned, bytes a multiple of 16), completion posted on `bar`
__device__ __forceinline__ void rs_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <typename T, typename Op>
__global__ void __launch_bounds__(RS_THREADS)
row_stream_kernel(const T* __restrict__ x, long long rows, int cols, Op op, int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t rs_smem[];
  __shared__ float sh[64];
  __shared__ __align__(8) uint64_t full[2];
  __shared__ int abort_flag;
  if (status_poisoned(status)) return;
  const uint32_t row_bytes = (uint32_t)cols * (uint32_t)sizeof(T);
  const long long stride = gridDim.x;
  if (threadIdx.x == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      const long long r = blockIdx.x + s * stride;
      if (r < rows) {
        mbar_expect_tx(&full[s], row_bytes);
        rs_bulk_load(rs_smem + (size_t)s * row_bytes, x + r * cols, row_bytes, &full[s]);
      }
    }
  }
  typename Op::State state;
  op.init(state, cols);
  int it = 0;
  for (long long r = blockIdx.x; r < rows; r += stride, ++it) {
    const int s = it & 1;
    const uint32_t ph = (it >> 1) & 1;
    const bool ok = mbar_wait(&full[s], ph, &abort_flag, status, 700);
    if (!__syncthreads_and(ok ? 1 : 0)) {
      // a copy that never arrived: the other stage may still be in flight; give it its own bounded wait so that
      // nothing is written into this CTA's shared memory after it has left
      if (threadIdx.x == 0 && r + stride < rows) mbar_wait(&full[s ^ 1], (uint32_t)(((it + 1) >> 1) & 1), &abort_flag, nullptr, 701);
      return;
    }
    op.row(state, reinterpret_cast<const T*>(rs_smem + (size_t)s * row_bytes), r, cols, sh);
    __syncthreads();                                   // every thread is done with this stage
    const long long nxt = r + 2 * stride;
    if (threadIdx.x == 0 && nxt < rows) {
      mbar_expect_tx(&full[s], row_bytes);
      rs_bulk_load(rs_smem + (size_t)s * row_bytes, x + nxt * cols, row_bytes, &full[s]);
    }
  }
}

// grid and shared-memory size of a launch; 0 CTAs when the shape does not qualify
template <typename T, typename Op>
static int rs_launch(const T* x, long long rows, int cols, const Op& op, int* status, unsigned long long& cfg_mask,
                     cudaStream_t st) {
  const long long row_bytes = (long long)cols * (long long)sizeof(T);
  const int smem = (int)(2 * row_bytes);
  auto kern = row_stream_kernel<T, Op>;
  if (int e = smem_opt_in(kern, 2 * RS_MAX_ROW_BYTES, cfg_mask)) return e;      // once per device: the largest row
  int per_sm = (int)((220 * 1024) / (smem + 1024));
  if (per_sm > 8) per_sm = 8;
  if (per_sm < 1) per_sm = 1;
  long long grid = 148ll * per_sm;
  if (grid > rows) grid = rows;
  kern<<<(unsigned)grid, RS_THREADS, smem, st>>>(x, rows, cols, op, status);
  return (int)cudaGetLastError();
}

static inline bool rs_shape_ok(const void* x, long long rows, long long cols, int elem_size) {
  const long long rb = cols * elem_size;
  return rows >= 64 && rb >= RS_MIN_ROW_BYTES && rb <= RS_MAX_ROW_BYTES && rb % 16 == 0 &&
         (reinterpret_cast<uintptr_t>(x) & 15) == 0;
}

}  // namespace gb
