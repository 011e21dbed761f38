// Shared pieces of the flash-attention kernels (forward in attention_sm100.cu, backward in
// attention_bwd_sm100.cu): parameters, swizzled tile stores, operand descriptors, tile loads, tensor maps.
#pragma once
#include "sm100_ptx.cuh"
#include "common.cuh"

namespace gb {

constexpr int AT_BM = 128;   // rows of a score tile (TMEM lanes)
constexpr int AT_BN = 128;   // columns of a score tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct AttnParams {
  void* o; float* lse;                       // forward outputs
  const float* lse_in; const float* delta;   // backward inputs
  void* dq; void* dk; void* dv;              // backward outputs
  int* status;
  int B, S, Sk, Hq, Hkv;
  int causal, is_bf16;
  float scale;                               // softmax scale
};

// 32 fp32 values of row `row`, columns c0..c0+31, into a K-major 128-byte-swizzled 16-bit tile whose
// 64-column chunks are `chunk_stride` bytes apart (the layout TMA SWIZZLE_128B produces).
template <bool BF16>
__device__ __forceinline__ void store_row_chunk_t(uint8_t* base, int u0, int row, const float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 w;
    w.x = pack2c<BF16>(v[i * 8 + 0], v[i * 8 + 1]);
    w.y = pack2c<BF16>(v[i * 8 + 2], v[i * 8 + 3]);
    w.z = pack2c<BF16>(v[i * 8 + 4], v[i * 8 + 5]);
    w.w = pack2c<BF16>(v[i * 8 + 6], v[i * 8 + 7]);
    *reinterpret_cast<uint4*>(base + (((u0 + i) ^ (row & 7)) << 4)) = w;
  }
}
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int row, int c0, const float (&v)[32], int is_bf16,
                                                int chunk_stride) {
  uint8_t* base = tile + (c0 >> 6) * chunk_stride + row * 128;
  const int u0 = (c0 & 63) >> 3;
  if (is_bf16) store_row_chunk_t<true>(base, u0, row, v);
  else store_row_chunk_t<false>(base, u0, row, v);
}

// K-major operand (contraction inside the 128-byte rows): k-step kk of 16 elements
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int kk, int rows) {
  return make_smem_desc(tile_addr + (kk >> 2) * rows * 128 + (kk & 3) * 32, 16, 1024);
}
// MN-major operand (contraction over the rows of the tile): k-step kk of 16 rows
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int kk, int rows) {
  return make_smem_desc(tile_addr + kk * 2048, rows * 128, 1024);
}

template <int D>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int head, int row0,
                                          int b, int rows) {
#pragma unroll
  for (int dc = 0; dc < D / 64; ++dc) tma_load_4d(dst + dc * rows * 128, m, bar, dc * 64, head, row0, b);
}

#define AT_WAIT(bar, ph, site) mbar_wait((bar), (ph), abort_flag, p.status, (site))

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


// ------------------------------------------------------------------------------------------------
// host
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn4)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn4 encode4() {
  static EncodeTiledFn4 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn4>(ptr);
  }
  return fn;
}

// [B, S, H, D] 16-bit tensor -> map with dims {D, H, S, B}, box {64, 1, 128, 1}, 128-byte swizzle
static inline int make_tmap_bshd(CUtensorMap* out, const void* base, int is_bf16, int B, int S, int H, int D,
                                 int box_rows = 128) {
  EncodeTiledFn4 enc = encode4();
  if (enc == nullptr) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)H * D * 2, (cuuint64_t)S * H * D * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  return (int)enc(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}



}  // namespace gb
