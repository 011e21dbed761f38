// GEMM for sm_100a on the 5th-generation tensor cores.
//
//   D[z][M,N] (+)= A[za] * B[zb]^T (+ bias)         fp32 accumulation in tensor memory
//
// One persistent, warp-specialised kernel:
//   warp 0    TMA producer   cp.async.bulk.tensor (128-byte swizzle) into a ring of smem stages
//   warp 1    MMA issuer     one elected thread issues tcgen05.mma (UMMA 128 x BN x 16); TMEM owner
//   warps 2-9 epilogue       tcgen05.ld of the finished accumulator -> bias/convert -> swizzled smem slab of the
//                            warp -> TMA store (or TMA add-reduce for fp32 accumulation and split-K); outputs
//                            whose base or pitch is not 16-byte aligned take plain per-thread stores instead
//                            (two warps per TMEM lane quarter, each takes half of the tile's columns)
// Two accumulators live in TMEM (2 x BN columns), so the epilogue of tile i overlaps the main loop of
// tile i+1.  Every load targets one CTA only: the kernel is safe in multi-GPU jobs.
//
// Operand layouts (what the backward passes of a linear layer need without transposes):
//   A "K-major"  : memory [M, K] row-major          A "MN-major": memory [K, M] row-major
//   B "K-major"  : memory [N, K] row-major          B "MN-major": memory [K, N] row-major
// Group modes for mixture-of-experts (segments padded to multiples of 128 rows):
//   GROUP_M : rows of A/D are split in segments, segment g multiplies B[g]
//   GROUP_K : the contraction runs over segment g of the rows of A and B, result goes to D[g]
//
// Reference counterpart: the Triton `matmul_kernel` / `bmm_kernel`, genesis/ops/cuda/matrix_ops.py:21-294.
#include "sm100_ptx.cuh"
#include "common.cuh"

namespace gb {

constexpr int BM = 128;
constexpr int BK_BYTES = 128;   // one swizzle row of K per stage: 64 x 16-bit or 32 x tf32

enum GroupMode : int { GROUP_NONE = 0, GROUP_M = 1, GROUP_K = 2 };

struct GemmParams {
  void* D;
  const void* bias;        // [N] or nullptr
  const int* group_offsets;  // [groups+1] or nullptr
  int* status;
  long long strideD;       // elements between batches / groups of D
  int M, N, K, batch;
  int ldd;
  int out_dtype;           // DT_F32 / DT_F16 / DT_BF16
  int bias_dtype;
  int accumulate;          // D += result
  int group_mode;
  int groups;
  int m_fastest;           // tile order
  int raster_group;        // tiles of the fast dimension swept together (keeps both operand panels in L2)
  int splits;              // split-K factor (>1: fp32 output, partial sums combined with adds in memory)
  int tma_out;             // 0: per-thread stores; 1: TMA store; 2: TMA add-reduce (fp32 output)
  int stream_k;            // 1: every CTA takes an equal, contiguous share of all (tile, k-iteration) units and adds
                           //    its partial tiles into the fp32 output (needs tma_out == 2)
  float alpha;
};

template <int BN, int STAGES, int ESIZE>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK_BYTES;
  static constexpr int B_BYTES = BN * BK_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BARRIER_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int SLAB_OFFSET = BARRIER_OFFSET + 1024;      // 8 epilogue warps x [32 rows x 128 bytes]
  static constexpr int SLAB_BYTES = 32 * 128;
  static constexpr int TOTAL = SLAB_OFFSET + 8 * SLAB_BYTES;
};

// Find the segment that contains row `m0` (offsets ascending, last = total padded rows).
__device__ __forceinline__ int find_group(const int* offs, int groups, int m0) {
  int lo = 0, hi = groups;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (offs[mid] <= m0) lo = mid; else hi = mid;
  }
  return lo;
}

template <int BN, int STAGES, int ESIZE, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(320, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
            const __grid_constant__ CUtensorMap tmapD, const GemmParams p) {
  using L = SmemLayout<BN, STAGES, ESIZE>;
  constexpr int BK = BK_BYTES / ESIZE;              // elements of K per stage
  constexpr int UMMA_K = 32 / ESIZE;                // 16 for 16-bit, 8 for tf32
  constexpr int KSTEPS = BK / UMMA_K;               // 4
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if (status_poisoned(p.status)) return;
  // No alignment pad: the kernel has no static shared memory, so the dynamic part starts 1024-aligned.  The 2 KB this
  // leaves free per SM is what lets a communication CTA (no shared memory of its own) share the SM with a GEMM CTA.
  if ((reinterpret_cast<uintptr_t>(smem_raw) & 1023) != 0) {
    if (threadIdx.x == 0) report_error(p.status, GB_ERR_BAD_ARG, 4, 0);
    return;
  }
  uint8_t* smem = smem_raw;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BARRIER_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  int* s_offs = reinterpret_cast<int*>(tmem_base_slot + 4);   // up to 200 group offsets

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 8); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmapA);
    tma_prefetch_desc(&tmapB);
    if (p.tma_out) tma_prefetch_desc(&tmapD);
  }
  if (p.group_mode != GROUP_NONE) {
    for (int i = threadIdx.x; i <= p.groups; i += blockDim.x) s_offs[i] = p.group_offsets[i];
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int nz = (p.group_mode == GROUP_K) ? p.groups : p.batch * p.splits;
  const long long total_tiles = (long long)tiles_m * tiles_n * nz;
  const int k_iters_per_split = (((p.K + BK - 1) / BK) + p.splits - 1) / p.splits;

  // z carries (batch, split) for plain GEMMs: z = batch * splits + split
  auto decode = [&](long long t, int& mi, int& ni, int& z) {
    z = (int)(t / ((long long)tiles_m * tiles_n));
    int r = (int)(t % ((long long)tiles_m * tiles_n));
    const int g = p.raster_group;
    if (p.m_fastest) {
      const int grp = r / (g * tiles_n), rr = r % (g * tiles_n);
      const int gs = (tiles_m - grp * g) < g ? (tiles_m - grp * g) : g;
      mi = grp * g + rr % gs; ni = rr / gs;
    } else {
      const int grp = r / (g * tiles_m), rr = r % (g * tiles_m);
      const int gs = (tiles_n - grp * g) < g ? (tiles_n - grp * g) : g;
      ni = grp * g + rr % gs; mi = rr / gs;
    }
  };
  // stream-K: this CTA's share of the tiles x k-iterations units
  const long long k_iters_total = (p.K + BK - 1) / BK;
  const long long sk_units = total_tiles * k_iters_total;
  const long long sk_u0 = p.stream_k ? sk_units * blockIdx.x / gridDim.x : 0;
  const long long sk_u1 = p.stream_k ? sk_units * (blockIdx.x + 1) / gridDim.x : 0;
  // k range of a tile, in elements
  auto krange = [&](int z, int& k_begin, int& k_end) {
    if (p.group_mode == GROUP_K) { k_begin = s_offs[z]; k_end = s_offs[z + 1]; }
    else if (p.splits > 1) {
      const int sp = z % p.splits;
      k_begin = sp * k_iters_per_split * BK;
      k_end = k_begin + k_iters_per_split * BK;
      if (k_end > p.K) k_end = p.K;
    } else { k_begin = 0; k_end = p.K; }
  };

  // Next piece of work of this CTA.  Classic: `cur` walks the tiles (stride gridDim.x), each with its whole k range.
  // Stream-K: `cur` walks this CTA's units; a piece is the part of one tile's k range that falls inside them.
  auto advance = [&](long long& cur, int& mi, int& ni, int& z, int& k_begin, int& k_end) -> bool {
    if (!p.stream_k) {
      if (cur >= total_tiles) return false;
      decode(cur, mi, ni, z);
      krange(z, k_begin, k_end);
      cur += gridDim.x;
      return true;
    }
    if (cur >= sk_u1) return false;
    const long long tile = cur / k_iters_total;
    const long long kb = cur % k_iters_total;
    long long len = k_iters_total - kb;
    if (len > sk_u1 - cur) len = sk_u1 - cur;
    decode(tile, mi, ni, z);
    k_begin = (int)(kb * BK);
    k_end = (int)((kb + len) * BK);
    if (k_end > p.K) k_end = p.K;
    cur += len;
    return true;
  };
  const long long cur0 = p.stream_k ? sk_u0 : (long long)blockIdx.x;

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (elect_one()) {
      uint32_t it = 0;
      long long cur = cur0;
      int mi, ni, z, k_begin, k_end;
      while (!*abort_flag && advance(cur, mi, ni, z, k_begin, k_end)) {
        const int m0 = mi * BM, n0 = ni * BN;
        int za = z / p.splits, zb = z / p.splits;
        if (p.group_mode == GROUP_M) {
          if (m0 >= s_offs[p.groups]) continue;
          za = 0; zb = find_group(s_offs, p.groups, m0);
        } else if (p.group_mode == GROUP_K) { za = 0; zb = 0; }
        for (int k0 = k_begin; k0 < k_end; k0 += BK, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, 100)) break;
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_3d(sa, &tmapA, &full_bar[s], k0, m0, za);
          } else {
#pragma unroll
            for (int c = 0; c < BM / (BK_BYTES / ESIZE); ++c)
              tma_load_3d(sa + c * (BK * BK_BYTES), &tmapA, &full_bar[s], m0 + c * (BK_BYTES / ESIZE), k0, za);
          }
          if constexpr (!B_MN) {
            tma_load_3d(sb, &tmapB, &full_bar[s], k0, n0, zb);
          } else {
#pragma unroll
            for (int c = 0; c < BN / (BK_BYTES / ESIZE); ++c)
              tma_load_3d(sb + c * (BK * BK_BYTES), &tmapB, &full_bar[s], n0 + c * (BK_BYTES / ESIZE), k0, zb);
          }
        }
      }
      // Drain: every load issued above has been (or will be) consumed by the MMA warp, which
      // waits on the full barriers; on abort, give in-flight copies a bounded time to land.
      if (*abort_flag) {
        for (int s = 0; s < STAGES; ++s) {
          uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full_bar[s], 0) && !mbar_try_wait(&full_bar[s], 1) &&
                 globaltimer_ns() - t0 < 1000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer (one thread) ===========================
    if (lane == 0) {
      const uint32_t fmt = (ESIZE == 4) ? 2u : (uint32_t)(p.out_dtype >> 8);   // operand format rides in bits 8+
      const uint32_t idesc = make_idesc(fmt, A_MN ? 1u : 0u, B_MN ? 1u : 0u, BM, BN);
      uint32_t it = 0, tile_no = 0;
      long long cur = cur0;
      int mi, ni, z, k_begin, k_end;
      while (!*abort_flag && advance(cur, mi, ni, z, k_begin, k_end)) {
        if (p.group_mode == GROUP_M && mi * BM >= s_offs[p.groups]) continue;
        const uint32_t acc = tile_no & 1;
        const uint32_t acc_ph = (tile_no >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag, p.status, 200)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool first = true;
        bool ok = true;
        for (int k0 = k_begin; k0 < k_end; k0 += BK, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, 201)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t b_addr = a_addr + L::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < KSTEPS; ++kk) {
            // K-major: advance 32 bytes inside the 128-byte swizzle row.
            // MN-major: advance UMMA_K k-rows of 128 bytes.
            const uint64_t da = A_MN ? make_smem_desc(a_addr + kk * UMMA_K * BK_BYTES, BK * BK_BYTES, 1024)
                                     : make_smem_desc(a_addr + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(b_addr + kk * UMMA_K * BK_BYTES, BK * BK_BYTES, 1024)
                                     : make_smem_desc(b_addr + kk * 32, 16, 1024);
            if constexpr (ESIZE == 4) umma_tf32(d_tmem, da, db, idesc, (first && kk == 0) ? 0u : 1u);
            else umma_f16(d_tmem, da, db, idesc, (first && kk == 0) ? 0u : 1u);
          }
          umma_commit(&empty_bar[s]);   // frees the smem stage once these MMAs have read it
          first = false;
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);
        ++tile_no;
      }
    }
    __syncwarp();
  } else {
    // =========================== epilogue warps ===========================
    const int q = warp & 3;                       // TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;             // which half of the tile's columns this warp stores
    constexpr int HALF_N = BN / 2;
    const bool use_atomics = p.splits > 1;
    uint8_t* slab = smem + L::SLAB_OFFSET + (warp - 2) * L::SLAB_BYTES;
    uint8_t* slab_row = slab + lane * 128;
    uint32_t tile_no = 0;
    long long cur = cur0;
    int mi, ni, z, k_begin, k_end;
    while (!*abort_flag && advance(cur, mi, ni, z, k_begin, k_end)) {
      const int m0 = mi * BM, n0 = ni * BN;
      if (p.group_mode == GROUP_M && m0 >= s_offs[p.groups]) continue;
      const uint32_t acc = tile_no & 1;
      const uint32_t acc_ph = (tile_no >> 1) & 1;
      const bool empty_k = (k_end <= k_begin);
      // all lanes must agree before the warp-collective tcgen05.ld below
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[acc], acc_ph, abort_flag, p.status, 300))) break;
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const int zd = (p.group_mode == GROUP_K) ? z : z / p.splits;
      const long long zoff = (p.group_mode == GROUP_M) ? 0 : (long long)zd * p.strideD;
      const size_t row_off = (size_t)zoff + (size_t)row * p.ldd;
      const int dt = p.out_dtype & 0xff;
#pragma unroll 1
      for (int c = half * HALF_N; c < (half + 1) * HALF_N; c += 64) {
        // 64 accumulator columns per TMEM round trip
        uint32_t r[2][32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c;
        tmem_ld_32x32b_x32(taddr, r[0]);
        tmem_ld_32x32b_x32(taddr + 32, r[1]);
        tmem_ld_wait();
        if (p.tma_out) {
          // the warp's 32 x 128-byte slab (128-byte swizzle, as the tensor map expects) goes out as one box
          const int zc = (p.group_mode == GROUP_M) ? 0 : zd;
          const int y0 = m0 + q * 32;
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int col0 = n0 + c + hh * 32;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = empty_k ? 0.f : __uint_as_float(r[hh][j]) * p.alpha;
            if (p.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] += load_as_float(p.bias, p.bias_dtype, col0 + j);
            }
            if (dt == DT_F32) {
              // 32 fp32 columns fill the slab: one box per half batch
              if (lane == 0) bulk_wait_group_read<0>();
              __syncwarp();
#pragma unroll
              for (int u = 0; u < 8; ++u)
                *reinterpret_cast<float4*>(slab_row + ((u ^ (lane & 7)) << 4)) =
                    make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0 && y0 < p.M && col0 < p.N) {
                if (p.tma_out == 2) tma_reduce_add_3d(&tmapD, slab, col0, y0, zc);
                else tma_store_3d(&tmapD, slab, col0, y0, zc);
                bulk_commit_group();
              }
            } else {
              // 64 16-bit columns fill the slab: this half batch writes units 4*hh .. 4*hh+3 of each row
              if (hh == 0) {
                if (lane == 0) bulk_wait_group_read<0>();
                __syncwarp();
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                uint4 o;
                o.x = pack2(v[8 * u], v[8 * u + 1], dt); o.y = pack2(v[8 * u + 2], v[8 * u + 3], dt);
                o.z = pack2(v[8 * u + 4], v[8 * u + 5], dt); o.w = pack2(v[8 * u + 6], v[8 * u + 7], dt);
                *reinterpret_cast<uint4*>(slab_row + (((4 * hh + u) ^ (lane & 7)) << 4)) = o;
              }
              if (hh == 1) {
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && y0 < p.M && n0 + c < p.N) {
                  tma_store_3d(&tmapD, slab, n0 + c, y0, zc);
                  bulk_commit_group();
                }
              }
            }
          }
          continue;
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int col0 = n0 + c + hh * 32;
          if (!(row_ok && col0 < p.N)) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = empty_k ? 0.f : __uint_as_float(r[hh][j]) * p.alpha;
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) v[j] += load_as_float(p.bias, p.bias_dtype, col0 + j);
          }
          const bool full = (col0 + 32 <= p.N);
          if (dt == DT_F32) {
            float* dst = reinterpret_cast<float*>(p.D) + row_off + col0;
            const bool vec = full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
            if (use_atomics) {
              if (vec) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  atomicAdd(reinterpret_cast<float4*>(dst + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
              } else {
                for (int j = 0; j < 32 && col0 + j < p.N; ++j) atomicAdd(dst + j, v[j]);
              }
            } else if (vec) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (p.accumulate) { float4 old = *reinterpret_cast<float4*>(dst + j); o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
                *reinterpret_cast<float4*>(dst + j) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = p.accumulate ? dst[j] + v[j] : v[j];
            }
          } else {
            uint16_t* dst = reinterpret_cast<uint16_t*>(p.D) + row_off + col0;
            if (p.accumulate) {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) v[j] += half_bits_to_float(dst[j], dt);
            }
            if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 o;
                o.x = pack2(v[j], v[j + 1], dt); o.y = pack2(v[j + 2], v[j + 3], dt);
                o.z = pack2(v[j + 4], v[j + 5], dt); o.w = pack2(v[j + 6], v[j + 7], dt);
                *reinterpret_cast<uint4*>(dst + j) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = float_to_half_bits(v[j], dt);
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      ++tile_no;
    }
    // the slab must outlive the last store's read of it
    if (lane == 0) bulk_wait_group_read<0>();
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 3-D map over (inner, outer, batch) with a {128 bytes, box_outer, 1} box and 128-byte swizzle.
int make_tmap_3d(CUtensorMap* out, const void* base, int dtype, long long inner, long long outer,
                 long long batch, long long ld_elems, long long batch_stride_elems, int box_outer) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -1;
  const int es = (dtype == DT_F32) ? 4 : 2;
  CUtensorMapDataType dt = dtype == DT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)(batch > 0 ? batch : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)ld_elems * es,
                           (cuuint64_t)(batch > 1 ? batch_stride_elems : (long long)outer * ld_elems) * es};
  cuuint32_t box[3] = {(cuuint32_t)(128 / es), (cuuint32_t)box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (int)r;
}

template <int BN, int STAGES, int ESIZE, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const GemmParams& p,
                       int sms, cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES, ESIZE>;
  auto kern = gemm_kernel<BN, STAGES, ESIZE, A_MN, B_MN>;
  static unsigned long long configured = 0;
  if (int e = smem_opt_in(kern, L::TOTAL, configured)) return e;
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int nz = (p.group_mode == GROUP_K) ? p.groups : p.batch * p.splits;
  long long total = (long long)tiles_m * tiles_n * nz;
  int grid = (int)(total < sms ? total : sms);
  if (p.stream_k) {
    // at least 16 k-iterations per CTA, so that a piece's main loop outweighs its 128 KB epilogue
    const long long units = total * ((p.K + (BK_BYTES / ESIZE) - 1) / (BK_BYTES / ESIZE));
    long long g = units / 16;
    grid = (int)(g < sms ? g : sms);
  }
  if (grid < 1) grid = 1;
  kern<<<grid, 320, L::TOTAL, stream>>>(ta, tb, td, p);
  return (int)cudaGetLastError();
}

template <int BN, int STAGES, int ESIZE>
static int dispatch_major(int a_mn, int b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                          const GemmParams& p, int sms, cudaStream_t s) {
  if (!a_mn && !b_mn) return launch_gemm<BN, STAGES, ESIZE, false, false>(ta, tb, td, p, sms, s);
  if (!a_mn && b_mn) return launch_gemm<BN, STAGES, ESIZE, false, true>(ta, tb, td, p, sms, s);
  if (a_mn && !b_mn) return launch_gemm<BN, STAGES, ESIZE, true, false>(ta, tb, td, p, sms, s);
  return launch_gemm<BN, STAGES, ESIZE, true, true>(ta, tb, td, p, sms, s);
}

}  // namespace gb

using namespace gb;

// C ABI.  in_dtype: DT_F32 (tf32 tensor cores) / DT_F16 / DT_BF16.  a_mn / b_mn: operand is stored
// with M (resp. N) contiguous.  lda / ldb: leading dimension of the stored matrix in elements.
// Requirements: base pointers 16-byte aligned, leading dimensions multiples of 16 bytes.
extern "C" int gb_gemm(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int batch,
                       long long lda, long long ldb, int ldd, long long strideA, long long strideB,
                       long long strideD, int a_mn, int b_mn, int in_dtype, int out_dtype, int bias_dtype,
                       int accumulate, float alpha, int group_mode, const int* group_offsets, int groups,
                       int splits, int bn_hint, int* status, int sm_count, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  const int es = (in_dtype == DT_F32) ? 4 : 2;
  const int bk = 128 / es;
  const int bn = (N <= 128 || bn_hint == 128) ? 128 : 256;
  // splits < 0 asks for stream-K (see GemmParams::stream_k); it needs what split-K needs, and the TMA add path
  const bool want_stream_k = splits < 0;
  if (splits < 1 || group_mode != GROUP_NONE || out_dtype != DT_F32) splits = 1;
  CUtensorMap ta, tb;
  int r;
  // A: K-major map dims (K, M); MN-major map dims (M, K); boxes: {bk, 128} resp. {bk(along M), bk rows of K}
  const long long a_batches = (group_mode == GROUP_NONE) ? batch : 1;
  const long long b_batches = (group_mode == GROUP_M) ? groups : ((group_mode == GROUP_K) ? 1 : batch);
  if (!a_mn) r = make_tmap_3d(&ta, A, in_dtype, K, M, a_batches, lda, strideA, BM);
  else r = make_tmap_3d(&ta, A, in_dtype, M, K, a_batches, lda, strideA, bk);
  if (r != 0) return 10000 + r;
  if (!b_mn) r = make_tmap_3d(&tb, B, in_dtype, K, N, b_batches, ldb, strideB, bn);
  else r = make_tmap_3d(&tb, B, in_dtype, N, K, b_batches, ldb, strideB, bk);
  if (r != 0) return 20000 + r;
  GemmParams p;
  p.D = D; p.bias = bias; p.group_offsets = group_offsets; p.status = status; p.strideD = strideD;
  p.M = M; p.N = N; p.K = K; p.batch = batch < 1 ? 1 : batch; p.ldd = ldd;
  p.out_dtype = out_dtype | ((in_dtype == DT_BF16 ? 1 : 0) << 8);
  p.bias_dtype = bias_dtype; p.accumulate = accumulate; p.group_mode = group_mode; p.groups = groups;
  p.alpha = alpha;
  p.splits = splits;
  // Output through TMA when the tensor-map rules allow it: 16-byte aligned base, pitch and batch stride.
  // fp32 accumulation and split-K become add-reductions in memory; 16-bit accumulation keeps the
  // read-modify-write path (one rounding instead of two).
  CUtensorMap td = ta;
  p.tma_out = 0;
  {
    const int eso = (out_dtype == DT_F32) ? 4 : 2;
    const bool adds = accumulate != 0 || splits > 1;
    const long long d_batches = (group_mode == GROUP_K) ? groups : ((group_mode == GROUP_M) ? 1 : p.batch);
    const bool aligned = (reinterpret_cast<uintptr_t>(D) & 15) == 0 && ((long long)ldd * eso) % 16 == 0 &&
                         (d_batches <= 1 || (strideD * eso) % 16 == 0);
    const bool sk_ok = want_stream_k && group_mode == GROUP_NONE && out_dtype == DT_F32 && p.batch == 1 &&
                       bias == nullptr;
    if (aligned && (!adds || out_dtype == DT_F32)) {
      r = make_tmap_3d(&td, D, out_dtype, N, M, d_batches, ldd, strideD, 32);
      if (r == 0) p.tma_out = (adds || sk_ok) ? 2 : 1;
    }
    p.stream_k = (sk_ok && p.tma_out == 2) ? 1 : 0;
    if (want_stream_k && !p.stream_k) return -5;      // the caller zeroed D for adds: refuse rather than overwrite
  }
  // Sweep the dimension whose operand is smaller fastest, so the larger one streams from HBM once
  // and the smaller one stays in L2.
  p.m_fastest = ((long long)M <= (long long)N) ? 1 : 0;
  {
    // If the operand of the fast dimension fits comfortably in L2, sweep it whole (the other operand then
    // streams from HBM exactly once); otherwise walk 16-tile groups so a wave touches ~16 + ~9 panels.
    const long long fast_bytes = (long long)(p.m_fastest ? M : N) * K * es;
    const int fast_tiles = p.m_fastest ? (M + BM - 1) / BM : (N + bn - 1) / bn;
    p.raster_group = (fast_bytes <= (48ll << 20)) ? fast_tiles : 16;
    if (p.raster_group < 1) p.raster_group = 1;
  }
  if (es == 4) {
    if (bn == 128) return dispatch_major<128, 4, 4>(a_mn, b_mn, ta, tb, td, p, sm_count, stream);
    return dispatch_major<256, 4, 4>(a_mn, b_mn, ta, tb, td, p, sm_count, stream);
  }
  if (bn == 128) return dispatch_major<128, 6, 2>(a_mn, b_mn, ta, tb, td, p, sm_count, stream);
  return dispatch_major<256, 4, 2>(a_mn, b_mn, ta, tb, td, p, sm_count, stream);
}
