// GEMM on CTA pairs: one tcgen05.mma.cta_group::2 instruction drives the tensor cores of two SMs.
//
//   D[M, N] (+)= A * B^T (+ bias)        16-bit operands, fp32 accumulation in the tensor memory of both SMs
//
// A cluster of two CTAs works on a 256 x BN tile (BN = 128 / 192 / 256).  CTA r of the pair
//   * loads ITS 128 rows of A and ITS BN/2 rows of B (plain per-CTA TMA loads, no cluster broadcast),
//   * owns accumulator rows [128 r, 128 r + 128) in its own tensor memory and stores them itself.
// The MMA thread of CTA 0 issues the instructions for the pair: the hardware reads each CTA's A rows and
// both halves of B out of the two shared memories, so every SM fetches 2/3 of the operand bytes per flop that
// the single-CTA 128 x 256 tile needs (32 KB instead of 48 KB per k-step of 64), which is what that kernel
// is bound by on shapes with a short k extent.
//
// Synchronisation (all mbarriers live at the same offsets in both CTAs):
//   full[s]       in CTA 0 only: both CTAs' TMA loads complete_tx on it, CTA 0's producer posts the byte count
//   empty[s]      per CTA: arrived by tcgen05.commit from CTA 0's MMA thread (one commit per CTA)
//   tmem_full[a]  per CTA: same, after the last k-step of a tile
//   tmem_empty[a] in CTA 0 only: the 8 epilogue warps of BOTH CTAs arrive (CTA 1 through its cluster address)
// Every wait is bounded; a CTA that gives up raises the abort flag of both CTAs, and both always reach the
// cluster barrier in front of the TMEM release.
//
// Epilogues: plain (bias, alpha, convert, TMA store or fp32 TMA add-reduce), or SwiGLU: the B operand is a stacked
// [gate; up] weight, CTA 0 loads gate rows and CTA 1 the matching up rows, so accumulator columns [0, 128) are
// gate and [128, 256) up of the same 128 hidden units, and the epilogue writes gate | up (for backward) and
// silu(gate) * up in one pass: the separate activation kernel and its read of gate | up disappear.
//
// SwiGLU backward epilogue: the product is dh (the gradient of silu(gate) * up, i.e. the data gradient of the down
// projection); the epilogue reads gate | up of the forward pass for its tile and stores d(gate) | d(up) directly, so
// dh is never written to memory and the stand-alone backward activation pass disappears.
//
// Reference counterpart: the Triton `matmul_kernel`, genesis/ops/cuda/matrix_ops.py:21-294, and the SiLU kernels
// of genesis/nn/triton_ops/silu.py:29-85.
#include <type_traits>
#include "sm100_ptx.cuh"
#include "common.cuh"

namespace gb {

int make_tmap_3d(CUtensorMap* out, const void* base, int dtype, long long inner, long long outer, long long batch,
                 long long ld_elems, long long batch_stride_elems, int box_outer);

namespace g2 {

constexpr int BM = 128;              // rows of A / D per CTA (256 per pair)
constexpr int BK = 64;               // 16-bit elements of K per stage (one 128-byte swizzle row)
constexpr int A_BYTES = BM * 128;    // 16 KB
constexpr int B_BYTES = 128 * 128;   // up to 128 rows of B per CTA
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SLAB_BYTES = 32 * 128;
constexpr int ACC_STRIDE = 256;      // TMEM columns between the two accumulators

enum : int { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_SWIGLU_BWD = 2 };

struct Params {
  const void* bias;
  int* status;
  int M, N, K;             // N: columns of D (plain) or hidden units (SwiGLU: D has 2 N columns, D2 has N)
  int bn;                  // pair tile width: 128 / 192 / 256 (SwiGLU: 256 = 128 gate + 128 up)
  int out_dtype, in_bf16, bias_dtype;
  int accumulate;          // fp32 output only: add into D (TMA add-reduce)
  int m_fastest, raster_group;
  int write_gu;            // SwiGLU: also store gate | up
  const void* gu;          // SwiGLU backward: gate | up of the forward pass, [M, 2 N] with pitch ld_gu elements
  int ld_gu;
  float alpha;
};

template <int STAGES, int SLABS>
struct Smem {
  static constexpr int BARRIER_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int SLAB_OFFSET = BARRIER_OFFSET + 1024;
  static constexpr int TOTAL = SLAB_OFFSET + 8 * SLABS * SLAB_BYTES;
};

// ---- cluster helpers ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cta_rank_in_cluster() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local` (a shared::cta address) inside CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
}

// ---- tcgen05, pair forms ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc2(uint32_t* dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t addr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}
// arrives on the mbarrier at shared::cluster address `bar` once all MMAs issued so far by this thread are done
__device__ __forceinline__ void umma2_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// per-CTA TMA load whose completion is posted on a barrier of the pair (shared::cluster address)
__device__ __forceinline__ void tma2_load_3d(void* smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Ties 16 registers to this point of the instruction stream: placed after tcgen05.wait::ld, it keeps every use of
// registers that an earlier tcgen05.ld fills asynchronously behind the wait.  Emits no instruction.
__device__ __forceinline__ void reg_fence16(uint32_t (&r)[16]) {
  asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                    "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                    "+r"(r[15]));
}

__device__ __forceinline__ void reg_fence32(uint32_t (&r)[32]) {
  asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                    "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                    "+r"(r[15]));
  asm volatile("" : "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]),
                    "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]),
                    "+r"(r[30]), "+r"(r[31]));
}

// two packed 16-bit values (low half first) -> floats
template <bool BF16>
__device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi) {
  if (BF16) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x; hi = f.y;
  }
}
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// 32 bytes from global memory through the read-only path (address 32-byte aligned)
__device__ __forceinline__ void ld_nc_v8(uint32_t* r, const void* p) {
  asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "l"(p));
}

__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.f + __expf(-x)); }

template <int STAGES, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(320, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
             const __grid_constant__ CUtensorMap tmapD, const __grid_constant__ CUtensorMap tmapD2, const Params p) {
  constexpr int SLABS = (EPI == EPI_SWIGLU) ? 3 : (EPI == EPI_SWIGLU_BWD ? 2 : 1);
  using L = Smem<STAGES, SLABS>;
  constexpr int UMMA_K = 16, KSTEPS = BK / UMMA_K;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BARRIER_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  uint32_t* poison_slot = tmem_base_slot + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cta_rank_in_cluster();          // 0 = leader
  const uint32_t peer = rank ^ 1u;
  const int cluster_id = blockIdx.x >> 1, nclusters = gridDim.x >> 1;
  const int bnh = p.bn >> 1;                             // rows of B per CTA

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 16); }
    *abort_flag = 0;
    // a status word that already holds an error turns the launch into a no-op; both CTAs must decide alike, so
    // each publishes what it read and both look at both after the cluster barrier
    *poison_slot = (status_poisoned(p.status) || (smem_u32(smem) & 1023) != 0) ? 1u : 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tmapA);
    tma_prefetch_desc(&tmapB);
    tma_prefetch_desc(&tmapD);
    if (EPI == EPI_SWIGLU) tma_prefetch_desc(&tmapD2);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_base_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  const bool poisoned = (*poison_slot | ld_cluster_u32(map_to_cta(smem_u32(poison_slot), peer))) != 0;
  if (poisoned && threadIdx.x == 0) {
    *abort_flag = 1;
    if ((smem_u32(smem) & 1023) != 0) report_error(p.status, GB_ERR_BAD_ARG, 4, 0);
  }
  __syncthreads();

  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int n_units = (EPI == EPI_SWIGLU) ? (p.N + 127) / 128 : (p.N + p.bn - 1) / p.bn;
  const long long total_tiles = (long long)tiles_m * n_units;
  auto decode = [&](long long t, int& mi, int& ni) {
    const int r = (int)t, g = p.raster_group;
    if (p.m_fastest) {
      const int grp = r / (g * n_units), rr = r % (g * n_units);
      const int gs = (tiles_m - grp * g) < g ? (tiles_m - grp * g) : g;
      mi = grp * g + rr % gs; ni = rr / gs;
    } else {
      const int grp = r / (g * tiles_m), rr = r % (g * tiles_m);
      const int gs = (n_units - grp * g) < g ? (n_units - grp * g) : g;
      ni = grp * g + rr % gs; mi = rr / gs;
    }
  };
  const uint32_t abort_peer = map_to_cta(smem_u32(const_cast<int*>(abort_flag)), peer);
  auto give_up = [&]() { st_cluster_u32(abort_peer, 1u); };

  if (warp == 0) {
    // =========================== TMA producer (one thread per CTA) ===========================
    if (elect_one()) {
      uint32_t it = 0;
      for (long long t = cluster_id; t < total_tiles && !*abort_flag; t += nclusters) {
        int mi, ni;
        decode(t, mi, ni);
        const int m0 = mi * 2 * BM + (int)rank * BM;
        // rows of B this CTA loads: its half of the tile, or (SwiGLU) the gate rows in CTA 0 and up rows in CTA 1
        const int nb0 = (EPI == EPI_SWIGLU) ? (int)rank * p.N + ni * 128 : ni * p.bn + (int)rank * bnh;
        bool ok = true;
        for (int k0 = 0; k0 < p.K; k0 += BK, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, 100)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t bar0 = map_to_cta(smem_u32(&full_bar[s]), 0);
          // the leader posts the bytes of both CTAs: 16 KB of A and bnh rows of B from each
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2u * (uint32_t)(A_BYTES + bnh * 128));
          if constexpr (!A_MN) {
            tma2_load_3d(sa, &tmapA, bar0, k0, m0, 0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma2_load_3d(sa + c * (BK * 128), &tmapA, bar0, m0 + c * 64, k0, 0);
          }
          if constexpr (!B_MN) {
            tma2_load_3d(sb, &tmapB, bar0, k0, nb0, 0);
          } else {
            for (int c = 0; c < bnh / 64; ++c) tma2_load_3d(sb + c * (BK * 128), &tmapB, bar0, nb0 + c * 64, k0, 0);
          }
        }
        if (!ok) { give_up(); break; }
      }
      if (*abort_flag && rank == 0) {
        // give loads in flight a bounded time to land before shared memory is given up
        for (int s = 0; s < STAGES; ++s) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full_bar[s], 0) && !mbar_try_wait(&full_bar[s], 1) &&
                 globaltimer_ns() - t0 < 1000000ull) {}
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =========================== MMA issuer: one thread of the leader CTA ===========================
    if (rank == 0 && lane == 0) {
      const uint32_t idesc = make_idesc(p.in_bf16 ? 1u : 0u, A_MN ? 1u : 0u, B_MN ? 1u : 0u, 2 * BM, p.bn);
      uint32_t it = 0, tile_no = 0;
      for (long long t = cluster_id; t < total_tiles && !*abort_flag; t += nclusters) {
        const uint32_t acc = tile_no & 1, acc_ph = (tile_no >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag, p.status, 200)) { give_up(); break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE;
        bool ok = true;
        for (int k0 = 0; k0 < p.K; k0 += BK, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, 201)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < KSTEPS; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc(a_addr + kk * UMMA_K * 128, BK * 128, 1024)
                                     : make_smem_desc(a_addr + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(b_addr + kk * UMMA_K * 128, BK * 128, 1024)
                                     : make_smem_desc(b_addr + kk * 32, 16, 1024);
            umma2_f16(d_tmem, da, db, idesc, (k0 == 0 && kk == 0) ? 0u : 1u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma2_commit(smem_u32(&empty_bar[s]));
          umma2_commit(map_to_cta(smem_u32(&empty_bar[s]), 1));
        }
        if (!ok) { give_up(); break; }
        umma2_commit(smem_u32(&tmem_full[acc]));
        umma2_commit(map_to_cta(smem_u32(&tmem_full[acc]), 1));
        ++tile_no;
      }
    }
    __syncwarp();
  } else {
    // =========================== epilogue warps (both CTAs, own accumulator rows) ===========================
    const int q = warp & 3;                        // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;              // which 64-column units of the tile this warp stores
    uint8_t* slab = smem + L::SLAB_OFFSET + (warp - 2) * SLABS * SLAB_BYTES;
    uint8_t* slab_row = slab + lane * 128;
    const uint32_t empty0 = map_to_cta(smem_u32(&tmem_empty[0]), 0);
    const int dt = p.out_dtype;
    // SwiGLU backward: gate (ng) and up (nu) of the next 32-column step of this lane's row, fetched one step ahead
    // with 32-byte read-only loads (two per 64-byte run, so every sector is requested once).  Rows past M and
    // columns past N keep whatever the registers held: their results are clipped by the TMA store.
    uint32_t ng[16], nu[16];
    auto gu_fetch = [&](int mi2, int ni2, int k) {
      const int row = mi2 * 2 * BM + (int)rank * BM + q * 32 + lane;
      const int col = ni2 * p.bn + half * 64 + (k >> 1) * 128 + (k & 1) * 32;
      if (row < p.M && col + 32 <= p.N) {
        const uint16_t* g = reinterpret_cast<const uint16_t*>(p.gu) + (size_t)row * p.ld_gu + col;
        ld_nc_v8(ng, g); ld_nc_v8(ng + 8, g + 16);
        ld_nc_v8(nu, g + p.N); ld_nc_v8(nu + 8, g + p.N + 16);
      }
    };
    if constexpr (EPI == EPI_SWIGLU_BWD) {
#pragma unroll
      for (int i = 0; i < 16; ++i) { ng[i] = 0u; nu[i] = 0u; }
      if (cluster_id < total_tiles) {
        int mi2, ni2;
        decode(cluster_id, mi2, ni2);
        gu_fetch(mi2, ni2, 0);
      }
    }
    uint32_t tile_no = 0;
    for (long long t = cluster_id; t < total_tiles && !*abort_flag; t += nclusters) {
      int mi, ni;
      decode(t, mi, ni);
      const int m0 = mi * 2 * BM + (int)rank * BM;
      const uint32_t acc = tile_no & 1, acc_ph = (tile_no >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[acc], acc_ph, abort_flag, p.status, 300))) {
        if (lane == 0) give_up();
        break;
      }
      tc_fence_after_sync();
      const int y0 = m0 + q * 32;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * ACC_STRIDE;
      if constexpr (EPI == EPI_SWIGLU) {
        // this warp: hidden units [64 half, 64 half + 64) of the tile; gate in columns c, up in columns 128 + c
        const int h0 = ni * 128 + half * 64;
        if (lane == 0) bulk_wait_group_read<0>();
        __syncwarp();
        auto run = [&](auto is_bf16) {
          constexpr bool BF = decltype(is_bf16)::value;
          // four steps of 16 hidden units; the accumulator columns of step s + 1 travel from tensor memory to
          // registers while step s is computed
          uint32_t ga[16], ua[16], gb_[16], ub[16];
          auto step = [&](const uint32_t (&rg)[16], const uint32_t (&ru)[16], int s) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              float g[8], v[8], h[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                g[j] = __uint_as_float(rg[8 * u + j]) * p.alpha;
                v[j] = __uint_as_float(ru[8 * u + j]) * p.alpha;
                h[j] = g[j] * rcp_approx(1.f + ex2_approx(g[j] * -1.4426950408889634f)) * v[j];
              }
              const int unit = ((2 * s + u) ^ (lane & 7)) << 4;
              uint4 o;
              o.x = pack2c<BF>(g[0], g[1]); o.y = pack2c<BF>(g[2], g[3]); o.z = pack2c<BF>(g[4], g[5]); o.w = pack2c<BF>(g[6], g[7]);
              *reinterpret_cast<uint4*>(slab_row + unit) = o;
              o.x = pack2c<BF>(v[0], v[1]); o.y = pack2c<BF>(v[2], v[3]); o.z = pack2c<BF>(v[4], v[5]); o.w = pack2c<BF>(v[6], v[7]);
              *reinterpret_cast<uint4*>(slab_row + SLAB_BYTES + unit) = o;
              o.x = pack2c<BF>(h[0], h[1]); o.y = pack2c<BF>(h[2], h[3]); o.z = pack2c<BF>(h[4], h[5]); o.w = pack2c<BF>(h[6], h[7]);
              *reinterpret_cast<uint4*>(slab_row + 2 * SLAB_BYTES + unit) = o;
            }
          };
          const uint32_t tg = t_row + half * 64, tu = t_row + 128 + half * 64;
          tmem_ld_32x32b_x16(tg, ga); tmem_ld_32x32b_x16(tu, ua);
          tmem_ld_wait(); reg_fence16(ga); reg_fence16(ua);
          tmem_ld_32x32b_x16(tg + 16, gb_); tmem_ld_32x32b_x16(tu + 16, ub);
          step(ga, ua, 0);
          tmem_ld_wait(); reg_fence16(gb_); reg_fence16(ub);
          tmem_ld_32x32b_x16(tg + 32, ga); tmem_ld_32x32b_x16(tu + 32, ua);
          step(gb_, ub, 1);
          tmem_ld_wait(); reg_fence16(ga); reg_fence16(ua);
          tmem_ld_32x32b_x16(tg + 48, gb_); tmem_ld_32x32b_x16(tu + 48, ub);
          step(ga, ua, 2);
          tmem_ld_wait(); reg_fence16(gb_); reg_fence16(ub);
          step(gb_, ub, 3);
        };
        if (dt == DT_BF16) run(std::true_type{});
        else run(std::false_type{});
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && y0 < p.M && h0 < p.N) {
          if (p.write_gu) {
            tma_store_3d(&tmapD, slab, h0, y0, 0);
            tma_store_3d(&tmapD, slab + SLAB_BYTES, p.N + h0, y0, 0);
          }
          tma_store_3d(&tmapD2, slab + 2 * SLAB_BYTES, h0, y0, 0);
          bulk_commit_group();
        }
      } else if constexpr (EPI == EPI_SWIGLU_BWD) {
        // accumulator = dh[rows, n0 .. n0 + 256); this warp takes the 64-column units half and half + 2 in four steps
        // of 32 columns.  gate | up of step k + 1 (of the next tile after the last step) is already on its way to
        // registers while step k is computed.  The element type is a compile-time constant inside `steps`: the
        // epilogue is bound by instruction issue (two warps per scheduler), so every select on the type counts.
        const int n0 = ni * p.bn;
        auto steps = [&](auto is_bf16) {
          constexpr bool BF = decltype(is_bf16)::value;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int c = half * 64 + (k >> 1) * 128, sub = k & 1;
            uint32_t cg[16], cu[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) { cg[i] = ng[i]; cu[i] = nu[i]; }
            if (k < 3) {
              gu_fetch(mi, ni, k + 1);
            } else if (t + nclusters < total_tiles) {
              int mi2, ni2;
              decode(t + nclusters, mi2, ni2);
              gu_fetch(mi2, ni2, 0);
            }
            if (n0 + c >= p.N) continue;                      // warp-uniform: a unit past the last hidden column
            if (sub == 0) {
              if (lane == 0) bulk_wait_group_read<0>();
              __syncwarp();
            }
            uint32_t rd[32];
            tmem_ld_32x32b_x32(t_row + c + sub * 32, rd);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float dg[8], du[8];
#pragma unroll
              for (int j = 0; j < 8; j += 2) {
                float x2[2], u2[2];
                unpack2<BF>(cg[4 * v + (j >> 1)], x2[0], x2[1]);
                unpack2<BF>(cu[4 * v + (j >> 1)], u2[0], u2[1]);
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  // s = sigmoid(x); d silu(x) u / dx = u s (1 + x (1 - s)); d silu(x) u / du = x s
                  const float x = x2[e];
                  const float s = rcp_approx(1.f + ex2_approx(x * -1.4426950408889634f));
                  const float a = __uint_as_float(rd[8 * v + j + e]) * p.alpha * s;
                  dg[j + e] = a * u2[e] * fmaf(x, 1.f - s, 1.f);
                  du[j + e] = a * x;
                }
              }
              const int unit = ((4 * sub + v) ^ (lane & 7)) << 4;
              uint4 o;
              o.x = pack2c<BF>(dg[0], dg[1]); o.y = pack2c<BF>(dg[2], dg[3]);
              o.z = pack2c<BF>(dg[4], dg[5]); o.w = pack2c<BF>(dg[6], dg[7]);
              *reinterpret_cast<uint4*>(slab_row + unit) = o;
              o.x = pack2c<BF>(du[0], du[1]); o.y = pack2c<BF>(du[2], du[3]);
              o.z = pack2c<BF>(du[4], du[5]); o.w = pack2c<BF>(du[6], du[7]);
              *reinterpret_cast<uint4*>(slab_row + SLAB_BYTES + unit) = o;
            }
            if (sub == 1) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0 && y0 < p.M) {
                tma_store_3d(&tmapD, slab, n0 + c, y0, 0);
                tma_store_3d(&tmapD, slab + SLAB_BYTES, p.N + n0 + c, y0, 0);
                bulk_commit_group();
              }
            }
          }
        };
        if (dt == DT_BF16) steps(std::true_type{});
        else steps(std::false_type{});
      } else {
        const int n0 = ni * p.bn;
        auto process = [&](uint32_t (&r)[2][32], int c) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int col0 = n0 + c + hh * 32;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[hh][j]) * p.alpha;
            if (p.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] += load_as_float(p.bias, p.bias_dtype, col0 + j);
            }
            if (dt == DT_F32) {
              if (lane == 0) bulk_wait_group_read<0>();
              __syncwarp();
#pragma unroll
              for (int u = 0; u < 8; ++u)
                *reinterpret_cast<float4*>(slab_row + ((u ^ (lane & 7)) << 4)) =
                    make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0 && y0 < p.M && col0 < p.N) {
                if (p.accumulate) tma_reduce_add_3d(&tmapD, slab, col0, y0, 0);
                else tma_store_3d(&tmapD, slab, col0, y0, 0);
                bulk_commit_group();
              }
            } else {
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
                  tma_store_3d(&tmapD, slab, n0 + c, y0, 0);
                  bulk_commit_group();
                }
              }
            }
          }
        };
        // this warp's 64-column units: half, and half + 2 when the tile is wider than 128 + 64 half; the second
        // unit's accumulator columns are on their way to registers while the first is converted and stored
        const int c0 = half * 64;
        const bool two = c0 + 128 < p.bn;
        uint32_t ra[2][32], rb[2][32];
        tmem_ld_32x32b_x32(t_row + c0, ra[0]);
        tmem_ld_32x32b_x32(t_row + c0 + 32, ra[1]);
        tmem_ld_wait();
        reg_fence32(ra[0]); reg_fence32(ra[1]);
        if (two) {
          tmem_ld_32x32b_x32(t_row + c0 + 128, rb[0]);
          tmem_ld_32x32b_x32(t_row + c0 + 160, rb[1]);
        }
        process(ra, c0);
        if (two) {
          tmem_ld_wait();
          reg_fence32(rb[0]); reg_fence32(rb[1]);
          process(rb, c0 + 128);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      // the accumulator may be overwritten once the 8 warps of both CTAs have read it
      if (lane == 0) mbar_arrive_cluster(empty0 + acc * 8);
      ++tile_no;
    }
    if (lane == 0) bulk_wait_group_read<0>();
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();            // nobody leaves (or frees tensor memory) while the peer may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

template <int STAGES, bool A_MN, bool B_MN, int EPI>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const CUtensorMap& td2,
                  const Params& p, cudaStream_t stream) {
  constexpr int SLABS = (EPI == EPI_SWIGLU) ? 3 : (EPI == EPI_SWIGLU_BWD ? 2 : 1);
  using L = Smem<STAGES, SLABS>;
  auto kern = gemm2_kernel<STAGES, A_MN, B_MN, EPI>;
  static unsigned long long configured = 0;
  static int max_clusters[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (int e = smem_opt_in(kern, L::TOTAL, configured)) return e;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(320); cfg.dynamicSmemBytes = L::TOTAL; cfg.stream = stream;
  cfg.attrs = attr; cfg.numAttrs = 1;
  if (max_clusters[dev & 63] == 0) {
    // how many CTA pairs the device can hold at once (pairs live inside one GPC): the persistent grid
    cfg.gridDim = dim3(2);
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess || n < 1) { cudaGetLastError(); return -7; }
    max_clusters[dev & 63] = n;
  }
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int n_units = (EPI == EPI_SWIGLU) ? (p.N + 127) / 128 : (p.N + p.bn - 1) / p.bn;
  long long total = (long long)tiles_m * n_units;
  long long clusters = total < max_clusters[dev & 63] ? total : max_clusters[dev & 63];
  if (clusters < 1) clusters = 1;
  cfg.gridDim = dim3((unsigned)(2 * clusters));
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, td, td2, p);
  return e == cudaSuccess ? (int)cudaGetLastError() : (int)e;
}

}  // namespace g2
}  // namespace gb

using namespace gb;

// C ABI of the pair kernel.  16-bit operands (in_dtype DT_F16 / DT_BF16), a_mn / b_mn / lda / ldb as in gb_gemm.
//   epi 0: D[M, N] = alpha * A B^T + bias, out_dtype f32 / f16 / bf16; accumulate (f32 only) adds into D.
//   epi 1: B is a stacked [2 N, K] K-major weight (gate rows, then up rows); D2[M, N] = silu(g) * u with
//          g | u = alpha * A B^T, and D[M, 2 N] = g | u when D is not null.  N must be a multiple of 128.
//   epi 2: dh = alpha * A B^T is the gradient of silu(g) * u; D2 [M, 2 N] holds g | u (input) and
//          D [M, 2 N] receives dg | du; dh itself is never stored.  N must be a multiple of 64.
// Requirements (the caller falls back to gb_gemm otherwise): D, D2 16-byte aligned with 16-byte multiples as pitch.
// bn: pair tile width 128 / 192 / 256 (0 = 256).  Returns 0, a cudaError_t, or a negative argument error.
extern "C" int gb_gemm_pair(const void* A, const void* B, void* D, void* D2, const void* bias, int M, int N, int K,
                            long long lda, long long ldb, int ldd, int ldd2, int a_mn, int b_mn, int in_dtype,
                            int out_dtype, int bias_dtype, int accumulate, float alpha, int epi, int bn,
                            int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (in_dtype != DT_F16 && in_dtype != DT_BF16) return -2;
  if (bn == 0) bn = 256;
  if (bn != 128 && bn != 192 && bn != 256) return -3;
  if (accumulate && out_dtype != DT_F32) return -4;
  g2::Params p;
  p.bias = bias; p.status = status; p.M = M; p.N = N; p.K = K; p.bn = bn; p.out_dtype = out_dtype;
  p.in_bf16 = in_dtype == DT_BF16 ? 1 : 0; p.bias_dtype = bias_dtype; p.accumulate = accumulate;
  p.alpha = alpha; p.write_gu = D != nullptr ? 1 : 0;
  p.gu = nullptr; p.ld_gu = 0;
  CUtensorMap ta, tb, td, td2;
  int r;
  if (epi == g2::EPI_SWIGLU_BWD) {
    // A = gy [M, K], B = the [N, K] K-major twin of the down weight; D2 = gate | up of the forward pass [M, 2 N]
    // (read), D = d(gate) | d(up) [M, 2 N] (written).  N = hidden width, a multiple of 64.
    if (a_mn || b_mn || N % 64 != 0 || out_dtype == DT_F32 || bias != nullptr || D == nullptr || D2 == nullptr)
      return -5;
    if ((reinterpret_cast<uintptr_t>(D2) & 31) != 0 || (ldd2 * 2) % 32 != 0) return -5;   // 32-byte loads of gate | up
    p.bn = 256;
    p.gu = D2; p.ld_gu = ldd2;
    if ((r = make_tmap_3d(&ta, A, in_dtype, K, M, 1, lda, 0, g2::BM)) != 0) return 10000 + r;
    if ((r = make_tmap_3d(&tb, B, in_dtype, K, N, 1, ldb, 0, 128)) != 0) return 20000 + r;
    if ((r = make_tmap_3d(&td, D, out_dtype, 2ll * N, M, 1, ldd, 0, 32)) != 0) return 30000 + r;
    td2 = td;
    p.m_fastest = 1;
    p.raster_group = (M + 255) / 256;
    return g2::launch<5, false, false, g2::EPI_SWIGLU_BWD>(ta, tb, td, td2, p, stream);
  }
  if (epi == g2::EPI_SWIGLU) {
    if (a_mn || b_mn || N % 128 != 0 || out_dtype == DT_F32 || bias != nullptr || D2 == nullptr) return -5;
    p.bn = 256;
    if ((r = make_tmap_3d(&ta, A, in_dtype, K, M, 1, lda, 0, g2::BM)) != 0) return 10000 + r;
    if ((r = make_tmap_3d(&tb, B, in_dtype, K, 2ll * N, 1, ldb, 0, 128)) != 0) return 20000 + r;
    if ((r = make_tmap_3d(&td2, D2, out_dtype, N, M, 1, ldd2, 0, 32)) != 0) return 40000 + r;
    if (D != nullptr) { if ((r = make_tmap_3d(&td, D, out_dtype, 2ll * N, M, 1, ldd, 0, 32)) != 0) return 30000 + r; }
    else td = td2;
    p.m_fastest = 1;
    p.raster_group = (M + 255) / 256;
    return g2::launch<4, false, false, g2::EPI_SWIGLU>(ta, tb, td, td2, p, stream);
  }
  const int bnh = bn / 2;
  if (b_mn && bnh % 64 != 0) return -6;
  if (!a_mn) r = make_tmap_3d(&ta, A, in_dtype, K, M, 1, lda, 0, g2::BM);
  else r = make_tmap_3d(&ta, A, in_dtype, M, K, 1, lda, 0, g2::BK);
  if (r != 0) return 10000 + r;
  if (!b_mn) r = make_tmap_3d(&tb, B, in_dtype, K, N, 1, ldb, 0, bnh);
  else r = make_tmap_3d(&tb, B, in_dtype, N, K, 1, ldb, 0, g2::BK);
  if (r != 0) return 20000 + r;
  if ((r = make_tmap_3d(&td, D, out_dtype, N, M, 1, ldd, 0, 32)) != 0) return 30000 + r;
  td2 = td;
  // sweep the dimension with the smaller operand fastest; whole sweeps when that operand sits in L2 comfortably
  p.m_fastest = ((long long)M <= (long long)N) ? 1 : 0;
  {
    const long long fast_bytes = (long long)(p.m_fastest ? M : N) * K * 2;
    const int fast_tiles = p.m_fastest ? (M + 255) / 256 : (N + bn - 1) / bn;
    p.raster_group = (fast_bytes <= (48ll << 20)) ? fast_tiles : 8;
    if (p.raster_group < 1) p.raster_group = 1;
  }
  if (!a_mn && !b_mn) return g2::launch<6, false, false, g2::EPI_PLAIN>(ta, tb, td, td2, p, stream);
  if (!a_mn && b_mn) return g2::launch<6, false, true, g2::EPI_PLAIN>(ta, tb, td, td2, p, stream);
  if (a_mn && !b_mn) return g2::launch<6, true, false, g2::EPI_PLAIN>(ta, tb, td, td2, p, stream);
  return g2::launch<6, true, true, g2::EPI_PLAIN>(ta, tb, td, td2, p, stream);
}
