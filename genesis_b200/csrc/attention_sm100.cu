// Flash attention for sm_100a on tcgen05 tensor cores: forward, dQ and dK/dV kernels.
//
// Layout: q [B, S, Hq, D], k/v [B, Sk, Hkv, D], o [B, S, Hq, D], lse [B, Hq, S] (natural log).
// Native GQA (Hkv divides Hq, K/V never replicated), optional causal mask (aligned to the end of
// the keys when Sk > S), any S / Sk, D in {64, 128}, bf16 / fp16.
//
// All three kernels share one scheme: 128 "row" threads own one row of a 128 x 128 score tile each
// (= one TMEM lane), so soft-max statistics never leave the thread; one TMA thread and one MMA thread
// feed the tensor cores.  Scores and accumulators live in tensor memory; probabilities go back to the
// tensor cores through a 128-byte-swizzled shared-memory tile written by the row threads.
//   forward : S = Q K^T (double-buffered in TMEM so the next QK^T overlaps the soft-max),
//             O += P V with O resident in TMEM, rescaled only when a row maximum moves
//   dQ      : per q tile, loop over kv tiles: S, dP = dO V^T, dS = P (dP - delta) scale, dQ += dS K
//   dK/dV   : per kv tile, loop over the query heads of the group and q tiles:
//             S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q   (no atomics, no K/V head copies)
// Operand tricks: V, dO and Q/K tiles are consumed by the second GEMMs as MN-major operands straight
// from the tile TMA wrote, so nothing is ever transposed in memory.
// Reference counterpart: Triton kernels of genesis/nn/attention.py:21-519 (32 x 32 tiles, Hq == Hkv only).
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
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int row, int c0, const float (&v)[32], int is_bf16,
                                                int chunk_stride) {
  uint8_t* base = tile + (c0 >> 6) * chunk_stride + row * 128;
  const int u0 = (c0 & 63) >> 3;
  const int dt = is_bf16 ? DT_BF16 : DT_F16;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 w;
    w.x = pack2(v[i * 8 + 0], v[i * 8 + 1], dt);
    w.y = pack2(v[i * 8 + 2], v[i * 8 + 3], dt);
    w.z = pack2(v[i * 8 + 4], v[i * 8 + 5], dt);
    w.w = pack2(v[i * 8 + 6], v[i * 8 + 7], dt);
    *reinterpret_cast<uint4*>(base + (((u0 + i) ^ (row & 7)) << 4)) = w;
  }
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

// =====================================================================================================
// forward
// =====================================================================================================
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// SB = number of score buffers in TMEM.  D = 64: one buffer, 256 TMEM columns and ~113 KB of shared
// memory, so two CTAs share an SM and cover each other's soft-max / MMA bubbles.  D = 128: two score
// buffers, 512 columns, one CTA per SM.
template <int D, int SB>
__global__ void __launch_bounds__(192, SB == 1 ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                const __grid_constant__ CUtensorMap tmv, const AttnParams p) {
  constexpr int TILE = AT_BM * D * 2;            // bytes of one [128 x D] 16-bit tile
  constexpr int PB = AT_BM * AT_BN * 2;
  constexpr uint32_t TCOLS = SB == 1 ? 256 : 512;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if (SB == 1 && (reinterpret_cast<uintptr_t>(smem_raw) & 1023) != 0) {
    // the two-CTA-per-SM configuration has no room for an alignment pad; refuse rather than overrun
    if (threadIdx.x == 0) report_error(p.status, GB_ERR_BAD_ARG, 1, 0);
    return;
  }
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE;          // 2 stages
  uint8_t* sV = sK + 2 * TILE;      // 2 stages
  uint8_t* sP = sV + 2 * TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + PB);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2]
  uint64_t* s_empty = bars + 11;      // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* pv_done = bars + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;     // longest (last) tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.Hq / p.Hkv);
  const int m0 = qt * AT_BM;
  const int off = p.Sk - p.S;
  int n_kv = (p.Sk + AT_BN - 1) / AT_BN;
  if (p.causal) {
    const int lim = (m0 + AT_BM + off + AT_BN - 1) / AT_BN;
    n_kv = lim < n_kv ? lim : n_kv;
  }
  if (n_kv < 1) n_kv = 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, TCOLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tO = tmem + SB * AT_BN;
  // score buffer and barrier phase of kv block j
  auto sbuf = [](int j) { return SB == 2 ? (j & 1) : 0; };
  auto sphase = [](int j) { return (uint32_t)(SB == 2 ? ((j >> 1) & 1) : (j & 1)); };

  if (warp == 4) {
    if (lane == 0) {   // ---------------- TMA ----------------
      tma_prefetch_desc(&tmq); tma_prefetch_desc(&tmk); tma_prefetch_desc(&tmv);
      mbar_expect_tx(q_full, TILE);
      load_tile<D>(sQ, &tmq, q_full, h, m0, b, AT_BM);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!AT_WAIT(&k_empty[s], ph ^ 1, 10)) break;
        mbar_expect_tx(&k_full[s], TILE);
        load_tile<D>(sK + s * TILE, &tmk, &k_full[s], kvh, j * AT_BN, b, AT_BN);
        if (!AT_WAIT(&v_empty[s], ph ^ 1, 11)) break;
        mbar_expect_tx(&v_full[s], TILE);
        load_tile<D>(sV + s * TILE, &tmv, &v_full[s], kvh, j * AT_BN, b, AT_BN);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {   // ---------------- MMA ----------------
      const uint32_t fmt = p.is_bf16 ? 1u : 0u;
      const uint32_t idesc_qk = make_idesc(fmt, 0, 0, AT_BM, AT_BN);
      const uint32_t idesc_pv = make_idesc(fmt, 0, 1, AT_BM, D);
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      bool ok = AT_WAIT(q_full, 0, 20);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!AT_WAIT(&k_full[s], ph, 21)) return false;
        if (!AT_WAIT(&s_empty[sbuf(j)], sphase(j) ^ 1, 22)) return false;
        tc_fence_after_sync();
        const uint32_t aK = smem_u32(sK + s * TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16(tmem + sbuf(j) * AT_BN, desc_kmajor(aQ, kk, AT_BM), desc_kmajor(aK, kk, AT_BN), idesc_qk, kk > 0);
        umma_commit(&k_empty[s]);
        umma_commit(&s_full[sbuf(j)]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; ok && j < n_kv; ++j) {
        if (j + 1 < n_kv && !issue_qk(j + 1)) break;
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!AT_WAIT(p_full, j & 1, 23)) break;
        if (!AT_WAIT(&v_full[s], ph, 24)) break;
        tc_fence_after_sync();
        const uint32_t aV = smem_u32(sV + s * TILE);
#pragma unroll
        for (int kk = 0; kk < AT_BN / 16; ++kk)
          umma_f16(tO, desc_kmajor(aP, kk, AT_BM), desc_mnmajor(aV, kk, AT_BN), idesc_pv, (j > 0 || kk > 0));
        umma_commit(&v_empty[s]);
        umma_commit(pv_done);
      }
    }
  } else {
    // ---------------- soft-max rows ----------------
    const int t = threadIdx.x;
    const int row = m0 + t;
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    const float sl2 = p.scale * LOG2E;
    float m = -INFINITY, l = 0.f;     // running max (scaled, log2 domain) and sum
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int sb = sbuf(j);
      if (!__all_sync(0xffffffffu, AT_WAIT(&s_full[sb], sphase(j), 30))) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t tS = tmem + lane_base + sb * AT_BN;
      // the whole score row goes to registers in one go, then the TMEM buffer is handed back
      uint32_t r[4][32];
      tmem_ld_32x32b_x32(tS, r[0]);
      tmem_ld_32x32b_x32(tS + 32, r[1]);
      tmem_ld_32x32b_x32(tS + 64, r[2]);
      tmem_ld_32x32b_x32(tS + 96, r[3]);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&s_empty[sb]);
      const int col0 = j * AT_BN;
      const bool need_mask = (col0 + AT_BN > p.Sk) || (p.causal && (col0 + AT_BN - 1 > m0 + off));
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = col0 + c * 32 + i;
            if (col >= p.Sk || (p.causal && col > row + off)) r[c][i] = 0xff800000u;   // -inf
          }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[c][i]));
      const float m_new = fmaxf(m, mx * sl2);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2(m - m_safe);
      if (j > 0) {
        if (!__all_sync(0xffffffffu, AT_WAIT(pv_done, (j - 1) & 1, 31))) { ok = false; break; }
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(tO + lane_base + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32b_x32(tO + lane_base + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      float rowsum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          pv[i] = fast_exp2(fmaf(__uint_as_float(r[c][i]), sl2, -m_safe));
          rowsum += pv[i];
        }
        store_row_chunk(sP, t, c * 32, pv, p.is_bf16, AT_BM * 128);
      }
      l = l * alpha + rowsum;
      m = m_new;
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(p_full);
    }
    if (ok && __all_sync(0xffffffffu, AT_WAIT(pv_done, (n_kv - 1) & 1, 32))) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int dt = p.is_bf16 ? DT_BF16 : DT_F16;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + (((size_t)b * p.S + row) * p.Hq + h) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tO + lane_base + c * 32, o);
        tmem_ld_wait();
        if (row < p.S) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv, dt);
            w.y = pack2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv, dt);
            w.z = pack2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv, dt);
            w.w = pack2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv, dt);
            *reinterpret_cast<uint4*>(orow + c * 32 + i) = w;
          }
        }
      }
      if (row < p.S) p.lse[((size_t)b * p.Hq + h) * p.S + row] = (l > 0.f) ? (m + log2f(l)) * LN2 : -INFINITY;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) { tc_fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}
// =====================================================================================================
// backward: dQ
// =====================================================================================================
template <int D>
__global__ void __launch_bounds__(160, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                   const __grid_constant__ CUtensorMap tmv, const __grid_constant__ CUtensorMap tmdo,
                   const AttnParams p) {
  constexpr int TILE = AT_BM * D * 2;
  constexpr int PB = AT_BM * AT_BN * 2;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + TILE;
  uint8_t* sK = sdO + TILE;
  uint8_t* sV = sK + TILE;
  uint8_t* sdS = sV + TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + PB);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* sdp_full = bars + 2;
  uint64_t* ds_ready = bars + 3;
  uint64_t* acc_done = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.Hq / p.Hkv);
  const int m0 = qt * AT_BM;
  const int off = p.Sk - p.S;
  int n_kv = (p.Sk + AT_BN - 1) / AT_BN;
  if (p.causal) {
    const int lim = (m0 + AT_BM + off + AT_BN - 1) / AT_BN;
    n_kv = lim < n_kv ? lim : n_kv;
  }
  if (n_kv < 1) n_kv = 1;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1); mbar_init(kv_full, 1); mbar_init(sdp_full, 1); mbar_init(ds_ready, 128);
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + AT_BN, tdQ = tmem + 2 * AT_BN;

  if (warp == 4) {
    if (lane == 0) {   // ---------------- TMA + MMA ----------------
      const uint32_t fmt = p.is_bf16 ? 1u : 0u;
      const uint32_t idesc_s = make_idesc(fmt, 0, 0, AT_BM, AT_BN);
      const uint32_t idesc_dq = make_idesc(fmt, 0, 1, AT_BM, D);
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO), aK = smem_u32(sK), aV = smem_u32(sV), adS = smem_u32(sdS);
      mbar_expect_tx(qdo_full, 2 * TILE);
      load_tile<D>(sQ, &tmq, qdo_full, h, m0, b, AT_BM);
      load_tile<D>(sdO, &tmdo, qdo_full, h, m0, b, AT_BM);
      for (int j = 0; j < n_kv; ++j) {
        if (j > 0 && !AT_WAIT(acc_done, (j - 1) & 1, 40)) break;
        mbar_expect_tx(kv_full, 2 * TILE);
        load_tile<D>(sK, &tmk, kv_full, kvh, j * AT_BN, b, AT_BN);
        load_tile<D>(sV, &tmv, kv_full, kvh, j * AT_BN, b, AT_BN);
        if (j == 0 && !AT_WAIT(qdo_full, 0, 41)) break;
        if (!AT_WAIT(kv_full, j & 1, 42)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          umma_f16(tS, desc_kmajor(aQ, kk, AT_BM), desc_kmajor(aK, kk, AT_BN), idesc_s, kk > 0);
          umma_f16(tdP, desc_kmajor(adO, kk, AT_BM), desc_kmajor(aV, kk, AT_BN), idesc_s, kk > 0);
        }
        umma_commit(sdp_full);
        if (!AT_WAIT(ds_ready, j & 1, 43)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < AT_BN / 16; ++kk)
          umma_f16(tdQ, desc_kmajor(adS, kk, AT_BM), desc_mnmajor(aK, kk, AT_BN), idesc_dq, (j > 0 || kk > 0));
        umma_commit(acc_done);
      }
    }
  } else {
    const int t = threadIdx.x;
    const int row = m0 + t;
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    const float sl2 = p.scale * LOG2E;
    const size_t stat = ((size_t)b * p.Hq + h) * p.S + row;
    const float lse2 = row < p.S ? p.lse_in[stat] * LOG2E : 0.f;
    const float dl = row < p.S ? p.delta[stat] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!__all_sync(0xffffffffu, AT_WAIT(sdp_full, j & 1, 50))) { ok = false; break; }
      tc_fence_after_sync();
      if (j > 0 && !__all_sync(0xffffffffu, AT_WAIT(acc_done, (j - 1) & 1, 51))) { ok = false; break; }
      const int col0 = j * AT_BN;
#pragma unroll 1
      for (int c = 0; c < AT_BN / 32; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld_32x32b_x32(tS + lane_base + c * 32, rs);
        tmem_ld_32x32b_x32(tdP + lane_base + c * 32, rp);
        tmem_ld_wait();
        float ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int col = col0 + c * 32 + i;
          const bool valid = row < p.S && col < p.Sk && (!p.causal || col <= row + off);
          const float pr = valid ? fast_exp2(fmaf(__uint_as_float(rs[i]), sl2, -lse2)) : 0.f;
          ds[i] = pr * (__uint_as_float(rp[i]) - dl) * p.scale;
        }
        store_row_chunk(sdS, t, c * 32, ds, p.is_bf16, AT_BM * 128);
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(ds_ready);
    }
    if (ok && __all_sync(0xffffffffu, AT_WAIT(acc_done, (n_kv - 1) & 1, 52))) {
      tc_fence_after_sync();
      const int dt = p.is_bf16 ? DT_BF16 : DT_F16;
      uint16_t* drow = reinterpret_cast<uint16_t*>(p.dq) + (((size_t)b * p.S + row) * p.Hq + h) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tdQ + lane_base + c * 32, r);
        tmem_ld_wait();
        if (row < p.S) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack2(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), dt);
            w.y = pack2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]), dt);
            w.z = pack2(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]), dt);
            w.w = pack2(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]), dt);
            *reinterpret_cast<uint4*>(drow + c * 32 + i) = w;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) { tc_fence_after_sync(); tmem_dealloc(tmem, 512); }
}

// =====================================================================================================
// backward: dK, dV
// =====================================================================================================
template <int D>
__global__ void __launch_bounds__(160, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                     const __grid_constant__ CUtensorMap tmv, const __grid_constant__ CUtensorMap tmdo,
                     const AttnParams p) {
  constexpr int TILE = AT_BM * D * 2;
  constexpr int PB = AT_BM * AT_BN * 2;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE;
  uint8_t* sQ = sV + TILE;
  uint8_t* sdO = sQ + TILE;
  uint8_t* sPT = sdO + TILE;
  uint8_t* sdST = sPT + PB;
  float* s_lse = reinterpret_cast<float*>(sdST + PB);   // [2][128]
  float* s_dl = s_lse + 2 * AT_BM;                      // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_dl + 2 * AT_BM);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* sdp_full = bars + 2;
  uint64_t* ds_ready = bars + 3;
  uint64_t* acc_done = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = blockIdx.x;
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int n0 = nt * AT_BN;
  const int off = p.Sk - p.S;
  const int nq = (p.S + AT_BM - 1) / AT_BM;
  int i_start = 0;
  if (p.causal) { i_start = (n0 - off) / AT_BM; if (i_start < 0) i_start = 0; }
  const int per_head = nq - i_start;
  const int n_it = per_head > 0 ? per_head * G : 0;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(qdo_full, 1); mbar_init(sdp_full, 1); mbar_init(ds_ready, 128);
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tST = tmem, tdPT = tmem + AT_BM, tdV = tmem + 2 * AT_BM, tdK = tmem + 2 * AT_BM + D;

  if (warp == 4) {
    if (lane == 0 && n_it > 0) {   // ---------------- TMA + MMA ----------------
      const uint32_t fmt = p.is_bf16 ? 1u : 0u;
      const uint32_t idesc_s = make_idesc(fmt, 0, 0, AT_BN, AT_BM);
      const uint32_t idesc_acc = make_idesc(fmt, 0, 1, AT_BN, D);
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO), aK = smem_u32(sK), aV = smem_u32(sV);
      const uint32_t aPT = smem_u32(sPT), adST = smem_u32(sdST);
      mbar_expect_tx(kv_full, 2 * TILE);
      load_tile<D>(sK, &tmk, kv_full, kvh, n0, b, AT_BN);
      load_tile<D>(sV, &tmv, kv_full, kvh, n0, b, AT_BN);
      for (int it = 0; it < n_it; ++it) {
        const int h = kvh * G + it / per_head;
        const int qi = i_start + it % per_head;
        if (it > 0 && !AT_WAIT(acc_done, (it - 1) & 1, 60)) break;
        mbar_expect_tx(qdo_full, 2 * TILE);
        load_tile<D>(sQ, &tmq, qdo_full, h, qi * AT_BM, b, AT_BM);
        load_tile<D>(sdO, &tmdo, qdo_full, h, qi * AT_BM, b, AT_BM);
        if (it == 0 && !AT_WAIT(kv_full, 0, 61)) break;
        if (!AT_WAIT(qdo_full, it & 1, 62)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          umma_f16(tST, desc_kmajor(aK, kk, AT_BN), desc_kmajor(aQ, kk, AT_BM), idesc_s, kk > 0);
          umma_f16(tdPT, desc_kmajor(aV, kk, AT_BN), desc_kmajor(adO, kk, AT_BM), idesc_s, kk > 0);
        }
        umma_commit(sdp_full);
        if (!AT_WAIT(ds_ready, it & 1, 63)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < AT_BM / 16; ++kk) {
          umma_f16(tdV, desc_kmajor(aPT, kk, AT_BN), desc_mnmajor(adO, kk, AT_BM), idesc_acc, (it > 0 || kk > 0));
          umma_f16(tdK, desc_kmajor(adST, kk, AT_BN), desc_mnmajor(aQ, kk, AT_BM), idesc_acc, (it > 0 || kk > 0));
        }
        umma_commit(acc_done);
      }
    }
  } else {
    const int t = threadIdx.x;
    const int kvrow = n0 + t;
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    const float sl2 = p.scale * LOG2E;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int h = kvh * G + it / per_head;
      const int qi = i_start + it % per_head;
      const int q0 = qi * AT_BM;
      float* lse_s = s_lse + (it & 1) * AT_BM;
      float* dl_s = s_dl + (it & 1) * AT_BM;
      {
        const int qr = q0 + t;
        const size_t stat = ((size_t)b * p.Hq + h) * p.S + qr;
        lse_s[t] = qr < p.S ? p.lse_in[stat] * LOG2E : INFINITY;
        dl_s[t] = qr < p.S ? p.delta[stat] : 0.f;
      }
      named_barrier(1, 128);
      if (!__all_sync(0xffffffffu, AT_WAIT(sdp_full, it & 1, 70))) { ok = false; break; }
      tc_fence_after_sync();
      if (it > 0 && !__all_sync(0xffffffffu, AT_WAIT(acc_done, (it - 1) & 1, 71))) { ok = false; break; }
#pragma unroll 1
      for (int c = 0; c < AT_BM / 32; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld_32x32b_x32(tST + lane_base + c * 32, rs);
        tmem_ld_32x32b_x32(tdPT + lane_base + c * 32, rp);
        tmem_ld_wait();
        float pt[32], dst[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int qcol = q0 + c * 32 + i;
          const bool valid = kvrow < p.Sk && qcol < p.S && (!p.causal || kvrow <= qcol + off);
          const float pr = valid ? fast_exp2(fmaf(__uint_as_float(rs[i]), sl2, -lse_s[c * 32 + i])) : 0.f;
          pt[i] = pr;
          dst[i] = pr * (__uint_as_float(rp[i]) - dl_s[c * 32 + i]) * p.scale;
        }
        store_row_chunk(sPT, t, c * 32, pt, p.is_bf16, AT_BN * 128);
        store_row_chunk(sdST, t, c * 32, dst, p.is_bf16, AT_BN * 128);
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(ds_ready);
    }
    const int dt = p.is_bf16 ? DT_BF16 : DT_F16;
    const size_t orow = (((size_t)b * p.Sk + kvrow) * p.Hkv + kvh) * D;
    if (n_it == 0) {
      if (kvrow < p.Sk)
        for (int c = 0; c < D; ++c) {
          reinterpret_cast<uint16_t*>(p.dk)[orow + c] = 0;
          reinterpret_cast<uint16_t*>(p.dv)[orow + c] = 0;
        }
    } else if (ok && __all_sync(0xffffffffu, AT_WAIT(acc_done, (n_it - 1) & 1, 72))) {
      tc_fence_after_sync();
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        uint16_t* out = reinterpret_cast<uint16_t*>(which == 0 ? p.dv : p.dk) + orow;
        const uint32_t tsrc = (which == 0 ? tdV : tdK) + lane_base;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tsrc + c * 32, r);
          tmem_ld_wait();
          if (kvrow < p.Sk) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 w;
              w.x = pack2(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), dt);
              w.y = pack2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]), dt);
              w.z = pack2(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]), dt);
              w.w = pack2(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]), dt);
              *reinterpret_cast<uint4*>(out + c * 32 + i) = w;
            }
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) { tc_fence_after_sync(); tmem_dealloc(tmem, 512); }
}

// delta[b, h, s] = sum_d dO * O ; one warp per row
template <typename T>
__global__ void attn_delta_kernel(const T* __restrict__ o, const T* __restrict__ dout, float* __restrict__ delta,
                                  int B, int S, int H, int D) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long rows = (long long)B * S * H;
  for (long long r = warp; r < rows; r += nwarps) {
    const int h = (int)(r % H);
    const long long bs = r / H;
    const int s = (int)(bs % S);
    const int b = (int)(bs / S);
    float acc = 0.f;
    for (int d = lane; d < D; d += 32) acc += Cvt<T>::to_f(o[r * D + d]) * Cvt<T>::to_f(dout[r * D + d]);
    acc = warp_sum(acc);
    if (lane == 0) delta[((long long)b * H + h) * S + s] = acc;
  }
}

// ------------------------------------------------------------------------------------------------
// host
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn4)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn4 encode4() {
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
static int make_tmap_bshd(CUtensorMap* out, const void* base, int is_bf16, int B, int S, int H, int D) {
  EncodeTiledFn4 enc = encode4();
  if (enc == nullptr) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)H * D * 2, (cuuint64_t)S * H * D * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  return (int)enc(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

template <typename KernT>
static int set_smem(KernT kern, int bytes) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

}  // namespace gb

using namespace gb;

extern "C" int gb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Sk,
                           int Hq, int Hkv, int D, int causal, float scale, int is_bf16, int* status,
                           cudaStream_t st) {
  if (D != 64 && D != 128) return -2;
  if (Hq % Hkv != 0 || Sk < S) return -3;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_tmap_bshd(&tq, q, is_bf16, B, S, Hq, D)) != 0) return 10000 + r;
  if ((r = make_tmap_bshd(&tk, k, is_bf16, B, Sk, Hkv, D)) != 0) return 20000 + r;
  if ((r = make_tmap_bshd(&tv, v, is_bf16, B, Sk, Hkv, D)) != 0) return 30000 + r;
  AttnParams p{};
  p.o = o; p.lse = lse; p.status = status; p.B = B; p.S = S; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
  p.causal = causal; p.is_bf16 = is_bf16; p.scale = scale;
  dim3 grid((S + AT_BM - 1) / AT_BM, Hq, B);
  // D = 64 runs two CTAs per SM: 2 x (114,944 + 1 KB reserved) just fits, an alignment pad would not
  const int smem = 5 * AT_BM * D * 2 + AT_BM * AT_BN * 2 + 256 + (D == 64 ? 0 : 1024);
  if (D == 64) {
    static bool cfg = false;
    if (!cfg) { if ((r = set_smem(attn_fwd_kernel<64, 1>, smem)) != 0) return r; cfg = true; }
    attn_fwd_kernel<64, 1><<<grid, 192, smem, st>>>(tq, tk, tv, p);
  } else {
    static bool cfg = false;
    if (!cfg) { if ((r = set_smem(attn_fwd_kernel<128, 2>, smem)) != 0) return r; cfg = true; }
    attn_fwd_kernel<128, 2><<<grid, 192, smem, st>>>(tq, tk, tv, p);
  }
  return (int)cudaGetLastError();
}

extern "C" int gb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                           const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S, int Sk,
                           int Hq, int Hkv, int D, int causal, float scale, int is_bf16, int* status,
                           cudaStream_t st) {
  if (D != 64 && D != 128) return -2;
  if (Hq % Hkv != 0 || Sk < S) return -3;
  CUtensorMap tq, tk, tv, tdo;
  int r;
  if ((r = make_tmap_bshd(&tq, q, is_bf16, B, S, Hq, D)) != 0) return 10000 + r;
  if ((r = make_tmap_bshd(&tk, k, is_bf16, B, Sk, Hkv, D)) != 0) return 20000 + r;
  if ((r = make_tmap_bshd(&tv, v, is_bf16, B, Sk, Hkv, D)) != 0) return 30000 + r;
  if ((r = make_tmap_bshd(&tdo, dout, is_bf16, B, S, Hq, D)) != 0) return 40000 + r;
  const long long rows = (long long)B * S * Hq;
  if (is_bf16) attn_delta_kernel<__nv_bfloat16><<<gb_grid(rows * 32, 256), 256, 0, st>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, S, Hq, D);
  else attn_delta_kernel<__half><<<gb_grid(rows * 32, 256), 256, 0, st>>>((const __half*)o, (const __half*)dout,
                                                                            delta, B, S, Hq, D);
  AttnParams p{};
  p.lse_in = lse; p.delta = delta; p.dq = dq; p.dk = dk; p.dv = dv; p.status = status;
  p.B = B; p.S = S; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.is_bf16 = is_bf16; p.scale = scale;
  const int smem_dq = 4 * AT_BM * D * 2 + AT_BM * AT_BN * 2 + 256 + 1024;
  const int smem_kv = 4 * AT_BM * D * 2 + 2 * AT_BM * AT_BN * 2 + 4 * AT_BM * 4 + 256 + 1024;
  dim3 gq((S + AT_BM - 1) / AT_BM, Hq, B), gk((Sk + AT_BN - 1) / AT_BN, Hkv, B);
  if (D == 64) {
    static bool cfg = false;
    if (!cfg) {
      if ((r = set_smem(attn_bwd_dq_kernel<64>, smem_dq)) != 0) return r;
      if ((r = set_smem(attn_bwd_dkdv_kernel<64>, smem_kv)) != 0) return r;
      cfg = true;
    }
    attn_bwd_dq_kernel<64><<<gq, 160, smem_dq, st>>>(tq, tk, tv, tdo, p);
    attn_bwd_dkdv_kernel<64><<<gk, 160, smem_kv, st>>>(tq, tk, tv, tdo, p);
  } else {
    static bool cfg = false;
    if (!cfg) {
      if ((r = set_smem(attn_bwd_dq_kernel<128>, smem_dq)) != 0) return r;
      if ((r = set_smem(attn_bwd_dkdv_kernel<128>, smem_kv)) != 0) return r;
      cfg = true;
    }
    attn_bwd_dq_kernel<128><<<gq, 160, smem_dq, st>>>(tq, tk, tv, tdo, p);
    attn_bwd_dkdv_kernel<128><<<gk, 160, smem_kv, st>>>(tq, tk, tv, tdo, p);
  }
  return (int)cudaGetLastError();
}
