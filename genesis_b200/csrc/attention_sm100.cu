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
#include "attention_common.cuh"

namespace gb {

// =====================================================================================================
// forward
// =====================================================================================================
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
  if (status_poisoned(p.status)) return;
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
    static unsigned long long cfg = 0;
    if ((r = smem_opt_in(attn_fwd_kernel<64, 1>, smem, cfg)) != 0) return r;
    attn_fwd_kernel<64, 1><<<grid, 192, smem, st>>>(tq, tk, tv, p);
  } else {
    static unsigned long long cfg = 0;
    if ((r = smem_opt_in(attn_fwd_kernel<128, 2>, smem, cfg)) != 0) return r;
    attn_fwd_kernel<128, 2><<<grid, 192, smem, st>>>(tq, tk, tv, p);
  }
  return (int)cudaGetLastError();
}

