// Flash-attention backward for sm_100a (tcgen05 / TMEM / TMA): dQ kernel, dK/dV kernel, delta pre-pass.
//
// Both kernels work on 128 x 64 score tiles: 128 row threads (one TMEM lane each) by 64 columns, which
// keeps S and dP (64 + 64 fp32 registers per thread) in registers after ONE tensor-memory round trip, so
// the TMEM tile is handed back at once and the next tile's QK^T / dO V^T run while the current tile's
// exponentials are computed.  Operand tiles arrive through a TMA ring (three stages in dQ, two in dK/dV).
//   dQ    : CTA = (q tile of 128 rows, head); loop over kv tiles of 64:
//           S = Q K^T, dP = dO V^T, dS = P o (dP - delta) * scale, dQ += dS K          (K tile reused MN-major)
//   dK/dV : CTA = (kv tile of 128 rows, query head); loop over q tiles of 64:
//           S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q                     (dO, Q tiles reused MN-major)
// With D = 64 a CTA needs 256 TMEM columns and at most 100.1 KB of shared memory: two CTAs share an SM.
// Reference counterpart: genesis/nn/attention.py:162-406 (Triton, 32 x 32 tiles, Hq == Hkv only).
#include "attention_common.cuh"

namespace gb {

constexpr int BW_C = 64;    // columns of a backward score tile
constexpr int BW_ST = 3;    // stages of the ring of streamed operand tiles in the dQ kernel
constexpr int KV_ST = 2;    // ... and in the dK/dV kernel, which spends the shared memory on per-warp statistics instead

__device__ __forceinline__ void store_out_row(uint16_t* dst, uint32_t tsrc, int ncols, bool valid, int dt,
                                              float mul = 1.f) {
#pragma unroll 1
  for (int c = 0; c < ncols; c += 32) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(tsrc + c, r);
    tmem_ld_wait();
    if (valid) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 w;
        w.x = pack2(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul, dt);
        w.y = pack2(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul, dt);
        w.z = pack2(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul, dt);
        w.w = pack2(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul, dt);
        *reinterpret_cast<uint4*>(dst + c + i) = w;
      }
    }
  }
}

// =====================================================================================================
// dQ
// =====================================================================================================
template <int D, int NCTA>
__global__ void __maxnreg__(NCTA == 2 ? 168 : 255)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                   const __grid_constant__ CUtensorMap tmv, const __grid_constant__ CUtensorMap tmdo,
                   const AttnParams p) {
  constexpr int QT = AT_BM * D * 2;          // [128 x D] tile
  constexpr int KT = BW_C * D * 2;           // [64 x D] tile
  constexpr uint32_t TCOLS = (D == 64) ? 256 : 512;   // 64 (S) + 64 (dP) + D (dQ) + 32 (dS as 16-bit pairs)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if (status_poisoned(p.status)) return;
  if ((reinterpret_cast<uintptr_t>(smem_raw) & 1023) != 0) {
    if (threadIdx.x == 0) report_error(p.status, GB_ERR_BAD_ARG, 2, 0);
    return;
  }
  uint8_t* sQ = smem_raw;
  uint8_t* sdO = sQ + QT;
  uint8_t* sK = sdO + QT;            // BW_ST stages
  uint8_t* sV = sK + BW_ST * KT;     // BW_ST stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + BW_ST * KT);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;      // [BW_ST]
  uint64_t* sdp_full = bars + 4;
  uint64_t* sdp_free = bars + 5;
  uint64_t* ds_ready = bars + 6;
  uint64_t* acc_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.Hq / p.Hkv);
  const int m0 = qt * AT_BM;
  const int off = p.Sk - p.S;
  int n_kv = (p.Sk + BW_C - 1) / BW_C;
  if (p.causal) {
    const int lim = (m0 + AT_BM + off + BW_C - 1) / BW_C;
    n_kv = lim < n_kv ? lim : n_kv;
  }
  if (n_kv < 1) n_kv = 1;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1); mbar_init(sdp_full, 1);
    for (int i = 0; i < BW_ST; ++i) mbar_init(&kv_full[i], 1);
    mbar_init(sdp_free, 128); mbar_init(ds_ready, 128); mbar_init(acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, TCOLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + BW_C, tdQ = tmem + 2 * BW_C, tdS = tmem + 2 * BW_C + D;

  if (warp == 4) {
    if (lane == 0) {   // ---------------- TMA + MMA ----------------
      const uint32_t fmt = p.is_bf16 ? 1u : 0u;
      const uint32_t idesc_s = make_idesc(fmt, 0, 0, AT_BM, BW_C);
      const uint32_t idesc_dq = make_idesc(fmt, 0, 1, AT_BM, D);
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO);
      auto load_kv = [&](int j) {
        const int st = j % BW_ST;
        mbar_expect_tx(&kv_full[st], 2 * KT);
        load_tile<D>(sK + st * KT, &tmk, &kv_full[st], kvh, j * BW_C, b, BW_C);
        load_tile<D>(sV + st * KT, &tmv, &kv_full[st], kvh, j * BW_C, b, BW_C);
      };
      auto issue_s = [&](int j) -> bool {
        const int st = j % BW_ST;
        if (!AT_WAIT(&kv_full[st], (j / BW_ST) & 1, 42)) return false;
        if (j > 0 && !AT_WAIT(sdp_free, (j - 1) & 1, 44)) return false;
        tc_fence_after_sync();
        const uint32_t aK = smem_u32(sK + st * KT), aV = smem_u32(sV + st * KT);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          umma_f16(tS, desc_kmajor(aQ, kk, AT_BM), desc_kmajor(aK, kk, BW_C), idesc_s, kk > 0);
          umma_f16(tdP, desc_kmajor(adO, kk, AT_BM), desc_kmajor(aV, kk, BW_C), idesc_s, kk > 0);
        }
        umma_commit(sdp_full);
        return true;
      };
      mbar_expect_tx(qdo_full, 2 * QT);
      load_tile<D>(sQ, &tmq, qdo_full, h, m0, b, AT_BM);
      load_tile<D>(sdO, &tmdo, qdo_full, h, m0, b, AT_BM);
      for (int j = 0; j < BW_ST && j < n_kv; ++j) load_kv(j);
      bool ok = AT_WAIT(qdo_full, 0, 41) && issue_s(0);
      for (int j = 0; ok && j < n_kv; ++j) {
        if (j + 1 < n_kv && !issue_s(j + 1)) break;
        if (!AT_WAIT(ds_ready, j & 1, 43)) break;
        tc_fence_after_sync();
        const uint32_t aK = smem_u32(sK + (j % BW_ST) * KT);
#pragma unroll
        for (int kk = 0; kk < BW_C / 16; ++kk)
          umma_f16_ts(tdQ, tdS + kk * 8, desc_mnmajor(aK, kk, BW_C), idesc_dq, (j > 0 || kk > 0));
        umma_commit(acc_done);
        // tile j - 1 is retired (the row threads waited for it before they signalled ds_ready(j)): refill
        // its stage with tile j - 1 + BW_ST, a full iteration before anything needs it
        // (no wait on acc_done here: its phase j - 1 is known complete, and a parity wait issued after the
        // commit above could alias phase j + 1)
        if (j >= 1 && j - 1 + BW_ST < n_kv) load_kv(j - 1 + BW_ST);
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
      uint32_t rs[2][32], rp[2][32];
      tmem_ld_32x32b_x32(tS + lane_base, rs[0]);
      tmem_ld_32x32b_x32(tS + lane_base + 32, rs[1]);
      tmem_ld_32x32b_x32(tdP + lane_base, rp[0]);
      tmem_ld_32x32b_x32(tdP + lane_base + 32, rp[1]);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(sdp_free);
      const int col0 = j * BW_C;
      const bool need_mask = (col0 + BW_C > p.Sk) || (p.causal && (col0 + BW_C - 1 > m0 + off)) || (m0 + AT_BM > p.S);
      if (need_mask) {
        // masked scores become -inf (probability 0) in a pass of their own: the main loop stays branch-free
        int lim = p.causal ? row + off : p.Sk - 1;            // last visible column of this row
        lim = lim < p.Sk - 1 ? lim : p.Sk - 1;
        if (row >= p.S) lim = -1;
        lim -= col0;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) rs[c][i] = (c * 32 + i <= lim) ? rs[c][i] : 0xff800000u;
      }
      // dS = P o (dP - delta) as 16-bit pairs (the softmax scale is applied once, to dQ at the end)
      uint32_t dsp[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(rs[c][i]), sl2, -lse2));
          const float p1 = fast_exp2(fmaf(__uint_as_float(rs[c][i + 1]), sl2, -lse2));
          const float d0 = p0 * (__uint_as_float(rp[c][i]) - dl);
          const float d1 = p1 * (__uint_as_float(rp[c][i + 1]) - dl);
          dsp[c * 16 + i / 2] = p.is_bf16 ? pack2c<true>(d0, d1) : pack2c<false>(d0, d1);
        }
      }
      // dS lives in tensor memory (A operand of the dQ MMA), single-buffered: the previous iteration's MMA has
      // to be done reading it
      if (j > 0 && !__all_sync(0xffffffffu, AT_WAIT(acc_done, (j - 1) & 1, 51))) { ok = false; break; }
      tc_fence_after_sync();
      tmem_st_32x32b_x32(tdS + lane_base, dsp);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(ds_ready);
    }
    if (ok && __all_sync(0xffffffffu, AT_WAIT(acc_done, (n_kv - 1) & 1, 52))) {
      tc_fence_after_sync();
      uint16_t* drow = reinterpret_cast<uint16_t*>(p.dq) + (((size_t)b * p.S + row) * p.Hq + h) * D;
      store_out_row(drow, tdQ + lane_base, D, row < p.S, p.is_bf16 ? DT_BF16 : DT_F16, p.scale);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) { tc_fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}

// =====================================================================================================
// dK / dV.  One CTA per (kv tile of 128 rows, QUERY head, batch): with grouped-query attention the heads of
// a group add their parts into an fp32 workspace (vector atomics), which keeps the grid large and the
// causal triangle balanced; with Hq == Hkv the CTA owns its output rows and stores them directly.
// =====================================================================================================
template <int D, int NCTA>
__global__ void __maxnreg__(NCTA == 2 ? 168 : 255)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                     const __grid_constant__ CUtensorMap tmv, const __grid_constant__ CUtensorMap tmdo,
                     const AttnParams p, float* __restrict__ ws) {
  constexpr int KT = AT_BM * D * 2;          // [128 x D] K / V tile
  constexpr int QT = BW_C * D * 2;           // [64 x D] Q / dO tile
  constexpr int PB = AT_BM * BW_C * 2;       // [128 x 64] 16-bit tile
  constexpr uint32_t TCOLS = (D == 64) ? 256 : 512;   // 64 (S^T) + 64 (dP^T) + D (dV) + D (dK)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if (status_poisoned(p.status)) return;
  if ((reinterpret_cast<uintptr_t>(smem_raw) & 1023) != 0) {
    if (threadIdx.x == 0) report_error(p.status, GB_ERR_BAD_ARG, 3, 0);
    return;
  }
  uint8_t* sK = smem_raw;
  uint8_t* sV = sK + KT;
  uint8_t* sQ = sV + KT;             // KV_ST stages
  uint8_t* sdO = sQ + KV_ST * QT;    // KV_ST stages
  uint8_t* sPT = sdO + KV_ST * QT;
  uint8_t* sdST = sPT + PB;
  float* lse_s = reinterpret_cast<float*>(sdST + PB);     // [4 warps][2][64] log2-domain row statistics, a copy per warp
  float* dl_s = lse_s + 8 * BW_C;                          // [4 warps][2][64] delta
  uint64_t* bars = reinterpret_cast<uint64_t*>(dl_s + 8 * BW_C);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;     // [KV_ST]
  uint64_t* sdp_full = bars + 4;
  uint64_t* sdp_free = bars + 5;
  uint64_t* ds_ready = bars + 6;
  uint64_t* acc_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int kvh = h / group;
  const int n0 = blockIdx.x * AT_BM;
  const int off = p.Sk - p.S;
  const int nq = (p.S + BW_C - 1) / BW_C;
  int i_start = 0;
  if (p.causal) { const int first = n0 - off; i_start = first > 0 ? first / BW_C : 0; }
  const int n_it = nq > i_start ? nq - i_start : 0;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(sdp_full, 1);
    for (int i = 0; i < KV_ST; ++i) mbar_init(&qdo_full[i], 1);
    mbar_init(sdp_free, 128); mbar_init(ds_ready, 128); mbar_init(acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, TCOLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tST = tmem, tdPT = tmem + BW_C, tdV = tmem + 2 * BW_C, tdK = tmem + 2 * BW_C + D;

  if (warp == 4) {
    if (lane == 0 && n_it > 0) {   // ---------------- TMA + MMA ----------------
      const uint32_t fmt = p.is_bf16 ? 1u : 0u;
      const uint32_t idesc_s = make_idesc(fmt, 0, 0, AT_BM, BW_C);
      const uint32_t idesc_acc = make_idesc(fmt, 0, 1, AT_BM, D);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aPT = smem_u32(sPT), adST = smem_u32(sdST);
      auto load_q = [&](int it) {
        const int st = it % KV_ST;
        const int q0 = (i_start + it) * BW_C;
        mbar_expect_tx(&qdo_full[st], 2 * QT);
        load_tile<D>(sQ + st * QT, &tmq, &qdo_full[st], h, q0, b, BW_C);
        load_tile<D>(sdO + st * QT, &tmdo, &qdo_full[st], h, q0, b, BW_C);
      };
      auto issue_s = [&](int it) -> bool {
        const int st = it % KV_ST;
        if (!AT_WAIT(&qdo_full[st], (it / KV_ST) & 1, 62)) return false;
        if (it > 0 && !AT_WAIT(sdp_free, (it - 1) & 1, 64)) return false;
        tc_fence_after_sync();
        const uint32_t aQ = smem_u32(sQ + st * QT), adO = smem_u32(sdO + st * QT);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          umma_f16(tST, desc_kmajor(aK, kk, AT_BM), desc_kmajor(aQ, kk, BW_C), idesc_s, kk > 0);
          umma_f16(tdPT, desc_kmajor(aV, kk, AT_BM), desc_kmajor(adO, kk, BW_C), idesc_s, kk > 0);
        }
        umma_commit(sdp_full);
        return true;
      };
      mbar_expect_tx(kv_full, 2 * KT);
      load_tile<D>(sK, &tmk, kv_full, kvh, n0, b, AT_BM);
      load_tile<D>(sV, &tmv, kv_full, kvh, n0, b, AT_BM);
      for (int it = 0; it < KV_ST && it < n_it; ++it) load_q(it);
      bool ok = AT_WAIT(kv_full, 0, 61) && issue_s(0);
      for (int it = 0; ok && it < n_it; ++it) {
        if (it + 1 < n_it && !issue_s(it + 1)) break;
        if (!AT_WAIT(ds_ready, it & 1, 63)) break;
        tc_fence_after_sync();
        const uint32_t aQ = smem_u32(sQ + (it % KV_ST) * QT), adO = smem_u32(sdO + (it % KV_ST) * QT);
#pragma unroll
        for (int kk = 0; kk < BW_C / 16; ++kk) {
          umma_f16(tdV, desc_kmajor(aPT, kk, AT_BM), desc_mnmajor(adO, kk, BW_C), idesc_acc, (it > 0 || kk > 0));
          umma_f16(tdK, desc_kmajor(adST, kk, AT_BM), desc_mnmajor(aQ, kk, BW_C), idesc_acc, (it > 0 || kk > 0));
        }
        umma_commit(acc_done);
        // two stages: the stage of tile `it` is free once the MMAs just committed are done (a wait on the phase
        // that was committed last cannot alias)
        if (it + KV_ST < n_it) {
          if (!AT_WAIT(acc_done, it & 1, 60)) break;
          load_q(it + KV_ST);
        }
      }
    }
  } else {
    const int t = threadIdx.x;
    const int kvrow = n0 + t;
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    const float sl2 = p.scale * LOG2E;
    const size_t stat0 = ((size_t)b * p.Hq + h) * p.S;
    bool ok = true;
    // Per-column statistics (log2-domain LSE, delta) of a q tile: each warp keeps its own copy in shared memory,
    // double-buffered; a lane fetches two columns of the NEXT tile into registers at the top of an iteration and
    // parks them in the other buffer at its end, so the global latency hides behind the tile's arithmetic.
    auto fetch_stats = [&](int it, float (&v)[4]) {
      const int q0n = (i_start + it) * BW_C;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int qr = q0n + lane + u * 32;
        v[u] = qr < p.S ? p.lse_in[stat0 + qr] * LOG2E : 0.f;
        v[2 + u] = qr < p.S ? p.delta[stat0 + qr] : 0.f;
      }
    };
    auto park_stats = [&](int it, const float (&v)[4]) {
      float* lb = lse_s + (warp * 2 + (it & 1)) * BW_C;
      float* db = dl_s + (warp * 2 + (it & 1)) * BW_C;
      lb[lane] = v[0]; lb[lane + 32] = v[1]; db[lane] = v[2]; db[lane + 32] = v[3];
    };
    if (n_it > 0) {
      float v0[4];
      fetch_stats(0, v0);
      park_stats(0, v0);
      __syncwarp();
    }
    for (int it = 0; it < n_it; ++it) {
      const int q0 = (i_start + it) * BW_C;
      float nxt[4] = {0.f, 0.f, 0.f, 0.f};
      if (it + 1 < n_it) fetch_stats(it + 1, nxt);
      const float* lse_b = lse_s + (warp * 2 + (it & 1)) * BW_C;
      const float* dl_b = dl_s + (warp * 2 + (it & 1)) * BW_C;
      if (!__all_sync(0xffffffffu, AT_WAIT(sdp_full, it & 1, 70))) { ok = false; break; }
      tc_fence_after_sync();
      const bool need_mask = (q0 + BW_C > p.S) || (n0 + AT_BM > p.Sk) || (p.causal && (n0 + AT_BM - 1 > q0 + off));
      // this kv row is visible to query columns first..last of the tile
      const int first = p.causal ? kvrow - off - q0 : 0;
      const int last = kvrow < p.Sk ? p.S - 1 - q0 : -1;
      // two half tiles of 32 columns, each read from tensor memory just before its use: 64 live accumulator
      // registers instead of 128 keep the kernel at two CTAs per SM
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld_32x32b_x32(tST + lane_base + c * 32, rs);
        tmem_ld_32x32b_x32(tdPT + lane_base + c * 32, rp);
        tmem_ld_wait();
        if (c == 1) { tc_fence_before_sync(); mbar_arrive(sdp_free); }
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int qc = c * 32 + i;
            rs[i] = (qc >= first && qc <= last) ? rs[i] : 0xff800000u;      // -inf: probability 0
          }
        }
        float pt[32], dst[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int qc = c * 32 + i;
          const float pr = fast_exp2(fmaf(__uint_as_float(rs[i]), sl2, -lse_b[qc]));
          pt[i] = pr;
          dst[i] = pr * (__uint_as_float(rp[i]) - dl_b[qc]);       // the softmax scale is applied once, to dK at the end
        }
        // the P^T / dS^T tiles are single-buffered: the previous iteration's MMAs have to be done with them
        if (c == 0 && it > 0 && !__all_sync(0xffffffffu, AT_WAIT(acc_done, (it - 1) & 1, 71))) { ok = false; break; }
        store_row_chunk(sPT, t, c * 32, pt, p.is_bf16, AT_BM * 128);
        store_row_chunk(sdST, t, c * 32, dst, p.is_bf16, AT_BM * 128);
      }
      if (!ok) break;
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(ds_ready);
      if (it + 1 < n_it) park_stats(it + 1, nxt);
      __syncwarp();
    }
    const size_t orow = (((size_t)b * p.Sk + kvrow) * p.Hkv + kvh) * D;
    const bool valid = kvrow < p.Sk;
    if (n_it == 0) {
      // no query row sees this kv tile: its gradient is zero (only the owning-store path has to write it)
      if (ws == nullptr && valid) {
        uint4 z = make_uint4(0, 0, 0, 0);
        uint4* a = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.dk) + orow);
        uint4* c = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.dv) + orow);
        for (int i = 0; i < D / 8; ++i) { a[i] = z; c[i] = z; }
      }
    } else if (ok && __all_sync(0xffffffffu, AT_WAIT(acc_done, (n_it - 1) & 1, 72))) {
      tc_fence_after_sync();
      if (ws == nullptr) {
        const int dt = p.is_bf16 ? DT_BF16 : DT_F16;
        store_out_row(reinterpret_cast<uint16_t*>(p.dv) + orow, tdV + lane_base, D, valid, dt);
        store_out_row(reinterpret_cast<uint16_t*>(p.dk) + orow, tdK + lane_base, D, valid, dt, p.scale);
      } else {
        // ws = [2][B, Sk, Hkv, D] fp32: dK first, dV second
        const size_t half = (size_t)p.B * p.Sk * p.Hkv * D;
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          float* dst = ws + (which ? half : 0) + orow;
          const uint32_t src = (which ? tdV : tdK) + lane_base;
          const float mul = which ? 1.f : p.scale;
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(src + c, r);
            tmem_ld_wait();
            if (valid) {
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                atomicAdd(reinterpret_cast<float4*>(dst + c + i),
                          make_float4(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul,
                                      __uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul));
            }
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) { tc_fence_after_sync(); tmem_dealloc(tmem, TCOLS); }
}

// delta[b, h, s] = sum_d dO * O ; D / 8 lanes per row, 16 bytes per lane
template <typename T, int D>
__global__ void attn_delta_kernel(const T* __restrict__ o, const T* __restrict__ dout, float* __restrict__ delta,
                                  int B, int S, int H) {
  constexpr int LPR = D / 8;                 // lanes per row (8 or 16)
  const long long rows = (long long)B * S * H;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const int sub = (int)(tid % LPR);
  // whole warps leave the loop together: rows per pass is a multiple of the rows a warp covers
  for (long long r0 = tid / LPR; r0 - (threadIdx.x & 31) / LPR < rows; r0 += nthreads / LPR) {
    float acc = 0.f;
    if (r0 < rows) {
      const Vec16<T> a = ld16(o + r0 * D + sub * 8);
      const Vec16<T> g = ld16(dout + r0 * D + sub * 8);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc += Cvt<T>::to_f(a.v[i]) * Cvt<T>::to_f(g.v[i]);
    }
#pragma unroll
    for (int m = LPR / 2; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
    if (sub == 0 && r0 < rows) {
      const int h = (int)(r0 % H);
      const long long bs = r0 / H;
      const int s_ = (int)(bs % S);
      const int b = (int)(bs / S);
      delta[((long long)b * H + h) * S + s_] = acc;
    }
  }
}

// fp32 workspace [2][n] (dK, dV) -> the 16-bit gradients
template <typename T>
__global__ void attn_dkv_convert_kernel(const float* __restrict__ ws, T* __restrict__ dk, T* __restrict__ dv,
                                        long long n) {
  const long long n4 = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < 2 * n4;
       i += (long long)gridDim.x * blockDim.x) {
    const bool second = i >= n4;
    const long long j = second ? i - n4 : i;
    const float4 v = reinterpret_cast<const float4*>(ws + (second ? n : 0))[j];
    T* dst = (second ? dv : dk) + 4 * j;
    uint2 w;
    w.x = pack2(v.x, v.y, std::is_same<T, __nv_bfloat16>::value ? DT_BF16 : DT_F16);
    w.y = pack2(v.z, v.w, std::is_same<T, __nv_bfloat16>::value ? DT_BF16 : DT_F16);
    *reinterpret_cast<uint2*>(dst) = w;
  }
}

template <int D, int NCTA>
static int launch_bwd(const CUtensorMap& tq128, const CUtensorMap& tdo128, const CUtensorMap& tk64,
                      const CUtensorMap& tv64, const CUtensorMap& tq64, const CUtensorMap& tdo64,
                      const CUtensorMap& tk128, const CUtensorMap& tv128, const AttnParams& p, float* ws,
                      cudaStream_t st) {
  // no alignment pad: shared memory of a CTA starts 1024-aligned (checked in the kernels), and at D = 64 two
  // CTAs have to fit in one SM
  const int smem_dq = 2 * AT_BM * D * 2 + 2 * BW_ST * BW_C * D * 2 + 128;
  const int smem_kv = 2 * AT_BM * D * 2 + 2 * KV_ST * BW_C * D * 2 + 2 * AT_BM * BW_C * 2 + 16 * BW_C * 4 + 128;
  static unsigned long long cfg_dq = 0, cfg_kv = 0;
  int r;
  if ((r = smem_opt_in(attn_bwd_dq_kernel<D, NCTA>, smem_dq, cfg_dq)) != 0) return r;
  if ((r = smem_opt_in(attn_bwd_dkdv_kernel<D, NCTA>, smem_kv, cfg_kv)) != 0) return r;
  dim3 gq((p.S + AT_BM - 1) / AT_BM, p.Hq, p.B), gk((p.Sk + AT_BM - 1) / AT_BM, p.Hq, p.B);
  attn_bwd_dq_kernel<D, NCTA><<<gq, 160, smem_dq, st>>>(tq128, tk64, tv64, tdo128, p);
  attn_bwd_dkdv_kernel<D, NCTA><<<gk, 160, smem_kv, st>>>(tq64, tk128, tv128, tdo64, p, ws);
  return (int)cudaGetLastError();
}

}  // namespace gb

using namespace gb;

// dkv_ws: fp32 scratch of 2 * B * Sk * Hkv * D elements, needed (and used) only when Hq != Hkv.
extern "C" int gb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                           const float* lse, float* delta, void* dq, void* dk, void* dv, float* dkv_ws, int B,
                           int S, int Sk, int Hq, int Hkv, int D, int causal, float scale, int is_bf16,
                           int* status, cudaStream_t st) {
  if (D != 64 && D != 128) return -2;
  if (Hq % Hkv != 0 || Sk < S) return -3;
  const bool gqa = Hq != Hkv;
  if (gqa && dkv_ws == nullptr) return -4;
  CUtensorMap tq, tk, tv, tdo, tq64, tk64, tv64, tdo64;
  int r;
  if ((r = make_tmap_bshd(&tq, q, is_bf16, B, S, Hq, D, 128)) != 0) return 10000 + r;
  if ((r = make_tmap_bshd(&tk, k, is_bf16, B, Sk, Hkv, D, 128)) != 0) return 20000 + r;
  if ((r = make_tmap_bshd(&tv, v, is_bf16, B, Sk, Hkv, D, 128)) != 0) return 30000 + r;
  if ((r = make_tmap_bshd(&tdo, dout, is_bf16, B, S, Hq, D, 128)) != 0) return 40000 + r;
  if ((r = make_tmap_bshd(&tq64, q, is_bf16, B, S, Hq, D, BW_C)) != 0) return 50000 + r;
  if ((r = make_tmap_bshd(&tk64, k, is_bf16, B, Sk, Hkv, D, BW_C)) != 0) return 60000 + r;
  if ((r = make_tmap_bshd(&tv64, v, is_bf16, B, Sk, Hkv, D, BW_C)) != 0) return 70000 + r;
  if ((r = make_tmap_bshd(&tdo64, dout, is_bf16, B, S, Hq, D, BW_C)) != 0) return 80000 + r;
  const long long rows = (long long)B * S * Hq;
  const int dgrid = gb_grid(rows * (D / 8), 256);
  if (is_bf16 && D == 64) attn_delta_kernel<__nv_bfloat16, 64><<<dgrid, 256, 0, st>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, S, Hq);
  else if (is_bf16) attn_delta_kernel<__nv_bfloat16, 128><<<dgrid, 256, 0, st>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, S, Hq);
  else if (D == 64) attn_delta_kernel<__half, 64><<<dgrid, 256, 0, st>>>((const __half*)o, (const __half*)dout,
                                                                        delta, B, S, Hq);
  else attn_delta_kernel<__half, 128><<<dgrid, 256, 0, st>>>((const __half*)o, (const __half*)dout, delta, B, S, Hq);
  const long long nkv = (long long)B * Sk * Hkv * D;
  if (gqa && (r = (int)cudaMemsetAsync(dkv_ws, 0, 2 * nkv * sizeof(float), st)) != 0) return r;
  AttnParams p{};
  p.lse_in = lse; p.delta = delta; p.dq = dq; p.dk = dk; p.dv = dv; p.status = status;
  p.B = B; p.S = S; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.is_bf16 = is_bf16; p.scale = scale;
  float* ws = gqa ? dkv_ws : nullptr;
  if (D == 64) r = launch_bwd<64, 2>(tq, tdo, tk64, tv64, tq64, tdo64, tk, tv, p, ws, st);
  else r = launch_bwd<128, 1>(tq, tdo, tk64, tv64, tq64, tdo64, tk, tv, p, ws, st);
  if (r != 0) return r;
  if (gqa) {
    if (is_bf16) attn_dkv_convert_kernel<__nv_bfloat16><<<gb_grid(nkv / 2, 256), 256, 0, st>>>(
        dkv_ws, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, nkv);
    else attn_dkv_convert_kernel<__half><<<gb_grid(nkv / 2, 256), 256, 0, st>>>(dkv_ws, (__half*)dk, (__half*)dv, nkv);
  }
  return (int)cudaGetLastError();
}
