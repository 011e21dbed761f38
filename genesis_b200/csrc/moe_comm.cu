// Expert-parallel dispatch and combine over peer memory (NVLink / NVSwitch): the all-to-alls of a
// mixture-of-experts layer as PULL kernels.  Nothing is packed or sent: the owner of an expert reads the
// token rows it needs straight out of the source ranks' activation buffers (plain peer loads), and the source
// rank later reads the expert outputs straight out of the owners' output buffers while it forms the weighted
// sum over the k slots.  No NCCL call, no host synchronisation, every wait bounded.
//
// Symmetric (peer-mapped) buffers per rank: x (token rows), tok (token index of every sorted (token, slot)
// pair, sorted by global expert id), ws (routing weight of every sorted pair), y (rows in the owner's
// receive layout) and a float-per-row buffer for the routing-weight gradient.
//
// Receive layout of rank r: expert-major over its local experts, inside an expert source-rank-minor, every
// expert segment padded to a multiple of `align` rows (one GEMM tile), so the grouped GEMMs run on it as is.
//
//   ep_layout          (local)  all ranks' per-expert offsets -> segment table, padded expert offsets,
//                               and for every global expert the row where THIS rank's rows start at its owner
//   ep_dispatch_pull   barrier, then row (e, p, i) <- x_p[tok_p[off_p[e] + i]]           (forward)
//                      or      row <- ws_p[..] * g_p[tok_p[..]],  dwr[row] = <g_p[..], y[row]>  (backward of combine)
//   ep_combine_pull    barrier, then out[t] = sum_j w[t, j] * y_d[row(t, j)]                (forward)
//                      or      dx[t] = sum_j dxe_d[row(t, j)],   dw[t, j] = dwr_d[row(t, j)] (backward of dispatch)
//
// Reference counterpart: none (the reference loops over all experts on one GPU,
// genesis/models/transformers/moe.py:317-361).
#include "comm_common.cuh"

namespace gb {

constexpr int EP_MAX_SEGS = 4096;      // local experts x world, held in shared memory for the row search

// all_off [W][E + 1]: offsets of every rank's pair list sorted by global expert.
__global__ void ep_layout_kernel(const int* __restrict__ all_off, int rank, int world, int E, int align,
                                 int capacity, int* __restrict__ local_offsets, int* __restrict__ seg_start,
                                 int* __restrict__ seg_src_off, int* __restrict__ dest_base, int* __restrict__ info,
                                 int* __restrict__ status) {
  const int El = E / world;
  extern __shared__ int sm[];
  int* padded = sm;                      // [world][El + 1] padded expert offsets of every rank's layout
  // one thread per destination rank computes that rank's padded expert offsets (El <= a few hundred)
  for (int d = threadIdx.x; d < world; d += blockDim.x) {
    int pos = 0;
    for (int e = 0; e < El; ++e) {
      padded[d * (El + 1) + e] = pos;
      int cnt = 0;
      const int g = d * El + e;
      for (int p = 0; p < world; ++p) cnt += all_off[p * (E + 1) + g + 1] - all_off[p * (E + 1) + g];
      pos += (cnt + align - 1) / align * align;
    }
    padded[d * (El + 1) + El] = pos;
  }
  __syncthreads();
  // rows of rank `rank` for global expert g start, in the owner's layout, after the rows of lower ranks
  for (int g = threadIdx.x; g < E; g += blockDim.x) {
    const int d = g / El, e = g % El;
    int before = 0;
    for (int p = 0; p < rank; ++p) before += all_off[p * (E + 1) + g + 1] - all_off[p * (E + 1) + g];
    dest_base[g] = padded[d * (El + 1) + e] + before;
  }
  // my own receive layout
  for (int e = threadIdx.x; e <= El; e += blockDim.x) local_offsets[e] = padded[rank * (El + 1) + e];
  for (int s = threadIdx.x; s < El * world; s += blockDim.x) {
    const int e = s / world, p = s % world;
    const int g = rank * El + e;
    int before = 0;
    for (int q = 0; q < p; ++q) before += all_off[q * (E + 1) + g + 1] - all_off[q * (E + 1) + g];
    seg_start[s] = padded[rank * (El + 1) + e] + before;
    seg_src_off[s] = all_off[p * (E + 1) + g];
  }
  if (threadIdx.x == 0) {
    const int total = padded[rank * (El + 1) + El];
    info[0] = total;
    if (total > capacity) report_error(status, GB_ERR_BAD_ARG, 900, total);
  }
}

// seg_cnt is implied: rows of segment s = off_p[g + 1] - off_p[g], read from all_off.
template <typename T>
__global__ void __launch_bounds__(512)
ep_dispatch_pull_kernel(PeerTable xs, PeerTable toks, PeerTable wss, PeerTable flags, const int* __restrict__ all_off,
                        const int* __restrict__ local_offsets, const int* __restrict__ seg_start,
                        const int* __restrict__ seg_src_off, T* __restrict__ out, const T* __restrict__ y_rows,
                        float* __restrict__ dwr, int H, int rank, int world, int E, int capacity, int mode,
                        uint32_t epoch, unsigned long long budget_ns, int* __restrict__ status) {
  __shared__ int s_fail;
  __shared__ int s_start[EP_MAX_SEGS + 1];
  if (threadIdx.x == 0) s_fail = 0;
  if (!peer_barrier(flags, rank, world, 0, epoch, budget_ns, status, &s_fail)) return;
  const int El = E / world;
  const int nseg = El * world;
  for (int s = threadIdx.x; s < nseg; s += blockDim.x) s_start[s] = seg_start[s];
  int total = local_offsets[El];
  if (total > capacity) total = capacity;
  if (threadIdx.x == 0) s_start[nseg] = total;
  __syncthreads();
  constexpr int V = Vec16<T>::N;
  const int nvec = H / V;
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  // A warp takes 32 consecutive rows of the layout: lane l resolves row base + l (segment search, then ONE peer
  // load of the token index), after which the rows are copied one by one with all 32 lanes on a row.
  for (int base = warp * 32; base < total; base += nwarps * 32) {
    const int my_row = base + lane;
    int my_p = -1, my_t = 0;
    float my_w = 0.f;
    if (my_row < total) {
      int lo = 0, hi = nseg;                             // last segment whose start is <= row
      while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (s_start[mid] <= my_row) lo = mid; else hi = mid; }
      const int e = lo / world, p = lo % world;
      const int g = rank * El + e;
      const int cnt = all_off[p * (E + 1) + g + 1] - all_off[p * (E + 1) + g];
      const int i = my_row - s_start[lo];
      if (i < cnt) {                                     // else: padding up to the next expert
        const int sp = seg_src_off[lo] + i;              // position in p's sorted pair list
        my_p = p;
        my_t = *reinterpret_cast<const volatile int*>(reinterpret_cast<const int*>(toks.ptr[p]) + sp);
        if (mode == 1) my_w = *reinterpret_cast<const volatile float*>(reinterpret_cast<const float*>(wss.ptr[p]) + sp);
      }
    }
    const int nrows = total - base < 32 ? total - base : 32;
    if (mode == 0 && nvec <= 256) {
      // plain row copies: two rows (2 x 8 vectors per lane) in flight per warp, so a pair costs one NVLink round trip
      for (int r = 0; r < nrows; r += 2) {
        uint4 q[2][8];
        int pp[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          const int rr = r + h2 < nrows ? r + h2 : r;
          pp[h2] = __shfl_sync(0xffffffffu, my_p, rr);
          const int t = __shfl_sync(0xffffffffu, my_t, rr);
          if (r + h2 >= nrows) pp[h2] = -2;                       // no such row
          if (pp[h2] >= 0) {
            const T* src = reinterpret_cast<const T*>(xs.ptr[pp[h2]]) + (size_t)t * H;
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (lane + u * 32 < nvec) q[h2][u] = ld_volatile_v4(src + (lane + u * 32) * V);
          }
        }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          if (pp[h2] == -2) continue;
          T* dst = out + (size_t)(base + r + h2) * H;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (lane + u * 32 >= nvec) continue;
            *reinterpret_cast<uint4*>(dst + (lane + u * 32) * V) = pp[h2] >= 0 ? q[h2][u] : make_uint4(0, 0, 0, 0);
          }
        }
      }
      continue;
    }
    for (int r = 0; r < nrows; ++r) {
      const int p = __shfl_sync(0xffffffffu, my_p, r);
      const int t = __shfl_sync(0xffffffffu, my_t, r);
      const float wgt = __shfl_sync(0xffffffffu, my_w, r);
      const int row = base + r;
      T* dst = out + (size_t)row * H;
      if (p < 0) {
        Vec16<T> z;
#pragma unroll
        for (int q = 0; q < V; ++q) z.v[q] = Cvt<T>::from_f(0.f);
        for (int v = lane; v < nvec; v += 32) st16(dst + v * V, z);
        if (mode == 1 && lane == 0) dwr[row] = 0.f;
        continue;
      }
      const T* src = reinterpret_cast<const T*>(xs.ptr[p]) + (size_t)t * H;
      if (mode == 0) {
        for (int v0 = lane; v0 < nvec; v0 += 256) {
          uint4 q[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) if (v0 + u * 32 < nvec) q[u] = ld_volatile_v4(src + (v0 + u * 32) * V);
#pragma unroll
          for (int u = 0; u < 8; ++u) if (v0 + u * 32 < nvec) *reinterpret_cast<uint4*>(dst + (v0 + u * 32) * V) = q[u];
        }
      } else {
        const T* yr = y_rows + (size_t)row * H;
        float dot = 0.f;
        for (int v0 = lane; v0 < nvec; v0 += 128) {
          uint4 q[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) if (v0 + u * 32 < nvec) q[u] = ld_volatile_v4(src + (v0 + u * 32) * V);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (v0 + u * 32 >= nvec) continue;
            const T* ge = reinterpret_cast<const T*>(&q[u]);
            const Vec16<T> yv = ld16(yr + (v0 + u * 32) * V);
            Vec16<T> o;
#pragma unroll
            for (int c = 0; c < V; ++c) {
              const float gj = Cvt<T>::to_f(ge[c]);
              dot += gj * Cvt<T>::to_f(yv.v[c]);
              o.v[c] = Cvt<T>::from_f(gj * wgt);
            }
            st16(dst + (v0 + u * 32) * V, o);
          }
        }
        dot = warp_sum(dot);
        if (lane == 0) dwr[row] = dot;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(512)
ep_combine_pull_kernel(PeerTable ys, PeerTable dwrs, PeerTable flags, const int* __restrict__ idx,
                       const int* __restrict__ pos, const float* __restrict__ w, const int* __restrict__ my_off,
                       const int* __restrict__ dest_base, T* __restrict__ out, float* __restrict__ dw, int T_tokens,
                       int k, int H, int rank, int world, int E, int capacity, int mode, uint32_t epoch,
                       unsigned long long budget_ns, int* __restrict__ status) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  if (!peer_barrier(flags, rank, world, 0, epoch, budget_ns, status, &s_fail)) return;
  const int El = E / world;
  constexpr int V = Vec16<T>::N;
  const int nvec = H / V;
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int t = warp; t < T_tokens; t += nwarps) {
    // lane j resolves slot j of the token once: owner rank, row in the owner's layout, weight
    int my_d = 0, my_row = -1;
    float my_w = 0.f;
    if (lane < k) {
      const int g = idx[t * k + lane];
      my_d = g / El;
      my_row = dest_base[g] + pos[t * k + lane] - my_off[g];
      if (my_row >= capacity) my_row = -1;              // the owner's layout overflowed (reported there)
      my_w = mode == 0 ? w[t * k + lane] : 1.f;
      if (mode == 1)
        dw[t * k + lane] = my_row < 0 ? 0.f
            : *reinterpret_cast<const volatile float*>(reinterpret_cast<const float*>(dwrs.ptr[my_d]) + my_row);
    }
    for (int v0 = lane; v0 < nvec; v0 += 32) {
      float acc[V];
#pragma unroll
      for (int c = 0; c < V; ++c) acc[c] = 0.f;
      // up to eight slots of the token in flight at once (one NVLink round trip per eight rows, not per four)
      for (int j0 = 0; j0 < k; j0 += 8) {
        uint4 q[8];
        float wt[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int j = j0 + u < k ? j0 + u : k - 1;
          const int d = __shfl_sync(0xffffffffu, my_d, j);
          const int row = __shfl_sync(0xffffffffu, my_row, j);
          const float wj = __shfl_sync(0xffffffffu, my_w, j);
          const bool ok = j0 + u < k && row >= 0;       // uniform over the warp
          wt[u] = ok ? wj : 0.f;
          q[u] = make_uint4(0, 0, 0, 0);
          if (ok) q[u] = ld_volatile_v4(reinterpret_cast<const T*>(ys.ptr[d]) + (size_t)row * H + v0 * V);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const T* e = reinterpret_cast<const T*>(&q[u]);
#pragma unroll
          for (int c = 0; c < V; ++c) acc[c] += wt[u] * Cvt<T>::to_f(e[c]);
        }
      }
      Vec16<T> o;
#pragma unroll
      for (int c = 0; c < V; ++c) o.v[c] = Cvt<T>::from_f(acc[c]);
      st16(out + (size_t)t * H + v0 * V, o);
    }
  }
}

// Copies the rows of the receive layout that exist (row < local_offsets[El], at most `capacity`) into the
// symmetric buffer the peers read from; the count lives on the device, so the host never waits for it.
__global__ void ep_stage_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                     const int* __restrict__ total_rows, long long vec_per_row, int capacity) {
  int total = *total_rows;
  if (total > capacity) total = capacity;
  const long long n = (long long)total * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = src[i];
}

static void fill_table(PeerTable& t, void* const* ptrs, int world) {
  for (int i = 0; i < COMM_MAX_WORLD; ++i) t.ptr[i] = (ptrs != nullptr && i < world) ? ptrs[i] : nullptr;
}

}  // namespace gb

using namespace gb;

// all_off: int32 [world][E + 1] (every rank's offsets, gathered).  Outputs: local_offsets [E / world + 1],
// seg_start / seg_src_off [E / world * world], dest_base [E], info [1] = rows of this rank's receive layout.
extern "C" int gb_ep_layout(const int* all_off, int rank, int world, int E, int align, int capacity,
                            int* local_offsets, int* seg_start, int* seg_src_off, int* dest_base, int* info,
                            int* status, cudaStream_t st) {
  if (world < 1 || world > COMM_MAX_WORLD || E % world != 0 || (E / world) * world > EP_MAX_SEGS) return -2;
  const size_t smem = (size_t)world * (E / world + 1) * sizeof(int);
  ep_layout_kernel<<<1, 256, smem, st>>>(all_off, rank, world, E, align, capacity, local_offsets, seg_start,
                                         seg_src_off, dest_base, info, status);
  return (int)cudaGetLastError();
}

// mode 0: out[row] = x_p[tok_p[..]];  mode 1: out[row] = ws_p[..] * x_p[tok_p[..]], dwr[row] = <x_p[..], y_rows[row]>.
extern "C" int gb_ep_dispatch_pull(void* const* xs, void* const* toks, void* const* wss, void* const* flags,
                                   const int* all_off, const int* local_offsets, const int* seg_start,
                                   const int* seg_src_off, void* out, const void* y_rows, float* dwr, int H,
                                   int rank, int world, int E, int capacity, int mode, unsigned int epoch, int dt,
                                   int ctas, unsigned long long budget_ns, int* status, cudaStream_t st) {
  if (world < 1 || world > COMM_MAX_WORLD || E % world != 0 || (E / world) * world > EP_MAX_SEGS) return -2;
  if (dt != DT_BF16 && dt != DT_F16 && dt != DT_F32) return -2;
  if (ctas > COMM_MAX_CTAS) ctas = COMM_MAX_CTAS;
  if (ctas < 1) ctas = 1;
  PeerTable tx, tt, tw, tf;
  fill_table(tx, xs, world); fill_table(tt, toks, world); fill_table(tw, wss, world); fill_table(tf, flags, world);
  GB_DISPATCH_FLOAT(dt, T, {
    if (H % Vec16<T>::N != 0) return -3;
    ep_dispatch_pull_kernel<T><<<ctas, 512, 0, st>>>(tx, tt, tw, tf, all_off, local_offsets, seg_start, seg_src_off,
                                                     reinterpret_cast<T*>(out), reinterpret_cast<const T*>(y_rows),
                                                     dwr, H, rank, world, E, capacity, mode, epoch, budget_ns, status);
  });
  return (int)cudaGetLastError();
}

// mode 0: out[t] = sum_j w[t, j] * y_d[row(t, j)];  mode 1: out[t] = sum_j y_d[row(t, j)], dw[t, j] = dwr_d[row(t, j)].
extern "C" int gb_ep_combine_pull(void* const* ys, void* const* dwrs, void* const* flags, const int* idx,
                                  const int* pos, const float* w, const int* my_off, const int* dest_base, void* out,
                                  float* dw, int tokens, int k, int H, int rank, int world, int E, int capacity,
                                  int mode, unsigned int epoch, int dt, int ctas, unsigned long long budget_ns, int* status,
                                  cudaStream_t st) {
  if (world < 1 || world > COMM_MAX_WORLD || E % world != 0 || k > 32) return -2;
  if (dt != DT_BF16 && dt != DT_F16 && dt != DT_F32) return -2;
  if (ctas > COMM_MAX_CTAS) ctas = COMM_MAX_CTAS;
  if (ctas < 1) ctas = 1;
  PeerTable ty, td, tf;
  fill_table(ty, ys, world); fill_table(td, dwrs, world); fill_table(tf, flags, world);
  GB_DISPATCH_FLOAT(dt, T, {
    if (H % Vec16<T>::N != 0) return -3;
    ep_combine_pull_kernel<T><<<ctas, 512, 0, st>>>(ty, td, tf, idx, pos, w, my_off, dest_base,
                                                    reinterpret_cast<T*>(out), dw, tokens, k, H, rank, world, E, capacity,
                                                    mode, epoch, budget_ns, status);
  });
  return (int)cudaGetLastError();
}

// dst[0 .. rows) = src[0 .. rows) with rows = min(*total_rows, capacity), rows of row_bytes (multiple of 16).
extern "C" int gb_ep_stage_rows(const void* src, void* dst, const int* total_rows, long long row_bytes, int capacity,
                                cudaStream_t st) {
  if (row_bytes % 16 != 0) return -3;
  ep_stage_rows_kernel<<<148 * 8, 256, 0, st>>>(reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst),
                                                total_rows, row_bytes / 16, capacity);
  return (int)cudaGetLastError();
}
