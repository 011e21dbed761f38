// Multi-tensor optimizer kernels: ONE launch updates every parameter of the model.
//
// The host passes a device table `meta` of int64 rows, each of length `nt` (number of tensors):
//   row 0 param ptr, 1 grad ptr, 2 state-1 ptr (m / momentum buffer), 3 state-2 ptr (v), 4 shadow ptr (or 0),
//   row 5 numel, 6 first chunk index (prefix sum of ceil(numel / CHUNK)), 7 grad dtype code.
// Block b finds its tensor by binary search over row 6 and handles CHUNK consecutive elements.
// AMP hooks: `grad_scale` (device float, multiplies gradients) and `found_inf` (device float; when it is
// non-zero the whole launch is a no-op), so a training step needs no host synchronisation.
// Reference counterpart: one Triton launch per parameter, genesis/optim/adamw.py:9-147.
#include "common.cuh"

namespace gb {

constexpr int OPT_CHUNK = 8192;
constexpr int OPT_THREADS = 256;

__device__ __forceinline__ int find_tensor(const long long* starts, int nt, long long chunk) {
  int lo = 0, hi = nt;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (starts[mid] <= chunk) lo = mid; else hi = mid;
  }
  return lo;
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;
  int decoupled;
  int shadow_dtype;
};

// Step-dependent scalars kept on the device so that a captured CUDA graph of the step stays valid when replayed:
// dyn[0] learning rate (written by the host between replays), dyn[1] / dyn[2] bias corrections, dyn[3] step count.
// The betas arrive as doubles so that the corrections round to the same floats as the host's 1 - beta ** step.
// A step that the overflow flag cancels does not count: the bias corrections follow the updates actually applied.
__global__ void adam_dyn_advance_kernel(float* __restrict__ dyn, double beta1, double beta2,
                                        const float* __restrict__ found_inf) {
  if (found_inf != nullptr && *found_inf != 0.f) return;
  const double step = (double)dyn[3] + 1.0;
  dyn[3] = (float)step;
  dyn[1] = (float)(1.0 - pow(beta1, step));
  dyn[2] = (float)(1.0 - pow(beta2, step));
}

__device__ __forceinline__ void adam_update(float& pi, float& mi, float& vi, float gi, const AdamArgs& a) {
  if (a.decoupled) pi *= (1.f - a.lr * a.weight_decay);
  else gi += a.weight_decay * pi;
  mi = a.beta1 * mi + (1.f - a.beta1) * gi;
  vi = a.beta2 * vi + (1.f - a.beta2) * gi * gi;
  pi -= a.lr * (mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps);
}

__global__ void __launch_bounds__(OPT_THREADS)
adam_multi_kernel(const long long* __restrict__ meta, int nt, AdamArgs a, const float* __restrict__ grad_scale,
                  const float* __restrict__ found_inf, const float* __restrict__ dyn) {
  if (found_inf != nullptr && *found_inf != 0.f) return;
  if (dyn != nullptr) { a.lr = dyn[0]; a.bc1 = dyn[1]; a.bc2 = dyn[2]; }
  const int t = find_tensor(meta + 6ll * nt, nt, blockIdx.x);
  float* p = reinterpret_cast<float*>(meta[0ll * nt + t]);
  const void* g = reinterpret_cast<const void*>(meta[1ll * nt + t]);
  float* m = reinterpret_cast<float*>(meta[2ll * nt + t]);
  float* v = reinterpret_cast<float*>(meta[3ll * nt + t]);
  void* sh = reinterpret_cast<void*>(meta[4ll * nt + t]);
  const long long n = meta[5ll * nt + t];
  const int gdt = (int)meta[7ll * nt + t];
  const long long base = (blockIdx.x - meta[6ll * nt + t]) * OPT_CHUNK;
  const float gs = grad_scale != nullptr ? *grad_scale : 1.f;
  const long long end = (base + OPT_CHUNK < n) ? base + OPT_CHUNK : n;
  // fp32 gradients, 16-byte aligned tensors (and an 8-byte aligned 16-bit shadow copy, if any): four elements per
  // thread and access
  const bool sh16 = a.shadow_dtype == DT_BF16 || a.shadow_dtype == DT_F16;
  const bool vec = gdt == DT_F32 && (sh == nullptr || (sh16 && ((uintptr_t)sh & 7) == 0)) &&
      (((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15) == 0;
  if (vec) {
    const long long end4 = base + ((end - base) & ~3ll);
    for (long long i = base + 4ll * threadIdx.x; i < end4; i += 4ll * OPT_THREADS) {
      float4 g4 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g) + i);
      float4 p4 = *reinterpret_cast<const float4*>(p + i);
      float4 m4 = *reinterpret_cast<const float4*>(m + i);
      float4 v4 = *reinterpret_cast<const float4*>(v + i);
      adam_update(p4.x, m4.x, v4.x, g4.x * gs, a);
      adam_update(p4.y, m4.y, v4.y, g4.y * gs, a);
      adam_update(p4.z, m4.z, v4.z, g4.z * gs, a);
      adam_update(p4.w, m4.w, v4.w, g4.w * gs, a);
      *reinterpret_cast<float4*>(p + i) = p4;
      *reinterpret_cast<float4*>(m + i) = m4;
      *reinterpret_cast<float4*>(v + i) = v4;
      if (sh != nullptr) {
        uint2 o;
        if (a.shadow_dtype == DT_BF16) { o.x = pack2c<true>(p4.x, p4.y); o.y = pack2c<true>(p4.z, p4.w); }
        else { o.x = pack2c<false>(p4.x, p4.y); o.y = pack2c<false>(p4.z, p4.w); }
        *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(sh) + i) = o;
      }
    }
    for (long long i = end4 + threadIdx.x; i < end; i += OPT_THREADS) {
      float pi = p[i], mi = m[i], vi = v[i];
      adam_update(pi, mi, vi, reinterpret_cast<const float*>(g)[i] * gs, a);
      p[i] = pi; m[i] = mi; v[i] = vi;
      if (sh != nullptr) store_from_float(sh, a.shadow_dtype, i, pi);
    }
    return;
  }
  for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) {
    float pi = p[i], mi = m[i], vi = v[i];
    adam_update(pi, mi, vi, load_as_float(g, gdt, i) * gs, a);
    p[i] = pi; m[i] = mi; v[i] = vi;
    if (sh != nullptr) store_from_float(sh, a.shadow_dtype, i, pi);
  }
}

// u = momentum*u + (1-momentum)*(g + wd*p); p -= lr*u
__global__ void __launch_bounds__(OPT_THREADS)
sgd_multi_kernel(const long long* __restrict__ meta, int nt, float lr, float momentum, float weight_decay) {
  const int t = find_tensor(meta + 6ll * nt, nt, blockIdx.x);
  float* p = reinterpret_cast<float*>(meta[0ll * nt + t]);
  const void* g = reinterpret_cast<const void*>(meta[1ll * nt + t]);
  float* u = reinterpret_cast<float*>(meta[2ll * nt + t]);
  const long long n = meta[5ll * nt + t];
  const int gdt = (int)meta[7ll * nt + t];
  const long long base = (blockIdx.x - meta[6ll * nt + t]) * OPT_CHUNK;
  const long long end = (base + OPT_CHUNK < n) ? base + OPT_CHUNK : n;
  for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) {
    const float pi = p[i];
    const float gi = load_as_float(g, gdt, i) + weight_decay * pi;
    const float ui = momentum * u[i] + (1.f - momentum) * gi;
    u[i] = ui;
    p[i] = pi - lr * ui;
  }
}

// mode bit 0: multiply by *scale; bit 1: raise found_inf on Inf/NaN; bit 2: accumulate sum of squares into norm_sq
__global__ void __launch_bounds__(OPT_THREADS)
grad_multi_kernel(const long long* __restrict__ meta, int nt, const float* __restrict__ scale, float fixed_scale,
                  float* __restrict__ found_inf, float* __restrict__ norm_sq, int mode) {
  __shared__ float shm[32];
  const int t = find_tensor(meta + 6ll * nt, nt, blockIdx.x);
  void* g = reinterpret_cast<void*>(meta[1ll * nt + t]);
  const long long n = meta[5ll * nt + t];
  const int gdt = (int)meta[7ll * nt + t];
  const long long base = (blockIdx.x - meta[6ll * nt + t]) * OPT_CHUNK;
  const long long end = (base + OPT_CHUNK < n) ? base + OPT_CHUNK : n;
  const float s = (mode & 1) ? (scale != nullptr ? *scale : fixed_scale) : 1.f;
  bool bad = false;
  float ss = 0.f;
  for (long long i = base + threadIdx.x; i < end; i += OPT_THREADS) {
    float gi = load_as_float(g, gdt, i);
    if (!isfinite(gi)) bad = true;
    if (mode & 1) { gi *= s; store_from_float(g, gdt, i, gi); }
    ss += gi * gi;
  }
  if ((mode & 2) && __syncthreads_or(bad) && threadIdx.x == 0) *found_inf = 1.f;
  if (mode & 4) {
    ss = block_sum(ss, shm);
    if (threadIdx.x == 0) atomicAdd(norm_sq, ss);
  }
}

}  // namespace gb

using namespace gb;

extern "C" int gb_opt_chunk() { return OPT_CHUNK; }

extern "C" int gb_adam_multi(const long long* meta, int nt, long long total_chunks, float lr, float beta1,
                             float beta2, float eps, float weight_decay, float bc1, float bc2, int decoupled,
                             int shadow_dtype, const float* grad_scale, const float* found_inf, const float* dyn,
                             cudaStream_t st) {
  if (total_chunks == 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bc1, bc2, decoupled, shadow_dtype};
  adam_multi_kernel<<<(unsigned)total_chunks, OPT_THREADS, 0, st>>>(meta, nt, a, grad_scale, found_inf, dyn);
  return (int)cudaGetLastError();
}

extern "C" int gb_adam_dyn_advance(float* dyn, double beta1, double beta2, const float* found_inf,
                                   cudaStream_t st) {
  adam_dyn_advance_kernel<<<1, 1, 0, st>>>(dyn, beta1, beta2, found_inf);
  return (int)cudaGetLastError();
}

extern "C" int gb_sgd_multi(const long long* meta, int nt, long long total_chunks, float lr, float momentum,
                            float weight_decay, cudaStream_t st) {
  if (total_chunks == 0) return 0;
  sgd_multi_kernel<<<(unsigned)total_chunks, OPT_THREADS, 0, st>>>(meta, nt, lr, momentum, weight_decay);
  return (int)cudaGetLastError();
}

extern "C" int gb_grad_multi(const long long* meta, int nt, long long total_chunks, const float* scale,
                             float fixed_scale, float* found_inf, float* norm_sq, int mode, cudaStream_t st) {
  if (total_chunks == 0) return 0;
  grad_multi_kernel<<<(unsigned)total_chunks, OPT_THREADS, 0, st>>>(meta, nt, scale, fixed_scale, found_inf,
                                                                    norm_sq, mode);
  return (int)cudaGetLastError();
}

// Plain asynchronous host-to-device copy on `st` (pointer tables uploaded while a CUDA graph is captured: the node
// reads the pinned source again on every replay, the caller keeps it alive).
extern "C" int gb_copy_h2d_async(void* dst, const void* src, long long bytes, cudaStream_t st) {
  return (int)cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, st);
}
