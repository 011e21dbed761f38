/* Entry points of libgenesis_b200.so that never allocate memory.
 *
 * There is no counterpart of this in the reference framework: it exists for users of this library
 * whose call site is not allowed to allocate.  Two kinds of callers are meant.  (1) Code that lives
 * under a memory manager it does not own and whose budget was fixed up front - an inference server
 * that sized its pools at start-up, or a plugin loaded into another runtime - where one more
 * cudaMalloc may fail or break the host's accounting.  (2) Code on a latency-critical path, where
 * cudaMalloc / cudaFree are ruled out because they synchronise the device and stall every stream.
 *
 * The scratch memory such a kernel needs is a file-scope `static __device__` array inside the library
 * (for gb_rmsnorm_bwd_noalloc: 296 x 4096 floats = 4.6 MiB).  Every GPU that loads the library holds
 * that array until the process exits.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* RMSNorm backward: dx = rstd * (g*w - xhat * mean(g*w*xhat)) and dw = sum over rows of g * xhat,
 * the same math as gb_rmsnorm_bwd, with the per-CTA partial sums of dw kept in the library's own
 * scratch array instead of a caller-provided buffer.
 *
 *   g, x, dx : [rows, cols] contiguous, 16-byte aligned, dtype code `dt` (0 = float32, 1 = float16,
 *              2 = bfloat16); w : [cols] of dtype code `wdt` (float32, or the same 16-bit type as x);
 *   rstd     : [rows] float32, as produced by gb_rmsnorm_fwd;   dw : [cols] float32 (overwritten).
 *   The caller owns and passes every input and output; nothing is allocated or freed in here, and no
 *   allocating library routine is called.
 *
 * Limits: cols <= gb_rmsnorm_bwd_noalloc_max_cols() (4096) and a multiple of 8 (16-bit) or 4 (float32)
 * elements.  Anything else is rejected before a launch with a negative code; gb_rmsnorm_bwd_noalloc_strerror
 * turns the code into text.  A positive return value is a cudaError_t from the runtime.
 *
 * First call on a device: looks up the device address of the scratch array (cudaGetSymbolAddress, with
 * that device current) and caches it.  Make this first call before you start capturing a stream.
 *
 * Sharing: all calls on a device use the same scratch array, which keeps whatever the previous call left
 * in it.  The kernels overwrite every element they later read, so no clearing is needed between calls,
 * but two calls that overlap on the GPU (different streams, no ordering between them) race on it.
 * Order them on one stream or with events.
 */
int gb_rmsnorm_bwd_noalloc(const void* g, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                           long long rows, int cols, int dt, int wdt, cudaStream_t stream);

int gb_rmsnorm_bwd_noalloc_max_cols(void);
const char* gb_rmsnorm_bwd_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
