// Native caching pool for device memory ("CUDA storage pool with statistics").
//
// Size classes: powers of two from 512 B to 1 MB ("small"), multiples of 2 MB up to 1 GB rounded to
// 1/8-octave steps ("large"), exact 2 MB multiples above.  A freed block goes back to the bin of
// its class tagged with the stream it was used on; the same stream reuses it immediately, another
// stream only after the CUDA event recorded at free time has completed (blocks wait in `pending`).
// Out of memory => every cached block is released and the allocation retried once.  Counters are
// always on (they are a few relaxed increments under the pool mutex).
//
// CUDA graphs: between `gb_pool_begin_capture` and `gb_pool_end_capture` every block handed out becomes the
// property of that capture.  Blocks of a capture that are freed (while capturing or later) go to the capture's
// private free list, which only allocations of the same capture may take from, so memory that a recorded kernel
// reads or writes on every replay is never handed to eager code; `gb_pool_release_capture` (graph destroyed)
// returns the private list to the common bins.  Allocation order inside a capture is the order of its replay, so
// reuse within the private list is safe on any stream of the capture.
//
// The two entry points `gb_pool_alloc` / `gb_pool_free` have the signature torch's
// CUDAPluggableAllocator expects, so the pool can back every torch CUDA tensor.
// Reference counterpart: genesis/backends/cuda_memory.py:30-848 (Python, cuda-python driver calls).
#include <cuda_runtime.h>
#include <stdint.h>
#include <sys/types.h>

#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

constexpr size_t kSmallMax = 1u << 20;
constexpr size_t kLargeStep = 2u << 20;
constexpr size_t kLargeMax = 1ull << 30;
constexpr int kMaxDevices = 16;

struct Block {
  void* ptr;
  size_t size;
  cudaStream_t stream;   // stream of the last use
  bool any_stream;       // the event recorded at free time has completed: every stream may take the block
                         // (a flag of its own: a null `stream` is the handle of the legacy default stream)
  int capture;           // 0, or the id of the graph capture that owns the block
};
struct Pending {
  Block b;
  cudaEvent_t ev;
};

struct DevicePool {
  std::mutex mu;
  std::map<size_t, std::vector<Block>> bins;   // free blocks by class size
  std::vector<Pending> pending;                 // freed on one stream, not yet reusable elsewhere
  std::unordered_map<void*, Block> live;
  int64_t alloc_count = 0, free_count = 0, cache_hits = 0, cuda_alloc_count = 0, pending_checks = 0;
  int64_t allocated = 0, max_allocated = 0, reserved = 0, max_reserved = 0, oom_retries = 0;
  int64_t limit = 0;   // 0 = none
  int capturing = 0;   // id of the capture in progress on this device (0 = none)
  int next_capture = 0;
  std::map<int, std::map<size_t, std::vector<Block>>> priv;   // capture id -> its private free lists
};

DevicePool g_pools[kMaxDevices];

size_t round_size(size_t n) {
  if (n <= 512) return 512;
  if (n <= kSmallMax) {
    size_t s = 512;
    while (s < n) s <<= 1;
    return s;
  }
  if (n <= kLargeMax) {
    // 8 classes per octave, each a multiple of 2 MB
    size_t oct = kLargeStep;
    while (oct * 2 < n) oct <<= 1;
    size_t step = oct / 8 < kLargeStep ? kLargeStep : oct / 8;
    return (n + step - 1) / step * step;
  }
  return (n + kLargeStep - 1) / kLargeStep * kLargeStep;
}

void drain_pending(DevicePool& P) {
  for (size_t i = 0; i < P.pending.size();) {
    ++P.pending_checks;
    if (cudaEventQuery(P.pending[i].ev) == cudaSuccess) {
      cudaEventDestroy(P.pending[i].ev);
      Block b = P.pending[i].b;
      b.any_stream = true;
      P.bins[b.size].push_back(b);
      P.pending[i] = P.pending.back();
      P.pending.pop_back();
    } else {
      ++i;
    }
  }
  cudaGetLastError();   // cudaErrorNotReady is not an error for us
}

int64_t release_cached(DevicePool& P) {
  int64_t freed = 0;
  for (auto& kv : P.bins) {
    for (Block& b : kv.second) {
      cudaFree(b.ptr);
      freed += (int64_t)b.size;
    }
    kv.second.clear();
  }
  P.bins.clear();
  P.reserved -= freed;
  return freed;
}

}  // namespace

extern "C" {

int64_t gb_pool_round_size(int64_t n) { return (int64_t)round_size((size_t)n); }

void* gb_pool_alloc(ssize_t size, int device, cudaStream_t stream) {
  if (size <= 0) return nullptr;
  if (device < 0 || device >= kMaxDevices) return nullptr;
  DevicePool& P = g_pools[device];
  const size_t cls = round_size((size_t)size);
  std::lock_guard<std::mutex> lock(P.mu);
  ++P.alloc_count;
  const int cap = P.capturing;
  // (event queries are not allowed while a stream of this thread is capturing)
  if (cap == 0 && !P.pending.empty() && (P.alloc_count % 16) == 0) drain_pending(P);
  if (cap != 0) {
    auto pit = P.priv.find(cap);
    if (pit != P.priv.end()) {
      auto cit = pit->second.find(cls);
      if (cit != pit->second.end() && !cit->second.empty()) {
        Block b = cit->second.back();
        cit->second.pop_back();
        b.stream = stream;
        P.live[b.ptr] = b;
        ++P.cache_hits;
        P.allocated += (int64_t)cls;
        if (P.allocated > P.max_allocated) P.max_allocated = P.allocated;
        return b.ptr;
      }
    }
  }
  auto it = P.bins.find(cls);
  if (it != P.bins.end()) {
    std::vector<Block>& v = it->second;
    for (size_t i = v.size(); i-- > 0;) {
      if (v[i].any_stream || v[i].stream == stream) {
        Block b = v[i];
        v[i] = v.back();
        v.pop_back();
        b.stream = stream;
        b.any_stream = false;
        b.capture = cap;
        P.live[b.ptr] = b;
        ++P.cache_hits;
        P.allocated += (int64_t)cls;
        if (P.allocated > P.max_allocated) P.max_allocated = P.allocated;
        return b.ptr;
      }
    }
  }
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != device) cudaSetDevice(device);
  void* p = nullptr;
  cudaError_t e = cudaErrorMemoryAllocation;
  if (P.limit == 0 || P.reserved + (int64_t)cls <= P.limit) e = cudaMalloc(&p, cls);
  if (e != cudaSuccess) {
    cudaGetLastError();
    ++P.oom_retries;
    drain_pending(P);
    release_cached(P);
    e = cudaMalloc(&p, cls);
    if (e != cudaSuccess) {
      cudaGetLastError();
      p = nullptr;
    }
  }
  if (prev != device) cudaSetDevice(prev);
  if (p == nullptr) return nullptr;
  ++P.cuda_alloc_count;
  P.reserved += (int64_t)cls;
  if (P.reserved > P.max_reserved) P.max_reserved = P.reserved;
  P.allocated += (int64_t)cls;
  if (P.allocated > P.max_allocated) P.max_allocated = P.allocated;
  P.live[p] = Block{p, cls, stream, false, cap};
  return p;
}

void gb_pool_free(void* ptr, ssize_t /*size*/, int device, cudaStream_t stream) {
  if (ptr == nullptr || device < 0 || device >= kMaxDevices) return;
  DevicePool& P = g_pools[device];
  std::lock_guard<std::mutex> lock(P.mu);
  auto it = P.live.find(ptr);
  if (it == P.live.end()) return;
  Block b = it->second;
  P.live.erase(it);
  ++P.free_count;
  P.allocated -= (int64_t)b.size;
  if (b.capture != 0) {
    P.priv[b.capture][b.size].push_back(b);
    return;
  }
  if (stream != b.stream && P.capturing == 0) {
    // used on a different stream than it was allocated on: park behind an event
    cudaEvent_t ev;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess &&
        cudaEventRecord(ev, stream) == cudaSuccess) {
      P.pending.push_back(Pending{b, ev});
      return;
    }
    cudaGetLastError();
  }
  P.bins[b.size].push_back(b);
}

// out[16]: alloc_count, free_count, cache_hits, cuda_alloc_count, small_pool_blocks, large_pool_blocks,
// small_pool_bytes, large_pool_bytes, total_cached_bytes, pending_deallocations, pending_checks,
// allocated_bytes, max_allocated_bytes, reserved_bytes, max_reserved_bytes, oom_retries
void gb_pool_stats(int device, int64_t* out) {
  for (int i = 0; i < 16; ++i) out[i] = 0;
  if (device < 0 || device >= kMaxDevices) return;
  DevicePool& P = g_pools[device];
  std::lock_guard<std::mutex> lock(P.mu);
  int64_t sb = 0, lb = 0, sby = 0, lby = 0;
  for (auto& kv : P.bins) {
    const int64_t n = (int64_t)kv.second.size();
    if (kv.first <= kSmallMax) { sb += n; sby += n * (int64_t)kv.first; }
    else { lb += n; lby += n * (int64_t)kv.first; }
  }
  out[0] = P.alloc_count; out[1] = P.free_count; out[2] = P.cache_hits; out[3] = P.cuda_alloc_count;
  out[4] = sb; out[5] = lb; out[6] = sby; out[7] = lby; out[8] = sby + lby;
  out[9] = (int64_t)P.pending.size(); out[10] = P.pending_checks;
  out[11] = P.allocated; out[12] = P.max_allocated; out[13] = P.reserved; out[14] = P.max_reserved;
  out[15] = P.oom_retries;
}

int64_t gb_pool_empty_cache(int device) {
  if (device < 0 || device >= kMaxDevices) return 0;
  DevicePool& P = g_pools[device];
  std::lock_guard<std::mutex> lock(P.mu);
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != device) cudaSetDevice(device);
  drain_pending(P);
  const int64_t freed = release_cached(P);
  if (prev != device) cudaSetDevice(prev);
  return freed;
}

// Graph capture brackets (see the header comment).  begin returns the id of the new capture, or 0 when another one
// is already in progress on the device (nested captures share the outer id).
int gb_pool_begin_capture(int device) {
  if (device < 0 || device >= kMaxDevices) return 0;
  DevicePool& P = g_pools[device];
  std::lock_guard<std::mutex> lock(P.mu);
  if (P.capturing != 0) return 0;
  P.capturing = ++P.next_capture;
  return P.capturing;
}

void gb_pool_end_capture(int device) {
  if (device < 0 || device >= kMaxDevices) return;
  DevicePool& P = g_pools[device];
  std::lock_guard<std::mutex> lock(P.mu);
  P.capturing = 0;
}

// The graph of capture `id` is gone (and the device idle with respect to it): its private blocks join the common
// bins, live blocks it still owns become ordinary blocks.  Returns the bytes moved to the bins.
int64_t gb_pool_release_capture(int device, int id) {
  if (device < 0 || device >= kMaxDevices || id == 0) return 0;
  DevicePool& P = g_pools[device];
  std::lock_guard<std::mutex> lock(P.mu);
  int64_t moved = 0;
  auto pit = P.priv.find(id);
  if (pit != P.priv.end()) {
    for (auto& kv : pit->second)
      for (Block b : kv.second) {
        b.capture = 0;
        b.any_stream = true;
        P.bins[b.size].push_back(b);
        moved += (int64_t)b.size;
      }
    P.priv.erase(pit);
  }
  for (auto& kv : P.live)
    if (kv.second.capture == id) kv.second.capture = 0;
  return moved;
}

// bytes parked in private free lists of captures
int64_t gb_pool_capture_cached(int device) {
  if (device < 0 || device >= kMaxDevices) return 0;
  DevicePool& P = g_pools[device];
  std::lock_guard<std::mutex> lock(P.mu);
  int64_t n = 0;
  for (auto& c : P.priv)
    for (auto& kv : c.second) n += (int64_t)kv.first * (int64_t)kv.second.size();
  return n;
}

void gb_pool_reset_peak(int device) {
  if (device < 0 || device >= kMaxDevices) return;
  DevicePool& P = g_pools[device];
  std::lock_guard<std::mutex> lock(P.mu);
  P.max_allocated = P.allocated;
  P.max_reserved = P.reserved;
}

void gb_pool_set_limit(int device, int64_t bytes) {
  if (device < 0 || device >= kMaxDevices) return;
  DevicePool& P = g_pools[device];
  std::lock_guard<std::mutex> lock(P.mu);
  P.limit = bytes;
}

}  // extern "C"
