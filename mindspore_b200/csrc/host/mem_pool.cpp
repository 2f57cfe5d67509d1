// C interface of the best-fit pool over the C heap: the pool logic (mem_pool.hpp) is exercised on a CPU through
// these entry points; the device pool (csrc/cuda/pool_alloc.cu) wraps the same class around cudaMalloc.
#include "mem_pool.hpp"

#include <cstdlib>

#define MSB_API extern "C" __attribute__((visibility("default")))

namespace {
void* heap_alloc(size_t n) { return std::malloc(n); }
void heap_free(void* p) { std::free(p); }
}  // namespace

MSB_API void* msb_pool_create(unsigned long long block_size, unsigned long long max_size) {
  return new msb::BestFitPool(block_size, max_size, heap_alloc, heap_free);
}

MSB_API void msb_pool_destroy(void* pool) { delete static_cast<msb::BestFitPool*>(pool); }

MSB_API void* msb_pool_alloc(void* pool, unsigned long long size, unsigned long long stream) {
  return static_cast<msb::BestFitPool*>(pool)->allocate(size, stream);
}

MSB_API unsigned long long msb_pool_free(void* pool, void* ptr) {
  return static_cast<msb::BestFitPool*>(pool)->deallocate(ptr);
}

MSB_API void msb_pool_mark_synchronized(void* pool) { static_cast<msb::BestFitPool*>(pool)->mark_synchronized(); }

MSB_API unsigned long long msb_pool_release_idle(void* pool) {
  return static_cast<msb::BestFitPool*>(pool)->release_idle();
}

// out: used, reserved, peak_used, peak_reserved, blocks, largest_idle, idle_bufs
MSB_API void msb_pool_stats(void* pool, unsigned long long* out) {
  const msb::BestFitPool::Stats s = static_cast<msb::BestFitPool*>(pool)->stats();
  out[0] = s.used; out[1] = s.reserved; out[2] = s.peak_used; out[3] = s.peak_reserved;
  out[4] = s.blocks; out[5] = s.largest_idle; out[6] = s.idle_bufs;
}
