// Device memory pool for torch's pluggable-allocator hook: msb_cuda_pool_malloc / msb_cuda_pool_free have the
// signatures torch.cuda.memory.CUDAPluggableAllocator expects and serve every tensor allocation of the process from
// one best-fit pool per device (csrc/host/mem_pool.hpp) over cudaMalloc.  Configure before the first allocation with
// msb_cuda_pool_configure (block size, limit); msb_cuda_pool_stats / _release_idle / _mark_synchronized expose the
// rest.  The reference's GPUMemoryAllocator is the same pairing (plugin/device/gpu/hal/device/gpu_memory_allocator.cc
// over DynamicMemPoolBestFit).
#include "host_common.h"

#include "../host/mem_pool.hpp"

#include <new>

namespace {

constexpr int kMaxDev = 64;
msb::BestFitPool* g_pools[kMaxDev] = {};
std::mutex g_mu;
size_t g_block_size = size_t(1) << 30;
size_t g_max_size = 0;

void* dev_alloc(size_t n) {
  void* p = nullptr;
  if (cudaMalloc(&p, n) != cudaSuccess) {
    cudaGetLastError();          // clear the sticky-less allocation error: the pool reports failure by nullptr
    return nullptr;
  }
  return p;
}
void dev_free(void* p) { cudaFree(p); }

msb::BestFitPool* pool_for(int device) {
  if (device < 0 || device >= kMaxDev) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_pools[device] == nullptr) g_pools[device] = new msb::BestFitPool(g_block_size, g_max_size, dev_alloc, dev_free);
  return g_pools[device];
}

}  // namespace

MSB_EXPORT void msb_cuda_pool_configure(unsigned long long block_size, unsigned long long max_size) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (block_size) g_block_size = block_size;
  g_max_size = max_size;
}

MSB_EXPORT void* msb_cuda_pool_malloc(long long size, int device, void* stream) {
  msb::BestFitPool* pool = pool_for(device);
  if (pool == nullptr) throw std::bad_alloc();
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != device) cudaSetDevice(device);
  void* p = pool->allocate(static_cast<size_t>(size), reinterpret_cast<uint64_t>(stream));
  if (p == nullptr) {
    // out of room: wait for the device, let every stream reuse what is idle, give idle blocks back and retry once
    cudaDeviceSynchronize();
    pool->mark_synchronized();
    pool->release_idle();
    p = pool->allocate(static_cast<size_t>(size), reinterpret_cast<uint64_t>(stream));
  }
  if (prev != device) cudaSetDevice(prev);
  if (p == nullptr) {
    // the hook has no error return and torch does not test the pointer: an exception is the only way to refuse
    // (it travels through torch's C++ frames and surfaces in Python as MemoryError)
    msb::set_last_error("device pool: cannot serve %lld bytes on device %d (limit %zu bytes)", size, device, g_max_size);
    throw std::bad_alloc();
  }
  return p;
}

MSB_EXPORT void msb_cuda_pool_free(void* ptr, long long /*size*/, int device, void* /*stream*/) {
  msb::BestFitPool* pool = pool_for(device);
  if (pool != nullptr && ptr != nullptr) pool->deallocate(ptr);
}

MSB_EXPORT void msb_cuda_pool_mark_synchronized(int device) {
  msb::BestFitPool* pool = pool_for(device);
  if (pool != nullptr) pool->mark_synchronized();
}

MSB_EXPORT unsigned long long msb_cuda_pool_release_idle(int device) {
  msb::BestFitPool* pool = pool_for(device);
  return pool != nullptr ? pool->release_idle() : 0;
}

MSB_EXPORT void msb_cuda_pool_stats(int device, unsigned long long* out) {
  msb::BestFitPool* pool = pool_for(device);
  if (pool == nullptr) return;
  const msb::BestFitPool::Stats s = pool->stats();
  out[0] = s.used; out[1] = s.reserved; out[2] = s.peak_used; out[3] = s.peak_reserved;
  out[4] = s.blocks; out[5] = s.largest_idle; out[6] = s.idle_bufs;
}
