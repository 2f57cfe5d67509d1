// Host-side helpers shared by the kernel launchers: error reporting, SM count,
// and TMA tensor-map encoding through the driver entry point (looked up at run
// time so the library links without libcuda on a machine that has no driver).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define MSB_EXPORT extern "C" __attribute__((visibility("default")))

namespace msb {

// Return codes of every exported launcher.
enum : int {
  kOk = 0,
  kBadArg = 1,       // unsupported shape / alignment (nothing was launched)
  kCudaError = 2,    // a CUDA runtime/driver call failed
  kTooLarge = 3,     // request beyond a fixed capacity
};

void set_last_error(const char* fmt, ...);
int sm_count();
// Device address of this device's status word (see AbortCtx in ptx.cuh); nullptr on failure.
int* status_ptr();

// Encodes a rank-3 bf16/fp32 tiled tensor map with 128-byte swizzle.
//   dims    : extents, innermost first
//   strides : byte strides of dims 1 and 2 (dim 0 is contiguous)
//   box     : tile extents, innermost first; box[0]*elem_size must be 128 bytes
int encode_tmap_3d(CUtensorMap* out, const void* base, int elem_size, uint64_t d0, uint64_t d1, uint64_t d2,
                   uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                   bool swizzle128 = true);

// Rank-4 bf16 tiled tensor map with 128-byte swizzle (NHWC activations: channels, width, height, image).
//   dims / box innermost first; strides_bytes are the byte strides of dims 1..3; box[0] must be 64 elements.
int encode_tmap_4d(CUtensorMap* out, const void* base, const uint64_t dims[4], const uint64_t strides_bytes[3],
                   const uint32_t box[4]);

}  // namespace msb

#define MSB_CUDA_CHECK(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      msb::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return msb::kCudaError;                                                             \
    }                                                                                     \
  } while (0)
