#include "host_common.h"

#include <mutex>
#include <stdarg.h>
#include <string.h>

#include "ptx.cuh"

namespace msb {

__device__ int g_msb_status = 0;

int* status_ptr() {
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_msb_status) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}

static thread_local char g_last_error[512] = {0};

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

int encode_tmap_3d(CUtensorMap* out, const void* base, int elem_size, uint64_t d0, uint64_t d1, uint64_t d2,
                   uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                   bool swizzle128) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled is not available from the driver");
    return kCudaError;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (stride1_bytes & 15) != 0 || (stride2_bytes & 15) != 0) {
    set_last_error("tensor map needs a 16-byte aligned base and strides (base=%p s1=%llu s2=%llu)", base,
                   (unsigned long long)stride1_bytes, (unsigned long long)stride2_bytes);
    return kBadArg;
  }
  CUtensorMapDataType dt = elem_size == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed with %d (dims %llu,%llu,%llu strides %llu,%llu box %u,%u,%u)",
                   (int)r, (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2,
                   (unsigned long long)stride1_bytes, (unsigned long long)stride2_bytes, b0, b1, b2);
    return kCudaError;
  }
  return kOk;
}

int encode_tmap_4d(CUtensorMap* out, const void* base, const uint64_t dims[4], const uint64_t strides_bytes[3],
                   const uint32_t box[4]) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled is not available from the driver");
    return kCudaError;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (strides_bytes[0] & 15) || (strides_bytes[1] & 15) ||
      (strides_bytes[2] & 15)) {
    set_last_error("4-D tensor map needs a 16-byte aligned base and strides (base=%p)", base);
    return kBadArg;
  }
  cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t st[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t b[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), d, st, b, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled (4-D) failed with %d (dims %llu,%llu,%llu,%llu box %u,%u,%u,%u)", (int)r,
                   (unsigned long long)d[0], (unsigned long long)d[1], (unsigned long long)d[2],
                   (unsigned long long)d[3], b[0], b[1], b[2], b[3]);
    return kCudaError;
  }
  return kOk;
}

}  // namespace msb

MSB_EXPORT const char* msb_last_error() { return msb::g_last_error; }

// Reads and clears the device status word (synchronises the device).
MSB_EXPORT int msb_read_status(int clear) {
  int h = 0;
  if (cudaMemcpyFromSymbol(&h, msb::g_msb_status, sizeof(int)) != cudaSuccess) return -1;
  if (clear && h != 0) {
    int z = 0;
    cudaMemcpyToSymbol(msb::g_msb_status, &z, sizeof(int));
  }
  return h;
}
