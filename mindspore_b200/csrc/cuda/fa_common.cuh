// Shared pieces of the FlashAttention forward / backward kernels: 4-D TMA loads of token-major
// [batch][token][head][128] tensors, the tensor-map encoder for them, and exp2.
#pragma once
#include "host_common.h"
#include "elem.cuh"

namespace msb {
namespace MSB_ELEM_NS {

constexpr int kFaD = 128;  // head dim served by these kernels

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y,
                                            int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Loads a [rows x 128] bf16 tile of head h starting at token t0 as two 128B-swizzled halves
// (d 0..63 at dst, d 64..127 at dst + rows*128 bytes).
__device__ __forceinline__ void fa_load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int rows, int h,
                                             int t0, int b) {
  tma_load_4d(dst, tm, bar, 0, h, t0, b);
  tma_load_4d(dst + rows * 128, tm, bar, 64, h, t0, b);
}

// dims (d, head, token, batch); box = 64 d x 1 head x box_rows tokens x 1 batch, 128-byte swizzle.
static inline int fa_encode_map(CUtensorMap* m, const void* base, int B, int S, int H, long long pitch,
                                int box_rows) {
  typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                         const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                         CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Fn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      set_last_error("cuTensorMapEncodeTiled unavailable");
      return kCudaError;
    }
    fn = reinterpret_cast<Fn>(ptr);
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch * 2) % 16) {
    set_last_error("flash attention: base pointer and token pitch must be 16-byte aligned");
    return kBadArg;
  }
  cuuint64_t dims[4] = {(cuuint64_t)kFaD, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)kFaD * 2, (cuuint64_t)pitch * 2, (cuuint64_t)pitch * 2 * S};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("flash attention: cuTensorMapEncodeTiled failed with %d", (int)r);
    return kCudaError;
  }
  return kOk;
}

// Writes 8 consecutive values of row `row` (16-byte chunk index `ch`) of a K-major 128B-swizzled bf16 tile whose
// 64-column halves are `half_stride` bytes apart.
__device__ __forceinline__ void fa_store_chunk(uint8_t* tile, int row, int ch, int half_stride, const float* v) {
  uint4 o;
  o.x = pack_e2(v[0], v[1]);
  o.y = pack_e2(v[2], v[3]);
  o.z = pack_e2(v[4], v[5]);
  o.w = pack_e2(v[6], v[7]);
  const int half = ch >> 3, cc = ch & 7;
  *reinterpret_cast<uint4*>(tile + half * half_stride + row * 128 + ((cc ^ (row & 7)) << 4)) = o;
}

}  // namespace MSB_ELEM_NS
}  // namespace msb
