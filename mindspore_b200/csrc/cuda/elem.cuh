// Element type of a translation unit whose text is compiled once per 16-bit float type.
//
// A kernel file that works on "the 16-bit tensor type" writes elem_t / elem2_t and the helpers below instead of
// __nv_bfloat16 and its intrinsics, wraps its exported names in MSB_FN(...), and keeps its device code inside
// namespace msb::MSB_ELEM_NS.  Compiled as is, it is the bf16 build; compiled with MSB_ELEM_FP16 defined (the
// *_fp16.cu files do that and include the text), it is the fp16 build and every entry point carries the suffix _fp16.
#pragma once
#include "ptx.cuh"

#ifdef MSB_ELEM_FP16
#define MSB_FN(name) name##_fp16
#define MSB_ELEM_NS fp16v
#else
#define MSB_FN(name) name
#define MSB_ELEM_NS bf16v
#endif

namespace msb {
namespace MSB_ELEM_NS {

#ifdef MSB_ELEM_FP16
using elem_t = __half;
using elem2_t = __half2;
constexpr bool kElemFp16 = true;
__device__ __forceinline__ float e_to_f(elem_t v) { return __half2float(v); }
__device__ __forceinline__ elem_t f_to_e(float v) { return __float2half_rn(v); }
__device__ __forceinline__ float2 e2_to_f2(elem2_t v) { return __half22float2(v); }
__device__ __forceinline__ elem2_t f2_to_e2(float a, float b) { return __floats2half2_rn(a, b); }
#else
using elem_t = __nv_bfloat16;
using elem2_t = __nv_bfloat162;
constexpr bool kElemFp16 = false;
__device__ __forceinline__ float e_to_f(elem_t v) { return __bfloat162float(v); }
__device__ __forceinline__ elem_t f_to_e(float v) { return __float2bfloat16(v); }
__device__ __forceinline__ float2 e2_to_f2(elem2_t v) { return __bfloat1622float2(v); }
__device__ __forceinline__ elem2_t f2_to_e2(float a, float b) { return __floats2bfloat162_rn(a, b); }
#endif

// Two fp32 values rounded to the element type, packed into 32 bits (low half first).
__device__ __forceinline__ uint32_t pack_e2(float lo, float hi) {
  elem2_t v = f2_to_e2(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// tcgen05 instruction descriptor for elem x elem -> fp32.
__host__ __device__ constexpr uint32_t umma_idesc_elem(int m, int n, bool a_mn_major, bool b_mn_major) {
  return kElemFp16 ? umma_idesc_f16(m, n, a_mn_major, b_mn_major) : umma_idesc_bf16(m, n, a_mn_major, b_mn_major);
}

}  // namespace MSB_ELEM_NS
}  // namespace msb
