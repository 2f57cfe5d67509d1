// BatchNorm / pooling kernels for fp16 tensors: the text of bn_pool.cu with fp16 element types; every entry point carries the
// suffix _fp16.
#define MSB_ELEM_FP16 1
#include "bn_pool_impl.cuh"
