// Norm / RoPE / SwiGLU / GELU kernels for fp16 tensors: the text of norm_act.cu with fp16 element types; every
// entry point carries the suffix _fp16 (msb_rmsnorm_fwd_fp16, ...).  The reference's GPU LayerNorm / GELU kernels are
// instantiated for half in the same way (plugin/device/gpu/kernel/cuda_impl/cuda_ops/layer_norm_impl.cu, gelu_impl.cu).
#define MSB_ELEM_FP16 1
#include "norm_act_impl.cuh"
