// Norm / RoPE / SwiGLU / GELU kernels for bf16 tensors; the fp16 build of the same text is norm_act_fp16.cu.
#include "norm_act_impl.cuh"
