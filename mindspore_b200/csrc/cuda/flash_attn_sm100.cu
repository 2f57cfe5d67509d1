// FlashAttention forward for bf16 tensors; the fp16 build of the same text is flash_attn_sm100_fp16.cu.
#include "flash_attn_sm100_impl.cuh"
