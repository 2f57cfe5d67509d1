// FlashAttention forward for fp16 tensors: the text of flash_attn_sm100.cu with fp16 element types; every entry point carries the
// suffix _fp16.
#define MSB_ELEM_FP16 1
#include "flash_attn_sm100_impl.cuh"
