// Entry points that allocate nothing: no device or host memory is obtained by the call or by anything it uses.
// This interface has no counterpart in the reference framework, whose kernels receive their workspace from the
// framework's memory pool.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest hidden size msb_rmsnorm_bwd_static accepts: its fp32 scratch is a fixed array of this many elements
// (64 KiB) in device global memory, declared at file scope of the translation unit that defines the function.
#define MSB_RMSNORM_BWD_STATIC_MAX_H 16384

// RMSNorm backward, same arithmetic and same kernels as msb_rmsnorm_bwd, but the fp32 [H] accumulator for the
// weight gradient is the library's own static device array instead of a caller-provided buffer.
//
//   dy, x, w   : bf16 [rows, H], [rows, H], [H];  rstd: fp32 [rows];  dres: optional bf16 [rows, H] added to dx
//   dx         : bf16 [rows, H] out
//   dw_out     : bf16 [H] (dw_fp32 == 0) or fp32 [H] (dw_fp32 != 0); receives the weight gradient, or has it
//                added when accumulate != 0
//   returns 0 on success; 1 for an unsupported H (not a positive multiple of 8); 3 when H exceeds
//   MSB_RMSNORM_BWD_STATIC_MAX_H; 2 when a CUDA call failed.  msb_last_error() gives the message.
//
// Set-up: the first call on each device looks up the device address of the static array once
// (cudaGetSymbolAddress) and keeps it; make that first call outside any stream capture.
// Contents: the array keeps whatever the previous call left in it.  The only part that must start at zero is the
// first H floats, and every call clears exactly those on `stream` (a memset node, not an allocation) before the
// kernel accumulates into them.
// Concurrency: all calls on one device share the one array, so two calls that may overlap in time (different
// streams, or different host threads on different streams) race on it; order them on one stream or with events.
int msb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                           void* dx, void* dw_out, int dw_fp32, int accumulate, long long rows, int H,
                           void* stream);

#ifdef __cplusplus
}
#endif
