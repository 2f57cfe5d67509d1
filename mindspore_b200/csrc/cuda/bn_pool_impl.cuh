// BatchNorm (training and inference), ReLU, residual add and pooling for NHWC bf16 activations.
//
// Forward in training: the convolution epilogue (conv_sm100.cu) or msb_channel_stats has left per-channel
// sum / sum-of-squares; msb_bn_finalize turns them into scale = gamma * rstd and shift = beta - mean * scale and
// updates the moving statistics; msb_bn_apply is one pass  y = relu(x * scale + shift (+ residual)).
// Backward: msb_bn_bwd_reduce (sum dy', sum dy' * xhat with the ReLU mask taken from y) and msb_bn_bwd_apply
// (dx, and the masked gradient for the residual branch), two passes over the activation in total.
// The reference runs cudnnBatchNormalizationForwardTrainingEx / BackwardEx with a fused activation
// (plugin/device/gpu/kernel/nn/batch_norm_gpu_kernel.cc:62, batch_norm_grad_gpu_kernel.cc) and cuDNN pooling
// (pooling_gpu_kernel.h).
//
// This text is compiled twice: for bf16 tensors (bn_pool.cu), and with MSB_ELEM_FP16 defined for fp16 tensors
// (bn_pool_fp16.cu), where every entry point carries the suffix _fp16 and "bf16" in a comment reads "fp16".
#include "host_common.h"
#include "elem.cuh"

namespace msb {
namespace MSB_ELEM_NS {

constexpr int kEwThreads = 256;

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const elem2_t* h = reinterpret_cast<const elem2_t*>(&raw);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 t = e2_to_f2(h[q]);
    f[2 * q] = t.x;
    f[2 * q + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_e2(f[0], f[1]);
  o.y = pack_e2(f[2], f[3]);
  o.z = pack_e2(f[4], f[5]);
  o.w = pack_e2(f[6], f[7]);
  return o;
}

// Column sums over rows of a [rows, C] matrix.  MODE 0: (x, x^2).  MODE 1: (dy', dy' * xhat) with
// dy' = dy masked by y > 0 when relu, xhat = (x - mean) * rstd.  Threads of a block tile (rows_per_iter x C/8).
template <int MODE>
__global__ void __launch_bounds__(kEwThreads)
column_reduce_kernel(const elem_t* __restrict__ a, const elem_t* __restrict__ x,
                     const elem_t* __restrict__ y, const float* __restrict__ mean,
                     const float* __restrict__ rstd, float* __restrict__ out, long long rows, int C, int relu) {
  extern __shared__ float red[];   // [2][rows_per_iter][C] would be too big: reduce through atomics on [2][C]
  const int vecs = C / 8;
  const int rows_per_iter = kEwThreads / vecs;
  const int lr = threadIdx.x / vecs, lc = threadIdx.x % vecs;
  for (int i = threadIdx.x; i < 2 * C; i += kEwThreads) red[i] = 0.f;
  __syncthreads();
  float s1[8] = {0, 0, 0, 0, 0, 0, 0, 0}, s2[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float mu[8], rs[8];
  if (MODE == 1 && lr < rows_per_iter) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mu[j] = mean[lc * 8 + j];
      rs[j] = rstd[lc * 8 + j];
    }
  }
  if (lr < rows_per_iter) {
    for (long long r = (long long)blockIdx.x * rows_per_iter + lr; r < rows; r += (long long)gridDim.x * rows_per_iter) {
      float av[8];
      unpack8(reinterpret_cast<const uint4*>(a + r * C)[lc], av);
      if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s1[j] += av[j];
          s2[j] += av[j] * av[j];
        }
      } else {
        float xv[8];
        unpack8(reinterpret_cast<const uint4*>(x + r * C)[lc], xv);
        if (relu) {
          float yv[8];
          unpack8(reinterpret_cast<const uint4*>(y + r * C)[lc], yv);
#pragma unroll
          for (int j = 0; j < 8; ++j) av[j] = yv[j] > 0.f ? av[j] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s1[j] += av[j];
          s2[j] += av[j] * (xv[j] - mu[j]) * rs[j];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      atomicAdd(&red[lc * 8 + j], s1[j]);
      atomicAdd(&red[C + lc * 8 + j], s2[j]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * C; i += kEwThreads) atomicAdd(out + i, red[i]);
}

// stats: [2C] sums.  Writes scale/shift (and mean/rstd for backward); updates the moving statistics
// moving = momentum * moving + (1 - momentum) * batch  (variance unbiased), as nn.BatchNorm2d does.
__global__ void bn_finalize_kernel(const float* __restrict__ stats, const float* __restrict__ gamma,
                                   const float* __restrict__ beta, float* __restrict__ moving_mean,
                                   float* __restrict__ moving_var, float* __restrict__ scale,
                                   float* __restrict__ shift, float* __restrict__ mean_out,
                                   float* __restrict__ rstd_out, int C, float count, float momentum, float eps,
                                   int training) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float mean, var;
  if (training) {
    mean = stats[c] / count;
    var = fmaxf(stats[C + c] / count - mean * mean, 0.f);
    if (moving_mean) {
      moving_mean[c] = momentum * moving_mean[c] + (1.f - momentum) * mean;
      moving_var[c] = momentum * moving_var[c] + (1.f - momentum) * var * (count > 1.f ? count / (count - 1.f) : 1.f);
    }
  } else {
    mean = moving_mean[c];
    var = moving_var[c];
  }
  const float r = rsqrtf(var + eps);
  const float sc = gamma[c] * r;
  scale[c] = sc;
  shift[c] = beta[c] - mean * sc;
  if (mean_out) {
    mean_out[c] = mean;
    rstd_out[c] = r;
  }
}

__global__ void __launch_bounds__(kEwThreads)
bn_apply_kernel(const elem_t* __restrict__ x, const float* __restrict__ scale, const float* __restrict__ shift,
                const elem_t* __restrict__ residual, elem_t* __restrict__ y, long long total_vecs,
                int vecs, int relu) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total_vecs;
       i += (long long)gridDim.x * blockDim.x) {
    const int c0 = (int)(i % vecs) * 8;
    float v[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], v);
    const float4 sa = *reinterpret_cast<const float4*>(scale + c0), sb = *reinterpret_cast<const float4*>(scale + c0 + 4);
    const float4 ha = *reinterpret_cast<const float4*>(shift + c0), hb = *reinterpret_cast<const float4*>(shift + c0 + 4);
    const float sc[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
    const float sh[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = v[j] * sc[j] + sh[j];
    if (residual) {
      float rv[8];
      unpack8(reinterpret_cast<const uint4*>(residual)[i], rv);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += rv[j];
    }
    if (relu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.f);
    }
    reinterpret_cast<uint4*>(y)[i] = pack8(v);
  }
}

// dx = gamma * rstd * (dy' - sum(dy')/count - xhat * sum(dy' xhat)/count) = A[c] * dy' + B[c] * x + D[c];
// dres = dy' (optional).  coef = [A | B | D], each C floats.
__global__ void bn_bwd_coeff_kernel(const float* __restrict__ gamma, const float* __restrict__ mean,
                                    const float* __restrict__ rstd, const float* __restrict__ sums,
                                    float* __restrict__ coef, int C, float inv_count) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float g = gamma[c], r = rstd[c], mu = mean[c];
  const float s1 = sums[c] * inv_count, s2 = sums[C + c] * inv_count;
  coef[c] = g * r;
  coef[C + c] = -g * r * r * s2;
  coef[2 * C + c] = -g * r * s1 + g * r * r * s2 * mu;
}

__global__ void __launch_bounds__(kEwThreads)
bn_bwd_apply_kernel(const elem_t* __restrict__ dy, const elem_t* __restrict__ x,
                    const elem_t* __restrict__ y, const float* __restrict__ coef,
                    elem_t* __restrict__ dx, elem_t* __restrict__ dres, long long total_vecs, int vecs,
                    int C, int relu) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total_vecs;
       i += (long long)gridDim.x * blockDim.x) {
    const int c0 = (int)(i % vecs) * 8;
    float g[8], xv[8];
    unpack8(reinterpret_cast<const uint4*>(dy)[i], g);
    unpack8(reinterpret_cast<const uint4*>(x)[i], xv);
    if (relu) {
      float yv[8];
      unpack8(reinterpret_cast<const uint4*>(y)[i], yv);
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = yv[j] > 0.f ? g[j] : 0.f;
    }
    if (dres) reinterpret_cast<uint4*>(dres)[i] = pack8(g);
    float ca[8], cb[8], cd[8];
    *reinterpret_cast<float4*>(ca) = *reinterpret_cast<const float4*>(coef + c0);
    *reinterpret_cast<float4*>(ca + 4) = *reinterpret_cast<const float4*>(coef + c0 + 4);
    *reinterpret_cast<float4*>(cb) = *reinterpret_cast<const float4*>(coef + C + c0);
    *reinterpret_cast<float4*>(cb + 4) = *reinterpret_cast<const float4*>(coef + C + c0 + 4);
    *reinterpret_cast<float4*>(cd) = *reinterpret_cast<const float4*>(coef + 2 * C + c0);
    *reinterpret_cast<float4*>(cd + 4) = *reinterpret_cast<const float4*>(coef + 2 * C + c0 + 4);
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = ca[j] * g[j] + cb[j] * xv[j] + cd[j];
    reinterpret_cast<uint4*>(dx)[i] = pack8(o);
  }
}

// 3x3 / stride 2 / pad 1 max pooling, NHWC.  The forward pass also records, per output element, which of the nine
// window positions (r*3 + s, first maximum in scan order) won; the backward pass routes dy by that record.
__global__ void __launch_bounds__(kEwThreads)
maxpool3x3s2_fwd_kernel(const elem_t* __restrict__ x, elem_t* __restrict__ y,
                        unsigned long long* __restrict__ idx, int N, int H, int W, int C, int Ho, int Wo) {
  const int vecs = C / 8;
  const long long total = (long long)N * Ho * Wo * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int cv = (int)(i % vecs);
    long long pix = i / vecs;
    const int wo = (int)(pix % Wo);
    pix /= Wo;
    const int ho = (int)(pix % Ho);
    const int n = (int)(pix / Ho);
    float m[8];
    unsigned long long win = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) m[j] = -INFINITY;
    for (int r = 0; r < 3; ++r) {
      const int h = ho * 2 - 1 + r;
      if (h < 0 || h >= H) continue;
      for (int s = 0; s < 3; ++s) {
        const int w = wo * 2 - 1 + s;
        if (w < 0 || w >= W) continue;
        float v[8];
        unpack8(reinterpret_cast<const uint4*>(x + (((long long)n * H + h) * W + w) * C)[cv], v);
        const unsigned long long pos = (unsigned long long)(r * 3 + s);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (v[j] > m[j]) {
            m[j] = v[j];
            win = (win & ~(0xffull << (8 * j))) | (pos << (8 * j));
          }
        }
      }
    }
    reinterpret_cast<uint4*>(y)[i] = pack8(m);
    if (idx) idx[i] = win;
  }
}

__global__ void __launch_bounds__(kEwThreads)
maxpool3x3s2_bwd_kernel(const unsigned long long* __restrict__ idx, const elem_t* __restrict__ dy,
                        elem_t* __restrict__ dx, int N, int H, int W, int C, int Ho, int Wo) {
  const int vecs = C / 8;
  const long long total = (long long)N * H * W * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int cv = (int)(i % vecs);
    long long pix = i / vecs;
    const int w = (int)(pix % W);
    pix /= W;
    const int h = (int)(pix % H);
    const int n = (int)(pix / H);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int ho = h / 2; ho <= (h + 1) / 2; ++ho) {        // windows with ho*2-1 <= h <= ho*2+1
      if (ho >= Ho) continue;
      for (int wo = w / 2; wo <= (w + 1) / 2; ++wo) {
        if (wo >= Wo) continue;
        const unsigned long long pos = (unsigned long long)((h - (ho * 2 - 1)) * 3 + (w - (wo * 2 - 1)));
        const long long o = (((long long)n * Ho + ho) * Wo + wo) * vecs + cv;
        const unsigned long long win = idx[o];
        float g[8];
        unpack8(reinterpret_cast<const uint4*>(dy)[o], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += (((win >> (8 * j)) & 0xffull) == pos) ? g[j] : 0.f;
      }
    }
    reinterpret_cast<uint4*>(dx)[i] = pack8(acc);
  }
}

// Global average pooling [N, HW, C] -> [N, C] and its gradient.
__global__ void avgpool_fwd_kernel(const elem_t* __restrict__ x, elem_t* __restrict__ y, int N, int HW,
                                   int C) {
  const int vecs = C / 8;
  const long long total = (long long)N * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int cv = (int)(i % vecs);
    const int n = (int)(i / vecs);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < HW; ++p) {
      float v[8];
      unpack8(reinterpret_cast<const uint4*>(x + ((long long)n * HW + p) * C)[cv], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] /= (float)HW;
    reinterpret_cast<uint4*>(y)[i] = pack8(acc);
  }
}
__global__ void avgpool_bwd_kernel(const elem_t* __restrict__ dy, elem_t* __restrict__ dx, int N, int HW,
                                   int C) {
  const int vecs = C / 8;
  const long long total = (long long)N * HW * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int cv = (int)(i % vecs);
    const int n = (int)(i / ((long long)HW * vecs));
    float v[8];
    unpack8(reinterpret_cast<const uint4*>(dy + (long long)n * C)[cv], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] /= (float)HW;
    reinterpret_cast<uint4*>(dx)[i] = pack8(v);
  }
}

static unsigned ew_grid(long long work) {
  long long b = (work + kEwThreads - 1) / kEwThreads;
  const long long cap = (long long)sm_count() * 8;
  b = b < 1 ? 1 : (b > cap ? cap : b);
  return (unsigned)b;
}

static int check_c(const char* what, int C) {
  if (C <= 0 || (C % 8) || C > 2048) {
    set_last_error("%s: channels %d must be a multiple of 8 in (0, 2048]", what, C);
    return kBadArg;
  }
  return kOk;
}

}  // namespace MSB_ELEM_NS
}  // namespace msb

using namespace msb;
using namespace msb::MSB_ELEM_NS;

// out[2C] += (sum x, sum x^2) over rows.
MSB_EXPORT int MSB_FN(msb_channel_stats)(const void* x, float* out, long long rows, int C, void* stream) {
  if (int rc = check_c("channel_stats", C)) return rc;
  if (rows <= 0) return kOk;
  const int rpi = kEwThreads / (C / 8);
  long long blocks = (rows + rpi - 1) / rpi;
  const long long cap = (long long)sm_count() * 4;
  blocks = blocks > cap ? cap : blocks;
  column_reduce_kernel<0><<<(unsigned)blocks, kEwThreads, 2 * C * sizeof(float), (cudaStream_t)stream>>>(
      (const elem_t*)x, nullptr, nullptr, nullptr, nullptr, out, rows, C, 0);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int MSB_FN(msb_bn_finalize)(const float* stats, const float* gamma, const float* beta, float* moving_mean,
                               float* moving_var, float* scale, float* shift, float* mean_out, float* rstd_out, int C,
                               float count, float momentum, float eps, int training, void* stream) {
  if (int rc = check_c("bn_finalize", C)) return rc;
  bn_finalize_kernel<<<(C + 127) / 128, 128, 0, (cudaStream_t)stream>>>(stats, gamma, beta, moving_mean, moving_var,
                                                                         scale, shift, mean_out, rstd_out, C, count,
                                                                         momentum, eps, training);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int MSB_FN(msb_bn_apply)(const void* x, const float* scale, const float* shift, const void* residual, void* y,
                            long long rows, int C, int relu, void* stream) {
  if (int rc = check_c("bn_apply", C)) return rc;
  if (rows <= 0) return kOk;
  const long long tv = rows * (C / 8);
  bn_apply_kernel<<<ew_grid(tv), kEwThreads, 0, (cudaStream_t)stream>>>(
      (const elem_t*)x, scale, shift, (const elem_t*)residual, (elem_t*)y, tv, C / 8, relu);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// sums[2C] += (sum dy', sum dy' xhat)
MSB_EXPORT int MSB_FN(msb_bn_bwd_reduce)(const void* dy, const void* x, const void* y, const float* mean, const float* rstd,
                                 float* sums, long long rows, int C, int relu, void* stream) {
  if (int rc = check_c("bn_bwd_reduce", C)) return rc;
  if (rows <= 0) return kOk;
  const int rpi = kEwThreads / (C / 8);
  long long blocks = (rows + rpi - 1) / rpi;
  const long long cap = (long long)sm_count() * 4;
  blocks = blocks > cap ? cap : blocks;
  column_reduce_kernel<1><<<(unsigned)blocks, kEwThreads, 2 * C * sizeof(float), (cudaStream_t)stream>>>(
      (const elem_t*)dy, (const elem_t*)x, (const elem_t*)y, mean, rstd, sums, rows, C, relu);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// coef: fp32 [3C] scratch owned by the caller (filled here).
MSB_EXPORT int MSB_FN(msb_bn_bwd_apply)(const void* dy, const void* x, const void* y, const float* gamma, const float* mean,
                                const float* rstd, const float* sums, float* coef, void* dx, void* dres,
                                long long rows, int C, int relu, void* stream) {
  if (int rc = check_c("bn_bwd_apply", C)) return rc;
  if (rows <= 0) return kOk;
  bn_bwd_coeff_kernel<<<(C + 127) / 128, 128, 0, (cudaStream_t)stream>>>(gamma, mean, rstd, sums, coef, C,
                                                                         1.f / (float)rows);
  const long long tv = rows * (C / 8);
  bn_bwd_apply_kernel<<<ew_grid(tv), kEwThreads, 0, (cudaStream_t)stream>>>(
      (const elem_t*)dy, (const elem_t*)x, (const elem_t*)y, coef, (elem_t*)dx,
      (elem_t*)dres, tv, C / 8, C, relu);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// Forward: x -> out (and idx: one byte per output element, 8-byte aligned, may be null).
// Backward: idx + dy -> out = dx.
MSB_EXPORT int MSB_FN(msb_maxpool3x3s2)(const void* x, const void* dy, void* out, void* idx, int N, int H, int W, int C,
                                int backward, void* stream) {
  if (int rc = check_c("maxpool", C)) return rc;
  const int Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
  if (!backward) {
    maxpool3x3s2_fwd_kernel<<<ew_grid((long long)N * Ho * Wo * (C / 8)), kEwThreads, 0, (cudaStream_t)stream>>>(
        (const elem_t*)x, (elem_t*)out, (unsigned long long*)idx, N, H, W, C, Ho, Wo);
  } else {
    if (!idx) { set_last_error("maxpool backward needs the index record of the forward pass"); return kBadArg; }
    maxpool3x3s2_bwd_kernel<<<ew_grid((long long)N * H * W * (C / 8)), kEwThreads, 0, (cudaStream_t)stream>>>(
        (const unsigned long long*)idx, (const elem_t*)dy, (elem_t*)out, N, H, W, C, Ho, Wo);
  }
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int MSB_FN(msb_global_avgpool)(const void* in, void* out, int N, int HW, int C, int backward, void* stream) {
  if (int rc = check_c("global_avgpool", C)) return rc;
  if (!backward) {
    avgpool_fwd_kernel<<<ew_grid((long long)N * (C / 8)), kEwThreads, 0, (cudaStream_t)stream>>>(
        (const elem_t*)in, (elem_t*)out, N, HW, C);
  } else {
    avgpool_bwd_kernel<<<ew_grid((long long)N * HW * (C / 8)), kEwThreads, 0, (cudaStream_t)stream>>>(
        (const elem_t*)in, (elem_t*)out, N, HW, C);
  }
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
