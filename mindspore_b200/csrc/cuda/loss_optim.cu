// Softmax-cross-entropy (one pass for statistics, one for the gradient, vocab-parallel capable),
// flat-arena optimizers (AdamW, Momentum), gradient statistics (sum of squares + finite check),
// embedding gather / scatter-add and dtype casts, for sm_100a.
//
// Reference counterparts: cuDNN softmax + cross_entropy_impl.cu:104-123 and the serial
// <<<1,1>>> sparse variant (sparse_cross_entropy_cuda_impl.cu:57); adam_impl.cu:100-109
// (AdamWeightDecay), momentum_impl.cu:253-280 (CombineMomentum), float_status_impl.cu:299-314,
// square_sum_all_impl.cu:86, embedding_lookup_impl.cu:46, cast_all_impl.cu:35, all under
// plugin/device/gpu/kernel/cuda_impl/cuda_ops/.
#include "host_common.h"
#include "ptx.cuh"

namespace msb {

constexpr int kCeThreads = 512;

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float nm = fmaxf(m, m2);
  if (nm == -INFINITY) { m = nm; s = 0.f; return; }
  s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  m = nm;
}

// Per-row statistics over this rank's vocabulary slice [vocab_start, vocab_start+V):
//   stats[row] = {max, sum exp(l - max), logit[label] if label in slice else 0}
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_stats_kernel(const T* __restrict__ logits, const int* __restrict__ labels, float* __restrict__ stats,
                int V, long long pitch, int vocab_start) {
  __shared__ float sm[kCeThreads / 32], ss[kCeThreads / 32];
  const long long row = blockIdx.x;
  const T* lr = logits + row * pitch;
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x; c < V; c += kCeThreads) {
    const float v = to_f<T>(lr[c]);
    if (v > m) { s = s * __expf(m - v) + 1.f; m = v; } else { s += __expf(v - m); }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sm[warp] = m; ss[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    m = lane < kCeThreads / 32 ? sm[lane] : -INFINITY;
    s = lane < kCeThreads / 32 ? ss[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_merge(m, s, m2, s2);
    }
    if (lane == 0) {
      const int lab = labels[row] - vocab_start;
      stats[row * 3 + 0] = m;
      stats[row * 3 + 1] = s;
      stats[row * 3 + 2] = (lab >= 0 && lab < V) ? to_f<T>(lr[lab]) : 0.f;
    }
  }
}

// Given (possibly cross-rank combined) stats, writes loss[row] = log(sum) + max - target (0 for ignored
// rows) and, if dlogits != nullptr, dlogits = (softmax - onehot) * grad_scale[0] * (row valid).
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_grad_kernel(const T* __restrict__ logits, const int* __restrict__ labels, const float* __restrict__ stats,
               float* __restrict__ loss, T* __restrict__ dlogits, const float* __restrict__ grad_scale, int V,
               long long pitch, int vocab_start, int ignore_index, int write_loss) {
  const long long row = blockIdx.x;
  const float m = stats[row * 3 + 0], s = stats[row * 3 + 1], tgt = stats[row * 3 + 2];
  const int label = labels[row];
  const bool valid = label != ignore_index;
  if (threadIdx.x == 0 && write_loss) loss[row] = valid ? (__logf(s) + m - tgt) : 0.f;
  if (!dlogits) return;
  const float scale = valid ? grad_scale[0] : 0.f;
  const float inv = 1.f / s;
  const int lab = label - vocab_start;
  const T* lr = logits + row * pitch;
  T* dr = dlogits + row * pitch;
  for (int c = threadIdx.x; c < V; c += kCeThreads) {
    float g = __expf(to_f<T>(lr[c]) - m) * inv;
    if (c == lab) g -= 1.f;
    g *= scale;
    if constexpr (sizeof(T) == 2) dr[c] = __float2bfloat16(g); else dr[c] = g;
  }
}

// ------------------------------------------------------------------------------------ optimizers
// Flat-arena AdamW step.  `grad` is fp32 or bf16.  hyper (device, fp32[8]):
//   {lr, beta1, beta2, eps, weight_decay, 1-beta1^t, 1-beta2^t, grad_scale}
// skip (device int): non-zero leaves everything untouched (overflow step).
template <typename G>
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ grad, __nv_bfloat16* __restrict__ param_lp, long long n,
                             const float* __restrict__ hyper, const int* __restrict__ skip) {
  if (skip && *skip) return;
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4];
  const float bc1 = hyper[5], bc2 = hyper[6], gs = hyper[7];
  const float step = lr / bc1;
  const float rsq_bc2 = rsqrtf(bc2);
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      float4 p4 = *reinterpret_cast<float4*>(master + i);
      float4 m4 = *reinterpret_cast<float4*>(m + i);
      float4 v4 = *reinterpret_cast<float4*>(v + i);
      float g[4];
      if constexpr (sizeof(G) == 4) {
        const float4 g4 = *reinterpret_cast<const float4*>(grad + i);
        g[0] = g4.x; g[1] = g4.y; g[2] = g4.z; g[3] = g4.w;
      } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(grad + i);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
      }
      float* pp = reinterpret_cast<float*>(&p4);
      float* mm = reinterpret_cast<float*>(&m4);
      float* vv = reinterpret_cast<float*>(&v4);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = g[j] * gs;
        mm[j] = b1 * mm[j] + (1.f - b1) * gj;
        vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
        const float denom = sqrtf(vv[j]) * rsq_bc2 + eps;
        pp[j] = pp[j] * (1.f - lr * wd) - step * mm[j] / denom;
      }
      *reinterpret_cast<float4*>(master + i) = p4;
      *reinterpret_cast<float4*>(m + i) = m4;
      *reinterpret_cast<float4*>(v + i) = v4;
      if (param_lp) {
        uint2 o;
        o.x = pack_bf16x2(pp[0], pp[1]);
        o.y = pack_bf16x2(pp[2], pp[3]);
        *reinterpret_cast<uint2*>(param_lp + i) = o;
      }
    } else {
      for (long long k = i; k < n; ++k) {
        const float gj = to_f<G>(grad[k]) * gs;
        const float mk = b1 * m[k] + (1.f - b1) * gj;
        const float vk = b2 * v[k] + (1.f - b2) * gj * gj;
        m[k] = mk; v[k] = vk;
        const float pk = master[k] * (1.f - lr * wd) - step * mk / (sqrtf(vk) * rsq_bc2 + eps);
        master[k] = pk;
        if (param_lp) param_lp[k] = __float2bfloat16(pk);
      }
    }
  }
}

// Momentum SGD (reference semantics of ApplyMomentum): accum = accum*mom + g ; p -= lr*accum
// (use_nesterov: p -= lr*(g + mom*accum)).  hyper: {lr, momentum, weight_decay, grad_scale, nesterov}
template <typename G>
__global__ void momentum_kernel(float* __restrict__ master, float* __restrict__ accum, const G* __restrict__ grad,
                                __nv_bfloat16* __restrict__ param_lp, long long n, const float* __restrict__ hyper,
                                const int* __restrict__ skip) {
  if (skip && *skip) return;
  const float lr = hyper[0], mom = hyper[1], wd = hyper[2], gs = hyper[3];
  const bool nesterov = hyper[4] != 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float p = master[i];
    const float g = to_f<G>(grad[i]) * gs + wd * p;
    const float a = accum[i] * mom + g;
    accum[i] = a;
    const float np = nesterov ? p - lr * (g + mom * a) : p - lr * a;
    master[i] = np;
    if (param_lp) param_lp[i] = __float2bfloat16(np);
  }
}

// out[0] += sum(x^2) ; flag |= any non-finite
template <typename T>
__global__ void sumsq_finite_kernel(const T* __restrict__ x, long long n, float* __restrict__ out,
                                    int* __restrict__ nonfinite) {
  __shared__ float red[32];
  float acc = 0.f;
  bool bad = false;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = to_f<T>(x[i]);
    acc += v * v;
    bad |= !isfinite(v);
  }
  acc = warp_sum(acc);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) atomicAdd(out, t);
  }
  if (bad) atomicOr(nonfinite, 1);
}

// hyper[7] (grad_scale of adamw) = inv_loss_scale * min(1, max_norm / (sqrt(sumsq)*inv_loss_scale + 1e-6)),
// skip = nonfinite.  Keeps clip + unscale decisions on the device (no host sync, graph-capturable).
__global__ void finalize_grad_scale_kernel(const float* __restrict__ sumsq, const int* __restrict__ nonfinite,
                                           float inv_loss_scale, float max_norm, float* __restrict__ hyper_scale,
                                           int* __restrict__ skip, float* __restrict__ norm_out) {
  const float norm = sqrtf(sumsq[0]) * inv_loss_scale;
  float s = inv_loss_scale;
  if (max_norm > 0.f) s *= fminf(1.f, max_norm / (norm + 1e-6f));
  *hyper_scale = s;
  if (skip) *skip = *nonfinite;
  if (norm_out) *norm_out = norm;
}

// ------------------------------------------------------------------------------------ embedding
// out[t,:] = (ids[t] in [vocab_start, vocab_start+rows)) ? table[ids[t]-vocab_start,:] : 0
__global__ void embedding_fwd_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids,
                                     __nv_bfloat16* __restrict__ out, long long tokens, int H, int rows,
                                     int vocab_start) {
  const int vecs = H / 8;
  const long long total = tokens * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vecs;
    const int c = (i % vecs) * 8;
    const int id = ids[t] - vocab_start;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < rows) v = *reinterpret_cast<const uint4*>(table + (long long)id * H + c);
    *reinterpret_cast<uint4*>(out + t * H + c) = v;
  }
}
// dtable[ids[t]-vocab_start,:] += dout[t,:]   (fp32 accumulation arena)
__global__ void embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const int* __restrict__ ids,
                                     float* __restrict__ dtable, long long tokens, int H, int rows, int vocab_start) {
  const int vecs = H / 2;
  const long long total = tokens * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vecs;
    const int c = (i % vecs) * 2;
    const int id = ids[t] - vocab_start;
    if (id < 0 || id >= rows) continue;
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dout + t * H + c));
    atomicAdd(dtable + (long long)id * H + c, g.x);
    atomicAdd(dtable + (long long)id * H + c + 1, g.y);
  }
}

// ------------------------------------------------------------------------------------ casts / axpy
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n,
                                        float scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(in[i] * scale);
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, long long n,
                                        float scale, int accumulate) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(in[i]) * scale;
    out[i] = accumulate ? out[i] + v : v;
  }
}
// y = a + b (bf16), 16 bytes per thread
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ y, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const uint4 ra = reinterpret_cast<const uint4*>(a)[i], rb = reinterpret_cast<const uint4*>(b)[i];
    uint4 o;
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&rb);
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) po[j] = __hadd2(pa[j], pb[j]);
    reinterpret_cast<uint4*>(y)[i] = o;
  }
}

static inline int grid_for(long long n, int threads, int per_sm = 8) {
  long long b = (n + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * per_sm;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace msb

using namespace msb;

MSB_EXPORT int msb_ce_stats(const void* logits, const int* labels, float* stats, long long rows, int V,
                            long long pitch, int vocab_start, int logits_fp32, void* stream) {
  if (rows <= 0) return kOk;
  if (logits_fp32)
    ce_stats_kernel<float><<<(unsigned)rows, kCeThreads, 0, (cudaStream_t)stream>>>((const float*)logits, labels,
                                                                                    stats, V, pitch, vocab_start);
  else
    ce_stats_kernel<__nv_bfloat16><<<(unsigned)rows, kCeThreads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)logits, labels, stats, V, pitch, vocab_start);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_ce_grad(const void* logits, const int* labels, const float* stats, float* loss, void* dlogits,
                           const float* grad_scale, long long rows, int V, long long pitch, int vocab_start,
                           int ignore_index, int write_loss, int logits_fp32, void* stream) {
  if (rows <= 0) return kOk;
  if (logits_fp32)
    ce_grad_kernel<float><<<(unsigned)rows, kCeThreads, 0, (cudaStream_t)stream>>>(
        (const float*)logits, labels, stats, loss, (float*)dlogits, grad_scale, V, pitch, vocab_start, ignore_index,
        write_loss);
  else
    ce_grad_kernel<__nv_bfloat16><<<(unsigned)rows, kCeThreads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)logits, labels, stats, loss, (__nv_bfloat16*)dlogits, grad_scale, V, pitch,
        vocab_start, ignore_index, write_loss);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_adamw(float* master, float* m, float* v, const void* grad, int grad_fp32, void* param_lp,
                         long long n, const float* hyper, const int* skip, void* stream) {
  if (n <= 0) return kOk;
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(grad)) & 15) {
    set_last_error("adamw: arena pointers must be 16-byte aligned");
    return kBadArg;
  }
  const int grid = grid_for((n + 3) / 4, 256);
  if (grad_fp32)
    adamw_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(master, m, v, (const float*)grad,
                                                                (__nv_bfloat16*)param_lp, n, hyper, skip);
  else
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(master, m, v, (const __nv_bfloat16*)grad,
                                                                        (__nv_bfloat16*)param_lp, n, hyper, skip);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_momentum(float* master, float* accum, const void* grad, int grad_fp32, void* param_lp, long long n,
                            const float* hyper, const int* skip, void* stream) {
  if (n <= 0) return kOk;
  const int grid = grid_for(n, 256);
  if (grad_fp32)
    momentum_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(master, accum, (const float*)grad,
                                                                   (__nv_bfloat16*)param_lp, n, hyper, skip);
  else
    momentum_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
        master, accum, (const __nv_bfloat16*)grad, (__nv_bfloat16*)param_lp, n, hyper, skip);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_sumsq_finite(const void* x, int is_fp32, long long n, float* out, int* nonfinite, void* stream) {
  if (n <= 0) return kOk;
  const int grid = grid_for(n, 512, 4);
  if (is_fp32)
    sumsq_finite_kernel<float><<<grid, 512, 0, (cudaStream_t)stream>>>((const float*)x, n, out, nonfinite);
  else
    sumsq_finite_kernel<__nv_bfloat16><<<grid, 512, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, n, out,
                                                                               nonfinite);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_finalize_grad_scale(const float* sumsq, const int* nonfinite, float inv_loss_scale, float max_norm,
                                       float* hyper_scale, int* skip, float* norm_out, void* stream) {
  finalize_grad_scale_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(sumsq, nonfinite, inv_loss_scale, max_norm,
                                                                hyper_scale, skip, norm_out);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_embedding_fwd(const void* table, const int* ids, void* out, long long tokens, int H, int rows,
                                 int vocab_start, void* stream) {
  if (H % 8) { set_last_error("embedding: H=%d must be a multiple of 8", H); return kBadArg; }
  if (tokens <= 0) return kOk;
  embedding_fwd_kernel<<<grid_for(tokens * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, tokens, H, rows, vocab_start);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
MSB_EXPORT int msb_embedding_bwd(const void* dout, const int* ids, float* dtable, long long tokens, int H, int rows,
                                 int vocab_start, void* stream) {
  if (H % 2) { set_last_error("embedding: H=%d must be even", H); return kBadArg; }
  if (tokens <= 0) return kOk;
  embedding_bwd_kernel<<<grid_for(tokens * (H / 2), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dout, ids, dtable, tokens, H, rows, vocab_start);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_cast_f32_to_bf16(const float* in, void* out, long long n, float scale, void* stream) {
  if (n <= 0) return kOk;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(in, (__nv_bfloat16*)out, n, scale);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
MSB_EXPORT int msb_cast_bf16_to_f32(const void* in, float* out, long long n, float scale, int accumulate,
                                    void* stream) {
  if (n <= 0) return kOk;
  cast_bf16_to_f32_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)in, out, n, scale,
                                                                              accumulate);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
MSB_EXPORT int msb_add_bf16(const void* a, const void* b, void* y, long long n, void* stream) {
  if (n % 8) { set_last_error("add_bf16: n=%lld must be a multiple of 8", n); return kBadArg; }
  if (n <= 0) return kOk;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, n / 8);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
