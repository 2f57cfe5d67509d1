// Memory-bound transformer kernels for sm_100a: RMSNorm / LayerNorm (forward, backward, fused
// residual add), RoPE, SwiGLU, GELU.  All move 16 bytes per thread per access and make one pass
// over HBM per tensor; reductions stay in registers / shared memory.
//
// The reference has a block-per-row Welford LayerNorm for GPU
// (plugin/device/gpu/kernel/cuda_impl/cuda_ops/layer_norm_impl.cu:218) and a half2 GELU
// (gelu_impl.cu:56); RmsNorm, ApplyRotaryPosEmb and SwiGLU have op definitions
// (core/ops/ops_def/rms_norm_op.yaml, apply_rotary_pos_emb_op.yaml) but no GPU kernel.
//
// This text is compiled twice: for bf16 tensors (norm_act.cu), and with MSB_ELEM_FP16 defined for fp16 tensors
// (norm_act_fp16.cu), where every entry point carries the suffix _fp16 and "bf16" in a comment reads "fp16".
#include "host_common.h"
#include "elem.cuh"

namespace msb {
namespace MSB_ELEM_NS {

constexpr int kNormThreads = 256;

struct alignas(16) bf16x8 {
  elem2_t v[4];
};

__device__ __forceinline__ void load8(const elem_t* p, float (&f)[8]) {
  const bf16x8 raw = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = e2_to_f2(raw.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(elem_t* p, const float (&f)[8]) {
  bf16x8 raw;
#pragma unroll
  for (int i = 0; i < 4; ++i) raw.v[i] = f2_to_e2(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = raw;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ------------------------------------------------------------------------------------ RMSNorm
// y = (x [+ res]) * rstd * w ; optionally writes the summed residual stream to `xsum`.
// H must be a multiple of 8 and <= kNormThreads*8*kMaxIter.
constexpr int kMaxIter = 8;  // H up to 16384

template <int ITER>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const elem_t* __restrict__ x, const elem_t* __restrict__ res,
                   const elem_t* __restrict__ w, elem_t* __restrict__ y,
                   elem_t* __restrict__ xsum, float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const elem_t* xr = x + row * H;
  float v[ITER][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = (it * kNormThreads + threadIdx.x) * 8;
    if (c < H) {
      load8(xr + c, v[it]);
      if (res) {
        float r[8];
        load8(res + row * H + c, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[it][j] += r[j];
        if (xsum) {
          // round once so that the normalised value matches what the backward pass re-reads
          store8(xsum + row * H + c, v[it]);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[it][j] = e_to_f(f_to_e(v[it][j]));
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[it][j] * v[it][j];
    }
  }
  ss = block_sum<kNormThreads>(ss, red);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = (it * kNormThreads + threadIdx.x) * 8;
    if (c < H) {
      float g[8], o[8];
      load8(w + c, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[it][j] * rstd * g[j];
      store8(y + row * H + c, o);
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres_in) ; dw = sum_rows dy * xhat.
// Persistent over rows; per-CTA partial dw kept in registers.  Two-stage reduction (ATOMIC = false): CTA b stores
// its partial as row b of dw_acc[gridDim.x][H] and reduce_partials_kernel sums the rows in a fixed order
// (deterministic).  ATOMIC = true adds into a single dw_acc[H] instead (the allocation-free entry point, whose
// scratch is one row).
template <int ITER, bool ATOMIC>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const elem_t* __restrict__ dy, const elem_t* __restrict__ x,
                   const elem_t* __restrict__ w, const float* __restrict__ rstd,
                   const elem_t* __restrict__ dres, elem_t* __restrict__ dx,
                   float* __restrict__ dw_acc, int rows, int H) {
  __shared__ float red[32];
  float wreg[ITER][8], dwreg[ITER][8];
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = (it * kNormThreads + threadIdx.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwreg[it][j] = 0.f;
    if (c < H) load8(w + c, wreg[it]);
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rs = rstd[row];
    float g[ITER][8], xh[ITER][8];
    float dot = 0.f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kNormThreads + threadIdx.x) * 8;
      if (c < H) {
        load8(dy + row * H + c, g[it]);
        load8(x + row * H + c, xh[it]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[it][j] *= rs;
          dwreg[it][j] += g[it][j] * xh[it][j];
          g[it][j] *= wreg[it][j];
          dot += g[it][j] * xh[it][j];
        }
      }
    }
    dot = block_sum<kNormThreads>(dot, red) / H;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kNormThreads + threadIdx.x) * 8;
      if (c < H) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (g[it][j] - xh[it][j] * dot);
        if (dres) {
          float r[8];
          load8(dres + row * H + c, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + row * H + c, o);
      }
    }
  }
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = (it * kNormThreads + threadIdx.x) * 8;
    if (c < H) {
      if (ATOMIC) {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(dw_acc + c + j, dwreg[it][j]);
      } else {
        float* dst = dw_acc + static_cast<long long>(blockIdx.x) * H + c;
        *reinterpret_cast<float4*>(dst) = make_float4(dwreg[it][0], dwreg[it][1], dwreg[it][2], dwreg[it][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(dwreg[it][4], dwreg[it][5], dwreg[it][6], dwreg[it][7]);
      }
    }
  }
}

// Second stage of the weight-gradient reduction: out[c] (+)= sum_b partial[b][c] for b = 0..parts-1, rows visited
// in a fixed order.  Block = 32 columns x 8 row lanes; lane r sums rows r, r+8, ... and the 8 lanes are combined
// through shared memory, always in the same order.
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const float* __restrict__ partial, int parts, int H, elem_t* __restrict__ out_bf16,
                       float* __restrict__ out_f32, int accumulate) {
  __shared__ float sm[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < H)
    for (int b = ry; b < parts; b += 8) s += partial[static_cast<long long>(b) * H + c];
  sm[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && c < H) {
    float v = sm[0][cx];
#pragma unroll
    for (int r = 1; r < 8; ++r) v += sm[r][cx];
    if (out_f32) out_f32[c] = accumulate ? out_f32[c] + v : v;
    if (out_bf16) out_bf16[c] = f_to_e(accumulate ? e_to_f(out_bf16[c]) + v : v);
  }
}

// ------------------------------------------------------------------------------------ LayerNorm
template <int ITER>
__global__ void __launch_bounds__(kNormThreads)
layernorm_fwd_kernel(const elem_t* __restrict__ x, const elem_t* __restrict__ w,
                     const elem_t* __restrict__ b, elem_t* __restrict__ y,
                     float* __restrict__ mean_out, float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  float v[ITER][8];
  float s = 0.f;
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = (it * kNormThreads + threadIdx.x) * 8;
    if (c < H) {
      load8(x + row * H + c, v[it]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[it][j];
    }
  }
  const float mean = block_sum<kNormThreads>(s, red) / H;
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = (it * kNormThreads + threadIdx.x) * 8;
    if (c < H) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[it][j] - mean;
        ss += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum<kNormThreads>(ss, red) / H + eps);
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = (it * kNormThreads + threadIdx.x) * 8;
    if (c < H) {
      float g[8], bb[8], o[8];
      load8(w + c, g);
      if (b) load8(b + c, bb);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[it][j] - mean) * rstd * g[j] + (b ? bb[j] : 0.f);
      store8(y + row * H + c, o);
    }
  }
}

template <int ITER>
__global__ void __launch_bounds__(kNormThreads)
layernorm_bwd_kernel(const elem_t* __restrict__ dy, const elem_t* __restrict__ x,
                     const elem_t* __restrict__ w, const float* __restrict__ mean,
                     const float* __restrict__ rstd, elem_t* __restrict__ dx, float* __restrict__ dw_acc,
                     float* __restrict__ db_acc, int rows, int H) {
  __shared__ float red[32];
  float wreg[ITER][8], dwreg[ITER][8], dbreg[ITER][8];
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = (it * kNormThreads + threadIdx.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwreg[it][j] = dbreg[it][j] = 0.f;
    if (c < H) load8(w + c, wreg[it]);
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mu = mean[row], rs = rstd[row];
    float g[ITER][8], xh[ITER][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kNormThreads + threadIdx.x) * 8;
      if (c < H) {
        load8(dy + row * H + c, g[it]);
        load8(x + row * H + c, xh[it]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[it][j] = (xh[it][j] - mu) * rs;
          dwreg[it][j] += g[it][j] * xh[it][j];
          dbreg[it][j] += g[it][j];
          g[it][j] *= wreg[it][j];
          s1 += g[it][j];
          s2 += g[it][j] * xh[it][j];
        }
      }
    }
    s1 = block_sum<kNormThreads>(s1, red) / H;
    s2 = block_sum<kNormThreads>(s2, red) / H;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kNormThreads + threadIdx.x) * 8;
      if (c < H) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (g[it][j] - s1 - xh[it][j] * s2);
        store8(dx + row * H + c, o);
      }
    }
  }
  // two-stage reduction: this CTA's partial sums are row blockIdx.x of dw_acc / db_acc ([gridDim.x][H] each)
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = (it * kNormThreads + threadIdx.x) * 8;
    if (c < H) {
      float* dw = dw_acc + static_cast<long long>(blockIdx.x) * H + c;
      *reinterpret_cast<float4*>(dw) = make_float4(dwreg[it][0], dwreg[it][1], dwreg[it][2], dwreg[it][3]);
      *reinterpret_cast<float4*>(dw + 4) = make_float4(dwreg[it][4], dwreg[it][5], dwreg[it][6], dwreg[it][7]);
      if (db_acc) {
        float* db = db_acc + static_cast<long long>(blockIdx.x) * H + c;
        *reinterpret_cast<float4*>(db) = make_float4(dbreg[it][0], dbreg[it][1], dbreg[it][2], dbreg[it][3]);
        *reinterpret_cast<float4*>(db + 4) = make_float4(dbreg[it][4], dbreg[it][5], dbreg[it][6], dbreg[it][7]);
      }
    }
  }
}

// fp32 accumulator -> bf16 parameter gradient (optionally accumulating into an existing bf16/fp32 grad)
__global__ void finalize_acc_kernel(const float* __restrict__ acc, elem_t* __restrict__ out_bf16,
                                    float* __restrict__ out_f32, int n, int accumulate) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = acc[i];
  if (out_f32) out_f32[i] = accumulate ? out_f32[i] + v : v;
  if (out_bf16) out_bf16[i] = f_to_e(accumulate ? e_to_f(out_bf16[i]) + v : v);
}

// ------------------------------------------------------------------------------------ RoPE
// x: [tokens, heads, D] (row pitch `pitch` elements per token), rotate-half convention:
//   out[..., i]       = x[i]*cos[i] - x[i+D/2]*sin[i]
//   out[..., i+D/2]   = x[i+D/2]*cos[i] + x[i]*sin[i]
// cos/sin: fp32 [seq, D/2]; position of token t is pos[t] if given, else (t % seq).
// sign = -1 gives the backward (inverse) rotation.
__global__ void rope_kernel(elem_t* __restrict__ x, const float* __restrict__ cosb,
                            const float* __restrict__ sinb, const int* __restrict__ pos, long long tokens,
                            int heads, int D, long long pitch, int seq, float sign) {
  const int half = D / 2;
  const int vec_per_head = half / 8;
  const long long total = tokens * heads * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int vi = i % vec_per_head;
    const long long th = i / vec_per_head;
    const int h = th % heads;
    const long long t = th / heads;
    const int p = pos ? pos[t] : static_cast<int>(t % seq);
    elem_t* base = x + t * pitch + (long long)h * D + vi * 8;
    float a[8], b[8], oa[8], ob[8];
    load8(base, a);
    load8(base + half, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c = cosb[(long long)p * half + vi * 8 + j];
      const float s = sign * sinb[(long long)p * half + vi * 8 + j];
      oa[j] = a[j] * c - b[j] * s;
      ob[j] = b[j] * c + a[j] * s;
    }
    store8(base, oa);
    store8(base + half, ob);
  }
}

// ------------------------------------------------------------------------------------ SwiGLU / GELU
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// gu: [rows, 2F] with gate in [:, :F], up in [:, F:]; out [rows, F] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const elem_t* __restrict__ gu, elem_t* __restrict__ out,
                                  long long rows, int F) {
  const int vecs = F / 8;
  const long long total = rows * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vecs;
    const int c = (i % vecs) * 8;
    float g[8], u[8], o[8];
    load8(gu + r * 2 * F + c, g);
    load8(gu + r * 2 * F + F + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] * sigmoidf_(g[j]) * u[j];
    store8(out + r * F + c, o);
  }
}
// dgu[:, :F] = dout * up * (s + g*s*(1-s)) ; dgu[:, F:] = dout * g*s
__global__ void swiglu_bwd_kernel(const elem_t* __restrict__ gu, const elem_t* __restrict__ dout,
                                  elem_t* __restrict__ dgu, long long rows, int F) {
  const int vecs = F / 8;
  const long long total = rows * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vecs;
    const int c = (i % vecs) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + r * 2 * F + c, g);
    load8(gu + r * 2 * F + F + c, u);
    load8(dout + r * F + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sigmoidf_(g[j]);
      dg[j] = d[j] * u[j] * (s + g[j] * s * (1.f - s));
      du[j] = d[j] * g[j] * s;
    }
    store8(dgu + r * 2 * F + c, dg);
    store8(dgu + r * 2 * F + F + c, du);
  }
}

// tanh-approximated GELU on x (+ bias[n]) ; mode 0 fwd: y = gelu(x+b); mode 1 bwd: y = dy * gelu'(x+b)
__global__ void gelu_kernel(const elem_t* __restrict__ x, const elem_t* __restrict__ bias,
                            const elem_t* __restrict__ dy, elem_t* __restrict__ y, long long rows,
                            int N, int mode) {
  const int vecs = N / 8;
  const long long total = rows * vecs;
  constexpr float k0 = 0.7978845608028654f, k1 = 0.044715f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (i % vecs) * 8;
    float v[8], o[8], b[8], d[8];
    load8(x + i * 8, v);
    if (bias) {
      load8(bias + c, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += b[j];
    }
    if (mode == 1) load8(dy + i * 8, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float t = tanhf(k0 * (v[j] + k1 * v[j] * v[j] * v[j]));
      if (mode == 0) {
        o[j] = 0.5f * v[j] * (1.f + t);
      } else {
        const float dt = (1.f - t * t) * k0 * (1.f + 3.f * k1 * v[j] * v[j]);
        o[j] = d[j] * (0.5f * (1.f + t) + 0.5f * v[j] * dt);
      }
    }
    store8(y + i * 8, o);
  }
}

static inline int ew_grid(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace MSB_ELEM_NS
}  // namespace msb

using namespace msb;
using namespace msb::MSB_ELEM_NS;

#define MSB_ITER_DISPATCH(H, CALL)                                           \
  do {                                                                       \
    const int _it = ((H) / 8 + kNormThreads - 1) / kNormThreads;             \
    if (_it <= 1) { CALL(1); } else if (_it <= 2) { CALL(2); }               \
    else if (_it <= 4) { CALL(4); } else { CALL(8); }                        \
  } while (0)

static int check_h(const char* what, int H) {
  if (H <= 0 || (H % 8) != 0 || H > kNormThreads * 8 * kMaxIter) {
    set_last_error("%s: hidden size %d must be a positive multiple of 8 and <= %d", what, H,
                   kNormThreads * 8 * kMaxIter);
    return kBadArg;
  }
  return kOk;
}

MSB_EXPORT int MSB_FN(msb_rmsnorm_fwd)(const void* x, const void* res, const void* w, void* y, void* xsum, float* rstd,
                               long long rows, int H, float eps, void* stream) {
  if (int rc = check_h("rmsnorm_fwd", H)) return rc;
  if (rows <= 0) return kOk;
#define CALL(I)                                                                                          \
  rmsnorm_fwd_kernel<I><<<(unsigned)rows, kNormThreads, 0, (cudaStream_t)stream>>>(                      \
      (const elem_t*)x, (const elem_t*)res, (const elem_t*)w, (elem_t*)y,    \
      (elem_t*)xsum, rstd, H, eps)
  MSB_ITER_DISPATCH(H, CALL);
#undef CALL
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// dw_out (bf16 or fp32 by dw_fp32) receives (accumulate ? dw_out + dw : dw), dw = sum_rows dy * xhat.
// Floats of scratch the norm backward launchers need for hidden size H: one partial row per CTA.
#ifndef MSB_ELEM_FP16
MSB_EXPORT long long msb_norm_bwd_scratch_elems(int H, int with_bias) {
  return 2LL * sm_count() * H * (with_bias ? 2 : 1);
}
#endif

// dw_acc: fp32 scratch of msb_norm_bwd_scratch_elems(H, 0) floats (per-CTA partial rows; nothing needs clearing).
MSB_EXPORT int MSB_FN(msb_rmsnorm_bwd)(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                               void* dx, float* dw_acc, void* dw_out, int dw_fp32, int accumulate, long long rows,
                               int H, void* stream_) {
  if (int rc = check_h("rmsnorm_bwd", H)) return rc;
  cudaStream_t stream = (cudaStream_t)stream_;
  int grid = 0;
  if (rows > 0) {
    grid = (int)(rows < 2LL * sm_count() ? rows : 2LL * sm_count());
#define CALL(I)                                                                                      \
  rmsnorm_bwd_kernel<I, false><<<grid, kNormThreads, 0, stream>>>(                                   \
      (const elem_t*)dy, (const elem_t*)x, (const elem_t*)w, rstd,              \
      (const elem_t*)dres, (elem_t*)dx, dw_acc, (int)rows, H)
    MSB_ITER_DISPATCH(H, CALL);
#undef CALL
  }
  if (dw_out) {
    reduce_partials_kernel<<<(H + 31) / 32, 256, 0, stream>>>(dw_acc, grid, H, dw_fp32 ? nullptr : (elem_t*)dw_out,
                                                             dw_fp32 ? (float*)dw_out : nullptr, accumulate);
  }
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int MSB_FN(msb_layernorm_fwd)(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                                 long long rows, int H, float eps, void* stream) {
  if (int rc = check_h("layernorm_fwd", H)) return rc;
  if (rows <= 0) return kOk;
#define CALL(I)                                                                                       \
  layernorm_fwd_kernel<I><<<(unsigned)rows, kNormThreads, 0, (cudaStream_t)stream>>>(                 \
      (const elem_t*)x, (const elem_t*)w, (const elem_t*)b, (elem_t*)y,   \
      mean, rstd, H, eps)
  MSB_ITER_DISPATCH(H, CALL);
#undef CALL
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// acc: fp32 scratch of msb_norm_bwd_scratch_elems(H, 1) floats: per-CTA partial rows of dw, then those of db.
MSB_EXPORT int MSB_FN(msb_layernorm_bwd)(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                 void* dx, float* acc, void* dw_out, void* db_out, int out_fp32, int accumulate,
                                 long long rows, int H, void* stream_) {
  if (int rc = check_h("layernorm_bwd", H)) return rc;
  cudaStream_t stream = (cudaStream_t)stream_;
  int grid = 0;
  float* db_part = acc + 2LL * sm_count() * H;
  if (rows > 0) {
    grid = (int)(rows < 2LL * sm_count() ? rows : 2LL * sm_count());
#define CALL(I)                                                                                   \
  layernorm_bwd_kernel<I><<<grid, kNormThreads, 0, stream>>>(                                     \
      (const elem_t*)dy, (const elem_t*)x, (const elem_t*)w, mean, rstd,     \
      (elem_t*)dx, acc, db_out ? db_part : nullptr, (int)rows, H)
    MSB_ITER_DISPATCH(H, CALL);
#undef CALL
  }
  if (dw_out)
    reduce_partials_kernel<<<(H + 31) / 32, 256, 0, stream>>>(acc, grid, H, out_fp32 ? nullptr : (elem_t*)dw_out,
                                                             out_fp32 ? (float*)dw_out : nullptr, accumulate);
  if (db_out)
    reduce_partials_kernel<<<(H + 31) / 32, 256, 0, stream>>>(db_part, grid, H,
                                                             out_fp32 ? nullptr : (elem_t*)db_out,
                                                             out_fp32 ? (float*)db_out : nullptr, accumulate);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int MSB_FN(msb_rope)(void* x, const float* cosb, const float* sinb, const int* pos, long long tokens, int heads,
                        int D, long long pitch, int seq, int backward, void* stream) {
  if (D % 16 != 0 || pitch % 8 != 0) {
    set_last_error("rope: head dim %d must be a multiple of 16 and pitch %lld a multiple of 8", D, pitch);
    return kBadArg;
  }
  const long long work = tokens * heads * (D / 16);
  if (work <= 0) return kOk;
  rope_kernel<<<ew_grid(work, 256), 256, 0, (cudaStream_t)stream>>>((elem_t*)x, cosb, sinb, pos, tokens, heads,
                                                                    D, pitch, seq, backward ? -1.f : 1.f);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int MSB_FN(msb_swiglu_fwd)(const void* gu, void* out, long long rows, int F, void* stream) {
  if (F % 8 != 0) { set_last_error("swiglu: F=%d must be a multiple of 8", F); return kBadArg; }
  if (rows <= 0) return kOk;
  swiglu_fwd_kernel<<<ew_grid(rows * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const elem_t*)gu, (elem_t*)out, rows, F);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
MSB_EXPORT int MSB_FN(msb_swiglu_bwd)(const void* gu, const void* dout, void* dgu, long long rows, int F, void* stream) {
  if (F % 8 != 0) { set_last_error("swiglu: F=%d must be a multiple of 8", F); return kBadArg; }
  if (rows <= 0) return kOk;
  swiglu_bwd_kernel<<<ew_grid(rows * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const elem_t*)gu, (const elem_t*)dout, (elem_t*)dgu, rows, F);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
MSB_EXPORT int MSB_FN(msb_gelu)(const void* x, const void* bias, const void* dy, void* y, long long rows, int N, int backward,
                        void* stream) {
  if (N % 8 != 0) { set_last_error("gelu: N=%d must be a multiple of 8", N); return kBadArg; }
  if (rows <= 0) return kOk;
  gelu_kernel<<<ew_grid(rows * (N / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const elem_t*)x, (const elem_t*)bias, (const elem_t*)dy, (elem_t*)y, rows, N,
      backward);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

#ifndef MSB_ELEM_FP16
// ----------------------------------------------------------------------------------------------------------------
// RMSNorm backward without any allocation (declared in no_alloc.h): the [H] fp32 weight-gradient accumulator is the
// static device array below.  One array per device (each device holds its own instance of a __device__ variable).
#include "no_alloc.h"

#include <atomic>

static __device__ __align__(256) float g_rmsnorm_bwd_static_acc[MSB_RMSNORM_BWD_STATIC_MAX_H];

namespace {
constexpr int kMaxDevices = 64;
std::atomic<float*> g_static_acc_ptr[kMaxDevices];

// Device address of this device's instance of the array; looked up on the first call per device and kept.
int static_acc_ptr(float** out) {
  int dev = 0;
  MSB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_last_error("rmsnorm_bwd_static: device ordinal %d is beyond %d", dev, kMaxDevices - 1);
    return kTooLarge;
  }
  float* p = g_static_acc_ptr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    MSB_CUDA_CHECK(cudaGetSymbolAddress((void**)&p, g_rmsnorm_bwd_static_acc));
    if (p == nullptr) {
      set_last_error("rmsnorm_bwd_static: cudaGetSymbolAddress returned a null address");
      return kCudaError;
    }
    g_static_acc_ptr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return kOk;
}
}  // namespace

MSB_EXPORT int msb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd,
                                      const void* dres, void* dx, void* dw_out, int dw_fp32, int accumulate,
                                      long long rows, int H, void* stream_) {
  if (H > MSB_RMSNORM_BWD_STATIC_MAX_H) {
    set_last_error("rmsnorm_bwd_static: hidden size %d exceeds the static scratch of %d floats", H,
                   MSB_RMSNORM_BWD_STATIC_MAX_H);
    return kTooLarge;
  }
  if (int rc = check_h("rmsnorm_bwd_static", H)) return rc;
  float* acc = nullptr;
  if (int rc = static_acc_ptr(&acc)) return rc;
  cudaStream_t stream = (cudaStream_t)stream_;
  MSB_CUDA_CHECK(cudaMemsetAsync(acc, 0, sizeof(float) * H, stream));
  if (rows > 0) {
    const int grid = (int)(rows < 2LL * sm_count() ? rows : 2LL * sm_count());
#define CALL(I)                                                                                      \
  rmsnorm_bwd_kernel<I, true><<<grid, kNormThreads, 0, stream>>>(                                    \
      (const elem_t*)dy, (const elem_t*)x, (const elem_t*)w, rstd,              \
      (const elem_t*)dres, (elem_t*)dx, acc, (int)rows, H)
    MSB_ITER_DISPATCH(H, CALL);
#undef CALL
  }
  if (dw_out) {
    finalize_acc_kernel<<<(H + 255) / 256, 256, 0, stream>>>(acc, dw_fp32 ? nullptr : (elem_t*)dw_out,
                                                             dw_fp32 ? (float*)dw_out : nullptr, H, accumulate);
  }
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
#endif  // MSB_ELEM_FP16
