// Mixture-of-experts routing and token movement.
//
//   msb_moe_router_step   : one routing round (the k-th choice of every token) in a single kernel: softmax over
//                           the expert logits, masking of experts the token already occupies, arg-max, position of
//                           the token inside its expert (exclusive count over tokens in index order, by a
//                           decoupled look-back scan across thread blocks), capacity cut, and the load-balance
//                           statistics (tokens per expert, mean renormalised probability per expert).
//   msb_moe_router_finish : closes a round: adds the round's load-balance loss, advances the per-expert fill level.
//   msb_moe_router_weights: combine weights = gates normalised over the rounds of one token (k > 1).
//   msb_moe_router_bwd    : gradient of (combine weights, loss) with respect to the router logits.
//   msb_moe_scatter_rows  : dispatch: every kept (token, choice) row is stored straight into the input buffer of
//                           the expert's owner rank (peer stores over NVLink), optionally scaled.
//   msb_moe_gather_rows   : combine: every token pulls its rows from the owners' output buffers (peer loads),
//                           applies the combine weights and sums; optionally also returns <g[t], row> per choice.
//
// The routing arithmetic is that of TopkRouter in the reference (python/mindspore/parallel/_transformer/moe.py:
// 604-693): ~40 small operators there, plus one-hot dispatch/combine BatchMatMuls and an AlltoAll lowered to
// ncclSend/ncclRecv pairs (plugin/device/gpu/kernel/nccl/nccl_p2p_gpu_kernel.h:133-168).
#include "host_common.h"
#include "ptx.cuh"

namespace msb {

constexpr int kRouterThreads = 256;
constexpr int kMaxExperts = 256;
constexpr int kMaxChoices = 4;
constexpr int kMoeMaxRanks = 8;

struct RouterParams {
  const float* logits;      // [T, E]
  int* expert;              // [T, K]
  int* slot;                // [T, K]  position inside the expert, -1 = dropped
  float* gate;              // [T, K]  router probability of the choice, 0 when dropped
  const int* fill;          // [E] rows already taken in each expert by earlier rounds
  float* proxy;             // [E] += sum over tokens of renormalised masked probability
  unsigned long long* scan; // [blocks, E] look-back words: (state << 32) | value; state 1 = aggregate, 2 = prefix
  int* ticket;              // dynamic block id
  int T, E, K, step, capacity;
  int* status;
};

__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kRouterThreads) moe_router_step_kernel(RouterParams p) {
  __shared__ int s_block;
  __shared__ int s_wcount[kRouterThreads / 32][kMaxExperts];
  __shared__ int s_excl[kMaxExperts];
  __shared__ float s_proxy[kMaxExperts];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_block = atomicAdd(p.ticket, 1);
  for (int i = tid; i < (kRouterThreads / 32) * kMaxExperts; i += kRouterThreads) (&s_wcount[0][0])[i] = 0;
  if (tid < kMaxExperts) s_proxy[tid] = 0.f;
  __syncthreads();
  const int block = s_block;
  const int t = block * kRouterThreads + tid;
  const bool valid = t < p.T;
  const int E = p.E;
  const float* row = p.logits + (size_t)(valid ? t : 0) * E;

  // experts this token already occupies (kept choices of earlier rounds)
  int taken[kMaxChoices];
#pragma unroll
  for (int j = 0; j < kMaxChoices; ++j) {
    taken[j] = -1;
    if (valid && j < p.step && p.slot[(size_t)t * p.K + j] >= 0) taken[j] = p.expert[(size_t)t * p.K + j];
  }
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) mx = fmaxf(mx, row[e]);
  float sum = 0.f;
  for (int e = 0; e < E; ++e) sum += expf(row[e] - mx);
  const float inv = 1.f / sum;
  float best = -1.f, msum = 0.f;
  int best_e = 0;
  for (int e = 0; e < E; ++e) {
    float pe = expf(row[e] - mx) * inv;
#pragma unroll
    for (int j = 0; j < kMaxChoices; ++j) pe = (taken[j] == e) ? 0.f : pe;
    msum += pe;
    if (pe > best) { best = pe; best_e = e; }
  }
  // load-balance proxy: mean over tokens of the renormalised masked probabilities
  const float rnorm = valid ? 1.f / (msum + 1e-9f) : 0.f;
  for (int e = 0; e < E; ++e) {
    float pe = expf(row[e] - mx) * inv;
#pragma unroll
    for (int j = 0; j < kMaxChoices; ++j) pe = (taken[j] == e) ? 0.f : pe;
    const float v = warp_sum(pe * rnorm);
    if (lane == 0) atomicAdd(&s_proxy[e], v);
  }
  // rank of the token among the tokens of this block that chose the same expert
  const int key = valid ? best_e : (kMaxExperts + lane);
  const unsigned same = __match_any_sync(0xffffffffu, key);
  const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
  if (valid && rank_in_warp == 0) s_wcount[warp][best_e] = __popc(same);
  __syncthreads();
  int before = 0;
  if (valid)
    for (int w = 0; w < warp; ++w) before += s_wcount[w][best_e];
  // decoupled look-back over blocks, one thread per expert
  if (tid < E) {
    int agg = 0;
    for (int w = 0; w < kRouterThreads / 32; ++w) agg += s_wcount[w][tid];
    unsigned long long* mine = p.scan + (size_t)block * E + tid;
    int excl = 0;
    if (block == 0) {
      atomicExch(mine, (2ull << 32) | (unsigned)agg);
    } else {
      atomicExch(mine, (1ull << 32) | (unsigned)agg);
      const unsigned long long t0 = globaltimer_ns();
      int j = block - 1;
      while (j >= 0) {
        const unsigned long long w = ld_volatile_u64(p.scan + (size_t)j * E + tid);
        const unsigned state = (unsigned)(w >> 32);
        if (state == 0) {
          if (globaltimer_ns() - t0 > kWaitLimitNs) {
            atomicOr(p.status, 4);
            break;
          }
          continue;
        }
        excl += (int)(unsigned)w;
        if (state == 2) break;
        --j;
      }
      atomicExch(mine, (2ull << 32) | (unsigned)(excl + agg));
    }
    s_excl[tid] = excl;
    atomicAdd(p.proxy + tid, s_proxy[tid]);
  }
  __syncthreads();
  if (valid) {
    const int pos = p.fill[best_e] + s_excl[best_e] + before + rank_in_warp;
    const bool keep = pos < p.capacity;
    const size_t o = (size_t)t * p.K + p.step;
    p.expert[o] = best_e;
    p.slot[o] = keep ? pos : -1;
    p.gate[o] = keep ? best : 0.f;
  }
}

// One block of E threads.  density[step][e] = tokens that chose e in this round / T.
__global__ void moe_router_finish_kernel(const unsigned long long* scan, int blocks, int* fill, float* proxy,
                                         float* density, float* loss, int T, int E, int step, int capacity) {
  __shared__ float red[kMaxExperts];
  const int e = threadIdx.x;
  float term = 0.f;
  if (e < E) {
    const int total = (int)(unsigned)scan[(size_t)(blocks - 1) * E + e];
    const float d = (float)total / (float)T;
    density[(size_t)step * E + e] = d;
    term = d * (proxy[e] / (float)T);
    proxy[e] = 0.f;
    const int f = fill[e];
    int room = capacity - f;
    room = room < 0 ? 0 : room;
    fill[e] = f + (total < room ? total : room);
  }
  red[e] = term;
  __syncthreads();
  for (int s = blockDim.x / 2; s > 0; s >>= 1) {
    if (e < s) red[e] += red[e + s];
    __syncthreads();
  }
  // mean over experts, times E twice (as the reference does)
  if (e == 0) *loss += red[0] / (float)E * (float)E * (float)E;
}

__global__ void moe_router_weights_kernel(const float* gate, float* weight, int T, int K) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float s = 0.f;
  for (int j = 0; j < K; ++j) s += gate[(size_t)t * K + j];
  const float inv = K > 1 ? 1.f / (s + 1e-9f) : 1.f;
  for (int j = 0; j < K; ++j) weight[(size_t)t * K + j] = gate[(size_t)t * K + j] * inv;
}

// d logits from d weights [T, K] and d loss (scalar).  One thread per token; probabilities are recomputed.
//   weights w_s = g_s / (sum_j g_j + eps)  (K > 1), g_s = p[e_s] * keep_s
//   loss    = sum_s E * sum_e density_s[e] * (1/T) sum_t m_s[t, e] / (M_s[t] + eps),  m_s = p * (1 - taken_s)
__global__ void moe_router_bwd_kernel(const float* logits, const int* expert, const int* slot, const float* gate,
                                      const float* dweight, const float* dloss, const float* density,
                                      float* dlogits, int T, int E, int K) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float* row = logits + (size_t)t * E;
  int ex[kMaxChoices];
  bool kept[kMaxChoices];
  float dg[kMaxChoices], g[kMaxChoices];
  float gs = 0.f, dot_w = 0.f;
  for (int j = 0; j < K; ++j) {
    ex[j] = expert[(size_t)t * K + j];
    kept[j] = slot[(size_t)t * K + j] >= 0;
    g[j] = gate[(size_t)t * K + j];
    gs += g[j];
  }
  if (K > 1) {
    const float S = gs + 1e-9f;
    for (int j = 0; j < K; ++j) dot_w += dweight[(size_t)t * K + j] * g[j];
    for (int j = 0; j < K; ++j) dg[j] = kept[j] ? (dweight[(size_t)t * K + j] / S - dot_w / (S * S)) : 0.f;
  } else {
    dg[0] = kept[0] ? dweight[t] : 0.f;
  }
  const float dl = dloss ? *dloss : 0.f;
  const float cscale = dl * (float)E / (float)T;
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) mx = fmaxf(mx, row[e]);
  float sum = 0.f;
  for (int e = 0; e < E; ++e) sum += expf(row[e] - mx);
  const float inv = 1.f / sum;
  // per round: M_s = sum of masked probabilities, Q_s = sum_e c_s[e] m_s[e]
  float M[kMaxChoices], Q[kMaxChoices];
  for (int s = 0; s < K; ++s) M[s] = Q[s] = 0.f;
  for (int e = 0; e < E; ++e) {
    const float pe = expf(row[e] - mx) * inv;
    bool masked = false;
    for (int s = 0; s < K; ++s) {
      if (!masked) {
        M[s] += pe;
        Q[s] += cscale * density[(size_t)s * E + e] * pe;
      }
      masked = masked || (kept[s] && ex[s] == e);     // rounds after s see expert ex[s] masked
    }
  }
  // dp[e] evaluated on the fly, twice: once for sum_e p[e] dp[e], once to write
  float pdot = 0.f;
  for (int pass = 0; pass < 2; ++pass) {
    for (int e = 0; e < E; ++e) {
      const float pe = expf(row[e] - mx) * inv;
      float dp = 0.f;
      bool masked = false;
      for (int s = 0; s < K; ++s) {
        if (!masked) {
          const float Ms = M[s] + 1e-9f;
          dp += cscale * density[(size_t)s * E + e] / Ms - Q[s] / (Ms * Ms);
        }
        if (ex[s] == e && kept[s]) dp += dg[s];
        masked = masked || (kept[s] && ex[s] == e);
      }
      if (pass == 0) pdot += pe * dp;
      else dlogits[(size_t)t * E + e] = pe * (dp - pdot);
    }
  }
}

struct MoePeers {
  void* p[kMoeMaxRanks];
};

// One block per token.  Row of (token t, choice j) goes to rank e / EL, offset ((e % EL) * n_src + me) * C + pos.
__global__ void moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, const float* __restrict__ scale,
                                        const int* __restrict__ expert, const int* __restrict__ slot, MoePeers dst,
                                        int T, int K, int H, int EL, int n_src, int me, int C) {
  const int t = blockIdx.x;
  const uint4* in = reinterpret_cast<const uint4*>(src + (size_t)t * H);
  for (int j = 0; j < K; ++j) {
    const int pos = slot[(size_t)t * K + j];
    if (pos < 0) continue;
    const int e = expert[(size_t)t * K + j];
    __nv_bfloat16* base = static_cast<__nv_bfloat16*>(dst.p[e / EL]) +
                          ((size_t)((e % EL) * n_src + me) * C + pos) * H;
    uint4* out = reinterpret_cast<uint4*>(base);
    if (scale == nullptr) {
      for (int i = threadIdx.x; i < H / 8; i += blockDim.x) out[i] = in[i];
    } else {
      const float s = scale[(size_t)t * K + j];
      for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
        uint4 v = in[i];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(h[q]);
          h[q] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
        out[i] = v;
      }
    }
  }
}

// One block per token: out[t] = sum_j scale[t, j] * row_j (scale null = 1); dots[t, j] = <g[t], row_j>.
__global__ void moe_gather_rows_kernel(MoePeers srcs, const float* __restrict__ scale,
                                       const int* __restrict__ expert, const int* __restrict__ slot,
                                       const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ out,
                                       float* __restrict__ dots, int T, int K, int H, int EL, int n_src, int me,
                                       int C) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const uint4* rows[kMaxChoices];
  float w[kMaxChoices];
  for (int j = 0; j < K; ++j) {
    const int pos = slot[(size_t)t * K + j];
    rows[j] = nullptr;
    w[j] = 0.f;
    if (pos >= 0) {
      const int e = expert[(size_t)t * K + j];
      rows[j] = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(srcs.p[e / EL]) +
                                               ((size_t)((e % EL) * n_src + me) * C + pos) * H);
      w[j] = scale ? scale[(size_t)t * K + j] : 1.f;
    }
  }
  float dot[kMaxChoices] = {0.f, 0.f, 0.f, 0.f};
  const uint4* gin = g ? reinterpret_cast<const uint4*>(g + (size_t)t * H) : nullptr;
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float gv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (gin) {
      const uint4 raw = gin[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        gv[2 * q] = f.x;
        gv[2 * q + 1] = f.y;
      }
    }
    for (int j = 0; j < K; ++j) {
      if (rows[j] == nullptr) continue;
      const uint4 raw = rows[j][i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        acc[2 * q] += w[j] * f.x;
        acc[2 * q + 1] += w[j] * f.y;
        dot[j] += gv[2 * q] * f.x + gv[2 * q + 1] * f.y;
      }
    }
    if (out) {
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out + (size_t)t * H)[i] = o;
    }
  }
  if (dots) {
    for (int j = 0; j < K; ++j) {
      float v = warp_sum(dot[j]);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
      __syncthreads();
      if (threadIdx.x == 0) {
        float s = 0.f;
        for (int wv = 0; wv < (int)(blockDim.x >> 5); ++wv) s += red[wv];
        dots[(size_t)t * K + j] = s;
      }
    }
  }
}

}  // namespace msb

using namespace msb;

static int check_router(const char* what, int T, int E, int K) {
  if (T <= 0 || E <= 0 || E > kMaxExperts || K <= 0 || K > kMaxChoices || K > E) {
    set_last_error("%s: need T > 0, 0 < E <= %d, 0 < K <= min(E, %d); got T=%d E=%d K=%d", what, kMaxExperts,
                   kMaxChoices, T, E, K);
    return kBadArg;
  }
  return kOk;
}

// scan: device scratch of ceil(T/256) * E 8-byte words; ticket: one int.  Both are cleared here.
MSB_EXPORT int msb_moe_router_step(const float* logits, int* expert, int* slot, float* gate, int* fill, float* proxy,
                                   float* density, float* loss, void* scan, int* ticket, int T, int E, int K,
                                   int step, int capacity, void* stream_) {
  if (int rc = check_router("moe_router_step", T, E, K)) return rc;
  if (step < 0 || step >= K) { set_last_error("moe_router_step: step %d outside [0, %d)", step, K); return kBadArg; }
  cudaStream_t stream = (cudaStream_t)stream_;
  const int blocks = (T + kRouterThreads - 1) / kRouterThreads;
  MSB_CUDA_CHECK(cudaMemsetAsync(scan, 0, sizeof(unsigned long long) * (size_t)blocks * E, stream));
  MSB_CUDA_CHECK(cudaMemsetAsync(ticket, 0, sizeof(int), stream));
  RouterParams p{logits, expert, slot, gate, fill, proxy, (unsigned long long*)scan, ticket,
                 T, E, K, step, capacity, status_ptr()};
  moe_router_step_kernel<<<blocks, kRouterThreads, 0, stream>>>(p);
  moe_router_finish_kernel<<<1, kMaxExperts, 0, stream>>>((const unsigned long long*)scan, blocks, fill, proxy,
                                                          density, loss, T, E, step, capacity);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_moe_router_weights(const float* gate, float* weight, int T, int K, void* stream) {
  moe_router_weights_kernel<<<(T + 255) / 256, 256, 0, (cudaStream_t)stream>>>(gate, weight, T, K);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_moe_router_bwd(const float* logits, const int* expert, const int* slot, const float* gate,
                                  const float* dweight, const float* dloss, const float* density, float* dlogits,
                                  int T, int E, int K, void* stream) {
  if (int rc = check_router("moe_router_bwd", T, E, K)) return rc;
  moe_router_bwd_kernel<<<(T + 127) / 128, 128, 0, (cudaStream_t)stream>>>(logits, expert, slot, gate, dweight,
                                                                           dloss, density, dlogits, T, E, K);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

static int check_rows(const char* what, int T, int K, int H, int EL, int n_src, int me, int C) {
  if (T < 0 || K <= 0 || K > kMaxChoices || H <= 0 || H % 8 || EL <= 0 || n_src <= 0 || n_src > kMoeMaxRanks ||
      me < 0 || me >= n_src || C <= 0) {
    set_last_error("%s: bad arguments T=%d K=%d H=%d (multiple of 8) experts/rank=%d ranks=%d me=%d capacity=%d",
                   what, T, K, H, EL, n_src, me, C);
    return kBadArg;
  }
  return kOk;
}

MSB_EXPORT int msb_moe_scatter_rows(const void* src, const float* scale, const int* expert, const int* slot,
                                    const unsigned long long* dst_ptrs, int T, int K, int H, int EL, int n_src,
                                    int me, int C, void* stream) {
  if (int rc = check_rows("moe_scatter_rows", T, K, H, EL, n_src, me, C)) return rc;
  if (T == 0) return kOk;
  MoePeers peers;
  for (int r = 0; r < kMoeMaxRanks; ++r) peers.p[r] = r < n_src ? (void*)dst_ptrs[r] : nullptr;
  moe_scatter_rows_kernel<<<T, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, scale, expert, slot, peers,
                                                               T, K, H, EL, n_src, me, C);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_moe_gather_rows(const unsigned long long* src_ptrs, const float* scale, const int* expert,
                                   const int* slot, const void* g, void* out, float* dots, int T, int K, int H,
                                   int EL, int n_src, int me, int C, void* stream) {
  if (int rc = check_rows("moe_gather_rows", T, K, H, EL, n_src, me, C)) return rc;
  if (T == 0) return kOk;
  MoePeers peers;
  for (int r = 0; r < kMoeMaxRanks; ++r) peers.p[r] = r < n_src ? (void*)src_ptrs[r] : nullptr;
  moe_gather_rows_kernel<<<T, 128, 0, (cudaStream_t)stream>>>(peers, scale, expert, slot, (const __nv_bfloat16*)g,
                                                              (__nv_bfloat16*)out, dots, T, K, H, EL, n_src, me, C);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
