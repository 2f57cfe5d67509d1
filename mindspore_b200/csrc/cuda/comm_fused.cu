// NVLink collectives over symmetric memory (peer pointers obtained once per group), written for one 8-GPU
// NVSwitch box.  All cross-GPU synchronisation is a stream-ordered barrier kernel whose waits are bounded; data
// kernels never wait on a peer.
//
//   msb_symm_barrier        : all ranks of the group rendezvous (flag exchange through peer stores)
//   msb_allreduce_symm      : two-shot all-reduce of a bucket held in symmetric memory: rank r sums slice r over
//                             all peers (peer loads), applies the 1/N or loss-scale factor, optionally checks
//                             finiteness, and writes the result into every peer's buffer (peer stores)
//   msb_reduce_slots        : sums the mp partial slices that peers pushed into this rank's staging buffer
//                             (second half of the fused MatMul->ReduceScatter; the first half is the GEMM epilogue
//                             storing its tiles straight into the owner's staging buffer, see gemm_sm100.cu)
//   msb_reduce_scatter_adamw: parallel-optimizer step on a gradient bucket: rank r sums its 1/N slice over peers,
//                             unscales, updates fp32 master + moments (AdamW) and writes the new bf16 weights of
//                             its slice into every peer's weight buffer - ReduceScatter + cast/scale + AdamW +
//                             parameter AllGather in one pass over the slice.
//
// The reference issues ncclAllReduce / ncclReduceScatter / ncclAllGather as separate kernels
// (plugin/device/gpu/kernel/nccl/nccl_collective_gpu_kernel.h:143-178) followed by separate Cast, Mul and
// AdamWeightDecay kernels.
#include "host_common.h"
#include "ptx.cuh"

namespace msb {

constexpr int kMaxRanks = 8;

struct PeerPtrs {
  void* p[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// pads.p[r] -> int[channels * world] flag words followed by int[channels] epoch counters on rank r.  The epoch
// lives in device memory and is advanced by the kernel itself, so the barrier can be captured in a CUDA graph
// and replayed.  Thread t tells peer t "rank `rank` reached epoch e", then waits until every peer has told us
// the same.  A wait that runs past the limit sets status bit 2 and returns.
__global__ void symm_barrier_kernel(PeerPtrs pads, int rank, int world, int channel, int channels, int* status) {
  __shared__ int epoch_s;
  const int t = threadIdx.x;
  if (t == 0) {
    int* ep = static_cast<int*>(pads.p[rank]) + channels * world + channel;
    epoch_s = *ep + 1;
    *ep = epoch_s;
  }
  __syncthreads();
  const int epoch = epoch_s;
  if (t >= world) return;
  __threadfence_system();
  int* remote = static_cast<int*>(pads.p[t]) + channel * world + rank;
  st_release_sys(remote, epoch);
  const int* mine = static_cast<const int*>(pads.p[rank]) + channel * world + t;
  const unsigned long long t0 = globaltimer_ns();
  while (ld_acquire_sys(mine) < epoch) {
    if (globaltimer_ns() - t0 > kWaitLimitNs) {
      atomicOr(status, 2);
      break;
    }
  }
  __threadfence_system();
}

// bufs.p[r]: fp32 buffer of n elements on rank r (same offset on every rank).
__global__ void allreduce_symm_kernel(PeerPtrs bufs, int rank, int world, long long n, float scale,
                                      int* nonfinite) {
  const long long per = ((n + world - 1) / world + 3) & ~3LL;
  const long long lo = per * rank;
  const long long hi = lo + per < n ? lo + per : n;
  bool bad = false;
  for (long long i = lo + (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < hi;
       i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= hi) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r < world) {
          const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(bufs.p[r]) + i);
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
      }
      acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
      bad |= !(isfinite(acc.x) && isfinite(acc.y) && isfinite(acc.z) && isfinite(acc.w));
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < world) *reinterpret_cast<float4*>(static_cast<float*>(bufs.p[r]) + i) = acc;
    } else {
      for (long long k = i; k < hi; ++k) {
        float a = 0.f;
        for (int r = 0; r < world; ++r) a += static_cast<const float*>(bufs.p[r])[k];
        a *= scale;
        bad |= !isfinite(a);
        for (int r = 0; r < world; ++r) static_cast<float*>(bufs.p[r])[k] = a;
      }
    }
  }
  if (bad && nonfinite) atomicOr(nonfinite, 1);
}

// stage: [slots][rows*cols] bf16 -> out[rows*cols] = sum over slots (fp32 accumulation)
__global__ void reduce_slots_kernel(const __nv_bfloat16* __restrict__ stage, __nv_bfloat16* __restrict__ out,
                                    int slots, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < slots; ++s) {
      const uint4 raw = reinterpret_cast<const uint4*>(stage + s * n8 * 8)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// Parallel-optimizer step for one bucket of n elements whose fp32 gradients sit at the same offset of every
// rank's symmetric gradient buffer and whose bf16 weights sit at the same offset of every rank's symmetric weight
// buffer.  Rank r owns elements [r*per, (r+1)*per): master/m/v hold only that slice (per elements).
// hyper: {lr, beta1, beta2, eps, weight_decay, 1-beta1^t, 1-beta2^t, grad_scale}
__global__ void reduce_scatter_adamw_kernel(PeerPtrs grads, PeerPtrs weights, float* __restrict__ master,
                                            float* __restrict__ m, float* __restrict__ v, int rank, int world,
                                            long long per, const float* __restrict__ hyper,
                                            const int* __restrict__ skip) {
  if (skip && *skip) return;
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4];
  const float bc1 = hyper[5], bc2 = hyper[6], gs = hyper[7];
  const float step = lr / bc1, rsq = rsqrtf(bc2);
  const long long base = per * rank;
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < per;
       i += (long long)gridDim.x * blockDim.x * 4) {
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r < world) {
        const float4 t = *reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[r]) + base + i);
        g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
      }
    }
    float4 p4 = *reinterpret_cast<float4*>(master + i);
    float4 m4 = *reinterpret_cast<float4*>(m + i);
    float4 v4 = *reinterpret_cast<float4*>(v + i);
    float* gg = reinterpret_cast<float*>(&g);
    float* pp = reinterpret_cast<float*>(&p4);
    float* mm = reinterpret_cast<float*>(&m4);
    float* vv = reinterpret_cast<float*>(&v4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gg[j] * gs;
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      pp[j] = pp[j] * (1.f - lr * wd) - step * mm[j] / (sqrtf(vv[j]) * rsq + eps);
    }
    *reinterpret_cast<float4*>(master + i) = p4;
    *reinterpret_cast<float4*>(m + i) = m4;
    *reinterpret_cast<float4*>(v + i) = v4;
    uint2 o;
    o.x = pack_bf16x2(pp[0], pp[1]);
    o.y = pack_bf16x2(pp[2], pp[3]);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < world) *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(weights.p[r]) + base + i) = o;
  }
}

// First half of the sharded optimizer step with gradient clipping: rank r replaces elements [base, base+n) of its
// own gradient buffer by scale * (sum over all ranks' buffers of the same elements).  Peers only ever read the
// slices they own, so the in-place write does not race with their loads.
__global__ void reduce_scatter_symm_kernel(PeerPtrs grads, int rank, int world, long long base, long long n,
                                           float scale) {
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r < world) {
        const float4 t = *reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[r]) + base + i);
        g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
      }
    }
    g.x *= scale; g.y *= scale; g.z *= scale; g.w *= scale;
    *reinterpret_cast<float4*>(static_cast<float*>(grads.p[rank]) + base + i) = g;
  }
}

// Second half: AdamW on n owned elements (master / m / v / grad are local, already offset) and the new bf16 weights
// written into every rank's weight buffer at element offset `base` (the parameter AllGather).
__global__ void adamw_allgather_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                       const float* __restrict__ grad, PeerPtrs weights, int world, long long base,
                                       long long n, const float* __restrict__ hyper, const int* __restrict__ skip) {
  if (skip && *skip) return;
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4];
  const float bc1 = hyper[5], bc2 = hyper[6], gs = hyper[7];
  const float step = lr / bc1, rsq = rsqrtf(bc2);
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    float4 g4 = *reinterpret_cast<const float4*>(grad + i);
    float4 p4 = *reinterpret_cast<float4*>(master + i);
    float4 m4 = *reinterpret_cast<float4*>(m + i);
    float4 v4 = *reinterpret_cast<float4*>(v + i);
    float* gg = reinterpret_cast<float*>(&g4);
    float* pp = reinterpret_cast<float*>(&p4);
    float* mm = reinterpret_cast<float*>(&m4);
    float* vv = reinterpret_cast<float*>(&v4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gg[j] * gs;
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      pp[j] = pp[j] * (1.f - lr * wd) - step * mm[j] / (sqrtf(vv[j]) * rsq + eps);
    }
    *reinterpret_cast<float4*>(master + i) = p4;
    *reinterpret_cast<float4*>(m + i) = m4;
    *reinterpret_cast<float4*>(v + i) = v4;
    uint2 o;
    o.x = pack_bf16x2(pp[0], pp[1]);
    o.y = pack_bf16x2(pp[2], pp[3]);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < world) *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(weights.p[r]) + base + i) = o;
  }
}

static int fill_peers(PeerPtrs* out, const unsigned long long* ptrs, int world, const char* what) {
  if (world < 1 || world > kMaxRanks) {
    set_last_error("%s: group size %d is outside [1, %d]", what, world, kMaxRanks);
    return kBadArg;
  }
  for (int i = 0; i < kMaxRanks; ++i) out->p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return kOk;
}

}  // namespace msb

using namespace msb;

MSB_EXPORT int msb_symm_barrier(const unsigned long long* pad_ptrs, int rank, int world, int channel, int channels,
                                void* stream) {
  PeerPtrs pads;
  if (int rc = fill_peers(&pads, pad_ptrs, world, "symm_barrier")) return rc;
  int* status = status_ptr();
  if (!status) { set_last_error("symm_barrier: no status word"); return kCudaError; }
  symm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pads, rank, world, channel, channels, status);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_allreduce_symm(const unsigned long long* buf_ptrs, int rank, int world, long long n, float scale,
                                  int* nonfinite, void* stream) {
  PeerPtrs bufs;
  if (int rc = fill_peers(&bufs, buf_ptrs, world, "allreduce_symm")) return rc;
  for (int r = 0; r < world; ++r)
    if (buf_ptrs[r] & 15) { set_last_error("allreduce_symm: buffers must be 16-byte aligned"); return kBadArg; }
  if (n <= 0) return kOk;
  const long long per = (n + world - 1) / world;
  long long blocks = (per / 4 + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 4;
  blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
  allreduce_symm_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      bufs, rank, world, n, scale, nonfinite);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_reduce_slots(const void* stage, void* out, int slots, long long n, void* stream) {
  if (n % 8) { set_last_error("reduce_slots: n=%lld must be a multiple of 8", n); return kBadArg; }
  if (n <= 0) return kOk;
  long long blocks = (n / 8 + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  blocks = blocks > cap ? cap : blocks;
  reduce_slots_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(stage), static_cast<__nv_bfloat16*>(out), slots, n / 8);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_reduce_scatter_adamw(const unsigned long long* grad_ptrs, const unsigned long long* weight_ptrs,
                                        float* master, float* m, float* v, int rank, int world, long long per,
                                        const float* hyper, const int* skip, void* stream) {
  PeerPtrs g, w;
  if (int rc = fill_peers(&g, grad_ptrs, world, "reduce_scatter_adamw")) return rc;
  if (int rc = fill_peers(&w, weight_ptrs, world, "reduce_scatter_adamw")) return rc;
  if (per % 4) { set_last_error("reduce_scatter_adamw: slice length %lld must be a multiple of 4", per); return kBadArg; }
  if (per <= 0) return kOk;
  long long blocks = (per / 4 + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 4;
  blocks = blocks > cap ? cap : blocks;
  reduce_scatter_adamw_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      g, w, master, m, v, rank, world, per, hyper, skip);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

static unsigned ew_blocks(long long n4) {
  long long blocks = (n4 + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 4;
  blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
  return static_cast<unsigned>(blocks);
}

MSB_EXPORT int msb_reduce_scatter_symm(const unsigned long long* grad_ptrs, int rank, int world, long long base,
                                       long long n, float scale, void* stream) {
  PeerPtrs g;
  if (int rc = fill_peers(&g, grad_ptrs, world, "reduce_scatter_symm")) return rc;
  if ((n % 4) || (base % 4)) {
    set_last_error("reduce_scatter_symm: base %lld and length %lld must be multiples of 4", base, n);
    return kBadArg;
  }
  if (n <= 0) return kOk;
  reduce_scatter_symm_kernel<<<ew_blocks(n / 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(g, rank, world, base, n,
                                                                                              scale);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

MSB_EXPORT int msb_adamw_allgather(float* master, float* m, float* v, const float* grad,
                                   const unsigned long long* weight_ptrs, int world, long long base, long long n,
                                   const float* hyper, const int* skip, void* stream) {
  PeerPtrs w;
  if (int rc = fill_peers(&w, weight_ptrs, world, "adamw_allgather")) return rc;
  if ((n % 4) || (base % 4)) {
    set_last_error("adamw_allgather: base %lld and length %lld must be multiples of 4", base, n);
    return kBadArg;
  }
  if (n <= 0) return kOk;
  adamw_allgather_kernel<<<ew_blocks(n / 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(master, m, v, grad, w, world,
                                                                                          base, n, hyper, skip);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
