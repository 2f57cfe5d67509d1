// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2, one 256 x 256 output tile per two SMs.
//
//   C[m][n] (+)= sum_k A[m][k] * B[n][k]       (operand storage flags as in gemm_sm100.cu)
//
// The two CTAs of a cluster share a tile: CTA r loads rows [m0 + 128 r, +128) of A and rows [n0 + 128 r, +128) of B
// (each CTA issues its own plain TMA loads), the leader (rank 0) issues one MMA per 16-wide k-step that reads
// both CTAs' shared memory and writes 128 accumulator lanes x 256 columns into each CTA's tensor memory, and each
// CTA drains and stores its own 128 rows.  Per k-block a CTA stages 32 KB instead of the 48 KB a lone CTA needs for
// a 128 x 256 tile, so the ring holds six stages instead of four.
//
// Synchronisation (every wait is bounded; a wait that runs out sets the status word and the CTA leaves):
//   full[s]      : in the leader; the TMA loads of BOTH CTAs count their bytes on it (.cta_group::2 loads may signal
//                  a barrier of the partner CTA), so the MMA thread waits once per stage.  A first version had the
//                  partner forward "my half has landed" with mbarrier.arrive.release.cluster from a relay thread;
//                  the release fence cost ~1 us per k-block and halved the throughput (660 vs 1230 TFLOP/s at 8192^3).
//   empty[s]     : in both CTAs; tcgen05.commit of the leader (multicast to the pair) releases the stage
//   tfull[a]     : in both CTAs; commit after the last k-block: accumulator a is complete
//   tempty[a]    : in the leader; 256 arrivals - the 128 epilogue threads of each CTA have drained accumulator a
#include <cooperative_groups.h>

#include "host_common.h"
#include "ptx.cuh"

namespace msb {

namespace cg = cooperative_groups;

constexpr int k2BM = 128;        // rows per CTA (tile M = 256)
constexpr int k2BN = 256;        // tile N (each CTA stages 128 of them)
constexpr int k2BK = 64;
constexpr int k2Threads = 192;
constexpr int k2Stages = 6;
constexpr int k2ABytes = k2BM * k2BK * 2;          // 16 KB
constexpr int k2BBytes = (k2BN / 2) * k2BK * 2;    // 16 KB
constexpr int k2StageBytes = k2ABytes + k2BBytes;
constexpr int k2StagingOffset = k2Stages * k2StageBytes;
constexpr int k2StagingBytes = 4 * 4096;
constexpr int k2BarOffset = k2StagingOffset + k2StagingBytes;
constexpr int k2SmemBytes = k2BarOffset + 512 + 1024;

struct Gemm2Params {
  const void* bias;
  int* status;
  int* debug;          // optional: [4] tensor-memory addresses returned to rank 0 / rank 1
  int M, N, K;
  int out_fp32, accumulate;
  float alpha;
  // split-K: every output tile is ksplit work items, item j covering k-blocks [j, j+1) * num_kb / ksplit; each item
  // adds its partial product into C with the TMA reduce epilogue (fp32 accumulate only).  It shortens the last,
  // partly filled round of tiles when the tile count is a poor multiple of the number of CTA pairs.
  int ksplit;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// address of `local_smem_addr` (shared::cta window of this CTA) as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_smem_addr), "r"(rank));
  return a;
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ uint32_t ld_remote_u32(uint32_t cluster_addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}
// Non-suspending test of a barrier that is signalled from the partner CTA (remote arrive, or the leader's
// tcgen05.commit): acquire at cluster scope.  try_wait may park the thread, and a parked thread was not woken
// promptly by remote arrivals.
__device__ __forceinline__ bool mbar_test_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, const AbortCtx& ab) {
#pragma unroll 1
  for (int i = 0; i < 256; ++i) {
    if (mbar_test_cluster(bar, parity)) return true;
  }
  const unsigned long long t0 = globaltimer_ns();
#pragma unroll 1
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 512; ++i) {
      if (mbar_test_cluster(bar, parity)) return true;
    }
    if (*ab.cta_abort) return false;
    if (globaltimer_ns() - t0 > kWaitLimitNs) {
      *ab.cta_abort = 1;
      atomicOr(ab.gstatus, 1);
      return false;
    }
  }
}

__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in both CTAs of the pair once the issued MMAs have finished
__device__ __forceinline__ void umma2_commit_pair(uint64_t* bar) {
  const uint16_t mask = 0x3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}
// 3-D tiled load into this CTA's shared memory whose bytes are counted on the mbarrier at `bar_cluster_addr`, an
// address in the cluster window: with .cta_group::2 that barrier may live in the partner CTA, so both halves of a
// stage complete on the leader's barrier and no thread has to forward "my half has landed".
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr,
                                                 int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d_2(const CUtensorMap* tmap, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d_2(const CUtensorMap* tmap, const void* smem_src, int x, int y,
                                                    int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}

template <bool A_MN, bool B_MN, int ACC>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(k2Threads, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, const Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + k2Stages * k2ABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + k2BarOffset);
  uint64_t* empty_bar = full_bar + k2Stages;
  uint64_t* tfull_bar = empty_bar + k2Stages;     // [2]
  uint64_t* tempty_bar = tfull_bar + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const AbortCtx ab{cta_abort, p.status};
  cg::cluster_group cluster = cg::this_cluster();

  const int tiles_m = (p.M + 2 * k2BM - 1) / (2 * k2BM);
  const int tiles_n = (p.N + k2BN - 1) / k2BN;
  const int ksplit = p.ksplit;
  const int total_tiles = tiles_m * tiles_n * ksplit;      // work items
  const int num_kb = (p.K + k2BK - 1) / k2BK;
  const int pairs = gridDim.x / 2;
  const int pair = blockIdx.x / 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < k2Stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 256);
    }
    *cta_abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, ACC * k2BN);
    tmem_relinquish2();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster.sync();                       // both CTAs' barriers and tensor-memory slots are ready
  tc_fence_after_sync();
  // the MMA of the leader addresses the accumulator in both CTAs by the leader's allocation
  const uint32_t my_alloc = *tmem_slot;
  const uint32_t tmem_base = leader ? my_alloc : ld_remote_u32(map_to_rank(smem_u32(tmem_slot), 0));
  if (p.debug && threadIdx.x == 0 && pair == 0) {
    p.debug[rank * 2] = static_cast<int>(my_alloc);
    p.debug[rank * 2 + 1] = static_cast<int>(tmem_base);
  }

  // k-block range [kb0, kb1) of a work item
  auto k_range = [&](int item, int& kb0, int& kb1) {
    const int ks = item % ksplit;
    kb0 = static_cast<int>(static_cast<long long>(ks) * num_kb / ksplit);
    kb1 = static_cast<int>(static_cast<long long>(ks + 1) * num_kb / ksplit);
  };
  auto tile_coords = [&](int item, int& m_blk, int& n_blk) {
    const int tile = item / ksplit;
    const int group_sz = 4 * tiles_n;            // groups of 4 m-tiles share B tiles in L2
    const int g = tile / group_sz;
    const int first_m = g * 4;
    const int gm = min(tiles_m - first_m, 4);
    const int r = tile - g * group_sz;
    m_blk = first_m + r % gm;
    n_blk = r / gm;
  };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer (each CTA, own halves)
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += pairs) {
        int m_blk, n_blk;
        tile_coords(tile, m_blk, n_blk);
        const int m0 = m_blk * 2 * k2BM + static_cast<int>(rank) * k2BM;
        const int n0 = n_blk * k2BN + static_cast<int>(rank) * (k2BN / 2);
        int kb0, kb1;
        k_range(tile, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_cluster(&empty_bar[s], ph ^ 1, ab)) { ok = false; break; }
          // both CTAs' bytes are counted on the leader's barrier; only the leader announces them
          if (leader) mbar_expect_tx(&full_bar[s], 2 * k2StageBytes);
          const uint32_t bar = map_to_rank(smem_u32(&full_bar[s]), 0);
          uint8_t* a_dst = smem_a + s * k2ABytes;
          uint8_t* b_dst = smem_b + s * k2BBytes;
          const int k0 = kb * k2BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < k2BM / 64; ++j) tma_load_3d_pair(a_dst + j * 8192, &tmA, bar, m0 + 64 * j, k0, 0);
          } else {
            tma_load_3d_pair(a_dst, &tmA, bar, k0, m0, 0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < k2BN / 128; ++j) tma_load_3d_pair(b_dst + j * 8192, &tmB, bar, n0 + 64 * j, k0, 0);
          } else {
            tma_load_3d_pair(b_dst, &tmB, bar, k0, n0, 0);
          }
          if (++s == k2Stages) { s = 0; ph ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      if (leader) {
        // ---------------------------------------------------------------- MMA issuer (leader CTA)
        constexpr uint32_t idesc = umma_idesc_bf16(2 * k2BM, k2BN, A_MN, B_MN);
        int s = 0;
        uint32_t ph = 0;
        int it = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles && ok; tile += pairs, ++it) {
          const int acc = ACC == 2 ? (it & 1) : 0;
          const uint32_t acc_ph = ACC == 2 ? ((it >> 1) & 1) : (it & 1);
          if (!mbar_wait_cluster(&tempty_bar[acc], acc_ph ^ 1, ab)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + acc * k2BN;
          int kb0, kb1;
          k_range(tile, kb0, kb1);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(&full_bar[s], ph, ab)) { ok = false; break; }      // both CTAs' halves have landed
            tc_fence_after_sync();
            const uint32_t a_addr = smem_u32(smem_a + s * k2ABytes);
            const uint32_t b_addr = smem_u32(smem_b + s * k2BBytes);
#pragma unroll
            for (int kk = 0; kk < k2BK / 16; ++kk) {
              const uint64_t adesc = A_MN ? umma_smem_desc(a_addr + kk * 2048, 8192, 1024)
                                          : umma_smem_desc(a_addr + kk * 32, 16, 1024);
              const uint64_t bdesc = B_MN ? umma_smem_desc(b_addr + kk * 2048, 8192, 1024)
                                          : umma_smem_desc(b_addr + kk * 32, 16, 1024);
              umma2_bf16(d_tmem, adesc, bdesc, idesc, ((kb - kb0) | kk) != 0);
            }
            umma2_commit_pair(&empty_bar[s]);
            if (++s == k2Stages) { s = 0; ph ^= 1; }
          }
          if (ok) umma2_commit_pair(&tfull_bar[acc]);
        }
      }
    }
    __syncwarp();
  } else {
    // -------------------------------------------------------------------- epilogue (each CTA, its 128 rows)
    const int q = warp & 3;
    int it = 0;
    bool ok = true;
    uint8_t* stage_base = smem + k2StagingOffset + q * 4096;
    const uint32_t tempty_leader0 = map_to_rank(smem_u32(&tempty_bar[0]), 0);
    const uint32_t tempty_leader1 = map_to_rank(smem_u32(&tempty_bar[1]), 0);
    const int sw = lane & 7;
    for (int tile = pair; tile < total_tiles && ok; tile += pairs, ++it) {
      int m_blk, n_blk;
      tile_coords(tile, m_blk, n_blk);
      const int acc = ACC == 2 ? (it & 1) : 0;
      const uint32_t acc_ph = ACC == 2 ? ((it >> 1) & 1) : (it & 1);
      if (!mbar_wait_cluster(&tfull_bar[acc], acc_ph, ab)) { ok = false; break; }
      tc_fence_after_sync();
      const int row0 = m_blk * 2 * k2BM + static_cast<int>(rank) * k2BM + q * 32;
      const int n0 = n_blk * k2BN;
      const uint32_t t_row = tmem_base + acc * k2BN + (static_cast<uint32_t>(q * 32) << 16);
      int nbuf = 0;
#pragma unroll 1
      for (int c = 0; c < k2BN; c += 32) {
        if (n0 + c >= p.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(t_row + c, r);
        tmem_ld_wait();
        const int col0 = n0 + c;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        if (p.bias) {
          const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(p.bias);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) v[j] += __bfloat162float(bias[col0 + j]);
        }
        uint8_t* rowp = stage_base + lane * 128;
        if (p.out_fp32) {
          if (nbuf >= 1) tma_store_wait_read<0>();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(rowp + ((j ^ sw) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2],
                                                                             v[4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (p.accumulate) tma_reduce_add_3d_2(&tmC, stage_base, col0, row0, 0);
            else tma_store_3d_2(&tmC, stage_base, col0, row0, 0);
            tma_store_commit();
          }
          ++nbuf;
        } else {
          const int half = (c >> 5) & 1;
          if (half == 0) {
            if (nbuf >= 1) tma_store_wait_read<0>();
            __syncwarp();
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
            o.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
            o.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
            o.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
            *reinterpret_cast<uint4*>(rowp + (((half * 4 + j) ^ sw) << 4)) = o;
          }
          const bool last = (c + 32 >= k2BN) || (n0 + c + 32 >= p.N);
          if (half == 1 || last) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d_2(&tmC, stage_base, col0 - half * 32, row0, 0);
              tma_store_commit();
            }
            ++nbuf;
          }
        }
      }
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
      tc_fence_before_sync();
      remote_arrive(acc == 0 ? tempty_leader0 : tempty_leader1);   // the leader's barrier counts both CTAs
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  cluster.sync();          // the partner no longer reads this CTA's shared memory or signals its barriers
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc2(my_alloc, ACC * k2BN);
  }
}

}  // namespace msb

using namespace msb;

static int g_pair_splitk_auto = 1;

// 1 (default): accumulating fp32 GEMMs choose a split-K factor by themselves; 0: never split.
MSB_EXPORT void msb_gemm_pair_set_splitk(int enabled) { g_pair_splitk_auto = enabled ? 1 : 0; }

template <bool A_MN, bool B_MN, int ACC>
static int launch_gemm2(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const Gemm2Params& p,
                        cudaStream_t stream) {
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, ACC>;
  static bool configured = false;
  if (!configured) {
    MSB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, k2SmemBytes));
    configured = true;
  }
  // The kernel is persistent: every cluster must be resident at once.  How many 2-CTA clusters fit depends on how
  // the SMs are grouped (a group with an odd number of SMs leaves one unpaired), so ask the runtime.
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sm_count() / 2), 1, 1);
    cfg.blockDim = dim3(k2Threads, 1, 1);
    cfg.dynamicSmemBytes = k2SmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    MSB_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    if (n <= 0) { set_last_error("gemm_pair: no 2-CTA cluster of this kernel can be resident"); return kCudaError; }
    max_pairs = n;
  }
  const int tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256);
  Gemm2Params q = p;
  q.ksplit = 1;
  if (p.ksplit == 0 && p.accumulate && p.out_fp32 && !p.bias && g_pair_splitk_auto) {
    // pick the split with the fewest (rounds x length): rounds = ceil(tiles * s / pairs), each 1/s long, plus a
    // per-item cost of about two k-blocks for the pipeline fill and the read-modify-write epilogue
    const int num_kb = (p.K + k2BK - 1) / k2BK;
    double best = 1e30;
    for (int s = 1; s <= 4; ++s) {
      if (num_kb / s < 8) break;
      const int rounds = (tiles * s + max_pairs - 1) / max_pairs;
      const double cost = rounds * (static_cast<double>(num_kb) / s + 2.0);
      if (cost < best * 0.97) { best = cost; q.ksplit = s; }
    }
  } else if (p.ksplit > 1) {
    if (!(p.accumulate && p.out_fp32)) {
      set_last_error("gemm_pair: split-K needs an fp32 output that is accumulated into");
      return kBadArg;
    }
    q.ksplit = p.ksplit;
  }
  const int items = tiles * q.ksplit;
  int pairs = max_pairs;
  if (items < pairs) pairs = items;
  kern<<<2 * pairs, k2Threads, k2SmemBytes, stream>>>(tmA, tmB, tmC, q);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// C (+)= alpha * A x B^T (+ bias) with CTA pairs.  Same operand conventions as msb_gemm_bf16 (no batch).  The output
// must satisfy the TMA rules (16-byte aligned base and row pitch); bf16 accumulation is not supported.
// acc_buffers: 1 or 2 accumulators in tensor memory.  debug: optional int[4] (device) receiving tensor-memory
// addresses.
MSB_EXPORT int msb_gemm_bf16_pair(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                                  int a_mn, int b_mn, long long lda, long long ldb, long long ldc, int out_fp32,
                                  int accumulate, float alpha, int acc_buffers, int* debug, void* stream_) {
  if (M <= 0 || N <= 0 || K <= 0) { set_last_error("gemm_pair: empty problem"); return kBadArg; }
  if ((lda % 8) || (ldb % 8)) { set_last_error("gemm_pair: operand pitches must be multiples of 8"); return kBadArg; }
  const int es = out_fp32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || ((ldc * es) & 15) || (accumulate && !out_fp32)) {
    set_last_error("gemm_pair: output needs a 16-byte aligned base and pitch, and fp32 when accumulating");
    return kBadArg;
  }
  if (acc_buffers != 1 && acc_buffers != 2) { set_last_error("gemm_pair: acc_buffers must be 1 or 2"); return kBadArg; }
  Gemm2Params p = {};
  p.bias = bias; p.status = status_ptr(); p.debug = debug;
  if (!p.status) { set_last_error("gemm_pair: no status word"); return kCudaError; }
  p.M = M; p.N = N; p.K = K; p.out_fp32 = out_fp32; p.accumulate = accumulate; p.alpha = alpha;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if (a_mn) rc = encode_tmap_3d(&tmA, A, 2, M, K, 1, lda * 2, (uint64_t)lda * 2 * K, 64, 64, 1);
  else      rc = encode_tmap_3d(&tmA, A, 2, K, M, 1, lda * 2, (uint64_t)lda * 2 * M, 64, k2BM, 1);
  if (rc) return rc;
  if (b_mn) rc = encode_tmap_3d(&tmB, B, 2, N, K, 1, ldb * 2, (uint64_t)ldb * 2 * K, 64, 64, 1);
  else      rc = encode_tmap_3d(&tmB, B, 2, K, N, 1, ldb * 2, (uint64_t)ldb * 2 * N, 64, k2BN / 2, 1);
  if (rc) return rc;
  if ((rc = encode_tmap_3d(&tmC, C, es, N, M, 1, (uint64_t)ldc * es, (uint64_t)ldc * es * M, 128 / es, 32, 1))) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
#define MSB_PAIR(ACC_)                                                                     \
  if (a_mn) {                                                                              \
    if (b_mn) return launch_gemm2<true, true, ACC_>(tmA, tmB, tmC, p, stream);             \
    return launch_gemm2<true, false, ACC_>(tmA, tmB, tmC, p, stream);                      \
  } else {                                                                                 \
    if (b_mn) return launch_gemm2<false, true, ACC_>(tmA, tmB, tmC, p, stream);            \
    return launch_gemm2<false, false, ACC_>(tmA, tmB, tmC, p, stream);                     \
  }
  if (acc_buffers == 2) { MSB_PAIR(2) } else { MSB_PAIR(1) }
#undef MSB_PAIR
}
