// bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
//   C[b][m][n] (+)= sum_k A[b][m][k] * B[b][n][k]   (+ bias[n])
//
// Either operand may be stored "K-major" (reduction dim contiguous) or "MN-major"
// (the M, resp. N, dim contiguous); the three GEMMs of a Dense layer map to
//   forward  Y  = X  W^T : A = X  (K-major),  B = W (K-major)
//   dgrad    dX = dY W   : A = dY (K-major),  B = W (MN-major)
//   wgrad    dW = dY^T X : A = dY (MN-major), B = X (MN-major)
// with no transposed copies.  This replaces the cublasGemmEx/StridedBatchedEx calls of
// plugin/device/gpu/kernel/math/matmul_gpu_kernel.cc:163-181 in the reference.
//
// Persistent kernel, one CTA per SM, 192 threads:
//   warp 0    : TMA producer (one lane)
//   warp 1    : TMEM allocation + MMA issue (one lane)
//   warps 2-5 : epilogue; warp w drains TMEM lanes 32*(w%4)..+31
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of tile i
// overlaps the main loop of tile i+1.  Shared-memory stages are recycled through
// full/empty mbarriers; tcgen05.commit releases a stage when the MMAs that read it retire.
#include "host_common.h"
#include "ptx.cuh"

namespace msb {

__device__ __forceinline__ bool row_ok_pre(int row, int M) { return row < M; }

constexpr int kBM = 128;       // tile rows (UMMA M)
constexpr int kBK = 64;        // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192;
constexpr int kGroupM = 8;     // m-tiles per scheduling group (L2 reuse of B tiles)

struct GemmParams {
  void* C;
  const void* bias;   // bf16 [N] or nullptr
  int* status;
  long long c_batch_stride;  // elements
  int M, N, K, batch;
  int ldc;            // elements
  int out_fp32;       // C is fp32 (else the operands' 16-bit type)
  int fp16;           // operands, bias and a 16-bit C are fp16 (else bf16)
  int accumulate;     // C += result (read-modify-write)
  float alpha;        // result scale applied before bias/accumulate
  // --- MatMul -> ReduceScatter (MODE 1): the epilogue stores each bf16 output tile straight into the staging
  // buffer of the rank that owns those token rows: rs_peer[owner] is bf16 [world][rows_per_rank][N] on `owner`.
  void* rs_peer[8];
  // --- AllGather -> MatMul (MODE 2): warp 6 of every CTA pulls its share of each peer's token shard
  // ag_src[c] ([rows_per_rank][K] bf16 on rank c) through shared memory into the local gathered operand ag_dst
  // ([world*rows_per_rank][K], what the A tensor map covers) and bumps ag_flags[c]; the TMA producer waits until
  // a chunk's counter reaches gridDim.x before it loads tiles of that chunk.
  const void* ag_src[8];
  void* ag_dst;
  int* ag_flags;
  // ag_in_kernel = 0: the chunks are brought in by the copy engines instead (peer -> local copies on side streams,
  // each followed by a copy of 1 into ag_flags[c]); warp 6 idles and a chunk is ready when its flag is >= 1.
  int ag_in_kernel, ag_flag_target;
  int world, rank, rows_per_rank;
  int rs_slot;        // MODE 1: which [rows_per_rank][N] slot of the owner's buffer this rank's rows go to
  // The epilogue stages 32 rows x 128 bytes per warp in shared memory (128-byte swizzle) and writes them with TMA
  // stores (fp32 accumulation = TMA reduce-add): full 128-byte lines instead of 16-byte fragments per row, which is
  // what makes stores into a peer's memory efficient.  0 = per-thread stores (unaligned C, bf16 accumulation).
  int tma_epilogue;
};

struct CMaps {
  CUtensorMap m[8];   // m[0]: C.  MatMul -> ReduceScatter: m[r] = staging buffer of rank r
};

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tmap, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* tmap, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read_n() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

constexpr int kBounceBytes = 8192;   // per bounce buffer of the AllGather copy warp (two buffers)

template <int BN>
struct GemmCfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // epilogue staging: 4 warps x (32 rows x 128 B), 1024-byte aligned (after the stage ring)
  static constexpr int kStagingOffset = kStages * kStageBytes;
  static constexpr int kStagingBytes = 4 * 4096;
  static constexpr int kBarOffset = kStagingOffset + kStagingBytes;
  static constexpr int kBounceOffset = kBarOffset + 256;
  static constexpr int kSmemBytes = kBarOffset + 256 + 1024;  // barriers + slack for 1024B alignment
  static constexpr int kSmemBytesAG = kBounceOffset + 2 * kBounceBytes + 1024;
};

// MODE: 0 plain GEMM, 1 MatMul->ReduceScatter push epilogue, 2 AllGather->MatMul pull loader.
template <int BN, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(MODE == 2 ? kGemmThreads + 32 : kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CMaps tmC, const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * Cfg::kABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;   // [2] accumulator ready for epilogue
  uint64_t* tempty_bar = tfull_bar + 2;        // [2] accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* issued_cnt = cta_abort + 1;    // k-blocks whose loads were issued
  volatile int* consumed_cnt = cta_abort + 2;  // k-blocks whose loads were observed complete

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AbortCtx ab{cta_abort, p.status};

  const int tiles_m = (p.M + kBM - 1) / kBM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_per_batch = tiles_m * tiles_n;
  const int total_tiles = tiles_per_batch * p.batch;
  const int num_kb = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    mbar_init(&tempty_bar[0], 128);
    mbar_init(&tempty_bar[1], 128);
    *cta_abort = 0;
    *issued_cnt = 0;
    *consumed_cnt = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_coords = [&](int tile, int& b, int& m_blk, int& n_blk) {
    b = tile / tiles_per_batch;
    int t = tile - b * tiles_per_batch;
    const int group_sz = kGroupM * tiles_n;
    const int g = t / group_sz;
    const int first_m = g * kGroupM;
    const int gm = min(tiles_m - first_m, kGroupM);
    const int r = t - g * group_sz;
    m_blk = first_m + r % gm;
    n_blk = r / gm;
    if (MODE != 0) {
      // start with the chunk whose data / destination is local-most: RS sends remote chunks first and keeps its
      // own chunk for last; AG starts on its own (already local) chunk while peers' chunks are in flight
      const int tiles_per_chunk = p.rows_per_rank / kBM;
      const int shift = (MODE == 1 ? (p.rank + 1) % p.world : p.rank) * tiles_per_chunk;
      m_blk = (m_blk + shift) % tiles_m;
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      int s = 0;
      uint32_t ph = 0;
      int issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int b, m_blk, n_blk;
        tile_coords(tile, b, m_blk, n_blk);
        const int m0 = m_blk * kBM, n0 = n_blk * BN;
        if (MODE == 2) {
          const int chunk = m0 / p.rows_per_rank;
          const volatile int* flag = p.ag_flags + chunk;
          const unsigned long long t0 = globaltimer_ns();
          while (*flag < p.ag_flag_target) {
            if (*cta_abort) { ok = false; break; }
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
              *cta_abort = 1;
              atomicOr(p.status, 2);
              ok = false;
              break;
            }
          }
          if (!ok) break;
          __threadfence();
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, ab)) { ok = false; break; }
          mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
          uint8_t* a_dst = smem_a + s * Cfg::kABytes;
          uint8_t* b_dst = smem_b + s * Cfg::kBBytes;
          const int k0 = kb * kBK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)
              tma_load_3d(a_dst + j * 8192, &tmA, &full_bar[s], m0 + 64 * j, k0, b);
          } else {
            tma_load_3d(a_dst, &tmA, &full_bar[s], k0, m0, b);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(b_dst + j * 8192, &tmB, &full_bar[s], n0 + 64 * j, k0, b);
          } else {
            tma_load_3d(b_dst, &tmB, &full_bar[s], k0, n0, b);
          }
          ++issued;
          *issued_cnt = issued;
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      const uint32_t idesc = p.fp16 ? umma_idesc_f16(kBM, BN, A_MN, B_MN) : umma_idesc_bf16(kBM, BN, A_MN, B_MN);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      int consumed = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, ab)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, ab)) { ok = false; break; }
          ++consumed;
          *consumed_cnt = consumed;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + s * Cfg::kABytes);
          const uint32_t b_addr = smem_u32(smem_b + s * Cfg::kBBytes);
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            // K-major: step 16 elements (32 B) inside the 128 B swizzle row.
            // MN-major: step 16 k-rows of 128 B (2048 B); 64-wide M/N groups are 8192 B apart.
            const uint64_t adesc = A_MN ? umma_smem_desc(a_addr + kk * 2048, 8192, 1024)
                                        : umma_smem_desc(a_addr + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(b_addr + kk * 2048, 8192, 1024)
                                        : umma_smem_desc(b_addr + kk * 32, 16, 1024);
            umma_bf16(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0);
          }
          umma_commit(&empty_bar[s]);  // stage reusable once these MMAs retire
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&tfull_bar[acc]);
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // -------------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      int b, m_blk, n_blk;
      tile_coords(tile, b, m_blk, n_blk);
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, ab)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = m_blk * kBM + q * 32 + lane;
      const int n0 = n_blk * BN;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const bool row_ok = row < p.M;
      const bool f16 = p.fp16 != 0;
      long long c_off = static_cast<long long>(b) * p.c_batch_stride + static_cast<long long>(row) * p.ldc;
      __nv_bfloat16* c_bf16 = static_cast<__nv_bfloat16*>(p.C);
      if (MODE == 1 && row_ok_pre(row, p.M)) {
        const int owner = row / p.rows_per_rank;
        c_bf16 = static_cast<__nv_bfloat16*>(p.rs_peer[owner]);
        c_off = (static_cast<long long>(p.rs_slot) * p.rows_per_rank + (row - owner * p.rows_per_rank)) * p.ldc;
      }
      if (p.tma_epilogue) {
        // ---- staged epilogue: registers -> swizzled shared memory -> TMA store / reduce
        uint8_t* stage_base = smem + Cfg::kStagingOffset + q * 4096;
        const int row0 = m_blk * kBM + q * 32;
        const CUtensorMap* cmap = &tmC.m[0];
        int store_row = row0;
        if (MODE == 1) {
          const int owner = (m_blk * kBM) / p.rows_per_rank;
          cmap = &tmC.m[owner];
          store_row = p.rs_slot * p.rows_per_rank + (row0 - owner * p.rows_per_rank);
        }
        const int sw = lane & 7;
        int nbuf = 0;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          if (n0 + c >= p.N) break;  // warp-uniform
          uint32_t r[32];
          tmem_ld_32x32(t_row + c, r);
          tmem_ld_wait();
          const int col0 = n0 + c;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) v[j] += load_16(p.bias, col0 + j, f16);
          }
          if (p.out_fp32) {
            // one chunk = 32 fp32 = a full 128-byte row
            uint8_t* buf = stage_base;
            if (nbuf >= 1) tma_store_wait_read_n<0>();   // the previous store has read the buffer
            __syncwarp();
            uint8_t* rowp = buf + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<float4*>(rowp + ((j ^ sw) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2],
                                                                               v[4 * j + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (p.accumulate) tma_reduce_add_3d(cmap, buf, col0, store_row, b);
              else tma_store_3d(cmap, buf, col0, store_row, b);
              tma_store_commit();
            }
            ++nbuf;
          } else {
            // two chunks (64 bf16) make one 128-byte row
            const int half = (c >> 5) & 1;
            uint8_t* buf = stage_base;
            if (half == 0) {
              if (nbuf >= 1) tma_store_wait_read_n<0>();
              __syncwarp();
            }
            uint8_t* rowp = buf + lane * 128;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_16x2(v[8 * j], v[8 * j + 1], f16);
              o.y = pack_16x2(v[8 * j + 2], v[8 * j + 3], f16);
              o.z = pack_16x2(v[8 * j + 4], v[8 * j + 5], f16);
              o.w = pack_16x2(v[8 * j + 6], v[8 * j + 7], f16);
              *reinterpret_cast<uint4*>(rowp + (((half * 4 + j) ^ sw) << 4)) = o;
            }
            const bool last = (c + 32 >= BN) || (n0 + c + 32 >= p.N);
            if (half == 1 || last) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(cmap, buf, col0 - half * 32, store_row, b);
                tma_store_commit();
              }
              ++nbuf;
            }
          }
        }
        if (lane == 0) tma_store_wait_read_n<0>();   // staging may be rewritten by the next tile
        __syncwarp();
        tc_fence_before_sync();
        mbar_arrive(&tempty_bar[acc]);
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        if (n0 + c >= p.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(t_row + c, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        const int col0 = n0 + c;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) v[j] += load_16(p.bias, col0 + j, f16);
        }
        const bool full = (col0 + 32 <= p.N);
        if (p.out_fp32) {
          float* dst = static_cast<float*>(p.C) + c_off + col0;
          if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              if (p.accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(dst + j);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(dst + j) = o;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dst[j] = p.accumulate ? dst[j] + v[j] : v[j];
          }
        } else {
          __nv_bfloat16* dst = c_bf16 + c_off + col0;
          if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (p.accumulate) {
                const uint4 old = *reinterpret_cast<const uint4*>(dst + j);
                const uint32_t* ob = reinterpret_cast<const uint32_t*>(&old);
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                  const float2 f = unpack_16x2(ob[t], f16);
                  v[j + 2 * t] += f.x;
                  v[j + 2 * t + 1] += f.y;
                }
              }
              uint4 o;
              o.x = pack_16x2(v[j], v[j + 1], f16);
              o.y = pack_16x2(v[j + 2], v[j + 3], f16);
              o.z = pack_16x2(v[j + 4], v[j + 5], f16);
              o.w = pack_16x2(v[j + 6], v[j + 7], f16);
              *reinterpret_cast<uint4*>(dst + j) = o;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) store_16(dst, j, p.accumulate ? load_16(dst, j, f16) + v[j] : v[j], f16);
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&tempty_bar[acc]);
    }
    if (p.tma_epilogue && lane == 0) {
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every staged store has been written out
      if (MODE == 1) __threadfence_system();
    }
  }

  if (MODE == 2 && warp == 6 && p.ag_in_kernel) {
    // ------------------------------------------------------------------ AllGather copy warp
    // One lane moves this CTA's share of every chunk peer -> shared bounce buffer -> local gathered operand
    // with bulk copies (two buffers in flight), own chunk first, then ranks rank+1, rank+2, ...
    if (lane == 0) {
      uint8_t* bounce = smem + Cfg::kBounceOffset;
      uint64_t* bfull = tempty_bar + 2 + 2;   // two barriers after tmem_slot/abort words (see layout below)
      mbar_init(&bfull[0], 1);
      mbar_init(&bfull[1], 1);
      fence_mbar_init();
      const long long chunk_bytes = static_cast<long long>(p.rows_per_rank) * p.K * 2;
      long long per = (chunk_bytes / gridDim.x + 15) & ~15LL;
      if (per * gridDim.x < chunk_bytes) per += 16;
      const long long lo = per * blockIdx.x;
      const long long hi = lo + per < chunk_bytes ? lo + per : chunk_bytes;
      const int pieces = hi > lo ? static_cast<int>((hi - lo + kBounceBytes - 1) / kBounceBytes) : 0;
      uint32_t gload = 0, gdrain = 0;   // running piece counters: buffer = counter & 1, phase = (counter >> 1) & 1
      bool okc = true;
      for (int sidx = 0; sidx < p.world && okc; ++sidx) {
        const int c = (p.rank + sidx) % p.world;
        const uint8_t* src = static_cast<const uint8_t*>(p.ag_src[c]);
        uint8_t* dst = static_cast<uint8_t*>(p.ag_dst) + static_cast<long long>(c) * chunk_bytes;
        int nload = 0, ndrain = 0;
        while (ndrain < pieces) {
          while (nload < pieces && nload - ndrain < 2) {
            const long long off = lo + static_cast<long long>(nload) * kBounceBytes;
            const int bytes = static_cast<int>(hi - off < kBounceBytes ? hi - off : kBounceBytes);
            const int bsel = gload & 1;
            mbar_expect_tx(&bfull[bsel], bytes);
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                    smem_u32(bounce + bsel * kBounceBytes)),
                "l"(src + off), "r"(bytes), "r"(smem_u32(&bfull[bsel]))
                : "memory");
            ++nload;
            ++gload;
          }
          const long long off = lo + static_cast<long long>(ndrain) * kBounceBytes;
          const int bytes = static_cast<int>(hi - off < kBounceBytes ? hi - off : kBounceBytes);
          const int d = gdrain & 1;
          if (!mbar_wait(&bfull[d], (gdrain >> 1) & 1, ab)) { okc = false; break; }
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + off),
                       "r"(smem_u32(bounce + d * kBounceBytes)), "r"(bytes)
                       : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // buffer d may be refilled
          ++ndrain;
          ++gdrain;
        }
        if (!okc) break;
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");          // stores of this chunk have landed
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
        atomicAdd(p.ag_flags + c, 1);
      }
    }
    __syncwarp();
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*cta_abort && threadIdx.x == 0) {
    // Loads that were issued but never observed complete may still be in flight:
    // give them a bounded time to land before shared memory is released.
    const int issued = *issued_cnt, consumed = *consumed_cnt;
    for (int i = consumed; i < issued; ++i) {
      const int s = i % kStages;
      const uint32_t ph = (i / kStages) & 1;
      const unsigned long long t0 = globaltimer_ns();
      while (!mbar_try_wait(&full_bar[s], ph)) {
        if (globaltimer_ns() - t0 > 200000000ull) break;
      }
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <int BN, bool A_MN, bool B_MN, int MODE>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CMaps& tmC, const GemmParams& p,
                       cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, MODE>;
  constexpr int smem = MODE == 2 ? Cfg::kSmemBytesAG : Cfg::kSmemBytes;
  static bool configured = false;  // per template instance
  if (!configured) {
    MSB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  const int tiles = ((p.M + kBM - 1) / kBM) * ((p.N + BN - 1) / BN) * p.batch;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, MODE == 2 ? kGemmThreads + 32 : kGemmThreads, smem, stream>>>(tmA, tmB, tmC, p);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

static int pick_bn(int M, int N, int batch, int bn_hint) {
  if (bn_hint == 128 || bn_hint == 256) return bn_hint;
  if (N <= 128) return 128;
  // persistent CTAs work through the tiles in rounds of one tile per SM: take the width with the smaller
  // (rounds x time per tile).  Measured per round at 4096 x 4096: a 128-wide tile takes 0.82 (K = 4096) to 0.87
  // (K = 11008) of a 256-wide one - it still loads the full 128 rows of A and drains as many accumulator rows
  const long long sms = sm_count();
  const long long t256 = static_cast<long long>((M + 127) / 128) * ((N + 255) / 256) * batch;
  const long long t128 = static_cast<long long>((M + 127) / 128) * ((N + 127) / 128) * batch;
  const double c256 = static_cast<double>((t256 + sms - 1) / sms);
  const double c128 = static_cast<double>((t128 + sms - 1) / sms) * 0.85;
  return c128 < c256 ? 128 : 256;
}

static int encode_operands(CUtensorMap* tmA, CUtensorMap* tmB, const void* A, const void* B, int M, int N, int K,
                           int batch, int a_mn, int b_mn, long long lda, long long ldb, long long a_batch_stride,
                           long long b_batch_stride, int bn) {
  if ((lda % 8) || (ldb % 8) || (a_batch_stride % 8) || (b_batch_stride % 8)) {
    set_last_error("gemm: pitches and batch strides must be multiples of 8 elements (lda=%lld ldb=%lld)", lda, ldb);
    return kBadArg;
  }
  const uint64_t abs_ = batch > 1 ? static_cast<uint64_t>(a_batch_stride) * 2
                                  : static_cast<uint64_t>(lda) * 2 * (a_mn ? K : M);
  const uint64_t bbs_ = batch > 1 ? static_cast<uint64_t>(b_batch_stride) * 2
                                  : static_cast<uint64_t>(ldb) * 2 * (b_mn ? K : N);
  int rc;
  if (a_mn) rc = encode_tmap_3d(tmA, A, 2, M, K, batch, lda * 2, abs_, 64, 64, 1);
  else      rc = encode_tmap_3d(tmA, A, 2, K, M, batch, lda * 2, abs_, 64, kBM, 1);
  if (rc != kOk) return rc;
  if (b_mn) rc = encode_tmap_3d(tmB, B, 2, N, K, batch, ldb * 2, bbs_, 64, 64, 1);
  else      rc = encode_tmap_3d(tmB, B, 2, K, N, batch, ldb * 2, bbs_, 64, bn, 1);
  return rc;
}

// Tensor map of an output matrix for the staged epilogue (128-byte rows of 32 output rows); returns 0 and leaves
// *ok = 0 when the matrix does not meet the TMA alignment rules (the kernel then stores per thread).
static int encode_output(CUtensorMap* map, const void* C, int M, int N, int batch, long long ldc,
                         long long c_batch_stride, int out_fp32, int* ok) {
  const int es = out_fp32 ? 4 : 2;
  *ok = 0;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || ((ldc * es) & 15) || (batch > 1 && ((c_batch_stride * es) & 15)))
    return kOk;
  const uint64_t bs = batch > 1 ? static_cast<uint64_t>(c_batch_stride) * es : static_cast<uint64_t>(ldc) * es * M;
  if (int rc = encode_tmap_3d(map, C, es, N, M, batch, static_cast<uint64_t>(ldc) * es, bs, 128 / es, 32, 1)) return rc;
  *ok = 1;
  return kOk;
}

}  // namespace msb

// C[b] (+)= alpha * A[b] x B[b]^T (+ bias).  A is [M,K] (a_mn=0, row pitch lda) or stored [K,M]
// (a_mn=1, row pitch lda); B is [N,K] (b_mn=0) or stored [K,N] (b_mn=1).  Pitches and batch
// strides are in elements and must be multiples of 8; base pointers 16-byte aligned.
// bn_hint: 0 = choose, else 128 or 256.
static int gemm_16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int batch,
                   int a_mn, int b_mn, long long lda, long long ldb, long long ldc, long long a_batch_stride,
                   long long b_batch_stride, long long c_batch_stride, int out_fp32, int accumulate, float alpha,
                   int bn_hint, int fp16, void* stream_) {
  using namespace msb;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) {
    set_last_error("gemm: empty problem M=%d N=%d K=%d batch=%d", M, N, K, batch);
    return kBadArg;
  }
  int* status = status_ptr();
  if (!status) {
    set_last_error("gemm: cannot resolve the device status word");
    return kCudaError;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int bn = pick_bn(M, N, batch, bn_hint);
  CUtensorMap tmA, tmB;
  if (int rc = encode_operands(&tmA, &tmB, A, B, M, N, K, batch, a_mn, b_mn, lda, ldb, a_batch_stride,
                               b_batch_stride, bn))
    return rc;
  GemmParams p = {};
  p.C = C; p.bias = bias; p.status = status; p.c_batch_stride = c_batch_stride;
  p.M = M; p.N = N; p.K = K; p.batch = batch; p.ldc = static_cast<int>(ldc);
  p.out_fp32 = out_fp32; p.accumulate = accumulate; p.alpha = alpha; p.fp16 = fp16;
  CMaps tmC = {};
  if (!(accumulate && !out_fp32)) {
    if (int rc = encode_output(&tmC.m[0], C, M, N, batch, ldc, c_batch_stride, out_fp32, &p.tma_epilogue)) return rc;
  }

#define MSB_DISPATCH(BN_)                                                          \
  if (a_mn) {                                                                      \
    if (b_mn) return launch_gemm<BN_, true, true, 0>(tmA, tmB, tmC, p, stream);    \
    return launch_gemm<BN_, true, false, 0>(tmA, tmB, tmC, p, stream);             \
  } else {                                                                         \
    if (b_mn) return launch_gemm<BN_, false, true, 0>(tmA, tmB, tmC, p, stream);   \
    return launch_gemm<BN_, false, false, 0>(tmA, tmB, tmC, p, stream);            \
  }
  if (bn == 256) { MSB_DISPATCH(256) } else { MSB_DISPATCH(128) }
#undef MSB_DISPATCH
}

MSB_EXPORT int msb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int batch,
                             int a_mn, int b_mn, long long lda, long long ldb, long long ldc,
                             long long a_batch_stride, long long b_batch_stride, long long c_batch_stride,
                             int out_fp32, int accumulate, float alpha, int bn_hint, void* stream_) {
  return gemm_16(A, B, C, bias, M, N, K, batch, a_mn, b_mn, lda, ldb, ldc, a_batch_stride, b_batch_stride,
                 c_batch_stride, out_fp32, accumulate, alpha, bn_hint, 0, stream_);
}

// The same GEMM on fp16 operands (fp16 bias; C fp16 or fp32): the tensor-core instruction takes the operand format
// from its descriptor, so this is the bf16 kernel with another descriptor and another 16-bit pack in the epilogue.
MSB_EXPORT int msb_gemm_fp16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int batch,
                             int a_mn, int b_mn, long long lda, long long ldb, long long ldc,
                             long long a_batch_stride, long long b_batch_stride, long long c_batch_stride,
                             int out_fp32, int accumulate, float alpha, int bn_hint, void* stream_) {
  return gemm_16(A, B, C, bias, M, N, K, batch, a_mn, b_mn, lda, ldb, ldc, a_batch_stride, b_batch_stride,
                 c_batch_stride, out_fp32, accumulate, alpha, bn_hint, 1, stream_);
}

namespace msb {

static __device__ int g_ag_ones[8] = {1, 1, 1, 1, 1, 1, 1, 1};

// Per-device side streams / events for the copy-engine all-gather of msb_gemm_ag.  Created on the first call of a
// device (outside any stream capture: the callers run eagerly before they capture).
struct AgDma {
  cudaStream_t side[2];
  cudaEvent_t fork, join[2];
  int* ones;
  bool ready;
};

static int ag_dma_state(AgDma** out) {
  static AgDma state[64] = {};
  int dev = 0;
  MSB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) { set_last_error("gemm_ag: device ordinal %d out of range", dev); return kBadArg; }
  AgDma* st = &state[dev];
  if (!st->ready) {
    for (int i = 0; i < 2; ++i) {
      MSB_CUDA_CHECK(cudaStreamCreateWithFlags(&st->side[i], cudaStreamNonBlocking));
      MSB_CUDA_CHECK(cudaEventCreateWithFlags(&st->join[i], cudaEventDisableTiming));
    }
    MSB_CUDA_CHECK(cudaEventCreateWithFlags(&st->fork, cudaEventDisableTiming));
    void* p = nullptr;
    MSB_CUDA_CHECK(cudaGetSymbolAddress(&p, g_ag_ones));
    st->ones = static_cast<int*>(p);
    st->ready = true;
  }
  *out = st;
  return kOk;
}

}  // namespace msb

static int check_chunks(const char* what, int M, int world, int rank) {
  using namespace msb;
  if (world < 2 || world > 8 || rank < 0 || rank >= world || M % world || (M / world) % kBM) {
    set_last_error("%s: M=%d must split into %d chunks that are multiples of %d rows (rank %d)", what, M, world,
                   kBM, rank);
    return kBadArg;
  }
  return kOk;
}

// MatMul -> ReduceScatter.  partial[M,N] = A[M,K] x B^T is never materialised locally: tile rows owned by rank o
// are stored into stage_ptrs[o] + (rank*rows_per_rank + local_row)*N  (bf16 staging of shape [world][M/world][N]
// on every rank).  After a group barrier each rank sums its `world` slots (msb_reduce_slots).
static int gemm_push(const char* what, const void* A, const void* B, const void* bias,
                     const unsigned long long* stage_ptrs, int M, int N, int K, int b_mn, long long lda,
                     long long ldb, int world, int rank, int slot, int slots, int bn_hint, void* stream_) {
  using namespace msb;
  if (int rc = check_chunks(what, M, world, rank)) return rc;
  if (N % 8) { set_last_error("%s: N=%d must be a multiple of 8", what, N); return kBadArg; }
  if (slot < 0 || slot >= slots) { set_last_error("%s: slot %d outside [0, %d)", what, slot, slots); return kBadArg; }
  int* status = status_ptr();
  if (!status) { set_last_error("%s: no status word", what); return kCudaError; }
  const int bn = pick_bn(M, N, 1, bn_hint);
  CUtensorMap tmA, tmB;
  if (int rc = encode_operands(&tmA, &tmB, A, B, M, N, K, 1, 0, b_mn, lda, ldb, 0, 0, bn)) return rc;
  GemmParams p = {};
  p.status = status; p.M = M; p.N = N; p.K = K; p.batch = 1; p.ldc = N; p.alpha = 1.f; p.bias = bias;
  p.world = world; p.rank = rank; p.rows_per_rank = M / world; p.rs_slot = slot;
  for (int i = 0; i < world; ++i) p.rs_peer[i] = reinterpret_cast<void*>(stage_ptrs[i]);
  p.C = p.rs_peer[rank];
  CMaps tmC = {};
  int all_ok = 1;
  for (int i = 0; i < world; ++i) {
    int ok = 0;
    if (int rc = encode_output(&tmC.m[i], p.rs_peer[i], slots * p.rows_per_rank, N, 1, N, 0, 0, &ok)) return rc;
    all_ok &= ok;
  }
  p.tma_epilogue = all_ok;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (bn == 256) {
    if (b_mn) return launch_gemm<256, false, true, 1>(tmA, tmB, tmC, p, stream);
    return launch_gemm<256, false, false, 1>(tmA, tmB, tmC, p, stream);
  }
  if (b_mn) return launch_gemm<128, false, true, 1>(tmA, tmB, tmC, p, stream);
  return launch_gemm<128, false, false, 1>(tmA, tmB, tmC, p, stream);
}

MSB_EXPORT int msb_gemm_rs(const void* A, const void* B, const unsigned long long* stage_ptrs, int M, int N, int K,
                           int b_mn, long long lda, long long ldb, int world, int rank, int bn_hint, void* stream_) {
  return gemm_push("gemm_rs", A, B, nullptr, stage_ptrs, M, N, K, b_mn, lda, ldb, world, rank, rank, world, bn_hint,
                   stream_);
}

// MatMul -> row exchange (an expert's GEMM whose rows go back to the ranks their tokens came from).  Rows
// [o*M/world, (o+1)*M/world) of  A x op(B) + bias  are stored into slot `slot` of rank o's buffer dst_ptrs[o], bf16
// [slots][M/world][N]; nothing is summed, the receiver reads the slots after a group barrier.
MSB_EXPORT int msb_gemm_push_rows(const void* A, const void* B, const void* bias, const unsigned long long* dst_ptrs,
                                  int M, int N, int K, int b_mn, long long lda, long long ldb, int world, int rank,
                                  int slot, int slots, int bn_hint, void* stream_) {
  return gemm_push("gemm_push_rows", A, B, bias, dst_ptrs, M, N, K, b_mn, lda, ldb, world, rank, slot, slots, bn_hint,
                   stream_);
}

// AllGather -> MatMul.  C[M,N] = gather(A)[M,K] x B^T (+ bias) where chunk c of the gathered operand is pulled from
// src_ptrs[c] (rank c's [M/world][K] shard in symmetric memory) into `gathered` ([M][K], local) while tiles of
// chunks that have already arrived are being multiplied.  flags: int[world], zeroed here.
//   use_dma = 0: a copy warp of every CTA pulls the chunks with bulk copies through shared memory;
//   use_dma = 1: the copy engines pull them - peer -> local cudaMemcpyAsync on two side streams in ring order
//                (rank+1, rank+2, ...), each followed by a 4-byte copy that raises the chunk's flag; the SMs only
//                multiply.  The side streams fork from and join `stream`, so the call also captures into a graph.
MSB_EXPORT int msb_gemm_ag(const unsigned long long* src_ptrs, void* gathered, int* flags, const void* B, void* C,
                           const void* bias, int M, int N, int K, int b_mn, long long ldb, long long ldc, int world,
                           int rank, int bn_hint, int use_dma, void* stream_) {
  using namespace msb;
  if (int rc = check_chunks("gemm_ag", M, world, rank)) return rc;
  if (K % 8) { set_last_error("gemm_ag: K=%d must be a multiple of 8", K); return kBadArg; }
  int* status = status_ptr();
  if (!status) { set_last_error("gemm_ag: no status word"); return kCudaError; }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MSB_CUDA_CHECK(cudaMemsetAsync(flags, 0, sizeof(int) * world, stream));
  const int bn = pick_bn(M, N, 1, bn_hint);
  CUtensorMap tmA, tmB;
  if (int rc = encode_operands(&tmA, &tmB, gathered, B, M, N, K, 1, 0, b_mn, K, ldb, 0, 0, bn)) return rc;
  GemmParams p = {};
  p.C = C; p.bias = bias; p.status = status; p.M = M; p.N = N; p.K = K; p.batch = 1;
  p.ldc = static_cast<int>(ldc); p.alpha = 1.f;
  p.world = world; p.rank = rank; p.rows_per_rank = M / world;
  for (int i = 0; i < world; ++i) p.ag_src[i] = reinterpret_cast<const void*>(src_ptrs[i]);
  p.ag_dst = gathered; p.ag_flags = flags;
  p.ag_in_kernel = use_dma ? 0 : 1;
  CMaps tmC = {};
  if (int rc = encode_output(&tmC.m[0], C, M, N, 1, ldc, 0, 0, &p.tma_epilogue)) return rc;
  const int tiles = ((M + kBM - 1) / kBM) * ((N + bn - 1) / bn);
  p.ag_flag_target = use_dma ? 1 : (tiles < sm_count() ? tiles : sm_count());
  AgDma* dma = nullptr;
  if (use_dma) {
    if (int rc = ag_dma_state(&dma)) return rc;
    const size_t chunk_bytes = static_cast<size_t>(p.rows_per_rank) * K * 2;
    char* dst = static_cast<char*>(gathered);
    MSB_CUDA_CHECK(cudaEventRecord(dma->fork, stream));
    for (int i = 0; i < 2; ++i) MSB_CUDA_CHECK(cudaStreamWaitEvent(dma->side[i], dma->fork, 0));
    for (int sidx = 1; sidx < world; ++sidx) {
      const int c = (rank + sidx) % world;
      cudaStream_t q = dma->side[(sidx - 1) & 1];
      MSB_CUDA_CHECK(cudaMemcpyAsync(dst + c * chunk_bytes, reinterpret_cast<const void*>(src_ptrs[c]), chunk_bytes,
                                     cudaMemcpyDeviceToDevice, q));
      MSB_CUDA_CHECK(cudaMemcpyAsync(flags + c, dma->ones, sizeof(int), cudaMemcpyDeviceToDevice, q));
    }
    // own shard: on the launching stream, so it is in place before the kernel starts
    MSB_CUDA_CHECK(cudaMemcpyAsync(dst + rank * chunk_bytes, reinterpret_cast<const void*>(src_ptrs[rank]),
                                   chunk_bytes, cudaMemcpyDeviceToDevice, stream));
    MSB_CUDA_CHECK(cudaMemcpyAsync(flags + rank, dma->ones, sizeof(int), cudaMemcpyDeviceToDevice, stream));
  }
  int rc;
  if (bn == 256) {
    rc = b_mn ? launch_gemm<256, false, true, 2>(tmA, tmB, tmC, p, stream)
              : launch_gemm<256, false, false, 2>(tmA, tmB, tmC, p, stream);
  } else {
    rc = b_mn ? launch_gemm<128, false, true, 2>(tmA, tmB, tmC, p, stream)
              : launch_gemm<128, false, false, 2>(tmA, tmB, tmC, p, stream);
  }
  if (use_dma) {
    // join even when the launch failed: a forked side stream must come back before a capture can end
    for (int i = 0; i < 2; ++i) {
      MSB_CUDA_CHECK(cudaEventRecord(dma->join[i], dma->side[i]));
      MSB_CUDA_CHECK(cudaStreamWaitEvent(stream, dma->join[i], 0));
    }
  }
  return rc;
}
