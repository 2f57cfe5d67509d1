// FlashAttention backward for sm_100a (head_dim 128, bf16, equal q/kv head counts), tcgen05 + TMEM + TMA.
//
// Three launches, all deterministic (no atomics):
//   1. delta[b][h][s] = sum_d O * dO
//   2. dK/dV kernel: one work item = (batch, head, 128 keys); loops over 64-row query blocks.  With keys as the
//      M dimension, thread t of the compute warps owns key row t:
//         S^T  = K Q^T          (TMEM, 64 columns, double-buffered)
//         P^T  = exp2(S^T * c - lse)            -> shared memory (A operand, K-major over queries)
//         dV  += P^T dO         (TMEM accumulator, 128 columns)
//         dP^T = V dO^T         (TMEM, 64 columns, double-buffered)
//         dS^T = P^T o (dP^T - delta) * scale   -> shared memory
//         dK  += dS^T Q         (TMEM accumulator, 128 columns)
//      The Q and dO tiles are read both K-major (as B of S^T / dP^T) and MN-major (as B of dK / dV) from the
//      same shared-memory bytes.
//   3. dQ kernel: one work item = (batch, head, 128 queries); loops over 128-key blocks, thread t owns query row t:
//         S = Q K^T, dP = dO V^T, dS = P o (dP - delta) * scale -> shared memory, dQ += dS K.
// Warp roles as in the forward kernel: warp 0 TMA, warp 1 MMA issue, warps 2-5 compute/epilogue.
//
// This text is compiled twice: for bf16 tensors (flash_attn_bwd_sm100.cu), and with MSB_ELEM_FP16 defined for fp16 tensors
// (flash_attn_bwd_sm100_fp16.cu), where every entry point carries the suffix _fp16 and "bf16" in a comment reads "fp16".
#include "fa_common.cuh"

namespace msb {
namespace MSB_ELEM_NS {

constexpr int kBwdThreads = 192;

struct FaBwdParams {
  const float* lse;     // [B][H][S] natural log
  const float* delta;   // [B][H][S]
  elem_t* dq;
  elem_t* dk;
  elem_t* dv;
  int* status;
  long long dq_pitch, dkv_pitch;
  int B, H, S;
  int causal;
  float scale, scale_log2;
};

// ------------------------------------------------------------------------------------------------ delta
__global__ void fa_delta_kernel(const elem_t* __restrict__ o, const elem_t* __restrict__ dout,
                                float* __restrict__ delta, int B, int S, int H, long long o_pitch,
                                long long do_pitch) {
  const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * H;
  if (wid >= total) return;
  const int h = wid % H;
  const long long tok = wid / H;
  const uint2 a = *reinterpret_cast<const uint2*>(o + tok * o_pitch + (long long)h * kFaD + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + tok * do_pitch + (long long)h * kFaD + lane * 4);
  const float2 a0 = e2_to_f2(*reinterpret_cast<const elem2_t*>(&a.x));
  const float2 a1 = e2_to_f2(*reinterpret_cast<const elem2_t*>(&a.y));
  const float2 b0 = e2_to_f2(*reinterpret_cast<const elem2_t*>(&b.x));
  const float2 b1 = e2_to_f2(*reinterpret_cast<const elem2_t*>(&b.y));
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  s = warp_sum(s);
  if (lane == 0) {
    const long long bb = tok / S, ss = tok % S;
    delta[(bb * H + h) * S + ss] = s;
  }
}

// ------------------------------------------------------------------------------------------------ dK / dV
struct KvSmem {
  static constexpr int kK = 0;                 // 32 KB
  static constexpr int kV = 32768;             // 32 KB
  static constexpr int kQ = 65536;             // 2 x 16 KB
  static constexpr int kDO = 98304;            // 2 x 16 KB
  static constexpr int kPT = 131072;           // 16 KB
  static constexpr int kDST = 147456;          // 16 KB
  static constexpr int kBar = 163840;
  static constexpr int kBytes = kBar + 512 + 1024;
};

__global__ void __launch_bounds__(kBwdThreads, 1)
fa_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const FaBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + KvSmem::kBar);
  uint64_t* kv_full = bars + 0;
  uint64_t* kv_empty = bars + 1;
  uint64_t* q_full = bars + 2;     // [2]
  uint64_t* q_empty = bars + 4;    // [2]
  uint64_t* do_full = bars + 6;    // [2]
  uint64_t* do_empty = bars + 8;   // [2]
  uint64_t* s_full = bars + 10;    // [2]
  uint64_t* s_empty = bars + 12;   // [2]
  uint64_t* dp_full = bars + 14;   // [2]
  uint64_t* dp_empty = bars + 16;  // [2]
  uint64_t* p_ready = bars + 18;
  uint64_t* p_empty = bars + 19;
  uint64_t* ds_ready = bars + 20;
  uint64_t* ds_empty = bars + 21;
  uint64_t* acc_done = bars + 22;
  uint64_t* acc_empty = bars + 23;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const AbortCtx ab{cta_abort, p.status};
  const int nkv = p.S / 128;
  const int nq64 = p.S / 64;
  const int total = p.B * p.H * nkv;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(kv_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&do_full[i], 1);
      mbar_init(&do_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
      mbar_init(&dp_full[i], 1);
      mbar_init(&dp_empty[i], 128);
    }
    mbar_init(p_ready, 128);
    mbar_init(p_empty, 1);
    mbar_init(ds_ready, 128);
    mbar_init(ds_empty, 1);
    mbar_init(acc_done, 1);
    mbar_init(acc_empty, 128);
    *cta_abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dv = tmem_base + 256, tm_dk = tmem_base + 384;

  // item w -> (b, h, key block jb); light-to-heavy would starve the tail, so heavy (small jb) first
  auto item = [&](int w, int& b, int& h, int& jb) {
    const int bh = p.B * p.H;
    jb = w / bh;
    const int r = w % bh;
    b = r / p.H;
    h = r % p.H;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t items = 0, qc = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++items) {
        int b, h, jb;
        item(w, b, h, jb);
        const int i0 = p.causal ? 2 * jb : 0;
        if (!mbar_wait(kv_empty, (items & 1) ^ 1, ab)) { ok = false; break; }
        mbar_expect_tx(kv_full, 65536);
        fa_load_tile(smem + KvSmem::kK, &tmK, kv_full, 128, h, jb * 128, b);
        fa_load_tile(smem + KvSmem::kV, &tmV, kv_full, 128, h, jb * 128, b);
        for (int i = i0; i < nq64; ++i, ++qc) {
          const int st = qc & 1;
          const uint32_t ph = (qc >> 1) & 1;
          if (!mbar_wait(&q_empty[st], ph ^ 1, ab)) { ok = false; break; }
          mbar_expect_tx(&q_full[st], 16384);
          fa_load_tile(smem + KvSmem::kQ + st * 16384, &tmQ, &q_full[st], 64, h, i * 64, b);
          if (!mbar_wait(&do_empty[st], ph ^ 1, ab)) { ok = false; break; }
          mbar_expect_tx(&do_full[st], 16384);
          fa_load_tile(smem + KvSmem::kDO + st * 16384, &tmDO, &do_full[st], 64, h, i * 64, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = umma_idesc_elem(128, 64, false, false);    // [keys x queries], K = d
      constexpr uint32_t idesc_acc = umma_idesc_elem(128, 128, false, true);   // [keys x d], K = queries, B MN-major
      const uint32_t k_addr = smem_u32(smem + KvSmem::kK), v_addr = smem_u32(smem + KvSmem::kV);
      const uint32_t pt_addr = smem_u32(smem + KvSmem::kPT), dst_addr = smem_u32(smem + KvSmem::kDST);
      uint32_t items = 0, qc = 0;
      bool ok = true;
      auto issue_front = [&](uint32_t c) -> bool {
        const int st = c & 1;
        const uint32_t ph = (c >> 1) & 1;
        const uint32_t q_addr = smem_u32(smem + KvSmem::kQ + st * 16384);
        const uint32_t do_addr = smem_u32(smem + KvSmem::kDO + st * 16384);
        if (!mbar_wait(&q_full[st], ph, ab)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, ab)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tm_s + st * 64, umma_smem_desc(k_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                    umma_smem_desc(q_addr + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), idesc_st, kk != 0);
        umma_commit(&s_full[st]);
        if (!mbar_wait(&do_full[st], ph, ab)) return false;
        if (!mbar_wait(&dp_empty[st], ph ^ 1, ab)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tm_dp + st * 64, umma_smem_desc(v_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                    umma_smem_desc(do_addr + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), idesc_st, kk != 0);
        umma_commit(&dp_full[st]);
        return true;
      };
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++items) {
        int b, h, jb;
        item(w, b, h, jb);
        const int nblk = nq64 - (p.causal ? 2 * jb : 0);
        if (!mbar_wait(kv_full, items & 1, ab)) { ok = false; break; }
        if (!issue_front(qc)) { ok = false; break; }
        for (int i = 0; i < nblk; ++i) {
          const uint32_t c = qc + i;
          const int st = c & 1;
          if (i + 1 < nblk && !issue_front(c + 1)) { ok = false; break; }
          if (i == 0 && !mbar_wait(acc_empty, (items & 1) ^ 1, ab)) { ok = false; break; }
          const uint32_t q_addr = smem_u32(smem + KvSmem::kQ + st * 16384);
          const uint32_t do_addr = smem_u32(smem + KvSmem::kDO + st * 16384);
          if (!mbar_wait(p_ready, c & 1, ab)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tm_dv, umma_smem_desc(pt_addr + kk * 32, 16, 1024),
                      umma_smem_desc(do_addr + kk * 2048, 8192, 1024), idesc_acc, (i | kk) != 0);
          umma_commit(p_empty);
          umma_commit(&do_empty[st]);
          if (!mbar_wait(ds_ready, c & 1, ab)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(tm_dk, umma_smem_desc(dst_addr + kk * 32, 16, 1024),
                      umma_smem_desc(q_addr + kk * 2048, 8192, 1024), idesc_acc, (i | kk) != 0);
          umma_commit(ds_empty);
          umma_commit(&q_empty[st]);
        }
        if (!ok) break;
        umma_commit(acc_done);
        umma_commit(kv_empty);
        qc += nblk;
      }
    }
    __syncwarp();
  } else {
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;   // key row inside the 128-key block == TMEM lane
    const uint32_t lane_sel = static_cast<uint32_t>(q4 * 32) << 16;
    uint8_t* pt = smem + KvSmem::kPT;
    uint8_t* dst = smem + KvSmem::kDST;
    uint32_t items = 0, qc = 0;
    bool ok = true;
    const float log2e = 1.4426950408889634f;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++items) {
      int b, h, jb;
      item(w, b, h, jb);
      const int i0 = p.causal ? 2 * jb : 0;
      const float* lse_row = p.lse + (static_cast<long long>(b) * p.H + h) * p.S;
      const float* delta_row = p.delta + (static_cast<long long>(b) * p.H + h) * p.S;
      const int key = jb * 128 + row;
      for (int i = i0; i < nq64; ++i, ++qc) {
        const int st = qc & 1;
        const uint32_t ph = (qc >> 1) & 1;
        float pv[64];
        if (!mbar_wait(&s_full[st], ph, ab)) { ok = false; break; }
        tc_fence_after_sync();
        {
          // both loads are issued before the one wait: a single TMEM round trip per tile
          uint32_t r[2][32];
          tmem_ld_32x32(tm_s + st * 64 + lane_sel, r[0]);
          tmem_ld_32x32(tm_s + st * 64 + lane_sel + 32, r[1]);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int t = 0; t < 32; ++t) pv[c * 32 + t] = __uint_as_float(r[c][t]);
        }
        tc_fence_before_sync();
        mbar_arrive(&s_empty[st]);
        const int q0 = i * 64;
        const bool diag = p.causal && (q0 < jb * 128 + 128);
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse_row + q0 + c4 * 4);
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const int c = c4 * 4 + t;
            float v = ex2(pv[c] * p.scale_log2 - lv[t] * log2e);
            if (diag && (q0 + c < key)) v = 0.f;
            pv[c] = v;
          }
        }
        if (!mbar_wait(p_empty, (qc & 1) ^ 1, ab)) { ok = false; break; }
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) fa_store_chunk(pt, row, ch, 0, &pv[ch * 8]);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(p_ready);
        // ---- dS^T
        if (!mbar_wait(&dp_full[st], ph, ab)) { ok = false; break; }
        tc_fence_after_sync();
        {
          uint32_t r[2][32];
          tmem_ld_32x32(tm_dp + st * 64 + lane_sel, r[0]);
          tmem_ld_32x32(tm_dp + st * 64 + lane_sel + 32, r[1]);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int t4 = 0; t4 < 8; ++t4) {
              const float4 d4 = *reinterpret_cast<const float4*>(delta_row + q0 + c * 32 + t4 * 4);
              const float dv4[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                const int cc = c * 32 + t4 * 4 + t;
                pv[cc] = pv[cc] * (__uint_as_float(r[c][t4 * 4 + t]) - dv4[t]) * p.scale;
              }
            }
          }
        }
        tc_fence_before_sync();
        mbar_arrive(&dp_empty[st]);
        if (!mbar_wait(ds_empty, (qc & 1) ^ 1, ab)) { ok = false; break; }
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) fa_store_chunk(dst, row, ch, 0, &pv[ch * 8]);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(ds_ready);
      }
      if (!ok) break;
      // ---- epilogue: dV, dK rows of this key
      if (!mbar_wait(acc_done, items & 1, ab)) { ok = false; break; }
      tc_fence_after_sync();
      const long long tok = static_cast<long long>(b) * p.S + key;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        elem_t* orow = (which == 0 ? p.dv : p.dk) + tok * p.dkv_pitch + static_cast<long long>(h) * kFaD;
        const uint32_t tm = which == 0 ? tm_dv : tm_dk;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tm + lane_sel + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 32; t += 8) {
            uint4 v;
            v.x = pack_e2(__uint_as_float(r[t + 0]), __uint_as_float(r[t + 1]));
            v.y = pack_e2(__uint_as_float(r[t + 2]), __uint_as_float(r[t + 3]));
            v.z = pack_e2(__uint_as_float(r[t + 4]), __uint_as_float(r[t + 5]));
            v.w = pack_e2(__uint_as_float(r[t + 6]), __uint_as_float(r[t + 7]));
            *reinterpret_cast<uint4*>(orow + c * 32 + t) = v;
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(acc_empty);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*cta_abort && threadIdx.x == 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000000ull) {
      if (mbar_try_wait(kv_full, 0) && mbar_try_wait(kv_full, 1)) break;
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------ dQ
struct DqSmem {
  static constexpr int kQ = 0;          // 32 KB
  static constexpr int kDO = 32768;     // 32 KB
  static constexpr int kK = 65536;      // 2 x 32 KB
  static constexpr int kV = 131072;     // 2 x 32 KB
  static constexpr int kDS = 196608;    // 32 KB
  static constexpr int kBar = 229376;
  static constexpr int kBytes = kBar + 256 + 1024;
};

__global__ void __launch_bounds__(kBwdThreads, 1)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const FaBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DqSmem::kBar);
  uint64_t* qdo_full = bars + 0;
  uint64_t* qdo_empty = bars + 1;
  uint64_t* k_full = bars + 2;    // [2]
  uint64_t* k_empty = bars + 4;   // [2]
  uint64_t* v_full = bars + 6;    // [2]
  uint64_t* v_empty = bars + 8;   // [2]
  uint64_t* s_full = bars + 10;   // [2]
  uint64_t* s_empty = bars + 12;  // [2]
  uint64_t* dp_full = bars + 14;
  uint64_t* dp_empty = bars + 15;
  uint64_t* ds_ready = bars + 16;
  uint64_t* ds_empty = bars + 17;
  uint64_t* dq_done = bars + 18;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const AbortCtx ab{cta_abort, p.status};
  const int nq = p.S / 128;
  const int total = p.B * p.H * nq;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
    }
    mbar_init(dp_full, 1);
    mbar_init(dp_empty, 128);
    mbar_init(ds_ready, 128);
    mbar_init(ds_empty, 1);
    mbar_init(dq_done, 1);
    *cta_abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 256, tm_dq = tmem_base + 384;

  auto item = [&](int w, int& b, int& h, int& qb) {
    const int bh = p.B * p.H;
    qb = nq - 1 - w / bh;
    const int r = w % bh;
    b = r / p.H;
    h = r % p.H;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t items = 0, kvc = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++items) {
        int b, h, qb;
        item(w, b, h, qb);
        const int nblk = p.causal ? qb + 1 : nq;
        if (!mbar_wait(qdo_empty, (items & 1) ^ 1, ab)) { ok = false; break; }
        mbar_expect_tx(qdo_full, 65536);
        fa_load_tile(smem + DqSmem::kQ, &tmQ, qdo_full, 128, h, qb * 128, b);
        fa_load_tile(smem + DqSmem::kDO, &tmDO, qdo_full, 128, h, qb * 128, b);
        for (int j = 0; j < nblk; ++j, ++kvc) {
          const int st = kvc & 1;
          const uint32_t ph = (kvc >> 1) & 1;
          if (!mbar_wait(&k_empty[st], ph ^ 1, ab)) { ok = false; break; }
          mbar_expect_tx(&k_full[st], 32768);
          fa_load_tile(smem + DqSmem::kK + st * 32768, &tmK, &k_full[st], 128, h, j * 128, b);
          if (!mbar_wait(&v_empty[st], ph ^ 1, ab)) { ok = false; break; }
          mbar_expect_tx(&v_full[st], 32768);
          fa_load_tile(smem + DqSmem::kV + st * 32768, &tmV, &v_full[st], 128, h, j * 128, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = umma_idesc_elem(128, 128, false, false);
      constexpr uint32_t idesc_mn = umma_idesc_elem(128, 128, false, true);
      const uint32_t q_addr = smem_u32(smem + DqSmem::kQ), do_addr = smem_u32(smem + DqSmem::kDO);
      const uint32_t ds_addr = smem_u32(smem + DqSmem::kDS);
      uint32_t items = 0, kvc = 0;
      bool ok = true;
      auto issue_s = [&](uint32_t c) -> bool {
        const int st = c & 1;
        const uint32_t ph = (c >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, ab)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, ab)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + DqSmem::kK + st * 32768);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tm_s + st * 128, umma_smem_desc(q_addr + off, 16, 1024), umma_smem_desc(k_addr + off, 16, 1024),
                    idesc_kk, kk != 0);
        }
        umma_commit(&s_full[st]);
        return true;
      };
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++items) {
        int b, h, qb;
        item(w, b, h, qb);
        const int nblk = p.causal ? qb + 1 : nq;
        if (!mbar_wait(qdo_full, items & 1, ab)) { ok = false; break; }
        if (!issue_s(kvc)) { ok = false; break; }
        for (int j = 0; j < nblk; ++j) {
          const uint32_t c = kvc + j;
          const int st = c & 1;
          const uint32_t ph = (c >> 1) & 1;
          const uint32_t k_addr = smem_u32(smem + DqSmem::kK + st * 32768);
          const uint32_t v_addr = smem_u32(smem + DqSmem::kV + st * 32768);
          if (!mbar_wait(&v_full[st], ph, ab)) { ok = false; break; }
          if (!mbar_wait(dp_empty, (c & 1) ^ 1, ab)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
            umma_bf16(tm_dp, umma_smem_desc(do_addr + off, 16, 1024), umma_smem_desc(v_addr + off, 16, 1024),
                      idesc_kk, kk != 0);
          }
          umma_commit(dp_full);
          umma_commit(&v_empty[st]);
          if (j + 1 < nblk && !issue_s(c + 1)) { ok = false; break; }
          if (!mbar_wait(ds_ready, c & 1, ab)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_bf16(tm_dq, umma_smem_desc(ds_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                      umma_smem_desc(k_addr + kk * 2048, 16384, 1024), idesc_mn, (j | kk) != 0);
          umma_commit(ds_empty);
          umma_commit(&k_empty[st]);
        }
        if (!ok) break;
        umma_commit(dq_done);
        umma_commit(qdo_empty);
        kvc += nblk;
      }
    }
    __syncwarp();
  } else {
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(q4 * 32) << 16;
    uint8_t* ds = smem + DqSmem::kDS;
    uint32_t items = 0, kvc = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++items) {
      int b, h, qb;
      item(w, b, h, qb);
      const int nblk = p.causal ? qb + 1 : nq;
      const long long stat = (static_cast<long long>(b) * p.H + h) * p.S + qb * 128 + row;
      const float lse2 = p.lse[stat] * 1.4426950408889634f;
      const float dl = p.delta[stat];
      for (int j = 0; j < nblk; ++j, ++kvc) {
        const int st = kvc & 1;
        const uint32_t ph = (kvc >> 1) & 1;
        float pv[128];
        if (!mbar_wait(&s_full[st], ph, ab)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          // two loads per wait (64 registers in flight beside the 128 of the row)
          uint32_t r[2][32];
          tmem_ld_32x32(tm_s + st * 128 + lane_sel + c2 * 64, r[0]);
          tmem_ld_32x32(tm_s + st * 128 + lane_sel + c2 * 64 + 32, r[1]);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int t = 0; t < 32; ++t)
              pv[c2 * 64 + c * 32 + t] = ex2(__uint_as_float(r[c][t]) * p.scale_log2 - lse2);
        }
        tc_fence_before_sync();
        mbar_arrive(&s_empty[st]);
        if (p.causal && j == qb) {
#pragma unroll
          for (int t = 0; t < 128; ++t)
            if (t > row) pv[t] = 0.f;
        }
        if (!mbar_wait(dp_full, kvc & 1, ab)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t r[2][32];
          tmem_ld_32x32(tm_dp + lane_sel + c2 * 64, r[0]);
          tmem_ld_32x32(tm_dp + lane_sel + c2 * 64 + 32, r[1]);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int t = 0; t < 32; ++t) {
              const int cc = c2 * 64 + c * 32 + t;
              pv[cc] = pv[cc] * (__uint_as_float(r[c][t]) - dl) * p.scale;
            }
        }
        tc_fence_before_sync();
        mbar_arrive(dp_empty);
        if (!mbar_wait(ds_empty, (kvc & 1) ^ 1, ab)) { ok = false; break; }
#pragma unroll
        for (int ch = 0; ch < 16; ++ch) fa_store_chunk(ds, row, ch, 16384, &pv[ch * 8]);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(ds_ready);
      }
      if (!ok) break;
      if (!mbar_wait(dq_done, items & 1, ab)) { ok = false; break; }
      tc_fence_after_sync();
      const long long tok = static_cast<long long>(b) * p.S + qb * 128 + row;
      elem_t* orow = p.dq + tok * p.dq_pitch + static_cast<long long>(h) * kFaD;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tm_dq + lane_sel + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; t += 8) {
          uint4 v;
          v.x = pack_e2(__uint_as_float(r[t + 0]), __uint_as_float(r[t + 1]));
          v.y = pack_e2(__uint_as_float(r[t + 2]), __uint_as_float(r[t + 3]));
          v.z = pack_e2(__uint_as_float(r[t + 4]), __uint_as_float(r[t + 5]));
          v.w = pack_e2(__uint_as_float(r[t + 6]), __uint_as_float(r[t + 7]));
          *reinterpret_cast<uint4*>(orow + c * 32 + t) = v;
        }
      }
      tc_fence_before_sync();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*cta_abort && threadIdx.x == 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000000ull) {
      if (mbar_try_wait(qdo_full, 0) && mbar_try_wait(qdo_full, 1)) break;
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace MSB_ELEM_NS
}  // namespace msb

using namespace msb;
using namespace msb::MSB_ELEM_NS;

static int fa_bwd_impl(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                       float* delta, void* dq, void* dk, void* dv, int B, int S, int H, int Hk, int D,
                       long long q_pitch, long long k_pitch, long long v_pitch, long long o_pitch, long long do_pitch,
                       long long dq_pitch, long long dkv_pitch, int causal, float scale, void* stream_) {
  if ((dq_pitch % 8) || (dkv_pitch % 8) || (reinterpret_cast<uintptr_t>(dq) & 15) ||
      (reinterpret_cast<uintptr_t>(dk) & 15) || (reinterpret_cast<uintptr_t>(dv) & 15)) {
    set_last_error("flash_attn_bwd: gradient pitches must be multiples of 8 elements and pointers 16-byte aligned");
    return kBadArg;
  }
  if (D != kFaD || S % 128 != 0 || S <= 0 || H != Hk || B <= 0) {
    set_last_error("flash_attn_bwd: needs head_dim 128, S a multiple of 128 and equal q/kv head counts "
                   "(got D=%d S=%d H=%d Hk=%d)", D, S, H, Hk);
    return kBadArg;
  }
  if (o_pitch % 4 || do_pitch % 8) {
    set_last_error("flash_attn_bwd: o/do pitches must be multiples of 8 elements");
    return kBadArg;
  }
  int* status = status_ptr();
  if (!status) { set_last_error("flash_attn_bwd: no status word"); return kCudaError; }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long warps = (long long)B * S * H;
  fa_delta_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const elem_t*>(o), static_cast<const elem_t*>(dout), delta, B, S, H, o_pitch,
      do_pitch);
  MSB_CUDA_CHECK(cudaGetLastError());

  CUtensorMap tq64, tdo64, tq128, tdo128, tk, tv;
  int rc;
  if ((rc = fa_encode_map(&tq64, q, B, S, H, q_pitch, 64)) != kOk) return rc;
  if ((rc = fa_encode_map(&tdo64, dout, B, S, H, do_pitch, 64)) != kOk) return rc;
  if ((rc = fa_encode_map(&tq128, q, B, S, H, q_pitch, 128)) != kOk) return rc;
  if ((rc = fa_encode_map(&tdo128, dout, B, S, H, do_pitch, 128)) != kOk) return rc;
  if ((rc = fa_encode_map(&tk, k, B, S, Hk, k_pitch, 128)) != kOk) return rc;
  if ((rc = fa_encode_map(&tv, v, B, S, Hk, v_pitch, 128)) != kOk) return rc;
  static bool configured = false;
  if (!configured) {
    MSB_CUDA_CHECK(cudaFuncSetAttribute(fa_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        KvSmem::kBytes));
    MSB_CUDA_CHECK(cudaFuncSetAttribute(fa_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        DqSmem::kBytes));
    configured = true;
  }
  FaBwdParams p;
  p.lse = lse; p.delta = delta;
  p.dq = static_cast<elem_t*>(dq);
  p.dk = static_cast<elem_t*>(dk);
  p.dv = static_cast<elem_t*>(dv);
  p.status = status;
  p.dq_pitch = dq_pitch;
  p.dkv_pitch = dkv_pitch;
  p.B = B; p.H = H; p.S = S; p.causal = causal;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int items = B * H * (S / 128);
  const int grid = items < sm_count() ? items : sm_count();
  fa_bwd_dkdv_kernel<<<grid, kBwdThreads, KvSmem::kBytes, stream>>>(tq64, tk, tv, tdo64, p);
  MSB_CUDA_CHECK(cudaGetLastError());
  fa_bwd_dq_kernel<<<grid, kBwdThreads, DqSmem::kBytes, stream>>>(tq128, tk, tv, tdo128, p);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

// All tensors token-major [B,S,H,128] with the given token pitches (elements).  delta: fp32 [B,H,S] scratch that
// this call fills.  dq / dk / dv are written densely ([B,S,H,128]).
MSB_EXPORT int MSB_FN(msb_flash_attn_bwd)(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                  const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S, int H,
                                  int Hk, int D, long long q_pitch, long long k_pitch, long long v_pitch,
                                  long long o_pitch, long long do_pitch, int causal, float scale, void* stream) {
  return fa_bwd_impl(q, k, v, o, dout, lse, delta, dq, dk, dv, B, S, H, Hk, D, q_pitch, k_pitch, v_pitch, o_pitch,
                     do_pitch, (long long)H * kFaD, (long long)Hk * kFaD, causal, scale, stream);
}

// Same, with the token pitches of the gradient outputs given: lets dq, dk, dv be column blocks of one packed
// [tokens, (H + 2 Hk) * 128] gradient of a fused QKV projection.
MSB_EXPORT int MSB_FN(msb_flash_attn_bwd_strided)(const void* q, const void* k, const void* v, const void* o,
                                          const void* dout, const float* lse, float* delta, void* dq, void* dk,
                                          void* dv, int B, int S, int H, int Hk, int D, long long q_pitch,
                                          long long k_pitch, long long v_pitch, long long o_pitch, long long do_pitch,
                                          long long dq_pitch, long long dkv_pitch, int causal, float scale,
                                          void* stream) {
  return fa_bwd_impl(q, k, v, o, dout, lse, delta, dq, dk, dv, B, S, H, Hk, D, q_pitch, k_pitch, v_pitch, o_pitch,
                     do_pitch, dq_pitch, dkv_pitch, causal, scale, stream);
}
