// FlashAttention forward for sm_100a (head_dim 128, bf16, causal or full), tcgen05 + TMEM + TMA.
//
// Tensors are token-major: q[b][s][h][d], k/v[b][s][hk][d], o[b][s][h][d]; row pitches are parameters so
// q/k/v may be column slices of one fused QKV GEMM output.  One work item = (batch, head, 128 query rows).
//
// Persistent CTA, 192 threads:
//   warp 0    : TMA producer  (Q once per item; K and V tiles of 128 keys, double-buffered)
//   warp 1    : MMA issuer    S[buf] = Q K^T into TMEM (double-buffered, so QK of block j+1 overlaps the
//                             softmax of block j), then O += P V
//   warps 2-5 : softmax       thread t owns query row t: reads its S row from TMEM (no shuffles), keeps the
//                             running max / sum, writes P (bf16) into 128B-swizzled shared memory as the A
//                             operand of the PV MMA, rescales O in TMEM only when the row max grew by more
//                             than 2^8 (warp-uniform decision), and finally normalises and stores O and LSE.
// TMEM: S0 [0,128) S1 [128,256) O [256,384) of a 512-column allocation.
//
// The reference defines FlashAttentionScore (core/ops/ops_def/flash_attention_score_op.yaml) but ships no GPU
// kernel for it; its GPU path would be BatchMatMul + Softmax + BatchMatMul through cuBLAS/cuDNN.
//
// This text is compiled twice: for bf16 tensors (flash_attn_sm100.cu), and with MSB_ELEM_FP16 defined for fp16 tensors
// (flash_attn_sm100_fp16.cu), where every entry point carries the suffix _fp16 and "bf16" in a comment reads "fp16".
#include "fa_common.cuh"

namespace msb {
namespace MSB_ELEM_NS {

constexpr int kFaBM = 128;       // query rows per item
constexpr int kFaBN = 128;       // keys per block
constexpr int kFaThreads = 192;
constexpr int kTileBytes = 128 * 128 * 2;  // 32 KB: one 128x128 bf16 tile (two 128B-swizzled halves)

struct FaParams {
  elem_t* o;
  float* lse;          // [B][H][S] natural-log sum-exp of scaled scores
  int* status;
  long long o_pitch;   // elements between consecutive tokens of o
  int B, H, Hk, S;
  int causal;
  float scale_log2;    // softmax scale * log2(e)
  float scale;
};

// shared memory map (1024B aligned): Q 32K | K0 32K | K1 32K | V0 32K | V1 32K | P 32K | barriers
struct FaSmem {
  static constexpr int kQ = 0;
  static constexpr int kK = kTileBytes;
  static constexpr int kV = 3 * kTileBytes;
  static constexpr int kP = 5 * kTileBytes;
  static constexpr int kBar = 6 * kTileBytes;
  static constexpr int kBytes = kBar + 256 + 1024;
};

__device__ __forceinline__ void fa_item(int w, const FaParams& p, int nq, int& b, int& h, int& qb) {
  const int bh = p.B * p.H;
  qb = nq - 1 - w / bh;     // longest (latest) query blocks first
  const int r = w % bh;
  b = r / p.H;
  h = r % p.H;
}

__global__ void __launch_bounds__(kFaThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FaSmem::kBar);
  uint64_t* q_full = bars + 0;
  uint64_t* q_empty = bars + 1;
  uint64_t* k_full = bars + 2;    // [2]
  uint64_t* k_empty = bars + 4;   // [2]
  uint64_t* v_full = bars + 6;    // [2]
  uint64_t* v_empty = bars + 8;   // [2]
  uint64_t* s_full = bars + 10;   // [2]
  uint64_t* s_empty = bars + 12;  // [2]
  uint64_t* p_ready = bars + 14;
  uint64_t* o_done = bars + 15;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const AbortCtx ab{cta_abort, p.status};
  const int nq = p.S / kFaBM;
  const int total = p.B * p.H * nq;
  const int group = p.H / p.Hk;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
    }
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
    *cta_abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      uint32_t items = 0, kvc = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++items) {
        int b, h, qb;
        fa_item(w, p, nq, b, h, qb);
        const int hk = h / group;
        const int nblk = p.causal ? qb + 1 : p.S / kFaBN;
        if (!mbar_wait(q_empty, (items & 1) ^ 1, ab)) { ok = false; break; }
        mbar_expect_tx(q_full, kTileBytes);
        tma_load_4d(smem + FaSmem::kQ, &tmQ, q_full, 0, h, qb * kFaBM, b);
        tma_load_4d(smem + FaSmem::kQ + 16384, &tmQ, q_full, 64, h, qb * kFaBM, b);
        for (int j = 0; j < nblk; ++j, ++kvc) {
          const int st = kvc & 1;
          const uint32_t ph = (kvc >> 1) & 1;
          if (!mbar_wait(&k_empty[st], ph ^ 1, ab)) { ok = false; break; }
          mbar_expect_tx(&k_full[st], kTileBytes);
          uint8_t* kd = smem + FaSmem::kK + st * kTileBytes;
          tma_load_4d(kd, &tmK, &k_full[st], 0, hk, j * kFaBN, b);
          tma_load_4d(kd + 16384, &tmK, &k_full[st], 64, hk, j * kFaBN, b);
          if (!mbar_wait(&v_empty[st], ph ^ 1, ab)) { ok = false; break; }
          mbar_expect_tx(&v_full[st], kTileBytes);
          uint8_t* vd = smem + FaSmem::kV + st * kTileBytes;
          tma_load_4d(vd, &tmV, &v_full[st], 0, hk, j * kFaBN, b);
          tma_load_4d(vd + 16384, &tmV, &v_full[st], 64, hk, j * kFaBN, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc_qk = umma_idesc_elem(128, 128, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_elem(128, 128, false, true);   // V is MN-major (d contiguous)
      const uint32_t q_addr = smem_u32(smem + FaSmem::kQ);
      const uint32_t p_addr = smem_u32(smem + FaSmem::kP);
      uint32_t items = 0, kvc = 0, sc = 0, pc = 0;
      bool ok = true;
      auto issue_qk = [&](uint32_t kv_index, uint32_t s_index) -> bool {
        const int st = kv_index & 1;
        const int sb = s_index & 1;
        if (!mbar_wait(&k_full[st], (kv_index >> 1) & 1, ab)) return false;
        if (!mbar_wait(&s_empty[sb], ((s_index >> 1) & 1) ^ 1, ab)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + FaSmem::kK + st * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < kFaD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem_base + sb * 128, umma_smem_desc(q_addr + off, 16, 1024),
                    umma_smem_desc(k_addr + off, 16, 1024), idesc_qk, kk != 0);
        }
        umma_commit(&s_full[sb]);
        umma_commit(&k_empty[st]);
        return true;
      };
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++items) {
        int b, h, qb;
        fa_item(w, p, nq, b, h, qb);
        const int nblk = p.causal ? qb + 1 : p.S / kFaBN;
        if (!mbar_wait(q_full, items & 1, ab)) { ok = false; break; }
        if (!issue_qk(kvc, sc)) { ok = false; break; }
        ++sc;
        for (int j = 0; j < nblk; ++j) {
          if (j + 1 < nblk) {
            if (!issue_qk(kvc + 1 + j, sc)) { ok = false; break; }
            ++sc;
          } else {
            umma_commit(q_empty);  // last QK of this item is in flight: Q may be reloaded when it retires
          }
          const uint32_t kv_index = kvc + j;
          const int st = kv_index & 1;
          if (!mbar_wait(p_ready, pc & 1, ab)) { ok = false; break; }
          ++pc;
          if (!mbar_wait(&v_full[st], (kv_index >> 1) & 1, ab)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t v_addr = smem_u32(smem + FaSmem::kV + st * kTileBytes);
#pragma unroll
          for (int kk = 0; kk < kFaBN / 16; ++kk) {
            const uint64_t adesc = umma_smem_desc(p_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
            const uint64_t bdesc = umma_smem_desc(v_addr + kk * 2048, 16384, 1024);
            umma_bf16(tmem_o, adesc, bdesc, idesc_pv, (j | kk) != 0);
          }
          umma_commit(&v_empty[st]);
          umma_commit(o_done);
        }
        kvc += nblk;
      }
    }
    __syncwarp();
  } else {
    // -------------------------------------------------------------------- softmax / correction / epilogue
    const int q = warp & 3;
    const int row = q * 32 + lane;                 // row inside the 128-row tile == TMEM lane
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* p_smem = smem + FaSmem::kP;
    uint32_t sc = 0, oc = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
      int b, h, qb;
      fa_item(w, p, nq, b, h, qb);
      const int nblk = p.causal ? qb + 1 : p.S / kFaBN;
      float m_used = -INFINITY;   // max the stored probabilities are relative to (log2 domain)
      float l = 0.f;
      for (int j = 0; j < nblk; ++j, ++sc) {
        const int sb = sc & 1;
        if (!mbar_wait(&s_full[sb], (sc >> 1) & 1, ab)) { ok = false; break; }
        tc_fence_after_sync();
        // raw scores; the softmax scale is folded into the exponent below (one FFMA per element) and every
        // reduction runs on four independent accumulators: with one warp per scheduler a serial chain of 128
        // dependent max / add instructions would cost its full latency 128 times
        float s[128];
        {
          // the four loads are issued back to back and waited for once: one TMEM round trip instead of four
          uint32_t r[4][32];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld_32x32(tmem_base + sb * 128 + lane_sel + c * 32, r[c]);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(r[c][i]);
        }
        tc_fence_before_sync();
        mbar_arrive(&s_empty[sb]);
        if (p.causal && j == qb) {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i > row) s[i] = -INFINITY;
        }
        float mx4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
        for (int i = 4; i < 128; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], s[i]);
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;   // scale > 0
        // rescale only when some row of this warp grew its max by more than 8 (in log2 units)
        const bool grow = mx > m_used + 8.f;
        const bool warp_grow = __any_sync(0xffffffffu, grow);
        float alpha = 1.f;
        if (warp_grow) {
          const float m_new = fmaxf(m_used, mx);
          alpha = (m_used == -INFINITY) ? 0.f : ex2(m_used - m_new);
          m_used = m_new;
        }
        const float neg_m = -m_used;
        float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          s[i] = ex2(fmaf(s[i], p.scale_log2, neg_m));
          rs4[i & 3] += s[i];
        }
        l = l * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
        if (j > 0) {
          // previous PV must have retired before O is rescaled or P is overwritten
          if (!mbar_wait(o_done, oc & 1, ab)) { ok = false; break; }
          ++oc;
          tc_fence_after_sync();
          if (warp_grow) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t r[32];
              tmem_ld_32x32(tmem_o + lane_sel + c * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32(tmem_o + lane_sel + c * 32, r);
            }
            tmem_st_wait();
          }
        }
        // P row -> shared memory, K-major 128B swizzle: 16-byte chunk ch of row r lands at chunk (ch ^ (r & 7))
#pragma unroll
        for (int ch = 0; ch < 16; ++ch) {
          uint4 v;
          v.x = pack_e2(s[ch * 8 + 0], s[ch * 8 + 1]);
          v.y = pack_e2(s[ch * 8 + 2], s[ch * 8 + 3]);
          v.z = pack_e2(s[ch * 8 + 4], s[ch * 8 + 5]);
          v.w = pack_e2(s[ch * 8 + 6], s[ch * 8 + 7]);
          const int half = ch >> 3, cc = ch & 7;
          *reinterpret_cast<uint4*>(p_smem + half * 16384 + row * 128 + ((cc ^ (row & 7)) << 4)) = v;
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(p_ready);
      }
      if (!ok) break;
      // ---- epilogue: O / l -> global, LSE
      if (!mbar_wait(o_done, oc & 1, ab)) { ok = false; break; }
      ++oc;
      tc_fence_after_sync();
      const float inv_l = 1.f / l;
      const long long tok = static_cast<long long>(b) * p.S + qb * kFaBM + row;
      elem_t* orow = p.o + tok * p.o_pitch + static_cast<long long>(h) * kFaD;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_o + lane_sel + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 v;
          v.x = pack_e2(__uint_as_float(r[i + 0]) * inv_l, __uint_as_float(r[i + 1]) * inv_l);
          v.y = pack_e2(__uint_as_float(r[i + 2]) * inv_l, __uint_as_float(r[i + 3]) * inv_l);
          v.z = pack_e2(__uint_as_float(r[i + 4]) * inv_l, __uint_as_float(r[i + 5]) * inv_l);
          v.w = pack_e2(__uint_as_float(r[i + 6]) * inv_l, __uint_as_float(r[i + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + c * 32 + i) = v;
        }
      }
      tc_fence_before_sync();
      if (p.lse) {
        p.lse[(static_cast<long long>(b) * p.H + h) * p.S + qb * kFaBM + row] =
            (m_used + log2f(l)) * 0.6931471805599453f;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*cta_abort && threadIdx.x == 0) {
    // a wait was abandoned: give bulk copies that may still be in flight a bounded time to land
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000000ull) {
      if (mbar_try_wait(q_full, 0) && mbar_try_wait(q_full, 1)) break;
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

// q [B,S,H,128], k/v [B,S,Hk,128] with token pitches (elements) q_pitch / k_pitch / v_pitch; o [B,S,H,128] with o_pitch.
// S must be a multiple of 128.  lse (fp32 [B,H,S]) may be null.
MSB_EXPORT int MSB_FN(msb_flash_attn_fwd)(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S,
                                  int H, int Hk, int D, long long q_pitch, long long k_pitch, long long v_pitch,
                                  long long o_pitch,
                                  int causal, float scale, void* stream_) {
  if (D != kFaD || S % 128 != 0 || S <= 0 || H % Hk != 0 || B <= 0) {
    set_last_error("flash_attn_fwd: needs head_dim 128, S a multiple of 128 and H a multiple of Hk "
                   "(got D=%d S=%d H=%d Hk=%d)", D, S, H, Hk);
    return kBadArg;
  }
  if (o_pitch % 8) {
    set_last_error("flash_attn_fwd: o_pitch must be a multiple of 8");
    return kBadArg;
  }
  int* status = status_ptr();
  if (!status) { set_last_error("flash_attn_fwd: no status word"); return kCudaError; }
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = fa_encode_map(&tq, q, B, S, H, q_pitch, 128)) != kOk) return rc;
  if ((rc = fa_encode_map(&tk, k, B, S, Hk, k_pitch, 128)) != kOk) return rc;
  if ((rc = fa_encode_map(&tv, v, B, S, Hk, v_pitch, 128)) != kOk) return rc;
  static bool configured = false;
  if (!configured) {
    MSB_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        FaSmem::kBytes));
    configured = true;
  }
  FaParams p;
  p.o = static_cast<elem_t*>(o);
  p.lse = lse;
  p.status = status;
  p.o_pitch = o_pitch;
  p.B = B; p.H = H; p.Hk = Hk; p.S = S;
  p.causal = causal;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int total = B * H * (S / 128);
  const int grid = total < sm_count() ? total : sm_count();
  flash_fwd_kernel<<<grid, kFaThreads, FaSmem::kBytes, static_cast<cudaStream_t>(stream_)>>>(tq, tk, tv, p);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
