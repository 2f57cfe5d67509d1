// NHWC bf16 convolution as an implicit GEMM on tcgen05: no im2col matrix is ever written.
//
// Forward / data gradient (WGRAD = false):  Y[pix, co] = sum_{tap, ci} X[pix + offset(tap), ci] * W[co, tap, ci]
//   GEMM M = output pixels, N = output channels, K = taps * Cin.  A tile of 128 output pixels is a box
//   (tw x th x tn) of the output grid; for filter tap t and channel block c the A operand of that k-block is one
//   4-D TMA load of the input at (c, w0 + dw[t], h0 + dh[t], n0): 128 rows of 64 channels, 128-byte swizzled, i.e.
//   exactly the K-major tile the MMA wants.  Padding is the TMA's out-of-bounds zero fill.  Strided convolutions
//   read one of up to four "parity planes" of the input (views with doubled W/H strides), chosen per tap, so the
//   same box load applies.  The epilogue writes bf16 NHWC rows and can accumulate the per-channel sum and sum of
//   squares of the output in shared memory (flushed once per CTA) - the BatchNorm statistics come for free.
// Weight gradient (WGRAD = true):  dW[co, tap, ci] = sum_pix dY[pix, co] * X[pix + offset(tap), ci]
//   GEMM M = Cout, N = Cin, K = pixels; both operands are MN-major 4-D box loads (64 pixels x 64 channels), the
//   k-loop runs over pixel tiles and is split across CTAs (fp32 atomic accumulation into dW).
//
// The reference calls cudnnConvolutionForward / BackwardData / BackwardFilter
// (plugin/device/gpu/kernel/nn/conv2d_gpu_kernel.h, conv2d_grad_input_gpu_kernel.h, conv2d_grad_filter_gpu_kernel.h)
// followed by a separate cuDNN BatchNorm pass over the output.
//
// This text is compiled twice: for bf16 tensors (conv_sm100.cu), and with MSB_ELEM_FP16 defined for fp16 tensors
// (conv_sm100_fp16.cu), where every entry point carries the suffix _fp16 and "bf16" in a comment reads "fp16".
#include "host_common.h"
#include "elem.cuh"

namespace msb {
namespace MSB_ELEM_NS {

constexpr int kConvBM = 128;
constexpr int kConvBK = 64;
constexpr int kConvThreads = 192;
constexpr int kMaxTaps = 49;
constexpr int kMaxStatChannels = 2048;

struct ConvParams {
  void* C;
  float* stats;          // fwd: [2 * Cout] running sum / sum of squares of the bf16 output, or nullptr
  int* status;
  int N, Ho, Wo;         // pixel grid that the boxes tile (fwd: output pixels; wgrad: dY pixels)
  int tw, th, tn;        // box extents (product 128 fwd, 64 wgrad)
  int tiles_w, tiles_h, tiles_n;
  int cin_blocks;        // fwd: Cin / 64
  int taps;
  int Cout, Cin;
  long long ldc;         // fwd: elements between output pixels; wgrad: elements between rows of dW
  int out_fp32, accumulate, ksplit;
  short tap_map[kMaxTaps], tap_dh[kMaxTaps], tap_dw[kMaxTaps];
};

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c, int w,
                                            int h, int n) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h),
      "r"(n)
      : "memory");
}

template <int BN>
struct ConvCfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = kConvBM * kConvBK * 2;
  static constexpr int kBBytes = BN * kConvBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kStatOffset = kBarOffset + 256;
  static constexpr int kSmemBytes = kStatOffset + 2 * kMaxStatChannels * 4 + 1024;
};

// Sum over the 32 lanes of a warp of v[j], for every j: afterwards lane j holds the total of column j in v[0].
__device__ __forceinline__ float warp_column_sums(float (&v)[32], int lane) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < off; ++i) {
      const float send = upper ? v[i] : v[i + off];
      const float keep = upper ? v[i + off] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  return v[0];
}

template <int BN, bool WGRAD>
__global__ void __launch_bounds__(kConvThreads, 1)
conv_igemm_kernel(const __grid_constant__ CUtensorMap tmX0, const __grid_constant__ CUtensorMap tmX1,
                  const __grid_constant__ CUtensorMap tmX2, const __grid_constant__ CUtensorMap tmX3,
                  const __grid_constant__ CUtensorMap tmO, const ConvParams p) {
  // tmX*: input activations (parity planes).  tmO: fwd = weights [Cout, taps*Cin] (3-D map, K-major);
  // wgrad = dY (4-D map).
  using Cfg = ConvCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * Cfg::kABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* issued_cnt = cta_abort + 1;
  volatile int* consumed_cnt = cta_abort + 2;
  float* s_stats = reinterpret_cast<float*>(smem + Cfg::kStatOffset);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AbortCtx ab{cta_abort, p.status};
  const CUtensorMap* maps[4] = {&tmX0, &tmX1, &tmX2, &tmX3};

  const int pix_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
  // GEMM tiling
  const int gemm_m = WGRAD ? p.Cout : 0;
  const int tiles_m = WGRAD ? (gemm_m + kConvBM - 1) / kConvBM : pix_tiles;
  const int gemm_n = WGRAD ? p.Cin : p.Cout;
  const int tiles_n = (gemm_n + BN - 1) / BN;
  const int outer = WGRAD ? p.taps * p.ksplit : 1;
  const int total_tiles = tiles_m * tiles_n * outer;
  const int kb_total = WGRAD ? pix_tiles : p.taps * p.cin_blocks;
  const int kb_per = WGRAD ? (kb_total + p.ksplit - 1) / p.ksplit : kb_total;
  const bool want_stats = !WGRAD && p.stats != nullptr;

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
    tma_prefetch_desc(&tmX0);
    tma_prefetch_desc(&tmO);
  }
  if (want_stats)
    for (int i = threadIdx.x; i < 2 * p.Cout; i += kConvThreads) s_stats[i] = 0.f;
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (outer index, m block, n block); m fastest so that CTAs running together share the weight tile
  auto tile_coords = [&](int tile, int& o, int& m_blk, int& n_blk) {
    o = tile / (tiles_m * tiles_n);
    const int t = tile - o * tiles_m * tiles_n;
    m_blk = t % tiles_m;
    n_blk = t / tiles_m;
  };
  auto pixel_origin = [&](int pt, int& n0, int& h0, int& w0) {
    const int iw = pt % p.tiles_w;
    const int ih = (pt / p.tiles_w) % p.tiles_h;
    const int in_ = pt / (p.tiles_w * p.tiles_h);
    n0 = in_ * p.tn;
    h0 = ih * p.th;
    w0 = iw * p.tw;
  };
  auto k_range = [&](int o, int& kb_lo, int& kb_hi) {
    if (WGRAD) {
      const int split = o % p.ksplit;
      kb_lo = split * kb_per;
      kb_hi = min(kb_lo + kb_per, kb_total);
    } else {
      kb_lo = 0;
      kb_hi = kb_total;
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
        int o, m_blk, n_blk, kb_lo, kb_hi;
        tile_coords(tile, o, m_blk, n_blk);
        k_range(o, kb_lo, kb_hi);
        const int nc0 = n_blk * BN;
        int n0 = 0, h0 = 0, w0 = 0;
        if (!WGRAD) pixel_origin(m_blk, n0, h0, w0);
        const int tap_w = WGRAD ? o / p.ksplit : 0;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, ab)) { ok = false; break; }
          mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
          uint8_t* a_dst = smem_a + s * Cfg::kABytes;
          uint8_t* b_dst = smem_b + s * Cfg::kBBytes;
          if (WGRAD) {
            pixel_origin(kb, n0, h0, w0);
            const int m0 = m_blk * kConvBM;
#pragma unroll
            for (int j = 0; j < kConvBM / 64; ++j)
              tma_load_4d(a_dst + j * 8192, &tmO, &full_bar[s], m0 + 64 * j, w0, h0, n0);
            const CUtensorMap* mx = maps[p.tap_map[tap_w]];
            const int dh = p.tap_dh[tap_w], dw = p.tap_dw[tap_w];
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_4d(b_dst + j * 8192, mx, &full_bar[s], nc0 + 64 * j, w0 + dw, h0 + dh, n0);
          } else {
            const int tap = kb / p.cin_blocks;
            const int cb = kb - tap * p.cin_blocks;
            tma_load_4d(a_dst, maps[p.tap_map[tap]], &full_bar[s], cb * 64, w0 + p.tap_dw[tap], h0 + p.tap_dh[tap],
                        n0);
            tma_load_3d(b_dst, &tmO, &full_bar[s], kb * kConvBK, nc0, 0);
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
      constexpr uint32_t idesc = umma_idesc_elem(kConvBM, BN, WGRAD, WGRAD);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      int consumed = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        int o, m_blk, n_blk, kb_lo, kb_hi;
        tile_coords(tile, o, m_blk, n_blk);
        k_range(o, kb_lo, kb_hi);
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, ab)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, ab)) { ok = false; break; }
          ++consumed;
          *consumed_cnt = consumed;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + s * Cfg::kABytes);
          const uint32_t b_addr = smem_u32(smem_b + s * Cfg::kBBytes);
#pragma unroll
          for (int kk = 0; kk < kConvBK / 16; ++kk) {
            const uint64_t adesc = WGRAD ? umma_smem_desc(a_addr + kk * 2048, 8192, 1024)
                                         : umma_smem_desc(a_addr + kk * 32, 16, 1024);
            const uint64_t bdesc = WGRAD ? umma_smem_desc(b_addr + kk * 2048, 8192, 1024)
                                         : umma_smem_desc(b_addr + kk * 32, 16, 1024);
            umma_bf16(d_tmem, adesc, bdesc, idesc, (kb != kb_lo) || (kk != 0));
          }
          umma_commit(&empty_bar[s]);
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&tfull_bar[acc]);
      }
    }
    __syncwarp();
  } else {
    // -------------------------------------------------------------------- epilogue (warps 2-5)
    const int q = warp & 3;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      int o, m_blk, n_blk, kb_lo, kb_hi;
      tile_coords(tile, o, m_blk, n_blk);
      k_range(o, kb_lo, kb_hi);
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, ab)) { ok = false; break; }
      tc_fence_after_sync();
      const int r = q * 32 + lane;
      const int nc0 = n_blk * BN;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      bool row_ok;
      long long c_off;
      if (WGRAD) {
        const int co = m_blk * kConvBM + r;
        row_ok = co < p.Cout && kb_lo < kb_hi;
        c_off = static_cast<long long>(co) * p.ldc + static_cast<long long>(o / p.ksplit) * p.Cin;
      } else {
        int n0, h0, w0;
        pixel_origin(m_blk, n0, h0, w0);
        const int n = n0 + r / (p.tw * p.th), h = h0 + (r / p.tw) % p.th, w = w0 + r % p.tw;
        row_ok = n < p.N && h < p.Ho && w < p.Wo;
        c_off = ((static_cast<long long>(n) * p.Ho + h) * p.Wo + w) * p.ldc;
      }
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        if (nc0 + c >= gemm_n) break;  // warp-uniform
        uint32_t rr[32];
        tmem_ld_32x32(t_row + c, rr);
        tmem_ld_wait();
        const int col0 = nc0 + c;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = row_ok ? __uint_as_float(rr[j]) : 0.f;
        if (WGRAD || p.out_fp32) {
          float* dst = static_cast<float*>(p.C) + c_off + col0;
          if (row_ok) {
            if (WGRAD && (p.ksplit > 1 || p.accumulate)) {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < gemm_n) atomicAdd(dst + j, v[j]);
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < gemm_n) dst[j] = v[j];
            }
          }
        } else {
          elem_t* dst = static_cast<elem_t*>(p.C) + c_off + col0;
          const bool full = (col0 + 32 <= gemm_n);
          if (row_ok) {
            if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 ov;
                ov.x = pack_e2(v[j], v[j + 1]);
                ov.y = pack_e2(v[j + 2], v[j + 3]);
                ov.z = pack_e2(v[j + 4], v[j + 5]);
                ov.w = pack_e2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(dst + j) = ov;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < gemm_n) dst[j] = f_to_e(v[j]);
            }
          }
          if (want_stats) {
            // statistics of what was stored (the rounded values); rows outside the image contribute zero
            float sq[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              v[j] = e_to_f(f_to_e(v[j]));
              sq[j] = v[j] * v[j];
            }
            const float s1 = warp_column_sums(v, lane);
            const float s2 = warp_column_sums(sq, lane);
            if (col0 + lane < p.Cout) {
              atomicAdd(&s_stats[col0 + lane], s1);
              atomicAdd(&s_stats[p.Cout + col0 + lane], s2);
            }
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&tempty_bar[acc]);
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (want_stats)
    for (int i = threadIdx.x; i < 2 * p.Cout; i += kConvThreads)
      if (s_stats[i] != 0.f) atomicAdd(p.stats + i, s_stats[i]);
  if (*cta_abort && threadIdx.x == 0) {
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

}  // namespace MSB_ELEM_NS
}  // namespace msb

using namespace msb;
using namespace msb::MSB_ELEM_NS;

namespace {

// Box (tw, th, tn) with tw*th*tn == pixels_per_tile (all powers of two) that covers the N x H x W grid with the
// fewest tiles; ties go to the widest box.
void pick_box(int N, int H, int W, int pixels_per_tile, int* tw, int* th, int* tn) {
  long long best = -1;
  for (int a = 1; a <= pixels_per_tile; a <<= 1) {
    for (int b = 1; a * b <= pixels_per_tile; b <<= 1) {
      const int c = pixels_per_tile / (a * b);
      if (a > 256 || b > 256 || c > 256) continue;
      const long long tiles = static_cast<long long>((W + a - 1) / a) * ((H + b - 1) / b) * ((N + c - 1) / c);
      if (best < 0 || tiles < best || (tiles == best && a > *tw)) {
        best = tiles;
        *tw = a; *th = b; *tn = c;
      }
    }
  }
}

// Tensor maps of the (parity planes of the) NHWC input and the tap table.
int setup_input(CUtensorMap maps[4], ConvParams* p, const void* x, int N, int H, int W, int C, long long ldx, int R,
                int S, int stride, int pad_h, int pad_w, int flip) {
  if (stride != 1 && stride != 2) { set_last_error("conv: stride %d is not supported (1 or 2)", stride); return kBadArg; }
  if (R * S > kMaxTaps) { set_last_error("conv: %dx%d filter has more than %d taps", R, S, kMaxTaps); return kBadArg; }
  if (ldx % 8) { set_last_error("conv: pixel pitch %lld must be a multiple of 8 elements", ldx); return kBadArg; }
  const uint32_t box[4] = {64u, (uint32_t)p->tw, (uint32_t)p->th, (uint32_t)p->tn};
  const int planes = stride == 1 ? 1 : 4;
  for (int pl = 0; pl < 4; ++pl) {
    const int ph = stride == 1 ? 0 : (pl >> 1), pw = stride == 1 ? 0 : (pl & 1);
    if (pl >= planes || ph >= H || pw >= W) { maps[pl] = maps[0]; continue; }
    const elem_t* base = static_cast<const elem_t*>(x) + (static_cast<long long>(ph) * W + pw) * ldx;
    const uint64_t dims[4] = {(uint64_t)C, (uint64_t)((W - pw + stride - 1) / stride),
                              (uint64_t)((H - ph + stride - 1) / stride), (uint64_t)N};
    const uint64_t st[3] = {(uint64_t)(stride * ldx * 2), (uint64_t)(stride * W * ldx * 2),
                            (uint64_t)((long long)H * W * ldx * 2)};
    if (int rc = encode_tmap_4d(&maps[pl], base, dims, st, box)) return rc;
  }
  p->taps = R * S;
  for (int r = 0; r < R; ++r) {
    for (int s = 0; s < S; ++s) {
      const int oh = flip ? pad_h - r : r - pad_h, ow = flip ? pad_w - s : s - pad_w;
      const int ph = stride == 1 ? 0 : (oh & 1), pw = stride == 1 ? 0 : (ow & 1);
      const int t = r * S + s;
      p->tap_map[t] = static_cast<short>(stride == 1 ? 0 : ph * 2 + pw);
      p->tap_dh[t] = static_cast<short>(stride == 1 ? oh : (oh - ph) / 2);
      p->tap_dw[t] = static_cast<short>(stride == 1 ? ow : (ow - pw) / 2);
    }
  }
  return kOk;
}

template <int BN, bool WGRAD>
int launch_conv(const CUtensorMap maps[4], const CUtensorMap& tmO, const ConvParams& p, int tiles,
                cudaStream_t stream) {
  using Cfg = ConvCfg<BN>;
  auto kern = conv_igemm_kernel<BN, WGRAD>;
  static bool configured = false;
  if (!configured) {
    MSB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kConvThreads, Cfg::kSmemBytes, stream>>>(maps[0], maps[1], maps[2], maps[3], tmO, p);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}

}  // namespace

// y[N, Ho, Wo, Cout] = conv(x[N, H, W, Cin], w[Cout, R, S, Cin]); bf16 NHWC; ldx / ldy = elements between pixels.
// flip = 0: y[ho, wo] += x[ho*stride + r - pad_h, wo*stride + s - pad_w] * w[r, s]      (forward)
// flip = 1: y[ho, wo] += x[ho + pad_h - r, wo + pad_w - s] * w[r, s]  (stride 1 only)   (data gradient, with
//           x = dY, w = weights permuted to [Cin, R, S, Cout])
// stats (optional): fp32 [2 * Cout], += per-channel sum and sum of squares of y (caller zeroes it).
// Cin must be a multiple of 64.
MSB_EXPORT int MSB_FN(msb_conv_fwd)(const void* x, const void* w, void* y, float* stats, int N, int H, int W, int Cin,
                            int Cout, int R, int S, int stride, int pad_h, int pad_w, int flip, int Ho, int Wo,
                            long long ldx, long long ldy, int out_fp32, void* stream_) {
  if (N <= 0 || H <= 0 || W <= 0 || Ho <= 0 || Wo <= 0 || Cin <= 0 || Cout <= 0 || (Cin % 64)) {
    set_last_error("conv_fwd: bad shape N=%d H=%d W=%d Cin=%d (multiple of 64) Cout=%d Ho=%d Wo=%d", N, H, W, Cin,
                   Cout, Ho, Wo);
    return kBadArg;
  }
  if (flip && stride != 1) { set_last_error("conv_fwd: the data-gradient form needs stride 1"); return kBadArg; }
  if (stats && (Cout > kMaxStatChannels || out_fp32)) {
    set_last_error("conv_fwd: fused statistics need bf16 output and at most %d channels", kMaxStatChannels);
    return kBadArg;
  }
  ConvParams p = {};
  p.C = y; p.stats = stats; p.status = status_ptr();
  if (!p.status) { set_last_error("conv_fwd: no status word"); return kCudaError; }
  p.N = N; p.Ho = Ho; p.Wo = Wo; p.Cin = Cin; p.Cout = Cout; p.ldc = ldy; p.out_fp32 = out_fp32; p.ksplit = 1;
  pick_box(N, Ho, Wo, kConvBM, &p.tw, &p.th, &p.tn);
  p.tiles_w = (Wo + p.tw - 1) / p.tw; p.tiles_h = (Ho + p.th - 1) / p.th; p.tiles_n = (N + p.tn - 1) / p.tn;
  p.cin_blocks = Cin / 64;
  CUtensorMap maps[4], tmW;
  if (int rc = setup_input(maps, &p, x, N, H, W, Cin, ldx, R, S, stride, pad_h, pad_w, flip)) return rc;
  const long long pix_tiles = static_cast<long long>(p.tiles_w) * p.tiles_h * p.tiles_n;
  const int bn = (Cout <= 128 || pix_tiles * ((Cout + 255) / 256) < sm_count()) ? 128 : 256;
  const long long K = static_cast<long long>(R) * S * Cin;
  if (int rc = encode_tmap_3d(&tmW, w, 2, K, Cout, 1, K * 2, K * 2 * Cout, 64, bn, 1)) return rc;
  const long long tiles = pix_tiles * ((Cout + bn - 1) / bn);
  if (tiles > 0x7fffffffLL) { set_last_error("conv_fwd: too many tiles"); return kTooLarge; }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (bn == 256) return launch_conv<256, false>(maps, tmW, p, (int)tiles, stream);
  return launch_conv<128, false>(maps, tmW, p, (int)tiles, stream);
}

// dw[Cout, R, S, Cin] (fp32) (+)= sum over pixels of dy[N, Ho, Wo, Cout] x shifted x[N, H, W, Cin].
MSB_EXPORT int MSB_FN(msb_conv_wgrad)(const void* x, const void* dy, float* dw, int N, int H, int W, int Cin, int Cout,
                              int R, int S, int stride, int pad_h, int pad_w, int Ho, int Wo, long long ldx,
                              long long ldy, int accumulate, void* stream_) {
  if (N <= 0 || H <= 0 || W <= 0 || Ho <= 0 || Wo <= 0 || Cin <= 0 || Cout <= 0 || (Cin % 8) || (Cout % 8) ||
      (ldy % 8)) {
    set_last_error("conv_wgrad: bad shape N=%d H=%d W=%d Cin=%d Cout=%d Ho=%d Wo=%d (channels multiples of 8)", N, H,
                   W, Cin, Cout, Ho, Wo);
    return kBadArg;
  }
  ConvParams p = {};
  p.C = dw; p.status = status_ptr();
  if (!p.status) { set_last_error("conv_wgrad: no status word"); return kCudaError; }
  p.N = N; p.Ho = Ho; p.Wo = Wo; p.Cin = Cin; p.Cout = Cout; p.out_fp32 = 1; p.accumulate = 1;
  p.ldc = static_cast<long long>(R) * S * Cin;
  pick_box(N, Ho, Wo, kConvBK, &p.tw, &p.th, &p.tn);
  p.tiles_w = (Wo + p.tw - 1) / p.tw; p.tiles_h = (Ho + p.th - 1) / p.th; p.tiles_n = (N + p.tn - 1) / p.tn;
  CUtensorMap maps[4], tmDY;
  if (int rc = setup_input(maps, &p, x, N, H, W, Cin, ldx, R, S, stride, pad_h, pad_w, 0)) return rc;
  const uint32_t box[4] = {64u, (uint32_t)p.tw, (uint32_t)p.th, (uint32_t)p.tn};
  const uint64_t dims[4] = {(uint64_t)Cout, (uint64_t)Wo, (uint64_t)Ho, (uint64_t)N};
  const uint64_t st[3] = {(uint64_t)(ldy * 2), (uint64_t)(Wo * ldy * 2), (uint64_t)((long long)Ho * Wo * ldy * 2)};
  if (int rc = encode_tmap_4d(&tmDY, dy, dims, st, box)) return rc;
  const int bn = Cin <= 128 ? 128 : 256;
  const long long base_tiles = static_cast<long long>((Cout + kConvBM - 1) / kConvBM) * ((Cin + bn - 1) / bn) * p.taps;
  const long long pix_tiles = static_cast<long long>(p.tiles_w) * p.tiles_h * p.tiles_n;
  long long split = (2LL * sm_count() + base_tiles - 1) / base_tiles;
  if (split > pix_tiles) split = pix_tiles;
  if (split < 1) split = 1;
  p.ksplit = static_cast<int>(split);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!accumulate)
    MSB_CUDA_CHECK(cudaMemsetAsync(dw, 0, sizeof(float) * static_cast<size_t>(Cout) * R * S * Cin, stream));
  const long long tiles = base_tiles * split;
  if (bn == 256) return launch_conv<256, true>(maps, tmDY, p, (int)tiles, stream);
  return launch_conv<128, true>(maps, tmDY, p, (int)tiles, stream);
}

namespace msb {
namespace MSB_ELEM_NS {
// Patch matrix for convolutions whose input has too few channels for the 64-channel box loads (the first layer of
// image networks): out[pix, (r*S + s)*Cin + c] = x[n, ho*stride + r - pad, wo*stride + s - pad, c], zero outside the
// image and in the padding columns k >= R*S*Cin.
__global__ void __launch_bounds__(256)
im2col_nhwc_kernel(const elem_t* __restrict__ x, elem_t* __restrict__ out, int N, int H, int W, int Cin,
                   int R, int S, int stride, int pad_h, int pad_w, int Ho, int Wo, int Kpad) {
  // One thread per 16-byte chunk (8 columns) of a patch row, so stores are coalesced; where column k comes from
  // (filter row, offset inside the contiguous S*Cin input segment) is looked up in a table built once per block.
  extern __shared__ short tab[];          // [Kpad][2]: filter row (or -1 for padding columns), segment offset
  const int K = R * S * Cin, seg = S * Cin;
  for (int k = threadIdx.x; k < Kpad; k += blockDim.x) {
    tab[2 * k] = k < K ? (short)(k / seg) : (short)-1;
    tab[2 * k + 1] = (short)(k % seg);
  }
  __syncthreads();
  const int chunks = Kpad / 8;
  const long long total = (long long)N * Ho * Wo * chunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % chunks);
    const long long pix = i / chunks;
    const int wo = (int)(pix % Wo);
    const int ho = (int)((pix / Wo) % Ho);
    const int n = (int)(pix / ((long long)Wo * Ho));
    const int h0 = ho * stride - pad_h, w0 = wo * stride - pad_w;
    const elem_t* img = x + (long long)n * H * W * Cin;
    __align__(16) elem_t v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int k = ch * 8 + j;
      const int r = tab[2 * k], off = tab[2 * k + 1];
      const int h = h0 + r, w = w0 + off / Cin;
      const bool in = r >= 0 && h >= 0 && h < H && w >= 0 && w < W;
      v[j] = in ? img[((long long)h * W + w0) * Cin + off] : f_to_e(0.f);
    }
    reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<const uint4*>(v);
  }
}
}  // namespace MSB_ELEM_NS
}  // namespace msb

MSB_EXPORT int MSB_FN(msb_im2col_nhwc)(const void* x, void* out, int N, int H, int W, int Cin, int R, int S, int stride,
                               int pad_h, int pad_w, int Ho, int Wo, int Kpad, void* stream) {
  if (Kpad < R * S * Cin || (Kpad % 8)) {
    set_last_error("im2col: padded width %d must be a multiple of 8 and at least %d", Kpad, R * S * Cin);
    return kBadArg;
  }
  const long long total = (long long)N * Ho * Wo * (Kpad / 8);
  if (total <= 0) return kOk;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  blocks = blocks > cap ? cap : blocks;
  im2col_nhwc_kernel<<<(unsigned)blocks, 256, Kpad * 4, (cudaStream_t)stream>>>(
      (const elem_t*)x, (elem_t*)out, N, H, W, Cin, R, S, stride, pad_h, pad_w, Ho, Wo, Kpad);
  MSB_CUDA_CHECK(cudaGetLastError());
  return kOk;
}
