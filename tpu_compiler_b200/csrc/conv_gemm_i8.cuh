// INT8 implicit-GEMM convolution / fully-connected kernel for sm_100a.
//
// Replaces, for INT8 graphs, the reference's Conv2DOpKernel::invoke
// (lib/Dialect/TPU/Interpreter/core/conv.cpp:80-104: fp32 MKL-DNN convolution on
// integer-valued floats followed by quantizeActivationInt8PerChannelMultiplierAndRShift,
// lib/Dialect/TPU/Quantization/QuantizationArithmetic.cpp:849-871) and
// FullyConnectedOpKernel::invoke (core/fullyconnected.cpp:44-91).
//
// D[M=128 output pixels][N<=256 output channels] is accumulated in int32 in
// tensor memory by tcgen05.mma kind::i8; the A tile (activations, NHWC int8) is
// fetched either by an im2col-mode TMA load (any kh/kw/stride/dilation/padding;
// out-of-image taps arrive as zeros) or by a plain 2-D tiled TMA load (1x1
// stride-1 convolutions, fully-connected, pre-expanded patch matrices); the B
// tile (weights, [Cout][tap][Cin] int8) by a 3-D tiled TMA load. Tiles land in
// shared memory in the 32/64/128-byte swizzled K-major layout the tensor core
// reads. The epilogue adds the int32 bias, applies the per-channel
// multiplier/rshift requantisation, saturates, applies ReLU and stores int8 NHWC.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA
// issuer, warps 2..5 = epilogue (each reads the 32 TMEM lanes it may access).
// Every wait is bounded: on expiry the CTA records an error code in p.err and
// leaves through the common tear-down (TMEM freed, in-flight copies drained).
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace tpucb {

struct ConvGemmParams {
  int M_total;    // rows of the implicit GEMM: N*OH*OW (or m for fully-connected)
  int OH, OW;     // output spatial size (im2col mode)
  int sh, sw;     // stride
  int pt, pl;     // top / left padding
  int dh, dw;     // dilation
  int kh, kw;     // filter size (taps = kh*kw; 1 in tiled mode)
  int c_chunks;   // ceil(Cin_pad / BK)
  int BK;         // K bytes per pipeline stage: 32, 64 or 128 (= swizzle span)
  int BN;         // tile width in output channels, multiple of 16, <= 256
  int n_valid;    // number of valid (padded) output channels
  int ldc;        // output row pitch in bytes
  int c_off;      // first output channel written inside a row
  int stages;     // pipeline depth
  int a_im2col;   // 1: A through im2col TMA, 0: A is a 2-D [M][K] matrix
  int act;        // 0 none, 1 ReLU, 2 leaky (non-QDM pos/neg rescale of the int8 result)
  int tmem_cols;  // power of two >= max(32, BN)
  int leaky_mp, leaky_rp, leaky_mn, leaky_rn;
  uint32_t idesc; // tcgen05 instruction descriptor
  const int32_t *bias;   // [n_valid]
  const int32_t *mult;   // [n_valid]
  const int32_t *rshift; // [n_valid]
  int8_t *out;
  int *err;       // device error word (0 = ok)
};

namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false when the barrier did not flip within the limit.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile int *abort_flag) {
  for (uint32_t it = 0; it < (1u << 20); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, uint32_t bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void *tmap, uint32_t bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const void *tmap, uint32_t bar,
                                                   int c, int w, int h, int n, uint16_t off_w,
                                                   uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}
__device__ __forceinline__ void tcgen05_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tcgen05_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

} // namespace ptx

// Shared-memory matrix descriptor for a K-major tile whose rows are `BK` bytes
// long and swizzled over `BK` bytes (BK in {32,64,128}): 8-row groups are
// 8*BK bytes apart (stride byte offset); the leading byte offset is unused for
// swizzled K-major tiles; bits 46-47 carry the sm_100 descriptor version.
__device__ __forceinline__ uint64_t make_kmajor_desc(uint32_t smem_addr, int BK) {
  uint64_t layout = BK == 128 ? 2ull : (BK == 64 ? 4ull : 6ull);
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;                            // leading byte offset (ignored)
  d |= (uint64_t)(((uint32_t)(8 * BK)) >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;                            // descriptor version (Blackwell)
  d |= layout << 61;
  return d;
}

constexpr int kConvThreads = 192;
constexpr int kMaxStages = 8;
constexpr int kSmemHeader = 4096; // barriers + staged per-channel parameters

enum ConvErr { kErrFullWait = 1, kErrEmptyWait = 2, kErrAccWait = 3 };

__global__ void __launch_bounds__(kConvThreads, 1)
conv_gemm_i8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const ConvGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw);

  // header layout
  const uint32_t bar_full = base;            // kMaxStages x 8 B
  const uint32_t bar_empty = base + 64;      // kMaxStages x 8 B
  const uint32_t bar_acc = base + 128;       // 8 B
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 136);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 140);
  int32_t *s_bias = reinterpret_cast<int32_t *>(smem + 256);
  int32_t *s_mult = s_bias + 256;
  int32_t *s_rsh = s_mult + 256;
  const uint32_t tiles = base + kSmemHeader;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * 128;
  const int n0 = blockIdx.y * p.BN;
  const uint32_t a_bytes = 128u * (uint32_t)p.BK;
  const uint32_t b_bytes = (uint32_t)p.BN * (uint32_t)p.BK;
  const uint32_t stage_bytes = a_bytes + b_bytes;
  const int taps = p.kh * p.kw;
  const int k_iters = taps * p.c_chunks;

  // A CTA of a launch in which an earlier CTA already gave up does no work at all, so that a
  // broken launch ends quickly instead of timing out once per tile.
  if (threadIdx.x == 0) *abort_flag = *reinterpret_cast<volatile int *>(p.err);
  __syncthreads();
  if (*abort_flag != 0) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 1);
    }
    ptx::mbar_init(bar_acc, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    ptx::tcgen05_alloc(ptx::smem_u32(tmem_slot), (uint32_t)p.tmem_cols);
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      int n_img = 0, h_base = 0, w_base = 0;
      if (p.a_im2col) {
        int q = m0 % p.OW;
        int t = m0 / p.OW;
        int pp = t % p.OH;
        n_img = t / p.OH;
        w_base = q * p.sw - p.pl;
        h_base = pp * p.sh - p.pt;
      }
      int issued = 0;
      bool ok = true;
      for (int kit = 0; kit < k_iters && ok; ++kit) {
        const int s = kit % p.stages;
        const uint32_t ph = (uint32_t)(kit / p.stages) & 1u;
        if (kit >= p.stages) {
          if (!ptx::mbar_wait_bounded(bar_empty + 8 * s, ph ^ 1u, abort_flag)) {
            if (!*abort_flag) atomicExch(p.err, kErrEmptyWait);
            *abort_flag = 1;
            ok = false;
            break;
          }
        }
        const int tap = kit / p.c_chunks;
        const int c0 = (kit % p.c_chunks) * p.BK;
        const uint32_t a_dst = tiles + s * stage_bytes;
        const uint32_t b_dst = a_dst + a_bytes;
        const uint32_t fb = bar_full + 8 * s;
        ptx::mbar_expect_tx(fb, stage_bytes);
        if (p.a_im2col) {
          const int r = tap / p.kw, ss = tap % p.kw;
          ptx::tma_load_im2col_4d(a_dst, &tmA, fb, c0, w_base, h_base, n_img,
                                  (uint16_t)(ss * p.dw), (uint16_t)(r * p.dh));
        } else {
          ptx::tma_load_2d(a_dst, &tmA, fb, c0, m0);
        }
        ptx::tma_load_3d(b_dst, &tmB, fb, c0, tap, n0);
        ++issued;
      }
      if (!ok) {
        // Drain: wait (bounded) until every copy this thread issued has landed, so
        // no bulk copy is in flight when the CTA's shared memory is released.
        int first = issued > p.stages ? issued - p.stages : 0;
        for (int kit = first; kit < issued; ++kit) {
          const int s = kit % p.stages;
          const uint32_t ph = (uint32_t)(kit / p.stages) & 1u;
          for (uint32_t it = 0; it < (1u << 20); ++it)
            if (ptx::mbar_try_wait(bar_full + 8 * s, ph)) break;
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      bool ok = true;
      for (int kit = 0; kit < k_iters; ++kit) {
        const int s = kit % p.stages;
        const uint32_t ph = (uint32_t)(kit / p.stages) & 1u;
        if (!ptx::mbar_wait_bounded(bar_full + 8 * s, ph, abort_flag)) {
          if (!*abort_flag) atomicExch(p.err, kErrFullWait);
          *abort_flag = 1;
          ok = false;
          break;
        }
        ptx::tcgen05_fence_after();
        const uint32_t a_src = tiles + s * stage_bytes;
        const uint32_t b_src = a_src + a_bytes;
        const uint64_t adesc = make_kmajor_desc(a_src, p.BK);
        const uint64_t bdesc = make_kmajor_desc(b_src, p.BK);
        const int ksteps = p.BK / 32;
        for (int k = 0; k < ksteps; ++k) {
          // advance 32 bytes of K inside the swizzle span: +2 in 16-byte units
          ptx::tcgen05_mma_i8(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k),
                              p.idesc, (kit > 0 || k > 0) ? 1u : 0u);
        }
        ptx::tcgen05_commit(bar_empty + 8 * s); // frees the stage when the MMAs retire
      }
      if (ok) ptx::tcgen05_commit(bar_acc);
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int et = threadIdx.x - 64; // 0..127
    for (int i = et; i < p.BN; i += 128) {
      const int n = n0 + i;
      const bool v = n < p.n_valid;
      s_bias[i] = v ? p.bias[n] : 0;
      s_mult[i] = v ? p.mult[n] : 0;
      s_rsh[i] = v ? p.rshift[n] : 0;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    bool ok = ptx::mbar_wait_bounded(bar_acc, 0u, abort_flag);
    if (!ok && !*abort_flag) {
      atomicExch(p.err, kErrAccWait);
      *abort_flag = 1;
    }
    // the wait result may differ between lanes only on the error path; make it uniform
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      ptx::tcgen05_fence_after();
      const int quarter = warp & 3; // TMEM lanes this warp may read
      const int row = quarter * 32 + lane;
      const int m = m0 + row;
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
      int8_t *orow = p.out + (size_t)m * p.ldc + p.c_off + n0;
      for (int col = 0; col < p.BN; col += 16) {
        if (n0 + col >= p.n_valid) break;
        uint32_t acc[16];
        ptx::tcgen05_ld_x16(lane_addr + (uint32_t)col, acc);
        ptx::tcgen05_wait_ld();
        uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          int32_t v = (int32_t)acc[j] + s_bias[col + j];
          int q = qdm_requant(v, s_mult[col + j], s_rsh[col + j]);
          if (p.act == 1) {
            q = q < 0 ? 0 : q;
          } else if (p.act == 2) {
            if (q > 0) {
              if (p.leaky_mp != 0) q = mul_rshift_sat8(q, p.leaky_mp, p.leaky_rp);
            } else {
              q = mul_rshift_sat8(q, p.leaky_mn, p.leaky_rn);
            }
          }
          if ((j & 3) == 0) packed[j >> 2] = 0;
          packed[j >> 2] |= ((uint32_t)(q & 0xff)) << (8 * (j & 3));
        }
        if (m < p.M_total) {
          *reinterpret_cast<uint4 *>(orow + col) =
              make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tcgen05_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

} // namespace tpucb
