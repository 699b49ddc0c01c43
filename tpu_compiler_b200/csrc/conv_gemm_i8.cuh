// INT8 implicit-GEMM convolution / fully-connected kernel for sm_100a.
//
// Replaces, for INT8 graphs, the reference's Conv2DOpKernel::invoke
// (lib/Dialect/TPU/Interpreter/core/conv.cpp:80-104: fp32 MKL-DNN convolution on
// integer-valued floats followed by quantizeActivationInt8PerChannelMultiplierAndRShift,
// lib/Dialect/TPU/Quantization/QuantizationArithmetic.cpp:849-871) and
// FullyConnectedOpKernel::invoke (core/fullyconnected.cpp:44-91).
//
// The product is computed transposed, D[128 output channels][128 output pixels]: the weight
// tile ([Cout][tap][Cin] int8, 3-D tiled TMA load) is the tensor core's A operand and the
// activation tile its B operand, fetched either by an im2col-mode TMA load (any kh/kw/
// stride/dilation/padding; out-of-image taps arrive as zeros) or by a plain 2-D tiled TMA
// load (1x1 stride-1 convolutions, fully-connected, pre-expanded patch matrices). Tiles land
// in shared memory in the 32/64/128-byte swizzled K-major layout the tensor core reads and
// accumulate in int32 in tensor memory (tcgen05.mma kind::i8). With channels on the TMEM
// lanes every epilogue thread owns ONE output channel, so its bias / multiplier / rshift
// constants sit in registers instead of being re-read per value; the epilogue requantises,
// saturates, applies ReLU, transposes 4 channels x 4 pixels between neighbouring lanes with
// byte permutes and two shuffles, and stores 4 channels of one pixel per lane (a warp
// writes whole 32-byte sectors of the NHWC output).
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA
// issuer, warps 2..9 = epilogue (two warps per TMEM lane quarter, alternating
// 32-column groups).
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
  int BN;         // channel tile = tensor-core M, always 128 (rows past n_valid are zero-filled)
  int n_valid;    // number of valid (padded) output channels
  int ldc;        // output row pitch in bytes
  int c_off;      // first output channel written inside a row
  int stages;     // pipeline depth
  int dual;       // 1: at most 64 channels: two 128-pixel sub-tiles share the 128 TMEM lanes (see kernel)
  int w_resident; // 1: the CTA keeps all K blocks of its channel tile's weights in shared memory
  int a_mode;     // 0: A is a 2-D [M][K] matrix, 1: im2col TMA, 2: row windows (stem)
  int win_g;      // mode 2: output pixels per copy
  int act;        // 0 none, 1 ReLU, 2 leaky (non-QDM pos/neg rescale of the int8 result),
                  // 3 the eltwise add that consumes this convolution, with the residual tensor `res` (see add_*)
  int tmem_cols;  // 256: two accumulator buffers of 128 pixel columns
  int leaky_mp, leaky_rp, leaky_mn, leaky_rn;
  uint32_t idesc; // tcgen05 instruction descriptor
  const int32_t *bias;   // [n_valid]
  const int32_t *mult;   // [n_valid]
  const int32_t *rshift; // [n_valid]
  int8_t *out;
  int fastq;      // bit 0: the multiply-high form of the requantisation applies (requant_fast; set by the host);
                  // bit 1: every rshift of the layer is >= 1
  int8_t *out2;   // act == 2 / 3: the activation (or sum) goes here and `out` keeps the plain convolution result
  // act == 3 (EltwiseAddOpKernel::i8_invoke, core/eltwise.cpp:52-85, applied to this convolution's int8 result x and the
  // tensor `res` of the same geometry): sat8(relu?((x * add_ms + res * add_mr + 2^(add_r - 1)) >> add_r))
  const int8_t *res;
  int add_ms, add_mr, add_r, add_relu;
  int *err;       // device error word (0 = ok)
  // Self-test of the bounded waits (interpreter option "selftest_lost_arrival"): wait_rounds > 0 shortens every wait of
  // this launch to that many rounds of 1024 polls, and with lose_arrival the epilogue warps never hand an accumulator
  // buffer back, so that the MMA issuer's wait for it runs out and the launch ends through its error path (status
  // kErrAccWait) with no copy in flight. 0 / 0 in every ordinary launch.
  int wait_rounds, lose_arrival;
  // Split K (launches with fewer tiles than CTA slots and a long K, e.g. every layer of the last two stages at batch
  // 1): split_k > 1 CTAs share a tile, each takes k_per K blocks, adds its int32 partial accumulator to `ws`
  // ([tile][pixel column][channel lane], zero between launches) with red.global.add and counts itself in `ws_count`;
  // the CTA whose count completes the tile (no CTA waits for another) reads the sums back, runs the ordinary epilogue
  // on them and leaves `ws` and the counter zero again. Plain tiles only (not dual, INT8).
  int split_k, k_per;
  int32_t *ws;
  unsigned int *ws_count;
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
// The same with a suspend-time hint (nanoseconds): the thread may sleep in the instruction until the phase completes
// or that much time has passed, instead of coming back after the (short) default limit; a waiting role then spends
// few issue slots on its polling loop.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false when the barrier did not flip within the limit.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile int *abort_flag, int rounds = 1024) {
  // `rounds` (1024 by default) rounds of 1024 polls of at most a microsecond each (about a second in all): the abort
  // flag (another role of this CTA gave up) is read once per round
  for (int round = 0; round < rounds; ++round) {
#pragma unroll 1
    for (int it = 1024; it > 0; --it)
      if (mbar_try_wait_hint(bar, parity, 1000u)) return true;
    if (*abort_flag) return false;
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
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void *tmap, uint32_t bar, int x,
                                            int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
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
// The same MMA with the descriptors given as 32-bit halves (only the low words change between
// K steps and stages) and, when ACCUMULATE, a constant-true accumulate predicate: the issuing
// thread's loop carries no 64-bit arithmetic.
template <bool ACCUMULATE>
__device__ __forceinline__ void tcgen05_mma_i8_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                    uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  if (ACCUMULATE) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// kind::f16 with BF16 operands and fp32 accumulation (BF16 graphs): 16 elements = 32 bytes of K per MMA
template <bool ACCUMULATE>
__device__ __forceinline__ void tcgen05_mma_f16_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                     uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  if (ACCUMULATE) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// kind::tf32 with fp32 words as operands (their low 13 mantissa bits do not take part) and fp32 accumulation:
// 8 elements = 32 bytes of K per MMA
template <bool ACCUMULATE>
__device__ __forceinline__ void tcgen05_mma_tf32_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                      uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  if (ACCUMULATE) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// KSTEPS MMAs of one K block (32 bytes of K each: +2 in the descriptors' 16-byte address units).
// KIND: 0 kind::i8, 1 kind::f16 on BF16 operands, 2 kind::tf32
template <int KSTEPS, int KIND = 0>
__device__ __forceinline__ void tcgen05_mma_i8_kblock(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                                      uint32_t idesc, uint32_t accumulate_first) {
  if (KIND == 2) tcgen05_mma_tf32_lohi<false>(d_tmem, a_lo, hi, b_lo, hi, idesc, accumulate_first);
  else if (KIND == 1) tcgen05_mma_f16_lohi<false>(d_tmem, a_lo, hi, b_lo, hi, idesc, accumulate_first);
  else tcgen05_mma_i8_lohi<false>(d_tmem, a_lo, hi, b_lo, hi, idesc, accumulate_first);
#pragma unroll
  for (int k = 1; k < KSTEPS; ++k) {
    if (KIND == 2) tcgen05_mma_tf32_lohi<true>(d_tmem, a_lo + 2 * k, hi, b_lo + 2 * k, hi, idesc, 1u);
    else if (KIND == 1) tcgen05_mma_f16_lohi<true>(d_tmem, a_lo + 2 * k, hi, b_lo + 2 * k, hi, idesc, 1u);
    else tcgen05_mma_i8_lohi<true>(d_tmem, a_lo + 2 * k, hi, b_lo + 2 * k, hi, idesc, 1u);
  }
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

constexpr int kEpilogueWarps = 8;
constexpr int kConvThreads = 64 + 32 * kEpilogueWarps;
constexpr int kMaxStages = 8;
constexpr int kMaxBN = 256;
constexpr int kSmemHeader = 8192; // barriers + staged per-channel parameters

enum ConvErr { kErrFullWait = 1, kErrEmptyWait = 2, kErrAccWait = 3 };

// Per-channel requantisation constants, held in registers by the thread that owns the channel.
// The reference computes, for s = acc + bias and multiplier M in [0, 2^31),
//   hi = SaturatingRoundingDoublingHighMul(s, M) = floor((s * M + 2^30) / 2^31)
//        (adding 2^30 and flooring equals its sign-dependent nudge followed by a division that
//        truncates toward zero, for either sign),
//   q  = RoundingDivideByPOT(hi, r) = (hi + rnd - [hi < 0 and r > 0]) >> r, rnd = 2^(r-1) (0 if r = 0),
// then saturates (and ReLU clamps at 0, so there rnd is folded into the constant and the sign term
// dropped). requant_one forms the product once, unsigned and doubled, so that hi is simply the HIGH
// WORD of one 32 x 32 + 64 multiply-add:
//   s' = s + 2^31 (offset binary, one add of `sbias` = bias + 2^31), M2 = 2 * M (fits unsigned 32),
//   2 * (s * M + C) = s' * M2 + (2 * C - 2^31 * M2)   (mod 2^64),  C = 2^30 (+ rnd * 2^31 with ReLU),
//   hi = that >> 32.
struct ChanConst {
  uint32_t M2, sbias;
  int32_t r, rnd, s1; // s1 = 31 when r > 0, 32 when r == 0: (uint)hi >> s1 is the "negative and r > 0" bit
  unsigned long long c2;
  uint32_t kc;        // multiply-high form only (requant_fast), where r holds r + 1
  int32_t r0mask;     // multiply-high form: -1 when r == 0 (no sign term for this channel), else 0
};

__device__ __forceinline__ ChanConst load_chan_const(const ConvGemmParams &p, int n) {
  ChanConst c;
  const bool v = n < p.n_valid;
  const int32_t M = v ? p.mult[n] : 0;
  const int32_t b = v ? p.bias[n] : 0;
  c.r = v ? p.rshift[n] : 0;
  const unsigned long long rnd = c.r > 0 ? (1ull << (c.r - 1)) : 0ull;
  unsigned long long C = 1ull << 30;
  if (p.act == 1) C += rnd << 31;
  c.M2 = (uint32_t)M << 1;
  c.c2 = 2ull * C - ((unsigned long long)c.M2 << 31);
  c.sbias = (uint32_t)b + 0x80000000u;
  c.rnd = (int32_t)rnd;
  c.s1 = c.r > 0 ? 31 : 32;
  c.kc = 0;
  c.r0mask = c.r == 0 ? -1 : 0;
  if (p.fastq & 1) {
    // multiply-high form: see requant_fast
    const uint32_t k = 1u + 2u * (uint32_t)rnd;
    c.sbias = 2u * (uint32_t)b + 0x80000000u;
    // the sign term costs 2 when s < 0: the constant carries the -2 and the kernel gives it back when s >= 0
    c.kc = p.act == 1 ? k - (uint32_t)M : k - (uint32_t)M - (c.r > 0 ? 2u : 0u);
    c.r = c.r + 1;
    if (!v) { // a lane past the layer's channels: s2 = 0, no sign term, result 0
      c.sbias = 0u;
      c.kc = 0u;
    }
  }
  return c;
}

// One requantised value BEFORE the final int8 saturation (pack4_sat applies it).
template <int ACT>
__device__ __forceinline__ int requant_one(int32_t acc, const ChanConst &q, const ConvGemmParams &p) {
  unsigned long long x;
  asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(x) : "r"((uint32_t)acc + q.sbias), "r"(q.M2), "l"(q.c2));
  const int32_t hi = (int32_t)(uint32_t)(x >> 32);
  if (ACT == 1) {
    return max(hi, 0) >> q.r; // rnd already folded into c2; the upper clamp happens in the pack
  }
  uint32_t adj;
  asm("shr.u32 %0, %1, %2;" : "=r"(adj) : "r"((uint32_t)hi), "r"((uint32_t)q.s1)); // shifts >= 32 give 0
  int v = (hi + q.rnd - (int)adj) >> q.r;
  if (ACT == 2) v = min(max(v, -128), 127); // the leaky rescale below works on the saturated int8 value
  return v;
}
// The same value from ONE multiply-high. With t = floor(s * M / 2^30), hi = floor((t + 1) / 2) and, nesting the
// floors, q = floor((t + k - 2 * neg) / 2^(r + 1)), k = 1 + 2 * rnd, neg = [hi < 0 and r > 0].
//   Offset binary: s2 = 2 * (s + 2^30) is a non-negative 32-bit number whose top bit says s >= 0, and
//   mulhi(s2, 2M) = t + M exactly, so the addend kc = k - M gives t + k.
//   ReLU (ACT 1): no sign term. For s >= 0 the value is (t + k) >> (r + 1); for s < 0 it is <= 0 ((t + k) < 2^(r + 1)
//         there), which the caller clamps to 0 on the packed bytes (relu4): no clamp per value.
//   else: neg may be replaced by [s < 0 and r > 0]: the two differ only for t = -1 (hi = 0), where both forms
//         give 0. With m = s2 >> 31 (arithmetic: -1 for s >= 0, 0 for s < 0) the term is -2 - 2m; the -2 sits in kc.
//         R1 = every channel of the layer has r > 0; otherwise the channels with r = 0 switch the term off (r0mask).
// Valid for |s| < 2^29 and r <= 29 (no 32-bit overflow); the host sets fastq only when every channel of the
// layer and the largest possible |acc| satisfy that, else requant_one runs.
template <int ACT, bool R1>
__device__ __forceinline__ int requant_fast(int32_t acc, const ChanConst &q, const ConvGemmParams &p) {
  // The instructions are spelled out. Measured rates on this SM, lanes per clock: add / min / max 127; shifts, logic,
  // permutes, saturating packs and 32-bit multiply-adds 64, the last on a pipe of their own; multiply-high and
  // shuffles 32; the 64-bit multiply-add 16. The doubling and the sign term are multiply-adds, which run beside the
  // two shifts on the ALU: 122 -> 112 us on a 64 -> 256 channel 1x1 layer at batch 256; written as adds instead,
  // both 123 us, the doubling alone 111, the sign term alone 114.
  uint32_t s2, tk;
  asm("mad.lo.u32 %0, %1, 2, %2;" : "=r"(s2) : "r"((uint32_t)acc), "r"(q.sbias));
  asm("mad.hi.u32 %0, %1, %2, %3;" : "=r"(tk) : "r"(s2), "r"(q.M2), "r"(q.kc));
  int32_t v;
  if (ACT == 1) {
    asm("shr.s32 %0, %1, %2;" : "=r"(v) : "r"((int32_t)tk), "r"((uint32_t)q.r));
    return v;
  }
  int32_t m, x;
  asm("shr.s32 %0, %1, 31;" : "=r"(m) : "r"((int32_t)s2));
  if (!R1) m &= ~q.r0mask; // r == 0: kc carries no -2 and nothing is given back
  asm("mad.lo.s32 %0, %1, -2, %2;" : "=r"(x) : "r"(m), "r"((int32_t)tk));
  asm("shr.s32 %0, %1, %2;" : "=r"(v) : "r"(x), "r"((uint32_t)q.r));
  if (ACT == 2) v = min(max(v, -128), 127);
  return v;
}
// byte j of a and byte j of b in the two low bytes of a word (the upper bytes are multiplied by zero afterwards)
template <int J> __device__ __forceinline__ uint32_t byte_pair(uint32_t a, uint32_t b) {
  return __byte_perm(a, b, (uint32_t)(J | ((4 + J) << 4) | (J << 8) | (J << 12)));
}
// The INT8 eltwise add of four packed convolution results x with four packed residual values y:
// (x * ms + y * mr + rnd) >> r per byte through one four-way dot product each; the saturating pack (and the ReLU on
// the packed bytes) follow in the caller. mm = (ms, mr, 0, 0) as bytes.
__device__ __forceinline__ uint32_t add4_packed(uint32_t x, uint32_t y, uint32_t mm, int rnd, int r, bool relu) {
  const int s0 = __dp4a((int)byte_pair<0>(x, y), (int)mm, rnd) >> r;
  const int s1 = __dp4a((int)byte_pair<1>(x, y), (int)mm, rnd) >> r;
  const int s2 = __dp4a((int)byte_pair<2>(x, y), (int)mm, rnd) >> r;
  const int s3 = __dp4a((int)byte_pair<3>(x, y), (int)mm, rnd) >> r;
  const uint32_t w = pack4_sat(s0, s1, s2, s3);
  return relu ? __vmaxs4(w, 0u) : w;
}
// ReLU of four packed int8 values
__device__ __forceinline__ uint32_t relu4(uint32_t w) { return __vmaxs4(w, 0u); }
// INT8 leaky ReLU of a saturated convolution result (core/activation.cpp:126-153).
__device__ __forceinline__ int leaky_of(int v, const ConvGemmParams &p) {
  if (v > 0) return p.leaky_mp != 0 ? mul_rshift_sat8(v, p.leaky_mp, p.leaky_rp) : v;
  return mul_rshift_sat8(v, p.leaky_mn, p.leaky_rn);
}

// Byte-permute selectors of the 4x4 transpose between the four lanes of a group (lane & 3): two exchange steps
// (lane ^ 1, then lane ^ 2); each lane sends its whole word and picks two of its own bytes and two of its
// partner's with one permute per step.
struct TransposeSel {
  uint32_t merge1, merge2;
};
__device__ __forceinline__ TransposeSel make_transpose_sel(int lane) {
  TransposeSel t;
  t.merge1 = (lane & 1) ? 0x3715u : 0x6240u;
  t.merge2 = (lane & 2) ? 0x3276u : 0x5410u;
  return t;
}
// In: lane i of a 4-lane group holds bytes (pixel 0..3) of channel i. Out: lane j holds bytes
// (channel 0..3) of pixel j.
__device__ __forceinline__ uint32_t transpose4x4(uint32_t w, const TransposeSel &t) {
  const uint32_t z = __byte_perm(w, __shfl_xor_sync(0xffffffffu, w, 1), t.merge1);
  return __byte_perm(z, __shfl_xor_sync(0xffffffffu, z, 2), t.merge2);
}

// Epilogue of one accumulator buffer for the 32 channels (TMEM lanes) of this warp.
//   lane_addr  TMEM address of the warp's lane quarter in the buffer
//   out4       output address of (pixel m0, this lane's 4-channel group)
//   ch4_ok     the 4-channel group lies inside the valid channels
//   ncols      pixel columns of the accumulator buffer (128; 256 for the two-SM tile)
template <int ACT, bool FAST, bool R1 = false, bool FROM_WS = false>
__device__ __forceinline__ void epilogue_channels_impl(const ConvGemmParams &p, uint32_t lane_addr, int8_t *out4,
                                                       bool ch4_ok, int m0, int half, int halves, int lane,
                                                       const ChanConst &cc, const TransposeSel &ts, int ncols,
                                                       int32_t *ws_lane = nullptr) {
  constexpr int QACT = ACT == 3 ? 0 : ACT; // the fused add works on the plain (no activation) int8 result
  auto rq = [&](uint32_t a) { return FAST ? requant_fast<QACT, R1>((int32_t)a, cc, p) : requant_one<QACT>((int32_t)a, cc, p); };
  const int pj = lane & 3;
  // (Software-pipelining these loads in 16-column pieces made the epilogue alone 14% faster and the whole
  // kernel 4% slower, so the two loads of a chunk are simply issued together.)
  for (int colg = half * 32; colg < ncols; colg += 32 * halves) {
    if (m0 + colg >= p.M_total) break;
    const bool whole = m0 + colg + 32 <= p.M_total; // whole chunk in range: one guard for the eight stores
    int8_t *o = out4 + (size_t)(colg + pj) * p.ldc;
    uint32_t y[8];
    if (ACT == 3) {
      // the residual words of the fused eltwise add sit where the results go (same geometry): fetched first, so
      // that their latency passes under the accumulator loads and the requantisation
      const int8_t *rp = p.res + (size_t)(o - p.out);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        y[k] = 0u;
        if (ch4_ok && (whole || m0 + colg + 4 * k + pj < p.M_total))
          y[k] = __ldg(reinterpret_cast<const uint32_t *>(rp + (size_t)(4 * k) * p.ldc));
      }
    }
    uint32_t acc0[16], acc1[16];
    if (FROM_WS) {
      // split K: the summed accumulators of all the tile's CTAs, [pixel column][128 channel lanes] in global memory;
      // read past L1 (other SMs wrote them) and left zero for the next launch
      int32_t *src = ws_lane + (size_t)colg * 128;
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        acc0[k] = (uint32_t)__ldcg(src + (size_t)k * 128);
        acc1[k] = (uint32_t)__ldcg(src + (size_t)(16 + k) * 128);
      }
#pragma unroll
      for (int k = 0; k < 32; ++k) __stcg(src + (size_t)k * 128, 0);
    } else {
      ptx::tcgen05_ld_x16(lane_addr + (uint32_t)colg, acc0);
      ptx::tcgen05_ld_x16(lane_addr + (uint32_t)colg + 16u, acc1);
      ptx::tcgen05_wait_ld();
    }
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      w[k] = pack4_sat(rq(acc0[4 * k + 0]), rq(acc0[4 * k + 1]), rq(acc0[4 * k + 2]), rq(acc0[4 * k + 3]));
      w[4 + k] = pack4_sat(rq(acc1[4 * k + 0]), rq(acc1[4 * k + 1]), rq(acc1[4 * k + 2]), rq(acc1[4 * k + 3]));
      if (FAST && ACT == 1) { // the multiply-high form leaves the ReLU clamp to the packed bytes
        w[k] = relu4(w[k]);
        w[4 + k] = relu4(w[4 + k]);
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) w[k] = transpose4x4(w[k], ts);
    if (ACT == 3) {
      // fused eltwise add: both tensors are written
      int8_t *sp = p.out2 + (size_t)(o - p.out);
      const uint32_t mm = (uint32_t)(uint8_t)p.add_ms | ((uint32_t)(uint8_t)p.add_mr << 8);
      const int rnd = p.add_r > 0 ? (1 << (p.add_r - 1)) : 0;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (ch4_ok && (whole || m0 + colg + 4 * k + pj < p.M_total)) {
          *reinterpret_cast<uint32_t *>(o + (size_t)(4 * k) * p.ldc) = w[k];
          *reinterpret_cast<uint32_t *>(sp + (size_t)(4 * k) * p.ldc) = add4_packed(w[k], y[k], mm, rnd, p.add_r, p.add_relu != 0);
        }
    } else if (ACT == 2) {
      // fused leaky ReLU: the activation works on the packed, saturated values after the transpose (four
      // channels of one pixel per word); the plain result goes to `out` when the graph keeps that tensor
      uint32_t l[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        l[k] = pack4_sat(leaky_of(sext_byte<0>(w[k]), p), leaky_of(sext_byte<1>(w[k]), p), leaky_of(sext_byte<2>(w[k]), p),
                         leaky_of(sext_byte<3>(w[k]), p));
      int8_t *o2 = (p.out2 ? p.out2 + (out4 - p.out) : out4) + (size_t)(colg + pj) * p.ldc;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (ch4_ok && (whole || m0 + colg + 4 * k + pj < p.M_total)) {
          if (p.out2) *reinterpret_cast<uint32_t *>(o + (size_t)(4 * k) * p.ldc) = w[k];
          *reinterpret_cast<uint32_t *>(o2 + (size_t)(4 * k) * p.ldc) = l[k];
        }
    } else if (whole) {
      if (ch4_ok) {
        // row addresses by one wide multiply-add each (the multiply-add pipe has room, the integer ALU has not)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          unsigned long long addr;
          asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(addr) : "r"((uint32_t)(4 * k)), "r"((uint32_t)p.ldc), "l"((unsigned long long)o));
          asm volatile("st.global.b32 [%0], %1;" ::"l"(addr), "r"(w[k]) : "memory");
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (ch4_ok && m0 + colg + 4 * k + pj < p.M_total) *reinterpret_cast<uint32_t *>(o + (size_t)(4 * k) * p.ldc) = w[k];
    }
  }
}

template <int ACT>
__device__ __forceinline__ void epilogue_channels(const ConvGemmParams &p, uint32_t lane_addr, int8_t *out4,
                                                  bool ch4_ok, int m0, int half, int halves, int lane,
                                                  const ChanConst &cc, const TransposeSel &ts, int ncols = 128) {
  if ((p.fastq & 3) == 3) epilogue_channels_impl<ACT, true, true>(p, lane_addr, out4, ch4_ok, m0, half, halves, lane, cc, ts, ncols);
  else if (p.fastq & 1) epilogue_channels_impl<ACT, true, false>(p, lane_addr, out4, ch4_ok, m0, half, halves, lane, cc, ts, ncols);
  else epilogue_channels_impl<ACT, false>(p, lane_addr, out4, ch4_ok, m0, half, halves, lane, cc, ts, ncols);
}

// Epilogue of a BF16 convolution (core/conv.cpp:90-98: fp32 result + fp32 bias, ReLU, BF16 rounding). The
// accumulators are fp32; a thread rounds two neighbouring pixels of its channel into one word, exchanges
// words with the lane of the neighbouring channel and stores two channels of one pixel (a warp writes
// 64 contiguous bytes per pixel). `out_pair` addresses (pixel m0, the even channel of this lane's pair);
// `pitch` is the output row pitch in bytes.
template <bool RELU>
__device__ __forceinline__ void epilogue_channels_bf16(const ConvGemmParams &p, uint32_t lane_addr, uint8_t *out_pair,
                                                       bool ch_ok, int m0, int half, int halves, int lane, float bias,
                                                       int ncols = 128) {
  const int odd = lane & 1;
  const size_t pitch = (size_t)p.ldc;
  for (int colg = half * 32; colg < ncols; colg += 32 * halves) {
    if (m0 + colg >= p.M_total) break;
    uint32_t acc0[16], acc1[16];
    ptx::tcgen05_ld_x16(lane_addr + (uint32_t)colg, acc0);
    ptx::tcgen05_ld_x16(lane_addr + (uint32_t)colg + 16u, acc1);
    ptx::tcgen05_wait_ld();
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint32_t b0 = j < 8 ? acc0[2 * j] : acc1[2 * j - 16], b1 = j < 8 ? acc0[2 * j + 1] : acc1[2 * j - 15];
      float v0 = __fadd_rn(bits_f32(b0), bias), v1 = __fadd_rn(bits_f32(b1), bias);
      if (RELU) {
        v0 = v0 > 0.0f ? v0 : 0.0f;
        v1 = v1 > 0.0f ? v1 : 0.0f;
      }
      const uint32_t w = bf16x2_round_bits(v0, v1); // low half: pixel 2j, high half: pixel 2j + 1
      const uint32_t o = __shfl_xor_sync(0xffffffffu, w, 1);
      // even lane: channels (c, c+1) of pixel 2j; odd lane: channels (c-1, c) of pixel 2j + 1
      const uint32_t y = odd ? __byte_perm(o, w, 0x7632) : __byte_perm(w, o, 0x5410);
      const int pix = colg + 2 * j + odd;
      if (ch_ok && m0 + pix < p.M_total) *reinterpret_cast<uint32_t *>(out_pair + (size_t)pix * pitch) = y;
    }
  }
}

// Epilogue of an fp32 convolution computed as three TF32 products (calibration forward; core/conv.cpp:80-89): fp32
// accumulator + fp32 bias, ReLU, stored as fp32. A lane owns a channel: for every pixel the warp writes 32 consecutive
// channels (128 contiguous bytes). `out_ch` addresses (pixel m0, this lane's channel); `pitch` is the row pitch in bytes.
template <bool RELU>
__device__ __forceinline__ void epilogue_channels_f32(const ConvGemmParams &p, uint32_t lane_addr, uint8_t *out_ch, bool ch_ok,
                                                      int m0, int half, int halves, float bias, int ncols = 128) {
  const size_t pitch = (size_t)p.ldc;
  uint8_t *lo_ch = p.out2 ? reinterpret_cast<uint8_t *>(p.out2) + (out_ch - reinterpret_cast<uint8_t *>(p.out)) : nullptr;
  for (int colg = half * 32; colg < ncols; colg += 32 * halves) {
    if (m0 + colg >= p.M_total) break;
    uint32_t acc0[16], acc1[16];
    ptx::tcgen05_ld_x16(lane_addr + (uint32_t)colg, acc0);
    ptx::tcgen05_ld_x16(lane_addr + (uint32_t)colg + 16u, acc1);
    ptx::tcgen05_wait_ld();
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float v = __fadd_rn(bits_f32(j < 16 ? acc0[j & 15] : acc1[j & 15]), bias);
      if (RELU) v = v > 0.0f ? v : 0.0f;
      if (ch_ok && m0 + colg + j < p.M_total) {
        *reinterpret_cast<float *>(out_ch + (size_t)(colg + j) * pitch) = v;
        // the remainder operand of a TF32 x 3 convolution that reads this result, when one does
        if (lo_ch) *reinterpret_cast<float *>(lo_ch + (size_t)(colg + j) * pitch) = __fsub_rn(v, __uint_as_float(__float_as_uint(v) & 0xffffe000u));
      }
    }
  }
}

// Persistent kernel: gridDim.x CTAs walk the tile list (tile = blockIdx.x + k * gridDim.x; n-tiles
// vary fastest so that CTAs working at the same time share activation tiles through L2). The
// producer runs ahead through the shared-memory ring across tile boundaries and the accumulator is
// double-buffered in TMEM, so the loads and MMAs of tile i+1 overlap the epilogue of tile i.
// TF32: an fp32 convolution as three kind::tf32 products accumulated in one pass over K: with x = xh + xl and
// w = wh + wl (h: the upper 19 bits of the fp32 word, l: the exact remainder), x w = xh wh + xl wh + xh wl up to
// 2^-22 relative. The K loop runs three times over the taps: term 0 reads (tmA2, tmB) = (xl, wh), term 1
// (tmA, tmB2) = (xh, wl), term 2 (tmA, tmB) = (xh, wh); the accumulator never leaves TMEM in between. The two small
// terms come first: the tensor core truncates every partial sum at the accumulator's own precision, so each MMA
// step costs up to an ulp of what has been accumulated so far, and only the steps of the last term see the
// full magnitude (measured: the error against a double-accumulated convolution drops by the expected factor 3).
template <bool BF16, bool FAST = true, bool TF32 = false, bool SPLIT = false, int ACTSEL = -1>
__device__ __forceinline__ void conv_gemm_body(const CUtensorMap &tmA, const CUtensorMap &tmB, const ConvGemmParams &p,
                                               const CUtensorMap &tmA2, const CUtensorMap &tmB2) {
  constexpr int KIND = TF32 ? 2 : (BF16 ? 1 : 0);
  constexpr int kTerms = TF32 ? 3 : 1;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw);

  // header layout
  const uint32_t bar_full = base;             // kMaxStages x 8 B
  const uint32_t bar_empty = base + 64;       // kMaxStages x 8 B
  const uint32_t bar_acc_full = base + 128;   // 2 x 8 B: accumulator buffer complete
  const uint32_t bar_acc_empty = base + 144;  // 2 x 8 B: accumulator buffer drained by the epilogue
  const uint32_t bar_w = base + 160;          // resident weights landed
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 168);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 172);
  volatile int *split_last = reinterpret_cast<volatile int *>(smem + 176); // split K: this CTA completes its tile

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = (p.n_valid + p.BN - 1) / p.BN;
  // Dual mode (<= 64 output channels): a tile covers 256 pixels. The weight tile is fetched as 192 rows
  // starting 64 rows BEFORE the first channel, i.e. [64 zero rows][64 weight rows][64 zero rows]; rows
  // 64..191 of it ([W; 0]) times the first 128 pixels fill TMEM lanes 0..63, rows 0..127 ([0; W]) times
  // the second 128 pixels accumulate into lanes 64..127, so all 128 lanes (and all epilogue warps) work.
  const int m_tile = p.dual ? 256 : 128;
  const int m_tiles = (p.M_total + m_tile - 1) / m_tile;
  int total_tiles = n_tiles * m_tiles; // set to 0 below when the launch is already marked as failed
  const uint32_t a_bytes = (uint32_t)m_tile * (uint32_t)p.BK;
  const uint32_t b_bytes = (uint32_t)(p.dual ? 192 : p.BN) * (uint32_t)p.BK;
  const int taps = p.kh * p.kw;
  const int k_iters = taps * p.c_chunks;
  // Weight-resident mode: [all K blocks of the weights][ring of activation tiles]; the launch grid is a
  // multiple of the channel-tile count, so a CTA's channel tile never changes. Otherwise the ring
  // holds (activation tile, weight tile) pairs.
  const uint32_t w_base = base + kSmemHeader;
  const uint32_t tiles = p.w_resident ? w_base + (uint32_t)k_iters * b_bytes : w_base;
  const uint32_t stage_bytes = p.w_resident ? a_bytes : a_bytes + b_bytes;
  const uint32_t acc_stride = (uint32_t)(p.tmem_cols >> 1); // columns per accumulator buffer
  // The tile walk (tile = blockIdx.x + k * gridDim.x, channel tiles fastest) as a running (pixel tile, channel tile)
  // pair: the per-tile code of every role carries no division.
  const int walk_m0 = (int)blockIdx.x / n_tiles, walk_n0 = (int)blockIdx.x % n_tiles;
  const int walk_dm = (int)gridDim.x / n_tiles, walk_dn = (int)gridDim.x % n_tiles;
  const int wait_rounds = p.wait_rounds > 0 ? p.wait_rounds : 1024;
  // split K: a work item is (tile, K range); item = tile * split_k + range, one loop over items in every role
  const int split_k = (!SPLIT || p.split_k < 1) ? 1 : p.split_k; // SPLIT is a compile-time switch: the ordinary kernels carry none of it

  // Programmatic dependent launch: the next kernel of the stream may start its own set-up as soon as every CTA
  // of this launch has got here; this kernel in turn sets up its barriers and tensor memory while the
  // previous one is still finishing and only then waits for that kernel's results (pdl_wait below).
  pdl_trigger();
  if (threadIdx.x == 0) {
    // A CTA of a launch in which an earlier CTA already gave up does no work at all, so that a broken launch ends
    // quickly instead of timing out once per tile. The flag is read first and stored last, so that the load's
    // latency passes behind the barrier set-up, and ahead of pdl_wait on purpose: a flag raised by the previous
    // kernel after this read only costs this CTA its own bounded wait, the host sees the error either way.
    const int gave_up = *reinterpret_cast<volatile int *>(p.err);
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_acc_full + 8 * b, 1);
      ptx::mbar_init(bar_acc_empty + 8 * b, kEpilogueWarps);
    }
    ptx::mbar_init(bar_w, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    *abort_flag = gave_up;
  }
  if (warp == 1) {
    ptx::tcgen05_alloc(ptx::smem_u32(tmem_slot), (uint32_t)p.tmem_cols);
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (*abort_flag != 0) total_tiles = 0;
  const int total_items = total_tiles * split_k;
  // What does not depend on the previous kernel is started before the wait for it: the tensor maps are fetched and a
  // CTA that keeps its weights resident starts their copies (weights are written at load time only).
  if (warp == 0 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    if (p.w_resident && (int)blockIdx.x < total_tiles) {
      const int n0w = ((int)blockIdx.x % n_tiles) * p.BN - (p.dual ? 64 : 0);
      ptx::mbar_expect_tx(bar_w, (uint32_t)k_iters * b_bytes);
      for (int kit = 0; kit < k_iters; ++kit)
        ptx::tma_load_3d(w_base + (uint32_t)kit * b_bytes, &tmB, bar_w, (kit % p.c_chunks) * p.BK, kit / p.c_chunks,
                         n0w);
    }
  }
  // From here on the kernel touches the activations: the previous kernel's writes must be complete and visible.
  pdl_wait();

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      int it = 0; // k-iterations issued so far, across tiles
      int ps = 0;        // ring stage of iteration `it`
      uint32_t pph = 0;  // its phase bit
      bool ok = true;
      int tm = walk_m0, tn = walk_n0; // (resident weights: their copies were started before the wait above)
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        int k_begin = 0, k_end = kTerms * k_iters;
        if (split_k > 1) { // few items per CTA: the divisions do not matter here
          const int tile = item / split_k;
          tm = tile / n_tiles;
          tn = tile - tm * n_tiles;
          k_begin = (item - tile * split_k) * p.k_per;
          k_end = min(k_iters, k_begin + p.k_per);
        }
        const int m0 = tm * m_tile;
        const int n0 = tn * p.BN - (p.dual ? 64 : 0);
        tm += walk_dm;
        tn += walk_dn;
        if (tn >= n_tiles) {
          tn -= n_tiles;
          ++tm;
        }
        int n_img = 0, h_base = 0, w_base = 0; // im2col: base coordinates of the tile's first pixel
        if (p.a_mode == 1) {
          const int q = m0 % p.OW;
          const int t = m0 / p.OW;
          const int pp = t % p.OH;
          n_img = t / p.OH;
          w_base = q * p.sw - p.pl;
          h_base = pp * p.sh - p.pt;
        }
        // mode 2: the (column, row, image) of the first pixel of each copy, computed once per tile
        int bx_q[16], bx_h[16], bx_n[16];
        const int n_boxes = p.a_mode == 2 ? 128 / p.win_g : 0;
        for (int i = 0; i < n_boxes; ++i) {
          const int m = m0 + i * p.win_g;
          const int t = m / p.OW;
          bx_q[i] = m - t * p.OW;
          bx_n[i] = t / p.OH;
          bx_h[i] = (t - bx_n[i] * p.OH) * p.sh - p.pt;
        }
        // running (tap row, tap column, channel chunk) and ring (stage, phase) counters: this loop
        // is a single thread's instruction stream, so it carries no divisions
        int tap = 0, tr = 0, ts = 0, chunk = 0, term = 0;
        if (k_begin > 0) {
          tap = k_begin / p.c_chunks;
          chunk = k_begin - tap * p.c_chunks;
          tr = tap / p.kw;
          ts = tap - tr * p.kw;
        }
        for (int kit = k_begin; kit < k_end; ++kit, ++it) {
          const CUtensorMap *mapA = (TF32 && term == 0) ? &tmA2 : &tmA;
          const CUtensorMap *mapB = (TF32 && term == 1) ? &tmB2 : &tmB;
          if (it >= p.stages) {
            if (!ptx::mbar_wait_bounded(bar_empty + 8 * ps, pph ^ 1u, abort_flag, wait_rounds)) {
              if (!*abort_flag) atomicExch(p.err, kErrEmptyWait);
              *abort_flag = 1;
              ok = false;
              break;
            }
          }
          const int c0 = chunk * p.BK;
          const uint32_t a_dst = tiles + (uint32_t)ps * stage_bytes;
          const uint32_t b_dst = a_dst + a_bytes;
          const uint32_t fb = bar_full + 8 * ps;
          ptx::mbar_expect_tx(fb, stage_bytes);
          if (p.a_mode == 1) {
            // one copy per tile, also in dual mode (the map's pixel count per copy is the tile's: every copy costs
            // its issuing thread about 430 cycles whatever its size)
            ptx::tma_load_im2col_4d(a_dst, mapA, fb, c0, w_base, h_base, n_img, (uint16_t)(ts * p.dw),
                                    (uint16_t)(tr * p.dh));
          } else if (p.a_mode == 2) {
            // `tap` is the filter row; each copy brings win_g consecutive output pixels' windows.
            for (int i = 0; i < n_boxes; ++i)
              ptx::tma_load_4d(a_dst + (uint32_t)(i * p.win_g * p.BK), &tmA, fb, 0, bx_q[i],
                               bx_h[i] + tap * p.dh, bx_n[i]);
          } else {
            ptx::tma_load_2d(a_dst, mapA, fb, c0, m0);
          }
          if (!p.w_resident) ptx::tma_load_3d(b_dst, mapB, fb, c0, tap, n0);
          if (++chunk == p.c_chunks) {
            chunk = 0;
            ++tap;
            if (++ts == p.kw) {
              ts = 0;
              ++tr;
            }
            if (TF32 && tap == taps) { // next term: the same taps over the other operand pair
              tap = 0;
              tr = 0;
              ts = 0;
              ++term;
            }
          }
          if (++ps == p.stages) {
            ps = 0;
            pph ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag) {
        if (p.w_resident && (int)blockIdx.x < total_tiles)
          for (uint32_t w = 0; w < (1u << 20); ++w)
            if (ptx::mbar_try_wait(bar_w, 0u)) break;
        // Drain: wait (bounded) until every copy this thread issued has landed, so that no bulk
        // copy is in flight when the CTA's shared memory is released.
        int first = it > p.stages ? it - p.stages : 0;
        for (int j = first; j < it; ++j) {
          const int s = j % p.stages;
          const uint32_t ph = (uint32_t)(j / p.stages) & 1u;
          for (uint32_t w = 0; w < (1u << 20); ++w)
            if (ptx::mbar_try_wait(bar_full + 8 * s, ph)) break;
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int it = 0, t = 0;
      int ms = 0;        // ring stage of iteration `it`
      uint32_t mph = 0;  // its phase bit
      bool ok = true;
      // Shared-memory descriptors differ between stages and K steps only in the start-address field of
      // their low word (16-byte units, no carry out of its 14 bits below 256 KB): the low words are
      // advanced by 32-bit adds and the issue loop stays short. A single thread feeds the tensor core,
      // and every instruction it spends per K block beyond the MMAs themselves shows up as idle tensor
      // cycles (measured: ~35 extra instructions per 4 MMAs cost a third of the MMA rate).
      const uint64_t desc_ring0 = make_kmajor_desc(tiles, p.BK);
      const uint32_t desc_hi = (uint32_t)(desc_ring0 >> 32);
      const uint32_t desc_ring_lo = (uint32_t)desc_ring0;
      const uint32_t desc_w_lo = (uint32_t)make_kmajor_desc(w_base, p.BK);
      const uint32_t stage_step = stage_bytes >> 4, a_step = a_bytes >> 4, w_step = b_bytes >> 4;
      const uint32_t sub_step = (128u * (uint32_t)p.BK) >> 4, dual_step = (64u * (uint32_t)p.BK) >> 4;
      uint32_t m_full = bar_full, m_empty = bar_empty, ring_lo = desc_ring_lo;
      const int ksteps = p.BK / 32;
      if (p.w_resident && (int)blockIdx.x < total_tiles) {
        if (!ptx::mbar_wait_bounded(bar_w, 0u, abort_flag, wait_rounds)) {
          if (!*abort_flag) atomicExch(p.err, kErrFullWait);
          *abort_flag = 1;
          ok = false;
        }
      }
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++t) {
        int k_begin = 0, k_end = kTerms * k_iters;
        if (split_k > 1) {
          k_begin = (item % split_k) * p.k_per;
          k_end = min(k_iters, k_begin + p.k_per);
        }
        const int buf = t & 1;
        if (t >= 2) {
          // the epilogue must have drained this accumulator buffer (its previous use)
          if (!ptx::mbar_wait_bounded(bar_acc_empty + 8 * buf, (uint32_t)(((t >> 1) - 1) & 1), abort_flag, wait_rounds)) {
            if (!*abort_flag) atomicExch(p.err, kErrAccWait);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after();
        }
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * acc_stride;
        uint32_t wres_lo = desc_w_lo; // weight-resident mode: descriptor (low word) of K block `kit`
        for (int kit = k_begin; kit < k_end; ++kit, ++it) {
          if (!ptx::mbar_try_wait(m_full, mph) && !ptx::mbar_wait_bounded(m_full, mph, abort_flag, wait_rounds)) {
            if (!*abort_flag) atomicExch(p.err, kErrFullWait);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after();
          // transposed product: weights are the A operand (M = channels), activations B (N = pixels)
          const uint32_t w_lo = p.w_resident ? wres_lo : ring_lo + a_step;
          const uint32_t acc_first = kit > k_begin ? 1u : 0u;
          if (!p.dual) {
            if (ksteps == 4) ptx::tcgen05_mma_i8_kblock<4, KIND>(d_tmem, w_lo, ring_lo, desc_hi, p.idesc, acc_first);
            else if (ksteps == 2) ptx::tcgen05_mma_i8_kblock<2, KIND>(d_tmem, w_lo, ring_lo, desc_hi, p.idesc, acc_first);
            else ptx::tcgen05_mma_i8_kblock<1, KIND>(d_tmem, w_lo, ring_lo, desc_hi, p.idesc, acc_first);
          } else {
            // dual mode: sub-tile 0 uses weight rows 64..191 ([W; 0]), sub-tile 1 rows 0..127 ([0; W])
            for (int sub = 0; sub < 2; ++sub) {
              const uint32_t a_lo = w_lo + (sub == 0 ? dual_step : 0u);
              const uint32_t b_lo = ring_lo + (uint32_t)sub * sub_step;
              const uint32_t first = (kit > k_begin || sub > 0) ? 1u : 0u;
              if (ksteps == 4) ptx::tcgen05_mma_i8_kblock<4, KIND>(d_tmem, a_lo, b_lo, desc_hi, p.idesc, first);
              else if (ksteps == 2) ptx::tcgen05_mma_i8_kblock<2, KIND>(d_tmem, a_lo, b_lo, desc_hi, p.idesc, first);
              else ptx::tcgen05_mma_i8_kblock<1, KIND>(d_tmem, a_lo, b_lo, desc_hi, p.idesc, first);
            }
          }
          ptx::tcgen05_commit(m_empty); // frees the stage when the MMAs retire
          wres_lo += w_step;
          m_full += 8;
          m_empty += 8;
          ring_lo += stage_step;
          if (++ms == p.stages) {
            ms = 0;
            mph ^= 1u;
            m_full = bar_full;
            m_empty = bar_empty;
            ring_lo = desc_ring_lo;
          }
        }
        if (ok) ptx::tcgen05_commit(bar_acc_full + 8 * buf);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;     // TMEM lanes (= channels of the tile) this warp may read
    const int half = (warp - 2) >> 2; // which alternate 32-pixel column groups it takes
    const TransposeSel ts = make_transpose_sel(lane);
    ChanConst cc = {};
    float bias_f = 0.0f;
    int staged_n0 = -1;
    int t = 0;
    bool ok = true;
    int tm = walk_m0, tn = walk_n0;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++t) {
      int tile = item;
      if (split_k > 1) {
        tile = item / split_k;
        tm = tile / n_tiles;
        tn = tile - tm * n_tiles;
      }
      // dual mode: lanes 0..63 are the channels of the first 128 pixels, lanes 64..127 of the second
      const int ch_base = p.dual ? (quarter & 1) * 32 : quarter * 32;
      const int m0 = tm * m_tile + (p.dual ? 128 * (quarter >> 1) : 0);
      const int n0 = tn * p.BN;
      tm += walk_dm;
      tn += walk_dn;
      if (tn >= n_tiles) {
        tn -= n_tiles;
        ++tm;
      }
      const int buf = t & 1;
      if (n0 != staged_n0) {
        if (BF16 || TF32) {
          const int ch = n0 + ch_base + lane;
          bias_f = ch < p.n_valid ? __int_as_float(p.bias[ch]) : 0.0f; // fp32 bias bits in the int32 array
        } else {
          cc = load_chan_const(p, n0 + ch_base + lane);
        }
        staged_n0 = n0;
      }
      ok = ptx::mbar_wait_bounded(bar_acc_full + 8 * buf, (uint32_t)((t >> 1) & 1), abort_flag, wait_rounds);
      if (!ok && !*abort_flag) {
        atomicExch(p.err, kErrAccWait);
        *abort_flag = 1;
      }
      // the wait result may differ between lanes only on the error path; make it uniform
      ok = __all_sync(0xffffffffu, ok);
      const bool split_item = SPLIT && split_k > 1;
      if (!ok && !split_item) break; // (a split item still passes its two barriers, see below)
      ptx::tcgen05_fence_after();
      const int ch4 = n0 + ch_base + (lane >> 2) * 4;
      int32_t *ws_lane = nullptr; // split K: this lane's channel column of the tile's partial-sum block
      if (split_item) {
        ws_lane = p.ws + (size_t)tile * (128 * 128) + quarter * 32 + lane;
        if (ok && n0 + ch_base < p.n_valid && m0 < p.M_total) {
          // this CTA's partial accumulator goes to the tile's block in global memory (one reduction per value,
          // 128 contiguous bytes per warp and column)
          const uint32_t lane_addr = tmem_base + (uint32_t)buf * acc_stride + ((uint32_t)(quarter * 32) << 16);
          for (int colg = half * 32; colg < 128; colg += 32 * (kEpilogueWarps / 4)) {
            if (m0 + colg >= p.M_total) break;
            uint32_t a0[16], a1[16];
            ptx::tcgen05_ld_x16(lane_addr + (uint32_t)colg, a0);
            ptx::tcgen05_ld_x16(lane_addr + (uint32_t)colg + 16u, a1);
            ptx::tcgen05_wait_ld();
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              atomicAdd(ws_lane + (size_t)(colg + k) * 128, (int)a0[k]);
              atomicAdd(ws_lane + (size_t)(colg + 16 + k) * 128, (int)a1[k]);
            }
          }
        }
        // the accumulator buffer is free again
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (ok && lane == 0 && !p.lose_arrival)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_acc_empty + 8 * buf) : "memory");
        // Count this CTA in once all of its epilogue warps have added their part; the CTA that completes the tile
        // goes on to the epilogue proper, the others are done with it (nobody waits for another CTA). The two
        // barriers are among the epilogue warps of this CTA only, and every one of them reaches both: a warp whose
        // wait ran out has raised the abort flag before the first, the leader turns that into "stop" for all (2),
        // so that no warp goes on to a barrier the others will not come to.
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpilogueWarps) : "memory");
        if (warp == 2 && lane == 0) {
          int verdict = 2;
          if (!*abort_flag) {
            const unsigned int before = atomicAdd(p.ws_count + tile, 1u);
            verdict = before == (unsigned int)(split_k - 1) ? 1 : 0;
            if (verdict) p.ws_count[tile] = 0u; // ready for the next launch
          }
          *split_last = verdict;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpilogueWarps) : "memory");
        const int verdict = *split_last;
        if (verdict == 2) {
          ok = false;
          break;
        }
        if (verdict == 0) continue;
        __threadfence();
      }
      if (n0 + ch_base < p.n_valid && m0 < p.M_total) { // warp-uniform: this lane quarter holds real outputs
        const uint32_t lane_addr = tmem_base + (uint32_t)buf * acc_stride + ((uint32_t)(quarter * 32) << 16);
        int8_t *out4 = p.out + (size_t)m0 * p.ldc + p.c_off + ch4;
        const bool ch4_ok = ch4 < p.n_valid;
        if (TF32) {
          // byte addressing: 4 bytes per channel
          const int ch = n0 + ch_base + lane;
          uint8_t *out_ch = reinterpret_cast<uint8_t *>(p.out) + (size_t)m0 * p.ldc + (size_t)(p.c_off + ch) * 4;
          if (p.act == 1) epilogue_channels_f32<true>(p, lane_addr, out_ch, ch < p.n_valid, m0, half, kEpilogueWarps / 4, bias_f);
          else epilogue_channels_f32<false>(p, lane_addr, out_ch, ch < p.n_valid, m0, half, kEpilogueWarps / 4, bias_f);
        } else if (BF16) {
          // byte addressing: 2 bytes per channel, this lane's pair starts at its even channel
          const int ch = n0 + ch_base + lane;
          uint8_t *out_pair = reinterpret_cast<uint8_t *>(p.out) + (size_t)m0 * p.ldc + (size_t)(p.c_off + (ch & ~1)) * 2;
          if (p.act == 1) epilogue_channels_bf16<true>(p, lane_addr, out_pair, ch < p.n_valid, m0, half, kEpilogueWarps / 4, lane, bias_f);
          else epilogue_channels_bf16<false>(p, lane_addr, out_pair, ch < p.n_valid, m0, half, kEpilogueWarps / 4, lane, bias_f);
        } else if (ACTSEL == 1) { // kernels specialised for one epilogue (ACTSEL: 1 = ReLU, 10 = none with every rshift >= 1)
          epilogue_channels_impl<1, FAST, false, SPLIT>(p, lane_addr, out4, ch4_ok, m0, half, kEpilogueWarps / 4, lane, cc, ts, 128, ws_lane);
        } else if (ACTSEL == 10) {
          epilogue_channels_impl<0, FAST, true, SPLIT>(p, lane_addr, out4, ch4_ok, m0, half, kEpilogueWarps / 4, lane, cc, ts, 128, ws_lane);
        } else if (p.act == 1) epilogue_channels_impl<1, FAST, false, SPLIT>(p, lane_addr, out4, ch4_ok, m0, half, kEpilogueWarps / 4, lane, cc, ts, 128, ws_lane);
        else if (p.act == 2) epilogue_channels_impl<2, FAST, false, SPLIT>(p, lane_addr, out4, ch4_ok, m0, half, kEpilogueWarps / 4, lane, cc, ts, 128, ws_lane);
        else if (p.act == 3 && FAST && (p.fastq & 2)) epilogue_channels_impl<3, FAST, true>(p, lane_addr, out4, ch4_ok, m0, half, kEpilogueWarps / 4, lane, cc, ts, 128);
        else if (p.act == 3) epilogue_channels_impl<3, FAST>(p, lane_addr, out4, ch4_ok, m0, half, kEpilogueWarps / 4, lane, cc, ts, 128);
        else if (FAST && (p.fastq & 2)) epilogue_channels_impl<0, FAST, true, SPLIT>(p, lane_addr, out4, ch4_ok, m0, half, kEpilogueWarps / 4, lane, cc, ts, 128, ws_lane);
        else epilogue_channels_impl<0, FAST, false, SPLIT>(p, lane_addr, out4, ch4_ok, m0, half, kEpilogueWarps / 4, lane, cc, ts, 128, ws_lane);
      }
      if (SPLIT && ws_lane) continue; // split K: the accumulator buffer was handed back above
      // hand the accumulator buffer back to the MMA issuer
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0 && !p.lose_arrival)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_acc_empty + 8 * buf) : "memory");
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tcgen05_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// p.fastq bit 0 must be set: the epilogue uses the multiply-high requantisation (requant_fast)
__global__ void __launch_bounds__(kConvThreads, 2)
conv_gemm_i8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const ConvGemmParams p) {
  conv_gemm_body<false, true>(tmA, tmB, p, tmA, tmB);
}
// The two epilogues that carry most launches as kernels of their own (ReLU; no activation with every rshift >= 1):
// the compiler allocates registers and schedules for that one epilogue instead of for all of them.
template <int ACTSEL>
__global__ void __launch_bounds__(kConvThreads, 2)
conv_gemm_i8_act_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const ConvGemmParams p) {
  conv_gemm_body<false, true, false, false, ACTSEL>(tmA, tmB, p, tmA, tmB);
}
// The split-K form of both (ConvGemmParams::split_k > 1): a kernel of its own, so that the ordinary ones carry none of
// its code (with the switch at run time the epilogue-bound layers were 14% slower).
template <bool FAST>
__global__ void __launch_bounds__(kConvThreads, 2)
conv_gemm_i8_split_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const ConvGemmParams p) {
  conv_gemm_body<false, FAST, false, true>(tmA, tmB, p, tmA, tmB);
}
// the same with the 64-bit multiply-add requantisation (requant_one), for layers outside requant_fast's domain
__global__ void __launch_bounds__(kConvThreads, 2)
conv_gemm_i8_wide_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const ConvGemmParams p) {
  conv_gemm_body<false, false>(tmA, tmB, p, tmA, tmB);
}
// The same pipeline for BF16 graphs: BF16 operands (tcgen05 kind::f16), fp32 accumulators, BF16 results.
// All sizes in ConvGemmParams that count K or row pitches are in BYTES, so only the MMA kind and the
// epilogue differ.
__global__ void __launch_bounds__(kConvThreads, 2)
conv_gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const ConvGemmParams p) {
  conv_gemm_body<true, false>(tmA, tmB, p, tmA, tmB);
}

// fp32 convolution on the tensor cores as three TF32 products (see conv_gemm_body): tmA / tmA2 are the upper and
// the remainder part of the activations, tmB / tmB2 of the weights.
__global__ void __launch_bounds__(kConvThreads, 2)
conv_gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                        const ConvGemmParams p) {
  conv_gemm_body<false, false, true>(tmA, tmB, p, tmA2, tmB2);
}

// x -> (upper part, remainder): hi keeps the sign, the exponent and the top 10 mantissa bits of the fp32 word (what
// a kind::tf32 product uses of it), lo = x - hi exactly. 16-byte vectors; `hi` may be null (the tensor core makes the
// same cut when it reads x itself).
__global__ void tf32_split_kernel(const float4 *__restrict__ x, float4 *__restrict__ hi, float4 *__restrict__ lo, size_t nvec) {
  pdl_prologue();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = x[i];
    float4 h, l;
    h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); l.x = __fsub_rn(v.x, h.x);
    h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); l.y = __fsub_rn(v.y, h.y);
    h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); l.z = __fsub_rn(v.z, h.z);
    h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); l.w = __fsub_rn(v.w, h.w);
    if (hi) hi[i] = h;
    lo[i] = l;
  }
}

} // namespace tpucb
