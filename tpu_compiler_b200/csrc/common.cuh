// Shared device/host helpers for the B200 interpreter backend.
//
// The requantisation and rounding primitives restate, for the device, the
// reference's QuantizationArithmetic.cpp free functions
// (lib/Dialect/TPU/Quantization/QuantizationArithmetic.cpp):
//   qdm_requant      <- applyMultiplierAndRShiftAndSaturateInt8(.., qdm=true)  :518-539
//                       (SaturatingRoundingDoublingHighMul :501-509,
//                        RoundingDivideByPOT :487-499, saturateInt8 :301-334)
//   mul_rshift_sat8  <- the same function with qdm=false                      :526
//   rshift_sat8      <- applyRShiftAndSaturateInt8                            :481-483
//   f32_to_bf16_bits <- F32ToBF16                                             :873-910
//   f32_to_int8_rne  <- F32ToInt8(v, 0) / F32ToInt (round half to even on |v|) :918-947
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#define TPUCB_HD __host__ __device__ __forceinline__

namespace tpucb {

TPUCB_HD int clamp_i8(int q) { return q > 127 ? 127 : (q < -128 ? -128 : q); }

// gemmlowp-style rounding doubling high multiply followed by a rounding right
// shift and int8 saturation. v: int32 accumulator (bias already added),
// M: multiplier as int32, r: right shift in [0,31].
TPUCB_HD int qdm_requant(int32_t v, int32_t M, int r) {
  long long ab = (long long)v * (long long)M;
  long long x = ab + (ab >= 0 ? (1ll << 30) : (1ll - (1ll << 30)));
  // C++ division by 2^31 truncates toward zero.
  long long fl = x >> 31;
  if (x < 0 && (x & 0x7fffffffll) != 0) fl += 1;
  int32_t hi = (int32_t)fl;
  int32_t q;
  if (hi == 0 || r == 0) {
    q = hi;
  } else {
    int32_t mask = (int32_t)((1ll << r) - 1);
    int32_t rem = hi & mask;
    int32_t thr = (mask >> 1) + (hi < 0 ? 1 : 0);
    q = (hi >> r) + (rem > thr ? 1 : 0);
  }
  return clamp_i8(q);
}

// saturateInt8(floor(v * M / 2^r + 0.5)) for small integer v (|v*M| < 2^24 in the
// reference's float; here integer, exact for |v*M| < 2^31): (v*M + 2^(r-1)) >> r.
TPUCB_HD int mul_rshift_sat8(int32_t v, int32_t M, int r) {
  int32_t t = v * M;
  int32_t q = r == 0 ? t : ((t + (1 << (r - 1))) >> r);
  return clamp_i8(q);
}

TPUCB_HD int rshift_sat8(int32_t v, int r) {
  int32_t q = r == 0 ? v : ((v + (1 << (r - 1))) >> r);
  return clamp_i8(q);
}

TPUCB_HD uint32_t f32_bits(float f) {
#ifdef __CUDA_ARCH__
  return __float_as_uint(f);
#else
  union { float f; uint32_t u; } c;
  c.f = f;
  return c.u;
#endif
}
TPUCB_HD float bits_f32(uint32_t u) {
#ifdef __CUDA_ARCH__
  return __uint_as_float(u);
#else
  union { float f; uint32_t u; } c;
  c.u = u;
  return c.f;
#endif
}

// Round-to-nearest-even BF16 with the hardware quirk that any exponent-all-ones
// result (inf/NaN, either sign) becomes +max-finite 0x7f7f.
TPUCB_HD uint16_t f32_to_bf16_bits(float f, bool rounding = true) {
  uint32_t u = f32_bits(f);
  if (!rounding) return (uint16_t)(u >> 16);
  u += 0x7fffu + ((u >> 16) & 1u);
  uint16_t h = (uint16_t)(u >> 16);
  if ((h & 0x7f80) == 0x7f80) h = 0x7f7f;
  return h;
}
TPUCB_HD float bf16_bits_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }
TPUCB_HD float bf16_round(float f, bool rounding = true) {
  return bf16_bits_to_f32(f32_to_bf16_bits(f, rounding));
}

#ifdef __CUDACC__
// Programmatic dependent launch (kernels launched through launch_k with the stream-serialisation attribute): a kernel
// lets its successor in the stream be scheduled early (pdl_trigger) and waits for its predecessor's memory operations
// before its own first global access (pdl_wait). Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// first statement of every kernel that has no set-up worth overlapping
__device__ __forceinline__ void pdl_prologue() {
  pdl_trigger();
  pdl_wait();
}

// Two F32ToBF16 roundings in one conversion instruction: {bf16(hi), bf16(lo)} packed in a word.
// The hardware conversion equals the reference's add-and-shift rule whenever its result is
// finite; a result with an all-ones exponent (inf/NaN in, or rounding past max-finite) takes
// the exact bit rule instead, which also covers the NaN payloads that wrap in the reference.
__device__ __forceinline__ uint32_t bf16x2_round_bits(float lo, float hi) {
  uint32_t p;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(hi), "f"(lo));
  if (((p & 0x7f807f80u) + 0x00800080u) & 0x80008000u)
    p = (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
  return p;
}
// round(v) half-to-even as int32 (saturating at the int32 range, NaN -> 0): the integer that
// F32ToInt8(v, 0) saturates to int8 afterwards.
__device__ __forceinline__ int f32_to_i32_rne(float v) {
  int r;
  asm("cvt.rni.s32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return r;
}

// Per-channel constants of the short form of qdm_requant(acc + bias, M, r):
//   x  = acc * M + c64,  c64 = bias * M + 2^30 (one wide multiply-add)
//   hi = x >> 31 (floor; one funnel shift): adding 2^30 and flooring equals the reference's
//        sign-dependent nudge followed by a division that truncates toward zero, for either sign
//   q  = (hi + rnd - [hi < 0 and r > 0]) >> r,  rnd = 2^(r-1) (0 when r = 0): round half away
//        from zero, as RoundingDivideByPOT does
// With ReLU, negative results become 0 anyway: rnd moves into c64 and the sign term is dropped.
// The value returned is not yet saturated; pack4_sat does that.
struct QdmConst {
  int32_t M, r, rnd, s1; // s1 = 31 when r > 0, else 32: (uint)hi >> s1 is the sign term
  long long c64;
};
__device__ __forceinline__ QdmConst make_qdm_const(int32_t bias, int32_t M, int32_t r, bool relu) {
  QdmConst c;
  c.M = M;
  c.r = r;
  const long long rnd = r > 0 ? (1ll << (r - 1)) : 0ll;
  c.c64 = (long long)bias * (long long)M + (1ll << 30);
  if (relu) c.c64 += rnd << 31;
  c.rnd = (int32_t)rnd;
  c.s1 = r > 0 ? 31 : 32;
  return c;
}
template <bool RELU> __device__ __forceinline__ int qdm_fast(int32_t acc, const QdmConst &q) {
  long long x;
  asm("mad.wide.s32 %0, %1, %2, %3;" : "=l"(x) : "r"(acc), "r"(q.M), "l"(q.c64));
  const int32_t hi = (int32_t)__funnelshift_r((uint32_t)x, (uint32_t)(x >> 32), 31);
  if (RELU) return max(hi, 0) >> q.r;
  uint32_t adj;
  asm("shr.u32 %0, %1, %2;" : "=r"(adj) : "r"((uint32_t)hi), "r"((uint32_t)q.s1)); // shifts >= 32 give 0
  return (hi + q.rnd - (int)adj) >> q.r;
}
#endif

// F32ToInt8(v, 0): round half to even on the magnitude, then saturate.
__device__ __forceinline__ int f32_to_int8_rne(float v) {
  // rintf is round-half-even and symmetric in sign, identical to the reference's
  // modf-based rule for every finite v; clamp before the int conversion.
  float r = rintf(v);
  r = fminf(fmaxf(r, -128.0f), 127.0f);
  return (int)r;
}
// F32ToInt8(v, 1): C cast (truncate) then saturate.
__device__ __forceinline__ int f32_to_int8_rz(float v) {
  float r = truncf(v);
  r = fminf(fmaxf(r, -128.0f), 127.0f);
  return (int)r;
}

// d = {c[15:0], sat8(a), sat8(b)}: two int32 saturated to int8 and merged below the low half of c.
__device__ __forceinline__ uint32_t pack_sat_s8(int a, int b, uint32_t c) {
  uint32_t d;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// bytes (q0, q1, q2, q3) from low to high, each saturated to [-128, 127]
__device__ __forceinline__ uint32_t pack4_sat(int q0, int q1, int q2, int q3) {
  return pack_sat_s8(q1, q0, pack_sat_s8(q3, q2, 0u));
}
// sign-extended byte J of a word in one byte-permute: in prmt's default mode bit 3 of a selector
// nibble replicates the sign of the selected byte (the __byte_perm intrinsic masks that bit off,
// hence the inline PTX).
template <int J> __device__ __forceinline__ int sext_byte(uint32_t w) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(0u), "r"((uint32_t)(J | ((8 | J) << 4) | ((8 | J) << 8) | ((8 | J) << 12))));
  return (int)d;
}

} // namespace tpucb
