// HBM-bound kernels of the interpreter backend: layout conversion at the host
// boundary, quant/dequant, eltwise, pooling, depthwise convolution, patch
// expansion, concat / upsample / pixel-shuffle, activations and lookup tables.
//
// Device tensors are NHWC with the channel pitch `cp` padded to 16 bytes
// (int8 and bf16: 16 channels, fp32: 4); one thread handles one 16-byte vector
// so that a warp moves 512 contiguous bytes. Grids are sized by the callers as
// a multiple of the SM count with a grid-stride loop.
//
// Reference bodies restated here (lib/Dialect/TPU/Interpreter/core/):
//   quant.cpp:9-166, eltwise.cpp:52-85,335-357, pooling.cpp:33-160, conv.cpp (depthwise),
//   concat.cpp:34-90, upsample.cpp:20-41, depthtospace.cpp:6-48, activation.cpp:49-153,
//   lut_func.cpp:136-187,306-333.
#pragma once
#include "common.cuh"

namespace tpucb {

enum DType { DT_I8 = 0, DT_BF16 = 1, DT_F32 = 2 };

struct TensorGeom {
  int n, c, h, w, cp; // logical NCHW extents and the padded channel pitch (elements)
  int wl, wphys;      // physical row: wl zero pixels, w real pixels, zeros up to wphys
};

// ------------------------------------------------------------------ host boundary
// Host tensors are fp32 NCHW "containers" (include/tpuc/Interpreter/cpukernel.h:15-78).
// upload: staging fp32 NCHW -> device NHWC of dtype; padded lanes are written as zero.
template <int DT>
__global__ void nchw_f32_to_dev_kernel(const float *__restrict__ src, void *__restrict__ dst,
                                       TensorGeom g) {
  pdl_prologue();
  const size_t total = (size_t)g.n * g.h * g.wphys * g.cp;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    int c = (int)(i % g.cp);
    size_t pix = i / g.cp;
    int x = (int)(pix % g.wphys) - g.wl;
    size_t t = pix / g.wphys;
    int y = (int)(t % g.h);
    int b = (int)(t / g.h);
    float v = (c < g.c && x >= 0 && x < g.w) ? src[(((size_t)b * g.c + c) * g.h + y) * g.w + x] : 0.0f;
    if (DT == DT_I8) reinterpret_cast<int8_t *>(dst)[i] = (int8_t)(int)v;
    else if (DT == DT_BF16) reinterpret_cast<uint16_t *>(dst)[i] = (uint16_t)(f32_bits(v) >> 16);
    else reinterpret_cast<float *>(dst)[i] = v;
  }
}

// upload of an image-like fp32 tensor (at most 4 channels, channel pitch 4): one thread per pixel reads
// its values from the channel planes (consecutive threads, consecutive addresses) and writes one
// 16-byte NHWC4 word. This is the per-step input path of a serving loop.
__global__ void nchw_f32_to_nhwc4_kernel(const float *__restrict__ src, float4 *__restrict__ dst, int n, int c,
                                         size_t hw) {
  pdl_prologue();
  const size_t total = (size_t)n * hw;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t b = i / hw, p = i - b * hw;
    const float *s = src + b * c * hw + p;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    v.x = s[0];
    if (c > 1) v.y = s[hw];
    if (c > 2) v.z = s[2 * hw];
    if (c > 3) v.w = s[3 * hw];
    dst[i] = v;
  }
}

// upload of already quantised int8 values (NCHW order) into an INT8 tensor: the generic form (any channel pitch,
// padded rows) and the image form (at most 4 channels, one 32-bit word per pixel).
__global__ void nchw_i8_to_dev_kernel(const int8_t *__restrict__ src, int8_t *__restrict__ dst, TensorGeom g) {
  pdl_prologue();
  const size_t total = (size_t)g.n * g.h * g.wphys * g.cp;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % g.cp);
    const size_t pix = i / g.cp;
    const int x = (int)(pix % g.wphys) - g.wl;
    const size_t t = pix / g.wphys;
    const int y = (int)(t % g.h);
    const int b = (int)(t / g.h);
    dst[i] = (c < g.c && x >= 0 && x < g.w) ? src[(((size_t)b * g.c + c) * g.h + y) * g.w + x] : (int8_t)0;
  }
}
__global__ void nchw_i8_to_nhwc4_kernel(const int8_t *__restrict__ src, uint32_t *__restrict__ dst, int n, int c, size_t hw) {
  pdl_prologue();
  const size_t total = (size_t)n * hw;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t b = i / hw, p = i - b * hw;
    const uint8_t *s = reinterpret_cast<const uint8_t *>(src) + b * c * hw + p;
    uint32_t v = s[0];
    if (c > 1) v |= (uint32_t)s[hw] << 8;
    if (c > 2) v |= (uint32_t)s[2 * hw] << 16;
    if (c > 3) v |= (uint32_t)s[3 * hw] << 24;
    dst[i] = v;
  }
}

// download: device NHWC -> fp32 NCHW. One thread per NCHW element; reads of a warp
// stride by cp but stay inside L2-resident rows for the sizes that are fetched.
template <int DT>
__global__ void dev_to_nchw_f32_kernel(const void *__restrict__ src, float *__restrict__ dst,
                                       TensorGeom g) {
  pdl_prologue();
  const size_t total = (size_t)g.n * g.c * g.h * g.w;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    int x = (int)(i % g.w);
    size_t t = i / g.w;
    int y = (int)(t % g.h);
    t /= g.h;
    int c = (int)(t % g.c);
    int b = (int)(t / g.c);
    size_t s = (((size_t)b * g.h + y) * g.wphys + g.wl + x) * g.cp + c;
    float v;
    if (DT == DT_I8) v = (float)reinterpret_cast<const int8_t *>(src)[s];
    else if (DT == DT_BF16) v = bits_f32((uint32_t)reinterpret_cast<const uint16_t *>(src)[s] << 16);
    else v = reinterpret_cast<const float *>(src)[s];
    dst[i] = v;
  }
}

// ------------------------------------------------------------------------- quant
// kind: 0 fp32->int8 host rounding (std::round, half away from zero)  quant.cpp:22-30
//       1 fp32->int8 TPU mode                                         quant.cpp:11-20
//       2 int8->fp32   3 int8->bf16                                   quant.cpp:78-85,97-104
//       4 bf16->int8                                                  quant.cpp:87-94
//       5 fp32->bf16 (truncate)                                       quant.cpp:41-52
// Source and destination may have different channel pitches (cps / cpd).
__device__ __forceinline__ float load_as_f32(const void *p, int dt, size_t i) {
  if (dt == DT_I8) return (float)reinterpret_cast<const int8_t *>(p)[i];
  if (dt == DT_BF16) return bits_f32((uint32_t)reinterpret_cast<const uint16_t *>(p)[i] << 16);
  return reinterpret_cast<const float *>(p)[i];
}
__device__ __forceinline__ void store_from_f32(void *p, int dt, size_t i, float v) {
  if (dt == DT_I8) reinterpret_cast<int8_t *>(p)[i] = (int8_t)(int)v;
  else if (dt == DT_BF16) reinterpret_cast<uint16_t *>(p)[i] = (uint16_t)(f32_bits(v) >> 16);
  else reinterpret_cast<float *>(p)[i] = v;
}

// fp32 NHWC4 input image -> BF16 tensor with a 16-channel pitch (quant NONE -> BF16: the upper half of each fp32
// word, no rounding, QuantOpKernel's cast): one pixel per thread, one 16-byte read, two 16-byte writes.
__global__ void quant_f32c4_to_bf16c16_kernel(const float4 *__restrict__ in, uint4 *__restrict__ out, size_t pixels, int c) {
  pdl_prologue();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < pixels; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = __ldg(in + i);
    const uint32_t h0 = __float_as_uint(v.x) >> 16, h1 = c > 1 ? __float_as_uint(v.y) >> 16 : 0u;
    const uint32_t h2 = c > 2 ? __float_as_uint(v.z) >> 16 : 0u, h3 = c > 3 ? __float_as_uint(v.w) >> 16 : 0u;
    out[2 * i] = make_uint4(h0 | (h1 << 16), h2 | (h3 << 16), 0u, 0u);
    out[2 * i + 1] = make_uint4(0u, 0u, 0u, 0u);
  }
}

__global__ void quant_kernel(const void *__restrict__ src, void *__restrict__ dst, size_t rows, int w,
                             int wl, int wphys, int c, int cps, int cpd, int sdt, int ddt, int kind,
                             float scale) {
  pdl_prologue();
  const size_t total = rows * (size_t)wphys * (size_t)cpd;
  const float sb = bf16_round(scale);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    int ch = (int)(i % cpd);
    size_t ppix = i / cpd;
    int xx = (int)(ppix % wphys) - wl;
    size_t pix = (ppix / wphys) * w + xx;
    float out = 0.0f;
    if (ch < c && xx >= 0 && xx < w) {
      float x = load_as_f32(src, sdt, pix * cps + ch);
      switch (kind) {
      case 0: {
        float r = roundf(__fmul_rn(x, scale));
        out = fminf(fmaxf(r, -128.0f), 127.0f);
        break;
      }
      case 1:
        out = (float)f32_to_int8_rne(bf16_round(__fmul_rn(bf16_round(x, false), sb)));
        break;
      case 2:
      case 3:
        out = bf16_round(__fmul_rn(x, sb));
        break;
      case 4:
        out = (float)f32_to_int8_rne(bf16_round(__fmul_rn(x, sb)));
        break;
      default:
        out = bf16_round(x, false);
      }
    }
    store_from_f32(dst, ddt, i, out);
  }
}

// int8 -> bf16 (kind 3) over tensors with equal channel pitch and no row padding: 16 values per
// thread, one 16-byte load and two 16-byte stores. Padding lanes hold zero and stay zero.
__device__ __forceinline__ void dequant_word_bf16(uint32_t w, float sb, uint32_t &o0, uint32_t &o1) {
  o0 = bf16x2_round_bits(__fmul_rn((float)sext_byte<0>(w), sb), __fmul_rn((float)sext_byte<1>(w), sb));
  o1 = bf16x2_round_bits(__fmul_rn((float)sext_byte<2>(w), sb), __fmul_rn((float)sext_byte<3>(w), sb));
}
__global__ void quant_i8_to_bf16_vec_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst,
                                            size_t nvec, float scale) {
  pdl_prologue();
  const float sb = bf16_round(scale);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    uint32_t o[8];
    dequant_word_bf16(v.x, sb, o[0], o[1]);
    dequant_word_bf16(v.y, sb, o[2], o[3]);
    dequant_word_bf16(v.z, sb, o[4], o[5]);
    dequant_word_bf16(v.w, sb, o[6], o[7]);
    dst[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// bf16 -> int8 (kind 4), same layout conditions: two 16-byte loads, one 16-byte store.
__device__ __forceinline__ uint32_t quant_bf16x4_to_i8(uint32_t a, uint32_t b, float sb) {
  uint32_t p0 = bf16x2_round_bits(__fmul_rn(bits_f32(a << 16), sb), __fmul_rn(bits_f32(a & 0xffff0000u), sb));
  uint32_t p1 = bf16x2_round_bits(__fmul_rn(bits_f32(b << 16), sb), __fmul_rn(bits_f32(b & 0xffff0000u), sb));
  return pack4_sat(f32_to_i32_rne(bits_f32(p0 << 16)), f32_to_i32_rne(bits_f32(p0 & 0xffff0000u)),
                   f32_to_i32_rne(bits_f32(p1 << 16)), f32_to_i32_rne(bits_f32(p1 & 0xffff0000u)));
}
__global__ void quant_bf16_to_i8_vec_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst,
                                            size_t nvec, float scale) {
  pdl_prologue();
  const float sb = bf16_round(scale);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    const uint4 a = src[2 * i], b = src[2 * i + 1];
    dst[i] = make_uint4(quant_bf16x4_to_i8(a.x, a.y, sb), quant_bf16x4_to_i8(a.z, a.w, sb),
                        quant_bf16x4_to_i8(b.x, b.y, sb), quant_bf16x4_to_i8(b.z, b.w, sb));
  }
}

// fp32 -> int8 at the graph input (kind 0) from an NHWC4 fp32 tensor (c <= 4) into an int8
// tensor with channel pitch 4, 8 or 16 and optionally zero-padded rows: one thread per physical
// destination pixel, one 16-byte load and one 8/16-byte store.
__global__ void quant_input_pix_kernel(const float4 *__restrict__ src, void *__restrict__ dst, int n,
                                       int h, int w, int c, int cpd, int wl, int wphys, float scale) {
  pdl_prologue();
  const size_t total = (size_t)n * h * wphys;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    int x = (int)(i % wphys) - wl;
    size_t row = i / wphys;
    uint32_t lo = 0;
    if (x >= 0 && x < w) {
      float4 v = src[row * w + x];
      float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (k < c) {
          float r = fminf(fmaxf(roundf(__fmul_rn(f[k], scale)), -128.0f), 127.0f);
          lo |= ((uint32_t)((int)r & 0xff)) << (8 * k);
        }
      }
    }
    if (cpd == 4) reinterpret_cast<uint32_t *>(dst)[i] = lo;
    else if (cpd == 8) reinterpret_cast<uint2 *>(dst)[i] = make_uint2(lo, 0u);
    else reinterpret_cast<uint4 *>(dst)[i] = make_uint4(lo, 0u, 0u, 0u);
  }
}

// ----------------------------------------------------------------------- eltwise
// INT8 add: sum_i x_i * (int8)M_i, ReLU, (v + 2^(r-1)) >> r, saturate. eltwise.cpp:52-85.
struct EltwiseArgs {
  const int8_t *in[4];
  int mult[4];
  int nin;
  int rshift;
  int do_relu;
  int qdm_mult; // eltwise mul: QDM multiplier (0 with rshift 0 = no requant)
};

__device__ __forceinline__ int sx8(uint32_t w, int j) { return (int)(int8_t)(w >> (8 * j)); }

// acc += x_j * m for the 16 int8 lanes of one 16-byte vector
__device__ __forceinline__ void madd_vec16(int (&acc)[16], const uint4 &v, int m) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    acc[4 * q + 0] += sext_byte<0>(w[q]) * m;
    acc[4 * q + 1] += sext_byte<1>(w[q]) * m;
    acc[4 * q + 2] += sext_byte<2>(w[q]) * m;
    acc[4 * q + 3] += sext_byte<3>(w[q]) * m;
  }
}

// The rounding term 2^(r-1) is folded into the accumulator's start value: with ReLU,
// max(sum + rnd, 0) >> r equals (max(sum, 0) + rnd) >> r because rnd < 2^r.
template <int NIN, bool RELU>
__global__ void eltwise_add_i8_kernel(EltwiseArgs a, int8_t *__restrict__ out, size_t nvec) {
  pdl_prologue();
  const int rnd = a.rshift > 0 ? (1 << (a.rshift - 1)) : 0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += 2 * stride) {
    const size_t i2 = i + stride;
    const bool two = i2 < nvec;
    uint4 v[2][NIN];
#pragma unroll
    for (int k = 0; k < NIN; ++k) {
      v[0][k] = __ldcs(reinterpret_cast<const uint4 *>(a.in[k]) + i);
      if (two) v[1][k] = __ldcs(reinterpret_cast<const uint4 *>(a.in[k]) + i2);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u == 1 && !two) break;
      int acc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = rnd;
#pragma unroll
      for (int k = 0; k < NIN; ++k) madd_vec16(acc, v[u][k], a.mult[k]);
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        int r0 = acc[4 * q], r1 = acc[4 * q + 1], r2 = acc[4 * q + 2], r3 = acc[4 * q + 3];
        if (RELU) {
          r0 = max(r0, 0); r1 = max(r1, 0); r2 = max(r2, 0); r3 = max(r3, 0);
        }
        o[q] = pack4_sat(r0 >> a.rshift, r1 >> a.rshift, r2 >> a.rshift, r3 >> a.rshift);
      }
      __stcs(reinterpret_cast<uint4 *>(out) + (u == 0 ? i : i2), make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
}

// INT8 mul: product, ReLU, QDM requant with a scalar (M, r). eltwise.cpp:335-357.
__global__ void eltwise_mul_i8_kernel(EltwiseArgs a, int8_t *__restrict__ out, size_t nvec) {
  pdl_prologue();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    int acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 1;
    for (int k = 0; k < a.nin; ++k) {
      uint4 v = reinterpret_cast<const uint4 *>(a.in[k])[i];
      uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] *= sx8(w[j >> 2], j & 3);
    }
    uint32_t o[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      int v = acc[j];
      if (a.do_relu && v < 0) v = 0;
      int q = (a.rshift != 0 || a.qdm_mult != 0) ? qdm_requant(v, a.qdm_mult, a.rshift) : v;
      o[j >> 2] |= ((uint32_t)(q & 0xff)) << (8 * (j & 3));
    }
    reinterpret_cast<uint4 *>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// fp32 add with coefficients (eltwise.cpp:39-50); optional BF16 rounding of the result.
struct EltwiseF32Args {
  const float *in[4];
  float coeff[4];
  int nin;
  int do_relu;
  float *lo; // when set: also write x - (upper 19 bits of x), the remainder operand of a TF32 x 3 convolution that reads x
};
// One 16-byte vector per thread and step (fp32 tensors are a whole number of them: the channel pitch is a
// multiple of 4); operand by operand, product and sum rounded separately, as the reference's loop.
__global__ void eltwise_add_f32_kernel(EltwiseF32Args a, float *__restrict__ out, size_t n) {
  pdl_prologue();
  const size_t nvec = n / 4;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int k = 0; k < a.nin; ++k) {
      const float4 v = __ldg(reinterpret_cast<const float4 *>(a.in[k]) + i);
      const float c = a.coeff[k];
      acc.x = __fadd_rn(acc.x, __fmul_rn(c, v.x));
      acc.y = __fadd_rn(acc.y, __fmul_rn(c, v.y));
      acc.z = __fadd_rn(acc.z, __fmul_rn(c, v.z));
      acc.w = __fadd_rn(acc.w, __fmul_rn(c, v.w));
    }
    if (a.do_relu) {
      acc.x = acc.x < 0 ? 0.0f : acc.x;
      acc.y = acc.y < 0 ? 0.0f : acc.y;
      acc.z = acc.z < 0 ? 0.0f : acc.z;
      acc.w = acc.w < 0 ? 0.0f : acc.w;
    }
    reinterpret_cast<float4 *>(out)[i] = acc;
    if (a.lo) {
      float4 l;
      l.x = __fsub_rn(acc.x, __uint_as_float(__float_as_uint(acc.x) & 0xffffe000u));
      l.y = __fsub_rn(acc.y, __uint_as_float(__float_as_uint(acc.y) & 0xffffe000u));
      l.z = __fsub_rn(acc.z, __uint_as_float(__float_as_uint(acc.z) & 0xffffe000u));
      l.w = __fsub_rn(acc.w, __uint_as_float(__float_as_uint(acc.w) & 0xffffe000u));
      reinterpret_cast<float4 *>(a.lo)[i] = l;
    }
  }
}

// ----------------------------------------------------------------------- pooling
// One thread per (output pixel, 16-channel vector). method 0 max, 1 avg (window sum,
// then (sum*M + 2^(r-1)) >> r, saturate). pooling.cpp:65-82,146-155.
struct PoolArgs {
  int n, c, cp, ih, iw, oh, ow, kh, kw, sh, sw, pt, pl;
  int method, mult, rshift;
};
// Max pooling on packed bytes: four signed 8-bit maxima per instruction, no unpacking.
__global__ void pool_max_i8_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, PoolArgs a) {
  pdl_prologue();
  const int vecs = a.cp / 16;
  const size_t total = (size_t)a.n * a.oh * a.ow * vecs;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    int v = (int)(i % vecs);
    size_t pix = i / vecs;
    int x = (int)(pix % a.ow);
    size_t t = pix / a.ow;
    int y = (int)(t % a.oh);
    int b = (int)(t / a.oh);
    uint4 m = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
    const int y0 = max(y * a.sh - a.pt, 0), y1 = min(y * a.sh - a.pt + a.kh, a.ih);
    const int x0 = max(x * a.sw - a.pl, 0), x1 = min(x * a.sw - a.pl + a.kw, a.iw);
    for (int yy = y0; yy < y1; ++yy) {
      const uint4 *row = reinterpret_cast<const uint4 *>(in + (((size_t)b * a.ih + yy) * a.iw) * a.cp + v * 16);
      for (int xx = x0; xx < x1; ++xx) {
        const uint4 q = row[(size_t)xx * vecs];
        m.x = __vmaxs4(m.x, q.x);
        m.y = __vmaxs4(m.y, q.y);
        m.z = __vmaxs4(m.z, q.z);
        m.w = __vmaxs4(m.w, q.w);
      }
    }
    *reinterpret_cast<uint4 *>(out + pix * a.cp + v * 16) = m;
  }
}

__global__ void pool_i8_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, PoolArgs a) {
  pdl_prologue();
  const int vecs = a.cp / 16;
  const size_t total = (size_t)a.n * a.oh * a.ow * vecs;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    int v = (int)(i % vecs);
    size_t pix = i / vecs;
    int x = (int)(pix % a.ow);
    size_t t = pix / a.ow;
    int y = (int)(t % a.oh);
    int b = (int)(t / a.oh);
    int acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = a.method == 0 ? -128 : 0;
    for (int r = 0; r < a.kh; ++r) {
      int yy = y * a.sh - a.pt + r;
      if (yy < 0 || yy >= a.ih) continue;
      for (int s = 0; s < a.kw; ++s) {
        int xx = x * a.sw - a.pl + s;
        if (xx < 0 || xx >= a.iw) continue;
        uint4 q = *reinterpret_cast<const uint4 *>(in + (((size_t)b * a.ih + yy) * a.iw + xx) * a.cp + v * 16);
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          int e = sx8(w[j >> 2], j & 3);
          acc[j] = a.method == 0 ? max(acc[j], e) : acc[j] + e;
        }
      }
    }
    uint32_t o[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      int q = a.method == 0 ? acc[j] : mul_rshift_sat8(acc[j], a.mult, a.rshift);
      o[j >> 2] |= ((uint32_t)(q & 0xff)) << (8 * (j & 3));
    }
    *reinterpret_cast<uint4 *>(out + pix * a.cp + v * 16) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Average pooling over large windows (the global 7x7 pool before a classifier): eight lanes share
// one (output pixel, 16-channel vector), each sums every eighth tap, and three shuffle steps add
// the partial sums; a window is otherwise one long serial chain per thread.
__global__ void pool_avg_wide_i8_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, PoolArgs a) {
  pdl_prologue();
  const int vecs = a.cp / 16;
  const size_t items = (size_t)a.n * a.oh * a.ow * vecs;
  const int sub = threadIdx.x & 7;
  const int taps = a.kh * a.kw;
  for (size_t i = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 3; i < ((items + 3) & ~(size_t)3);
       i += ((size_t)gridDim.x * blockDim.x) >> 3) {
    const bool live = i < items; // a warp holds four items; dead ones still take part in the shuffles
    const size_t ii = live ? i : items - 1;
    int v = (int)(ii % vecs);
    size_t pix = ii / vecs;
    int x = (int)(pix % a.ow);
    size_t t = pix / a.ow;
    int y = (int)(t % a.oh);
    int b = (int)(t / a.oh);
    int acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0;
    for (int tap = sub; tap < taps; tap += 8) {
      const int yy = y * a.sh - a.pt + tap / a.kw, xx = x * a.sw - a.pl + tap % a.kw;
      if (yy < 0 || yy >= a.ih || xx < 0 || xx >= a.iw) continue;
      const uint4 q = *reinterpret_cast<const uint4 *>(in + (((size_t)b * a.ih + yy) * a.iw + xx) * a.cp + v * 16);
      madd_vec16(acc, q, 1);
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 1);
      acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 2);
      acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 4);
    }
    if (live && sub == 0) {
      const int rnd = a.rshift > 0 ? (1 << (a.rshift - 1)) : 0;
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        o[q] = pack4_sat((acc[4 * q] * a.mult + rnd) >> a.rshift, (acc[4 * q + 1] * a.mult + rnd) >> a.rshift,
                         (acc[4 * q + 2] * a.mult + rnd) >> a.rshift, (acc[4 * q + 3] * a.mult + rnd) >> a.rshift);
      *reinterpret_cast<uint4 *>(out + pix * a.cp + v * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ------------------------------------------------------------- depthwise 3x3 etc.
// Depthwise convolution (groups == channels), any kh/kw/stride/dilation, zero padding.
// Weights are packed tap-major [kh*kw][cp] so that a thread reads 16 consecutive
// channels per tap; the epilogue is the conv epilogue (bias + QDM + saturate + ReLU).
struct DwArgs {
  int n, c, cp, ih, iw, oh, ow, kh, kw, sh, sw, pt, pl, dh, dw, do_relu;
  const int8_t *wgt;  // [kh*kw][cp]
  const int32_t *bias, *mult, *rshift; // [cp]
};
__global__ void dwconv_i8_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, DwArgs a) {
  pdl_prologue();
  const int vecs = a.cp / 16;
  const size_t total = (size_t)a.n * a.oh * a.ow * vecs;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    int v = (int)(i % vecs);
    size_t pix = i / vecs;
    int x = (int)(pix % a.ow);
    size_t t = pix / a.ow;
    int y = (int)(t % a.oh);
    int b = (int)(t / a.oh);
    int acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0;
    for (int r = 0; r < a.kh; ++r) {
      int yy = y * a.sh - a.pt + r * a.dh;
      if (yy < 0 || yy >= a.ih) continue;
      for (int s = 0; s < a.kw; ++s) {
        int xx = x * a.sw - a.pl + s * a.dw;
        if (xx < 0 || xx >= a.iw) continue;
        uint4 q = *reinterpret_cast<const uint4 *>(in + (((size_t)b * a.ih + yy) * a.iw + xx) * a.cp + v * 16);
        uint4 f = *reinterpret_cast<const uint4 *>(a.wgt + (size_t)(r * a.kw + s) * a.cp + v * 16);
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t g[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] += sx8(w[j >> 2], j & 3) * sx8(g[j >> 2], j & 3);
      }
    }
    uint32_t o[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      int ch = v * 16 + j;
      int q = qdm_requant(acc[j] + a.bias[ch], a.mult[ch], a.rshift[ch]);
      if (a.do_relu && q < 0) q = 0;
      o[j >> 2] |= ((uint32_t)(q & 0xff)) << (8 * (j & 3));
    }
    *reinterpret_cast<uint4 *>(out + pix * a.cp + v * 16) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// 3x3 depthwise convolution, dilation 1, stride S in both directions: the layers of the
// MobileNet family. One thread owns one 4-channel word and TW consecutive output pixels of a row:
// the 36 unpacked weights stay in registers, every loaded input word is unpacked once and feeds
// up to three outputs, and the requantisation is the short per-channel form. The work is integer
// multiply-adds (9 per output value), so registers are blocked to keep the unpack and address
// instructions per value low; rows are re-read from L1/L2 by the threads of neighbouring rows.
template <int S, int TW, bool RELU>
__global__ void __launch_bounds__(128)
dwconv3x3_i8_kernel(const uint32_t *__restrict__ in, uint32_t *__restrict__ out, DwArgs a) {
  pdl_prologue();
  constexpr int WC = (TW - 1) * S + 3; // input columns under TW outputs
  const int cw = a.cp / 4;
  const int xg = (a.ow + TW - 1) / TW;
  const size_t total = (size_t)a.n * a.oh * xg * cw;
  const uint32_t *wgt = reinterpret_cast<const uint32_t *>(a.wgt);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int w4 = (int)(i % cw);
    size_t t = i / cw;
    const int gx = (int)(t % xg);
    t /= xg;
    const int y = (int)(t % a.oh);
    const int b = (int)(t / a.oh);
    int wk[9][4];
#pragma unroll
    for (int tap = 0; tap < 9; ++tap) {
      const uint32_t f = wgt[tap * cw + w4];
      wk[tap][0] = sext_byte<0>(f);
      wk[tap][1] = sext_byte<1>(f);
      wk[tap][2] = sext_byte<2>(f);
      wk[tap][3] = sext_byte<3>(f);
    }
    int acc[TW][4];
#pragma unroll
    for (int p = 0; p < TW; ++p)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[p][k] = 0;
    const int x0 = gx * TW * S - a.pl;
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int yy = y * S - a.pt + r;
      if (yy < 0 || yy >= a.ih) continue;
      const uint32_t *row = in + ((size_t)b * a.ih + yy) * a.iw * cw + w4;
#pragma unroll
      for (int col = 0; col < WC; ++col) {
        const int xx = x0 + col;
        const uint32_t v = (xx >= 0 && xx < a.iw) ? row[(size_t)xx * cw] : 0u;
        const int e[4] = {sext_byte<0>(v), sext_byte<1>(v), sext_byte<2>(v), sext_byte<3>(v)};
#pragma unroll
        for (int s = 0; s < 3; ++s) {
          if (col - s >= 0 && (col - s) % S == 0 && (col - s) / S < TW) {
            const int p = (col - s) / S;
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[p][k] += e[k] * wk[r * 3 + s][k];
          }
        }
      }
    }
    const int4 bi = reinterpret_cast<const int4 *>(a.bias)[w4];
    const int4 mu = reinterpret_cast<const int4 *>(a.mult)[w4];
    const int4 rs = reinterpret_cast<const int4 *>(a.rshift)[w4];
    const QdmConst q0 = make_qdm_const(bi.x, mu.x, rs.x, RELU), q1 = make_qdm_const(bi.y, mu.y, rs.y, RELU),
                   q2 = make_qdm_const(bi.z, mu.z, rs.z, RELU), q3 = make_qdm_const(bi.w, mu.w, rs.w, RELU);
    uint32_t *orow = out + (((size_t)b * a.oh + y) * a.ow) * cw + w4;
#pragma unroll
    for (int p = 0; p < TW; ++p) {
      const int x = gx * TW + p;
      if (x < a.ow)
        orow[(size_t)x * cw] = pack4_sat(qdm_fast<RELU>(acc[p][0], q0), qdm_fast<RELU>(acc[p][1], q1),
                                         qdm_fast<RELU>(acc[p][2], q2), qdm_fast<RELU>(acc[p][3], q3));
    }
  }
}

// The same layers with the multiply-adds as four-way dot products (dp4a). Every integer instruction costs a thread
// two issue cycles on this SM whatever it does, so the kernel above, at nine multiply-adds plus the byte unpacking per
// output value, is bound by instruction issue at a fraction of the HBM rate. Here a thread still owns one 4-channel
// word and TW = 8 / S outputs of a row, but it first turns each group of four input columns into four words that hold ONE
// channel's four columns each (a 4 x 4 byte transpose: 8 permutes per 16 values); an output's three taps of a filter
// row are then three neighbouring bytes of such a word (or of the funnel shift of two of them), and one dp4a against
// the row's packed weights (w0, w1, w2, 0) -- or (0, w0, w1, w2) for the window that starts one byte later -- adds all
// three. Per output value: 3 dp4a + 1.5 shifts + 2.25 permutes instead of 9 multiply-adds + 3.75 permutes, and the
// requantisation in the multiply-high form of the tensor-core epilogue (|acc + bias| < 2^29 always holds here).
// `wt`: the weights packed on the host as [cp / 4][3 rows][4 channels] words (w0 | w1 << 8 | w2 << 16).
template <int S, bool RELU>
__global__ void __launch_bounds__(128)
dwconv3x3_dp4a_kernel(const uint32_t *__restrict__ in, uint32_t *__restrict__ out, const uint32_t *__restrict__ wt, DwArgs a) {
  pdl_prologue();
  constexpr int TW = 8 / S;             // outputs per thread: 8 (stride 1) or 4 (stride 2)
  const int cw = a.cp / 4;
  const int xg = (a.ow + TW - 1) / TW;
  const size_t total = (size_t)a.n * a.oh * xg * cw;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int w4 = (int)(i % cw);
    size_t t = i / cw;
    const int gx = (int)(t % xg);
    t /= xg;
    const int y = (int)(t % a.oh);
    const int b = (int)(t / a.oh);
    int acc[TW][4];
#pragma unroll
    for (int p = 0; p < TW; ++p)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[p][k] = 0;
    const int x0 = gx * 8 - a.pl; // first input column under this thread's outputs (TW * S = 8 in both cases)
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int yy = y * S - a.pt + r;
      if (yy < 0 || yy >= a.ih) continue;
      const uint32_t *row = in + ((size_t)b * a.ih + yy) * a.iw * cw + w4;
      const uint4 wr = __ldg(reinterpret_cast<const uint4 *>(wt) + (size_t)w4 * 3 + r); // (w0, w1, w2, 0) per channel
      const uint32_t wa[4] = {wr.x, wr.y, wr.z, wr.w};
      // twelve columns, three groups of four, each transposed to one word per channel
      uint32_t tch[3][4];
#pragma unroll
      for (int g = 0; g < 3; ++g) {
        uint32_t v[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int xx = x0 + 4 * g + c;
          // columns 10 and 11 lie beyond the last window (stride 1: columns 0..9; stride 2: 0..8)
          v[c] = (4 * g + c < (S == 1 ? 10 : 9) && xx >= 0 && xx < a.iw) ? __ldg(row + (size_t)xx * cw) : 0u;
        }
        const uint32_t a01 = __byte_perm(v[0], v[1], 0x5140), b01 = __byte_perm(v[0], v[1], 0x7362);
        const uint32_t a23 = __byte_perm(v[2], v[3], 0x5140), b23 = __byte_perm(v[2], v[3], 0x7362);
        tch[g][0] = __byte_perm(a01, a23, 0x5410);
        tch[g][1] = __byte_perm(a01, a23, 0x7632);
        tch[g][2] = __byte_perm(b01, b23, 0x5410);
        tch[g][3] = __byte_perm(b01, b23, 0x7632);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int w0 = (int)wa[k], w1 = (int)(wa[k] << 8); // taps on bytes 0..2, or on bytes 1..3
        const uint32_t t0 = tch[0][k], t1 = tch[1][k], t2 = tch[2][k];
        if (S == 1) {
          acc[0][k] = __dp4a((int)t0, w0, acc[0][k]);                                 // columns 0..2
          acc[1][k] = __dp4a((int)t0, w1, acc[1][k]);                                 // 1..3
          acc[2][k] = __dp4a((int)__funnelshift_r(t0, t1, 16), w0, acc[2][k]);        // 2..4
          acc[3][k] = __dp4a((int)__funnelshift_r(t0, t1, 24), w0, acc[3][k]);        // 3..5
          acc[4][k] = __dp4a((int)t1, w0, acc[4][k]);                                 // 4..6
          acc[5][k] = __dp4a((int)t1, w1, acc[5][k]);                                 // 5..7
          acc[6][k] = __dp4a((int)__funnelshift_r(t1, t2, 16), w0, acc[6][k]);        // 6..8
          acc[7][k] = __dp4a((int)__funnelshift_r(t1, t2, 24), w0, acc[7][k]);        // 7..9
        } else {
          acc[0][k] = __dp4a((int)t0, w0, acc[0][k]);                                 // columns 0..2
          acc[1][k] = __dp4a((int)__funnelshift_r(t0, t1, 16), w0, acc[1][k]);        // 2..4
          acc[2][k] = __dp4a((int)t1, w0, acc[2][k]);                                 // 4..6
          acc[3][k] = __dp4a((int)__funnelshift_r(t1, t2, 16), w0, acc[3][k]);        // 6..8
        }
      }
    }
    // requantisation: the multiply-high form (see requant_fast in conv_gemm_i8.cuh), constants per channel
    const int4 bi = __ldg(reinterpret_cast<const int4 *>(a.bias) + w4);
    const int4 mu = __ldg(reinterpret_cast<const int4 *>(a.mult) + w4);
    const int4 rs = __ldg(reinterpret_cast<const int4 *>(a.rshift) + w4);
    const int bb[4] = {bi.x, bi.y, bi.z, bi.w}, mm[4] = {mu.x, mu.y, mu.z, mu.w}, rr[4] = {rs.x, rs.y, rs.z, rs.w};
    uint32_t sb[4], m2[4], kc[4];
    int r1[4], corr[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t rnd = rr[k] > 0 ? (1u << (rr[k] - 1)) : 0u;
      sb[k] = 2u * (uint32_t)bb[k] + 0x80000000u;
      m2[k] = (uint32_t)mm[k] << 1;
      corr[k] = (!RELU && rr[k] > 0) ? 2 : 0; // the sign term of RoundingDivideByPOT, see requant_fast
      kc[k] = 1u + 2u * rnd - (uint32_t)mm[k] - (uint32_t)corr[k];
      r1[k] = rr[k] + 1;
    }
    uint32_t *orow = out + (((size_t)b * a.oh + y) * a.ow) * cw + w4;
#pragma unroll
    for (int p = 0; p < TW; ++p) {
      int q[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t s2 = 2u * (uint32_t)acc[p][k] + sb[k];
        const int tk = (int)(__umulhi(s2, m2[k]) + kc[k]);
        q[k] = RELU ? (tk >> r1[k]) : ((tk + (((int)s2 >> 31) & corr[k])) >> r1[k]);
      }
      uint32_t w = pack4_sat(q[0], q[1], q[2], q[3]);
      if (RELU) w = __vmaxs4(w, 0u);
      const int x = gx * TW + p;
      if (x < a.ow) orow[(size_t)x * cw] = w;
    }
  }
}

// ---------------------------------------------------------------- patch expansion
// Writes the patch matrix A[M = n*oh*ow][kp] (kp = padded kh*kw*c, K order (r, s, c) over
// the REAL channels) for convolutions the im2col TMA path does not take: very few
// input channels (the 3-channel stems), input zero-insertion, grouped convolution.
struct PatchArgs {
  int n, c, cp, ih, iw, oh, ow, kh, kw, sh, sw, pt, pl, dh, dw, ins_h, ins_w;
  int c_first, c_count; // channel slice (grouped convolution)
  int kp;
  int wl, wphys;        // physical row layout of the input
  int cv = 0;           // 4: patch_expand_tap_kernel's layout, four channel slots per filter tap (k = tap * 4 + c)
};
__global__ void patch_expand_i8_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out,
                                       PatchArgs a) {
  pdl_prologue();
  const size_t total = (size_t)a.n * a.oh * a.ow * a.kp;
  const int ihd = (a.ih - 1) * (a.ins_h + 1) + 1, iwd = (a.iw - 1) * (a.ins_w + 1) + 1;
  const int kreal = a.kh * a.kw * a.c_count;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    int k = (int)(i % a.kp);
    size_t pix = i / a.kp;
    int8_t v = 0;
    if (k < kreal) {
      int c = k % a.c_count;
      int tap = k / a.c_count;
      int s = tap % a.kw, r = tap / a.kw;
      int x = (int)(pix % a.ow);
      size_t t = pix / a.ow;
      int y = (int)(t % a.oh);
      int b = (int)(t / a.oh);
      int yy = y * a.sh - a.pt + r * a.dh, xx = x * a.sw - a.pl + s * a.dw;
      if (yy >= 0 && yy < ihd && xx >= 0 && xx < iwd && (yy % (a.ins_h + 1)) == 0 &&
          (xx % (a.ins_w + 1)) == 0) {
        v = in[(((size_t)b * a.ih + yy / (a.ins_h + 1)) * a.wphys + a.wl + xx / (a.ins_w + 1)) * a.cp + a.c_first + c];
      }
    }
    out[i] = v;
  }
}

// The same expansion for 2-byte (BF16) and 4-byte (fp32) elements, one thread per 16-byte vector of the patch
// matrix: few-channel BF16 / fp32 convolutions (3-channel stems) would otherwise run one 32-byte K step per filter
// tap; the expanded matrix [M][kp] is a plain K-major operand with a handful of 128-byte K blocks.
template <typename T>
__global__ void patch_expand_kernel(const T *__restrict__ in, T *__restrict__ out, PatchArgs a) {
  pdl_prologue();
  constexpr int V = 16 / (int)sizeof(T);
  const size_t total = (size_t)a.n * a.oh * a.ow * (a.kp / V);
  const int kreal = a.kh * a.kw * a.c_count;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int kv = (int)(i % (a.kp / V));
    const size_t pix = i / (a.kp / V);
    const int x = (int)(pix % a.ow);
    const size_t t = pix / a.ow;
    const int y = (int)(t % a.oh);
    const int b = (int)(t / a.oh);
    T v[V];
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const int k = kv * V + j;
      v[j] = (T)0;
      if (k < kreal) {
        const int c = k % a.c_count, tap = k / a.c_count;
        const int s = tap % a.kw, r = tap / a.kw;
        const int yy = y * a.sh - a.pt + r * a.dh, xx = x * a.sw - a.pl + s * a.dw;
        if (yy >= 0 && yy < a.ih && xx >= 0 && xx < a.iw)
          v[j] = in[(((size_t)b * a.ih + yy) * a.wphys + a.wl + xx) * a.cp + a.c_first + c];
      }
    }
    reinterpret_cast<uint4 *>(out)[i] = *reinterpret_cast<const uint4 *>(v);
  }
}

// At most 4 input channels (image stems): every filter tap keeps four channel slots in the patch matrix,
// k = tap * 4 + c, so a thread copies one tap of one output pixel as ONE vector (16 bytes of fp32, 8 bytes of BF16)
// without any per-element index arithmetic. With `lo` (fp32) the remainder part of the TF32 x 3 product,
// x - (upper 19 bits of x), is written beside it, which saves the separate split pass over the matrix.
template <typename T>
__global__ void patch_expand_tap_kernel(const T *__restrict__ in, T *__restrict__ out, T *__restrict__ lo, PatchArgs a) {
  pdl_prologue();
  const int taps = a.kh * a.kw;
  const int slots = a.kp / 4; // vectors per row, the last ones are padding
  const size_t total = (size_t)a.n * a.oh * a.ow * slots;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int tap = (int)(i % slots);
    const size_t pix = i / slots;
    const int x = (int)(pix % a.ow);
    const size_t t = pix / a.ow;
    const int y = (int)(t % a.oh);
    const int b = (int)(t / a.oh);
    T v[4] = {(T)0, (T)0, (T)0, (T)0};
    if (tap < taps) {
      const int s = tap % a.kw, r = tap / a.kw;
      const int yy = y * a.sh - a.pt + r * a.dh, xx = x * a.sw - a.pl + s * a.dw;
      if (yy >= 0 && yy < a.ih && xx >= 0 && xx < a.iw) {
        const T *src = in + (((size_t)b * a.ih + yy) * a.wphys + a.wl + xx) * a.cp;
        if (sizeof(T) == 4) *reinterpret_cast<uint4 *>(v) = __ldg(reinterpret_cast<const uint4 *>(src));
        else *reinterpret_cast<uint2 *>(v) = __ldg(reinterpret_cast<const uint2 *>(src));
      }
    }
    if (sizeof(T) == 4) {
      reinterpret_cast<uint4 *>(out)[i] = *reinterpret_cast<const uint4 *>(v);
      if (lo) {
        float l[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float f = reinterpret_cast<const float *>(v)[j];
          l[j] = __fsub_rn(f, __uint_as_float(__float_as_uint(f) & 0xffffe000u));
        }
        reinterpret_cast<uint4 *>(lo)[i] = *reinterpret_cast<const uint4 *>(l);
      }
    } else {
      reinterpret_cast<uint2 *>(out)[i] = *reinterpret_cast<const uint2 *>(v);
    }
  }
}

// ------------------------------------------------------------------ data movement
// Channel concat of one input into a slice of the output, with the optional non-QDM
// rescale and ReLU of concat.cpp:70-85. Byte granular so that unaligned slices
// (e.g. 255-channel heads) work; the 16-byte fast path is taken when everything aligns.
__global__ void concat_slice_i8_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out,
                                       size_t pixels, int c, int cps, int cpd, int c_off, int mult,
                                       int rshift, int requant, int do_relu) {
  pdl_prologue();
  const size_t total = pixels * (size_t)c;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    int ch = (int)(i % c);
    size_t pix = i / c;
    int v = in[pix * cps + ch];
    if (requant) v = mul_rshift_sat8(v, mult, rshift);
    if (do_relu && v < 0) v = 0;
    out[pix * cpd + c_off + ch] = (int8_t)v;
  }
}

// The same slice copy on 16-byte vectors, for channel counts, offsets and pitches that are all
// multiples of 16 (every concat of the detection backbones except the 255-channel heads).
__global__ void concat_slice_i8_vec_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out,
                                           size_t pixels, int cv, int cpsv, int cpdv, int offv, int mult,
                                           int rshift, int requant, int do_relu) {
  pdl_prologue();
  const size_t total = pixels * (size_t)cv;
  const int rnd = rshift > 0 ? (1 << (rshift - 1)) : 0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % cv);
    const size_t pix = i / cv;
    uint4 x = in[pix * cpsv + v];
    if (requant || do_relu) {
      uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        int e[4] = {sext_byte<0>(w[q]), sext_byte<1>(w[q]), sext_byte<2>(w[q]), sext_byte<3>(w[q])};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (requant) e[k] = (e[k] * mult + rnd) >> rshift; // saturated by the pack below
          if (do_relu) e[k] = max(e[k], 0);
        }
        w[q] = pack4_sat(e[0], e[1], e[2], e[3]);
      }
      x = make_uint4(w[0], w[1], w[2], w[3]);
    }
    out[pix * cpdv + offv + v] = x;
  }
}

// Generic element copy with an index map; element size es bytes (1, 2 or 4).
// mode 0: nearest upsample (upsample.cpp:20-41); mode 1/2: pixel shuffle CRD / DCR
// (depthtospace.cpp:6-48), expressed as a gather over the OUTPUT index.
struct MoveArgs {
  int n, ic, ih, iw, icp, oc, oh, ow, ocp, es, mode, r, scale_h, scale_w;
};
__global__ void move_kernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out, MoveArgs a) {
  pdl_prologue();
  const size_t total = (size_t)a.n * a.oh * a.ow * a.ocp;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    int c = (int)(i % a.ocp);
    size_t pix = i / a.ocp;
    int x = (int)(pix % a.ow);
    size_t t = pix / a.ow;
    int y = (int)(t % a.oh);
    int b = (int)(t / a.oh);
    bool valid = c < a.oc;
    int sc = c, sy = y, sx = x;
    if (a.mode == 0) {
      sy = y / a.scale_h;
      sx = x / a.scale_w;
    } else {
      int r = a.r;
      sy = y / r;
      sx = x / r;
      int dy = y % r, dx = x % r;
      sc = a.mode == 1 ? (c * r * r + dy * r + dx) : ((dy * r + dx) * a.oc + c);
    }
    size_t s = (((size_t)b * a.ih + sy) * a.iw + sx) * a.icp + sc;
    for (int e = 0; e < a.es; ++e) out[i * a.es + e] = valid ? in[s * a.es + e] : 0;
  }
}

// ------------------------------------------------------------------- activations
// INT8 leaky ReLU (activation.cpp:126-153) and plain ReLU (internal.cpp:13-18).
__global__ void leaky_relu_i8_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out,
                                     size_t nvec, int mp, int rp, int mn, int rn, int plain_relu) {
  pdl_prologue();
  // positive side without a multiplier is the identity: (x * 1 + 0) >> 0
  const int mpe = mp != 0 ? mp : 1, rpe = mp != 0 ? rp : 0;
  const int rndp = rpe > 0 ? (1 << (rpe - 1)) : 0, rndn = rn > 0 ? (1 << (rn - 1)) : 0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    uint4 v = reinterpret_cast<const uint4 *>(in)[i];
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (plain_relu) {
        w[q] = __vmaxs4(w[q], 0u);
      } else {
        int e[4] = {sext_byte<0>(w[q]), sext_byte<1>(w[q]), sext_byte<2>(w[q]), sext_byte<3>(w[q])};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int pos = (e[k] * mpe + rndp) >> rpe, neg = (e[k] * mn + rndn) >> rn;
          e[k] = e[k] > 0 ? pos : neg; // saturated by the pack
        }
        w[q] = pack4_sat(e[0], e[1], e[2], e[3]);
      }
    }
    reinterpret_cast<uint4 *>(out)[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// INT8 256-entry table (activation.cpp:49-53): out = table[(uint8)x]; table staged in smem.
__global__ void lut_i8_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, size_t nvec,
                              const int8_t *__restrict__ table) {
  pdl_prologue();
  __shared__ int8_t s_t[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) s_t[i] = table[i];
  __syncthreads();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    uint4 v = reinterpret_cast<const uint4 *>(in)[i];
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      uint32_t idx = (w[j >> 2] >> (8 * (j & 3))) & 0xff;
      o[j >> 2] |= ((uint32_t)(uint8_t)s_t[idx]) << (8 * (j & 3));
    }
    reinterpret_cast<uint4 *>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// BF16 slope-interpolated table (lut_func.cpp:169-186). Tables are 256 fp32 values holding
// bf16-representable numbers; `scale` is BF16(256 / (2 * range)). Multiply and add are kept
// separate (no FMA contraction), as the x86 reference computes them.
// one word (two bf16 values) through the slope table; s_t holds (base, slope) per segment
__device__ __forceinline__ uint32_t lut_slope_pair(uint32_t w, float scale, const float2 *s_t) {
  const uint32_t rp = bf16x2_round_bits(__fmul_rn(bits_f32(w << 16), scale),
                                        __fmul_rn(bits_f32(w & 0xffff0000u), scale));
  const float r0 = bits_f32(rp << 16), r1 = bits_f32(rp & 0xffff0000u);
  const int i0 = f32_to_int8_rz(r0), i1 = f32_to_int8_rz(r1);
  const uint32_t dp = bf16x2_round_bits(__fsub_rn(r0, (float)i0), __fsub_rn(r1, (float)i1));
  const float2 t0 = s_t[i0 & 0xff], t1 = s_t[i1 & 0xff];
  return bf16x2_round_bits(__fadd_rn(t0.x, __fmul_rn(bits_f32(dp << 16), t0.y)),
                           __fadd_rn(t1.x, __fmul_rn(bits_f32(dp & 0xffff0000u), t1.y)));
}
__global__ void lut_bf16_slope_kernel(const uint16_t *__restrict__ in, uint16_t *__restrict__ out,
                                      size_t n, const float *__restrict__ base,
                                      const float *__restrict__ slope, float scale) {
  pdl_prologue();
  __shared__ float2 s_t[256]; // (base, slope) of one segment side by side: one 8-byte lookup
  for (int i = threadIdx.x; i < 256; i += blockDim.x) s_t[i] = make_float2(base[i], slope[i]);
  __syncthreads();
  const size_t nvec = n / 8;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4 *>(in)[i];
    reinterpret_cast<uint4 *>(out)[i] = make_uint4(lut_slope_pair(v.x, scale, s_t), lut_slope_pair(v.y, scale, s_t),
                                                   lut_slope_pair(v.z, scale, s_t), lut_slope_pair(v.w, scale, s_t));
  }
}

// The chain the reference's mixed-precision graphs use around a BF16 activation,
//   quant INT8->BF16  ->  slope-table activation (BF16)  ->  quant BF16->INT8,
// in one pass: 16 values per thread, all three results are written (each stays a fetchable
// tensor) but nothing is read back: 6 bytes per value instead of 10 over three launches.
__global__ void act_chain_i8_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ deq, uint4 *__restrict__ act,
                                    uint4 *__restrict__ out, size_t nvec, float scale_in, float lut_scale,
                                    const float *__restrict__ base, const float *__restrict__ slope,
                                    float scale_out) {
  pdl_prologue();
  __shared__ float2 s_t[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) s_t[i] = make_float2(base[i], slope[i]);
  __syncthreads();
  const float sbi = bf16_round(scale_in), sbo = bf16_round(scale_out);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = in[i];
    uint32_t d[8], a[8];
    dequant_word_bf16(v.x, sbi, d[0], d[1]);
    dequant_word_bf16(v.y, sbi, d[2], d[3]);
    dequant_word_bf16(v.z, sbi, d[4], d[5]);
    dequant_word_bf16(v.w, sbi, d[6], d[7]);
    deq[2 * i] = make_uint4(d[0], d[1], d[2], d[3]);
    deq[2 * i + 1] = make_uint4(d[4], d[5], d[6], d[7]);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = lut_slope_pair(d[j], lut_scale, s_t);
    act[2 * i] = make_uint4(a[0], a[1], a[2], a[3]);
    act[2 * i + 1] = make_uint4(a[4], a[5], a[6], a[7]);
    out[i] = make_uint4(quant_bf16x4_to_i8(a[0], a[1], sbo), quant_bf16x4_to_i8(a[2], a[3], sbo),
                        quant_bf16x4_to_i8(a[4], a[5], sbo), quant_bf16x4_to_i8(a[6], a[7], sbo));
  }
}

// BF16 exponent x mantissa table (lut_func.cpp:306-333, "mantissa" method; reciprocal is the
// pow table with coefficient -1). floor(log2|x|) is the unbiased exponent field for normal x.
__global__ void lut_bf16_mantissa_kernel(const uint16_t *__restrict__ in, uint16_t *__restrict__ out,
                                         size_t n, const float *__restrict__ exp_table,
                                         const float *__restrict__ mant_table) {
  pdl_prologue();
  __shared__ float s_e[256], s_m[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) {
    s_e[i] = exp_table[i];
    s_m[i] = mant_table[i];
  }
  __syncthreads();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    uint32_t h = in[i];
    float x = bits_f32(h << 16);
    int e;
    if (x == 0.0f) e = 0;
    else {
      int ex = (int)((h >> 7) & 0xff) - 127; // floor(log2 |x|) for normal bf16 values
      e = ex + 63 + ((h & 0x8000u) ? 128 : 0);
      e = min(max(e, 0), 255);
    }
    float y = bf16_round(__fmul_rn(s_e[e], s_m[h & 0xff]));
    out[i] = (uint16_t)(f32_bits(y) >> 16);
  }
}

} // namespace tpucb
