// CPU oracle: a plain restatement of the arithmetic of the tpu_compiler
// interpreter's op kernels (sophgo/tpu_compiler, lib/Dialect/TPU/Interpreter).
//
// TEST INFRASTRUCTURE ONLY. Nothing in the product path links, loads or calls
// this file; it exists so that the parity tests, the smoke check and the CPU
// baseline leg of the benchmark have something independent to compare the CUDA
// kernels with. Tensors follow the reference's container convention: every
// value (int8, bf16 or fp32) is held in a `float`, NCHW.
//
// Pinning: the scalar primitives below (QDM requant, non-QDM requant, BF16
// rounding, F32->int8, LUT slope/mantissa, KLD) are checked against the
// reference's own QuantizationArithmetic.cpp / lut_func.cpp /
// calibration_math.cpp compiled unmodified into oracle/_ref (see
// oracle/build_oracle.py) and against golden vectors generated from that
// build. The conv / inner-product / pooling contraction itself is performed by
// Intel MKL-DNN v1.0.2 in the reference (not vendored there): for that step the
// oracle uses an exact integer (INT8 mode) or double (FP32 mode) direct loop and
// parity is unpinned by any in-tree golden vector of the reference.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

extern "C" {

// ---------------------------------------------------------------------------
// Scalar primitives.
// ---------------------------------------------------------------------------

// saturateInt8: QuantizationArithmetic.cpp:301-334 (floor(f + 0.5), clamp).
static inline int sat8f(float f) {
  int q = (int)std::floor(f + 0.5);
  return q > 127 ? 127 : (q < -128 ? -128 : q);
}

// RoundingDivideByPOT: QuantizationArithmetic.cpp:487-499.
static inline int32_t rdiv_pot(int32_t x, int e) {
  if (x == 0) return 0;
  if (e == 0) return x;
  const int32_t mask = (int32_t)((1ll << e) - 1);
  const int32_t rem = x & mask;
  const int32_t thr = (mask >> 1) + (x < 0 ? 1 : 0);
  return (x >> e) + (rem > thr ? 1 : 0);
}

// SaturatingRoundingDoublingHighMul: QuantizationArithmetic.cpp:501-509.
static inline int32_t srdhm(int32_t a, int32_t b) {
  int64_t ab = (int64_t)a * (int64_t)b;
  int32_t nudge = ab >= 0 ? (1 << 30) : (1 - (1 << 30));
  return (int32_t)((ab + nudge) / (1ll << 31));
}

// applyMultiplierAndRShiftAndSaturateInt8(int32, ..., qdm=true):
// QuantizationArithmetic.cpp:529-539.
int orc_qdm_i32(int32_t v, uint32_t rshift, uint32_t multiplier) {
  int32_t q = rdiv_pot(srdhm(v, (int32_t)multiplier), (int)rshift);
  return sat8f((float)q);
}

// float overload, qdm=true: QuantizationArithmetic.cpp:518-527 ((int32_t)v cast).
int orc_qdm_f32(float v, uint32_t rshift, uint32_t multiplier) {
  return orc_qdm_i32((int32_t)v, rshift, multiplier);
}

// float overload, qdm=false: saturateInt8((v * multiplier) / (1 << rshift)),
// QuantizationArithmetic.cpp:526. `v * multiplier` is float * uint32 -> float.
int orc_mul_rshift_f32(float v, uint32_t rshift, uint32_t multiplier) {
  return sat8f((float)((v * multiplier) / (1 << rshift)));
}

// applyRShiftAndSaturateInt8: QuantizationArithmetic.cpp:481-483.
int orc_rshift_f32(float v, uint32_t rshift) { return sat8f(v / (1 << rshift)); }

// F32ToBF16: QuantizationArithmetic.cpp:873-910.
uint16_t orc_f32_to_bf16(float src, int rounding) {
  uint32_t u;
  std::memcpy(&u, &src, 4);
  uint16_t h;
  if (rounding) {
    uint32_t lsb = (u >> 16) & 1;
    u += 0x7fff + lsb;
    h = (uint16_t)(u >> 16);
    if ((h & 0x7f80) == 0x7f80) h = 0x7f7f;
  } else {
    h = (uint16_t)(u >> 16);
  }
  return h;
}

// BF16(float): QuantizationArithmetic.cpp:958-964.
float orc_bf16(float src, int rounding) {
  uint32_t u = (uint32_t)orc_f32_to_bf16(src, rounding) << 16;
  float d;
  std::memcpy(&d, &u, 4);
  return d;
}

// F32ToInt / F32ToInt8: QuantizationArithmetic.cpp:918-947.
static inline int32_t f32_to_int(float v, int round_mode) {
  if (round_mode == 1) return (int)v;
  float integer;
  float abs_v = std::fabs(v);
  float fraction = std::modf(abs_v, &integer);
  int32_t i = (int)integer;
  if (fraction > 0.5f) i += 1;
  else if (fraction == 0.5f && (i & 1)) i += 1;
  return v < 0 ? -i : i;
}
int orc_f32_to_int8(float v, int round_mode) {
  int32_t i = f32_to_int(v, round_mode);
  return i > 127 ? 127 : (i < -128 ? -128 : i);
}

// ---------------------------------------------------------------------------
// Conv2D. core/conv.cpp:11-104 with the MKL-DNN contraction
// (NativeCpuImplementation.h:11-102) replaced by a direct loop. Weights are
// [g][oc/g][ic/g][kh][kw]; zero padding; dilation; optional input insertion.
// mode: 0 = INT8 (int32 accumulate, bias + QDM + saturate + ReLU per
// QuantizationArithmetic.cpp:849-871), 1 = FP32 (double accumulate, bias, ReLU),
// 2 = BF16 (as FP32 then BF16 rounding, conv.cpp:94-98).
// ---------------------------------------------------------------------------
void orc_conv2d(const float *in, const float *filter, const float *bias,
                const float *rshift, const float *multiplier, float *out, int n,
                int ic, int ih, int iw, int oc, int oh, int ow, int g, int kh,
                int kw, int sh, int sw, int pt, int pl, int dh, int dw,
                int ins_h, int ins_w, int do_relu, int mode) {
  const int ihd = (ih - 1) * (ins_h + 1) + 1, iwd = (iw - 1) * (ins_w + 1) + 1;
  const int icg = ic / g, ocg = oc / g;
#pragma omp parallel for collapse(2)
  for (int b = 0; b < n; ++b)
    for (int o = 0; o < oc; ++o) {
      const int grp = o / ocg;
      for (int y = 0; y < oh; ++y)
        for (int x = 0; x < ow; ++x) {
          int64_t acc_i = 0;
          double acc_f = 0.0;
          for (int c = 0; c < icg; ++c)
            for (int r = 0; r < kh; ++r) {
              int yy = y * sh - pt + r * dh;
              if (yy < 0 || yy >= ihd || (yy % (ins_h + 1)) != 0) continue;
              for (int s = 0; s < kw; ++s) {
                int xx = x * sw - pl + s * dw;
                if (xx < 0 || xx >= iwd || (xx % (ins_w + 1)) != 0) continue;
                float a = in[(((size_t)b * ic + grp * icg + c) * ih + yy / (ins_h + 1)) * iw + xx / (ins_w + 1)];
                float w = filter[(((size_t)o * icg + c) * kh + r) * kw + s];
                if (mode == 0) acc_i += (int64_t)((int32_t)a * (int32_t)w);
                else acc_f += (double)a * (double)w;
              }
            }
          size_t oi = (((size_t)b * oc + o) * oh + y) * ow + x;
          if (mode == 0) {
            int32_t v = (int32_t)acc_i;
            if (bias) v += (int32_t)bias[o];
            int q = orc_qdm_i32(v, (uint32_t)rshift[o], (uint32_t)multiplier[o]);
            if (do_relu && q < 0) q = 0;
            out[oi] = (float)q;
          } else {
            float v = (float)(acc_f + (bias ? (double)bias[o] : 0.0));
            if (do_relu && v < 0) v = 0;
            if (mode == 2) v = orc_bf16(v, 1);
            out[oi] = v;
          }
        }
    }
}

// ---------------------------------------------------------------------------
// FullyConnected. core/fullyconnected.cpp:44-91: Y[m,n] = X[m,k] . W[n,k]^T + b,
// ReLU on the float, then (INT8) the float overload of the QDM requant with a
// single (rshift, multiplier) per batch slice. The filter is stored [n][k]
// (mkldnn_ip weights, NativeCpuImplementation.cpp:185-288).
// ---------------------------------------------------------------------------
void orc_fc(const float *in, const float *filter, const float *bias,
            const float *rshift, const float *multiplier, float *out, int batch,
            int m, int k, int n, int do_relu, int mode) {
  for (int b = 0; b < batch; ++b) {
#pragma omp parallel for collapse(2)
    for (int i = 0; i < m; ++i)
      for (int j = 0; j < n; ++j) {
        int64_t acc_i = 0;
        double acc_f = 0;
        const float *x = in + ((size_t)b * m + i) * k;
        const float *w = filter + ((size_t)b * n + j) * k;
        for (int t = 0; t < k; ++t) {
          if (mode == 0) acc_i += (int64_t)((int32_t)x[t] * (int32_t)w[t]);
          else acc_f += (double)x[t] * (double)w[t];
        }
        float v = mode == 0 ? (float)((double)acc_i + (bias ? (double)bias[(size_t)b * n + j] : 0.0))
                            : (float)(acc_f + (bias ? (double)bias[(size_t)b * n + j] : 0.0));
        if (do_relu && v < 0) v = 0;
        if (mode == 0) v = (float)orc_qdm_f32(v, (uint32_t)rshift[b], (uint32_t)multiplier[b]);
        else if (mode == 2) v = orc_bf16(v, 1);
        out[((size_t)b * m + i) * n + j] = v;
      }
  }
}

// ---------------------------------------------------------------------------
// Pooling. core/pooling.cpp:33-160. method 0 = max (padded taps ignored, as
// MKL-DNN pooling_max), 1 = avg. INT8 avg sums the zero-padded window and
// applies the non-QDM (multiplier, rshift) rule (pooling.cpp:146-155); fp32 avg
// divides by kh*kw when count_include_pad, else by the number of valid taps
// (NativeCpuImplementation.h:123-125).
// ---------------------------------------------------------------------------
void orc_pool(const float *in, float *out, int n, int c, int ih, int iw, int oh,
              int ow, int kh, int kw, int sh, int sw, int pt, int pl,
              int method, int is_int8, int count_include_pad, float rshift,
              float multiplier) {
#pragma omp parallel for collapse(2)
  for (int b = 0; b < n; ++b)
    for (int ch = 0; ch < c; ++ch)
      for (int y = 0; y < oh; ++y)
        for (int x = 0; x < ow; ++x) {
          const float *p = in + ((size_t)b * c + ch) * ih * iw;
          float mx = -INFINITY;
          double sum = 0;
          int cnt = 0;
          for (int r = 0; r < kh; ++r)
            for (int s = 0; s < kw; ++s) {
              int yy = y * sh - pt + r, xx = x * sw - pl + s;
              if (yy < 0 || yy >= ih || xx < 0 || xx >= iw) continue;
              float v = p[yy * iw + xx];
              mx = std::max(mx, v);
              sum += v;
              ++cnt;
            }
          float res;
          if (method == 0) res = mx;
          else if (is_int8) res = (float)orc_mul_rshift_f32((float)sum, (uint32_t)rshift, (uint32_t)multiplier);
          else res = (float)(sum / (count_include_pad ? kh * kw : cnt));
          out[(((size_t)b * c + ch) * oh + y) * ow + x] = res;
        }
}

// ---------------------------------------------------------------------------
// Eltwise add / mul. core/eltwise.cpp:39-85, 318-357.
// ---------------------------------------------------------------------------
void orc_eltwise_add_i8(const float *const *ins, int nin, const float *multiplier,
                        float rshift, int do_relu, float *out, size_t size) {
  for (size_t i = 0; i < size; ++i) {
    float acc = 0;
    for (int k = 0; k < nin; ++k) acc += ins[k][i] * (float)(int8_t)multiplier[k];
    if (do_relu && acc < 0) acc = 0;
    out[i] = (float)orc_rshift_f32(acc, (uint32_t)rshift);
  }
}

void orc_eltwise_add_f32(const float *const *ins, int nin, const float *coeff,
                         int do_relu, int to_bf16, float *out, size_t size) {
  for (size_t i = 0; i < size; ++i) {
    float acc = 0;
    for (int k = 0; k < nin; ++k) acc += (coeff ? coeff[k] : 1.0f) * ins[k][i];
    if (do_relu && acc < 0) acc = 0;
    out[i] = to_bf16 ? orc_bf16(acc, 1) : acc;
  }
}

void orc_eltwise_mul_i8(const float *const *ins, int nin, float multiplier,
                        float rshift, int do_relu, float *out, size_t size) {
  for (size_t i = 0; i < size; ++i) {
    float acc = 1;
    for (int k = 0; k < nin; ++k) acc *= ins[k][i];
    if (do_relu && acc < 0) acc = 0;
    if (rshift != 0 || multiplier != 0)
      acc = (float)orc_qdm_f32(acc, (uint32_t)rshift, (uint32_t)multiplier);
    out[i] = acc;
  }
}

// ---------------------------------------------------------------------------
// Concat along the channel axis with optional per-input non-QDM requant.
// core/concat.cpp:34-90 (identity when multiplier==1 && rshift==0).
// ---------------------------------------------------------------------------
void orc_concat_c(const float *const *ins, int nin, const int *in_c, int n,
                  int hw, const float *multiplier, const float *rshift,
                  int need_quant, int do_relu, float *out) {
  int oc = 0;
  for (int k = 0; k < nin; ++k) oc += in_c[k];
  int coff = 0;
  for (int k = 0; k < nin; ++k) {
    for (int b = 0; b < n; ++b)
      for (size_t i = 0; i < (size_t)in_c[k] * hw; ++i) {
        float v = ins[k][(size_t)b * in_c[k] * hw + i];
        if (need_quant && !(multiplier[k] == 1 && rshift[k] == 0))
          v = (float)orc_mul_rshift_f32(v, (uint32_t)rshift[k], (uint32_t)multiplier[k]);
        if (do_relu && v < 0) v = 0;
        out[((size_t)b * oc + coff) * hw + i] = v;
      }
    coff += in_c[k];
  }
}

// Nearest upsample: core/upsample.cpp:20-41.
void orc_upsample(const float *in, float *out, int n, int c, int ih, int iw,
                  int scale_h, int scale_w) {
  int h = ih * scale_h, w = iw * scale_w;
  for (int nc = 0; nc < n * c; ++nc)
    for (int y = 0; y < h; ++y)
      for (int x = 0; x < w; ++x)
        out[((size_t)nc * h + y) * w + x] = in[((size_t)nc * ih + y / scale_h) * iw + x / scale_w];
}

// Pixel shuffle (depth to space): core/depthtospace.cpp:6-48.
void orc_pixelshuffle(const float *in, float *out, int n, int ic, int ih, int iw,
                      int r, int dcr_mode) {
  int oc = ic / (r * r), oh = ih * r, ow = iw * r;
  size_t idx = 0;
  for (int b = 0; b < n; ++b)
    for (int c = 0; c < ic; ++c)
      for (int h = 0; h < ih; ++h)
        for (int w = 0; w < iw; ++w) {
          int nc, nh, nw;
          if (dcr_mode) {
            nc = c % oc;
            nh = h * r + (c / oc) / r;
            nw = w * r + (c / oc) % r;
          } else {
            nc = c / (r * r);
            nh = h * r + (c / r) % r;
            nw = w * r + (c % (r * r)) % r;
          }
          out[(((size_t)b * oc + nc) * oh + nh) * ow + nw] = in[idx++];
        }
}

// ---------------------------------------------------------------------------
// Quant op family. core/quant.cpp:9-166.
// kind: 0 fp32->int8 host rounding (directly after the input op, :22-30)
//       1 fp32->int8 TPU mode (:11-20)      2 int8->fp32 (:97-104)
//       3 int8->bf16 (:78-85)               4 bf16->int8 (:87-94)
//       5 fp32->bf16 truncation (:41-52)
// ---------------------------------------------------------------------------
void orc_quant(const float *in, float *out, size_t size, float scale, int zp, int kind) {
  for (size_t i = 0; i < size; ++i) {
    float x = in[i];
    switch (kind) {
    case 0: {
      int v = (int)std::round(x * scale) + zp;
      out[i] = (float)(v > 127 ? 127 : (v < -128 ? -128 : v));
      break;
    }
    case 1: {
      float s = orc_bf16(scale, 1);
      float v = orc_bf16(orc_bf16(orc_bf16(x, 0) * s, 1) + zp, zp != 0);
      out[i] = (float)orc_f32_to_int8(v, 0);
      break;
    }
    case 2:
    case 3: {
      float s = orc_bf16(scale, 1);
      float z = kind == 3 ? (float)(int)orc_bf16((float)zp, 1) : (float)zp;
      out[i] = orc_bf16(orc_bf16(x + z, z != 0) * s, 1);
      break;
    }
    case 4: {
      float s = orc_bf16(scale, 1);
      out[i] = (float)orc_f32_to_int8(orc_bf16(x * s, 1), 0);
      break;
    }
    default:
      out[i] = orc_bf16(x, 0);
    }
  }
}

// Leaky ReLU INT8: core/activation.cpp:126-153.
void orc_leaky_relu_i8(const float *in, float *out, size_t size, float rshift_pos,
                       float mult_pos, float rshift_neg, float mult_neg) {
  for (size_t i = 0; i < size; ++i) {
    if (in[i] > 0) {
      out[i] = mult_pos != 0.0f
                   ? (float)orc_mul_rshift_f32(in[i], (uint32_t)rshift_pos, (uint32_t)mult_pos)
                   : in[i];
    } else {
      out[i] = (float)orc_mul_rshift_f32(in[i], (uint32_t)rshift_neg, (uint32_t)mult_neg);
    }
  }
}

// ReLU: core/internal.cpp:13-18.
void orc_relu(const float *in, float *out, size_t size) {
  for (size_t i = 0; i < size; ++i) out[i] = in[i] > 0 ? in[i] : 0;
}

// ---------------------------------------------------------------------------
// BF16 lookup tables. core/lut_func.cpp.
// ---------------------------------------------------------------------------
typedef float (*actf_t)(float, float, float);
static float f_sigmoid(float x, float s, float b) { return s / (1 + expf(-x)) + b; }
static float f_exp(float x, float s, float b) { return s * expf(x) + b; }
static float f_softplus(float x, float s, float b) { return s * logf(expf(x) + 1) + b; }
static float f_mish(float x, float, float) { return x * tanh(f_softplus(x, 1, 0)); }
static float f_tanh(float x, float, float) { return tanh(x); }

// kind: 0 sigmoid (range 12), 1 mish (8), 2 exp (15), 3 tanh (15): lut_func.hpp:8-15.
static actf_t lut_fn(int kind, float *range) {
  switch (kind) {
  case 0: *range = 12; return f_sigmoid;
  case 1: *range = 8; return f_mish;
  case 2: *range = 15; return f_exp;
  default: *range = 15; return f_tanh;
  }
}

// Table generation: lut_func.cpp:32-134.
void orc_lut_gen_slope_tables(int kind, float p0, float p1, float *base, float *slope) {
  float R;
  actf_t f = lut_fn(kind, &R);
  float start = -R, end = R;
  const int hw = 256, half = 128;
  int range = std::abs((int)(end - start));
  float interval = (float)range / (float)hw;
  for (int i = 0; i < half; ++i) base[i] = orc_bf16(f(0 + i * interval, p0, p1), 1);
  for (int i = half, j = 0; i < hw; ++i, ++j) base[i] = orc_bf16(f(start + j * interval, p0, p1), 1);
  float scale = ((float)hw) / (end - start);
  for (int i = 0; i < half - 1; ++i) {
    float x0 = base[i], x1 = base[i + 1];
    slope[i] = orc_f32_to_bf16(x0, 0) == orc_f32_to_bf16(x1, 0) ? 0 : orc_bf16(x1 - x0, 1);
  }
  slope[half - 1] = orc_bf16((f(3 * end, p0, p1) - f(end, p0, p1)) / (2 * end * scale), 1);
  for (int i = hw - 1; i > half; --i) {
    float x0 = base[i], x1 = base[i - 1];
    slope[i] = orc_f32_to_bf16(x0, 0) == orc_f32_to_bf16(x1, 0) ? 0 : orc_bf16(x0 - x1, 1);
  }
  slope[half] = orc_bf16((f(3 * start, p0, p1) - f(start, p0, p1)) / (std::abs(2 * start) * scale), 1);
}

// Slope interpolation: lut_func.cpp:136-187 (offset is always 0 for these ranges).
void orc_lut_bf16_slope(int kind, const float *in, float *out, size_t size,
                        const float *base, const float *slope) {
  float R;
  lut_fn(kind, &R);
  float scale = orc_bf16((float)(256.0 / (2 * R)), 1);
  for (size_t i = 0; i < size; ++i) {
    float r = orc_bf16(orc_bf16(in[i] - 0.0f, 0) * scale, 1);
    int idx = orc_f32_to_int8(r, 1);
    float dx = orc_bf16(r - idx, 1);
    float s = slope[idx & 0xff], b = base[idx & 0xff];
    volatile float prod = dx * s; // keep multiply and add separate (no FMA)
    out[i] = orc_bf16(b + prod, 1);
  }
}

// Exponent / mantissa tables for pow (reciprocal is coeff = -1): lut_func.cpp:189-274.
void orc_lut_gen_pow_tables(float coeff, float *exp_table, float *mant_table) {
  const int half = 128, start = -62;
  uint32_t maxu = 0x7F7F0000u;
  float maxf;
  std::memcpy(&maxf, &maxu, 4);
  for (int i = 0; i < 256; ++i) exp_table[i] = 0;
  float edge = coeff < 0 ? maxf : (coeff == 0 ? orc_bf16(1.0f, 1) : orc_bf16(0.0f, 1));
  int idx = 0;
  exp_table[idx++] = edge;
  for (int i = 0; i < half - 1; ++i) exp_table[idx++] = orc_bf16((float)pow(2, coeff * (float)(start + i)), 1);
  exp_table[idx++] = edge;
  if (coeff == (int)coeff) {
    int sgn = ((int)coeff % 2 == 0) ? 1 : -1;
    for (int i = 0; i < half - 1; ++i) exp_table[idx++] = orc_bf16(sgn * (float)pow(2, coeff * (float)(start + i)), 1);
  }
  for (int i = 0; i < half; ++i) {
    float d = (float)(1 + i * 1 / 128.0);
    d = (float)pow(d, coeff);
    mant_table[i] = mant_table[128 + i] = orc_bf16(d, 1);
  }
}

// Exponent / mantissa tables of the logarithm: lut_func.cpp:238-286. log(x) = e*ln2 + log(1.m); entry 0 and
// the negative half hold the most negative BF16 number.
void orc_lut_gen_log_tables(float *exp_table, float *mant_table) {
  const int half = 128, start = -62;
  uint32_t negu = 0xFF7F0000u;
  float negmax;
  std::memcpy(&negmax, &negu, 4);
  for (int i = 0; i < 256; ++i) exp_table[i] = 0;
  exp_table[0] = negmax;
  for (int i = 0; i < half - 1; ++i) {
    float e = (float)(start + i);
    exp_table[1 + i] = orc_bf16((float)(e * log(2.)), 1);
    exp_table[128 + 1 + i] = negmax;
  }
  for (int i = 0; i < half; ++i) {
    float d = (float)(1 + i * 1 / 128.0);
    mant_table[i] = mant_table[128 + i] = orc_bf16((float)log(d), 1);
  }
}

// Exponent x mantissa lookup: lut_func.cpp:306-333; method "mantissa" multiplies the two entries
// (is_log 0), method "log" adds them (is_log 1).
static inline float orc_lut_mantissa_one(float v, const float *exp_table, const float *mant_table, int is_log) {
  uint16_t h = orc_f32_to_bf16(v, 0);
  int e;
  if (v == 0) e = 0;
  else if (v >= 0) e = (int)floor(log2(v)) + 63;
  else e = (int)floor(log2(-1 * v)) + 62 + 129;
  volatile float ex = exp_table[e], ma = mant_table[h & 0xff];
  return orc_bf16(is_log ? ex + ma : ex * ma, 1);
}
void orc_lut_bf16_mantissa(const float *in, float *out, size_t size,
                           const float *exp_table, const float *mant_table) {
  for (size_t i = 0; i < size; ++i) out[i] = orc_lut_mantissa_one(in[i], exp_table, mant_table, 0);
}
void orc_lut_bf16_mantissa_log(const float *in, float *out, size_t size,
                               const float *exp_table, const float *mant_table) {
  for (size_t i = 0; i < size; ++i) out[i] = orc_lut_mantissa_one(in[i], exp_table, mant_table, 1);
}

// BF16 softmax over one axis (core/softmax.cpp:88-151): max, BF16(x - max), exp through the slope table,
// sum_j ex_j * BF16(BF16(C)/C) accumulated in fp32 in channel order and rounded once, reciprocal (or log)
// through the exponent / mantissa tables, BF16(ex * 1/sum) or BF16(sub - log(sum)).
void orc_softmax_bf16(const float *in, float *out, int outer, int channel, int inner, int do_log,
                      const float *exp_table, const float *exp_slope, const float *rec_table, const float *rec_mant) {
  std::vector<float> mx(inner), sum(inner), sub((size_t)channel * inner), ex((size_t)channel * inner);
  for (int i = 0; i < outer; ++i) {
    const float *x = in + (size_t)i * channel * inner;
    float *y = out + (size_t)i * channel * inner;
    for (int k = 0; k < inner; ++k) mx[k] = x[k];
    for (int j = 0; j < channel; ++j)
      for (int k = 0; k < inner; ++k)
        if (mx[k] < x[(size_t)j * inner + k]) mx[k] = x[(size_t)j * inner + k];
    for (int j = 0; j < channel; ++j)
      for (int k = 0; k < inner; ++k) sub[(size_t)j * inner + k] = orc_bf16(x[(size_t)j * inner + k] - mx[k], 1);
    orc_lut_bf16_slope(2, sub.data(), ex.data(), (size_t)channel * inner, exp_table, exp_slope);
    const float const_val = orc_bf16(orc_bf16(1.0f * channel, 1) / channel, 1);
    for (int k = 0; k < inner; ++k) sum[k] = 0;
    for (int j = 0; j < channel; ++j)
      for (int k = 0; k < inner; ++k) {
        volatile float t = ex[(size_t)j * inner + k] * const_val;
        sum[k] += t;
      }
    for (int k = 0; k < inner; ++k) sum[k] = orc_lut_mantissa_one(orc_bf16(sum[k], 1), rec_table, rec_mant, do_log);
    for (int j = 0; j < channel; ++j)
      for (int k = 0; k < inner; ++k) {
        size_t idx = (size_t)j * inner + k;
        y[idx] = do_log ? orc_bf16(sub[idx] - sum[k], 1) : orc_bf16(ex[idx] * sum[k], 1);
      }
  }
}

// INT8 256-entry table: core/activation.cpp:49-53.
void orc_lut_i8(const float *in, float *out, size_t size, const float *table) {
  for (size_t i = 0; i < size; ++i) out[i] = table[(unsigned char)in[i]];
}

// ---------------------------------------------------------------------------
// fp32 graph ops used by the calibration forward.
// ---------------------------------------------------------------------------
// Scale: core/scale.cpp:15-37.
void orc_scale_f32(const float *in, const float *scale, const float *bias, float *out,
                   int n, int c, int hw) {
  for (int b = 0; b < n; ++b)
    for (int ch = 0; ch < c; ++ch)
      for (int i = 0; i < hw; ++i) {
        size_t o = ((size_t)b * c + ch) * hw + i;
        float y = in[o] * scale[ch];
        if (bias) y += bias[ch];
        out[o] = y;
      }
}

// BatchNorm: core/batchnorm.cpp:20-68.
void orc_batchnorm_f32(const float *in, const float *mean, const float *var, float scale0,
                       float eps, float *out, int n, int c, int hw) {
  float sf = 1 / scale0;
  for (int b = 0; b < n; ++b)
    for (int ch = 0; ch < c; ++ch) {
      float m = mean[ch] * sf, v = var[ch] * sf;
      for (int i = 0; i < hw; ++i) {
        size_t o = ((size_t)b * c + ch) * hw + i;
        float x = in[o] - m;
        float d = std::sqrt(v + eps); // `auto d = sqrt(float)`: the float overload
        out[o] = x / d;
      }
    }
}

// Softmax over axis with [outer, channel, inner]: core/softmax.cpp:49-86.
void orc_softmax_f32(const float *in, float *out, int outer, int channel, int inner) {
  for (int i = 0; i < outer; ++i)
    for (int k = 0; k < inner; ++k) {
      const float *p = in + (size_t)i * channel * inner + k;
      float *q = out + (size_t)i * channel * inner + k;
      float mx = p[0];
      for (int j = 0; j < channel; ++j) mx = std::max(mx, p[(size_t)j * inner]);
      float sum = 0;
      for (int j = 0; j < channel; ++j) {
        q[(size_t)j * inner] = std::exp(p[(size_t)j * inner] - mx);
        sum += q[(size_t)j * inner];
      }
      for (int j = 0; j < channel; ++j) q[(size_t)j * inner] /= sum;
    }
}

// ---------------------------------------------------------------------------
// Calibration statistics.
// ---------------------------------------------------------------------------
// 2048-bin |x| histogram: python/cvi_toolkit/calibration/kld_calibrator.py:31-43
// (fp32 arithmetic throughout; zero elements skipped; np.histogram over
// range (0, bins-1) maps an integral index to itself for bins <= 4096).
void orc_histogram(const float *x, size_t size, float abs_max, int bins, int64_t *hist) {
  float width = abs_max / (float)(bins - 1);
  for (size_t i = 0; i < size; ++i) {
    float t = std::fabs(x[i]);
    if (t == 0) continue;
    float idx = std::floor(t / width + 0.5f);
    int b = (int)idx;
    if (b > bins - 1) continue; // outside np.histogram's range
    hist[b] += 1;
  }
}

// KLD threshold search: bindings/python/kld/calibration_math.cpp:169-223, 283-344.
float orc_kld_threshold(const int *data, float width, long long N, float *kl_out) {
  const long long BINS = 128;
  const long long KL_NUM = N / BINS;
  std::vector<long long> hist(N);
  std::vector<float> kl(KL_NUM, 0.0f);
  long long count = 0;
  for (long long i = 0; i < N; ++i) {
    hist[i] = data[i];
    count += hist[i];
  }
  long long m = 0;
  for (long long i = BINS; i < N + 1; i += BINS, ++m) {
    std::vector<float> P(i, 0.0f), Q(i, 0.0f);
    for (long long j = 0; j < N; ++j) {
      long long index = (j > (i - 1)) ? (i - 1) : j;
      P[index] += hist[j];
    }
    for (long long j = 0; j < i; ++j) P[j] /= count;
    float sum = 0.0;
    long long expand = i / BINS, idx = 0;
    for (long long j = 0; j < i; ++j) sum += hist[j];
    for (long long j = 0; j < BINS; ++j) {
      float sum_bin = 0, pos = 0;
      long long bin_idx = idx;
      for (long long k = 0; k < expand; ++k) {
        sum_bin += hist[idx];
        pos += (hist[idx] > 0) ? 1 : 0;
        idx++;
      }
      pos = (pos == 0) ? 1 : pos;
      float Q_base = sum_bin / pos / sum;
      while (bin_idx < idx) {
        Q[bin_idx] = hist[bin_idx] ? Q_base : 0;
        bin_idx++;
      }
    }
    for (idx = 0; idx < i; ++idx)
      kl[m] += P[idx] * (log10(P[idx] + 1e-30) - log10(Q[idx] + 1e-30));
  }
  long long m_min = 0;
  float best = kl[0];
  for (long long i = 1; i < m; ++i)
    if (best > kl[i]) {
      best = kl[i];
      m_min = i;
    }
  if (kl_out)
    for (long long i = 0; i < m; ++i) kl_out[i] = kl[i];
  return width * (m_min + 1) * BINS;
}

// ---------------------------------------------------------------------------
// Eltwise max / min, INT8 (core/eltwise.cpp:143-181 and :225-263): every input is multiplied by
// its int8 multiplier, the extremum taken, optional ReLU, then one rshift + saturation.
// ---------------------------------------------------------------------------
void orc_eltwise_maxmin_i8(const float *const *ins, int nin, const float *multiplier, float rshift,
                           int do_relu, int is_min, float *out, size_t size) {
  for (size_t i = 0; i < size; ++i) {
    float v = ins[0][i] * (float)(int8_t)multiplier[0];
    for (int k = 1; k < nin; ++k) {
      float x = ins[k][i] * (float)(int8_t)multiplier[k];
      v = is_min ? (v < x ? v : x) : (v > x ? v : x);
    }
    if (do_relu && v < 0) v = 0;
    out[i] = (float)orc_rshift_f32(v, (uint32_t)rshift);
  }
}

// ---------------------------------------------------------------------------
// Broadcast add / sub / mul (core/broadcast.cpp:45-156). op: 0 add, 1 sub, 2 mul. A dimension of
// extent 1 repeats. INT8: add/sub scale each input by its int8 multiplier and end with rshift +
// saturation; mul ends with the QDM requantisation by multiplier[0]. fp32: plain arithmetic.
// ---------------------------------------------------------------------------
void orc_broadcast(const float *a, const int *sa, const float *b, const int *sb, int op, int is_int8,
                   const float *multiplier, float rshift, int do_relu, float *out) {
  const int on = std::max(sa[0], sb[0]), oc = std::max(sa[1], sb[1]), oh = std::max(sa[2], sb[2]),
            ow = std::max(sa[3], sb[3]);
  size_t idx = 0;
  for (int n = 0; n < on; ++n)
    for (int c = 0; c < oc; ++c)
      for (int h = 0; h < oh; ++h)
        for (int w = 0; w < ow; ++w) {
          size_t i0 = (((size_t)(sa[0] == 1 ? 0 : n) * sa[1] + (sa[1] == 1 ? 0 : c)) * sa[2] + (sa[2] == 1 ? 0 : h)) * sa[3] +
                      (sa[3] == 1 ? 0 : w);
          size_t i1 = (((size_t)(sb[0] == 1 ? 0 : n) * sb[1] + (sb[1] == 1 ? 0 : c)) * sb[2] + (sb[2] == 1 ? 0 : h)) * sb[3] +
                      (sb[3] == 1 ? 0 : w);
          float x = a[i0], y = b[i1], v;
          if (op == 2) {
            v = x * y;
          } else {
            if (is_int8) {
              x *= (float)(int8_t)multiplier[0];
              y *= (float)(int8_t)multiplier[1];
            }
            v = op == 0 ? x + y : x - y;
          }
          if (do_relu && v < 0) v = 0;
          if (is_int8)
            v = op == 2 ? (float)orc_qdm_f32(v, (uint32_t)rshift, (uint32_t)multiplier[0])
                        : (float)orc_rshift_f32(v, (uint32_t)rshift);
          out[idx++] = v;
        }
}

// ---------------------------------------------------------------------------
// Pad (core/pad.cpp:7-141). pads = {n, c, h, w begin; n, c, h, w end}. mode 0 ("constant"): the body
// is copied, negative pads cut; the reference never writes const_val, the border keeps the zero the
// result tensor was created with. mode 1 ("edge"): h/w borders replicate the nearest body value.
// ---------------------------------------------------------------------------
void orc_pad(const float *in, const int *s, const int *pads, int mode, float *out) {
  const int on = s[0] + pads[0] + pads[4], oc = s[1] + pads[1] + pads[5], oh = s[2] + pads[2] + pads[6],
            ow = s[3] + pads[3] + pads[7];
  for (int n = 0; n < on; ++n)
    for (int c = 0; c < oc; ++c)
      for (int h = 0; h < oh; ++h)
        for (int w = 0; w < ow; ++w) {
          int in_n = n - pads[0], in_c = c - pads[1], in_h = h - pads[2], in_w = w - pads[3];
          if (mode == 1) {
            in_h = std::min(std::max(in_h, 0), s[2] - 1);
            in_w = std::min(std::max(in_w, 0), s[3] - 1);
          }
          float v = 0.0f;
          if (in_n >= 0 && in_n < s[0] && in_c >= 0 && in_c < s[1] && in_h >= 0 && in_h < s[2] && in_w >= 0 &&
              in_w < s[3])
            v = in[(((size_t)in_n * s[1] + in_c) * s[2] + in_h) * s[3] + in_w];
          out[(((size_t)n * oc + c) * oh + h) * ow + w] = v;
        }
}

// Crop (core/crop.cpp:18-92): out[n,c,h,w] = in[n*step0 + off0, c*step1 + off1, ...].
void orc_crop(const float *in, const int *s, const int *os, const int *off, const int *steps, float *out) {
  for (int n = 0; n < os[0]; ++n)
    for (int c = 0; c < os[1]; ++c)
      for (int h = 0; h < os[2]; ++h)
        for (int w = 0; w < os[3]; ++w)
          out[(((size_t)n * os[1] + c) * os[2] + h) * os[3] + w] =
              in[(((size_t)(n * steps[0] + off[0]) * s[1] + (c * steps[1] + off[1])) * s[2] + (h * steps[2] + off[2])) * s[3] +
                 (w * steps[3] + off[3])];
}

// Permute (core/permute.cpp:6-33): output dimension k is input dimension order[k].
void orc_permute(const float *in, const int *s, const int *order, float *out) {
  for (int n = 0; n < s[0]; ++n)
    for (int c = 0; c < s[1]; ++c)
      for (int h = 0; h < s[2]; ++h)
        for (int w = 0; w < s[3]; ++w) {
          const int cur[4] = {n, c, h, w};
          size_t o = (((size_t)cur[order[0]] * s[order[1]] + cur[order[1]]) * s[order[2]] + cur[order[2]]) * s[order[3]] +
                     cur[order[3]];
          out[o] = in[(((size_t)n * s[1] + c) * s[2] + h) * s[3] + w];
        }
}

// Reduce over consecutive axes (core/reduce.cpp:52-115). type: 0 mean, 1 sum, 2 max, 3 min. INT8 mean
// leaves the division to the multiplier / rshift pair (non-QDM) that follows when it is not (1, 0).
void orc_reduce(const float *in, int outer, int axis, int inner, int type, int is_int8, float multiplier,
                float rshift, float *out) {
  for (int o = 0; o < outer; ++o)
    for (int i = 0; i < inner; ++i) {
      float v;
      if (type <= 1) {
        float sum = 0.0f;
        for (int a = 0; a < axis; ++a) sum += in[((size_t)o * axis + a) * inner + i];
        v = (type == 0 && !is_int8) ? sum / axis : sum;
      } else {
        v = in[(size_t)o * axis * inner + i];
        for (int a = 1; a < axis; ++a) {
          float x = in[((size_t)o * axis + a) * inner + i];
          if (type == 2 ? x > v : x < v) v = x;
        }
      }
      if (is_int8 && (rshift != 0 || multiplier != 1))
        v = (float)orc_mul_rshift_f32(v, (uint32_t)rshift, (uint32_t)multiplier);
      out[(size_t)o * inner + i] = v;
    }
}

// REDUCE_L2 in fp32 (core/reduce.cpp:91-103): `sum += std::pow(x, 2)` promotes to double (the square is exact
// there) and rounds the running sum to float at every step; the result is std::pow(sum, coeff) on floats.
void orc_reduce_l2_f32(const float *in, int outer, int axis, int inner, float coeff, float *out) {
  for (int o = 0; o < outer; ++o)
    for (int i = 0; i < inner; ++i) {
      float sum = 0.0f;
      for (int a = 0; a < axis; ++a) sum += std::pow(in[((size_t)o * axis + a) * inner + i], 2);
      out[(size_t)o * inner + i] = std::pow(sum, coeff);
    }
}

// ---------------------------------------------------------------------------
// DeConv2D, INT8 (core/deconv.cpp:6-73). The reference runs MKL-DNN's deconvolution_forward on
// oihw / goihw weights (NativeCpuImplementation.h:197-283), whose definition is the scatter
//   dst[n, oc, ih*sh + kh*dh - pt, iw*sw + kw*dw - pl] += src[n, ic, ih, iw] * w[oc, ic, kh, kw],
// then adds the int32 bias and requantises per channel (QuantizationArithmetic.cpp:849-871).
// ---------------------------------------------------------------------------
void orc_deconv2d_i8(const float *in, const float *filter, const float *bias, const float *rshift,
                     const float *multiplier, float *out, int n, int ic, int ih, int iw, int oc, int oh, int ow,
                     int g, int kh, int kw, int sh, int sw, int pt, int pl, int dh, int dw, int do_relu) {
  const int icg = ic / g, ocg = oc / g;
  std::vector<int64_t> acc((size_t)n * oc * oh * ow, 0);
  for (int b = 0; b < n; ++b)
    for (int o = 0; o < oc; ++o) {
      const int grp = o / ocg;
      for (int c = 0; c < icg; ++c)
        for (int y = 0; y < ih; ++y)
          for (int x = 0; x < iw; ++x) {
            const int32_t a = (int32_t)in[(((size_t)b * ic + grp * icg + c) * ih + y) * iw + x];
            if (a == 0) continue;
            for (int r = 0; r < kh; ++r) {
              const int oy = y * sh + r * dh - pt;
              if (oy < 0 || oy >= oh) continue;
              for (int q = 0; q < kw; ++q) {
                const int ox = x * sw + q * dw - pl;
                if (ox < 0 || ox >= ow) continue;
                acc[(((size_t)b * oc + o) * oh + oy) * ow + ox] +=
                    (int64_t)(a * (int32_t)filter[(((size_t)o * icg + c) * kh + r) * kw + q]);
              }
            }
          }
    }
  for (int b = 0; b < n; ++b)
    for (int o = 0; o < oc; ++o)
      for (int i = 0; i < oh * ow; ++i) {
        const size_t oi = ((size_t)b * oc + o) * oh * ow + i;
        int32_t v = (int32_t)acc[oi];
        if (bias) v += (int32_t)bias[o];
        int q = orc_qdm_i32(v, (uint32_t)rshift[o], (uint32_t)multiplier[o]);
        if (do_relu && q < 0) q = 0;
        out[oi] = (float)q;
      }
}

// The same scatter for fp32 and BF16 graphs (core/deconv.cpp:56-68: MKL-DNN deconvolution with the fp32 bias, ReLU,
// and for BF16 one rounding of the result). Sums in double: the order of MKL-DNN's own sum is not known.
void orc_deconv2d_f(const float *in, const float *filter, const float *bias, float *out, int n, int ic, int ih, int iw,
                    int oc, int oh, int ow, int g, int kh, int kw, int sh, int sw, int pt, int pl, int dh, int dw,
                    int do_relu, int to_bf16) {
  const int icg = ic / g, ocg = oc / g;
  std::vector<double> acc((size_t)n * oc * oh * ow, 0.0);
  for (int b = 0; b < n; ++b)
    for (int o = 0; o < oc; ++o) {
      const int grp = o / ocg;
      for (int c = 0; c < icg; ++c)
        for (int y = 0; y < ih; ++y)
          for (int x = 0; x < iw; ++x) {
            const double a = in[(((size_t)b * ic + grp * icg + c) * ih + y) * iw + x];
            for (int r = 0; r < kh; ++r) {
              const int oy = y * sh + r * dh - pt;
              if (oy < 0 || oy >= oh) continue;
              for (int q = 0; q < kw; ++q) {
                const int ox = x * sw + q * dw - pl;
                if (ox < 0 || ox >= ow) continue;
                acc[(((size_t)b * oc + o) * oh + oy) * ow + ox] += a * (double)filter[(((size_t)o * icg + c) * kh + r) * kw + q];
              }
            }
          }
    }
  for (int b = 0; b < n; ++b)
    for (int o = 0; o < oc; ++o)
      for (int i = 0; i < oh * ow; ++i) {
        const size_t oi = ((size_t)b * oc + o) * oh * ow + i;
        float v = (float)(acc[oi] + (bias ? (double)bias[o] : 0.0));
        if (do_relu && v < 0) v = 0;
        out[oi] = to_bf16 ? orc_bf16(v, 1) : v;
      }
}

// MatMul of two activations (core/matmul.cpp:33-97; dimensions per TPUOperationSupport.cpp:615-655).
// The transposes only change where element (batch, row, col) is stored: [bh, rows, bl, cols] instead of
// [bh, bl, rows, cols]. mode 0 INT8 (QDM requant unless multiplier and rshift are both 0), 1 fp32, 2 BF16.
static inline size_t orc_mm_index(int trans, int bh, int bl, int nbl, int rows, int cols, int r, int c) {
  return trans ? (((size_t)bh * rows + r) * nbl + bl) * cols + c : (((size_t)bh * nbl + bl) * rows + r) * cols + c;
}
void orc_matmul(const float *left, const float *right, float *out, int nbh, int nbl, int M, int K, int N, int ltrans,
                int rtrans, int otrans, int do_relu, int mode, float rshift, float multiplier) {
#pragma omp parallel for collapse(2)
  for (int b = 0; b < nbh * nbl; ++b)
    for (int m = 0; m < M; ++m) {
      const int bh = b / nbl, bl = b % nbl;
      for (int n = 0; n < N; ++n) {
        double acc = 0;
        for (int k = 0; k < K; ++k)
          acc += (double)left[orc_mm_index(ltrans, bh, bl, nbl, M, K, m, k)] *
                 (double)right[orc_mm_index(rtrans, bh, bl, nbl, K, N, k, n)];
        float v = (float)acc;
        if (do_relu && v < 0) v = 0;
        if (mode == 0) {
          if (rshift != 0 || multiplier != 0) v = (float)orc_qdm_f32(v, (uint32_t)rshift, (uint32_t)multiplier);
        } else if (mode == 2) {
          v = orc_bf16(v, 1);
        }
        out[orc_mm_index(otrans, bh, bl, nbl, M, N, m, n)] = v;
      }
    }
}

} // extern "C"
