// C-callable shims over the UNMODIFIED reference arithmetic sources
// (QuantizationArithmetic.cpp, core/lut_func.cpp), which are compiled from
// where they lie in the reference checkout into oracle/_ref/. Test
// infrastructure only: used to pin the oracle restatement and to generate the
// golden vectors under tests/golden/.
#include "tpuc/QuantizationArithmetic.h"
#include "tpuc/Interpreter/cpu/lut_func.hpp"
#include <string>
#include <vector>

extern "C" {
int ref_qdm_i32(int32_t v, uint32_t rshift, uint32_t multiplier) {
  return mlir::applyMultiplierAndRShiftAndSaturateInt8(v, rshift, multiplier, true);
}
int ref_qdm_f32(float v, uint32_t rshift, uint32_t multiplier) {
  return mlir::applyMultiplierAndRShiftAndSaturateInt8(v, rshift, multiplier, true);
}
int ref_mul_rshift_f32(float v, uint32_t rshift, uint32_t multiplier) {
  return mlir::applyMultiplierAndRShiftAndSaturateInt8(v, rshift, multiplier, false);
}
int ref_rshift_f32(float v, uint32_t rshift) {
  return mlir::applyRShiftAndSaturateInt8(v, rshift);
}
uint16_t ref_f32_to_bf16(float v, int rounding) { return mlir::F32ToBF16(v, rounding != 0); }
float ref_bf16(float v, int rounding) { return mlir::BF16(v, rounding != 0); }
int ref_f32_to_int8(float v, int round_mode) { return mlir::F32ToInt8(v, round_mode); }
void ref_requant_per_channel(float *output, float *input, float *bias, int do_relu,
                             int64_t on, int64_t oc, int64_t isz, float *rshift,
                             float *multiplier) {
  mlir::quantizeActivationInt8PerChannelMultiplierAndRShift(
      output, input, bias, do_relu != 0, on, oc, isz, rshift, multiplier);
}
void ref_lut_gen_slope_tables(const char *name, float p0, float p1, float *base, float *slope) {
  float rs, re;
  bf16_gen_base_slope_table(name, base, slope, rs, re, p0, p1);
}
void ref_lut_bf16_slope(const char *name, float *in, float *out, int size, float *base,
                        float *slope) {
  bf16_lut_slope(name, in, out, size, base, slope);
}
void ref_lut_gen_expmant_tables(const char *name, float p0, float *exp_table, float *mant) {
  bf16_gen_exponent_mantissa_table(name, exp_table, mant, p0, 0.0f);
}
void ref_lut_bf16_mantissa(float *in, float *out, int size, float *exp_table, float *mant) {
  bf16_lut_mantissa(in, out, size, exp_table, mant, "mantissa");
}
void ref_lut_bf16_mantissa_log(float *in, float *out, int size, float *exp_table, float *mant) {
  bf16_lut_mantissa(in, out, size, exp_table, mant, "log");
}
// Weight quantisers the auto-tuner re-runs per candidate threshold (QuantizationArithmetic.cpp:630-818).
void ref_quantize_weight_int8_multiplier(float *filter, float *bias, int64_t oc, int64_t isz,
                                         float threshold_y, float threshold_x, float *new_filter,
                                         float *new_bias, float *rshift, float *multiplier) {
  std::vector<float> none;
  mlir::quantizeWeightInt8Multiplier(filter, bias, oc, isz, threshold_y, threshold_x, new_filter,
                                     new_bias, rshift, multiplier, none);
}
void ref_quantize_weight_int8_fc(float *filter, float *bias, int64_t n, int64_t k, float threshold_y,
                                 float threshold_x, float *new_filter, float *new_bias,
                                 float *rshift, float *multiplier) {
  mlir::quantizeWeightInt8ForFC(filter, bias, 1, n, k, threshold_y, threshold_x, new_filter, new_bias,
                                rshift, multiplier);
}
// The (rshift, int8 multipliers) of quantizeInt8RescaleNoWeightOps (QuantizeInt8.cpp:798-815).
int ref_rescale_no_weight(const float *qscale, int n, float *multipliers) {
  float max_qscale = 0.0f;
  for (int i = 0; i < n; ++i) {
    float p = qscale[i] > 0.0f ? qscale[i] : 0.0f - qscale[i];
    if (max_qscale < p) max_qscale = p;
  }
  int8_t rshift = mlir::findRShiftAndMultiplierFromQScale(max_qscale);
  for (int i = 0; i < n; ++i)
    multipliers[i] = (float)mlir::findMultiplierI8FromQScaleAndRShift(qscale[i], rshift);
  return rshift;
}
}
