// Layout and arithmetic kernels of the networks next to the benchmark graphs: eltwise max / min,
// broadcast add / sub / mul, pad, crop, permute and reduce. Reference bodies restated here
// (lib/Dialect/TPU/Interpreter/core/): eltwise.cpp:143-181,225-263, broadcast.cpp:45-156,
// pad.cpp:7-141, crop.cpp:18-92, permute.cpp:6-33, reduce.cpp:52-115.
//
// The reference indexes fp32 NCHW containers by their flat row-major index; device tensors are NHWC
// with a padded channel pitch, so every kernel here maps a logical flat index to the physical offset
// of its tensor (phys_offset) and is written per output element. They are HBM-bound gathers whose
// reads are strided in the general case; none of them is on the path of the benchmark graphs.
#pragma once
#include "mem_kernels.cuh"

namespace tpucb {

// physical element offset of the logical (row-major NCHW) flat index of a tensor
__device__ __forceinline__ size_t phys_offset(const TensorGeom &g, size_t flat) {
  const int w = (int)(flat % g.w);
  size_t t = flat / g.w;
  const int h = (int)(t % g.h);
  t /= g.h;
  const int c = (int)(t % g.c);
  const int n = (int)(t / g.c);
  return (((size_t)n * g.h + h) * g.wphys + g.wl + w) * g.cp + c;
}
__device__ __forceinline__ size_t phys_offset4(const TensorGeom &g, int n, int c, int h, int w) {
  return (((size_t)n * g.h + h) * g.wphys + g.wl + w) * g.cp + c;
}
__device__ __forceinline__ float load_elem(const void *p, int dt, size_t off) { return load_as_f32(p, dt, off); }

// ---------------------------------------------------------------- eltwise max / min (INT8)
struct MaxMinArgs {
  const int8_t *in[4];
  int mult[4];
  int nin, rshift, do_relu, is_min;
};
__global__ void eltwise_maxmin_i8_kernel(MaxMinArgs a, int8_t *__restrict__ out, size_t nvec) {
  pdl_prologue();
  const int rnd = a.rshift > 0 ? (1 << (a.rshift - 1)) : 0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    int v[16];
    {
      const uint4 x = reinterpret_cast<const uint4 *>(a.in[0])[i];
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        v[4 * q + 0] = sext_byte<0>(w[q]) * a.mult[0];
        v[4 * q + 1] = sext_byte<1>(w[q]) * a.mult[0];
        v[4 * q + 2] = sext_byte<2>(w[q]) * a.mult[0];
        v[4 * q + 3] = sext_byte<3>(w[q]) * a.mult[0];
      }
    }
    for (int k = 1; k < a.nin; ++k) {
      const uint4 x = reinterpret_cast<const uint4 *>(a.in[k])[i];
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
      const int m = a.mult[k];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int e[4] = {sext_byte<0>(w[q]) * m, sext_byte<1>(w[q]) * m, sext_byte<2>(w[q]) * m, sext_byte<3>(w[q]) * m};
#pragma unroll
        for (int j = 0; j < 4; ++j) v[4 * q + j] = a.is_min ? min(v[4 * q + j], e[j]) : max(v[4 * q + j], e[j]);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      int e[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int t = v[4 * q + j];
        if (a.do_relu) t = max(t, 0);
        e[j] = (t + rnd) >> a.rshift;
      }
      o[q] = pack4_sat(e[0], e[1], e[2], e[3]);
    }
    reinterpret_cast<uint4 *>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---------------------------------------------------------------- broadcast add / sub / mul
struct BroadcastArgs {
  TensorGeom ga, gb, go;
  int sa[4], sb[4], so[4]; // the reference's 4-D (right-aligned) shapes
  int op;                  // 0 add, 1 sub, 2 mul
  int dt;                  // DT_I8 or DT_F32 (all three tensors)
  int mult0, mult1, rshift, do_relu;
};
__global__ void broadcast_kernel(const void *__restrict__ a, const void *__restrict__ b, void *__restrict__ out,
                                 BroadcastArgs p) {
  pdl_prologue();
  const size_t total = (size_t)p.so[0] * p.so[1] * p.so[2] * p.so[3];
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int w = (int)(i % p.so[3]);
    size_t t = i / p.so[3];
    const int h = (int)(t % p.so[2]);
    t /= p.so[2];
    const int c = (int)(t % p.so[1]);
    const int n = (int)(t / p.so[1]);
    const size_t ia = (((size_t)(p.sa[0] == 1 ? 0 : n) * p.sa[1] + (p.sa[1] == 1 ? 0 : c)) * p.sa[2] + (p.sa[2] == 1 ? 0 : h)) * p.sa[3] +
                      (p.sa[3] == 1 ? 0 : w);
    const size_t ib = (((size_t)(p.sb[0] == 1 ? 0 : n) * p.sb[1] + (p.sb[1] == 1 ? 0 : c)) * p.sb[2] + (p.sb[2] == 1 ? 0 : h)) * p.sb[3] +
                      (p.sb[3] == 1 ? 0 : w);
    const size_t po = phys_offset(p.go, i);
    if (p.dt == DT_I8) {
      const int x = reinterpret_cast<const int8_t *>(a)[phys_offset(p.ga, ia)];
      const int y = reinterpret_cast<const int8_t *>(b)[phys_offset(p.gb, ib)];
      int q;
      if (p.op == 2) {
        int v = x * y;
        if (p.do_relu) v = max(v, 0);
        q = qdm_requant(v, p.mult0, p.rshift);
      } else {
        int v = p.op == 0 ? x * p.mult0 + y * p.mult1 : x * p.mult0 - y * p.mult1;
        if (p.do_relu) v = max(v, 0);
        q = rshift_sat8(v, p.rshift);
      }
      reinterpret_cast<int8_t *>(out)[po] = (int8_t)q;
    } else {
      const float x = reinterpret_cast<const float *>(a)[phys_offset(p.ga, ia)];
      const float y = reinterpret_cast<const float *>(b)[phys_offset(p.gb, ib)];
      float v = p.op == 0 ? __fadd_rn(x, y) : (p.op == 1 ? __fsub_rn(x, y) : __fmul_rn(x, y));
      if (p.do_relu) v = fmaxf(v, 0.0f);
      reinterpret_cast<float *>(out)[po] = v;
    }
  }
}

// ---------------------------------------------------------------- pad / crop / permute
struct RemapArgs {
  TensorGeom gi, go;
  int si[4], so[4]; // logical 4-D shapes of input and output
  int mode;         // 0 pad constant (negative pads cut), 1 pad edge, 2 crop, 3 permute
  int a[4];         // pad: begin pads; crop: offsets; permute: order
  int b[4];         // crop: steps
  int es;           // element size in bytes
};
__global__ void remap_kernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out, RemapArgs p) {
  pdl_prologue();
  const size_t total = (size_t)p.so[0] * p.so[1] * p.so[2] * p.so[3];
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    int o[4];
    o[3] = (int)(i % p.so[3]);
    size_t t = i / p.so[3];
    o[2] = (int)(t % p.so[2]);
    t /= p.so[2];
    o[1] = (int)(t % p.so[1]);
    o[0] = (int)(t / p.so[1]);
    int s[4];
    bool inside = true;
    if (p.mode <= 1) {
#pragma unroll
      for (int d = 0; d < 4; ++d) s[d] = o[d] - p.a[d];
      if (p.mode == 1) {
        s[2] = min(max(s[2], 0), p.si[2] - 1);
        s[3] = min(max(s[3], 0), p.si[3] - 1);
      }
#pragma unroll
      for (int d = 0; d < 4; ++d) inside = inside && s[d] >= 0 && s[d] < p.si[d];
    } else if (p.mode == 2) {
#pragma unroll
      for (int d = 0; d < 4; ++d) s[d] = o[d] * p.b[d] + p.a[d];
    } else {
      // output dimension k is input dimension order[k]
#pragma unroll
      for (int d = 0; d < 4; ++d) s[d] = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
#pragma unroll
        for (int d = 0; d < 4; ++d)
          if (p.a[k] == d) s[d] = o[k];
      }
    }
    const size_t po = phys_offset(p.go, i) * p.es;
    if (inside) {
      const size_t flat = (((size_t)s[0] * p.si[1] + s[1]) * p.si[2] + s[2]) * p.si[3] + s[3];
      const size_t pi = phys_offset(p.gi, flat) * p.es;
      for (int k = 0; k < p.es; ++k) out[po + k] = in[pi + k];
    } else {
      for (int k = 0; k < p.es; ++k) out[po + k] = 0;
    }
  }
}

// ---------------------------------------------------------------- reduce over consecutive axes
struct ReduceArgs {
  TensorGeom gi, go;
  int outer, axis, inner;
  int type; // 0 mean, 1 sum, 2 max, 3 min, 4 l2 (fp32 only: (sum of squares) ^ coeff)
  int dt;   // DT_I8 or DT_F32
  int mult, rshift, requant;
  float coeff;
};
__global__ void reduce_kernel(const void *__restrict__ in, void *__restrict__ out, ReduceArgs p) {
  pdl_prologue();
  const size_t total = (size_t)p.outer * p.inner;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % p.inner);
    const size_t o = idx / p.inner;
    const size_t po = phys_offset(p.go, idx);
    if (p.dt == DT_I8) {
      int v = 0;
      for (int a = 0; a < p.axis; ++a) {
        const int x = reinterpret_cast<const int8_t *>(in)[phys_offset(p.gi, (o * p.axis + a) * p.inner + i)];
        if (p.type <= 1) v += x;
        else if (a == 0) v = x;
        else v = p.type == 2 ? max(v, x) : min(v, x);
      }
      // without a rescale the reference stores the raw value in its fp32 container; int8 storage saturates
      reinterpret_cast<int8_t *>(out)[po] = (int8_t)(p.requant ? mul_rshift_sat8(v, p.mult, p.rshift) : clamp_i8(v));
    } else {
      float v = 0.0f;
      for (int a = 0; a < p.axis; ++a) {
        const float x = reinterpret_cast<const float *>(in)[phys_offset(p.gi, (o * p.axis + a) * p.inner + i)];
        // l2 (core/reduce.cpp:91-103): `sum += std::pow(x, 2)` squares in double (exact) and rounds the sum to fp32
        if (p.type == 4) v = __double2float_rn((double)v + (double)x * (double)x);
        else if (p.type <= 1) v = __fadd_rn(v, x);
        else if (a == 0) v = x;
        else v = p.type == 2 ? fmaxf(v, x) : fminf(v, x);
      }
      if (p.type == 0) v = __fdiv_rn(v, (float)p.axis);
      if (p.type == 4) v = powf(v, p.coeff);
      reinterpret_cast<float *>(out)[po] = v;
    }
  }
}

// ------------------------------------------------------------------ BF16 element-wise / pooling
// BF16 tensors hold 8 values per 16-byte vector (channel pitch a multiple of 16 values).
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// ReLU and leaky ReLU of BF16 tensors (core/activation.cpp:150-152, 168-180): x > 0 ? x : x * slope in fp32 and one
// BF16 rounding; slope 0 is the plain ReLU (the product rounds to a signed zero, which the reference's relu() writes as
// +0: handled apart). Eight values per thread.
__global__ void leaky_relu_bf16_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out, size_t nvec, float slope,
                                       int plain_relu) {
  pdl_prologue();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = __ldg(in + i);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t r = 0;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint16_t bits = (uint16_t)(w[q] >> (16 * h));
        const float x = bf16_bits_to_f32(bits);
        uint16_t y;
        if (x > 0.0f) y = bits;
        else if (plain_relu) y = 0;
        else y = f32_to_bf16_bits(__fmul_rn(x, slope));
        r |= (uint32_t)y << (16 * h);
      }
      w[q] = r;
    }
    out[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// Grouped and depthwise BF16 convolution (core/conv.cpp:90-98 with g > 1: the fp32 convolution of BF16-valued operands,
// fp32 bias, ReLU, one BF16 rounding) and, through input insertion (ins_h / ins_w zeros between the input pixels), the
// BF16 deconvolution (core/deconv.cpp:56-68). One thread per output value, fp32 accumulation over (filter row, filter
// column, input channel of the group); consecutive threads take consecutive output channels, so the stores and, for
// depthwise layers, the loads are coalesced. Weights as fp32 [oc][kh][kw][ic / g].
struct ConvBf16GroupArgs {
  int n, ic, icp, ih, iw, oc, ocp, oh, ow, kh, kw, sh, sw, pt, pl, dh, dw, g, do_relu, ins_h, ins_w;
};
__global__ void conv_bf16_grouped_kernel(const uint16_t *__restrict__ in, const float *__restrict__ w,
                                         const float *__restrict__ bias, uint16_t *__restrict__ out, ConvBf16GroupArgs a) {
  pdl_prologue();
  const int icg = a.ic / a.g, ocg = a.oc / a.g;
  const size_t total = (size_t)a.n * a.oh * a.ow * a.ocp;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int o = (int)(i % a.ocp);
    const size_t pix = i / a.ocp;
    uint16_t r = 0;
    if (o < a.oc) {
      const int x = (int)(pix % a.ow);
      const size_t t = pix / a.ow;
      const int y = (int)(t % a.oh);
      const int b = (int)(t / a.oh);
      const int c0 = (o / ocg) * icg;
      const float *wo = w + (size_t)o * a.kh * a.kw * icg;
      float acc = 0.0f;
      for (int kr = 0; kr < a.kh; ++kr) {
        int yy = y * a.sh - a.pt + kr * a.dh; // row of the zero-inserted input
        if (yy < 0 || yy % (a.ins_h + 1) != 0) continue;
        yy /= a.ins_h + 1;
        if (yy >= a.ih) continue;
        for (int ks = 0; ks < a.kw; ++ks) {
          int xx = x * a.sw - a.pl + ks * a.dw;
          if (xx < 0 || xx % (a.ins_w + 1) != 0) continue;
          xx /= a.ins_w + 1;
          if (xx >= a.iw) continue;
          const uint16_t *src = in + (((size_t)b * a.ih + yy) * a.iw + xx) * a.icp + c0;
          const float *wt = wo + (size_t)(kr * a.kw + ks) * icg;
          for (int c = 0; c < icg; ++c) acc = fmaf(bf16_bits_to_f32(src[c]), wt[c], acc);
        }
      }
      acc = __fadd_rn(acc, bias[o]);
      if (a.do_relu && acc < 0.0f) acc = 0.0f;
      r = f32_to_bf16_bits(acc);
    }
    out[i] = r;
  }
}

struct EltwiseBf16Args {
  const uint4 *in[4];
  float coeff[4];
  int nin;
  int do_relu;
};
// EltwiseAddOpKernel / EltwiseMulOpKernel in BF16 (core/eltwise.cpp:41-52, 101-104, 320-333): the fp32
// form, operand by operand from 0 (add) or 1 (mul), product and sum rounded separately, ReLU, then one
// BF16 rounding of the result.
template <bool MUL> __global__ void eltwise_bf16_kernel(EltwiseBf16Args a, uint4 *__restrict__ out, size_t nvec) {
  pdl_prologue();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = MUL ? 1.0f : 0.0f;
    for (int k = 0; k < a.nin; ++k) {
      const uint4 v = __ldg(a.in[k] + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      const float co = a.coeff[k];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = bf16_lo(w[j]), hi = bf16_hi(w[j]);
        if (MUL) {
          acc[2 * j] = __fmul_rn(acc[2 * j], lo);
          acc[2 * j + 1] = __fmul_rn(acc[2 * j + 1], hi);
        } else {
          acc[2 * j] = __fadd_rn(acc[2 * j], __fmul_rn(co, lo));
          acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __fmul_rn(co, hi));
        }
      }
    }
    if (a.do_relu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = acc[j] > 0.0f ? acc[j] : 0.0f;
    }
    uint4 o;
    o.x = bf16x2_round_bits(acc[0], acc[1]);
    o.y = bf16x2_round_bits(acc[2], acc[3]);
    o.z = bf16x2_round_bits(acc[4], acc[5]);
    o.w = bf16x2_round_bits(acc[6], acc[7]);
    out[i] = o;
  }
}

// PoolingOpKernel in BF16 (core/pooling.cpp:91-94): the fp32 pooling on BF16 values. The maximum of
// BF16 values is a BF16 value; the average (sum over the valid taps in row order, divided by kh*kw
// or by the number of valid taps) is rounded to BF16 when stored, where the reference's fp32
// container keeps the unrounded quotient: at most half a BF16 ulp apart.
__global__ void pool_bf16_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out, PoolArgs a, int count_include_pad) {
  pdl_prologue();
  const int vecs = a.cp / 8;
  const size_t total = (size_t)a.n * a.oh * a.ow * vecs;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vecs);
    size_t pix = i / vecs;
    const int x = (int)(pix % a.ow);
    size_t t = pix / a.ow;
    const int y = (int)(t % a.oh);
    const int b = (int)(t / a.oh);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = a.method == 0 ? -INFINITY : 0.0f;
    int cnt = 0;
    for (int r = 0; r < a.kh; ++r) {
      const int yy = y * a.sh - a.pt + r;
      if (yy < 0 || yy >= a.ih) continue;
      for (int s = 0; s < a.kw; ++s) {
        const int xx = x * a.sw - a.pl + s;
        if (xx < 0 || xx >= a.iw) continue;
        const uint4 q = __ldg(in + (((size_t)b * a.ih + yy) * a.iw + xx) * vecs + v);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = bf16_lo(w[j]), hi = bf16_hi(w[j]);
          if (a.method == 0) {
            acc[2 * j] = fmaxf(acc[2 * j], lo);
            acc[2 * j + 1] = fmaxf(acc[2 * j + 1], hi);
          } else {
            acc[2 * j] = __fadd_rn(acc[2 * j], lo);
            acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], hi);
          }
        }
        ++cnt;
      }
    }
    if (a.method != 0) {
      const float d = (float)(count_include_pad ? a.kh * a.kw : cnt);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __fdiv_rn(acc[j], d);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v * 8 + j >= a.c) acc[j] = 0.0f;
    uint4 o;
    o.x = bf16x2_round_bits(acc[0], acc[1]);
    o.y = bf16x2_round_bits(acc[2], acc[3]);
    o.z = bf16x2_round_bits(acc[4], acc[5]);
    o.w = bf16x2_round_bits(acc[6], acc[7]);
    out[i] = o;
  }
}

// ----------------------------------------------------------------------- matmul (two activations)
// MatMulOpKernel (core/matmul.cpp:33-97): out[b] = left[b] (M x K) * right[b] (K x N) over
// batch = batch_high * batch_low, optional ReLU, then QDM requantisation with one (multiplier, rshift)
// pair (INT8, skipped when both are zero), one BF16 rounding (BF16) or nothing (fp32). The transposes
// are storage orders, not arithmetic: left [bh, M, bl, K], right [bh, K, bl, N], out [bh, M, bl, N]
// instead of [bh, bl, rows, cols]. Both operands are activations, so neither is packed beforehand:
// 16 x 16 tiles of each are staged in shared memory through the tensors' own geometry.
struct MatMulArgs {
  TensorGeom ga, gb, go;
  int bh, bl, M, K, N;
  int lt, rt, ot;
  int dt, do_relu, mult, rshift, requant;
};
__device__ __forceinline__ size_t matmul_index(int trans, int bh, int bl, int nbl, int rows, int cols, int r, int c) {
  return trans ? (((size_t)bh * rows + r) * nbl + bl) * cols + c : (((size_t)bh * nbl + bl) * rows + r) * cols + c;
}
template <int DT> __global__ void matmul_kernel(const void *__restrict__ a, const void *__restrict__ b, void *__restrict__ out, MatMulArgs p) {
  pdl_prologue();
  __shared__ float As[16][17], Bs[16][17];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int bh = blockIdx.z / p.bl, bl = blockIdx.z % p.bl;
  const int m = blockIdx.y * 16 + ty, n = blockIdx.x * 16 + tx;
  float accf = 0.0f;
  int acci = 0;
  for (int k0 = 0; k0 < p.K; k0 += 16) {
    float av = 0.0f, bv = 0.0f;
    if (m < p.M && k0 + tx < p.K) av = load_as_f32(a, DT, phys_offset(p.ga, matmul_index(p.lt, bh, bl, p.bl, p.M, p.K, m, k0 + tx)));
    if (k0 + ty < p.K && n < p.N) bv = load_as_f32(b, DT, phys_offset(p.gb, matmul_index(p.rt, bh, bl, p.bl, p.K, p.N, k0 + ty, n)));
    As[ty][tx] = av;
    Bs[ty][tx] = bv;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      if (DT == DT_I8) acci += (int)As[ty][k] * (int)Bs[k][tx];
      else accf = fmaf(As[ty][k], Bs[k][tx], accf);
    }
    __syncthreads();
  }
  if (m >= p.M || n >= p.N) return;
  const size_t po = phys_offset(p.go, matmul_index(p.ot, bh, bl, p.bl, p.M, p.N, m, n));
  if (DT == DT_I8) {
    if (p.do_relu) acci = max(acci, 0);
    const int q = p.requant ? qdm_requant(acci, p.mult, p.rshift) : clamp_i8(acci);
    reinterpret_cast<int8_t *>(out)[po] = (int8_t)q;
  } else {
    if (p.do_relu) accf = fmaxf(accf, 0.0f);
    if (DT == DT_BF16) reinterpret_cast<uint16_t *>(out)[po] = f32_to_bf16_bits(accf);
    else reinterpret_cast<float *>(out)[po] = accf;
  }
}

// ------------------------------------------------------------ batched INT8 inner product
// FullyConnectedOpKernel with a filter of rank 3 (core/fullyconnected.cpp:59-88; parseFullyConnectedParam,
// lib/Dialect/TPU/IR/TPUOperationSupport.cpp:569-605): `batch` independent products Y[b] = X[b] (m x k) * W[b]^T
// (n x k) + bias[b], ReLU on the sum, then the QDM requantisation with ONE (multiplier, rshift) pair PER BATCH
// index. The rank-3 activations [batch, m, k] and [batch, m, n] sit in the device layout with m on the channel axis
// (pitch mp): consecutive threads take consecutive rows m, so both the reads and the writes are coalesced. The
// weights are int8 [batch][n][k]. An integer loop on the FMA / integer pipe: graphs with this op (attention-style
// products against constant matrices) are not on a benchmark path.
__global__ void fc_batched_i8_kernel(const int8_t *__restrict__ x, const int8_t *__restrict__ w, const int32_t *__restrict__ bias,
                                     const int32_t *__restrict__ mult, const int32_t *__restrict__ rshift,
                                     int8_t *__restrict__ y, int batch, int m, int k, int n, int mp, int do_relu) {
  pdl_prologue();
  const size_t total = (size_t)batch * n * mp;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % mp);
    const size_t bj = idx / mp;
    const int j = (int)(bj % n), b = (int)(bj / n);
    int v = 0;
    if (i < m) {
      int acc = bias ? bias[(size_t)b * n + j] : 0;
      const int8_t *xr = x + (size_t)b * k * mp + i;
      const int8_t *wr = w + ((size_t)b * n + j) * k;
      for (int t = 0; t < k; ++t) acc += (int)xr[(size_t)t * mp] * (int)wr[t];
      if (do_relu) acc = max(acc, 0);
      v = qdm_requant(acc, mult[b], rshift[b]);
    }
    y[idx] = (int8_t)v;
  }
}

// ----------------------------------------------------------------------------- BF16 softmax
// SoftmaxOpKernel::invoke_bf16 (core/softmax.cpp:88-151) over the channel axis, one pixel per CTA:
// max, BF16(x - max), exp through the 256-entry slope table (lut_func.cpp:169-186, range 15),
// sum_j ex_j * BF16(BF16(C)/C), reciprocal (or logarithm, do_log) of the BF16-rounded sum through the
// exponent / mantissa tables (lut_func.cpp:306-333), BF16(ex * 1/sum) or BF16(sub - log sum).
// The reference accumulates the sum in fp32 in channel order and rounds it once; an fp32 sum depends on
// its order, so one thread adds the channels in that order from shared memory (4 cycles per add:
// 2 us for 1000 channels) while every other step is spread over the CTA.
struct SoftmaxBf16Args {
  const float *exp_base, *exp_slope, *rec_exp, *rec_mant;
  int c, cp, do_log;
  float lut_scale, const_val;
};
__global__ void softmax_bf16_kernel(const uint16_t *__restrict__ in, uint16_t *__restrict__ out, SoftmaxBf16Args a) {
  pdl_prologue();
  extern __shared__ float sm_buf[]; // sub[c], ex[c]
  __shared__ float red[32];
  __shared__ float s_r;
  float *sub = sm_buf, *ex = sm_buf + a.c;
  const uint16_t *p = in + (size_t)blockIdx.x * a.cp;
  uint16_t *q = out + (size_t)blockIdx.x * a.cp;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < a.c; i += blockDim.x) {
    const float x = bf16_bits_to_f32(p[i]);
    sub[i] = x;
    mx = fmaxf(mx, x);
  }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for (int i = 1; i < (int)(blockDim.x >> 5); ++i) mx = fmaxf(mx, red[i]);
  for (int i = threadIdx.x; i < a.c; i += blockDim.x) {
    const float d = bf16_round(__fsub_rn(sub[i], mx));
    sub[i] = d;
    const float r = bf16_round(__fmul_rn(d, a.lut_scale));
    const int idx = f32_to_int8_rz(r);
    const float dx = bf16_round(__fsub_rn(r, (float)idx));
    ex[i] = bf16_round(__fadd_rn(__ldg(a.exp_base + (idx & 0xff)), __fmul_rn(dx, __ldg(a.exp_slope + (idx & 0xff)))));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float sum = 0.0f;
    for (int j = 0; j < a.c; ++j) sum = __fadd_rn(sum, __fmul_rn(ex[j], a.const_val));
    const uint32_t h = f32_to_bf16_bits(sum);
    const float v = bf16_bits_to_f32((uint16_t)h);
    int e;
    if (v == 0.0f) e = 0;
    else {
      e = (int)((h >> 7) & 0xff) - 127 + 63 + ((h & 0x8000u) ? 128 : 0); // floor(log2 |v|) of a normal value
      e = min(max(e, 0), 255);
    }
    const float te = __ldg(a.rec_exp + e), tm = __ldg(a.rec_mant + (h & 0xff));
    s_r = bf16_round(a.do_log ? __fadd_rn(te, tm) : __fmul_rn(te, tm));
  }
  __syncthreads();
  const float r = s_r;
  for (int i = threadIdx.x; i < a.cp; i += blockDim.x) {
    float y = 0.0f;
    if (i < a.c) y = a.do_log ? __fsub_rn(sub[i], r) : __fmul_rn(ex[i], r);
    q[i] = f32_to_bf16_bits(y);
  }
}

} // namespace tpucb
