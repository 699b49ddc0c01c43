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
  int type; // 0 mean, 1 sum, 2 max, 3 min
  int dt;   // DT_I8 or DT_F32
  int mult, rshift, requant;
};
__global__ void reduce_kernel(const void *__restrict__ in, void *__restrict__ out, ReduceArgs p) {
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
        if (p.type <= 1) v = __fadd_rn(v, x);
        else if (a == 0) v = x;
        else v = p.type == 2 ? fmaxf(v, x) : fminf(v, x);
      }
      if (p.type == 0) v = __fdiv_rn(v, (float)p.axis);
      reinterpret_cast<float *>(out)[po] = v;
    }
  }
}

} // namespace tpucb
