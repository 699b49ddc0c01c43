// Calibration statistics on device.
//   minmax_f32_kernel  find_min_max_abs          python/cvi_toolkit/calibration/kld_calibrator.py:269-296
//   hist_f32_kernel    BaseKldCalibrator.histogram                       kld_calibrator.py:31-43
//   kld_kernel         kl_diversity_hist / kl_calc_thread   bindings/python/kld/calibration_math.cpp:169-223, 283-344
//   tuner_distance_kernel  the two norms of SimpleTuner.run                  kld_calibrator.py:184-196
// Tensors are fp32 NHWC with channel pitch cp; padded lanes are skipped.
#pragma once
#include "common.cuh"

namespace tpucb {

__device__ __forceinline__ void atomic_max_f32(float *addr, float v) {
  if (v >= 0) atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}
__device__ __forceinline__ void atomic_min_f32(float *addr, float v) {
  if (v >= 0) atomicMin(reinterpret_cast<int *>(addr), __float_as_int(v));
  else atomicMax(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

// stats[0] = running min, stats[1] = running max. With `keep` the real lanes are also written to a second buffer of the
// same layout in the same pass (the copy the histogram pass reads when the activations of all batches stay resident).
__global__ void minmax_f32_kernel(const float *__restrict__ x, size_t pixels, int c, int cp, float *stats,
                                  float *__restrict__ keep) {
  pdl_prologue();
  float mn = INFINITY, mx = -INFINITY;
  const size_t total = pixels * (size_t)cp;
  if ((cp & 3) == 0 && (c & 3) == 0) {
    const size_t nvec = total / 4;
    const int vpp = cp / 4, vreal = c / 4;
    const bool dense = vreal == vpp; // no padded channels: no position arithmetic at all
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    float4 *k4 = reinterpret_cast<float4 *>(keep);
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    // four independent 16-byte loads in flight per thread (padded lanes hold zeros and are masked after the load)
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      float4 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = __ldg(x4 + i + k * stride);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (!dense && (int)((i + k * stride) % vpp) >= vreal) continue;
        if (keep) k4[i + k * stride] = v[k];
        mn = fminf(fminf(mn, v[k].x), fminf(fminf(v[k].y, v[k].z), v[k].w));
        mx = fmaxf(fmaxf(mx, v[k].x), fmaxf(fmaxf(v[k].y, v[k].z), v[k].w));
      }
    }
    for (; i < nvec; i += stride) {
      if (!dense && (int)(i % vpp) >= vreal) continue;
      float4 v = __ldg(x4 + i);
      if (keep) k4[i] = v;
      mn = fminf(fminf(mn, v.x), fminf(fminf(v.y, v.z), v.w));
      mx = fmaxf(fmaxf(mx, v.x), fmaxf(fmaxf(v.y, v.z), v.w));
    }
  } else {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
      if ((int)(i % cp) >= c) continue;
      float v = x[i];
      if (keep) keep[i] = v;
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  __shared__ float smn[32], smx[32];
  if ((threadIdx.x & 31) == 0) {
    smn[threadIdx.x >> 5] = mn;
    smx[threadIdx.x >> 5] = mx;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) {
      mn = fminf(mn, smn[i]);
      mx = fmaxf(mx, smx[i]);
    }
    if (mn <= mx) {
      atomic_min_f32(stats, mn);
      atomic_max_f32(stats + 1, mx);
    }
  }
}

// bins <= 4096. idx = floor(|x| / width + 0.5) in fp32 for x != 0; CTA-private shared histogram with
// warp-aggregated atomics (lanes that hit the same bin elect one adder), flushed with 64-bit atomics.
__global__ void hist_f32_kernel(const float *__restrict__ x, size_t pixels, int c, int cp, float width, int bins,
                                unsigned long long *__restrict__ hist) {
  pdl_prologue();
  extern __shared__ unsigned int s_h[];
  for (int i = threadIdx.x; i < bins; i += blockDim.x) s_h[i] = 0;
  __syncthreads();
  const size_t total = pixels * (size_t)cp;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  if ((cp & 3) == 0 && (c & 3) == 0) {
    // 16-byte vectors, one shared-memory atomic per non-zero value: the bins of one warp's values are spread over
    // the table, so the few collisions cost less than electing one adder per bin did.
    const size_t nvec = total / 4;
    const int vpp = cp / 4, vreal = c / 4;
    const bool dense = vreal == vpp;
    const float top = (float)(bins - 1);
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += stride) {
      if (!dense && (int)(i % vpp) >= vreal) continue;
      const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + i);
      const float t4[4] = {fabsf(v.x), fabsf(v.y), fabsf(v.z), fabsf(v.w)};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (t4[k] != 0.0f) {
          const float f = floorf(__fadd_rn(__fdiv_rn(t4[k], width), 0.5f));
          if (f <= top) atomicAdd(&s_h[(int)f], 1u);
        }
      }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < bins; j += blockDim.x)
      if (s_h[j]) atomicAdd(&hist[j], (unsigned long long)s_h[j]);
    return;
  }
  const size_t rounds = (total + stride - 1) / stride;
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  for (size_t rd = 0; rd < rounds; ++rd, i += stride) {
    int b = -1;
    if (i < total && (int)(i % cp) < c) {
      float t = fabsf(x[i]);
      if (t != 0.0f) {
        float f = floorf(__fadd_rn(__fdiv_rn(t, width), 0.5f));
        if (f <= (float)(bins - 1)) b = (int)f;
      }
    }
    unsigned active = __ballot_sync(0xffffffffu, b >= 0);
    if (b >= 0) {
      unsigned peers = __match_any_sync(active, b);
      int leader = __ffs(peers) - 1;
      if ((int)(threadIdx.x & 31) == leader) atomicAdd(&s_h[b], (unsigned)__popc(peers));
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < bins; j += blockDim.x)
    if (s_h[j]) atomicAdd(&hist[j], (unsigned long long)s_h[j]);
}

// a / w, correctly rounded, for a divisor that is constant over many values: r = RN(1 / w) is taken once
// (quot_setup) and every quotient costs one multiply and four fused multiply-adds on the FMA pipe instead of the
// reciprocal unit and the fix-up code of a division. q0 = RN(a r) is within 1.5 ulp of a / w; the residual
// e = a - q0 w is exact in one FMA, so q1 = RN(q0 + e r) is a faithful quotient, and one more step from a faithful
// quotient with a correctly rounded reciprocal gives RN(a / w) (Markstein's theorem). That holds while nothing
// overflows or goes subnormal; quot_ok tells whether w is in the range (2^-60 .. 2^60) where this is so for every
// |a| <= 2^40 w that is either zero or at least 2^-60 (smaller quotients differ from the division's by less than
// 2^-80 and are used here only after 0.5 is added). Callers take the plain division when quot_ok is false.
__device__ __forceinline__ bool quot_ok(float w) { return w > 8.673617e-19f && w < 1.1529215e18f; }
__device__ __forceinline__ float quot_by_const(float a, float w, float r) {
  const float q0 = __fmul_rn(a, r);
  const float q1 = __fmaf_rn(__fmaf_rn(-q0, w, a), r, q0);
  return __fmaf_rn(__fmaf_rn(-q1, w, a), r, q1);
}

// ---- all tensors of a module in one launch ------------------------------------------------------------------------
// One descriptor per fp32 tensor (channel pitch a multiple of 4). The kernels below are persistent: every block walks
// the tensor list and takes its stripe of each tensor, so small tensors cost no launch of their own and the tail of
// one tensor overlaps the head of the next. Lanes past the real channel count are masked per value.
struct StatDesc {
  const float *x;           // the values (the tensor's storage, or its kept copy)
  float *keep;              // minmax only: where to copy the storage, or null
  unsigned long long nvec;  // 16-byte vectors in the storage
  int vpp;                  // vectors per pixel (channel pitch / 4)
  int c;                    // real channels
  float width;              // histogram only: bin width
  int pad_;
};

__global__ void __launch_bounds__(1024) minmax_multi_kernel(const StatDesc *__restrict__ descs, int count, float *stats) {
  pdl_prologue();
  __shared__ float smn[32], smx[32];
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (int t = 0; t < count; ++t) {
    const StatDesc d = descs[t];
    const float4 *x4 = reinterpret_cast<const float4 *>(d.x);
    float4 *k4 = reinterpret_cast<float4 *>(d.keep);
    const bool dense = d.c == d.vpp * 4;
    float mn = INFINITY, mx = -INFINITY;
    auto take = [&](const float4 &v, size_t i) {
      if (k4) k4[i] = v;
      if (dense) {
        mn = fminf(fminf(mn, v.x), fminf(fminf(v.y, v.z), v.w));
        mx = fmaxf(fmaxf(mx, v.x), fmaxf(fmaxf(v.y, v.z), v.w));
      } else {
        const int ch = (int)(i % d.vpp) * 4;
        const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (ch + k < d.c) {
            mn = fminf(mn, e[k]);
            mx = fmaxf(mx, e[k]);
          }
      }
    };
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    for (; i + 3 * stride < d.nvec; i += 4 * stride) {
      float4 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = __ldg(x4 + i + k * stride);
#pragma unroll
      for (int k = 0; k < 4; ++k) take(v[k], i + k * stride);
    }
    for (; i < d.nvec; i += stride) take(__ldg(x4 + i), i);
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) {
      smn[threadIdx.x >> 5] = mn;
      smx[threadIdx.x >> 5] = mx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
        mn = fminf(mn, smn[w]);
        mx = fmaxf(mx, smx[w]);
      }
      if (mn <= mx) {
        atomic_min_f32(stats + 2 * t, mn);
        atomic_max_f32(stats + 2 * t + 1, mx);
      }
    }
    __syncthreads();
  }
}

// hist [count][bins]; the bin rule of hist_f32_kernel.
__global__ void __launch_bounds__(1024) hist_multi_kernel(const StatDesc *__restrict__ descs, int count, int bins,
                                                           unsigned long long *__restrict__ hist) {
  pdl_prologue();
  extern __shared__ unsigned int s_h[];
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const float top = (float)bins;
  for (int t = 0; t < count; ++t) {
    const StatDesc d = descs[t];
    const float4 *x4 = reinterpret_cast<const float4 *>(d.x);
    const bool dense = d.c == d.vpp * 4;
    // the bin width is constant over the tensor: its reciprocal is taken once and every quotient is formed, still
    // correctly rounded, with multiply-adds (quot_by_const); widths outside its range keep the division
    const bool fast = quot_ok(d.width);
    const float rw = fast ? __frcp_rn(d.width) : 0.0f;
    for (int j = threadIdx.x; j < bins; j += blockDim.x) s_h[j] = 0;
    __syncthreads();
    // One value: branch-free up to the (predicated) shared-memory increment. A zero takes the arithmetic too and is
    // dropped by the predicate, which costs less than a divergent branch per value.
    auto one = [&](float x, bool in_range, auto quotient) {
      const float a = fabsf(x);
      // floor(f) <= bins - 1 is f < bins; for 0 <= f < 2^23 the round-down sum f + 2^23 carries floor(f) in its low
      // mantissa bits: no rounding or conversion instruction of the (narrow) conversion pipe
      const float f = __fadd_rn(quotient(a), 0.5f);
      const int bin = __float_as_int(__fadd_rd(f, 8388608.0f)) - 0x4B000000;
      if (in_range && a != 0.0f && f < top) atomicAdd(&s_h[bin], 1u);
    };
    auto sweep = [&](auto quotient) {
      if (dense && d.nvec < 0x40000000ull) { // the usual case: every lane of every vector counts, 32-bit indices
        const uint32_t n = (uint32_t)d.nvec, st = (uint32_t)stride;
        uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
        for (; i + st < n; i += 2 * st) {
          const float4 v0 = __ldg(x4 + i), v1 = __ldg(x4 + i + st);
          one(v0.x, true, quotient); one(v0.y, true, quotient); one(v0.z, true, quotient); one(v0.w, true, quotient);
          one(v1.x, true, quotient); one(v1.y, true, quotient); one(v1.z, true, quotient); one(v1.w, true, quotient);
        }
        for (; i < n; i += st) {
          const float4 v = __ldg(x4 + i);
          one(v.x, true, quotient); one(v.y, true, quotient); one(v.z, true, quotient); one(v.w, true, quotient);
        }
      } else {
        for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < d.nvec; i += stride) {
          const float4 v = __ldg(x4 + i);
          const int ch = dense ? 0 : (int)(i % d.vpp) * 4;
          one(v.x, dense || ch + 0 < d.c, quotient); one(v.y, dense || ch + 1 < d.c, quotient);
          one(v.z, dense || ch + 2 < d.c, quotient); one(v.w, dense || ch + 3 < d.c, quotient);
        }
      }
    };
    const float w = d.width;
    if (fast) sweep([=](float a) { return quot_by_const(a, w, rw); });
    else sweep([=](float a) { return __fdiv_rn(a, w); });
    __syncthreads();
    unsigned long long *h = hist + (size_t)t * bins;
    for (int j = threadIdx.x; j < bins; j += blockDim.x)
      if (s_h[j]) atomicAdd(&h[j], (unsigned long long)s_h[j]);
    __syncthreads();
  }
}

// One CTA per (histogram, candidate). N <= 4096 bins, 128-bin target. The float / double mix and
// the accumulation order of kl_calc_thread are kept: P and the running sums are sequential fp32
// additions of the converted counts; each KL term is formed in double and added into an fp32
// accumulator in index order.
__global__ void kld_kernel(const long long *__restrict__ hists, int N, float *__restrict__ kl_out) {
  pdl_prologue();
  extern __shared__ unsigned char kld_smem[];
  float *P = reinterpret_cast<float *>(kld_smem);
  float *Q = P + N;
  double *term = reinterpret_cast<double *>(Q + N);
  __shared__ float s_sum, s_tail;
  __shared__ long long s_count;
  const int BINS = 128;
  const int KL_NUM = N / BINS;
  const long long *hist = hists + (size_t)(blockIdx.x / KL_NUM) * N;
  const int i = (blockIdx.x % KL_NUM + 1) * BINS;
  const int tid = threadIdx.x;
  if (tid == 0) {
    long long cnt = 0;
    for (int j = 0; j < N; ++j) cnt += hist[j];
    s_count = cnt;
  } else if (tid == 32) {
    float tail = 0.0f;
    for (int j = i - 1; j < N; ++j) tail += (float)hist[j];
    s_tail = tail;
  } else if (tid == 64) {
    float sum = 0.0f;
    for (int j = 0; j < i; ++j) sum += (float)hist[j];
    s_sum = sum;
  }
  __syncthreads();
  const float fcount = (float)s_count;
  for (int j = tid; j < i; j += blockDim.x) {
    float p = j == i - 1 ? s_tail : (float)hist[j];
    P[j] = p / fcount;
  }
  const int expand = i / BINS;
  for (int j = tid; j < BINS; j += blockDim.x) {
    float sum_bin = 0.0f, pos = 0.0f;
    for (int k = 0; k < expand; ++k) {
      long long h = hist[j * expand + k];
      sum_bin += (float)h;
      pos += h > 0 ? 1.0f : 0.0f;
    }
    pos = pos == 0.0f ? 1.0f : pos;
    float q_base = sum_bin / pos / s_sum;
    for (int k = 0; k < expand; ++k) Q[j * expand + k] = hist[j * expand + k] ? q_base : 0.0f;
  }
  __syncthreads();
  for (int j = tid; j < i; j += blockDim.x)
    term[j] = (double)P[j] * (log10((double)P[j] + 1e-30) - log10((double)Q[j] + 1e-30));
  __syncthreads();
  if (tid == 0) {
    float kl = 0.0f;
    for (int j = 0; j < i; ++j) kl = (float)((double)kl + term[j]);
    kl_out[blockIdx.x] = kl;
  }
}

// Geometry of one NHWC tensor for kernels that walk two tensors of the same logical shape but different
// physical layouts (channel pitch, zero-padded rows).
struct DistGeom {
  const void *dev;
  int cp, wl, wphys;
};

// Per image i: sums[2i] += sum (ref - scale * tgt)^2, sums[2i+1] += sum |ref| over the image's real elements
// (the terms of `np.linalg.norm(diff) / np.linalg.norm(ref, ord=1)`, kld_calibrator.py:189-195). ref is fp32;
// tgt is int8 (TGT = 0), bf16 (1) or fp32 (2). The difference is formed in fp32 as numpy forms it, the sums
// in double. One thread handles four channels of one pixel per step; grid = (blocks per image, images).
template <int TGT>
__global__ void tuner_distance_kernel(DistGeom ref, DistGeom tgt, int c, int h, int w, float scale, double *sums) {
  pdl_prologue();
  const int img = blockIdx.y;
  const int c4 = (c + 3) >> 2;
  const size_t quads = (size_t)h * w * c4;
  double d2 = 0.0, s1 = 0.0;
  // four channels of one pixel: the fp32 reference vector and the candidate's raw bytes (4, 8 or 16 of them)
  auto load = [&](size_t q, float4 &r4, uint4 &raw, int &cq) {
    cq = (int)(q % c4);
    const size_t pix = q / c4;
    const int x = (int)(pix % w), y = (int)(pix / w);
    const size_t ro = (((size_t)img * h + y) * ref.wphys + ref.wl + x) * ref.cp + cq * 4;
    const size_t to = (((size_t)img * h + y) * tgt.wphys + tgt.wl + x) * tgt.cp + cq * 4;
    r4 = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(ref.dev) + ro));
    raw = make_uint4(0, 0, 0, 0);
    if (TGT == 0) {
      raw.x = (unsigned)__ldg(reinterpret_cast<const int *>(reinterpret_cast<const signed char *>(tgt.dev) + to));
    } else if (TGT == 1) {
      const uint2 wd = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const unsigned short *>(tgt.dev) + to));
      raw.x = wd.x;
      raw.y = wd.y;
    } else {
      raw = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const float *>(tgt.dev) + to));
    }
  };
  auto take = [&](const float4 &r4, const uint4 &raw, int cq) {
    float t[4];
    if (TGT == 0) {
      const int wd = (int)raw.x;
      t[0] = (float)(signed char)(wd & 0xff);
      t[1] = (float)(signed char)((wd >> 8) & 0xff);
      t[2] = (float)(signed char)((wd >> 16) & 0xff);
      t[3] = (float)(signed char)((wd >> 24) & 0xff);
    } else if (TGT == 1) {
      t[0] = __uint_as_float(raw.x << 16);
      t[1] = __uint_as_float(raw.x & 0xffff0000u);
      t[2] = __uint_as_float(raw.y << 16);
      t[3] = __uint_as_float(raw.y & 0xffff0000u);
    } else {
      t[0] = __uint_as_float(raw.x); t[1] = __uint_as_float(raw.y); t[2] = __uint_as_float(raw.z); t[3] = __uint_as_float(raw.w);
    }
    const float r[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (cq * 4 + j < c) {
        const float diff = __fsub_rn(r[j], __fmul_rn(t[j], scale));
        d2 += (double)diff * (double)diff;
        s1 += (double)fabsf(r[j]);
      }
    }
  };
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t q = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  for (; q + stride < quads; q += 2 * stride) {  // two independent load pairs in flight per thread
    float4 ra, rb;
    uint4 ta, tb;
    int ca, cb;
    load(q, ra, ta, ca);
    load(q + stride, rb, tb, cb);
    take(ra, ta, ca);
    take(rb, tb, cb);
  }
  for (; q < quads; q += stride) {
    float4 ra;
    uint4 ta;
    int ca;
    load(q, ra, ta, ca);
    take(ra, ta, ca);
  }
  for (int o = 16; o > 0; o >>= 1) {
    d2 += __shfl_xor_sync(0xffffffffu, d2, o);
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
  }
  __shared__ double sd[32], ss[32];
  if ((threadIdx.x & 31) == 0) {
    sd[threadIdx.x >> 5] = d2;
    ss[threadIdx.x >> 5] = s1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) {
      d2 += sd[i];
      s1 += ss[i];
    }
    atomicAdd(sums + 2 * img, d2);
    atomicAdd(sums + 2 * img + 1, s1);
  }
}

} // namespace tpucb
