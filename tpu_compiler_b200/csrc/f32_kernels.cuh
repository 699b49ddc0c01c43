// fp32 op kernels used by the calibration forward pass (the reference runs these through
// MKL-DNN in fp32: core/conv.cpp:90-93, core/fullyconnected.cpp, core/pooling.cpp:87-90,
// core/scale.cpp:15-37, core/softmax.cpp:49-86). Tensors are NHWC fp32 with the channel pitch
// padded to 4. The convolution is an implicit GEMM on the FP32 FMA pipe: 64 output pixels x
// 64 output channels per CTA, K consumed 16 at a time through shared memory, 4x4 outputs per
// thread. Accumulation order differs from MKL-DNN's blocked order, so parity with the
// reference is to 1e-4 relative, not bit-exact.
#pragma once
#include "common.cuh"
#include "host_common.h"
#include "mem_kernels.cuh"

namespace tpucb {

struct ConvGeom;

struct ConvF32Args {
  int n, ic, icp, ih, iw, oc, ocp, oh, ow, kh, kw, sh, sw, pt, pl, dh, dw, do_relu;
  int K;    // kh*kw*ic
  int wld;  // weight row pitch (oc padded to 64)
  int M;    // n*oh*ow
};

// weights [K = (r, s, c)][wld]
__global__ void __launch_bounds__(256)
conv2d_f32_kernel(const float *__restrict__ in, const float *__restrict__ w, const float *__restrict__ bias,
                  float *__restrict__ out, ConvF32Args a) {
  __shared__ float As[16][64 + 4];
  __shared__ float Bs[16][64];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.x * 64, n0 = blockIdx.y * 64;
  const int ty = tid / 16, tx = tid % 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  // A gather assignment: k = tid % 16, rows tid/16 + 16*i
  const int ak = tid % 16;
  int a_b[4], a_y[4], a_x[4];
  bool a_ok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int m = m0 + tid / 16 + 16 * i;
    a_ok[i] = m < a.M;
    int mm = a_ok[i] ? m : 0;
    int x = mm % a.ow;
    int t = mm / a.ow;
    a_x[i] = x * a.sw - a.pl;
    a_y[i] = (t % a.oh) * a.sh - a.pt;
    a_b[i] = t / a.oh;
  }
  const int bk = tid / 64, bn = tid % 64;

  for (int k0 = 0; k0 < a.K; k0 += 16) {
    {
      int k = k0 + ak;
      int c = 0, r = 0, s = 0;
      bool kok = k < a.K;
      if (kok) {
        c = k % a.ic;
        int tap = k / a.ic;
        s = tap % a.kw;
        r = tap / a.kw;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = 0.0f;
        int yy = a_y[i] + r * a.dh, xx = a_x[i] + s * a.dw;
        if (kok && a_ok[i] && yy >= 0 && yy < a.ih && xx >= 0 && xx < a.iw)
          v = in[(((size_t)a_b[i] * a.ih + yy) * a.iw + xx) * a.icp + c];
        As[ak][tid / 16 + 16 * i] = v;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int k = k0 + bk + 4 * i;
      Bs[bk + 4 * i][bn] = k < a.K ? w[(size_t)k * a.wld + n0 + bn] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int m = m0 + ty * 4 + i;
    if (m >= a.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx * 4 + j;
      if (n >= a.ocp) continue;
      float v = 0.0f;
      if (n < a.oc) {
        v = acc[i][j] + bias[n];
        if (a.do_relu && v < 0) v = 0;
      }
      out[(size_t)m * a.ocp + n] = v;
    }
  }
}

inline std::vector<float> pack_conv_weights_f32(const float *w, int oc, int icg, int kh, int kw, int groups) {
  TPUCB_CHECK(groups == 1, "fp32 convolution: grouped convolution is not implemented");
  const int wld = round_up(oc, 64);
  std::vector<float> out((size_t)kh * kw * icg * wld, 0.0f);
  for (int o = 0; o < oc; ++o)
    for (int c = 0; c < icg; ++c)
      for (int r = 0; r < kh; ++r)
        for (int s = 0; s < kw; ++s)
          out[((size_t)(r * kw + s) * icg + c) * wld + o] = w[(((size_t)o * icg + c) * kh + r) * kw + s];
  return out;
}

template <class G>
inline void launch_conv2d_f32(const float *in, const float *w, const float *bias, float *out, const G &g, int icp,
                              int ocp, int do_relu, cudaStream_t s, int) {
  ConvF32Args a;
  a.n = g.n; a.ic = g.ic; a.icp = icp; a.ih = g.ih; a.iw = g.iw; a.oc = g.oc; a.ocp = ocp; a.oh = g.oh; a.ow = g.ow;
  a.kh = g.kh; a.kw = g.kw; a.sh = g.sh; a.sw = g.sw; a.pt = g.pt; a.pl = g.pl; a.dh = g.dh; a.dw = g.dw;
  a.do_relu = do_relu;
  a.K = g.kh * g.kw * g.ic;
  a.wld = round_up(g.oc, 64);
  a.M = g.n * g.oh * g.ow;
  dim3 grid((a.M + 63) / 64, a.wld / 64);
  conv2d_f32_kernel<<<grid, 256, 0, s>>>(in, w, bias, out, a);
}

// Y[m][n] = X[m][k] . W[n][k] + b, optional ReLU; one warp per output element.
__global__ void fc_f32_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
                              float *__restrict__ y, int m, int k, int n, int ldy, int do_relu) {
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32, lane = threadIdx.x & 31;
  if (warp >= m * n) return;
  int i = warp / n, j = warp % n;
  float acc = 0.0f;
  for (int t = lane; t < k; t += 32) acc = fmaf(x[(size_t)i * k + t], w[(size_t)j * k + t], acc);
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    float v = acc + bias[j];
    if (do_relu && v < 0) v = 0;
    y[(size_t)i * ldy + j] = v;
  }
}
inline void launch_fc_f32(const float *x, const float *w, const float *b, float *y, int m, int k, int n, int ldy,
                          int do_relu, cudaStream_t s) {
  size_t threads = (size_t)m * n * 32;
  fc_f32_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(x, w, b, y, m, k, n, ldy, do_relu);
}

// fp32 pooling: max ignores padded taps; avg divides by kh*kw (count_include_pad) or by the
// number of valid taps (NativeCpuImplementation.h:104-160).
__global__ void pool_f32_kernel(const float *__restrict__ in, float *__restrict__ out, PoolArgs a, int count_include_pad) {
  const size_t total = (size_t)a.n * a.oh * a.ow * a.cp;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    int c = (int)(i % a.cp);
    size_t pix = i / a.cp;
    int x = (int)(pix % a.ow);
    size_t t = pix / a.ow;
    int y = (int)(t % a.oh);
    int b = (int)(t / a.oh);
    float mx = -INFINITY, sum = 0.0f;
    int cnt = 0;
    for (int r = 0; r < a.kh; ++r) {
      int yy = y * a.sh - a.pt + r;
      if (yy < 0 || yy >= a.ih) continue;
      for (int s = 0; s < a.kw; ++s) {
        int xx = x * a.sw - a.pl + s;
        if (xx < 0 || xx >= a.iw) continue;
        float v = in[(((size_t)b * a.ih + yy) * a.iw + xx) * a.cp + c];
        mx = fmaxf(mx, v);
        sum += v;
        ++cnt;
      }
    }
    float res = a.method == 0 ? mx : sum / (float)(count_include_pad ? a.kh * a.kw : cnt);
    out[i] = c < a.c ? res : 0.0f;
  }
}
inline void launch_pool_f32(const float *in, float *out, const PoolArgs &a, int cip, cudaStream_t s, int sm_count) {
  size_t total = (size_t)a.n * a.oh * a.ow * a.cp;
  pool_f32_kernel<<<grid_for(total, 256, sm_count), 256, 0, s>>>(in, out, a, cip);
}

__global__ void scale_f32_kernel(const float *__restrict__ in, const float *__restrict__ sc, const float *__restrict__ bi,
                                 float *__restrict__ out, size_t n, int cp) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    int c = (int)(i % cp);
    out[i] = __fadd_rn(__fmul_rn(in[i], sc[c]), bi[c]);
  }
}

// softmax over the channel axis of one pixel per CTA.
__global__ void softmax_f32_kernel(const float *__restrict__ in, float *__restrict__ out, int c, int cp) {
  __shared__ float red[32];
  const float *p = in + (size_t)blockIdx.x * cp;
  float *q = out + (size_t)blockIdx.x * cp;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < c; i += blockDim.x) mx = fmaxf(mx, p[i]);
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for (int i = 1; i < (int)(blockDim.x >> 5); ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float sum = 0.0f;
  for (int i = threadIdx.x; i < c; i += blockDim.x) {
    float e = expf(p[i] - mx);
    q[i] = e;
    sum += e;
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  sum = 0.0f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) sum += red[i];
  for (int i = threadIdx.x; i < cp; i += blockDim.x) q[i] = i < c ? q[i] / sum : 0.0f;
}

} // namespace tpucb
