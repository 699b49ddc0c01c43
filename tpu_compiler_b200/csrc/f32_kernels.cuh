// fp32 op kernels used by the calibration forward pass (the reference runs these through
// MKL-DNN in fp32: core/conv.cpp:90-93, core/fullyconnected.cpp, core/pooling.cpp:87-90,
// core/scale.cpp:15-37, core/softmax.cpp:49-86). Tensors are NHWC fp32 with the channel pitch
// padded to 4. The convolution is an implicit GEMM on the FP32 FMA pipe: 128 x 128 outputs per CTA
// with 8x8 per thread when the input channels are a multiple of 16, else 64 x 64 with 4x4 per thread;
// K is consumed 16 at a time through shared memory. Accumulation order differs from MKL-DNN's blocked order, so parity with the
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
  pdl_prologue();
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

// The same convolution for input channel counts that are multiples of 16 (every layer but a
// 3-channel stem): 128 pixels x 128 channels per CTA, K consumed 16 at a time, 8x8 outputs per
// thread, 16-byte global loads (a K chunk never straddles a filter tap, so the tap is uniform per
// chunk and a thread fetches 4 consecutive channels of one pixel), next chunk prefetched into
// registers while the current one is multiplied.
__global__ void __launch_bounds__(256, 2)
conv2d_f32_tile128_kernel(const float *__restrict__ in, const float *__restrict__ w, const float *__restrict__ bias,
                          float *__restrict__ out, ConvF32Args a) {
  pdl_prologue();
  __shared__ __align__(16) float As[16][128 + 4];
  __shared__ __align__(16) float Bs[16][128];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.x * 128, n0 = blockIdx.y * 128;
  const int ty = tid / 16, tx = tid % 16;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

  // A: thread loads channels (tid % 4) * 4 .. +3 of pixels tid / 4 and tid / 4 + 64
  const int a_c = (tid & 3) * 4;
  int a_y[2], a_x[2];
  const float *a_img[2];
  bool a_ok[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    int m = m0 + (tid >> 2) + 64 * i;
    a_ok[i] = m < a.M;
    int mm = a_ok[i] ? m : 0;
    int x = mm % a.ow;
    int t = mm / a.ow;
    a_x[i] = x * a.sw - a.pl;
    a_y[i] = (t % a.oh) * a.sh - a.pt;
    a_img[i] = in + (size_t)(t / a.oh) * a.ih * a.iw * a.icp;
  }
  // B: thread loads columns (tid % 32) * 4 .. +3 of rows tid / 32 and tid / 32 + 8
  const int b_k = tid >> 5, b_n = (tid & 31) * 4;

  float4 ra[2], rb[2];
  int c0 = 0, tr = 0, ts = 0; // channel offset and filter tap of the chunk being fetched
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int yy = a_y[i] + tr * a.dh, xx = a_x[i] + ts * a.dw;
      ra[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (a_ok[i] && yy >= 0 && yy < a.ih && xx >= 0 && xx < a.iw)
        ra[i] = *reinterpret_cast<const float4 *>(a_img[i] + ((size_t)yy * a.iw + xx) * a.icp + c0 + a_c);
      rb[i] = *reinterpret_cast<const float4 *>(w + (size_t)(k0 + b_k + 8 * i) * a.wld + n0 + b_n);
    }
    c0 += 16;
    if (c0 == a.ic) {
      c0 = 0;
      if (++ts == a.kw) {
        ts = 0;
        ++tr;
      }
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < a.K; k0 += 16) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int m = (tid >> 2) + 64 * i;
      As[a_c + 0][m] = ra[i].x;
      As[a_c + 1][m] = ra[i].y;
      As[a_c + 2][m] = ra[i].z;
      As[a_c + 3][m] = ra[i].w;
      *reinterpret_cast<float4 *>(&Bs[b_k + 8 * i][b_n]) = rb[i];
    }
    __syncthreads();
    if (k0 + 16 < a.K) fetch(k0 + 16);
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const float4 a0 = *reinterpret_cast<const float4 *>(&As[k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4 *>(&As[k][ty * 4 + 64]);
      const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4 + 64]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + ty * 4 + (i & 3) + 64 * (i >> 2);
    if (m >= a.M) continue;
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int n = n0 + tx * 4 + 64 * jh;
      if (n >= a.ocp) continue;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[j] = 0.0f;
        if (n + j < a.oc) {
          v[j] = acc[i][4 * jh + j] + bias[n + j];
          if (a.do_relu && v[j] < 0) v[j] = 0;
        }
      }
      *reinterpret_cast<float4 *>(out + (size_t)m * a.ocp + n) = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
}

inline std::vector<float> pack_conv_weights_f32(const float *w, int oc, int icg, int kh, int kw, int groups) {
  TPUCB_CHECK(groups == 1, "fp32 convolution: grouped convolution is not implemented");
  const int wld = round_up(oc, 128);
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
                              int ocp, int do_relu, cudaStream_t s, int sm_count) {
  ConvF32Args a;
  a.n = g.n; a.ic = g.ic; a.icp = icp; a.ih = g.ih; a.iw = g.iw; a.oc = g.oc; a.ocp = ocp; a.oh = g.oh; a.ow = g.ow;
  a.kh = g.kh; a.kw = g.kw; a.sh = g.sh; a.sw = g.sw; a.pt = g.pt; a.pl = g.pl; a.dh = g.dh; a.dw = g.dw;
  a.do_relu = do_relu;
  a.K = g.kh * g.kw * g.ic;
  a.wld = round_up(g.oc, 128);
  a.M = g.n * g.oh * g.ow;
  (void)sm_count; // the large tile also wins on the layers that leave SMs without a CTA (measured)
  if (g.ic % 16 == 0 && icp == g.ic) {
    dim3 grid((a.M + 127) / 128, a.wld / 128);
    launch_k(conv2d_f32_tile128_kernel, grid, 256, 0, s, in, w, bias, out, a);
    return;
  }
  dim3 grid((a.M + 63) / 64, a.wld / 64);
  launch_k(conv2d_f32_kernel, grid, 256, 0, s, in, w, bias, out, a);
}

// Y[m][n] = X[m][k] . W[n][k] + b, optional ReLU; one warp per output element.
__global__ void fc_f32_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
                              float *__restrict__ y, int m, int k, int n, int ldy, int do_relu) {
  pdl_prologue();
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
  launch_k(fc_f32_kernel, (unsigned)((threads + 255) / 256), 256, 0, s, x, w, b, y, m, k, n, ldy, do_relu);
}

// fp32 pooling: max ignores padded taps; avg divides by kh*kw (count_include_pad) or by the
// number of valid taps (NativeCpuImplementation.h:104-160).
// Four channels (one 16-byte vector) per thread; per element the same operations in the same order as the scalar form.
__global__ void pool_f32_kernel(const float *__restrict__ in, float *__restrict__ out, PoolArgs a, int count_include_pad) {
  pdl_prologue();
  const int vpp = a.cp / 4; // fp32 tensors have a channel pitch that is a multiple of 4
  const size_t total = (size_t)a.n * a.oh * a.ow * vpp;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c4 = (int)(i % vpp) * 4;
    const size_t pix = i / vpp;
    const int x = (int)(pix % a.ow);
    const size_t t = pix / a.ow;
    const int y = (int)(t % a.oh);
    const int b = (int)(t / a.oh);
    float4 mx = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY), sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    int cnt = 0;
    for (int r = 0; r < a.kh; ++r) {
      const int yy = y * a.sh - a.pt + r;
      if (yy < 0 || yy >= a.ih) continue;
      for (int s = 0; s < a.kw; ++s) {
        const int xx = x * a.sw - a.pl + s;
        if (xx < 0 || xx >= a.iw) continue;
        const float4 v = __ldg(reinterpret_cast<const float4 *>(in + (((size_t)b * a.ih + yy) * a.iw + xx) * a.cp + c4));
        mx.x = fmaxf(mx.x, v.x); mx.y = fmaxf(mx.y, v.y); mx.z = fmaxf(mx.z, v.z); mx.w = fmaxf(mx.w, v.w);
        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        ++cnt;
      }
    }
    const float div = (float)(count_include_pad ? a.kh * a.kw : cnt);
    float4 res = a.method == 0 ? mx : make_float4(sum.x / div, sum.y / div, sum.z / div, sum.w / div);
    if (c4 + 0 >= a.c) res.x = 0.0f;
    if (c4 + 1 >= a.c) res.y = 0.0f;
    if (c4 + 2 >= a.c) res.z = 0.0f;
    if (c4 + 3 >= a.c) res.w = 0.0f;
    *reinterpret_cast<float4 *>(out + pix * a.cp + c4) = res;
  }
}

inline void launch_pool_f32(const float *in, float *out, const PoolArgs &a, int cip, cudaStream_t s, int sm_count) {
  size_t total = (size_t)a.n * a.oh * a.ow * (a.cp / 4);
  launch_k(pool_f32_kernel, grid_for(total, 256, sm_count), 256, 0, s, in, out, a, cip);
}

__global__ void scale_f32_kernel(const float *__restrict__ in, const float *__restrict__ sc, const float *__restrict__ bi,
                                 float *__restrict__ out, size_t n, int cp) {
  pdl_prologue();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    int c = (int)(i % cp);
    out[i] = __fadd_rn(__fmul_rn(in[i], sc[c]), bi[c]);
  }
}

// BatchNormOpKernel (core/batchnorm.cpp:20-68): (x - mean') / d per channel, with mean' and d = sqrt(var' + eps)
// prepared per channel by the host in fp32 as the reference forms them; a subtraction and an IEEE division per value.
__global__ void batchnorm_f32_kernel(const float *__restrict__ in, const float *__restrict__ mean, const float *__restrict__ den,
                                     float *__restrict__ out, size_t n, int cp) {
  pdl_prologue();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    int c = (int)(i % cp);
    out[i] = __fdiv_rn(__fsub_rn(in[i], mean[c]), den[c]);
  }
}

// softmax over the channel axis of one pixel per CTA.
__global__ void softmax_f32_kernel(const float *__restrict__ in, float *__restrict__ out, int c, int cp) {
  pdl_prologue();
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
