// Host planner for the INT8 implicit-GEMM kernel: weight packing, TMA tensor
// maps, tile-shape heuristics and the launch. The geometry follows parseConvParam
// (lib/Dialect/TPU/IR/TPUOperationSupport.cpp:366-428): four independent pads, the
// output size taken from the result type, dilation, optional input zero-insertion.
#pragma once
#include "conv_gemm_i8.cuh"
#include "conv_stem_i8.cuh"
#include "host_common.h"
#include "mem_kernels.cuh"

#include <cstdlib>
#include <cstring>
#include <cudaTypedefs.h>

namespace tpucb {

struct ConvGeom {
  int n, ic, ih, iw, oc, oh, ow, g, kh, kw, sh, sw, pt, pb, pl, pr, dh, dw, ins_h, ins_w;
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const int *, const int *,
                                   cuuint32_t, cuuint32_t, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

struct TmaApi {
  EncodeTiledFn tiled = nullptr;
  EncodeIm2colFn im2col = nullptr;
  int driver_version = 0;
};

// The driver entry points are fetched through the runtime so that the library carries no
// link-time dependency on the driver library (it must load on machines without a GPU).
inline const TmaApi &tma_api() {
  static TmaApi api = [] {
    TmaApi a;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    TPUCB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    TPUCB_CHECK(fn && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled not available");
    a.tiled = (EncodeTiledFn)fn;
    fn = nullptr;
    TPUCB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q));
    TPUCB_CHECK(fn && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeIm2col not available");
    a.im2col = (EncodeIm2colFn)fn;
    TPUCB_CUDA(cudaDriverGetVersion(&a.driver_version));
    return a;
  }();
  return api;
}

inline CUtensorMapSwizzle swizzle_for(int BK) {
  return BK == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                   : (BK == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

// tcgen05 instruction descriptor for kind::i8: D = s32 (bits 4-5 = 2), A and B signed
// 8-bit (bits 7-9 and 10-12 = 1), both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
inline uint32_t make_idesc_i8(int M, int N) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

// kind::f16 with BF16 operands and an fp32 accumulator: D = f32 (bits 4-5 = 1), A and B = BF16 (1)
inline uint32_t make_idesc_bf16(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// kind::tf32 with an fp32 accumulator: D = f32 (1), A and B = TF32 (2)
inline uint32_t make_idesc_tf32(int M, int N) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

struct ConvPlan {
  CUtensorMap tmA, tmB;
  ConvGemmParams p;
  dim3 grid;
  size_t smem = 0;
  int ws_tiles = 0;  // split K: tiles of the partial-sum workspace (p.ws, p.ws_count), allocated by the op that owns the plan
  bool bf16 = false; // runs conv_gemm_bf16_kernel (K sizes and pitches in bytes, 2 per element)
  bool tf32 = false; // runs conv_gemm_tf32x3_kernel (fp32 operands, 4 bytes per element; three K passes)
  CUtensorMap tmA2, tmB2;           // tf32: remainder parts of the activations and of the weights
  const float *split_src = nullptr; // tf32: the fp32 input, split into split_hi / split_lo before the launch
  float *split_hi = nullptr, *split_lo = nullptr;
  size_t split_nvec = 0;
  bool use_patch = false;
  int patch_elsize = 1; // bytes per element of the patch matrix: 1 INT8, 2 BF16, 4 fp32
  PatchArgs patch;
  int8_t *patch_buf = nullptr; // scratch: expanded patch matrix [M][kp]
  size_t patch_bytes = 0;
  const int8_t *in = nullptr;
  double ops = 0, bytes = 0; // algorithmic work of one launch
};

// K block width in bytes for `k_bytes` of K per tap. The main loop's time follows the NUMBER of K blocks (a block
// costs a barrier round trip and a copy issue whatever its width), so the fewest blocks win and, among equal counts,
// the narrower block (less zero padding through the tensor pipe): 96 bytes -> one 128-byte block, not three of 32.
inline int pick_bk(int k_bytes) {
  int best = 128, best_blocks = 1 << 30;
  for (int bk : {128, 64, 32}) {
    int blocks = (k_bytes + bk - 1) / bk;
    if (blocks <= best_blocks) {
      best_blocks = blocks;
      best = bk;
    }
  }
  return best;
}

// Pack OIHW fp32 weights (integer-valued) to int8 [oc_pad][taps][cin_pad] for the im2col
// path, or [oc_pad][1][kp] with K order (r, s, c) for the patch path. For grouped
// convolution the caller passes one group's slice.
inline std::vector<int8_t> pack_conv_weights(const float *w, int oc, int icg, int kh, int kw,
                                             int oc_pad, int cin_pad, bool patch, int kp) {
  const int taps = kh * kw;
  std::vector<int8_t> out((size_t)oc_pad * (patch ? kp : taps * cin_pad), 0);
  for (int o = 0; o < oc; ++o)
    for (int c = 0; c < icg; ++c)
      for (int r = 0; r < kh; ++r)
        for (int s = 0; s < kw; ++s) {
          int8_t v = (int8_t)(int)w[(((size_t)o * icg + c) * kh + r) * kw + s];
          if (patch) out[(size_t)o * kp + (size_t)(r * kw + s) * icg + c] = v;
          else out[((size_t)o * taps + (r * kw + s)) * cin_pad + c] = v;
        }
  return out;
}

// BF16 weights [oc_pad][tap][cin_pad] as 16-bit patterns (the values of a BF16 graph's filter are
// BF16-representable floats: the upper 16 bits are the value), returned as bytes
inline std::vector<int8_t> pack_conv_weights_bf16(const float *w, int oc, int icg, int kh, int kw, int oc_pad,
                                                  int cin_pad) {
  const int taps = kh * kw;
  std::vector<uint16_t> out((size_t)oc_pad * taps * cin_pad, 0);
  for (int o = 0; o < oc; ++o)
    for (int c = 0; c < icg; ++c)
      for (int r = 0; r < kh; ++r)
        for (int s = 0; s < kw; ++s)
          out[((size_t)o * taps + (r * kw + s)) * cin_pad + c] =
              (uint16_t)(f32_bits(w[(((size_t)o * icg + c) * kh + r) * kw + s]) >> 16);
  std::vector<int8_t> bytes(out.size() * 2);
  std::memcpy(bytes.data(), out.data(), bytes.size());
  return bytes;
}

// fp32 weights for the TF32 x 3 convolution, K-major [oc_pad][tap][cin_pad] as bytes: part 0 = the upper 19 bits of
// every word, part 1 = the exact remainder.
inline std::vector<int8_t> pack_conv_weights_tf32(const float *w, int oc, int icg, int kh, int kw, int oc_pad, int cin_pad,
                                                  int part) {
  const int taps = kh * kw;
  std::vector<float> out((size_t)oc_pad * taps * cin_pad, 0.0f);
  for (int o = 0; o < oc; ++o)
    for (int c = 0; c < icg; ++c)
      for (int r = 0; r < kh; ++r)
        for (int s = 0; s < kw; ++s) {
          const float v = w[(((size_t)o * icg + c) * kh + r) * kw + s];
          const float hi = bits_f32(f32_bits(v) & 0xffffe000u);
          out[((size_t)o * taps + (r * kw + s)) * cin_pad + c] = part == 0 ? hi : v - hi;
        }
  std::vector<int8_t> bytes(out.size() * 4);
  std::memcpy(bytes.data(), out.data(), bytes.size());
  return bytes;
}

// Weights of the patch-matrix form [oc_pad][kp], k = (r * kw + s) * icg + c, as 2-byte BF16 (part < 0) or as fp32
// parts of a TF32 x 3 product (part 0: upper 19 bits, part 1: remainder).
inline std::vector<int8_t> pack_patch_weights(const float *w, int oc, int icg, int kh, int kw, int oc_pad, int kp, int part,
                                              int cstride = 0) {
  if (cstride == 0) cstride = icg; // channel slots per tap (4 in patch_expand_tap_kernel's layout)
  const size_t n = (size_t)oc_pad * kp;
  std::vector<uint16_t> h(part < 0 ? n : 0, 0);
  std::vector<float> f(part < 0 ? 0 : n, 0.0f);
  for (int o = 0; o < oc; ++o)
    for (int c = 0; c < icg; ++c)
      for (int r = 0; r < kh; ++r)
        for (int s = 0; s < kw; ++s) {
          const float v = w[(((size_t)o * icg + c) * kh + r) * kw + s];
          const size_t k = (size_t)o * kp + (size_t)(r * kw + s) * cstride + c;
          if (part < 0) h[k] = (uint16_t)(f32_bits(v) >> 16);
          else {
            const float hi = bits_f32(f32_bits(v) & 0xffffe000u);
            f[k] = part == 0 ? hi : v - hi;
          }
        }
  std::vector<int8_t> bytes(part < 0 ? n * 2 : n * 4);
  std::memcpy(bytes.data(), part < 0 ? (const void *)h.data() : (const void *)f.data(), bytes.size());
  return bytes;
}

inline void encode_weight_map(CUtensorMap *tm, const int8_t *d_w, int oc_pad, int taps, int k_inner,
                              int BK, int BN) {
  cuuint64_t dims[3] = {(cuuint64_t)k_inner, (cuuint64_t)taps, (cuuint64_t)oc_pad};
  cuuint64_t strides[2] = {(cuuint64_t)k_inner, (cuuint64_t)k_inner * taps};
  cuuint32_t box[3] = {(cuuint32_t)BK, 1, (cuuint32_t)BN};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = tma_api().tiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void *)d_w, dims, strides, box,
                               es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(BK),
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPUCB_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(weights) failed: %d", (int)r);
}

// `tile_rows`: rows (pixels) per copy = the plan's pixel tile: 128, or 256 in dual mode (a_tile_rows)
inline int a_tile_rows(const ConvGemmParams &p) { return p.dual ? 256 : 128; }

inline void encode_matrix_map(CUtensorMap *tm, const int8_t *d_a, int rows, int k_inner, int ld,
                              int BK, int tile_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)k_inner, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)tile_rows};
  cuuint32_t es[2] = {1, 1};
  CUresult r = tma_api().tiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)d_a, dims, strides, box,
                               es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(BK),
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPUCB_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(matrix) failed: %d", (int)r);
}

inline void encode_im2col_map(CUtensorMap *tm, const int8_t *d_in, const ConvGeom &g, int cp,
                              int BK, int tile_rows) {
  cuuint64_t dims[4] = {(cuuint64_t)cp, (cuuint64_t)g.iw, (cuuint64_t)g.ih, (cuuint64_t)g.n};
  cuuint64_t strides[3] = {(cuuint64_t)cp, (cuuint64_t)cp * g.iw, (cuuint64_t)cp * g.iw * g.ih};
  // Base-pixel bounding box: lower corner = -pad_lo, upper corner chosen so that the number
  // of base positions along each axis equals the op's output extent:
  //   (extent + upper - lower - 1) / stride + 1 == out
  int lower[2] = {-g.pl, -g.pt};
  // Textbook value: pad_hi - (k - 1) * dilation. When the op's output extent does not follow
  // from its pads by the usual formula (the result type rules), use the tight value instead.
  int upper[2] = {g.pr - (g.kw - 1) * g.dw, g.pb - (g.kh - 1) * g.dh};
  if ((g.iw + upper[0] - lower[0] - 1) / g.sw + 1 != g.ow)
    upper[0] = (g.ow - 1) * g.sw + 1 - g.iw - g.pl;
  if ((g.ih + upper[1] - lower[1] - 1) / g.sh + 1 != g.oh)
    upper[1] = (g.oh - 1) * g.sh + 1 - g.ih - g.pt;
  cuuint32_t es[4] = {1, (cuuint32_t)g.sw, (cuuint32_t)g.sh, 1};
  CUresult r = tma_api().im2col(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void *)d_in, dims, strides,
                                lower, upper, (cuuint32_t)BK, (cuuint32_t)tile_rows, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                swizzle_for(BK), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPUCB_CHECK(r == CUDA_SUCCESS,
              "cuTensorMapEncodeIm2col failed: %d (iw=%d ih=%d lower=%d,%d upper=%d,%d)", (int)r,
              g.iw, g.ih, lower[0], lower[1], upper[0], upper[1]);
  // Drivers up to CUDA 13.1 encode im2col maps of tensors smaller than 128 KiB with a flag
  // (bit 21 of the second 64-bit word) that makes the load misbehave; the same correction
  // is applied by NVIDIA's open-source CUTLASS when it builds these maps.
  size_t tensor_bytes = (size_t)cp * g.iw * g.ih * g.n;
  if (tma_api().driver_version <= 13010 && tensor_bytes < 131072)
    reinterpret_cast<uint64_t *>(tm)[1] &= ~(1ull << 21);
}

// Few-channel ("stem") convolutions: with the input stored as zero-padded NHWC rows whose pixel
// pitch is cp = 16 / stride_w bytes, the kw taps of one filter row of one output pixel are a
// contiguous window that starts on a 16-byte boundary, and neighbouring output pixels' windows
// start 16 bytes apart. A 4-D tiled tensor map with OVERLAPPING strides
//   (window byte, output column q [16 B], input row [row pitch], image)
// then delivers g consecutive output pixels' windows per copy; K has one step per filter row.
struct StemLayout {
  int cp = 0;     // channel pitch of the input tensor (bytes per pixel)
  int wl = 0;     // zero pixels on the left of each row
  int wphys = 0;  // physical row width in pixels
  int bk = 0;     // window bytes, rounded up to a swizzle span (32/64/128)
  int g = 0;      // output pixels per copy: gcd(OW, 128), at least 8
};

inline int gcd_int(int a, int b) { return b == 0 ? a : gcd_int(b, a % b); }

inline bool stem_layout_for(const ConvGeom &g, StemLayout *out) {
  if (g.g != 1 || g.ins_h || g.ins_w || g.dw != 1) return false;
  if (!(g.sw == 1 || g.sw == 2 || g.sw == 4)) return false;
  const int cp = 16 / g.sw;
  if (g.ic > cp || g.ic >= 16) return false;
  const int wl = round_up(g.pl, g.sw);
  const int win_px = (wl - g.pl) + g.kw;
  const int wb = win_px * cp;
  if (wb > 128) return false;
  const int bk = wb <= 32 ? 32 : (wb <= 64 ? 64 : 128);
  const int gg = gcd_int(g.ow, 128);
  if (gg < 8) return false;
  int wphys = (g.ow - 1) * g.sw + bk / cp;
  if (wphys < wl + g.iw) wphys = wl + g.iw;
  wphys = round_up(wphys, g.sw);
  if (((size_t)wphys * cp) % 16 != 0) return false;
  out->cp = cp; out->wl = wl; out->wphys = wphys; out->bk = bk; out->g = gg;
  return true;
}

inline void encode_window_map(CUtensorMap *tm, const int8_t *d_in, const ConvGeom &g, int cp, int wphys,
                              int BK, int gpix) {
  const cuuint64_t row_pitch = (cuuint64_t)wphys * cp;
  cuuint64_t dims[4] = {(cuuint64_t)BK, (cuuint64_t)g.ow, (cuuint64_t)g.ih, (cuuint64_t)g.n};
  cuuint64_t strides[3] = {(cuuint64_t)g.sw * cp, row_pitch, row_pitch * g.ih};
  cuuint32_t box[4] = {(cuuint32_t)BK, (cuuint32_t)gpix, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = tma_api().tiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void *)d_in, dims, strides, box, es,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(BK),
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPUCB_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(row window) failed: %d", (int)r);
}

// Thread-gathered stem convolution (conv_stem_i8_kernel): at most 4 input channels stored as one
// 32-bit word per pixel, kw <= 8, kh <= 8, no groups / insertion / horizontal dilation.
inline bool stem4_applies(const ConvGeom &g) {
  return g.g == 1 && !g.ins_h && !g.ins_w && g.dw == 1 && g.ic <= 4 && g.kw <= 8 && g.kh <= 8;
}

struct StemPlan {
  CUtensorMap tmB;
  ConvStemParams p;
  dim3 grid;
  size_t smem = 0;
};

inline void stem_kernel_setup_once() {
  static bool done = [] {
    TPUCB_CUDA(cudaFuncSetAttribute(conv_stem_i8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    TPUCB_CUDA(cudaFuncSetAttribute(conv_stem_i8_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    TPUCB_CUDA(cudaFuncSetAttribute(conv_stem_i8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    return true;
  }();
  (void)done;
}

// weights [kh][oc_pad][32]: byte s*4 + c of filter row r
inline std::vector<int8_t> pack_stem_weights(const float *w, int oc, int ic, int kh, int kw, int oc_pad) {
  std::vector<int8_t> out((size_t)kh * oc_pad * 32, 0);
  for (int o = 0; o < oc; ++o)
    for (int c = 0; c < ic; ++c)
      for (int r = 0; r < kh; ++r)
        for (int s = 0; s < kw; ++s)
          out[((size_t)r * oc_pad + o) * 32 + s * 4 + c] = (int8_t)(int)w[(((size_t)o * ic + c) * kh + r) * kw + s];
  return out;
}

inline void finish_stem_plan(StemPlan &sp, const int8_t *d_w, int rows, int kh, int oc_pad, int sm_count) {
  ConvStemParams &p = sp.p;
  const int bn = 128; // channel tile = tensor-core M; rows past oc_pad are zero-filled by TMA
  p.BN = bn;
  p.n_valid = oc_pad;
  p.tmem_cols = 128;
  p.idesc = make_idesc_i8(128, bn);
  p.M_total = rows;
  p.kh = kh;
  p.dual = (oc_pad <= 64 && rows > 128) ? 1 : 0;
  const int m_tile = p.dual ? 256 : 128;
  const int w_rows = p.dual ? 192 : bn;
  sp.smem = kSmemHeader + 1024 + (size_t)kh * ((size_t)m_tile * 32 + (size_t)w_rows * 32);
  const int m_tiles = (rows + m_tile - 1) / m_tile;
  const int n_tiles = (oc_pad + bn - 1) / bn;
  // persistent: two CTAs per SM, a multiple of the channel-tile count (a CTA's weights never change)
  int grid = 2 * sm_count / n_tiles * n_tiles;
  if (grid < n_tiles) grid = n_tiles;
  if (grid > m_tiles * n_tiles) grid = m_tiles * n_tiles;
  sp.grid = dim3((unsigned)grid, 1, 1);
  cuuint64_t dims[3] = {32, (cuuint64_t)oc_pad, (cuuint64_t)kh};
  cuuint64_t strides[2] = {32, (cuuint64_t)32 * oc_pad};
  cuuint32_t box[3] = {32, (cuuint32_t)w_rows, (cuuint32_t)kh};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = tma_api().tiled(&sp.tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void *)d_w, dims, strides, box, es,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TPUCB_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(stem weights) failed: %d", (int)r);
}

// Build the launch plan for one GEMM-shaped problem.
//   rows       implicit-GEMM M
//   k_inner    K bytes per tap (padded input channels, or the whole K in matrix mode)
//   oc_pad     padded output channels (multiple of 16)
inline void finish_plan(ConvPlan &pl, int rows, int taps, int k_inner, int oc_pad, int sm_count) {
  ConvGemmParams &p = pl.p;
  p.M_total = rows;
  p.BK = pick_bk(k_inner);
  p.c_chunks = (k_inner + p.BK - 1) / p.BK;
  // Dual mode: layers with at most 64 output channels would leave half of the TMEM lanes (and half of
  // the epilogue warps) idle; they run 256-pixel tiles instead (see the kernel). Not combined with the
  // row-window activation mode.
  {
    // ... unless the whole weight set is small enough to stay resident in plain mode, which feeds
    // fewer bytes per pixel (measured faster for the 1x1 layers with 64 outputs).
    const size_t w_plain = (size_t)taps * p.c_chunks * 128 * p.BK;
    const bool plain_resident = w_plain <= 48 * 1024 && 113 * 1024 - kSmemHeader - 1024 - w_plain >= 3 * (size_t)128 * p.BK;
    p.dual = (oc_pad <= 64 && p.a_mode != 2 && rows > 128 && !plain_resident && !pl.tf32) ? 1 : 0;
  }
  const int m_tiles = (rows + (p.dual ? 255 : 127)) / (p.dual ? 256 : 128);
  // Transposed product: the channel tile is the tensor core's M (128 TMEM lanes, rows past the
  // padded channel count are zero-filled by TMA), the pixel tile its N (128 TMEM columns), and
  // the accumulator is double-buffered: 256 TMEM columns.
  const int bn = 128;
  p.BN = bn;
  p.n_valid = oc_pad;
  p.tmem_cols = 256;
  p.idesc = make_idesc_i8(128, bn);
  const int k_iters = taps * p.c_chunks;
  const int n_tiles = (oc_pad + bn - 1) / bn;
  const long long total_tiles = (long long)m_tiles * n_tiles;
  const size_t a_bytes = (size_t)(p.dual ? 256 : 128) * p.BK, b_bytes = (size_t)(p.dual ? 192 : bn) * p.BK;
  const size_t w_all = (size_t)k_iters * b_bytes;
  // Weight-resident mode: when all K blocks of one channel tile's weights fit in 48 KB beside a useful
  // ring of activation tiles (two CTAs per SM are kept), a CTA loads them once and streams only
  // activations, which halves the bytes that have to reach shared memory per MAC. Larger weight
  // sets would force one CTA per SM, which measured slower than re-fetching the weights from L2.
  const int ctas_per_sm = 2;
  const size_t budget = 113 * 1024;
  p.w_resident = (!pl.tf32 && total_tiles >= 2LL * n_tiles && w_all <= 48 * 1024 &&
                  budget - kSmemHeader - 1024 - w_all >= 3 * a_bytes) ? 1 : 0;
  const size_t stage_bytes = p.w_resident ? a_bytes : a_bytes + b_bytes;
  const size_t ring_budget = budget - kSmemHeader - 1024 - (p.w_resident ? w_all : 0);
  int stages = (int)(ring_budget / stage_bytes);
  if (stages < 2) stages = 2;
  if (stages > kMaxStages) stages = kMaxStages;
  int grid = ctas_per_sm * sm_count;
  if (grid > total_tiles) grid = (int)total_tiles;
  if (p.w_resident) {
    grid = grid / n_tiles * n_tiles; // a CTA's channel tile must not change
    if (grid < n_tiles) grid = n_tiles;
  }
  // Split K: a launch with fewer tiles than CTA slots and a long K gives each tile to several CTAs (ConvGemmParams::
  // split_k): at least six K blocks per CTA, at most sixteen CTAs per tile, no more CTAs than slots. The exchange
  // through global memory costs about 3 us of latency (reductions, fence, count, read back) and a K block 0.4 us, so
  // only layers of 24 K blocks or more are split (3x3 with 512 channels: 36 blocks, 16.4 -> 10.3 us at batch 1; with 16
  // or 18 blocks the two forms measured equal, below that the split is slower). The weights are then not kept resident
  // (a CTA needs only its own K range once).
  p.split_k = 1;
  p.k_per = k_iters;
  if (conv_split_k_enabled() && !pl.tf32 && !pl.bf16 && !p.dual && k_iters >= 24 && total_tiles * 2 <= ctas_per_sm * sm_count) {
    int want = (int)((ctas_per_sm * sm_count) / total_tiles);
    if (want > 16) want = 16;
    if (want > k_iters / 6) want = k_iters / 6;
    if (want >= 2) {
      p.k_per = (k_iters + want - 1) / want;
      p.split_k = (k_iters + p.k_per - 1) / p.k_per;
      if (p.split_k < 2) {
        p.split_k = 1;
        p.k_per = k_iters;
      }
    }
  }
  if (p.split_k > 1) {
    if (p.w_resident) {
      p.w_resident = 0;
      stages = (int)((budget - kSmemHeader - 1024) / (a_bytes + b_bytes));
      if (stages < 2) stages = 2;
      if (stages > kMaxStages) stages = kMaxStages;
    }
    grid = (int)total_tiles * p.split_k;
    pl.ws_tiles = (int)total_tiles;
  }
  const size_t stage_bytes_final = p.w_resident ? a_bytes : a_bytes + b_bytes;
  const long long iters_per_cta = p.split_k > 1 ? p.k_per
                                                : ((total_tiles + grid - 1) / grid) * k_iters * (pl.tf32 ? 3 : 1);
  if (stages > iters_per_cta) stages = (int)iters_per_cta;
  if (stages < 1) stages = 1;
  p.stages = stages;
  pl.smem = kSmemHeader + 1024 + (p.w_resident ? w_all : 0) + stages * stage_bytes_final;
  pl.grid = dim3((unsigned)grid, 1, 1);
}

inline void launch_conv_plan(const ConvPlan &pl, cudaStream_t stream, int sm_count) {
  if (pl.use_patch) {
    size_t total = (size_t)pl.p.M_total * pl.patch.kp;
    if (pl.patch.cv == 4 && pl.patch_elsize == 4)
      launch_k(patch_expand_tap_kernel<float>, grid_for(total / 4, 256, sm_count), 256, 0, stream, 
          reinterpret_cast<const float *>(pl.in), reinterpret_cast<float *>(pl.patch_buf), pl.split_lo, pl.patch);
    else if (pl.patch.cv == 4)
      launch_k(patch_expand_tap_kernel<uint16_t>, grid_for(total / 4, 256, sm_count), 256, 0, stream, 
          reinterpret_cast<const uint16_t *>(pl.in), reinterpret_cast<uint16_t *>(pl.patch_buf), nullptr, pl.patch);
    else if (pl.patch_elsize == 2)
      launch_k(patch_expand_kernel<uint16_t>, grid_for(total / 8, 256, sm_count), 256, 0, stream, 
          reinterpret_cast<const uint16_t *>(pl.in), reinterpret_cast<uint16_t *>(pl.patch_buf), pl.patch);
    else
      launch_k(patch_expand_i8_kernel, grid_for(total, 256, sm_count), 256, 0, stream, pl.in, pl.patch_buf, pl.patch);
  }
  const int threads = kConvThreads;
  PdlConvScope conv_class; // the tensor-core kernel and its helper passes may start while the predecessor finishes
  if (pl.tf32) {
    if (pl.split_src)
      launch_k(tf32_split_kernel, grid_for(pl.split_nvec, 256, sm_count), 256, 0, stream, 
        reinterpret_cast<const float4 *>(pl.split_src), reinterpret_cast<float4 *>(pl.split_hi),
        reinterpret_cast<float4 *>(pl.split_lo), pl.split_nvec);
    launch_k(conv_gemm_tf32x3_kernel, pl.grid, threads, pl.smem, stream, pl.tmA, pl.tmB, pl.tmA2, pl.tmB2, pl.p);
  } else if (pl.bf16) launch_k(conv_gemm_bf16_kernel, pl.grid, threads, pl.smem, stream, pl.tmA, pl.tmB, pl.p);
  else if (pl.p.split_k > 1 && (pl.p.fastq & 1)) launch_k(conv_gemm_i8_split_kernel<true>, pl.grid, threads, pl.smem, stream, pl.tmA, pl.tmB, pl.p);
  else if (pl.p.split_k > 1) launch_k(conv_gemm_i8_split_kernel<false>, pl.grid, threads, pl.smem, stream, pl.tmA, pl.tmB, pl.p);
  else if ((pl.p.fastq & 1) && pl.p.act == 1) launch_k(conv_gemm_i8_act_kernel<1>, pl.grid, threads, pl.smem, stream, pl.tmA, pl.tmB, pl.p);
  else if ((pl.p.fastq & 3) == 3 && pl.p.act == 0) launch_k(conv_gemm_i8_act_kernel<10>, pl.grid, threads, pl.smem, stream, pl.tmA, pl.tmB, pl.p);
  else if (!(pl.p.fastq & 1)) launch_k(conv_gemm_i8_wide_kernel, pl.grid, threads, pl.smem, stream, pl.tmA, pl.tmB, pl.p);
  else launch_k(conv_gemm_i8_kernel, pl.grid, threads, pl.smem, stream, pl.tmA, pl.tmB, pl.p);
}

inline void conv_kernel_setup_once() {
  static bool done = [] {
    TPUCB_CUDA(cudaFuncSetAttribute(conv_gemm_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    227 * 1024));
    TPUCB_CUDA(cudaFuncSetAttribute(conv_gemm_i8_act_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TPUCB_CUDA(cudaFuncSetAttribute(conv_gemm_i8_act_kernel<10>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    TPUCB_CUDA(cudaFuncSetAttribute(conv_gemm_i8_split_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    227 * 1024));
    TPUCB_CUDA(cudaFuncSetAttribute(conv_gemm_i8_split_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    227 * 1024));
    TPUCB_CUDA(cudaFuncSetAttribute(conv_gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    227 * 1024));
    TPUCB_CUDA(cudaFuncSetAttribute(conv_gemm_i8_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    227 * 1024));
    TPUCB_CUDA(cudaFuncSetAttribute(conv_gemm_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    227 * 1024));
    return true;
  }();
  (void)done;
}

} // namespace tpucb
