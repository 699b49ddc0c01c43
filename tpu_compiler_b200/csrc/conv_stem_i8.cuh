// INT8 convolution for stems with at most 4 input channels (the 3-channel first layer of
// ResNet / MobileNet / Darknet), same arithmetic as conv_gemm_i8_kernel (core/conv.cpp:80-104 of
// the reference followed by the per-channel requantisation of QuantizationArithmetic.cpp:849-871).
//
// With 3 channels an im2col TMA row would be 16 bytes, far too small for the TMA unit to be
// efficient, so here the A tile is built by CUDA threads: the input is stored with a 4-byte pixel
// (NHWC4), each of 128 threads owns one output pixel, gathers its kh x kw pixel words with bounds
// checks (zero padding) and writes them as kh rows of 32 bytes (kw <= 8 taps x 4 channels) into
// shared memory in the 32-byte-swizzled K-major layout the tensor core reads; a proxy fence hands
// the tile to tcgen05.mma (one K=32 step per filter row). Weights [kh][Cout_pad][32] arrive by one
// TMA copy, once per CTA: the kernel is persistent. The gathering warps then run the epilogue
// (channels on TMEM lanes, as in conv_gemm_i8_kernel). Two CTAs share an SM and overlap gather, MMA
// and epilogue.
#pragma once
#include "conv_gemm_i8.cuh"

namespace tpucb {

struct ConvStemParams {
  int M_total, OH, OW, H, W;
  int sh, sw, pt, pl, dh;
  int kh, kw;
  int BN, n_valid, ldc, c_off, act, tmem_cols, dual, fastq;
  int leaky_mp, leaky_rp, leaky_mn, leaky_rn;
  uint32_t idesc;
  const uint32_t *in; // NHWC4 int8, one 32-bit word per pixel
  const int32_t *bias, *mult, *rshift;
  int8_t *out;
  int *err;
};

constexpr int kStemThreads = 32 + 256; // warp 0: weights + MMA; warps 1..8: gather + epilogue

// Dual mode (p.dual, at most 64 output channels): the tile covers 256 pixels; the weight rows are
// fetched as [64 zero rows][64 weight rows][64 zero rows] per filter row, and the two 128-pixel halves
// fill TMEM lanes 0..63 and 64..127 (same construction as in conv_gemm_i8_kernel).
// FAST: the multiply-high requantisation (p.fastq bit 0 set), else the 64-bit multiply-add form
constexpr int kStemRows = 4; // filter rows whose loads are in flight together (7 measured slower: 252 -> 266 us)

template <bool FAST, bool RELU_ONLY = false>
__global__ void __launch_bounds__(kStemThreads, 2)
conv_stem_i8_kernel(const __grid_constant__ CUtensorMap tmB, const ConvStemParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw);

  const uint32_t bar_a = base;        // activation tile written (one arrival per gathering thread)
  const uint32_t bar_b = base + 8;    // weights landed (TMA)
  const uint32_t bar_acc = base + 16; // accumulator complete
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 24);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 28);
  const int m_tile = p.dual ? 256 : 128;
  const int subs = p.dual ? 2 : 1;
  const uint32_t w_rows = p.dual ? 192u : (uint32_t)p.BN;
  const uint32_t a_row_bytes = (uint32_t)m_tile * 32u;                 // one filter row of the pixel tile
  const uint32_t a_tiles = base + kSmemHeader;                           // kh x m_tile x 32 B
  const uint32_t b_tiles = a_tiles + (uint32_t)p.kh * a_row_bytes;       // kh x w_rows x 32 B

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Persistent: the CTA keeps its channel tile's weights (one TMA copy) and walks pixel tiles
  // tile = blockIdx.x + k * gridDim.x; the grid is a multiple of the channel-tile count, so the
  // channel tile (tile % n_tiles) never changes for a CTA.
  const int n_tiles = (p.n_valid + p.BN - 1) / p.BN;
  const int m_tiles = (p.M_total + m_tile - 1) / m_tile;
  int total_tiles = n_tiles * m_tiles; // set to 0 below when the launch is already marked as failed
  const int n0 = (int)(blockIdx.x % n_tiles) * p.BN;
  ConvGemmParams ep; // the shared epilogue reads these fields
  ep.BN = p.BN; ep.n_valid = p.n_valid; ep.act = p.act; ep.M_total = p.M_total; ep.ldc = p.ldc;
  ep.mult = p.mult; ep.bias = p.bias; ep.rshift = p.rshift;
  ep.leaky_mp = p.leaky_mp; ep.leaky_rp = p.leaky_rp; ep.leaky_mn = p.leaky_mn; ep.leaky_rn = p.leaky_rn;
  ep.out = p.out; ep.out2 = nullptr; ep.fastq = p.fastq;

  pdl_trigger(); // see conv_gemm_body: set-up overlaps the previous kernel's tail
  if (threadIdx.x == 0) {
    const int gave_up = *reinterpret_cast<volatile int *>(p.err); // read early, as in conv_gemm_body
    // every gathering thread arrives once per tile (also those without a pixel), so that the next
    // tile's MMAs cannot start before all epilogue warps have left the accumulator
    ptx::mbar_init(bar_a, (uint32_t)(kStemThreads - 32));
    ptx::mbar_init(bar_b, 1);
    ptx::mbar_init(bar_acc, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    *abort_flag = gave_up;
  }
  if (warp == 0) ptx::tcgen05_alloc(ptx::smem_u32(tmem_slot), (uint32_t)p.tmem_cols);
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (*abort_flag != 0) total_tiles = 0;
  // the weights do not depend on the previous kernel: their copy starts before the wait for it
  if (warp == 0 && lane == 0 && (int)blockIdx.x < total_tiles) {
    const uint32_t b_bytes = (uint32_t)p.kh * w_rows * 32u;
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    ptx::mbar_expect_tx(bar_b, b_bytes);
    ptx::tma_load_3d(b_tiles, &tmB, bar_b, 0, n0 - (p.dual ? 64 : 0), 0);
  }
  pdl_wait(); // the activations from here on

  if (warp == 0) {
    if (lane == 0 && (int)blockIdx.x < total_tiles) {
      bool ok = ptx::mbar_wait_bounded(bar_b, 0u, abort_flag);
      if (!ok) {
        // the copy is still owed: wait for it (bounded) before the CTA may release shared memory
        for (uint32_t it = 0; it < (1u << 20); ++it)
          if (ptx::mbar_try_wait(bar_b, 0u)) break;
        if (!*abort_flag) atomicExch(p.err, kErrFullWait);
        *abort_flag = 1;
      }
      int t = 0;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++t) {
        ok = ptx::mbar_wait_bounded(bar_a, (uint32_t)(t & 1), abort_flag);
        if (!ok) {
          if (!*abort_flag) atomicExch(p.err, kErrFullWait);
          *abort_flag = 1;
          break;
        }
        ptx::tcgen05_fence_after();
        for (int r = 0; r < p.kh; ++r)
          for (int sub = 0; sub < subs; ++sub) {
            // transposed product: weights are the A operand (M = channels), the gathered pixels B
            const uint32_t w_r = b_tiles + (uint32_t)r * w_rows * 32u + ((p.dual && sub == 0) ? 64u * 32u : 0u);
            const uint64_t adesc = make_kmajor_desc(w_r, 32);
            const uint64_t bdesc = make_kmajor_desc(a_tiles + (uint32_t)r * a_row_bytes + (uint32_t)sub * 4096u, 32);
            ptx::tcgen05_mma_i8(tmem_base, adesc, bdesc, p.idesc, (r > 0 || sub > 0) ? 1u : 0u);
          }
        ptx::tcgen05_commit(bar_acc);
      }
    }
  } else {
    const int g = threadIdx.x - 32; // thread g of 256 owns pixel g of the tile
    const int quarter = warp & 3;   // epilogue: 8 warps, two per TMEM lane quarter, alternating 32-pixel groups
    const int half = (warp - 1) >> 2;
    const int ch_base = p.dual ? (quarter & 1) * 32 : quarter * 32;
    const ChanConst cc = load_chan_const(ep, n0 + ch_base + lane);
    const TransposeSel ts = make_transpose_sel(lane);
    const uint32_t sw_bit = (uint32_t)((g >> 2) & 1); // 32-byte swizzle: 16-byte chunk ^= address bit 7
    uint8_t *a_row = smem + kSmemHeader + g * 32;
    int t = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++t) {
      const int m0 = (tile / n_tiles) * m_tile;
      // ---- gather (the previous tile's MMAs have retired: this thread saw bar_acc in its epilogue)
      if (g < m_tile) {
        const int m = m0 + g;
        const bool row_ok = m < p.M_total;
        int q = 0, pp = 0, nimg = 0;
        if (row_ok) {
          const int tt = m / p.OW;
          q = m - tt * p.OW;
          nimg = tt / p.OH;
          pp = tt - nimg * p.OH;
        }
        const int x0 = q * p.sw - p.pl;
        const int y0 = pp * p.sh - p.pt;
        const bool x_inside = x0 >= 0 && x0 + 8 <= p.W; // all eight words in range (weights past kw are zero): no per-tap checks
        // Four filter rows at a time: their 32 loads are all issued before the first is used, so that a thread has
        // four rows' worth of memory latency in flight instead of one (the row count is a run-time value; a plain
        // loop over the rows would wait for each row's loads before it starts the next).
        for (int r0 = 0; r0 < p.kh; r0 += kStemRows) {
          uint32_t w[kStemRows][8];
#pragma unroll
          for (int j = 0; j < kStemRows; ++j) {
#pragma unroll
            for (int s = 0; s < 8; ++s) w[j][s] = 0u;
            const int r = r0 + j;
            const int y = y0 + r * p.dh;
            if (r < p.kh && row_ok && y >= 0 && y < p.H) {
              const uint32_t *src = p.in + ((size_t)nimg * p.H + y) * p.W + x0;
              if (x_inside) {
#pragma unroll
                for (int s = 0; s < 8; ++s) w[j][s] = __ldg(src + s);
              } else {
#pragma unroll
                for (int s = 0; s < 8; ++s)
                  if (s < p.kw && x0 + s >= 0 && x0 + s < p.W) w[j][s] = __ldg(src + s);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < kStemRows; ++j) {
            if (r0 + j < p.kh) {
              uint4 *dst = reinterpret_cast<uint4 *>(a_row + (size_t)(r0 + j) * a_row_bytes);
              dst[0 ^ sw_bit] = make_uint4(w[j][0], w[j][1], w[j][2], w[j][3]);
              dst[1 ^ sw_bit] = make_uint4(w[j][4], w[j][5], w[j][6], w[j][7]);
            }
          }
        }
        // make the generic-proxy writes visible to the tensor core (async proxy)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      ptx::tcgen05_fence_before(); // orders this thread's accumulator reads of the previous tile
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_a) : "memory");

      // ---- epilogue
      ok = ptx::mbar_wait_bounded(bar_acc, (uint32_t)(t & 1), abort_flag);
      if (!ok && !*abort_flag) {
        atomicExch(p.err, kErrAccWait);
        *abort_flag = 1;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tcgen05_fence_after();
      const int m0e = m0 + (p.dual ? 128 * (quarter >> 1) : 0);
      const int ch4 = n0 + ch_base + (lane >> 2) * 4;
      if (n0 + ch_base < p.n_valid && m0e < p.M_total) {
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        int8_t *out4 = p.out + (size_t)m0e * p.ldc + p.c_off + ch4;
        const bool ch4_ok = ch4 < p.n_valid;
        if (RELU_ONLY || p.act == 1) epilogue_channels_impl<1, FAST>(ep, lane_addr, out4, ch4_ok, m0e, half, 2, lane, cc, ts, 128);
        else if (p.act == 2) epilogue_channels_impl<2, FAST>(ep, lane_addr, out4, ch4_ok, m0e, half, 2, lane, cc, ts, 128);
        else if (FAST && (p.fastq & 2)) epilogue_channels_impl<0, FAST, true>(ep, lane_addr, out4, ch4_ok, m0e, half, 2, lane, cc, ts, 128);
        else epilogue_channels_impl<0, FAST>(ep, lane_addr, out4, ch4_ok, m0e, half, 2, lane, cc, ts, 128);
      }
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tcgen05_fence_after();
    ptx::tcgen05_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

} // namespace tpucb
