// Two-SM variant of the INT8 implicit-GEMM convolution (same arithmetic and epilogue as
// conv_gemm_i8_kernel; reference: core/conv.cpp:80-104 + QuantizationArithmetic.cpp:849-871).
//
// A cluster of two CTAs (one per SM) computes a 256-channel x 256-pixel tile with
// tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 32 per instruction): CTA r holds the weights of
// channels [128 r, 128 r + 128) and the activations of pixels [128 r, 128 r + 128) of the tile, the
// tensor core reads both CTAs' shared memory, and CTA r's TMEM receives its 128 channels x all 256
// pixels. Per MAC this needs half the shared-memory fill of the one-SM 128 x 128 tile, which is
// what bounds the layers with a long K loop. No multicast copies: every CTA loads only its own
// halves; completion of both CTAs' copies is counted on the leader's barrier (copies are issued
// with .cta_group::2 so that they may signal the peer CTA's barrier).
//
// Protocol (barriers live at the same shared-memory offsets in both CTAs):
//   full[s]      leader's copy only; one arrival (the leader's expect_tx of both CTAs' bytes)
//   empty[s]     one per CTA; the leader's MMA thread commits to its own and to the peer's
//   acc_full[b]  one per CTA; committed by the leader after the tile's last MMA
//   acc_empty[b] leader's copy only; one arrival per epilogue warp of both CTAs (32)
// Every wait is bounded and also gives up when the launch's error word is set; all exit paths meet
// at a cluster barrier before TMEM is released, so no CTA leaves while its peer may still touch it.
#pragma once
#include "conv_gemm_i8.cuh"

namespace tpucb {

namespace ptx {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the shared::cluster address of `addr` (a shared address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// copies whose completion bytes are counted on a barrier of the peer CTA (cluster address `bar`)
__device__ __forceinline__ void tma2_load_2d(uint32_t dst, const void *tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(uint32_t dst, const void *tmap, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma2_load_im2col_4d(uint32_t dst, const void *tmap, uint32_t bar, int c, int w,
                                                    int h, int n, uint16_t off_w, uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}
__device__ __forceinline__ void tcgen05_alloc2(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrival on `cluster_bar` (either CTA's barrier) once all MMAs issued so far have retired
__device__ __forceinline__ void tcgen05_commit2(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma2_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// The same with the descriptors passed as (low, high) words, the high word shared: the issuing thread's loop
// advances 32-bit start-address fields only.
template <bool ACCUMULATE>
__device__ __forceinline__ void tcgen05_mma2_i8_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                                     uint32_t idesc, uint32_t accumulate) {
  if (ACCUMULATE) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %4, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(0u)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %4, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(0u), "r"(accumulate)
        : "memory");
  }
}
template <int KSTEPS>
__device__ __forceinline__ void tcgen05_mma2_i8_kblock(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                                       uint32_t idesc, uint32_t accumulate_first) {
  tcgen05_mma2_i8_lohi<false>(d_tmem, a_lo, b_lo, hi, idesc, accumulate_first);
#pragma unroll
  for (int k = 1; k < KSTEPS; ++k) tcgen05_mma2_i8_lohi<true>(d_tmem, a_lo + 2 * k, b_lo + 2 * k, hi, idesc, 1u);
}

} // namespace ptx

constexpr int kPairEpilogueWarps = 16;
// producer (activations), MMA issuer, 16 epilogue warps, second producer (weights)
constexpr int kPairThreads = 64 + 32 * kPairEpilogueWarps + 32;
constexpr int kPairWeightWarp = 2 + kPairEpilogueWarps;

// Bounded wait that also ends when this CTA or any CTA of the launch has recorded an error.
__device__ __forceinline__ bool pair_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          const volatile int *err) {
  for (uint32_t it = 0; it < (1u << 20); ++it) {
    if (ptx::mbar_try_wait_cluster(bar, parity)) return true;
    if ((it & 255u) == 255u && (*abort_flag || *err)) return false;
  }
  return false;
}

template <bool PROF>
__device__ __forceinline__ void conv_gemm2_body(const CUtensorMap &tmA, const CUtensorMap &tmB, const ConvGemmParams &p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw);

  const uint32_t bar_full = base;            // kMaxStages x 8 B (leader's copy is the one in use)
  const uint32_t bar_empty = base + 64;      // kMaxStages x 8 B
  const uint32_t bar_acc_full = base + 128;  // 2 x 8 B
  const uint32_t bar_acc_empty = base + 144; // 2 x 8 B (leader's copy is the one in use)
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 168);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 172);
  const volatile int *gerr = reinterpret_cast<const volatile int *>(p.err);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank(); // 0 = leader
  const int cluster_id = (int)(blockIdx.x >> 1);
  const int n_clusters = (int)(gridDim.x >> 1);
  const int n_tiles = p.n_valid / 256;
  const int m_tiles = (p.M_total + 255) / 256;
  const int total_tiles = n_tiles * m_tiles;
  const uint32_t half_bytes = 128u * (uint32_t)p.BK;   // one operand half of one CTA
  const uint32_t stage_bytes = 2u * half_bytes;         // weights + activations of this CTA
  const uint32_t tiles = base + kSmemHeader;
  const int taps = p.kh * p.kw;
  const int k_iters = taps * p.c_chunks;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(bar_acc_full + 8 * b, 1);
      ptx::mbar_init(bar_acc_empty + 8 * b, 2 * kPairEpilogueWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) ptx::tcgen05_alloc2(ptx::smem_u32(tmem_slot), 512u);
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::cluster_arrive(); // the peer's barriers are initialised before anything remote touches them
  ptx::cluster_wait();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // One thread can start only one bulk tensor copy per ~410 cycles whatever its size (measured), and a K block
  // of a tile pair is 534 tensor-pipe cycles: the activation half and the weight half of every stage are
  // started by two threads of two warps. The activation thread of the leader arms the stage's barrier.
  auto produce = [&](const bool do_a) {
    {
      long long pf_p0 = PROF ? clock64() : 0ll, pf_pwait = 0;
      int it = 0, ps = 0;
      uint32_t pph = 0;
      bool ok = *gerr == 0;
      const uint32_t leader_full = ptx::mapa(bar_full, 0u);
      for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters) {
        const int m0 = (tile / n_tiles) * 256 + (int)rank * 128; // this CTA's 128 pixels
        const int n0 = (tile % n_tiles) * 256 + (int)rank * 128; // this CTA's 128 channels
        int n_img = 0, h_base = 0, w_base = 0;
        if (p.a_mode == 1) {
          int q = m0 % p.OW;
          int t = m0 / p.OW;
          int pp = t % p.OH;
          n_img = t / p.OH;
          w_base = q * p.sw - p.pl;
          h_base = pp * p.sh - p.pt;
        }
        int tap = 0, tr = 0, ts = 0, chunk = 0; // running counters: no divisions in this loop
        for (int kit = 0; kit < k_iters; ++kit, ++it) {
          const long long pf_e0 = PROF ? clock64() : 0ll;
          if (it >= p.stages) {
            if (!pair_wait(bar_empty + 8 * ps, pph ^ 1u, abort_flag, gerr)) {
              if (!*abort_flag && !*gerr) atomicExch(p.err, kErrEmptyWait);
              *abort_flag = 1;
              ok = false;
              break;
            }
          }
          if (PROF) pf_pwait += clock64() - pf_e0;
          const int c0 = chunk * p.BK;
          const uint32_t w_dst = tiles + (uint32_t)ps * stage_bytes; // weights first, activations behind
          const uint32_t a_dst = w_dst + half_bytes;
          const uint32_t fb = leader_full + 8 * ps; // the leader's barrier
          if (do_a) {
            if (rank == 0) ptx::mbar_expect_tx(bar_full + 8 * ps, 2u * stage_bytes);
            if (p.a_mode == 1)
              ptx::tma2_load_im2col_4d(a_dst, &tmA, fb, c0, w_base, h_base, n_img, (uint16_t)(ts * p.dw),
                                       (uint16_t)(tr * p.dh));
            else
              ptx::tma2_load_2d(a_dst, &tmA, fb, c0, m0);
          } else {
            ptx::tma2_load_3d(w_dst, &tmB, fb, c0, tap, n0);
          }
          if (++chunk == p.c_chunks) {
            chunk = 0;
            ++tap;
            if (++ts == p.kw) {
              ts = 0;
              ++tr;
            }
          }
          if (++ps == p.stages) {
            ps = 0;
            pph ^= 1u;
          }
        }
      }
      if (PROF && do_a && rank == 0) {
        atomicAdd(&g_conv_prof[5], (unsigned long long)(clock64() - pf_p0));
        atomicAdd(&g_conv_prof[6], (unsigned long long)pf_pwait);
      }
      if (!ok || *abort_flag) {
        // Failure path: give copies that are still in flight time to land before shared memory is
        // released (the leader also waits for every stage it armed).
        if (rank == 0) {
          int first = it > p.stages ? it - p.stages : 0;
          for (int j = first; j < it; ++j)
            for (uint32_t w = 0; w < (1u << 16); ++w)
              if (ptx::mbar_try_wait_cluster(bar_full + 8 * (j % p.stages), (uint32_t)(j / p.stages) & 1u)) break;
        } else {
          for (int w = 0; w < 64; ++w) __nanosleep(1000);
        }
      }
    }
  };
  if (warp == 0) {
    // ------------------------------------------------------------ producer of the activation halves
    if (lane == 0) produce(true);
  } else if (warp == kPairWeightWarp) {
    // ------------------------------------------------------------ producer of the weight halves
    if (lane == 0) produce(false);
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0 && *gerr == 0) {
      int it = 0, t = 0, ms = 0;
      uint32_t mph = 0;
      bool ok = true;
      const uint64_t desc0 = make_kmajor_desc(tiles, p.BK); // stages differ in the start-address field only
      const uint32_t desc_hi = (uint32_t)(desc0 >> 32), desc_ring_lo = (uint32_t)desc0;
      const uint32_t stage_step = stage_bytes >> 4, half_step = half_bytes >> 4;
      const int ksteps = p.BK / 32;
      const uint32_t peer_empty0 = ptx::mapa(bar_empty, 1u);
      const uint32_t peer_acc_full = ptx::mapa(bar_acc_full, 1u);
      uint32_t m_full = bar_full, m_empty = bar_empty, m_peer_empty = peer_empty0, ring_lo = desc_ring_lo;
      long long pf_t0 = PROF ? clock64() : 0ll, pf_wait = 0, pf_accwait = 0, pf_blocks = 0;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters, ++t) {
        const int buf = t & 1;
        const long long pf_a0 = PROF ? clock64() : 0ll;
        if (t >= 2) {
          if (!pair_wait(bar_acc_empty + 8 * buf, (uint32_t)(((t >> 1) - 1) & 1), abort_flag, gerr)) {
            if (!*abort_flag && !*gerr) atomicExch(p.err, kErrAccWait);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after();
        }
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * 256u;
        if (PROF) pf_accwait += clock64() - pf_a0;
        for (int kit = 0; kit < k_iters; ++kit, ++it) {
          const long long pf_w0 = PROF ? clock64() : 0ll;
          if (!ptx::mbar_try_wait_cluster(m_full, mph) && !pair_wait(m_full, mph, abort_flag, gerr)) {
            if (!*abort_flag && !*gerr) atomicExch(p.err, kErrFullWait);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if (PROF) {
            pf_wait += clock64() - pf_w0;
            ++pf_blocks;
          }
          ptx::tcgen05_fence_after();
          // transposed product: weights are the A operand (M = 256 channels over the two CTAs), the
          // activations the B operand (N = 256 pixels, 128 rows of it in each CTA)
          const uint32_t acc_first = kit > 0 ? 1u : 0u;
          if (ksteps == 4) ptx::tcgen05_mma2_i8_kblock<4>(d_tmem, ring_lo, ring_lo + half_step, desc_hi, p.idesc, acc_first);
          else if (ksteps == 2) ptx::tcgen05_mma2_i8_kblock<2>(d_tmem, ring_lo, ring_lo + half_step, desc_hi, p.idesc, acc_first);
          else ptx::tcgen05_mma2_i8_kblock<1>(d_tmem, ring_lo, ring_lo + half_step, desc_hi, p.idesc, acc_first);
          ptx::tcgen05_commit2(m_empty);   // frees the stage in both CTAs once the MMAs retire
          ptx::tcgen05_commit2(m_peer_empty);
          m_full += 8;
          m_empty += 8;
          m_peer_empty += 8;
          ring_lo += stage_step;
          if (++ms == p.stages) {
            ms = 0;
            mph ^= 1u;
            m_full = bar_full;
            m_empty = bar_empty;
            m_peer_empty = peer_empty0;
            ring_lo = desc_ring_lo;
          }
        }
        if (ok) {
          ptx::tcgen05_commit2(bar_acc_full + 8 * buf);
          ptx::tcgen05_commit2(peer_acc_full + 8 * buf);
        }
      }
      if (PROF) {
        atomicAdd(&g_conv_prof[0], (unsigned long long)(clock64() - pf_t0));
        atomicAdd(&g_conv_prof[1], (unsigned long long)pf_wait);
        atomicAdd(&g_conv_prof[2], (unsigned long long)pf_accwait);
        atomicAdd(&g_conv_prof[3], (unsigned long long)pf_blocks);
        atomicAdd(&g_conv_prof[4], 1ull);
      }
    }
  } else if (warp < kPairWeightWarp) {
    // ------------------------------------------------------------ epilogue (16 warps per CTA)
    const int quarter = warp & 3;        // TMEM lanes (= channels of this CTA's half) this warp may read
    const int cgroup = (warp - 2) >> 2;  // 0..3: takes the 32-pixel column groups cgroup, cgroup + 4
    const TransposeSel ts = make_transpose_sel(lane);
    const uint32_t leader_acc_empty = ptx::mapa(bar_acc_empty, 0u);
    ChanConst cc;
    int staged_n0 = -1;
    int t = 0;
    bool ok = *gerr == 0;
    for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters, ++t) {
      const int m0 = (tile / n_tiles) * 256;
      const int n0 = (tile % n_tiles) * 256 + (int)rank * 128;
      const int buf = t & 1;
      if (n0 != staged_n0) {
        cc = load_chan_const(p, n0 + quarter * 32 + lane);
        staged_n0 = n0;
      }
      const long long pf_q0 = PROF ? clock64() : 0ll;
      ok = pair_wait(bar_acc_full + 8 * buf, (uint32_t)((t >> 1) & 1), abort_flag, gerr);
      if (PROF && warp == 2 && lane == 0 && rank == 0) atomicAdd(&g_conv_prof[7], (unsigned long long)(clock64() - pf_q0));
      const long long pf_q1 = PROF ? clock64() : 0ll;
      if (!ok && !*abort_flag && !*gerr) {
        atomicExch(p.err, kErrAccWait);
        *abort_flag = 1;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tcgen05_fence_after();
      const int ch4 = n0 + quarter * 32 + (lane >> 2) * 4;
      const uint32_t lane_addr = tmem_base + (uint32_t)buf * 256u + ((uint32_t)(quarter * 32) << 16);
      int8_t *out4 = p.out + (size_t)m0 * p.ldc + p.c_off + ch4;
      const bool ch4_ok = ch4 < p.n_valid;
      if (p.act == 1) epilogue_channels<1>(p, lane_addr, out4, ch4_ok, m0, cgroup, 4, lane, cc, ts, 256);
      else if (p.act == 2) epilogue_channels<2>(p, lane_addr, out4, ch4_ok, m0, cgroup, 4, lane, cc, ts, 256);
      else epilogue_channels<0>(p, lane_addr, out4, ch4_ok, m0, cgroup, 4, lane, cc, ts, 256);
      if (PROF && warp == 2 && lane == 0 && rank == 0) atomicAdd(&g_conv_prof[8], (unsigned long long)(clock64() - pf_q1));
      // hand the accumulator buffer back to the leader's MMA issuer
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(leader_acc_empty + 8 * buf);
    }
  }

  // Teardown: nobody releases shared memory or TMEM while the peer may still read or signal it.
  ptx::tcgen05_fence_before();
  __syncthreads();
  __syncwarp();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tcgen05_dealloc2(tmem_base, 512u);
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
conv_gemm2_i8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const ConvGemmParams p) {
  conv_gemm2_body<false>(tmA, tmB, p);
}
// the same with the loop-profile counters on (see conv_gemm_prof_kernel; the leader CTA of each pair reports)
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
conv_gemm2_prof_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const ConvGemmParams p) {
  conv_gemm2_body<true>(tmA, tmB, p);
}

} // namespace tpucb
