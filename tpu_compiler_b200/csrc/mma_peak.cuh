// Microbenchmark of the INT8 tensor pipe: every SM issues a long chain of
// tcgen05.mma.cta_group::1.kind::i8 (M=128, N=n_cols, K=32) on operand tiles that already sit in
// shared memory, so nothing but the tensor pipe (and its shared-memory operand reads) is timed.
// The driver-measured peaks carry no INT8 figure; this gives the roofline denominator for the
// convolution kernel as measured on the device it runs on.
#pragma once
#include "conv_gemm_i8.cuh"

namespace tpucb {

__global__ void __launch_bounds__(64, 1) mma_i8_peak_kernel(int iters, int n_cols, uint32_t idesc, int *err) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw);
  const uint32_t bar = base;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 16);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 20);
  const uint32_t a_tile = base + 1024;            // 128 rows x 128 B
  const uint32_t b_tile = a_tile + 128 * 128;     // n_cols rows x 128 B
  // operands: any values do; zero them so the accumulators stay finite
  for (int i = threadIdx.x; i < (128 + n_cols) * 128 / 16; i += blockDim.x)
    reinterpret_cast<uint4 *>(smem + 1024)[i] = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    ptx::mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  const int warp = threadIdx.x >> 5;
  if (warp == 0) ptx::tcgen05_alloc(ptx::smem_u32(tmem_slot), 256u);
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) {
    const uint64_t adesc = make_kmajor_desc(a_tile, 128);
    const uint64_t bdesc = make_kmajor_desc(b_tile, 128);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        ptx::tcgen05_mma_i8(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                            (it > 0 || k > 0) ? 1u : 0u);
    }
    ptx::tcgen05_commit(bar);
    bool ok = false;
    for (int rep = 0; rep < 64 && !ok; ++rep) ok = ptx::mbar_wait_bounded(bar, 0u, abort_flag);
    if (!ok) atomicExch(err, kErrAccWait);
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tcgen05_fence_after();
    ptx::tcgen05_dealloc(tmem_base, 256u);
  }
}

} // namespace tpucb
