// Host-side plumbing shared by the interpreter translation units: error type,
// CUDA call checking, the device tensor record and launch sizing.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace tpucb {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

inline std::string strfmt(const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  return buf;
}

#define TPUCB_CUDA(call)                                                                       \
  do {                                                                                         \
    cudaError_t e__ = (call);                                                                  \
    if (e__ != cudaSuccess)                                                                    \
      throw ::tpucb::Error(::tpucb::strfmt("%s failed: %s (%s:%d)", #call,                     \
                                           cudaGetErrorString(e__), __FILE__, __LINE__));      \
  } while (0)

#define TPUCB_CHECK(cond, ...)                                            \
  do {                                                                    \
    if (!(cond)) throw ::tpucb::Error(::tpucb::strfmt(__VA_ARGS__));      \
  } while (0)

inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

// Device tensor. Mirrors the role of TensorData (include/tpuc/Interpreter/cpukernel.h:15-78):
// one per op result, owned by the interpreter, shared by producer and consumers.
// Storage is NHWC with channel pitch cp; logical shape is what the module text gave.
struct DevTensor {
  std::string name;
  int dtype = 2; // DType
  std::vector<int64_t> shape;
  int n = 1, c = 1, h = 1, w = 1, cp = 1;
  int slot_n = 1; // leading-dimension extent of one batch slot (n / the interpreter's max_batch_size)
  // Physical row layout: `wl` zero pixels, the w real pixels, then zeros up to `wphys` pixels.
  // Every tensor has wl = 0, wphys = w except the input of a few-channel stem convolution.
  int wl = 0, wphys = 1;
  void *dev = nullptr;
  bool owns = true;
  // fp32 tensors read by a TF32 x 3 convolution: the remainder part x - (upper 19 bits of x), same layout as `dev`,
  // and who fills it (0 nobody yet, 1 the producing kernel, 2 the first consuming convolution's split pass)
  void *lo_dev = nullptr;
  int lo_by = 0;
  bool padded_rows() const { return wl != 0 || wphys != w; }
  size_t elsize() const { return dtype == 0 ? 1 : (dtype == 1 ? 2 : 4); }
  size_t pixels() const { return (size_t)n * h * wphys; }
  size_t bytes() const { return pixels() * cp * elsize(); }
  size_t numel() const { return (size_t)n * c * h * w; }
};
using TensorPtr = std::shared_ptr<DevTensor>;

struct HostWeight {
  std::vector<float> data;
  std::vector<int64_t> shape;
};

// Whether launch_k marks its launches for programmatic dependent launch. Set per launch: the interpreter's option
// "pdl" says which class of kernels gets the mark (pdl_mode: 0 none, 1 the tensor-core convolution kernels, 2 all), and
// the code that launches a kernel of the convolution class says so with PdlConvScope.
inline bool &launch_pdl_flag() {
  static thread_local bool on = true;
  return on;
}

// Whether launch plans may split K over several CTAs (option "split_k" of the interpreter that builds them).
inline bool &conv_split_k_enabled() {
  static thread_local bool on = true;
  return on;
}

inline int &pdl_mode() {
  static thread_local int v = 1;
  return v;
}
// While one lives, launch_k marks launches when the mode includes the convolution class; afterwards as before.
struct PdlConvScope {
  bool before;
  PdlConvScope() : before(launch_pdl_flag()) { launch_pdl_flag() = pdl_mode() >= 1; }
  ~PdlConvScope() { launch_pdl_flag() = before; }
};

#ifdef __CUDACC__
// Launch of an op kernel. With the flag above the launch carries the programmatic stream serialisation
// attribute: the kernel may be scheduled while its predecessor in the stream is still running and orders itself
// behind it with pdl_wait (every kernel launched this way begins with pdl_prologue or places pdl_wait itself).
template <typename... KArgs, typename G, typename B, typename... Args>
inline void launch_k(void (*kernel)(KArgs...), G grid, B block, size_t smem, cudaStream_t stream, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const bool pdl = launch_pdl_flag();
  // The arguments are converted to the kernel's own parameter types and passed by address; without the attribute the
  // launch goes through the classic entry point.
  auto go = [&](KArgs... a) {
    void *pa[sizeof...(KArgs) + 1] = {(void *)&a...};
    return pdl ? cudaLaunchKernelExC(&cfg, (const void *)kernel, pa)
               : cudaLaunchKernel((const void *)kernel, cfg.gridDim, cfg.blockDim, pa, smem, stream);
  };
  TPUCB_CUDA(go(std::forward<Args>(args)...));
}
#endif

// Grid for a grid-stride kernel: a multiple of the SM count, capped by the work.
inline int grid_for(size_t work_items, int block, int sm_count) {
  size_t blocks = (work_items + block - 1) / block;
  size_t cap = (size_t)sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

} // namespace tpucb
