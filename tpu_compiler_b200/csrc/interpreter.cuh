// Host-side interpreter: the device counterpart of MlirModuleInterpreter
// (include/tpuc/MlirModuleInterpreter.h:32-83, lib/Dialect/TPU/Interpreter/
// MlirModuleInterpreter.cpp) and of the CPUOpKernel hierarchy
// (include/tpuc/Interpreter/cpukernel.h:87-159). One OpKernel object per op, built at
// loadModule time from the op's attributes and operands; invoke() enqueues the op's
// CUDA kernel(s) on the interpreter's stream. All activations stay resident so that
// get_tensor / get_all_tensor work as in the reference.
#pragma once
#include "conv_plan.cuh"
#include "f32_kernels.cuh"
#include "calib_kernels.cuh"
#include "extra_kernels.cuh"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <sstream>

namespace tpucb {

using Attrs = std::map<std::string, std::string>;

struct ParsedOp {
  std::string type, name;
  std::vector<std::string> in;
  std::vector<int64_t> shape;
  std::string dtype = "FP32";
  Attrs attrs;
  std::string line; // the text the op was parsed from
  int geti(const char *k, int def = 0) const {
    auto it = attrs.find(k);
    return it == attrs.end() ? def : atoi(it->second.c_str());
  }
  double getf(const char *k, double def = 0) const {
    auto it = attrs.find(k);
    return it == attrs.end() ? def : atof(it->second.c_str());
  }
  std::string gets(const char *k, const char *def = "") const {
    auto it = attrs.find(k);
    return it == attrs.end() ? std::string(def) : it->second;
  }
  // comma-separated integer list attribute (I32ArrayAttr in the reference's op definitions)
  std::vector<int> getl(const char *k) const {
    std::vector<int> v;
    auto it = attrs.find(k);
    if (it == attrs.end()) return v;
    std::stringstream ss(it->second);
    std::string tok;
    while (std::getline(ss, tok, ',')) v.push_back(atoi(tok.c_str()));
    return v;
  }
};

class Interpreter;

// Device counterpart of CPUOpKernel: shape / name / op_type / datatype are public as in
// cpukernel.h:144-149; invoke() is the one virtual the driver loop calls (cpukernel.h:101).
class OpKernel {
public:
  virtual ~OpKernel() {}
  virtual void invoke(cudaStream_t s) = 0;
  // what the op loops call: an op whose result is currently supplied from outside (see set_tensor_async_i8) is skipped
  void run(cudaStream_t s) {
    if (!disabled) invoke(s);
  }
  virtual int kernel_launches() const { return 1; }
  bool disabled = false;
  std::string name, op_type;
  std::vector<int64_t> shape;
  int datatype = DT_F32;
  TensorPtr result;
  double alg_ops = 0, alg_bytes = 0; // algorithmic work of one invoke (for roofline reports)
  bool dirty = true;                 // cpukernel.h:152: not yet run since it was built (fastInvokeAllBatch clears it)
  std::string line;                  // the module-text line the op was built from (dump)
};

inline int dtype_from_string(const std::string &s) {
  if (s == "INT8" || s == "UINT8") return DT_I8;
  if (s == "BF16") return DT_BF16;
  return DT_F32;
}
inline const char *dtype_to_string(int dt) { return dt == DT_I8 ? "INT8" : (dt == DT_BF16 ? "BF16" : "FP32"); }

class Interpreter {
public:
  explicit Interpreter(int device) : device_(device) {
    TPUCB_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    TPUCB_CUDA(cudaGetDeviceProperties(&prop, device));
    TPUCB_CHECK(prop.major == 10, "this backend is written for sm_100a (B200); device %d is sm_%d%d",
                device, prop.major, prop.minor);
    sm_count = prop.multiProcessorCount;
    TPUCB_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    TPUCB_CUDA(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      TPUCB_CUDA(cudaEventCreateWithFlags(&upload_done[i], cudaEventDisableTiming));
      TPUCB_CUDA(cudaEventCreateWithFlags(&staging_free[i], cudaEventDisableTiming));
    }
    TPUCB_CUDA(cudaMalloc(&d_err, sizeof(int)));
    TPUCB_CUDA(cudaMemset(d_err, 0, sizeof(int)));
  }
  ~Interpreter() {
    cudaSetDevice(device_);
    cudaStreamSynchronize(stream);
    if (graph_exec) cudaGraphExecDestroy(graph_exec);
    kernels.clear();
    for (auto &kv : tensors)
      if (kv.second->owns && kv.second->dev) cudaFree(kv.second->dev);
    for (void *p : allocations) cudaFree(p);
    if (staging) cudaFree(staging);
    for (int i = 0; i < 2; ++i) {
      if (async_staging[i]) cudaFree(async_staging[i]);
      cudaEventDestroy(upload_done[i]);
      cudaEventDestroy(staging_free[i]);
    }
    cudaFree(d_err);
    cudaStreamDestroy(copy_stream);
    cudaStreamDestroy(stream);
  }

  void bind() {
    TPUCB_CUDA(cudaSetDevice(device_));
    pdl_mode() = use_pdl;
    launch_pdl_flag() = use_pdl >= 2;
    conv_split_k_enabled() = split_k && selftest_lost_arrival == 0; // the self-test needs tiles that follow one another in a CTA
  }
  int device() const { return device_; }

  // ---- device memory owned by the interpreter
  void *dalloc(size_t bytes) {
    void *p = nullptr;
    TPUCB_CUDA(cudaMalloc(&p, bytes ? bytes : 16));
    allocations.push_back(p);
    return p;
  }
  template <class T> T *upload(const std::vector<T> &v) {
    T *p = (T *)dalloc(v.size() * sizeof(T));
    if (!v.empty()) TPUCB_CUDA(cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    return p;
  }
  float *ensure_staging(size_t bytes) {
    if (bytes > staging_bytes) {
      TPUCB_CUDA(cudaStreamSynchronize(stream));
      if (staging) cudaFree(staging);
      TPUCB_CUDA(cudaMalloc(&staging, bytes));
      staging_bytes = bytes;
    }
    return (float *)staging;
  }

  // Row layout requested for a tensor by its (sole) consumer: channel pitch and zero-padded rows.
  struct RowLayout {
    int cp = 0, wl = 0, wphys = 0;
  };
  std::map<std::string, RowLayout> layout_requests;

  TensorPtr make_tensor(const std::string &name, const std::vector<int64_t> &shape, int dtype) {
    auto t = std::make_shared<DevTensor>();
    t->name = name;
    t->dtype = dtype;
    t->shape = shape;
    TPUCB_CHECK(shape.size() >= 1 && shape.size() <= 4, "tensor %s: rank %zu not supported", name.c_str(),
                shape.size());
    int64_t d[4] = {1, 1, 1, 1};
    for (size_t i = 0; i < shape.size(); ++i) d[i] = shape[i];
    t->n = (int)d[0];
    t->c = (int)d[1];
    t->h = (int)d[2];
    t->w = (int)d[3];
    // INT8 and BF16 tensors share a channel pitch (a multiple of 16) so that the conversions
    // between them run on whole 16-element vectors; fp32 pads to one 16-byte vector.
    int lanes = dtype == DT_F32 ? 4 : 16;
    t->cp = round_up(t->c, lanes);
    t->wphys = t->w;
    auto lr = layout_requests.find(name);
    if (lr != layout_requests.end() && dtype == DT_I8) {
      t->cp = lr->second.cp;
      t->wl = lr->second.wl;
      t->wphys = lr->second.wphys;
    }
    TPUCB_CUDA(cudaMalloc(&t->dev, t->bytes()));
    TPUCB_CUDA(cudaMemset(t->dev, 0, t->bytes()));
    return t;
  }

  const HostWeight &weight(const std::string &name) const {
    auto it = weights.find(name);
    TPUCB_CHECK(it != weights.end(), "weight '%s' was not registered", name.c_str());
    return it->second;
  }
  bool has_weight(const std::string &name) const {
    return !name.empty() && name != "-" && weights.count(name);
  }
  TensorPtr tensor(const std::string &name) const {
    auto it = tensors.find(name);
    TPUCB_CHECK(it != tensors.end(), "tensor '%s' not found", name.c_str());
    return it->second;
  }

  void load_module(const std::string &text);
  // one op of the module: builds its kernel from the operands already present and registers its result
  // (the body of the CPUOpKernel constructors, cpukernel.h:89-90); returns the index in `kernels`, or -1 for a
  // reshape, which is an alias and has no kernel
  int add_op(const ParsedOp &op);
  void reset_module();
  void finish_module();
  // slot < 0: the whole tensor (every batch slot); else the images of one slot (MlirModuleInterpreter::setTensor /
  // getTensor with bidx, MlirModuleInterpreter.cpp:407-427)
  void set_tensor(const std::string &name, const float *data, size_t numel, int slot = -1);
  void get_tensor(const std::string &name, float *out, size_t numel, int slot = -1);
  void fast_invoke_all_batch(const std::string &name, int batch);
  void launch_all();
  void launch_to(const std::string &name);
  void sync_and_check();
  void invalidate_graph() {
    if (graph_exec) {
      cudaGraphExecDestroy(graph_exec);
      graph_exec = nullptr;
    }
  }

  int device_;
  // MlirModuleInterpreter(int32_t batch) (MlirModuleInterpreter.h:35): the reference keeps `batch` copies ("slots") of
  // every activation and runs the kernels on one slot at a time. Here slot b is image group b of ONE device tensor
  // whose leading dimension is max_batch x the module's, so one launch covers every slot.
  int max_batch = 1;
  std::map<std::string, std::string> producer_type;
  std::map<std::string, int> uses;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  int *d_err = nullptr;
  bool use_graph = true;
  // Programmatic dependent launch (option "pdl"): a kernel launched with the attribute may be scheduled while its
  // predecessor in the stream is still running; it sets up its barriers and tensor memory and then waits for that
  // kernel's results (pdl_wait). 1 (default): the tensor-core convolution kernels carry the attribute; 0: none; 2: every
  // kernel. Measured per class (ms per graph launch, off / all / convolutions only): INT8 ResNet-50 batch 1 0.379 / 0.348 /
  // 0.334, batch 32 0.697 / 0.668 / 0.657, batch 256 3.074 / 3.193 / 3.063; YOLOv4-style batch 8 2.361 / 2.412 / 2.265;
  // MobileNet-v2 batch 32 0.526 / 0.504 / 0.485. On the memory-bound kernels alone the attribute costs 1-5%: their blocks
  // then take their SMs in the order the predecessor's CTAs leave instead of evenly.
  int use_pdl = 1;
  cudaGraphExec_t capture_graph();
  // Self-test (option "selftest_lost_arrival", read by the next load_module): > 0 makes every INT8 tensor-core
  // convolution built from then on lose its accumulator hand-back and wait only that many rounds of 1024 polls
  // (ConvGemmParams::wait_rounds / lose_arrival), so that a launch ends with a bounded-wait error status.
  int selftest_lost_arrival = 0;
  bool split_k = true; // set before load_module: launches with few tiles and a long K share each tile among CTAs
  // partial-sum workspaces of the split-K plans (zero between launches; cleared again after a failed launch)
  std::vector<std::pair<void *, size_t>> split_ws;
  void attach_split_ws(ConvPlan &pl) {
    if (pl.p.split_k <= 1) return;
    const size_t bytes = (size_t)pl.ws_tiles * 128 * 128 * sizeof(int32_t), cbytes = (size_t)pl.ws_tiles * sizeof(unsigned int);
    pl.p.ws = (int32_t *)dalloc(bytes);
    pl.p.ws_count = (unsigned int *)dalloc(cbytes);
    TPUCB_CUDA(cudaMemset(pl.p.ws, 0, bytes));
    TPUCB_CUDA(cudaMemset(pl.p.ws_count, 0, cbytes));
    split_ws.push_back({pl.p.ws, bytes});
    split_ws.push_back({pl.p.ws_count, cbytes});
  }
  bool fuse_activations = true; // set before load_module
  bool fuse_residual_add = false; // set before load_module: eltwise adds run in the producing convolution's epilogue
  bool fp32_tensor_cores = true; // set before load_module: fp32 convolutions as three TF32 products
  void fuse_activation_chains(const std::map<std::string, int> &uses);
  void link_tf32_remainders();
  cudaGraphExec_t graph_exec = nullptr;
  std::map<std::string, HostWeight> weights;
  std::map<std::string, TensorPtr> tensors;
  std::vector<std::string> tensor_order;
  std::vector<std::unique_ptr<OpKernel>> kernels;
  std::vector<std::pair<std::string, size_t>> input_details, output_details;
  std::vector<void *> allocations;
  void *staging = nullptr;
  size_t staging_bytes = 0;
  // asynchronous uploads: host -> staging on the copy stream, staging -> tensor on the compute stream
  cudaStream_t copy_stream = nullptr;
  void *async_staging[2] = {nullptr, nullptr};
  size_t async_staging_bytes[2] = {0, 0};
  cudaEvent_t upload_done[2], staging_free[2];
  bool staging_used[2] = {false, false};
  int async_next = 0;
  void set_tensor_async(const std::string &name, const float *pinned, size_t numel);
  void set_tensor_async_i8(const std::string &name, const int8_t *pinned, size_t numel);
  void reenable_quant_of(const DevTensor *input);
};

// =========================================================================== op kernels

inline std::vector<int32_t> to_i32(const std::vector<float> &v, int pad_to, bool as_u32 = false) {
  std::vector<int32_t> o(std::max<size_t>(pad_to, v.size()), 0);
  for (size_t i = 0; i < v.size(); ++i)
    o[i] = as_u32 ? (int32_t)(uint32_t)v[i] : (int32_t)v[i];
  return o;
}

// The tensor-core epilogue forms 2 * multiplier in 32 unsigned bits: multipliers are the
// non-negative Q31 values the reference's quantizer emits (QuantizationArithmetic.cpp:207-247).
inline void check_q31_multipliers(const std::vector<float> &m, const std::string &op_name) {
  for (float v : m)
    TPUCB_CHECK(v >= 0.0f && v < 2147483648.0f, "%s: multiplier %g is outside [0, 2^31)", op_name.c_str(), (double)v);
}

// The multiply-high form of the tensor-core requantisation (requant_fast) needs |acc + bias| < 2^29 and
// rshift <= 29: true when every shift is that small and K * 127 * 128 + max |bias| stays below 2^29.
inline bool requant_fast_applies(const std::vector<float> &rshift, const std::vector<float> &bias, long long k_total) {
  double bmax = 0;
  for (float b : bias) bmax = std::max(bmax, std::fabs((double)b));
  for (float r : rshift)
    if (!(r >= 0.0f && r <= 29.0f)) return false;
  return (double)k_total * 127.0 * 128.0 + bmax < 536870912.0;
}
// ConvGemmParams::fastq: bit 0 the multiply-high form applies, bit 1 every rshift is >= 1
inline int requant_fast_flags(const std::vector<float> &rshift, const std::vector<float> &bias, long long k_total) {
  if (!requant_fast_applies(rshift, bias, k_total)) return 0;
  int f = 1 | 2;
  for (float r : rshift)
    if (r < 1.0f) f = 1;
  return f;
}

// ---------------------------------------------------------------------------- Input
// InputOpKernel (core/input.cpp:7-24): holds the tensor set_tensor writes; no device work.
class InputOp : public OpKernel {
public:
  void invoke(cudaStream_t) override {}
  int kernel_launches() const override { return 0; }
};

// ---------------------------------------------------------------------------- Quant
// QuantOpKernel (core/quant.cpp:113-166).
class QuantOp : public OpKernel {
public:
  QuantOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out, bool prev_is_input)
      : I_(I), in_(in), out_(out) {
    std::string from = op.gets("from", "NONE"), to = op.gets("to", "NONE");
    scale_ = (float)op.getf("scale", 1.0);
    TPUCB_CHECK(op.geti("zero_point", 0) == 0, "quant %s: zero_point != 0 is not supported",
                op.name.c_str());
    if (from == "NONE" && to == "INT8") kind_ = prev_is_input ? 0 : 1;
    else if ((from == "INT8" || from == "UINT8") && to == "NONE") kind_ = 2;
    else if ((from == "INT8" || from == "UINT8") && to == "BF16") kind_ = 3;
    else if (from == "BF16" && to == "INT8") kind_ = 4;
    else if (from == "NONE" && to == "BF16") kind_ = 5;
    else if (from == "BF16" && to == "NONE") kind_ = 6;
    else throw Error(strfmt("quant %s: %s -> %s is not supported", op.name.c_str(), from.c_str(), to.c_str()));
    alg_bytes = (double)in->numel() * in->elsize() + (double)out->numel() * out->elsize();
  }
  void invoke(cudaStream_t s) override {
    TPUCB_CHECK(!in_->padded_rows(), "quant %s: padded-row input is not supported", name.c_str());
    if (kind_ == 0 && in_->dtype == DT_F32 && in_->cp == 4 && (out_->cp == 4 || out_->cp == 8 || out_->cp == 16)) {
      size_t total = out_->pixels();
      launch_k(quant_input_pix_kernel, grid_for(total, 256, I_.sm_count), 256, 0, s, 
          (const float4 *)in_->dev, out_->dev, out_->n, out_->h, out_->w, out_->c, out_->cp, out_->wl,
          out_->wphys, scale_);
      return;
    }
    if (kind_ == 5 && in_->dtype == DT_F32 && in_->cp == 4 && out_->cp == 16 && !out_->padded_rows()) {
      launch_k(quant_f32c4_to_bf16c16_kernel, grid_for(out_->pixels(), 256, I_.sm_count), 256, 0, s, 
          (const float4 *)in_->dev, (uint4 *)out_->dev, out_->pixels(), out_->c);
      return;
    }
    const bool same_layout = in_->cp == out_->cp && !out_->padded_rows() && out_->cp % 16 == 0;
    if (same_layout && (kind_ == 3 || kind_ == 4)) {
      size_t nvec = out_->pixels() * out_->cp / 16;
      if (kind_ == 3)
        launch_k(quant_i8_to_bf16_vec_kernel, grid_for(nvec, 256, I_.sm_count), 256, 0, s, 
            (const uint4 *)in_->dev, (uint4 *)out_->dev, nvec, scale_);
      else
        launch_k(quant_bf16_to_i8_vec_kernel, grid_for(nvec, 256, I_.sm_count), 256, 0, s, 
            (const uint4 *)in_->dev, (uint4 *)out_->dev, nvec, scale_);
      return;
    }
    size_t total = out_->pixels() * out_->cp;
    launch_k(quant_kernel, grid_for(total, 256, I_.sm_count), 256, 0, s, 
        in_->dev, out_->dev, (size_t)out_->n * out_->h, out_->w, out_->wl, out_->wphys, out_->c, in_->cp,
        out_->cp, in_->dtype, out_->dtype, kind_ == 6 ? 5 : kind_, scale_);
  }

  int kind() const { return kind_; }
  float scale() const { return scale_; }
  const TensorPtr &in() const { return in_; }
  const TensorPtr &out() const { return out_; }

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  int kind_ = 0;
  float scale_ = 1;
};

// --------------------------------------------------------------------------- Conv2D
// Conv2DOpKernel (core/conv.cpp:11-104). INT8: dense -> tcgen05 implicit GEMM; depthwise ->
// the HBM-bound kernel. FP32: direct fp32 kernel (calibration forward).
class Conv2DOp : public OpKernel {
public:
  Conv2DOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out) : I_(I), in_(in), out_(out) {
    ConvGeom g;
    g.n = in->n; g.ic = in->c; g.ih = in->h; g.iw = in->w;
    g.oc = out->c; g.oh = out->h; g.ow = out->w;
    g.g = op.geti("g", 1);
    g.kh = op.geti("kh", 1); g.kw = op.geti("kw", 1);
    g.sh = op.geti("sh", 1); g.sw = op.geti("sw", 1);
    g.pt = op.geti("pt", 0); g.pb = op.geti("pb", 0); g.pl = op.geti("pl", 0); g.pr = op.geti("pr", 0);
    g.dh = op.geti("dh", 1); g.dw = op.geti("dw", 1);
    g.ins_h = op.geti("ins_h", 0); g.ins_w = op.geti("ins_w", 0);
    g_ = g;
    do_relu_ = op.geti("do_relu", 0);
    TPUCB_CHECK(op.in.size() >= 3, "conv %s: expects input, filter, bias[, scale, zeropoint, rshift, multiplier]",
                op.name.c_str());
    const HostWeight &filt = I.weight(op.in[1]);
    const int icg = g.ic / g.g, ocg = g.oc / g.g;
    TPUCB_CHECK((size_t)g.oc * icg * g.kh * g.kw == filt.data.size(), "conv %s: filter has %zu values, expected %zu",
                op.name.c_str(), filt.data.size(), (size_t)g.oc * icg * g.kh * g.kw);
    const bool with_bias = I.has_weight(op.in[2]);
    std::vector<float> bias(g.oc, 0.0f);
    if (with_bias) bias = I.weight(op.in[2]).data;
    alg_ops = 2.0 * g.n * g.oc * g.oh * g.ow * icg * g.kh * g.kw;
    if (out->dtype == DT_BF16) {
      // BF16 graphs (core/conv.cpp:90-98: fp32 convolution of BF16-valued operands, fp32 bias, ReLU, BF16 rounding):
      // the tensor-core pipeline with BF16 operands and fp32 accumulators; every K size and pitch is in bytes.
      TPUCB_CHECK(in->dtype == DT_BF16, "conv %s: a BF16 convolution needs a BF16 input", op.name.c_str());
      if ((g.g > 1 || g.ins_h || g.ins_w) && !in->padded_rows()) {
        // grouped / depthwise layers and deconvolutions (input insertion): the direct kernel
        // (conv_bf16_grouped_kernel); weights as fp32 [oc][kh][kw][ic / g]
        std::vector<float> wt((size_t)g.oc * g.kh * g.kw * icg);
        for (int o = 0; o < g.oc; ++o)
          for (int c = 0; c < icg; ++c)
            for (int t = 0; t < g.kh * g.kw; ++t)
              wt[((size_t)o * g.kh * g.kw + t) * icg + c] = filt.data[((size_t)o * icg + c) * g.kh * g.kw + t];
        bf16g_w_ = I.upload(wt);
        bf16g_b_ = I.upload(bias);
        bf16g_ = true;
        alg_bytes = 2.0 * ((double)in->numel() + out->numel()) + 4.0 * (filt.data.size() + g.oc);
        return;
      }
      TPUCB_CHECK(g.g == 1 && !g.ins_h && !g.ins_w && !in->padded_rows() && g.pl <= 127 && g.pt <= 127 &&
                      (g.kw - 1) * g.dw <= 255 && (g.kh - 1) * g.dh <= 255,
                  "conv %s: BF16 convolution supports dense, ungrouped layers", op.name.c_str());
      conv_kernel_setup_once();
      std::vector<int32_t> bias_bits(out->cp, 0);
      for (int o = 0; o < g.oc; ++o) bias_bits[o] = (int32_t)f32_bits(bias[o]);
      d_bias_ = I.upload(bias_bits);
      act_ = do_relu_ ? 1 : 0;
      ConvPlan pl;
      std::memset(&pl.p, 0, sizeof(pl.p));
      pl.bf16 = true;
      pl.in = (const int8_t *)in->dev;
      ConvGemmParams &p = pl.p;
      p.OH = g.oh; p.OW = g.ow; p.sh = g.sh; p.sw = g.sw; p.pt = g.pt; p.pl = g.pl; p.dh = g.dh; p.dw = g.dw;
      p.act = act_;
      p.bias = d_bias_; p.mult = d_bias_; p.rshift = d_bias_;
      p.out = (int8_t *)out->dev;
      p.ldc = out->cp * 2; // bytes
      p.c_off = 0;
      p.err = I.d_err;
      const int rows = g.n * g.oh * g.ow;
      const int k_bytes = in->cp * 2;
      const bool one_by_one_bf = g.kh == 1 && g.kw == 1 && g.sh == 1 && g.sw == 1 && g.pt == 0 && g.pl == 0 && g.pb == 0 && g.pr == 0;
      if (g.ic < 8 && !one_by_one_bf) {
        // few input channels (3-channel stems): expand the patches into a K-major matrix first
        pl.use_patch = true;
        pl.patch_elsize = 2;
        PatchArgs &a = pl.patch;
        a.n = g.n; a.c = g.ic; a.cp = in->cp; a.ih = g.ih; a.iw = g.iw; a.oh = g.oh; a.ow = g.ow;
        a.kh = g.kh; a.kw = g.kw; a.sh = g.sh; a.sw = g.sw; a.pt = g.pt; a.pl = g.pl; a.dh = g.dh; a.dw = g.dw;
        a.ins_h = 0; a.ins_w = 0; a.c_first = 0; a.c_count = g.ic; a.wl = in->wl; a.wphys = in->wphys;
        a.cv = g.ic <= 4 ? 4 : 0; // four channel slots per tap: one 8-byte copy per tap
        a.kp = a.cv ? round_up(g.kh * g.kw * 4, 8) : round_up(g.kh * g.kw * g.ic, 16);
        pl.patch_bytes = (size_t)rows * a.kp * 2;
        pl.patch_buf = (int8_t *)I.dalloc(pl.patch_bytes);
        const int8_t *d_wp = I.upload(pack_patch_weights(filt.data.data(), g.oc, g.ic, g.kh, g.kw, out->cp, a.kp, -1, a.cv));
        p.kh = p.kw = 1;
        p.a_mode = 0;
        finish_plan(pl, rows, 1, a.kp * 2, out->cp, I.sm_count);
        encode_matrix_map(&pl.tmA, pl.patch_buf, rows, a.kp * 2, a.kp * 2, p.BK, a_tile_rows(p));
        encode_weight_map(&pl.tmB, d_wp, out->cp, 1, a.kp * 2, p.BK, p.dual ? 192 : p.BN);
        p.idesc = make_idesc_bf16(128, p.BN);
        pl.ops = alg_ops;
        I.attach_split_ws(pl);
        plans_.push_back(pl);
        alg_bytes = 2.0 * ((double)in->numel() + out->numel() + filt.data.size()) + 4.0 * g.oc;
        return;
      }
      const int8_t *d_w = I.upload(pack_conv_weights_bf16(filt.data.data(), g.oc, g.ic, g.kh, g.kw, out->cp, in->cp));
      if (one_by_one_bf) {
        p.kh = p.kw = 1;
        p.a_mode = 0;
        finish_plan(pl, rows, 1, k_bytes, out->cp, I.sm_count);
        encode_matrix_map(&pl.tmA, (const int8_t *)in->dev, rows, k_bytes, k_bytes, p.BK, a_tile_rows(p));
        encode_weight_map(&pl.tmB, d_w, out->cp, 1, k_bytes, p.BK, p.dual ? 192 : p.BN);
      } else {
        p.kh = g.kh; p.kw = g.kw;
        p.a_mode = 1;
        finish_plan(pl, rows, g.kh * g.kw, k_bytes, out->cp, I.sm_count);
        encode_im2col_map(&pl.tmA, (const int8_t *)in->dev, g, k_bytes, p.BK, a_tile_rows(p));
        encode_weight_map(&pl.tmB, d_w, out->cp, g.kh * g.kw, k_bytes, p.BK, p.dual ? 192 : p.BN);
      }
      p.idesc = make_idesc_bf16(128, p.BN);
      pl.ops = alg_ops;
      I.attach_split_ws(pl);
      plans_.push_back(pl);
      alg_bytes = 2.0 * ((double)in->numel() + out->numel() + filt.data.size()) + 4.0 * g.oc;
      return;
    }
    if (out->dtype == DT_F32) {
      TPUCB_CHECK(in->dtype == DT_F32, "conv %s: an fp32 convolution needs an fp32 input", op.name.c_str());
      if (I.fp32_tensor_cores && g.g == 1 && !g.ins_h && !g.ins_w && g.ic <= 4 && in->cp == 4 && !(g.kh == 1 && g.kw == 1)) {
        // Image stem (at most 4 channels, NHWC4 input): the patches are expanded into a K-major matrix with four channel
        // slots per tap (one 16-byte copy per tap; the expansion also writes the remainder part), which is then the
        // activation operand of the TF32 x 3 product: 49 taps become 7 K blocks per term.
        conv_kernel_setup_once();
        std::vector<int32_t> bias_bits(out->cp, 0);
        for (int o = 0; o < g.oc; ++o) bias_bits[o] = (int32_t)f32_bits(bias[o]);
        d_bias_ = I.upload(bias_bits);
        act_ = do_relu_ ? 1 : 0;
        ConvPlan pl;
        std::memset(&pl.p, 0, sizeof(pl.p));
        pl.tf32 = true;
        pl.use_patch = true;
        pl.patch_elsize = 4;
        pl.in = (const int8_t *)in->dev;
        const int rows = g.n * g.oh * g.ow;
        PatchArgs &a = pl.patch;
        a.n = g.n; a.c = g.ic; a.cp = in->cp; a.ih = g.ih; a.iw = g.iw; a.oh = g.oh; a.ow = g.ow;
        a.kh = g.kh; a.kw = g.kw; a.sh = g.sh; a.sw = g.sw; a.pt = g.pt; a.pl = g.pl; a.dh = g.dh; a.dw = g.dw;
        a.ins_h = 0; a.ins_w = 0; a.c_first = 0; a.c_count = g.ic; a.wl = in->wl; a.wphys = in->wphys;
        a.cv = 4;
        a.kp = g.kh * g.kw * 4;
        pl.patch_bytes = (size_t)rows * a.kp * 4;
        pl.patch_buf = (int8_t *)I.dalloc(pl.patch_bytes);
        pl.split_src = nullptr; // the expansion writes the remainder itself
        pl.split_hi = nullptr;
        pl.split_lo = (float *)I.dalloc(pl.patch_bytes);
        ConvGemmParams &p = pl.p;
        p.OH = g.oh; p.OW = g.ow; p.sh = p.sw = p.dh = p.dw = 1;
        p.act = act_;
        p.bias = d_bias_; p.mult = d_bias_; p.rshift = d_bias_;
        p.out = (int8_t *)out->dev;
        p.ldc = out->cp * 4;
        p.c_off = 0;
        p.err = I.d_err;
        p.kh = p.kw = 1;
        p.a_mode = 0;
        const int kb = a.kp * 4;
        const int8_t *d_ph = I.upload(pack_patch_weights(filt.data.data(), g.oc, g.ic, g.kh, g.kw, out->cp, a.kp, 0, 4));
        const int8_t *d_pl = I.upload(pack_patch_weights(filt.data.data(), g.oc, g.ic, g.kh, g.kw, out->cp, a.kp, 1, 4));
        finish_plan(pl, rows, 1, kb, out->cp, I.sm_count);
        encode_matrix_map(&pl.tmA, pl.patch_buf, rows, kb, kb, p.BK, a_tile_rows(p));
        encode_matrix_map(&pl.tmA2, (const int8_t *)pl.split_lo, rows, kb, kb, p.BK, a_tile_rows(p));
        encode_weight_map(&pl.tmB, d_ph, out->cp, 1, kb, p.BK, p.BN);
        encode_weight_map(&pl.tmB2, d_pl, out->cp, 1, kb, p.BK, p.BN);
        p.idesc = make_idesc_tf32(128, p.BN);
        pl.ops = alg_ops;
        I.attach_split_ws(pl);
        plans_.push_back(pl);
        alg_bytes = 4.0 * ((double)in->numel() + out->numel() + filt.data.size() + g.oc);
        return;
      }
      if (I.fp32_tensor_cores && g.g == 1 && !g.ins_h && !g.ins_w && !in->padded_rows() && in->cp % 8 == 0 &&
          g.pl <= 127 && g.pt <= 127 && (g.kw - 1) * g.dw <= 255 && (g.kh - 1) * g.dh <= 255) {
        // fp32 convolution on the tensor cores as three TF32 products with fp32 accumulation (x w = xh wh + xl wh +
        // xh wl, 2^-22 relative: inside the 1e-4 of the fp32 path, where a single TF32 product would not be). The
        // activations are split into their two parts by a vector kernel right before the launch; the weights once, here.
        conv_kernel_setup_once();
        std::vector<int32_t> bias_bits(out->cp, 0);
        for (int o = 0; o < g.oc; ++o) bias_bits[o] = (int32_t)f32_bits(bias[o]);
        d_bias_ = I.upload(bias_bits);
        act_ = do_relu_ ? 1 : 0;
        ConvPlan pl;
        std::memset(&pl.p, 0, sizeof(pl.p));
        pl.tf32 = true;
        pl.in = (const int8_t *)in->dev;
        pl.split_src = (const float *)in->dev;
        // The tensor core ignores the low 13 mantissa bits of an fp32 operand (measured: results are bit-identical with
        // the upper part materialised or not), so the tensor itself serves as xh and only xl is written.
        pl.split_hi = nullptr;
        if (!in->lo_dev) in->lo_dev = I.dalloc(in->bytes()); // shared by every convolution that reads this tensor
        pl.split_lo = (float *)in->lo_dev;
        pl.split_nvec = in->bytes() / 16;
        ConvGemmParams &p = pl.p;
        p.OH = g.oh; p.OW = g.ow; p.sh = g.sh; p.sw = g.sw; p.pt = g.pt; p.pl = g.pl; p.dh = g.dh; p.dw = g.dw;
        p.act = act_;
        p.bias = d_bias_; p.mult = d_bias_; p.rshift = d_bias_;
        p.out = (int8_t *)out->dev;
        p.ldc = out->cp * 4; // bytes
        p.c_off = 0;
        p.err = I.d_err;
        const int rows = g.n * g.oh * g.ow;
        const int k_bytes = in->cp * 4;
        const bool one = g.kh == 1 && g.kw == 1 && g.sh == 1 && g.sw == 1 && g.pt == 0 && g.pl == 0 && g.pb == 0 && g.pr == 0;
        const int8_t *d_wh = I.upload(pack_conv_weights_tf32(filt.data.data(), g.oc, g.ic, g.kh, g.kw, out->cp, in->cp, 0));
        const int8_t *d_wl = I.upload(pack_conv_weights_tf32(filt.data.data(), g.oc, g.ic, g.kh, g.kw, out->cp, in->cp, 1));
        const int taps = one ? 1 : g.kh * g.kw;
        p.kh = one ? 1 : g.kh; p.kw = one ? 1 : g.kw;
        p.a_mode = one ? 0 : 1;
        finish_plan(pl, rows, taps, k_bytes, out->cp, I.sm_count);
        if (one) {
          encode_matrix_map(&pl.tmA, pl.split_hi ? (const int8_t *)pl.split_hi : (const int8_t *)in->dev, rows, k_bytes, k_bytes, p.BK, a_tile_rows(p));
          encode_matrix_map(&pl.tmA2, (const int8_t *)pl.split_lo, rows, k_bytes, k_bytes, p.BK, a_tile_rows(p));
        } else {
          encode_im2col_map(&pl.tmA, pl.split_hi ? (const int8_t *)pl.split_hi : (const int8_t *)in->dev, g, k_bytes, p.BK, a_tile_rows(p));
          encode_im2col_map(&pl.tmA2, (const int8_t *)pl.split_lo, g, k_bytes, p.BK, a_tile_rows(p));
        }
        encode_weight_map(&pl.tmB, d_wh, out->cp, taps, k_bytes, p.BK, p.BN);
        encode_weight_map(&pl.tmB2, d_wl, out->cp, taps, k_bytes, p.BK, p.BN);
        p.idesc = make_idesc_tf32(128, p.BN);
        pl.ops = alg_ops;
        I.attach_split_ws(pl);
        plans_.push_back(pl);
        alg_bytes = 4.0 * ((double)in->numel() + out->numel() + filt.data.size() + g.oc);
        return;
      }
      f32_ = true;
      f32_w_ = I.upload(pack_conv_weights_f32(filt.data.data(), g.oc, icg, g.kh, g.kw, g.g));
      f32_b_ = I.upload(bias);
      alg_bytes = 4.0 * ((double)in->numel() + out->numel() + filt.data.size() + g.oc);
      return;
    }
    TPUCB_CHECK(in->dtype == DT_I8, "conv %s: INT8 convolution needs an INT8 input", op.name.c_str());
    TPUCB_CHECK(op.in.size() >= 7 && I.has_weight(op.in[5]) && I.has_weight(op.in[6]),
                "conv %s: INT8 convolution needs rshift and multiplier operands (RSHIFT_AND_M_I32)", op.name.c_str());
    const int oc_pad = out->cp;
    check_q31_multipliers(I.weight(op.in[6]).data, op.name);
    d_bias_ = I.upload(to_i32(bias, oc_pad));
    d_mult_ = I.upload(to_i32(I.weight(op.in[6]).data, oc_pad, true));
    d_rsh_ = I.upload(to_i32(I.weight(op.in[5]).data, oc_pad, true));
    alg_bytes = (double)in->numel() + out->numel() + filt.data.size() + 12.0 * g.oc;
    act_ = do_relu_ ? 1 : 0;
    const int fastq = requant_fast_flags(I.weight(op.in[5]).data, bias, (long long)(g.ic / g.g) * g.kh * g.kw);

    if (g.g == g.ic && g.g == g.oc && g.g > 1 && g.ins_h == 0 && g.ins_w == 0) {
      // depthwise
      dw_ = true;
      std::vector<int8_t> w((size_t)g.kh * g.kw * in->cp, 0);
      for (int c = 0; c < g.ic; ++c)
        for (int t = 0; t < g.kh * g.kw; ++t) w[(size_t)t * in->cp + c] = (int8_t)(int)filt.data[(size_t)c * g.kh * g.kw + t];
      DwArgs a;
      a.n = g.n; a.c = g.ic; a.cp = in->cp; a.ih = g.ih; a.iw = g.iw; a.oh = g.oh; a.ow = g.ow;
      a.kh = g.kh; a.kw = g.kw; a.sh = g.sh; a.sw = g.sw; a.pt = g.pt; a.pl = g.pl; a.dh = g.dh; a.dw = g.dw;
      a.do_relu = do_relu_;
      a.wgt = I.upload(w);
      a.bias = d_bias_; a.mult = d_mult_; a.rshift = d_rsh_;
      dwargs_ = a;
      if (g.kh == 3 && g.kw == 3 && g.dh == 1 && g.dw == 1 && g.sh == g.sw && (g.sh == 1 || g.sh == 2) && (fastq & 1)) {
        // the dot-product kernel: weights as one word per (channel word, filter row, channel): w0 | w1 << 8 | w2 << 16
        const int cw = in->cp / 4;
        std::vector<uint32_t> wt((size_t)cw * 12, 0u);
        for (int c = 0; c < g.ic; ++c)
          for (int r = 0; r < 3; ++r) {
            uint32_t word = 0;
            for (int ss = 0; ss < 3; ++ss)
              word |= (uint32_t)(uint8_t)(int8_t)(int)filt.data[(size_t)c * 9 + r * 3 + ss] << (8 * ss);
            wt[((size_t)(c / 4) * 3 + r) * 4 + (c % 4)] = word;
          }
        dw_wt_ = I.upload(wt);
      }
      return;
    }

    if (in->cp == 4 && !in->padded_rows() && stem4_applies(g)) {
      stem_kernel_setup_once();
      StemPlan sp;
      std::memset(&sp.p, 0, sizeof(sp.p));
      ConvStemParams &p = sp.p;
      p.OH = g.oh; p.OW = g.ow; p.H = g.ih; p.W = g.iw;
      p.sh = g.sh; p.sw = g.sw; p.pt = g.pt; p.pl = g.pl; p.dh = g.dh; p.kw = g.kw;
      p.act = act_;
      p.fastq = fastq;
      p.in = (const uint32_t *)in->dev;
      p.bias = d_bias_; p.mult = d_mult_; p.rshift = d_rsh_;
      p.out = (int8_t *)out->dev;
      p.ldc = out->cp;
      p.c_off = 0;
      p.err = I.d_err;
      const int8_t *d_w = I.upload(pack_stem_weights(filt.data.data(), g.oc, g.ic, g.kh, g.kw, oc_pad));
      finish_stem_plan(sp, d_w, g.n * g.oh * g.ow, g.kh, oc_pad, I.sm_count);
      stem_plans_.push_back(sp);
      return;
    }

    conv_kernel_setup_once();
    const bool one_by_one = g.kh == 1 && g.kw == 1 && g.sh == 1 && g.sw == 1 && g.pt == 0 && g.pl == 0 &&
                            g.oh == g.ih && g.ow == g.iw;
    const bool small_c = g.ic < 16;
    StemLayout stem;
    bool stem_ok = in->padded_rows() && stem_layout_for(g, &stem) && stem.cp == in->cp &&
                   stem.wl == in->wl && stem.wphys == in->wphys;
    if (stem_ok) {
      // The window tensor map has overlapping strides; if the driver refuses to encode it, the
      // patch-expansion path (which understands padded rows) takes over.
      try {
        CUtensorMap probe;
        encode_window_map(&probe, (const int8_t *)in->dev, g, in->cp, in->wphys, stem.bk, stem.g);
      } catch (const Error &) {
        stem_ok = false;
      }
    }
    const bool need_patch = !stem_ok && (g.g > 1 || g.ins_h || g.ins_w || (small_c && !one_by_one) || in->padded_rows() || in->cp % 16 != 0 ||
                            g.pl > 127 || g.pt > 127 || (g.kw - 1) * g.dw > 255 || (g.kh - 1) * g.dh > 255);
    const int groups = g.g;
    for (int grp = 0; grp < groups; ++grp) {
      ConvPlan pl;
      std::memset(&pl.p, 0, sizeof(pl.p));
      pl.in = (const int8_t *)in->dev;
      ConvGemmParams &p = pl.p;
      p.OH = g.oh; p.OW = g.ow; p.sh = g.sh; p.sw = g.sw; p.pt = g.pt; p.pl = g.pl; p.dh = g.dh; p.dw = g.dw;
      p.act = act_;
      p.fastq = fastq;
      p.bias = d_bias_ + grp * ocg; p.mult = d_mult_ + grp * ocg; p.rshift = d_rsh_ + grp * ocg;
      p.out = (int8_t *)out->dev;
      p.ldc = out->cp;
      p.c_off = grp * ocg;
      p.err = I.d_err;
      const int rows = g.n * g.oh * g.ow;
      const float *wsrc = filt.data.data() + (size_t)grp * ocg * icg * g.kh * g.kw;
      int ocg_pad = groups == 1 ? oc_pad : ocg;
      TPUCB_CHECK(groups == 1 || ocg % 16 == 0, "conv %s: grouped convolution needs oc/g to be a multiple of 16",
                  op.name.c_str());
      if (stem_ok) {
        // Row-window path: one K step per filter row; the window of (left slack + kw) pixels x
        // cp channels is contiguous in the zero-padded NHWC rows.
        const int BKs = stem.bk;
        std::vector<int8_t> w((size_t)ocg_pad * g.kh * BKs, 0);
        for (int o = 0; o < ocg; ++o)
          for (int c = 0; c < icg; ++c)
            for (int r = 0; r < g.kh; ++r)
              for (int ss = 0; ss < g.kw; ++ss)
                w[((size_t)o * g.kh + r) * BKs + (size_t)(ss + stem.wl - g.pl) * in->cp + c] =
                    (int8_t)(int)wsrc[(((size_t)o * icg + c) * g.kh + r) * g.kw + ss];
        const int8_t *d_w = I.upload(w);
        p.kh = g.kh;
        p.kw = 1;
        p.a_mode = 2;
        p.win_g = stem.g;
        finish_plan(pl, rows, g.kh, BKs, ocg_pad, I.sm_count);
        TPUCB_CHECK(p.BK == BKs && p.c_chunks == 1, "conv %s: stem tile shape mismatch", op.name.c_str());
        encode_window_map(&pl.tmA, (const int8_t *)in->dev, g, in->cp, in->wphys, BKs, stem.g);
        encode_weight_map(&pl.tmB, d_w, ocg_pad, g.kh, BKs, p.BK, p.dual ? 192 : p.BN);
      } else if (need_patch) {
        pl.use_patch = true;
        PatchArgs &a = pl.patch;
        a.n = g.n; a.c = g.ic; a.cp = in->cp; a.ih = g.ih; a.iw = g.iw; a.oh = g.oh; a.ow = g.ow;
        a.kh = g.kh; a.kw = g.kw; a.sh = g.sh; a.sw = g.sw; a.pt = g.pt; a.pl = g.pl; a.dh = g.dh; a.dw = g.dw;
        a.ins_h = g.ins_h; a.ins_w = g.ins_w;
        a.c_first = grp * icg; a.c_count = icg;
        a.wl = in->wl; a.wphys = in->wphys;
        a.kp = round_up(g.kh * g.kw * icg, 16);
        pl.patch_bytes = (size_t)rows * a.kp;
        pl.patch_buf = (int8_t *)I.dalloc(pl.patch_bytes);
        auto w = pack_conv_weights(wsrc, ocg, icg, g.kh, g.kw, ocg_pad, 0, true, a.kp);
        const int8_t *d_w = I.upload(w);
        p.kh = p.kw = 1;
        p.a_mode = 0;
        finish_plan(pl, rows, 1, a.kp, ocg_pad, I.sm_count);
        encode_matrix_map(&pl.tmA, pl.patch_buf, rows, a.kp, a.kp, p.BK, a_tile_rows(p));
        encode_weight_map(&pl.tmB, d_w, ocg_pad, 1, a.kp, p.BK, p.dual ? 192 : p.BN);
      } else if (one_by_one) {
        auto w = pack_conv_weights(wsrc, ocg, icg, 1, 1, ocg_pad, in->cp, false, 0);
        const int8_t *d_w = I.upload(w);
        p.kh = p.kw = 1;
        p.a_mode = 0;
        finish_plan(pl, rows, 1, in->cp, ocg_pad, I.sm_count);
        encode_matrix_map(&pl.tmA, (const int8_t *)in->dev, rows, in->cp, in->cp, p.BK, a_tile_rows(p));
        encode_weight_map(&pl.tmB, d_w, ocg_pad, 1, in->cp, p.BK, p.dual ? 192 : p.BN);
      } else {
        auto w = pack_conv_weights(wsrc, ocg, icg, g.kh, g.kw, ocg_pad, in->cp, false, 0);
        const int8_t *d_w = I.upload(w);
        p.kh = g.kh; p.kw = g.kw;
        p.a_mode = 1;
        finish_plan(pl, rows, g.kh * g.kw, in->cp, ocg_pad, I.sm_count);
        encode_im2col_map(&pl.tmA, (const int8_t *)in->dev, g, in->cp, p.BK, a_tile_rows(p));
        encode_weight_map(&pl.tmB, d_w, ocg_pad, g.kh * g.kw, in->cp, p.BK, p.dual ? 192 : p.BN);
      }
      if (I.selftest_lost_arrival > 0) {
        pl.p.wait_rounds = I.selftest_lost_arrival;
        pl.p.lose_arrival = 1;
      }
      I.attach_split_ws(pl);
      plans_.push_back(pl);
    }
  }
  // Fused leaky ReLU (tensor-core plans only): the epilogue writes the plain result to this op's tensor
  // and the activation result to `act_out`.
  bool can_fuse_leaky() const {
    return !(f32_ || dw_ || bf16g_ || !stem_plans_.empty() || act_ != 0 || plans_.empty()) && in_->dtype == DT_I8;
  }
  void set_leaky(int mp, int rp, int mn, int rn, int8_t *act_out) {
    for (auto &pl : plans_) {
      pl.p.act = 2;
      pl.p.leaky_mp = mp; pl.p.leaky_rp = rp; pl.p.leaky_mn = mn; pl.p.leaky_rn = rn;
      pl.p.out2 = act_out;
    }
    act_ = 2;
  }
  // Fused eltwise add (tensor-core INT8 plans without an activation of their own): the epilogue also forms
  // sat8(relu?((conv * ms + residual * mr + 2^(r-1)) >> r)) into `sum_out`; this op's own tensor is still written.
  bool can_fuse_add() const {
    return can_fuse_leaky() && plans_.size() == 1 && in_->dtype == DT_I8 && plans_[0].p.split_k <= 1;
  }
  void set_residual_add(const int8_t *residual, int8_t *sum_out, int ms, int mr, int rshift, int relu) {
    for (auto &pl : plans_) {
      pl.p.act = 3;
      pl.p.res = residual;
      pl.p.out2 = sum_out;
      pl.p.add_ms = ms; pl.p.add_mr = mr; pl.p.add_r = rshift; pl.p.add_relu = relu;
    }
    act_ = 3;
    alg_bytes += 2.0 * out_->numel(); // the residual read and the sum written
  }
  const TensorPtr &out() const { return out_; }
  const TensorPtr &in() const { return in_; }
  // TF32 x 3 plans (not the patch-matrix stem, whose remainder belongs to the patch matrix)
  bool is_tf32() const { return !plans_.empty() && plans_[0].tf32 && !plans_[0].use_patch; }
  bool can_write_remainder() const { return !plans_.empty() && plans_[0].tf32; }
  void set_remainder_out(void *lo) {
    for (auto &pl : plans_) pl.p.out2 = (int8_t *)lo;
  }
  void skip_split() {
    for (auto &pl : plans_) pl.split_src = nullptr;
  }
  void invoke(cudaStream_t s) override {
    if (bf16g_) {
      ConvBf16GroupArgs a{g_.n, g_.ic, in_->cp, g_.ih, g_.iw, g_.oc, out_->cp, g_.oh, g_.ow, g_.kh, g_.kw, g_.sh, g_.sw,
                          g_.pt, g_.pl, g_.dh, g_.dw, g_.g, do_relu_, g_.ins_h, g_.ins_w};
      const size_t total = (size_t)g_.n * g_.oh * g_.ow * out_->cp;
      launch_k(conv_bf16_grouped_kernel, grid_for(total, 256, I_.sm_count), 256, 0, s, (const uint16_t *)in_->dev, bf16g_w_,
               bf16g_b_, (uint16_t *)out_->dev, a);
    } else if (f32_) {
      launch_conv2d_f32((const float *)in_->dev, f32_w_, f32_b_, (float *)out_->dev, g_, in_->cp, out_->cp, do_relu_,
                        s, I_.sm_count);
    } else if (dw_) {
      const DwArgs &d = dwargs_;
      if (d.kh == 3 && d.kw == 3 && d.dh == 1 && d.dw == 1 && d.sh == d.sw && (d.sh == 1 || d.sh == 2) &&
          in_->cp == out_->cp && !in_->padded_rows() && !out_->padded_rows()) {
        const int tw = d.sh == 1 ? 8 : 4;
        size_t items = (size_t)d.n * d.oh * ((d.ow + tw - 1) / tw) * (d.cp / 4);
        int grid = grid_for(items, 128, I_.sm_count);
        const uint32_t *src = (const uint32_t *)in_->dev;
        uint32_t *dst = (uint32_t *)out_->dev;
        if (dw_wt_) {
          if (d.sh == 1 && d.do_relu) launch_k(dwconv3x3_dp4a_kernel<1, true>, grid, 128, 0, s, src, dst, dw_wt_, d);
          else if (d.sh == 1) launch_k(dwconv3x3_dp4a_kernel<1, false>, grid, 128, 0, s, src, dst, dw_wt_, d);
          else if (d.do_relu) launch_k(dwconv3x3_dp4a_kernel<2, true>, grid, 128, 0, s, src, dst, dw_wt_, d);
          else launch_k(dwconv3x3_dp4a_kernel<2, false>, grid, 128, 0, s, src, dst, dw_wt_, d);
          return;
        }
        if (d.sh == 1 && d.do_relu) launch_k(dwconv3x3_i8_kernel<1, 8, true>, grid, 128, 0, s, src, dst, d);
        else if (d.sh == 1) launch_k(dwconv3x3_i8_kernel<1, 8, false>, grid, 128, 0, s, src, dst, d);
        else if (d.do_relu) launch_k(dwconv3x3_i8_kernel<2, 4, true>, grid, 128, 0, s, src, dst, d);
        else launch_k(dwconv3x3_i8_kernel<2, 4, false>, grid, 128, 0, s, src, dst, d);
        return;
      }
      size_t total = out_->pixels() * (out_->cp / 16);
      launch_k(dwconv_i8_kernel, grid_for(total, 128, I_.sm_count), 128, 0, s, (const int8_t *)in_->dev,
                                                                          (int8_t *)out_->dev, dwargs_);
    } else {
      for (auto &sp : stem_plans_) {
        PdlConvScope conv_class;
        if ((sp.p.fastq & 1) && sp.p.act == 1) // the ReLU epilogue alone: most stems
          launch_k(conv_stem_i8_kernel<true, true>, sp.grid, kStemThreads, sp.smem, s, sp.tmB, sp.p);
        else if (sp.p.fastq & 1) launch_k(conv_stem_i8_kernel<true>, sp.grid, kStemThreads, sp.smem, s, sp.tmB, sp.p);
        else launch_k(conv_stem_i8_kernel<false>, sp.grid, kStemThreads, sp.smem, s, sp.tmB, sp.p);
      }
      for (auto &pl : plans_) launch_conv_plan(pl, s, I_.sm_count);
    }
  }
  int kernel_launches() const override {
    if (f32_ || dw_ || bf16g_) return 1;
    int k = (int)stem_plans_.size();
    for (auto &pl : plans_) k += 1 + (pl.use_patch ? 1 : 0) + ((pl.tf32 && pl.split_src) ? 1 : 0);
    return k;
  }
  bool is_tensor_core() const { return !f32_ && !dw_ && !bf16g_; }
  std::vector<ConvPlan> plans_;
  std::vector<StemPlan> stem_plans_;

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  ConvGeom g_;
  int do_relu_ = 0, act_ = 0;
  bool dw_ = false, f32_ = false;
  DwArgs dwargs_;
  const int32_t *d_bias_ = nullptr, *d_mult_ = nullptr, *d_rsh_ = nullptr;
  const float *f32_w_ = nullptr, *f32_b_ = nullptr;
  bool bf16g_ = false; // grouped / depthwise BF16 convolution on conv_bf16_grouped_kernel
  const float *bf16g_w_ = nullptr, *bf16g_b_ = nullptr;
  const uint32_t *dw_wt_ = nullptr; // depthwise 3x3: weights packed for dwconv3x3_dp4a_kernel (null: the multiply-add kernel)
};

// ------------------------------------------------------------------- FullyConnected
// FullyConnectedOpKernel (core/fullyconnected.cpp:7-91), batch == 1, no transposes.
class FullyConnectedOp : public OpKernel {
public:
  FullyConnectedOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out) : I_(I), in_(in), out_(out) {
    do_relu_ = op.geti("do_relu", 0);
    if (I.weight(op.in.at(1)).shape.size() >= 3) {
      setup_batched(I, op);
      return;
    }
    m_ = in->n;
    const int hw = in->h * in->w;
    k_ = in->c * hw;
    n_ = out->c;
    TPUCB_CHECK(out->n == m_ && out->h * out->w == 1, "fc %s: output must be [m, n]", op.name.c_str());
    const HostWeight &filt = I.weight(op.in[1]);
    TPUCB_CHECK(filt.data.size() == (size_t)n_ * k_, "fc %s: filter has %zu values, expected n*k = %zu",
                op.name.c_str(), filt.data.size(), (size_t)n_ * k_);
    std::vector<float> bias(n_, 0.0f);
    if (op.in.size() > 2 && I.has_weight(op.in[2])) bias = I.weight(op.in[2]).data;
    alg_ops = 2.0 * m_ * k_ * n_;
    if (out->dtype == DT_BF16) {
      // BF16 inner product (core/fullyconnected.cpp:44-91 with the BF16 rounding of the result): the tensor-core
      // pipeline with BF16 operands, fp32 accumulators and fp32 bias; K sizes and pitches in bytes.
      TPUCB_CHECK(in->dtype == DT_BF16, "fc %s: a BF16 inner product needs a BF16 input", op.name.c_str());
      conv_kernel_setup_once();
      const int n_pad = out->cp;
      kdev_ = hw * in->cp;
      std::vector<uint16_t> w((size_t)n_pad * kdev_, 0);
      for (int j = 0; j < n_; ++j)
        for (int c = 0; c < in->c; ++c)
          for (int p = 0; p < hw; ++p)
            w[(size_t)j * kdev_ + (size_t)p * in->cp + c] = (uint16_t)(f32_bits(filt.data[(size_t)j * k_ + (size_t)c * hw + p]) >> 16);
      std::vector<int8_t> wb(w.size() * 2);
      std::memcpy(wb.data(), w.data(), wb.size());
      const int8_t *d_w = I.upload(wb);
      std::vector<int32_t> bias_bits(n_pad, 0);
      for (int j = 0; j < n_; ++j) bias_bits[j] = (int32_t)f32_bits(bias[j]);
      ConvPlan pl;
      std::memset(&pl.p, 0, sizeof(pl.p));
      pl.bf16 = true;
      ConvGemmParams &p = pl.p;
      p.bias = I.upload(bias_bits);
      p.mult = p.bias; p.rshift = p.bias;
      p.out = (int8_t *)out->dev;
      p.ldc = out->cp * 2;
      p.c_off = 0;
      p.err = I.d_err;
      p.OH = p.OW = 1; p.sh = p.sw = p.dh = p.dw = 1; p.kh = p.kw = 1;
      p.act = do_relu_ ? 1 : 0;
      p.a_mode = 0;
      finish_plan(pl, m_, 1, kdev_ * 2, n_pad, I.sm_count);
      encode_matrix_map(&pl.tmA, (const int8_t *)in->dev, m_, kdev_ * 2, kdev_ * 2, p.BK, a_tile_rows(p));
      encode_weight_map(&pl.tmB, d_w, n_pad, 1, kdev_ * 2, p.BK, p.dual ? 192 : p.BN);
      p.idesc = make_idesc_bf16(128, p.BN);
      I.attach_split_ws(pl);
      plan_ = pl;
      alg_bytes = 2.0 * ((double)m_ * k_ + (double)n_ * k_ + (double)m_ * n_) + 4.0 * n_;
      return;
    }
    if (out->dtype != DT_I8) {
      TPUCB_CHECK(in->dtype == DT_F32 && out->dtype == DT_F32, "fc %s: an fp32 inner product needs an fp32 input", op.name.c_str());
      f32_ = true;
      // weights in device K order: (y, x, c) with pitch in->cp
      kdev_ = hw * in->cp;
      std::vector<float> w((size_t)n_ * kdev_, 0.0f);
      for (int j = 0; j < n_; ++j)
        for (int c = 0; c < in->c; ++c)
          for (int p = 0; p < hw; ++p) w[(size_t)j * kdev_ + (size_t)p * in->cp + c] = filt.data[(size_t)j * k_ + (size_t)c * hw + p];
      f32_w_ = I.upload(w);
      f32_b_ = I.upload(bias);
      alg_bytes = 4.0 * ((double)m_ * k_ + (double)n_ * k_ + (double)m_ * n_ + n_);
      return;
    }
    TPUCB_CHECK(in->dtype == DT_I8, "fc %s: INT8 needs an INT8 input", op.name.c_str());
    TPUCB_CHECK(op.in.size() >= 7 && I.has_weight(op.in[5]) && I.has_weight(op.in[6]),
                "fc %s: INT8 needs rshift and multiplier operands", op.name.c_str());
    conv_kernel_setup_once();
    const int n_pad = out->cp;
    kdev_ = hw * in->cp;
    std::vector<int8_t> w((size_t)n_pad * kdev_, 0);
    for (int j = 0; j < n_; ++j)
      for (int c = 0; c < in->c; ++c)
        for (int p = 0; p < hw; ++p)
          w[(size_t)j * kdev_ + (size_t)p * in->cp + c] = (int8_t)(int)filt.data[(size_t)j * k_ + (size_t)c * hw + p];
    const int8_t *d_w = I.upload(w);
    // one (rshift, multiplier) pair per batch slice (fullyconnected.cpp:78-88) -> broadcast per column
    std::vector<float> rs(n_, I.weight(op.in[5]).data.at(0)), mu(n_, I.weight(op.in[6]).data.at(0));
    check_q31_multipliers(mu, op.name);
    ConvPlan pl;
    std::memset(&pl.p, 0, sizeof(pl.p));
    ConvGemmParams &p = pl.p;
    p.bias = I.upload(to_i32(bias, n_pad));
    p.mult = I.upload(to_i32(mu, n_pad, true));
    p.rshift = I.upload(to_i32(rs, n_pad, true));
    p.out = (int8_t *)out->dev;
    p.ldc = out->cp;
    p.c_off = 0;
    p.err = I.d_err;
    p.OH = p.OW = 1; p.sh = p.sw = p.dh = p.dw = 1; p.kh = p.kw = 1;
    // The reference applies ReLU to the float before the QDM requant; with a positive
    // multiplier the two orders give the same int8 result.
    p.act = do_relu_ ? 1 : 0;
    p.fastq = requant_fast_flags(rs, bias, k_);
    p.a_mode = 0;
    finish_plan(pl, m_, 1, kdev_, n_pad, I.sm_count);
    encode_matrix_map(&pl.tmA, (const int8_t *)in->dev, m_, kdev_, kdev_, p.BK, a_tile_rows(p));
    encode_weight_map(&pl.tmB, d_w, n_pad, 1, kdev_, p.BK, p.dual ? 192 : p.BN);
    I.attach_split_ws(pl);
    plan_ = pl;
    alg_bytes = (double)m_ * k_ + (double)n_ * k_ + (double)m_ * n_ + 4.0 * n_ + 8;
  }
  // A filter of rank 3, [batch, n, k]: one product per batch index with its own bias row and its own (multiplier,
  // rshift) pair (core/fullyconnected.cpp:59-88). INT8, rank-3 activations [batch, m, k] -> [batch, m, n], no
  // input / output transposes.
  void setup_batched(Interpreter &I, const ParsedOp &op) {
    const HostWeight &filt = I.weight(op.in[1]);
    TPUCB_CHECK(filt.shape.size() == 3 && in_->shape.size() == 3 && out_->shape.size() == 3,
                "fc %s: a batched inner product needs rank-3 input, filter and result", op.name.c_str());
    TPUCB_CHECK(!op.geti("input_transpose", 0) && !op.geti("output_transpose", 0),
                "fc %s: batched inner products with transposes are not implemented", op.name.c_str());
    TPUCB_CHECK(in_->dtype == DT_I8 && out_->dtype == DT_I8, "fc %s: batched inner products are implemented for INT8 only",
                op.name.c_str());
    batch_ = (int)filt.shape[0];
    n_ = (int)filt.shape[1];
    k_ = (int)filt.shape[2];
    m_ = (int)in_->shape[1];
    TPUCB_CHECK(in_->shape[0] == batch_ && in_->shape[2] == k_ && out_->shape[0] == batch_ && out_->shape[1] == m_ &&
                    out_->shape[2] == n_,
                "fc %s: shapes do not agree with filter [%d, %d, %d]", op.name.c_str(), batch_, n_, k_);
    TPUCB_CHECK(op.in.size() >= 7 && I.has_weight(op.in[5]) && I.has_weight(op.in[6]),
                "fc %s: INT8 needs rshift and multiplier operands", op.name.c_str());
    const auto &rs = I.weight(op.in[5]).data, &mu = I.weight(op.in[6]).data;
    TPUCB_CHECK((int)rs.size() >= batch_ && (int)mu.size() >= batch_, "fc %s: one (rshift, multiplier) pair per batch index is needed",
                op.name.c_str());
    check_q31_multipliers(mu, op.name);
    TPUCB_CHECK((double)k_ * 127.0 * 128.0 < 2147483648.0, "fc %s: K = %d overflows the int32 sum", op.name.c_str(), k_);
    std::vector<int8_t> w(filt.data.size());
    for (size_t i = 0; i < w.size(); ++i) w[i] = (int8_t)(int)filt.data[i];
    bw_ = I.upload(w);
    if (op.in.size() > 2 && I.has_weight(op.in[2])) {
      const auto &b = I.weight(op.in[2]).data;
      TPUCB_CHECK(b.size() == (size_t)batch_ * n_, "fc %s: bias needs batch * n values", op.name.c_str());
      bb_ = I.upload(to_i32(b, (int)b.size()));
    }
    bm_ = I.upload(to_i32(mu, batch_, true));
    br_ = I.upload(to_i32(rs, batch_, true));
    alg_ops = 2.0 * batch_ * m_ * k_ * n_;
    alg_bytes = (double)batch_ * ((double)m_ * k_ + (double)n_ * k_ + (double)m_ * n_ + 4.0 * n_ + 8);
  }
  void invoke(cudaStream_t s) override {
    if (batch_ > 0) {
      const size_t total = (size_t)batch_ * n_ * out_->cp;
      launch_k(fc_batched_i8_kernel, grid_for(total, 128, I_.sm_count), 128, 0, s, (const int8_t *)in_->dev, bw_, bb_, bm_, br_,
               (int8_t *)out_->dev, batch_, m_, k_, n_, out_->cp, do_relu_);
    } else if (f32_) launch_fc_f32((const float *)in_->dev, f32_w_, f32_b_, (float *)out_->dev, m_, kdev_, n_, out_->cp, do_relu_, s);
    else launch_conv_plan(plan_, s, I_.sm_count);
  }
  bool is_batched() const { return batch_ > 0; }
  ConvPlan plan_;

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  int m_ = 1, k_ = 1, n_ = 1, kdev_ = 1, do_relu_ = 0;
  bool f32_ = false;
  const float *f32_w_ = nullptr, *f32_b_ = nullptr;
  int batch_ = 0; // > 0: batched inner product (setup_batched)
  const int8_t *bw_ = nullptr;
  const int32_t *bb_ = nullptr, *bm_ = nullptr, *br_ = nullptr;
};

// -------------------------------------------------------------------------- Pooling
// PoolingOpKernel (core/pooling.cpp:33-160).
class PoolOp : public OpKernel {
public:
  PoolOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out, bool is_avg) : I_(I), in_(in), out_(out) {
    PoolArgs a;
    a.n = in->n; a.c = in->c; a.cp = in->cp; a.ih = in->h; a.iw = in->w; a.oh = out->h; a.ow = out->w;
    a.kh = op.geti("kh", 1); a.kw = op.geti("kw", 1); a.sh = op.geti("sh", 1); a.sw = op.geti("sw", 1);
    a.pt = op.geti("pt", 0); a.pl = op.geti("pl", 0);
    a.method = is_avg ? 1 : 0;
    a.mult = 0; a.rshift = 0;
    count_include_pad_ = op.geti("count_include_pad", 0);
    TPUCB_CHECK(!op.geti("do_relu", 0), "pool %s: do_relu is not supported (the reference asserts it off)", op.name.c_str());
    if (in->dtype == DT_I8 && is_avg) {
      TPUCB_CHECK(op.in.size() >= 5 && I.has_weight(op.in[3]) && I.has_weight(op.in[4]),
                  "pool_avg %s: INT8 needs rshift and multiplier operands", op.name.c_str());
      a.rshift = (int)(uint32_t)I.weight(op.in[3]).data.at(0);
      a.mult = (int)(uint32_t)I.weight(op.in[4]).data.at(0);
    }
    a_ = a;
    alg_bytes = ((double)in->numel() + out->numel()) * in->elsize();
  }
  void invoke(cudaStream_t s) override {
    if (in_->dtype == DT_I8) {
      size_t total = out_->pixels() * (out_->cp / 16);
      if (a_.method == 0)
        launch_k(pool_max_i8_kernel, grid_for(total, 128, I_.sm_count), 128, 0, s, (const int8_t *)in_->dev, (int8_t *)out_->dev, a_);
      else if (a_.kh * a_.kw >= 16)
        launch_k(pool_avg_wide_i8_kernel, grid_for(total * 8, 128, I_.sm_count), 128, 0, s, (const int8_t *)in_->dev, (int8_t *)out_->dev, a_);
      else
        launch_k(pool_i8_kernel, grid_for(total, 128, I_.sm_count), 128, 0, s, (const int8_t *)in_->dev, (int8_t *)out_->dev, a_);
    } else if (in_->dtype == DT_BF16) {
      size_t total = out_->pixels() * (out_->cp / 8);
      launch_k(pool_bf16_kernel, grid_for(total, 128, I_.sm_count), 128, 0, s, (const uint4 *)in_->dev, (uint4 *)out_->dev, a_, count_include_pad_);
    } else {
      launch_pool_f32((const float *)in_->dev, (float *)out_->dev, a_, count_include_pad_, s, I_.sm_count);
    }
  }

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  PoolArgs a_;
  int count_include_pad_ = 0;
};

// -------------------------------------------------------------------------- Eltwise
// EltwiseAddOpKernel / EltwiseMulOpKernel (core/eltwise.cpp:7-107, 318-357).
class EltwiseOp : public OpKernel {
public:
  EltwiseOp(Interpreter &I, const ParsedOp &op, std::vector<TensorPtr> ins, TensorPtr out, bool is_mul)
      : I_(I), ins_(ins), out_(out), is_mul_(is_mul) {
    const int nin = (int)ins.size();
    TPUCB_CHECK(nin >= 1 && nin <= 4, "eltwise %s: %d inputs not supported (max 4)", op.name.c_str(), nin);
    for (auto &t : ins)
      TPUCB_CHECK(t->bytes() == out->bytes() && t->dtype == out->dtype, "eltwise %s: operand %s differs in shape or type",
                  op.name.c_str(), t->name.c_str());
    do_relu_ = op.geti("do_relu", 0);
    alg_bytes = (double)(nin + 1) * out->numel() * out->elsize();
    if (out->dtype == DT_I8) {
      // operands: inputs..., quant_scale, quant_zeropoint, quant_rshift, quant_multiplier
      TPUCB_CHECK((int)op.in.size() >= nin + 4 && I.has_weight(op.in[nin + 2]) && I.has_weight(op.in[nin + 3]),
                  "eltwise %s: INT8 needs rshift and multiplier operands", op.name.c_str());
      const auto &rs = I.weight(op.in[nin + 2]).data;
      const auto &mu = I.weight(op.in[nin + 3]).data;
      a_.nin = nin;
      a_.do_relu = do_relu_;
      a_.rshift = (int)(uint32_t)rs.at(0);
      a_.qdm_mult = 0;
      for (int i = 0; i < nin; ++i) a_.in[i] = (const int8_t *)ins[i]->dev;
      if (is_mul) a_.qdm_mult = (int)(uint32_t)mu.at(0);
      else
        for (int i = 0; i < nin; ++i) a_.mult[i] = (int)(int8_t)mu.at(i);
    } else if (out->dtype == DT_BF16) {
      b_.nin = nin;
      b_.do_relu = do_relu_;
      for (int i = 0; i < nin; ++i) {
        b_.in[i] = (const uint4 *)ins[i]->dev;
        b_.coeff[i] = 1.0f;
      }
      parse_coeff(op, b_.coeff, is_mul ? 0 : nin);
    } else {
      TPUCB_CHECK(out->dtype == DT_F32 && !is_mul, "eltwise %s: fp32 supports add only", op.name.c_str());
      f_.nin = nin;
      f_.lo = nullptr;
      f_.do_relu = do_relu_;
      for (int i = 0; i < nin; ++i) {
        f_.in[i] = (const float *)ins[i]->dev;
        f_.coeff[i] = 1.0f;
      }
      parse_coeff(op, f_.coeff, nin);
    }
  }
  // INT8 two-input add that a producing convolution's epilogue can take over
  bool is_plain_i8_add() const { return out_->dtype == DT_I8 && !is_mul_ && ins_.size() == 2; }
  const std::vector<TensorPtr> &inputs() const { return ins_; }
  const TensorPtr &out() const { return out_; }
  const EltwiseArgs &i8_args() const { return a_; }
  // fp32 add whose result feeds a TF32 x 3 convolution: also write that convolution's remainder operand
  bool can_write_remainder() const { return out_->dtype == DT_F32 && !is_mul_; }
  void set_remainder_out(float *lo) { f_.lo = lo; }
  static void parse_coeff(const ParsedOp &op, float *coeff, int nin) {
    std::string co = op.gets("coeff", "");
    if (co.empty()) return;
    std::stringstream ss(co);
    std::string tok;
    int i = 0;
    while (std::getline(ss, tok, ',') && i < nin) coeff[i++] = (float)atof(tok.c_str());
  }
  void invoke(cudaStream_t s) override {
    if (out_->dtype == DT_BF16) {
      size_t nvec = out_->bytes() / 16;
      if (is_mul_) launch_k(eltwise_bf16_kernel<true>, grid_for(nvec, 256, I_.sm_count), 256, 0, s, b_, (uint4 *)out_->dev, nvec);
      else launch_k(eltwise_bf16_kernel<false>, grid_for(nvec, 256, I_.sm_count), 256, 0, s, b_, (uint4 *)out_->dev, nvec);
    } else if (out_->dtype == DT_I8) {
      size_t nvec = out_->bytes() / 16;
      if (is_mul_) launch_k(eltwise_mul_i8_kernel, grid_for(nvec, 256, I_.sm_count), 256, 0, s, a_, (int8_t *)out_->dev, nvec);
      else {
        const int grid = grid_for((nvec + 1) / 2, 256, I_.sm_count);
        int8_t *o = (int8_t *)out_->dev;
#define TPUCB_ELT(N)                                                                               \
  if (a_.do_relu) launch_k(eltwise_add_i8_kernel<N, true>, grid, 256, 0, s, a_, o, nvec);               \
  else launch_k(eltwise_add_i8_kernel<N, false>, grid, 256, 0, s, a_, o, nvec);
        switch (a_.nin) {
        case 1: TPUCB_ELT(1) break;
        case 2: TPUCB_ELT(2) break;
        case 3: TPUCB_ELT(3) break;
        default: TPUCB_ELT(4) break;
        }
#undef TPUCB_ELT
      }
    } else {
      size_t n = out_->bytes() / 4;
      launch_k(eltwise_add_f32_kernel, grid_for(n / 4, 256, I_.sm_count), 256, 0, s, f_, (float *)out_->dev, n);
    }
  }

private:
  Interpreter &I_;
  std::vector<TensorPtr> ins_;
  TensorPtr out_;
  bool is_mul_;
  int do_relu_ = 0;
  EltwiseArgs a_;
  EltwiseF32Args f_;
  EltwiseBf16Args b_;
};

// --------------------------------------------------------------------------- Concat
// ConcatOpKernel (core/concat.cpp:7-90), channel axis: INT8 with per-input rescale; BF16 as a plain copy (the byte
// kernels with two bytes per channel).
class ConcatOp : public OpKernel {
public:
  ConcatOp(Interpreter &I, const ParsedOp &op, std::vector<TensorPtr> ins, TensorPtr out) : I_(I), ins_(ins), out_(out) {
    TPUCB_CHECK(op.geti("axis", 1) == 1, "concat %s: only the channel axis is supported", op.name.c_str());
    TPUCB_CHECK(out->dtype == DT_I8 || out->dtype == DT_BF16, "concat %s: INT8 and BF16 are implemented", op.name.c_str());
    const int nin = (int)ins.size();
    do_relu_ = op.geti("do_relu", 0);
    es_ = (int)out->elsize();
    TPUCB_CHECK(es_ == 1 || !do_relu_, "concat %s: BF16 concat with do_relu is not implemented", op.name.c_str());
    for (auto &t : ins) TPUCB_CHECK(t->dtype == out->dtype, "concat %s: input and output types differ", op.name.c_str());
    mult_.assign(nin, 1);
    rsh_.assign(nin, 0);
    if (es_ == 1 && (int)op.in.size() >= nin + 4 && I.has_weight(op.in[nin + 2]) && I.has_weight(op.in[nin + 3])) {
      need_quant_ = true;
      const auto &rs = I.weight(op.in[nin + 2]).data;
      const auto &mu = I.weight(op.in[nin + 3]).data;
      for (int i = 0; i < nin; ++i) {
        rsh_[i] = (int)(uint32_t)rs.at(i);
        mult_[i] = (int)(uint32_t)mu.at(i);
      }
    }
    int c = 0;
    for (auto &t : ins) c += t->c;
    TPUCB_CHECK(c == out->c, "concat %s: channel counts do not add up", op.name.c_str());
    alg_bytes = 2.0 * out->numel() * es_;
  }
  void invoke(cudaStream_t s) override {
    int off = 0; // in bytes of a pixel row of the output
    const int ocp = out_->cp * es_;
    for (size_t i = 0; i < ins_.size(); ++i) {
      auto &t = ins_[i];
      const int cb = t->c * es_, cpb = t->cp * es_; // channel bytes: BF16 moves as two bytes per channel
      size_t total = t->pixels() * cb;
      int requant = need_quant_ && !(mult_[i] == 1 && rsh_[i] == 0);
      if (cb % 16 == 0 && off % 16 == 0 && cpb % 16 == 0 && ocp % 16 == 0) {
        size_t nvec = t->pixels() * (cb / 16);
        launch_k(concat_slice_i8_vec_kernel, grid_for(nvec, 256, I_.sm_count), 256, 0, s, 
            (const uint4 *)t->dev, (uint4 *)out_->dev, t->pixels(), cb / 16, cpb / 16, ocp / 16, off / 16,
            mult_[i], rsh_[i], requant, do_relu_);
        off += cb;
        continue;
      }
      launch_k(concat_slice_i8_kernel, grid_for(total, 256, I_.sm_count), 256, 0, s, 
          (const int8_t *)t->dev, (int8_t *)out_->dev, t->pixels(), cb, cpb, ocp, off, mult_[i], rsh_[i],
          requant, do_relu_);
      off += cb;
    }
  }
  int kernel_launches() const override { return (int)ins_.size(); }

private:
  Interpreter &I_;
  std::vector<TensorPtr> ins_;
  TensorPtr out_;
  std::vector<int> mult_, rsh_;
  bool need_quant_ = false;
  int do_relu_ = 0;
  int es_ = 1; // bytes per channel value
};

// ------------------------------------------------------------ Upsample / PixelShuffle
// UpsampleOpKernel (core/upsample.cpp:20-41), DepthToSpaceOpKernel (core/depthtospace.cpp:50-80).
class MoveOp : public OpKernel {
public:
  MoveOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out, int mode) : I_(I), in_(in), out_(out) {
    MoveArgs a;
    a.n = in->n; a.ic = in->c; a.ih = in->h; a.iw = in->w; a.icp = in->cp;
    a.oc = out->c; a.oh = out->h; a.ow = out->w; a.ocp = out->cp;
    a.es = (int)in->elsize();
    a.scale_h = op.geti("scale_h", 1); a.scale_w = op.geti("scale_w", 1);
    a.r = op.geti("upscale_factor", 1);
    a.mode = mode == 0 ? 0 : (op.gets("mode", "CRD") == "DCR" ? 2 : 1);
    TPUCB_CHECK(in->dtype == out->dtype, "%s: input and output types differ", op.name.c_str());
    a_ = a;
    alg_bytes = ((double)in->numel() + out->numel()) * in->elsize();
  }
  void invoke(cudaStream_t s) override {
    size_t total = out_->pixels() * out_->cp;
    launch_k(move_kernel, grid_for(total, 256, I_.sm_count), 256, 0, s, (const uint8_t *)in_->dev, (uint8_t *)out_->dev, a_);
  }

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  MoveArgs a_;
};

// ------------------------------------------------------------------- ReLU / LeakyReLU
// ReluOpKernel, LeakyReluOpKernel (core/activation.cpp:104-180).
class LeakyReluOp : public OpKernel {
public:
  LeakyReluOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out, bool plain) : I_(I), in_(in), out_(out), plain_(plain) {
    TPUCB_CHECK(in->dtype == out->dtype && (in->dtype == DT_I8 || in->dtype == DT_BF16), "%s: INT8 and BF16 are implemented",
                op.name.c_str());
    bf16_ = in->dtype == DT_BF16;
    slope_ = (float)op.getf("negative_slope", 0.0);
    alg_bytes = 2.0 * out->numel() * (bf16_ ? 2 : 1);
    if (bf16_) return;
    if (!plain) {
      // operands 5..8: rshift_pos, multiplier_pos, rshift_neg, multiplier_neg (activation.cpp:113-124)
      TPUCB_CHECK(op.in.size() >= 9, "leaky_relu %s: INT8 needs 4 rescale operands", op.name.c_str());
      rp = (int)(uint32_t)I.weight(op.in[5]).data.at(0);
      mp = (int)I.weight(op.in[6]).data.at(0);
      rn = (int)(uint32_t)I.weight(op.in[7]).data.at(0);
      mn = (int)I.weight(op.in[8]).data.at(0);
    }
    alg_bytes = 2.0 * out->numel();
  }
  void invoke(cudaStream_t s) override {
    size_t nvec = out_->bytes() / 16;
    if (bf16_) {
      launch_k(leaky_relu_bf16_kernel, grid_for(nvec, 256, I_.sm_count), 256, 0, s, (const uint4 *)in_->dev, (uint4 *)out_->dev,
               nvec, slope_, plain_ ? 1 : 0);
      return;
    }
    launch_k(leaky_relu_i8_kernel, grid_for(nvec, 256, I_.sm_count), 256, 0, s, (const int8_t *)in_->dev, (int8_t *)out_->dev,
                                                                          nvec, mp, rp, mn, rn, plain_ ? 1 : 0);
  }
  int mp = 0, rp = 0, mn = 0, rn = 0;
  bool plain() const { return plain_; }
  const TensorPtr &in() const { return in_; }
  const TensorPtr &out() const { return out_; }

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  bool plain_;
  bool bf16_ = false;
  float slope_ = 0.0f;
};

// ---------------------------------------------------------------------- LUT activations
// SigmoidOpKernel / MishOpKernel / ExpOpKernel (core/activation.cpp:47-102, 251-268): INT8 mode is a
// 256-entry table gather, BF16 mode the slope-interpolated table of bf16_lut_slope.
// ReciprocalOpKernel BF16: bf16_lut_mantissa with the pow(-1) tables.
class LutOp : public OpKernel {
public:
  LutOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out) : I_(I), in_(in), out_(out) {
    TPUCB_CHECK(in->dtype == out->dtype, "%s: input and output types differ", op.name.c_str());
    TPUCB_CHECK(op.in.size() >= 3, "%s: expects input and two table operands", op.name.c_str());
    const auto &t0 = I.weight(op.in[1]).data;
    const auto &t1 = I.weight(op.in[2]).data;
    TPUCB_CHECK(t0.size() >= 256, "%s: table operand needs at least 256 entries", op.name.c_str());
    if (in->dtype == DT_I8) {
      std::vector<int8_t> t(256);
      for (int i = 0; i < 256; ++i) t[i] = (int8_t)(int)t0[i];
      tab_i8_ = I.upload(t);
      alg_bytes = 2.0 * out->numel();
    } else {
      TPUCB_CHECK(in->dtype == DT_BF16, "%s: lookup tables run in INT8 or BF16", op.name.c_str());
      TPUCB_CHECK(t1.size() >= 256, "%s: second table needs at least 256 entries", op.name.c_str());
      t0_ = I.upload(std::vector<float>(t0.begin(), t0.begin() + 256));
      t1_ = I.upload(std::vector<float>(t1.begin(), t1.begin() + 256));
      mantissa_ = op.type == "reciprocal";
      double range = op.type == "sigmoid" ? 12 : (op.type == "mish" ? 8 : 15); // lut_func.hpp:8-15
      scale_ = bf16_round((float)(256.0 / (2 * range)));
      alg_bytes = 4.0 * out->numel();
    }
  }
  void invoke(cudaStream_t s) override {
    if (in_->dtype == DT_I8) {
      size_t nvec = out_->bytes() / 16;
      launch_k(lut_i8_kernel, grid_for(nvec, 256, I_.sm_count), 256, 0, s, (const int8_t *)in_->dev, (int8_t *)out_->dev, nvec, tab_i8_);
    } else if (mantissa_) {
      size_t n = out_->bytes() / 2;
      launch_k(lut_bf16_mantissa_kernel, grid_for(n, 256, I_.sm_count), 256, 0, s, (const uint16_t *)in_->dev, (uint16_t *)out_->dev, n, t0_, t1_);
    } else {
      size_t n = out_->bytes() / 2;
      launch_k(lut_bf16_slope_kernel, grid_for(n / 8, 256, I_.sm_count), 256, 0, s, (const uint16_t *)in_->dev, (uint16_t *)out_->dev, n, t0_, t1_, scale_);
    }
  }

  bool is_bf16_slope() const { return in_->dtype == DT_BF16 && !mantissa_; }
  const float *base_table() const { return t0_; }
  const float *slope_table() const { return t1_; }
  float scale() const { return scale_; }
  const TensorPtr &in() const { return in_; }
  const TensorPtr &out() const { return out_; }

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  const int8_t *tab_i8_ = nullptr;
  const float *t0_ = nullptr, *t1_ = nullptr;
  bool mantissa_ = false;
  float scale_ = 1;
};

// ------------------------------------------------ fused INT8 -> BF16 activation -> INT8
// quant(INT8->BF16), a slope-table activation and quant(BF16->INT8) whose intermediate tensors have
// no other consumer run as one launch at the position of the first quant; all three tensors are
// still written. The two later ops become placeholders that launch nothing.
class ActChainOp : public OpKernel {
public:
  ActChainOp(Interpreter &I, const QuantOp &q0, const LutOp &lut, const QuantOp &q1)
      : I_(I), in_(q0.in()), deq_(q0.out()), act_(lut.out()), out_(q1.out()), s_in_(q0.scale()),
        s_lut_(lut.scale()), s_out_(q1.scale()), base_(lut.base_table()), slope_(lut.slope_table()) {
    alg_bytes = 6.0 * out_->numel();
  }
  void invoke(cudaStream_t s) override {
    size_t nvec = out_->pixels() * out_->cp / 16;
    launch_k(act_chain_i8_kernel, grid_for(nvec, 256, I_.sm_count), 256, 0, s, 
        (const uint4 *)in_->dev, (uint4 *)deq_->dev, (uint4 *)act_->dev, (uint4 *)out_->dev, nvec, s_in_, s_lut_,
        base_, slope_, s_out_);
  }

private:
  Interpreter &I_;
  TensorPtr in_, deq_, act_, out_;
  float s_in_, s_lut_, s_out_;
  const float *base_, *slope_;
};

class FusedAwayOp : public OpKernel {
public:
  void invoke(cudaStream_t) override {}
  int kernel_launches() const override { return 0; }
};

// ------------------------------------------------- ops of neighbouring networks
inline TensorGeom geom_of(const TensorPtr &t) { return TensorGeom{t->n, t->c, t->h, t->w, t->cp, t->wl, t->wphys}; }
// the reference's getNCHW: a shape of rank < 4 padded with ones on the left (align_right) or right
inline void shape4_of(const TensorPtr &t, bool align_right, int (&s)[4]) {
  const int r = (int)t->shape.size();
  for (int i = 0; i < 4; ++i) s[i] = 1;
  for (int i = 0; i < r; ++i) s[align_right ? 4 - r + i : i] = (int)t->shape[i];
}

// EltwiseMaxOpKernel / EltwiseMinOpKernel, INT8 (core/eltwise.cpp:100-263).
class EltwiseMaxMinOp : public OpKernel {
public:
  EltwiseMaxMinOp(Interpreter &I, const ParsedOp &op, std::vector<TensorPtr> ins, TensorPtr out, bool is_min)
      : I_(I), out_(out) {
    const int nin = (int)ins.size();
    TPUCB_CHECK(nin >= 1 && nin <= 4, "%s %s: %d inputs not supported (max 4)", op.type.c_str(), op.name.c_str(), nin);
    TPUCB_CHECK(out->dtype == DT_I8, "%s %s: only INT8 is implemented", op.type.c_str(), op.name.c_str());
    for (auto &t : ins)
      TPUCB_CHECK(t->bytes() == out->bytes() && t->dtype == DT_I8 && !t->padded_rows(), "%s %s: operand %s differs in shape or type",
                  op.type.c_str(), op.name.c_str(), t->name.c_str());
    TPUCB_CHECK((int)op.in.size() >= nin + 4 && I.has_weight(op.in[nin + 2]) && I.has_weight(op.in[nin + 3]),
                "%s %s: INT8 needs rshift and multiplier operands", op.type.c_str(), op.name.c_str());
    a_.nin = nin;
    a_.do_relu = op.geti("do_relu", 0);
    a_.is_min = is_min ? 1 : 0;
    a_.rshift = (int)(uint32_t)I.weight(op.in[nin + 2]).data.at(0);
    for (int i = 0; i < nin; ++i) {
      a_.in[i] = (const int8_t *)ins[i]->dev;
      a_.mult[i] = (int)(int8_t)I.weight(op.in[nin + 3]).data.at(i);
    }
    alg_bytes = (double)(nin + 1) * out->numel();
  }
  void invoke(cudaStream_t s) override {
    size_t nvec = out_->bytes() / 16;
    launch_k(eltwise_maxmin_i8_kernel, grid_for(nvec, 256, I_.sm_count), 256, 0, s, a_, (int8_t *)out_->dev, nvec);
  }

private:
  Interpreter &I_;
  TensorPtr out_;
  MaxMinArgs a_;
};

// BroadcastAdd / Sub / Mul (core/broadcast.cpp:8-156), INT8 and fp32.
class BroadcastOp : public OpKernel {
public:
  BroadcastOp(Interpreter &I, const ParsedOp &op, TensorPtr a, TensorPtr b, TensorPtr out) : I_(I), a_(a), b_(b), out_(out) {
    TPUCB_CHECK(a->dtype == out->dtype && b->dtype == out->dtype && (out->dtype == DT_I8 || out->dtype == DT_F32),
                "%s %s: operands and result must all be INT8 or all fp32", op.type.c_str(), op.name.c_str());
    const bool align_right = op.geti("align_right", 1) != 0;
    shape4_of(a, align_right, p_.sa);
    shape4_of(b, align_right, p_.sb);
    size_t total = 1;
    for (int i = 0; i < 4; ++i) {
      p_.so[i] = std::max(p_.sa[i], p_.sb[i]);
      TPUCB_CHECK((p_.sa[i] == p_.so[i] || p_.sa[i] == 1) && (p_.sb[i] == p_.so[i] || p_.sb[i] == 1),
                  "%s %s: shapes do not broadcast", op.type.c_str(), op.name.c_str());
      total *= (size_t)p_.so[i];
    }
    TPUCB_CHECK(total == out->numel(), "%s %s: result has %zu values, broadcast gives %zu", op.type.c_str(), op.name.c_str(),
                out->numel(), total);
    p_.ga = geom_of(a); p_.gb = geom_of(b); p_.go = geom_of(out);
    p_.op = op.type == "broadcast_add" ? 0 : (op.type == "broadcast_sub" ? 1 : 2);
    p_.dt = out->dtype;
    p_.do_relu = op.geti("do_relu", 0);
    p_.mult0 = p_.mult1 = 1;
    p_.rshift = 0;
    if (out->dtype == DT_I8) {
      // operands: a, b, quant_scale, quant_zeropoint, quant_rshift, quant_multiplier
      TPUCB_CHECK(op.in.size() >= 6 && I.has_weight(op.in[4]) && I.has_weight(op.in[5]),
                  "%s %s: INT8 needs rshift and multiplier operands", op.type.c_str(), op.name.c_str());
      const auto &mu = I.weight(op.in[5]).data;
      p_.rshift = (int)(uint32_t)I.weight(op.in[4]).data.at(0);
      if (p_.op == 2) {
        p_.mult0 = (int)(uint32_t)mu.at(0);
      } else {
        p_.mult0 = (int)(int8_t)mu.at(0);
        p_.mult1 = (int)(int8_t)mu.at(1);
      }
    }
    alg_bytes = ((double)a->numel() + b->numel() + out->numel()) * out->elsize();
  }
  void invoke(cudaStream_t s) override {
    launch_k(broadcast_kernel, grid_for(out_->numel(), 256, I_.sm_count), 256, 0, s, a_->dev, b_->dev, out_->dev, p_);
  }

private:
  Interpreter &I_;
  TensorPtr a_, b_, out_;
  BroadcastArgs p_;
};

// PadOpKernel (core/pad.cpp:112-141), CropOpKernel (core/crop.cpp:45-92), PermuteOpKernel (core/permute.cpp:35-45).
class RemapOp : public OpKernel {
public:
  RemapOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out) : I_(I), in_(in), out_(out) {
    TPUCB_CHECK(in->dtype == out->dtype, "%s %s: input and result types differ", op.type.c_str(), op.name.c_str());
    shape4_of(in, false, p_.si);
    shape4_of(out, false, p_.so);
    p_.gi = geom_of(in); p_.go = geom_of(out);
    p_.es = (int)out->elsize();
    for (int i = 0; i < 4; ++i) { p_.a[i] = 0; p_.b[i] = 1; }
    if (op.type == "pad") {
      std::vector<int> pads = op.getl("pads");
      TPUCB_CHECK(pads.size() == 8, "pad %s: pads needs 8 entries", op.name.c_str());
      p_.mode = op.gets("mode", "constant") == "edge" ? 1 : 0;
      for (int i = 0; i < 4; ++i) {
        p_.a[i] = pads[i];
        TPUCB_CHECK(p_.si[i] + pads[i] + pads[i + 4] == p_.so[i], "pad %s: result shape does not match the pads", op.name.c_str());
      }
      if (p_.mode == 1)
        TPUCB_CHECK(pads[0] == 0 && pads[1] == 0 && pads[4] == 0 && pads[5] == 0, "pad %s: edge mode pads height and width only",
                    op.name.c_str());
    } else if (op.type == "crop") {
      std::vector<int> off = op.getl("crop_offset"), steps = op.getl("steps");
      p_.mode = 2;
      for (int i = 0; i < 4; ++i) {
        p_.a[i] = i < (int)off.size() ? off[i] : 0;
        p_.b[i] = i < (int)steps.size() ? steps[i] : 1;
        TPUCB_CHECK(p_.b[i] >= 1 && p_.a[i] >= 0 && (p_.so[i] - 1) * p_.b[i] + p_.a[i] < p_.si[i],
                    "crop %s: window leaves the input in dimension %d", op.name.c_str(), i);
      }
    } else {
      std::vector<int> order = op.getl("order");
      TPUCB_CHECK(order.size() == 4, "permute %s: order needs 4 entries", op.name.c_str());
      p_.mode = 3;
      int seen = 0;
      for (int i = 0; i < 4; ++i) {
        TPUCB_CHECK(order[i] >= 0 && order[i] < 4, "permute %s: bad order", op.name.c_str());
        seen |= 1 << order[i];
        p_.a[i] = order[i];
        TPUCB_CHECK(p_.so[i] == p_.si[order[i]], "permute %s: result shape does not match the order", op.name.c_str());
      }
      TPUCB_CHECK(seen == 15, "permute %s: order is not a permutation", op.name.c_str());
    }
    alg_bytes = ((double)std::min(in->numel(), out->numel()) + out->numel()) * out->elsize();
  }
  void invoke(cudaStream_t s) override {
    launch_k(remap_kernel, grid_for(out_->numel(), 256, I_.sm_count), 256, 0, s, (const uint8_t *)in_->dev, (uint8_t *)out_->dev, p_);
  }

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  RemapArgs p_;
};

// ReduceOpKernel (core/reduce.cpp:10-115): mean / sum / max / min over consecutive axes, INT8 and fp32.
class ReduceOp : public OpKernel {
public:
  ReduceOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out) : I_(I), in_(in), out_(out) {
    TPUCB_CHECK(in->dtype == out->dtype && (out->dtype == DT_I8 || out->dtype == DT_F32), "%s %s: INT8 or fp32 only",
                op.type.c_str(), op.name.c_str());
    std::vector<int> axes = op.getl("axes");
    TPUCB_CHECK(!axes.empty(), "%s %s: axes missing", op.type.c_str(), op.name.c_str());
    for (size_t i = 1; i < axes.size(); ++i)
      TPUCB_CHECK(axes[i] == axes[i - 1] + 1, "%s %s: axes must be consecutive", op.type.c_str(), op.name.c_str());
    const int rank = (int)in->shape.size();
    TPUCB_CHECK(axes.front() >= 0 && axes.back() < rank, "%s %s: axis out of range", op.type.c_str(), op.name.c_str());
    long long outer = 1, axis = 1, inner = 1;
    for (int i = 0; i < rank; ++i) {
      if (i < axes.front()) outer *= in->shape[i];
      else if (i <= axes.back()) axis *= in->shape[i];
      else inner *= in->shape[i];
    }
    TPUCB_CHECK((size_t)(outer * inner) == out->numel(), "%s %s: result has %zu values, expected %lld", op.type.c_str(),
                op.name.c_str(), out->numel(), outer * inner);
    p_.gi = geom_of(in); p_.go = geom_of(out);
    p_.outer = (int)outer; p_.axis = (int)axis; p_.inner = (int)inner;
    p_.type = op.type == "reduce_mean" ? 0 : (op.type == "reduce_sum" ? 1 : (op.type == "reduce_max" ? 2 : (op.type == "reduce_min" ? 3 : 4)));
    p_.dt = out->dtype;
    p_.coeff = (float)op.getf("coeff", 0.5);
    // reduce_l2 ends in pow(sum, coeff) on the fp32 sum; the INT8 form would requantise that float and the BF16 form
    // goes through lookup tables: only the fp32 form is implemented
    TPUCB_CHECK(p_.type != 4 || out->dtype == DT_F32, "reduce_l2 %s: only fp32 is implemented", op.name.c_str());
    p_.mult = 1; p_.rshift = 0;
    if (out->dtype == DT_I8) {
      // operands: input, quant_scale, quant_zeropoint, quant_rshift, quant_multiplier
      if (op.in.size() > 3 && I.has_weight(op.in[3])) p_.rshift = (int)(uint32_t)I.weight(op.in[3]).data.at(0);
      if (op.in.size() > 4 && I.has_weight(op.in[4])) p_.mult = (int)(uint32_t)I.weight(op.in[4]).data.at(0);
    }
    p_.requant = (p_.rshift != 0 || p_.mult != 1) ? 1 : 0;
    alg_bytes = ((double)in->numel() + out->numel()) * out->elsize();
  }
  void invoke(cudaStream_t s) override {
    launch_k(reduce_kernel, grid_for(out_->numel(), 128, I_.sm_count), 128, 0, s, in_->dev, out_->dev, p_);
  }

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  ReduceArgs p_;
};

// --------------------------------------------------------------------------- MatMul
// MatMulOpKernel (core/matmul.cpp:9-97) with the dimension rule of parseMatMulParam
// (lib/Dialect/TPU/IR/TPUOperationSupport.cpp:615-655).
class MatMulOp : public OpKernel {
public:
  MatMulOp(Interpreter &I, const ParsedOp &op, TensorPtr a, TensorPtr b, TensorPtr out) : I_(I), a_(a), b_(b), out_(out) {
    TPUCB_CHECK(a->dtype == out->dtype && b->dtype == out->dtype, "matmul %s: operands and result must share a type", op.name.c_str());
    const auto &as = a->shape, &bs = b->shape, &os = out->shape;
    const int rank = (int)os.size();
    TPUCB_CHECK(rank >= 2 && rank <= 4 && (int)as.size() == rank && (int)bs.size() == rank, "matmul %s: operands and result need the same rank (2 to 4)",
                op.name.c_str());
    MatMulArgs &p = p_;
    p.lt = op.geti("left_transpose", 0); p.rt = op.geti("right_transpose", 0); p.ot = op.geti("output_transpose", 0);
    const int axis = rank - 1;
    p.bh = p.bl = 1;
    if (p.lt || p.rt || p.ot) {
      TPUCB_CHECK(rank >= 3, "matmul %s: transposes need rank 3 or 4", op.name.c_str());
      p.K = (int)as[axis]; p.N = (int)os[axis];
      if (p.lt) { p.bl = (int)as[axis - 1]; p.M = (int)as[axis - 2]; }
      else { p.bl = (int)as[axis - 2]; p.M = (int)as[axis - 1]; }
      if (axis == 3) p.bh = (int)as[0];
    } else {
      for (int i = 0; i < axis - 1; ++i) {
        TPUCB_CHECK(as[i] == os[i] && as[i] == bs[i], "matmul %s: batch dimensions differ", op.name.c_str());
        p.bh *= (int)as[i];
      }
      p.M = (int)as[axis - 1]; p.K = (int)as[axis]; p.N = (int)bs[axis];
      TPUCB_CHECK(p.K == bs[axis - 1] && p.M == os[axis - 1] && p.N == os[axis], "matmul %s: [M,K] x [K,N] -> [M,N] shapes do not agree", op.name.c_str());
    }
    const size_t batch = (size_t)p.bh * p.bl;
    TPUCB_CHECK(a->numel() == batch * p.M * p.K && b->numel() == batch * p.K * p.N && out->numel() == batch * p.M * p.N,
                "matmul %s: tensor sizes do not match batch %zu, M %d, K %d, N %d", op.name.c_str(), batch, p.M, p.K, p.N);
    TPUCB_CHECK(batch <= 65535, "matmul %s: batch %zu is beyond one launch", op.name.c_str(), batch);
    p.ga = geom_of(a); p.gb = geom_of(b); p.go = geom_of(out);
    p.dt = out->dtype;
    p.do_relu = op.geti("do_relu", 0);
    p.mult = 0; p.rshift = 0;
    if (out->dtype == DT_I8) {
      // operands: left, right, quant_scale, quant_zeropoint, quant_rshift, quant_multiplier
      TPUCB_CHECK(op.in.size() > 5 && I.has_weight(op.in[4]) && I.has_weight(op.in[5]), "matmul %s: INT8 needs rshift and multiplier operands", op.name.c_str());
      p.rshift = (int)(uint32_t)I.weight(op.in[4]).data.at(0);
      p.mult = (int)(uint32_t)I.weight(op.in[5]).data.at(0);
      TPUCB_CHECK((double)p.K * 127.0 * 128.0 < 2147483648.0, "matmul %s: K = %d overflows the int32 sum", op.name.c_str(), p.K);
    }
    p.requant = (p.rshift != 0 || p.mult != 0) ? 1 : 0;
    alg_ops = 2.0 * batch * p.M * p.K * p.N;
    alg_bytes = ((double)a->numel() + b->numel() + out->numel()) * out->elsize();
  }
  void invoke(cudaStream_t s) override {
    const dim3 grid((p_.N + 15) / 16, (p_.M + 15) / 16, p_.bh * p_.bl), block(16, 16);
    if (p_.dt == DT_I8) launch_k(matmul_kernel<DT_I8>, grid, block, 0, s, a_->dev, b_->dev, out_->dev, p_);
    else if (p_.dt == DT_BF16) launch_k(matmul_kernel<DT_BF16>, grid, block, 0, s, a_->dev, b_->dev, out_->dev, p_);
    else launch_k(matmul_kernel<DT_F32>, grid, block, 0, s, a_->dev, b_->dev, out_->dev, p_);
  }

private:
  Interpreter &I_;
  TensorPtr a_, b_, out_;
  MatMulArgs p_;
};

// ------------------------------------------------------------ fp32 Scale / Softmax
// ScaleOpKernel (core/scale.cpp:15-37), SoftmaxOpKernel::invoke_fp32 (core/softmax.cpp:49-86).
class ScaleOp : public OpKernel {
public:
  ScaleOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out) : I_(I), in_(in), out_(out) {
    TPUCB_CHECK(in->dtype == DT_F32 && out->dtype == DT_F32, "scale %s: fp32 only (as the reference)", op.name.c_str());
    std::vector<float> sc = I.weight(op.in[1]).data, bi(in->c, 0.0f);
    if (op.in.size() > 2 && I.has_weight(op.in[2])) bi = I.weight(op.in[2]).data;
    sc.resize(in->cp, 0.0f);
    bi.resize(in->cp, 0.0f);
    d_s_ = I.upload(sc);
    d_b_ = I.upload(bi);
    alg_bytes = 8.0 * out->numel();
  }
  void invoke(cudaStream_t s) override {
    size_t n = out_->bytes() / 4;
    launch_k(scale_f32_kernel, grid_for(n, 256, I_.sm_count), 256, 0, s, (const float *)in_->dev, d_s_, d_b_, (float *)out_->dev, n, out_->cp);
  }

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  const float *d_s_ = nullptr, *d_b_ = nullptr;
};

// BatchNormOpKernel (core/batchnorm.cpp:6-68), fp32 only as in the reference ("other mode please fused batchnorm").
// Operands: input, mean, variance, scale (one value). The reference scales mean and variance by 1 / scale[0] in
// fp32 for the duration of the call; the per-channel mean' and d = sqrt(variance' + epsilon) are formed here, once,
// with the same fp32 operations.
class BatchNormOp : public OpKernel {
public:
  BatchNormOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out) : I_(I), in_(in), out_(out) {
    TPUCB_CHECK(in->dtype == DT_F32 && out->dtype == DT_F32, "batchnorm %s: fp32 only (as the reference)", op.name.c_str());
    TPUCB_CHECK(op.in.size() >= 4, "batchnorm %s: expects input, mean, variance, scale", op.name.c_str());
    const auto &mean = I.weight(op.in[1]).data, &var = I.weight(op.in[2]).data, &scale = I.weight(op.in[3]).data;
    TPUCB_CHECK((int)mean.size() >= in->c && (int)var.size() >= in->c && !scale.empty(),
                "batchnorm %s: mean / variance need %d values and scale one", op.name.c_str(), in->c);
    const float eps = (float)op.getf("variance_epsilon", 1e-5);
    const float sf = 1.0f / scale[0];
    std::vector<float> m(in->cp, 0.0f), d(in->cp, 1.0f);
    for (int c = 0; c < in->c; ++c) {
      m[c] = mean[c] * sf;
      const float v = var[c] * sf;
      d[c] = sqrtf(v + eps);
    }
    d_m_ = I.upload(m);
    d_d_ = I.upload(d);
    alg_bytes = 8.0 * out->numel();
  }
  void invoke(cudaStream_t s) override {
    size_t n = out_->bytes() / 4;
    launch_k(batchnorm_f32_kernel, grid_for(n, 256, I_.sm_count), 256, 0, s, (const float *)in_->dev, d_m_, d_d_, (float *)out_->dev, n, out_->cp);
  }

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  const float *d_m_ = nullptr, *d_d_ = nullptr;
};

class SoftmaxOp : public OpKernel {
public:
  SoftmaxOp(Interpreter &I, const ParsedOp &op, TensorPtr in, TensorPtr out) : I_(I), in_(in), out_(out) {
    TPUCB_CHECK(in->dtype == out->dtype && out->dtype != DT_I8, "softmax %s: fp32 or BF16 (as the reference)", op.name.c_str());
    TPUCB_CHECK(op.geti("axis", 1) == 1, "softmax %s: channel axis only", op.name.c_str());
    alg_bytes = 2.0 * out->numel() * out->elsize();
    if (out->dtype == DT_BF16) {
      // operands: input, exponential_table, exponential_slope_table, reciprocal_table, reciprocal_mantissa_table
      TPUCB_CHECK(op.in.size() >= 5, "softmax %s: BF16 needs the four table operands", op.name.c_str());
      const float *t[4];
      for (int i = 0; i < 4; ++i) {
        const auto &w = I.weight(op.in[1 + i]).data;
        TPUCB_CHECK(w.size() >= 256, "softmax %s: table %s has %zu entries, expected 256", op.name.c_str(), op.in[1 + i].c_str(), w.size());
        t[i] = I.upload(std::vector<float>(w.begin(), w.begin() + 256));
      }
      b_.exp_base = t[0]; b_.exp_slope = t[1]; b_.rec_exp = t[2]; b_.rec_mant = t[3];
      b_.c = out->c; b_.cp = out->cp;
      b_.do_log = op.geti("do_log", 0);
      b_.lut_scale = bf16_round(256.0f / 30.0f); // the exp table spans [-15, 15] (lut_func.hpp:8-15)
      b_.const_val = bf16_round(bf16_round((float)out->c) / (float)out->c);
      smem_ = 2 * (size_t)out->c * sizeof(float);
      TPUCB_CHECK(smem_ <= 200 * 1024, "softmax %s: %d channels do not fit one CTA's shared memory", op.name.c_str(), out->c);
      if (smem_ > 48 * 1024)
        TPUCB_CUDA(cudaFuncSetAttribute(softmax_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_));
    }
  }
  void invoke(cudaStream_t s) override {
    if (out_->dtype == DT_BF16)
      launch_k(softmax_bf16_kernel, (unsigned)out_->pixels(), 128, smem_, s, (const uint16_t *)in_->dev, (uint16_t *)out_->dev, b_);
    else
      launch_k(softmax_f32_kernel, (unsigned)out_->pixels(), 128, 0, s, (const float *)in_->dev, (float *)out_->dev, out_->c, out_->cp);
  }

private:
  Interpreter &I_;
  TensorPtr in_, out_;
  SoftmaxBf16Args b_;
  size_t smem_ = 0;
};

// ====================================================================== Interpreter bodies

inline std::vector<std::string> split(const std::string &s, char sep) {
  std::vector<std::string> out;
  std::stringstream ss(s);
  std::string tok;
  while (std::getline(ss, tok, sep)) out.push_back(tok);
  return out;
}

inline ParsedOp parse_line(const std::string &line) {
  ParsedOp op;
  op.line = line;
  std::stringstream ss(line);
  std::string tok;
  ss >> op.type;
  while (ss >> tok) {
    auto eq = tok.find('=');
    TPUCB_CHECK(eq != std::string::npos, "module text: token '%s' is not key=value", tok.c_str());
    std::string k = tok.substr(0, eq), v = tok.substr(eq + 1);
    if (k == "name") op.name = v;
    else if (k == "in") op.in = split(v, ',');
    else if (k == "shape") {
      for (auto &d : split(v, ',')) op.shape.push_back(atoll(d.c_str()));
    } else if (k == "dtype") op.dtype = v;
    else op.attrs[k] = v;
  }
  TPUCB_CHECK(!op.name.empty(), "module text: op '%s' has no name", op.type.c_str());
  return op;
}

// Replaces every quant(INT8->BF16) -> slope-table activation -> quant(BF16->INT8) chain whose
// intermediates feed nothing else by one ActChainOp at the first op's position.
// Who writes the remainder operand (x minus the upper 19 bits of x) of the fp32 tensors that TF32 x 3 convolutions read:
// the kernel that produces the tensor when it can (an fp32 eltwise add or another TF32 x 3 convolution: 4 more bytes
// written per value, no separate pass), else the split pass of the FIRST convolution that reads it; later readers of
// the same tensor reuse the buffer. Ops run in program order, so the first reader always runs before the others.
inline void Interpreter::link_tf32_remainders() {
  for (auto &k : kernels) {
    auto *cv = dynamic_cast<Conv2DOp *>(k.get());
    if (!cv || !cv->is_tf32()) continue;
    DevTensor *t = cv->in().get();
    if (t->lo_by != 0) { // already filled by the producer or by an earlier reader
      cv->skip_split();
      continue;
    }
    OpKernel *prod = nullptr;
    for (auto &q : kernels)
      if (q->result.get() == t) prod = q.get();
    if (auto *pe = dynamic_cast<EltwiseOp *>(prod)) {
      if (pe->can_write_remainder()) {
        pe->set_remainder_out((float *)t->lo_dev);
        t->lo_by = 1;
      }
    } else if (auto *pc = dynamic_cast<Conv2DOp *>(prod)) {
      if (pc->can_write_remainder()) {
        pc->set_remainder_out(t->lo_dev);
        t->lo_by = 1;
      }
    }
    if (t->lo_by == 1) cv->skip_split();
    else t->lo_by = 2; // this convolution's split pass fills it
  }
}

inline void Interpreter::fuse_activation_chains(const std::map<std::string, int> &uses) {
  auto single_use = [&](const std::string &nm) {
    auto it = uses.find(nm);
    return it != uses.end() && it->second == 1;
  };
  const size_t n = kernels.size();
  // INT8 leaky ReLU directly behind a tensor-core convolution that feeds nothing else: the convolution's
  // epilogue applies it and writes both tensors; the leaky op becomes a placeholder.
  for (size_t j = 0; j < n; ++j) {
    auto *lk = dynamic_cast<LeakyReluOp *>(kernels[j].get());
    if (!lk || lk->plain() || lk->in()->dtype != DT_I8) continue;
    for (size_t i = 0; i < j; ++i) {
      auto *cv = dynamic_cast<Conv2DOp *>(kernels[i].get());
      if (!cv || cv->out() != lk->in()) continue;
      const TensorPtr &a = cv->out(), &b = lk->out();
      if (!cv->can_fuse_leaky() || !single_use(cv->name) || a->cp != b->cp || a->padded_rows() || b->padded_rows() ||
          a->bytes() != b->bytes())
        break;
      cv->set_leaky(lk->mp, lk->rp, lk->mn, lk->rn, (int8_t *)b->dev);
      std::unique_ptr<OpKernel> away(new FusedAwayOp());
      away->name = lk->name; away->op_type = lk->op_type; away->shape = lk->shape; away->datatype = lk->datatype;
      away->result = lk->result;
      kernels[j] = std::move(away);
      break;
    }
  }
  // INT8 eltwise add of two tensors, one of them the result of a tensor-core convolution that feeds nothing else and
  // runs after the other operand's producer (the last convolution of a residual block): that convolution's epilogue
  // reads the other operand, forms the sum and writes both tensors; the add op becomes a placeholder
  // (EltwiseAddOpKernel::i8_invoke, core/eltwise.cpp:52-85, on top of Conv2DOpKernel::invoke, core/conv.cpp:80-104).
  for (size_t j = 0; j < n && fuse_residual_add; ++j) {
    auto *ad = dynamic_cast<EltwiseOp *>(kernels[j].get());
    if (!ad || !ad->is_plain_i8_add()) continue;
    const auto &ins = ad->inputs();
    // the producers' positions; the later one must be the convolution
    int pos[2] = {-1, -1};
    for (size_t i = 0; i < j; ++i)
      for (int k = 0; k < 2; ++k)
        if (kernels[i]->result == ins[k]) pos[k] = (int)i;
    if (pos[0] < 0 || pos[1] < 0 || ins[0] == ins[1]) continue;
    const int self = pos[0] > pos[1] ? 0 : 1, other = 1 - self;
    auto *cv = dynamic_cast<Conv2DOp *>(kernels[pos[self]].get());
    if (!cv || !cv->can_fuse_add() || !single_use(cv->name)) continue;
    const TensorPtr &a = cv->out(), &r = ins[other], &o = ad->out();
    if (a->cp != r->cp || a->cp != o->cp || a->bytes() != r->bytes() || a->bytes() != o->bytes() || a->padded_rows() ||
        r->padded_rows() || o->padded_rows() || a->cp % 4 != 0)
      continue;
    const EltwiseArgs &ea = ad->i8_args();
    cv->set_residual_add((const int8_t *)r->dev, (int8_t *)o->dev, ea.mult[self], ea.mult[other], ea.rshift, ea.do_relu);
    std::unique_ptr<OpKernel> away(new FusedAwayOp());
    away->name = ad->name; away->op_type = ad->op_type; away->shape = ad->shape; away->datatype = ad->datatype;
    away->result = ad->result; away->line = ad->line; away->dirty = ad->dirty;
    kernels[j] = std::move(away);
  }
  for (size_t i = 0; i < n; ++i) {
    auto *q0 = dynamic_cast<QuantOp *>(kernels[i].get());
    if (!q0 || q0->kind() != 3 || !single_use(q0->name)) continue;
    size_t j = n, k = n;
    for (size_t t = i + 1; t < n && j == n; ++t) {
      auto *l = dynamic_cast<LutOp *>(kernels[t].get());
      if (l && l->in() == q0->out()) j = t;
    }
    if (j == n) continue;
    auto *lut = static_cast<LutOp *>(kernels[j].get());
    if (!lut->is_bf16_slope() || !single_use(lut->name)) continue;
    for (size_t t = j + 1; t < n && k == n; ++t) {
      auto *q = dynamic_cast<QuantOp *>(kernels[t].get());
      if (q && q->in() == lut->out()) k = t;
    }
    if (k == n) continue;
    auto *q1 = static_cast<QuantOp *>(kernels[k].get());
    if (q1->kind() != 4) continue;
    const TensorPtr &a = q0->in(), &b = q0->out(), &c = lut->out(), &d = q1->out();
    const bool same = a->cp == b->cp && b->cp == c->cp && c->cp == d->cp && a->cp % 16 == 0 && !a->padded_rows() &&
                      !d->padded_rows() && a->pixels() == d->pixels();
    if (!same) continue;
    std::unique_ptr<OpKernel> fused(new ActChainOp(*this, *q0, *lut, *q1));
    auto take_identity = [](OpKernel &dst, const OpKernel &src) {
      dst.name = src.name; dst.op_type = src.op_type; dst.shape = src.shape; dst.datatype = src.datatype;
      dst.result = src.result;
    };
    take_identity(*fused, *q0);
    std::unique_ptr<OpKernel> n1(new FusedAwayOp()), n2(new FusedAwayOp());
    take_identity(*n1, *lut);
    take_identity(*n2, *q1);
    kernels[i] = std::move(fused);
    kernels[j] = std::move(n1);
    kernels[k] = std::move(n2);
  }
}

// loadModule / updateKernelList (MlirModuleInterpreter.cpp:73-83, 118-350).
inline void Interpreter::reset_module() {
  bind();
  invalidate_graph();
  kernels.clear();
  for (auto &kv : tensors)
    if (kv.second->owns && kv.second->dev) cudaFree(kv.second->dev);
  tensors.clear();
  tensor_order.clear();
  input_details.clear();
  output_details.clear();
  producer_type.clear();
  uses.clear();
  layout_requests.clear();
}

// Op types whose kernels treat the leading dimension as independent images, so that batch slots can be laid side by
// side in it. The others (matmul, permute, reduce, pad, crop, broadcast of unequal batch ...) may mix it with other
// dimensions and are refused on an interpreter built with max_batch_size > 1.
inline bool op_is_slot_safe(const std::string &t) {
  static const char *ok[] = {"input", "quant", "conv_2d", "deconv_2d", "fully_connected", "pool_max_2d", "pool_avg_2d",
                             "eltwise_add", "eltwise_mul", "eltwise_max", "eltwise_min", "concat", "upsample", "pixelshuffle",
                             "relu", "leaky_relu", "sigmoid", "mish", "exp", "tanh", "reciprocal", "scale", "batchnorm",
                             "softmax", "reshape"};
  for (const char *o : ok)
    if (t == o) return true;
  return false;
}

inline int Interpreter::add_op(const ParsedOp &op_in) {
  bind();
  invalidate_graph();
  ParsedOp op = op_in;
  if (max_batch > 1) {
    TPUCB_CHECK(op_is_slot_safe(op.type), "%s %s: this op type is not supported on an interpreter with max_batch_size %d",
                op.type.c_str(), op.name.c_str(), max_batch);
    TPUCB_CHECK(!op.shape.empty(), "%s %s: no shape", op.type.c_str(), op.name.c_str());
    op.shape[0] *= max_batch;
  }
  {
    TPUCB_CHECK(!tensors.count(op.name), "module text: duplicate result name '%s'", op.name.c_str());
    const int dt = dtype_from_string(op.dtype);
    auto opd = [&](size_t i) -> TensorPtr {
      TPUCB_CHECK(i < op.in.size(), "%s %s: operand %zu missing", op.type.c_str(), op.name.c_str(), i);
      return tensor(op.in[i]);
    };
    for (auto &nm : op.in)
      if (tensors.count(nm)) uses[nm]++;
    std::unique_ptr<OpKernel> k;
    TensorPtr out;
    for (size_t oi = (op.type == "conv_2d" ? 1 : 0); oi < op.in.size(); ++oi)
      if (tensors.count(op.in[oi]))
        TPUCB_CHECK(!tensors[op.in[oi]]->padded_rows(), "%s %s: operand %s has padded rows", op.type.c_str(),
                    op.name.c_str(), op.in[oi].c_str());
    if (op.type == "reshape") {
      // tpu.reshape is a pure alias of its operand's storage (MlirModuleInterpreter.cpp:331-338);
      // valid on NHWC storage only when the element order is unchanged.
      TensorPtr in = opd(0);
      out = std::make_shared<DevTensor>(*in);
      out->name = op.name;
      out->shape = op.shape;
      out->owns = false;
      int64_t d[4] = {1, 1, 1, 1};
      for (size_t i = 0; i < op.shape.size() && i < 4; ++i) d[i] = op.shape[i];
      TPUCB_CHECK(in->h * in->w == 1 || (d[0] == in->n && d[1] == in->c && d[2] == in->h && d[3] == in->w),
                  "reshape %s: only reshapes of [n,c,1,1] tensors (or identity) are supported", op.name.c_str());
      if (in->h * in->w == 1) {
        TPUCB_CHECK(d[0] == in->n && d[1] * d[2] * d[3] == in->c && (d[2] * d[3] == 1),
                    "reshape %s: unsupported target shape", op.name.c_str());
      }
      out->slot_n = out->n / max_batch;
      tensors[op.name] = out;
      tensor_order.push_back(op.name);
      producer_type[op.name] = "reshape";
      return -1;
    }
    out = make_tensor(op.name, op.shape, dt);
    if (op.type == "input") {
      k.reset(new InputOp());
      input_details.push_back({op.name, out->numel() / (size_t)max_batch});
    } else if (op.type == "quant") {
      std::string pt = producer_type[op.in.at(0)];
      k.reset(new QuantOp(*this, op, opd(0), out, pt == "input"));
    } else if (op.type == "conv_2d") {
      k.reset(new Conv2DOp(*this, op, opd(0), out));
    } else if (op.type == "deconv_2d") {
      // DeConv2DOpKernel (core/deconv.cpp:6-73; MKL-DNN deconvolution on oihw / goihw weights): the scatter
      //   dst[oh = ih*sh + kh*dh - pt] += src[ih] * w[kh]
      // equals a stride-1 convolution of the zero-inserted input (sh-1 zeros between pixels) with the
      // spatially flipped filter and padding dh*(kh-1) - pt, which is what the convolution op runs.
      TPUCB_CHECK(dt == DT_I8 || dt == DT_BF16, "deconv_2d %s: INT8 and BF16 are implemented", op.name.c_str());
      TPUCB_CHECK(op.in.size() >= 2 && has_weight(op.in[1]), "deconv_2d %s: filter operand missing", op.name.c_str());
      const int kh = op.geti("kh", 1), kw = op.geti("kw", 1), sh = op.geti("sh", 1), sw = op.geti("sw", 1);
      const int dh = op.geti("dh", 1), dw = op.geti("dw", 1);
      const HostWeight &filt = weight(op.in[1]);
      TPUCB_CHECK(filt.data.size() % ((size_t)kh * kw) == 0, "deconv_2d %s: filter size does not match kh x kw", op.name.c_str());
      HostWeight flipped = filt;
      for (size_t base = 0; base < filt.data.size(); base += (size_t)kh * kw)
        for (int t = 0; t < kh * kw; ++t) flipped.data[base + t] = filt.data[base + kh * kw - 1 - t];
      ParsedOp cop = op;
      cop.in[1] = op.in[1] + "#flipped";
      weights[cop.in[1]] = flipped;
      auto set = [&](const char *key, int v) { cop.attrs[key] = std::to_string(v); };
      set("ins_h", sh - 1); set("ins_w", sw - 1); set("sh", 1); set("sw", 1);
      set("pt", dh * (kh - 1) - op.geti("pt", 0)); set("pb", dh * (kh - 1) - op.geti("pb", 0));
      set("pl", dw * (kw - 1) - op.geti("pl", 0)); set("pr", dw * (kw - 1) - op.geti("pr", 0));
      TPUCB_CHECK(cop.geti("pt") >= 0 && cop.geti("pl") >= 0, "deconv_2d %s: padding larger than the dilated filter extent",
                  op.name.c_str());
      k.reset(new Conv2DOp(*this, cop, opd(0), out));
    } else if (op.type == "fully_connected") {
      k.reset(new FullyConnectedOp(*this, op, opd(0), out));
    } else if (op.type == "pool_max_2d" || op.type == "pool_avg_2d") {
      k.reset(new PoolOp(*this, op, opd(0), out, op.type == "pool_avg_2d"));
    } else if (op.type == "eltwise_add" || op.type == "eltwise_mul") {
      std::vector<TensorPtr> ins;
      for (auto &nm : op.in)
        if (tensors.count(nm)) ins.push_back(tensors[nm]);
      k.reset(new EltwiseOp(*this, op, ins, out, op.type == "eltwise_mul"));
    } else if (op.type == "eltwise_max" || op.type == "eltwise_min") {
      std::vector<TensorPtr> ins;
      for (auto &nm : op.in)
        if (tensors.count(nm)) ins.push_back(tensors[nm]);
      k.reset(new EltwiseMaxMinOp(*this, op, ins, out, op.type == "eltwise_min"));
    } else if (op.type == "broadcast_add" || op.type == "broadcast_sub" || op.type == "broadcast_mul") {
      k.reset(new BroadcastOp(*this, op, opd(0), opd(1), out));
    } else if (op.type == "pad" || op.type == "crop" || op.type == "permute") {
      k.reset(new RemapOp(*this, op, opd(0), out));
    } else if (op.type == "reduce_mean" || op.type == "reduce_sum" || op.type == "reduce_max" || op.type == "reduce_min" ||
               op.type == "reduce_l2") {
      k.reset(new ReduceOp(*this, op, opd(0), out));
    } else if (op.type == "matmul") {
      k.reset(new MatMulOp(*this, op, opd(0), opd(1), out));
    } else if (op.type == "concat") {
      std::vector<TensorPtr> ins;
      for (auto &nm : op.in)
        if (tensors.count(nm)) ins.push_back(tensors[nm]);
      k.reset(new ConcatOp(*this, op, ins, out));
    } else if (op.type == "upsample") {
      k.reset(new MoveOp(*this, op, opd(0), out, 0));
    } else if (op.type == "pixelshuffle") {
      k.reset(new MoveOp(*this, op, opd(0), out, 1));
    } else if (op.type == "relu" && dt == DT_F32) {
      // fp32 ReLU (core/activation.cpp:168-180): the one-input fp32 eltwise kernel with its ReLU on
      ParsedOp r = op;
      r.attrs["do_relu"] = "1";
      k.reset(new EltwiseOp(*this, r, {opd(0)}, out, false));
    } else if (op.type == "relu" || op.type == "leaky_relu") {
      k.reset(new LeakyReluOp(*this, op, opd(0), out, op.type == "relu"));
    } else if (op.type == "sigmoid" || op.type == "mish" || op.type == "exp" || op.type == "tanh" ||
               op.type == "reciprocal") {
      k.reset(new LutOp(*this, op, opd(0), out));
    } else if (op.type == "scale") {
      k.reset(new ScaleOp(*this, op, opd(0), out));
    } else if (op.type == "batchnorm") {
      k.reset(new BatchNormOp(*this, op, opd(0), out));
    } else if (op.type == "softmax") {
      k.reset(new SoftmaxOp(*this, op, opd(0), out));
    } else {
      cudaFree(out->dev);
      throw Error(strfmt("op type '%s' (%s) is not implemented by the B200 backend", op.type.c_str(), op.name.c_str()));
    }
    k->name = op.name;
    k->op_type = op.type;
    k->shape = op_in.shape; // the module's shape (one batch slot)
    k->datatype = dt;
    k->result = out;
    tensors[op.name] = out;
    tensor_order.push_back(op.name);
    producer_type[op.name] = op.type;
    k->line = op_in.line;
    out->slot_n = out->n / max_batch;
    kernels.push_back(std::move(k));
    return (int)kernels.size() - 1;
  }
}

inline void Interpreter::finish_module() {
  if (fuse_activations) fuse_activation_chains(uses);
  link_tf32_remainders();
  output_details.clear();
  for (auto &k : kernels)
    if (!uses.count(k->name) && k->op_type != "input") output_details.push_back({k->name, k->result->numel() / (size_t)max_batch});
  TPUCB_CUDA(cudaDeviceSynchronize());
}

inline void Interpreter::load_module(const std::string &text) {
  reset_module();
  std::vector<ParsedOp> parsed;
  {
    std::stringstream ss(text);
    std::string line;
    while (std::getline(ss, line)) {
      size_t b = line.find_first_not_of(" \t\r");
      if (b == std::string::npos || line[b] == '#') continue;
      parsed.push_back(parse_line(line.substr(b)));
    }
  }
  // Pre-pass: a few-channel convolution whose input is produced by an input or quant op and has
  // no other consumer asks for that tensor to be stored with zero-padded rows (stem path).
  layout_requests.clear();
  {
    std::map<std::string, const ParsedOp *> by_name;
    std::map<std::string, int> n_uses;
    for (auto &op : parsed) {
      by_name[op.name] = &op;
      for (auto &nm : op.in) n_uses[nm]++;
    }
    for (auto &op : parsed) {
      if (op.type != "conv_2d" || op.dtype != "INT8" || op.in.empty()) continue;
      auto it = by_name.find(op.in[0]);
      if (it == by_name.end() || n_uses[op.in[0]] != 1) continue;
      const ParsedOp &src = *it->second;
      if (!(src.type == "input" || src.type == "quant") || src.dtype != "INT8" || src.shape.size() != 4 ||
          op.shape.size() != 4)
        continue;
      ConvGeom g;
      g.n = (int)src.shape[0]; g.ic = (int)src.shape[1]; g.ih = (int)src.shape[2]; g.iw = (int)src.shape[3];
      g.oc = (int)op.shape[1]; g.oh = (int)op.shape[2]; g.ow = (int)op.shape[3];
      g.g = op.geti("g", 1); g.kh = op.geti("kh", 1); g.kw = op.geti("kw", 1); g.sh = op.geti("sh", 1);
      g.sw = op.geti("sw", 1); g.pt = op.geti("pt", 0); g.pb = op.geti("pb", 0); g.pl = op.geti("pl", 0);
      g.pr = op.geti("pr", 0); g.dh = op.geti("dh", 1); g.dw = op.geti("dw", 1);
      g.ins_h = op.geti("ins_h", 0); g.ins_w = op.geti("ins_w", 0);
      StemLayout st;
      if (stem4_applies(g)) {
        RowLayout rl;
        rl.cp = 4; rl.wl = 0; rl.wphys = g.iw;
        layout_requests[src.name] = rl;
      } else if (stem_layout_for(g, &st)) {
        RowLayout rl;
        rl.cp = st.cp; rl.wl = st.wl; rl.wphys = st.wphys;
        layout_requests[src.name] = rl;
      }
    }
  }
  for (const ParsedOp &op : parsed) add_op(op);
  finish_module();
}

// Geometry and storage of one batch slot of a tensor (slot < 0: the whole tensor).
struct SlotView {
  TensorGeom g;
  void *dev;
  size_t numel;
};
inline SlotView slot_view(const DevTensor &t, int slot, int max_batch, const char *who) {
  SlotView v;
  v.g = TensorGeom{t.n, t.c, t.h, t.w, t.cp, t.wl, t.wphys};
  v.dev = t.dev;
  v.numel = t.numel();
  if (slot >= 0) {
    TPUCB_CHECK(slot < max_batch, "%s %s: batch slot %d is outside [0, %d)", who, t.name.c_str(), slot, max_batch);
    v.g.n = t.slot_n;
    v.numel = (size_t)t.slot_n * t.c * t.h * t.w;
    v.dev = (uint8_t *)t.dev + (size_t)slot * t.slot_n * t.h * t.wphys * t.cp * t.elsize();
  }
  return v;
}

// setTensor (MlirModuleInterpreter.cpp:407-417): fp32 NCHW host values -> device storage.
inline void Interpreter::set_tensor(const std::string &name, const float *data, size_t numel, int slot) {
  bind();
  TensorPtr t = tensor(name);
  reenable_quant_of(t.get());
  const SlotView v = slot_view(*t, slot, max_batch, "set_tensor");
  TPUCB_CHECK(numel == v.numel, "set_tensor %s: got %zu values, tensor has %zu", name.c_str(), numel, v.numel);
  float *stg = ensure_staging(numel * sizeof(float));
  TPUCB_CUDA(cudaMemcpyAsync(stg, data, numel * sizeof(float), cudaMemcpyHostToDevice, stream));
  const TensorGeom &g = v.g;
  const size_t pixels = (size_t)g.n * g.h * g.wphys;
  size_t total = pixels * t->cp;
  int grid = grid_for(total, 256, sm_count);
  if (t->dtype == DT_F32 && t->cp == 4 && !t->padded_rows())
    launch_k(nchw_f32_to_nhwc4_kernel, grid_for(pixels, 256, sm_count), 256, 0, stream, stg, (float4 *)v.dev, g.n, t->c,
                                                                                 (size_t)t->h * t->w);
  else if (t->dtype == DT_I8) launch_k(nchw_f32_to_dev_kernel<DT_I8>, grid, 256, 0, stream, stg, v.dev, g);
  else if (t->dtype == DT_BF16) launch_k(nchw_f32_to_dev_kernel<DT_BF16>, grid, 256, 0, stream, stg, v.dev, g);
  else launch_k(nchw_f32_to_dev_kernel<DT_F32>, grid, 256, 0, stream, stg, v.dev, g);
  TPUCB_CUDA(cudaGetLastError());
}

// Pipelined form of setTensor for serving loops: the host-to-device copy runs on a second stream
// into one of two staging buffers, so it overlaps the module launch that is still executing; the
// (short) layout conversion into the tensor is ordered on the compute stream behind that launch
// and behind the copy. `pinned` must stay valid until the next sync.
inline void Interpreter::set_tensor_async(const std::string &name, const float *pinned, size_t numel) {
  bind();
  TensorPtr t = tensor(name);
  TPUCB_CHECK(numel == t->numel(), "set_tensor_async %s: got %zu values, tensor has %zu", name.c_str(), numel,
              t->numel());
  reenable_quant_of(t.get());
  const int k = async_next;
  async_next ^= 1;
  const size_t bytes = numel * sizeof(float);
  if (bytes > async_staging_bytes[k]) {
    TPUCB_CUDA(cudaStreamSynchronize(stream));
    TPUCB_CUDA(cudaStreamSynchronize(copy_stream));
    if (async_staging[k]) cudaFree(async_staging[k]);
    TPUCB_CUDA(cudaMalloc(&async_staging[k], bytes));
    async_staging_bytes[k] = bytes;
    staging_used[k] = false;
  }
  // the previous conversion out of this staging buffer must have finished
  if (staging_used[k]) TPUCB_CUDA(cudaStreamWaitEvent(copy_stream, staging_free[k], 0));
  TPUCB_CUDA(cudaMemcpyAsync(async_staging[k], pinned, bytes, cudaMemcpyHostToDevice, copy_stream));
  TPUCB_CUDA(cudaEventRecord(upload_done[k], copy_stream));
  TPUCB_CUDA(cudaStreamWaitEvent(stream, upload_done[k], 0));
  TensorGeom g{t->n, t->c, t->h, t->w, t->cp, t->wl, t->wphys};
  size_t total = t->pixels() * t->cp;
  int grid = grid_for(total, 256, sm_count);
  const float *stg = (const float *)async_staging[k];
  if (t->dtype == DT_F32 && t->cp == 4 && !t->padded_rows())
    launch_k(nchw_f32_to_nhwc4_kernel, grid_for(t->pixels(), 256, sm_count), 256, 0, stream, stg, (float4 *)t->dev, t->n, t->c,
                                                                                     (size_t)t->h * t->w);
  else if (t->dtype == DT_I8) launch_k(nchw_f32_to_dev_kernel<DT_I8>, grid, 256, 0, stream, stg, t->dev, g);
  else if (t->dtype == DT_BF16) launch_k(nchw_f32_to_dev_kernel<DT_BF16>, grid, 256, 0, stream, stg, t->dev, g);
  else launch_k(nchw_f32_to_dev_kernel<DT_F32>, grid, 256, 0, stream, stg, t->dev, g);
  TPUCB_CUDA(cudaGetLastError());
  TPUCB_CUDA(cudaEventRecord(staging_free[k], stream));
  staging_used[k] = true;
}

// A quant op that was switched off by set_tensor_async_i8 runs again once its fp32 input is set the ordinary way.
inline void Interpreter::reenable_quant_of(const DevTensor *input) {
  for (auto &k : kernels) {
    auto *q = dynamic_cast<QuantOp *>(k.get());
    if (q && q->disabled && q->in().get() == input) {
      q->disabled = false;
      invalidate_graph();
    }
  }
}

// Pipelined upload of ALREADY QUANTISED input values (int8, NCHW order, PINNED host memory): one byte per value crosses
// the host link instead of the four of the fp32 container. `name` is an INT8 tensor that is either a module input or
// the result of the tpu.quant (NONE -> INT8) op directly behind an fp32 input; in the second case that quant op is
// switched off (its result now comes from the caller) until the fp32 input is set again with set_tensor /
// set_tensor_async. The caller quantises as the op would: sat8(round-half-away-from-zero(x * scale)) (core/quant.cpp:22-30).
inline void Interpreter::set_tensor_async_i8(const std::string &name, const int8_t *pinned, size_t numel) {
  bind();
  TensorPtr t = tensor(name);
  TPUCB_CHECK(t->dtype == DT_I8, "set_tensor_async_i8 %s: the tensor is not INT8", name.c_str());
  TPUCB_CHECK(numel == t->numel(), "set_tensor_async_i8 %s: got %zu values, tensor has %zu", name.c_str(), numel, t->numel());
  OpKernel *prod = nullptr;
  for (auto &k : kernels)
    if (k->result == t) prod = k.get();
  TPUCB_CHECK(prod != nullptr, "set_tensor_async_i8 %s: no op produces this tensor", name.c_str());
  if (prod->op_type != "input") {
    auto *q = dynamic_cast<QuantOp *>(prod);
    bool ok = q && (q->kind() == 0 || q->kind() == 1);
    if (ok) {
      ok = false;
      for (auto &k : kernels)
        if (k->result == q->in() && k->op_type == "input") ok = true;
    }
    TPUCB_CHECK(ok, "set_tensor_async_i8 %s: only a module input or the quant op directly behind one can be supplied", name.c_str());
    if (!q->disabled) {
      q->disabled = true;
      invalidate_graph();
    }
  }
  const int k = async_next;
  async_next ^= 1;
  if (numel > async_staging_bytes[k]) {
    TPUCB_CUDA(cudaStreamSynchronize(stream));
    TPUCB_CUDA(cudaStreamSynchronize(copy_stream));
    if (async_staging[k]) cudaFree(async_staging[k]);
    TPUCB_CUDA(cudaMalloc(&async_staging[k], numel));
    async_staging_bytes[k] = numel;
    staging_used[k] = false;
  }
  if (staging_used[k]) TPUCB_CUDA(cudaStreamWaitEvent(copy_stream, staging_free[k], 0));
  TPUCB_CUDA(cudaMemcpyAsync(async_staging[k], pinned, numel, cudaMemcpyHostToDevice, copy_stream));
  TPUCB_CUDA(cudaEventRecord(upload_done[k], copy_stream));
  TPUCB_CUDA(cudaStreamWaitEvent(stream, upload_done[k], 0));
  TensorGeom g{t->n, t->c, t->h, t->w, t->cp, t->wl, t->wphys};
  const int8_t *stg = (const int8_t *)async_staging[k];
  if (t->cp == 4 && !t->padded_rows())
    launch_k(nchw_i8_to_nhwc4_kernel, grid_for(t->pixels(), 256, sm_count), 256, 0, stream, stg, (uint32_t *)t->dev, t->n, t->c,
             (size_t)t->h * t->w);
  else
    launch_k(nchw_i8_to_dev_kernel, grid_for(t->pixels() * t->cp, 256, sm_count), 256, 0, stream, stg, (int8_t *)t->dev, g);
  TPUCB_CUDA(cudaEventRecord(staging_free[k], stream));
  staging_used[k] = true;
}

// getTensor (MlirModuleInterpreter.cpp:419-427): deep copy out as fp32 NCHW.
inline void Interpreter::get_tensor(const std::string &name, float *out, size_t numel, int slot) {
  bind();
  TensorPtr t = tensor(name);
  const SlotView v = slot_view(*t, slot, max_batch, "get_tensor");
  TPUCB_CHECK(numel == v.numel, "get_tensor %s: buffer has %zu values, tensor has %zu", name.c_str(), numel, v.numel);
  float *stg = ensure_staging(numel * sizeof(float));
  int grid = grid_for(numel, 256, sm_count);
  if (t->dtype == DT_I8) launch_k(dev_to_nchw_f32_kernel<DT_I8>, grid, 256, 0, stream, v.dev, stg, v.g);
  else if (t->dtype == DT_BF16) launch_k(dev_to_nchw_f32_kernel<DT_BF16>, grid, 256, 0, stream, v.dev, stg, v.g);
  else launch_k(dev_to_nchw_f32_kernel<DT_F32>, grid, 256, 0, stream, v.dev, stg, v.g);
  TPUCB_CUDA(cudaGetLastError());
  TPUCB_CUDA(cudaMemcpyAsync(out, stg, numel * sizeof(float), cudaMemcpyDeviceToHost, stream));
  TPUCB_CUDA(cudaStreamSynchronize(stream));
}

// The op list captured as one CUDA graph, with the launch flag of the moment.
inline cudaGraphExec_t Interpreter::capture_graph() {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  TPUCB_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
  try {
    for (auto &k : kernels) k->run(stream);
  } catch (...) {
    cudaStreamEndCapture(stream, &graph);
    if (graph) cudaGraphDestroy(graph);
    throw;
  }
  TPUCB_CUDA(cudaStreamEndCapture(stream, &graph));
  cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  TPUCB_CUDA(e);
  return exec;
}

// invoke (MlirModuleInterpreter.cpp:371-381): the op loop; replayed as one CUDA graph.
inline void Interpreter::launch_all() {
  bind();
  if (use_graph) {
    if (!graph_exec) graph_exec = capture_graph();
    TPUCB_CUDA(cudaGraphLaunch(graph_exec, stream));
  } else {
    for (auto &k : kernels) k->run(stream);
    TPUCB_CUDA(cudaGetLastError());
  }
}

inline void Interpreter::launch_to(const std::string &name) {
  bind();
  if (name.empty()) return launch_all();
  tensor(name);
  for (auto &k : kernels) {
    k->run(stream);
    if (k->name == name) break;
  }
  TPUCB_CUDA(cudaGetLastError());
}

// fastInvokeAllBatch (MlirModuleInterpreter.cpp:383-405): the reference loops over the batch slots and runs, per slot,
// every kernel that is still dirty (built since the last such call) up to `name`. Here the slots are image groups of
// one device tensor: the same kernels run ONCE, over all slots, and are marked clean.
inline void Interpreter::fast_invoke_all_batch(const std::string &name, int batch) {
  bind();
  TPUCB_CHECK(batch >= 1 && batch <= max_batch, "fastInvokeAllBatch: batch %d is outside [1, %d]", batch, max_batch);
  if (!name.empty()) tensor(name);
  for (auto &k : kernels) {
    if (k->dirty) {
      k->run(stream);
      k->dirty = false;
    }
    if (!name.empty() && k->name == name) break;
  }
  TPUCB_CUDA(cudaGetLastError());
}

inline void Interpreter::sync_and_check() {
  bind();
  TPUCB_CUDA(cudaStreamSynchronize(stream));
  int err = 0;
  TPUCB_CUDA(cudaMemcpy(&err, d_err, sizeof(int), cudaMemcpyDeviceToHost));
  if (err != 0) {
    TPUCB_CUDA(cudaMemset(d_err, 0, sizeof(int)));
    for (auto &w : split_ws) TPUCB_CUDA(cudaMemset(w.first, 0, w.second)); // a failed launch may leave partial sums
    throw Error(strfmt("a convolution kernel gave up on a bounded wait (code %d: 1 = tile load never arrived, "
                       "2 = stage never freed, 3 = accumulator never completed or never handed back); the launch's "
                       "results are incomplete, the interpreter stays usable", err));
  }
}

} // namespace tpucb
