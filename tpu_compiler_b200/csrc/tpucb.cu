// C ABI of libtpucb.so: a thin extern "C" layer over tpucb::Interpreter. See include/tpucb.h
// for the reference interface each entry point stands in for.
#include "../../include/tpucb.h"
#include "interpreter.cuh"
#include "mma_peak.cuh"

#include <algorithm>
#include <cmath>
#include <mutex>
#include <string>

using namespace tpucb;

struct tpucb_op {
  tpucb_interp *ctx;
  int index;        // position in the context's kernel list; -1 for a reshape (an alias: nothing to run)
  std::string name; // result name
  bool stale = false; // its interpreter has loaded another module since
};

struct tpucb_interp {
  Interpreter impl;
  std::vector<std::unique_ptr<tpucb_op>> ops; // handles given out by tpucb_op_create
  double *tuner_sums = nullptr; // device scratch of tpucb_tuner_distance, grown on demand
  int tuner_sums_cap = 0;
  StatDesc *stat_descs = nullptr; // device descriptor list of the all-tensor statistics launches, grown on demand
  int stat_descs_cap = 0;
  explicit tpucb_interp(int device) : impl(device) {}
  ~tpucb_interp() {
    if (tuner_sums) cudaFree(tuner_sums);
    if (stat_descs) cudaFree(stat_descs);
  }
};

static thread_local std::string g_last_error;

#define TPUCB_API_BEGIN try {
#define TPUCB_API_END                                  \
  }                                                    \
  catch (const std::exception &e) {                    \
    g_last_error = e.what();                           \
    return 1;                                          \
  }                                                    \
  catch (...) {                                        \
    g_last_error = "unknown error";                    \
    return 1;                                          \
  }                                                    \
  return 0;

static int copy_out(const std::string &s, char *out, size_t cap, size_t *needed) {
  if (needed) *needed = s.size() + 1;
  if (out && cap > 0) {
    size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
    memcpy(out, s.data(), n);
    out[n] = 0;
  }
  return 0;
}

extern "C" {

const char *tpucb_last_error(void) { return g_last_error.c_str(); }
int tpucb_version(void) { return 1; }

int tpucb_interp_create(int device, tpucb_interp **out) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(out != nullptr, "tpucb_interp_create: out is NULL");
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  TPUCB_CHECK(e == cudaSuccess && count > 0,
              "no CUDA device is available (%s); this backend has no CPU fallback",
              e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  TPUCB_CHECK(device >= 0 && device < count, "device %d out of range (have %d)", device, count);
  *out = new tpucb_interp(device);
  TPUCB_API_END
}

int tpucb_interp_create_batched(int device, int max_batch_size, tpucb_interp **out) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(max_batch_size >= 1 && max_batch_size <= 65536, "tpucb_interp_create_batched: max_batch_size %d is outside [1, 65536]",
              max_batch_size);
  if (tpucb_interp_create(device, out) != 0) return 1;
  (*out)->impl.max_batch = max_batch_size;
  TPUCB_API_END
}

int tpucb_interp_destroy(tpucb_interp *it) {
  TPUCB_API_BEGIN
  delete it;
  TPUCB_API_END
}

int tpucb_interp_set_weight(tpucb_interp *it, const char *name, const float *data, const int64_t *shape, int rank) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && name && data && rank >= 0, "tpucb_interp_set_weight: bad argument");
  HostWeight w;
  size_t n = 1;
  for (int i = 0; i < rank; ++i) {
    w.shape.push_back(shape[i]);
    n *= (size_t)shape[i];
  }
  w.data.assign(data, data + n);
  it->impl.weights[name] = std::move(w);
  TPUCB_API_END
}

int tpucb_interp_load_module(tpucb_interp *it, const char *module_text) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && module_text, "tpucb_interp_load_module: bad argument");
  for (auto &o : it->ops) o->stale = true; // handles into the previous module stay allocated, but refuse to run
  it->impl.load_module(module_text);
  TPUCB_API_END
}

int tpucb_interp_set_tensor(tpucb_interp *it, const char *name, const float *data, size_t numel) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && name && data, "tpucb_interp_set_tensor: bad argument");
  it->impl.set_tensor(name, data, numel);
  TPUCB_API_END
}

int tpucb_interp_set_tensor_slot(tpucb_interp *it, const char *name, const float *data, size_t numel, int bidx) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && name && data && bidx >= 0, "tpucb_interp_set_tensor_slot: bad argument");
  it->impl.set_tensor(name, data, numel, bidx);
  TPUCB_API_END
}

int tpucb_interp_get_tensor_slot(tpucb_interp *it, const char *name, float *out, size_t numel, int bidx) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && name && out && bidx >= 0, "tpucb_interp_get_tensor_slot: bad argument");
  it->impl.get_tensor(name, out, numel, bidx);
  TPUCB_API_END
}

int tpucb_interp_invoke_slot(tpucb_interp *it, const char *name, int bidx) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it, "tpucb_interp_invoke_slot: bad argument");
  TPUCB_CHECK(bidx >= 0 && bidx < it->impl.max_batch, "tpucb_interp_invoke_slot: batch slot %d is outside [0, %d)", bidx,
              it->impl.max_batch);
  it->impl.launch_to(name ? name : "");
  it->impl.sync_and_check();
  TPUCB_API_END
}

int tpucb_interp_fast_invoke_all_batch(tpucb_interp *it, const char *name, int batch) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it, "tpucb_interp_fast_invoke_all_batch: bad argument");
  it->impl.fast_invoke_all_batch(name ? name : "", batch);
  it->impl.sync_and_check();
  TPUCB_API_END
}

int tpucb_interp_max_batch_size(tpucb_interp *it, int *max_batch_size) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && max_batch_size, "tpucb_interp_max_batch_size: bad argument");
  *max_batch_size = it->impl.max_batch;
  TPUCB_API_END
}

int tpucb_interp_dump(tpucb_interp *it, const char *name, char *out, size_t cap, size_t *needed) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && name, "tpucb_interp_dump: bad argument");
  std::string s;
  for (auto &k : it->impl.kernels)
    if (k->name == name) {
      s = "name: " + k->name + "\nop_type: " + k->op_type + "\ndata_type: " + dtype_to_string(k->datatype) + "\nshape: ";
      for (size_t i = 0; i < k->shape.size(); ++i) s += (i ? "x" : "") + std::to_string(k->shape[i]);
      s += "\nmax_batch_size: " + std::to_string(it->impl.max_batch) + "\ndirty: " + (k->dirty ? "1" : "0") +
           "\nkernel_launches: " + std::to_string(k->kernel_launches()) + "\nop: " + k->line + "\n";
    }
  TPUCB_CHECK(!s.empty(), "tpucb_interp_dump: no op named '%s'", name);
  copy_out(s, out, cap, needed);
  TPUCB_API_END
}

// ---- per-op surface (CPUOpKernel, include/tpuc/Interpreter/cpukernel.h:87-159) -------------------------------------

int tpucb_op_create(tpucb_interp *ctx, const char *op_line, tpucb_op **out) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(ctx && op_line && out, "tpucb_op_create: bad argument");
  std::string line = op_line;
  size_t b = line.find_first_not_of(" \t\r\n");
  TPUCB_CHECK(b != std::string::npos, "tpucb_op_create: empty op line");
  size_t e = line.find_last_not_of(" \t\r\n");
  ParsedOp op = parse_line(line.substr(b, e - b + 1));
  const int index = ctx->impl.add_op(op);
  // the result of an op without consumers is an output until a later op reads it
  ctx->impl.output_details.clear();
  for (auto &k : ctx->impl.kernels)
    if (!ctx->impl.uses.count(k->name) && k->op_type != "input")
      ctx->impl.output_details.push_back({k->name, k->result->numel() / (size_t)ctx->impl.max_batch});
  ctx->ops.emplace_back(new tpucb_op{ctx, index, op.name, false});
  *out = ctx->ops.back().get();
  TPUCB_API_END
}

static OpKernel *op_kernel(tpucb_op *op, const char *who) {
  TPUCB_CHECK(op && op->ctx, "%s: bad argument", who);
  auto &ks = op->ctx->impl.kernels;
  TPUCB_CHECK(!op->stale && (op->index < 0 || (op->index < (int)ks.size() && ks[op->index]->name == op->name)),
              "%s: the op handle of '%s' is stale (its interpreter loaded another module)", who, op->name.c_str());
  if (op->index < 0) return nullptr;
  return ks[op->index].get();
}

int tpucb_op_invoke(tpucb_op *op) {
  TPUCB_API_BEGIN
  OpKernel *k = op_kernel(op, "tpucb_op_invoke");
  Interpreter &I = op->ctx->impl;
  I.bind();
  if (k) {
    k->run(I.stream);
    k->dirty = false;
    TPUCB_CUDA(cudaGetLastError());
  }
  I.sync_and_check();
  TPUCB_API_END
}

int tpucb_op_set_tensor(tpucb_op *op, const float *data, size_t numel, int bidx) {
  TPUCB_API_BEGIN
  OpKernel *k = op_kernel(op, "tpucb_op_set_tensor");
  TPUCB_CHECK(data, "tpucb_op_set_tensor: bad argument");
  // CPUOpKernel::set_tensor is implemented by the input op only (core/input.cpp:17-24); the others reject it
  TPUCB_CHECK(k && k->op_type == "input", "tpucb_op_set_tensor: op '%s' is not an input op", op->name.c_str());
  op->ctx->impl.set_tensor(op->name, data, numel, bidx);
  TPUCB_API_END
}

int tpucb_op_get_tensor(tpucb_op *op, float *out, size_t numel, int bidx) {
  TPUCB_API_BEGIN
  op_kernel(op, "tpucb_op_get_tensor");
  TPUCB_CHECK(out, "tpucb_op_get_tensor: bad argument");
  op->ctx->impl.get_tensor(op->name, out, numel, bidx);
  TPUCB_API_END
}

int tpucb_op_info(tpucb_op *op, char *out, size_t cap, size_t *needed) {
  TPUCB_API_BEGIN
  OpKernel *k = op_kernel(op, "tpucb_op_info");
  auto t = op->ctx->impl.tensor(op->name);
  std::string s = op->name + "\t" + (k ? k->op_type : std::string("reshape")) + "\t" + dtype_to_string(t->dtype) + "\t";
  for (size_t i = 0; i < t->shape.size(); ++i)
    s += (i ? "," : "") + std::to_string(i == 0 ? t->shape[i] / op->ctx->impl.max_batch : t->shape[i]);
  s += std::string("\t") + ((k && k->dirty) ? "1" : "0");
  copy_out(s, out, cap, needed);
  TPUCB_API_END
}

int tpucb_interp_set_tensor_async(tpucb_interp *it, const char *name, const float *pinned, size_t numel) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && name && pinned, "tpucb_interp_set_tensor_async: bad argument");
  it->impl.set_tensor_async(name, pinned, numel);
  TPUCB_API_END
}

int tpucb_interp_set_tensor_async_i8(tpucb_interp *it, const char *name, const int8_t *pinned, size_t numel) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && name && pinned, "tpucb_interp_set_tensor_async_i8: bad argument");
  it->impl.set_tensor_async_i8(name, pinned, numel);
  TPUCB_API_END
}

int tpucb_interp_wait_uploads(tpucb_interp *it) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it, "tpucb_interp_wait_uploads: bad argument");
  it->impl.bind();
  TPUCB_CUDA(cudaStreamSynchronize(it->impl.copy_stream));
  TPUCB_API_END
}

int tpucb_interp_invoke(tpucb_interp *it) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it, "tpucb_interp_invoke: bad argument");
  it->impl.launch_all();
  it->impl.sync_and_check();
  TPUCB_API_END
}

int tpucb_interp_invoke_to(tpucb_interp *it, const char *name) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it, "tpucb_interp_invoke_to: bad argument");
  it->impl.launch_to(name ? name : "");
  it->impl.sync_and_check();
  TPUCB_API_END
}

int tpucb_interp_launch(tpucb_interp *it) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it, "tpucb_interp_launch: bad argument");
  it->impl.launch_all();
  TPUCB_API_END
}

int tpucb_interp_sync(tpucb_interp *it) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it, "tpucb_interp_sync: bad argument");
  it->impl.sync_and_check();
  TPUCB_API_END
}

int tpucb_interp_get_tensor(tpucb_interp *it, const char *name, float *out, size_t numel) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && name && out, "tpucb_interp_get_tensor: bad argument");
  it->impl.get_tensor(name, out, numel);
  TPUCB_API_END
}

int tpucb_interp_get_tensor_shape(tpucb_interp *it, const char *name, int64_t *shape, int *rank) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && name && shape && rank, "tpucb_interp_get_tensor_shape: bad argument");
  auto t = it->impl.tensor(name);
  *rank = (int)t->shape.size();
  // the module's shape: one batch slot (MlirModuleInterpreter::getTensorShape)
  for (size_t i = 0; i < t->shape.size(); ++i) shape[i] = i == 0 ? t->shape[i] / it->impl.max_batch : t->shape[i];
  TPUCB_API_END
}

int tpucb_interp_get_data_type(tpucb_interp *it, const char *name, char *out, size_t cap) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && name && out, "tpucb_interp_get_data_type: bad argument");
  copy_out(dtype_to_string(it->impl.tensor(name)->dtype), out, cap, nullptr);
  TPUCB_API_END
}

int tpucb_interp_get_all_tensor_names(tpucb_interp *it, char *out, size_t cap, size_t *needed) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it, "tpucb_interp_get_all_tensor_names: bad argument");
  std::string s;
  for (auto &n : it->impl.tensor_order) s += n + "\n";
  copy_out(s, out, cap, needed);
  TPUCB_API_END
}

int tpucb_interp_get_details(tpucb_interp *it, int outputs, char *out, size_t cap, size_t *needed) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it, "tpucb_interp_get_details: bad argument");
  std::string s;
  for (auto &d : outputs ? it->impl.output_details : it->impl.input_details)
    s += d.first + ":" + std::to_string(d.second) + "\n";
  copy_out(s, out, cap, needed);
  TPUCB_API_END
}

int tpucb_interp_get_op_info(tpucb_interp *it, char *out, size_t cap, size_t *needed) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it, "tpucb_interp_get_op_info: bad argument");
  std::string s;
  for (auto &k : it->impl.kernels) {
    s += k->name + "\t" + k->op_type + "\t" + dtype_to_string(k->datatype) + "\t";
    for (size_t i = 0; i < k->shape.size(); ++i) s += (i ? "," : "") + std::to_string(k->shape[i]);
    s += "\t" + std::to_string(k->alg_ops) + "\t" + std::to_string(k->alg_bytes);
    auto *cv = dynamic_cast<Conv2DOp *>(k.get());
    auto *fc = dynamic_cast<FullyConnectedOp *>(k.get());
    s += std::string("\t") + ((cv && cv->is_tensor_core()) || (fc && !fc->is_batched()) ? "tensor" : "hbm") + "\n";
  }
  copy_out(s, out, cap, needed);
  TPUCB_API_END
}

int tpucb_interp_set_option(tpucb_interp *it, const char *key, int value) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && key, "tpucb_interp_set_option: bad argument");
  std::string k = key;
  if (k == "cuda_graph") {
    it->impl.use_graph = value != 0;
    it->impl.invalidate_graph();
  } else if (k == "pdl") {
    TPUCB_CHECK(value >= -1 && value <= 2, "pdl: 0 (off), 1 (convolution kernels, the default) or 2 (every kernel)");
    it->impl.use_pdl = value < 0 ? 1 : value;
    it->impl.invalidate_graph();
  } else if (k == "selftest_lost_arrival") {
    TPUCB_CHECK(value >= 0 && value <= 1024, "selftest_lost_arrival: rounds must be in [0, 1024]");
    it->impl.selftest_lost_arrival = value; // takes effect at the next load_module
  } else if (k == "split_k") {
    it->impl.split_k = value != 0; // takes effect at the next load_module
  } else if (k == "fuse_activations") {
    it->impl.fuse_activations = value != 0; // takes effect at the next load_module
  } else if (k == "fuse_residual_add") {
    it->impl.fuse_residual_add = value != 0; // takes effect at the next load_module
  } else if (k == "fp32_tensor_cores") {
    it->impl.fp32_tensor_cores = value != 0; // takes effect at the next load_module
  } else {
    throw Error("unknown option '" + k + "'");
  }
  TPUCB_API_END
}

int tpucb_interp_profile(tpucb_interp *it, float *ms, int cap, int *count) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && ms && count, "tpucb_interp_profile: bad argument");
  Interpreter &I = it->impl;
  I.bind();
  const int n = (int)I.kernels.size();
  *count = n;
  TPUCB_CHECK(cap >= n, "tpucb_interp_profile: buffer holds %d entries, need %d", cap, n);
  std::vector<cudaEvent_t> ev(n + 1);
  for (auto &e : ev) TPUCB_CUDA(cudaEventCreate(&e));
  TPUCB_CUDA(cudaEventRecord(ev[0], I.stream));
  for (int i = 0; i < n; ++i) {
    I.kernels[i]->run(I.stream);
    TPUCB_CUDA(cudaEventRecord(ev[i + 1], I.stream));
  }
  I.sync_and_check();
  for (int i = 0; i < n; ++i) TPUCB_CUDA(cudaEventElapsedTime(&ms[i], ev[i], ev[i + 1]));
  for (auto &e : ev) cudaEventDestroy(e);
  TPUCB_API_END
}

int tpucb_interp_time_launches(tpucb_interp *it, int iters, float *ms_total) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && ms_total && iters > 0, "tpucb_interp_time_launches: bad argument");
  Interpreter &I = it->impl;
  I.bind();
  cudaEvent_t a, b;
  TPUCB_CUDA(cudaEventCreate(&a));
  TPUCB_CUDA(cudaEventCreate(&b));
  TPUCB_CUDA(cudaStreamSynchronize(I.stream));
  TPUCB_CUDA(cudaEventRecord(a, I.stream));
  for (int i = 0; i < iters; ++i) I.launch_all();
  TPUCB_CUDA(cudaEventRecord(b, I.stream));
  I.sync_and_check();
  TPUCB_CUDA(cudaEventElapsedTime(ms_total, a, b));
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  TPUCB_API_END
}

int tpucb_interp_kernel_count(tpucb_interp *it, int *count) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && count, "tpucb_interp_kernel_count: bad argument");
  int c = 0;
  for (auto &k : it->impl.kernels) c += k->disabled ? 0 : k->kernel_launches();
  *count = c;
  TPUCB_API_END
}

int tpucb_interp_tensor_device(tpucb_interp *it, const char *name, void **dev, size_t *bytes, int *channels,
                               int *channel_pitch, int *dtype) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && name, "tpucb_interp_tensor_device: bad argument");
  auto t = it->impl.tensor(name);
  if (dev) *dev = t->dev;
  if (bytes) *bytes = t->bytes();
  if (channels) *channels = t->c;
  if (channel_pitch) *channel_pitch = t->cp;
  if (dtype) *dtype = t->dtype;
  TPUCB_API_END
}

int tpucb_interp_copy_tensor(tpucb_interp *dst, const char *dst_name, tpucb_interp *src, const char *src_name) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(dst && src && dst_name && src_name, "tpucb_interp_copy_tensor: bad argument");
  Interpreter &D = dst->impl, &S = src->impl;
  TPUCB_CHECK(D.device() == S.device(), "tpucb_interp_copy_tensor: the two interpreters live on different devices");
  auto d = D.tensor(dst_name);
  auto s = S.tensor(src_name);
  TPUCB_CHECK(d->dtype == s->dtype && d->n == s->n && d->c == s->c && d->h == s->h && d->w == s->w && d->cp == s->cp &&
                  d->wl == s->wl && d->wphys == s->wphys,
              "tpucb_interp_copy_tensor: %s and %s differ in type, shape or device layout", dst_name, src_name);
  D.bind();
  TPUCB_CUDA(cudaStreamSynchronize(S.stream)); // the source's producers have finished
  TPUCB_CUDA(cudaMemcpyAsync(d->dev, s->dev, s->bytes(), cudaMemcpyDeviceToDevice, D.stream));
  TPUCB_CUDA(cudaStreamSynchronize(D.stream)); // the source may be overwritten once this returns
  TPUCB_API_END
}

int tpucb_tuner_distance(tpucb_interp *ref, const char *ref_name, tpucb_interp *tgt, const char *tgt_name, float scale,
                         double *sums, int images) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(ref && tgt && ref_name && tgt_name && sums, "tpucb_tuner_distance: bad argument");
  Interpreter &R = ref->impl, &T = tgt->impl;
  TPUCB_CHECK(R.device() == T.device(), "tpucb_tuner_distance: the two interpreters live on different devices");
  auto r = R.tensor(ref_name);
  auto t = T.tensor(tgt_name);
  TPUCB_CHECK(r->dtype == DT_F32, "tpucb_tuner_distance: reference tensor %s is not fp32", ref_name);
  TPUCB_CHECK(r->n == t->n && r->c == t->c && r->h == t->h && r->w == t->w,
              "tpucb_tuner_distance: %s and %s differ in shape", ref_name, tgt_name);
  TPUCB_CHECK(images == r->n, "tpucb_tuner_distance: %d images asked, the tensors hold %d", images, r->n);
  TPUCB_CHECK(r->cp % 4 == 0 && t->cp % 4 == 0, "tpucb_tuner_distance: channel pitch is not a multiple of 4");
  T.bind();
  if (tgt->tuner_sums_cap < images) {
    if (tgt->tuner_sums) TPUCB_CUDA(cudaFree(tgt->tuner_sums));
    tgt->tuner_sums = nullptr;
    tgt->tuner_sums_cap = 0;
    TPUCB_CUDA(cudaMalloc(&tgt->tuner_sums, sizeof(double) * 2 * images));
    tgt->tuner_sums_cap = images;
  }
  TPUCB_CUDA(cudaStreamSynchronize(R.stream)); // the reference activations are complete
  TPUCB_CUDA(cudaMemsetAsync(tgt->tuner_sums, 0, sizeof(double) * 2 * images, T.stream));
  DistGeom rg{r->dev, r->cp, r->wl, r->wphys}, tg{t->dev, t->cp, t->wl, t->wphys};
  const size_t quads = (size_t)r->h * r->w * ((r->c + 3) / 4);
  int bx = (int)((quads + 1023) / 1024); // four steps per thread at least, when there is that much work
  const int per_image_cap = (T.sm_count * 8 + images - 1) / images;
  if (bx > per_image_cap) bx = per_image_cap;
  if (bx < 1) bx = 1;
  dim3 grid(bx, images);
  if (t->dtype == DT_I8)
    tuner_distance_kernel<0><<<grid, 256, 0, T.stream>>>(rg, tg, r->c, r->h, r->w, scale, tgt->tuner_sums);
  else if (t->dtype == DT_BF16)
    tuner_distance_kernel<1><<<grid, 256, 0, T.stream>>>(rg, tg, r->c, r->h, r->w, scale, tgt->tuner_sums);
  else
    tuner_distance_kernel<2><<<grid, 256, 0, T.stream>>>(rg, tg, r->c, r->h, r->w, scale, tgt->tuner_sums);
  TPUCB_CUDA(cudaGetLastError());
  TPUCB_CUDA(cudaMemcpyAsync(sums, tgt->tuner_sums, sizeof(double) * 2 * images, cudaMemcpyDeviceToHost, T.stream));
  TPUCB_CUDA(cudaStreamSynchronize(T.stream));
  TPUCB_API_END
}

int tpucb_host_alloc(void **ptr, size_t bytes) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(ptr, "tpucb_host_alloc: bad argument");
  TPUCB_CUDA(cudaHostAlloc(ptr, bytes, cudaHostAllocDefault));
  TPUCB_API_END
}

int tpucb_host_alloc_write_combined(void **ptr, size_t bytes) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(ptr, "tpucb_host_alloc_write_combined: bad argument");
  TPUCB_CUDA(cudaHostAlloc(ptr, bytes, cudaHostAllocWriteCombined));
  TPUCB_API_END
}

int tpucb_host_free(void *ptr) {
  TPUCB_API_BEGIN
  TPUCB_CUDA(cudaFreeHost(ptr));
  TPUCB_API_END
}

int tpucb_measure_i8_mma_peak(int device, int n_cols, double *tops) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(tops && (n_cols == 64 || n_cols == 128 || n_cols == 256), "tpucb_measure_i8_mma_peak: n_cols must be 64, 128 or 256");
  TPUCB_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  TPUCB_CUDA(cudaGetDeviceProperties(&prop, device));
  TPUCB_CHECK(prop.major == 10, "tpucb_measure_i8_mma_peak: needs an sm_100 device");
  int *d_err = nullptr;
  TPUCB_CUDA(cudaMalloc(&d_err, sizeof(int)));
  TPUCB_CUDA(cudaMemset(d_err, 0, sizeof(int)));
  const size_t smem = 2048 + (size_t)(128 + n_cols) * 128;
  TPUCB_CUDA(cudaFuncSetAttribute(mma_i8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const uint32_t idesc = make_idesc_i8(128, n_cols);
  const int iters = 8192, grid = prop.multiProcessorCount;
  cudaEvent_t a, b;
  TPUCB_CUDA(cudaEventCreate(&a));
  TPUCB_CUDA(cudaEventCreate(&b));
  float best = 1e30f;
  for (int rep = 0; rep < 4; ++rep) {
    TPUCB_CUDA(cudaEventRecord(a, 0));
    mma_i8_peak_kernel<<<grid, 64, smem, 0>>>(iters, n_cols, idesc, d_err);
    TPUCB_CUDA(cudaEventRecord(b, 0));
    TPUCB_CUDA(cudaEventSynchronize(b));
    float ms = 0;
    TPUCB_CUDA(cudaEventElapsedTime(&ms, a, b));
    if (rep > 0 && ms < best) best = ms;
  }
  int err = 0;
  TPUCB_CUDA(cudaMemcpy(&err, d_err, sizeof(int), cudaMemcpyDeviceToHost));
  cudaFree(d_err);
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  TPUCB_CHECK(err == 0, "tpucb_measure_i8_mma_peak: the MMA chain did not complete within the wait limit");
  const double ops = 2.0 * 128.0 * n_cols * 32.0 * 4.0 * iters * grid;
  *tops = ops / (best * 1e-3) / 1e12;
  TPUCB_API_END
}

// ---------------------------------------------------------------- calibration statistics

// dynamic shared memory of kld_kernel at the largest supported bin count (4096): two float arrays and one double array
static constexpr int kKldMaxSmem = 4096 * (2 * (int)sizeof(float) + (int)sizeof(double));

static void calib_minmax_impl(tpucb_interp *it, const char *name, float *d_stats, float *d_keep, const char *who) {
  TPUCB_CHECK(it && name && d_stats, "%s: bad argument", who);
  Interpreter &I = it->impl;
  I.bind();
  auto t = I.tensor(name);
  TPUCB_CHECK(t->dtype == DT_F32, "%s: tensor %s is not fp32", who, name);
  TPUCB_CHECK(((uintptr_t)d_keep & 15) == 0, "%s: the copy must be 16-byte aligned", who);
  size_t total = t->pixels() * t->cp;
  minmax_f32_kernel<<<grid_for(total / 4 + 1, 256, I.sm_count), 256, 0, I.stream>>>((const float *)t->dev, t->pixels(),
                                                                                    t->c, t->cp, d_stats, d_keep);
  TPUCB_CUDA(cudaGetLastError());
}

static void calib_hist_impl(tpucb_interp *it, const char *name, const float *d_values, float abs_max, int bins,
                            int64_t *d_hist, const char *who) {
  TPUCB_CHECK(it && name && d_hist, "%s: bad argument", who);
  TPUCB_CHECK(bins >= 128 && bins <= 4096, "%s: bins must be in [128, 4096]", who);
  Interpreter &I = it->impl;
  I.bind();
  auto t = I.tensor(name);
  TPUCB_CHECK(t->dtype == DT_F32, "%s: tensor %s is not fp32", who, name);
  TPUCB_CHECK(((uintptr_t)d_values & 15) == 0, "%s: the values must be 16-byte aligned", who);
  // width = abs_max / (bin_num - 1), in fp32 as numpy computes it (kld_calibrator.py:34)
  float width = abs_max / (float)(bins - 1);
  size_t total = t->pixels() * t->cp;
  // Every block ends by adding its private histogram to the global one (up to `bins` 64-bit atomics), so few, large
  // blocks: 1024 threads, at most two per SM, and at least four vectors per thread.
  const int threads = 1024;
  int grid = (int)std::min<size_t>((total / 4 + (size_t)threads * 4 - 1) / ((size_t)threads * 4),
                                   (size_t)I.sm_count * (2048 / threads));
  if (grid < 1) grid = 1;
  hist_f32_kernel<<<grid, threads, bins * sizeof(unsigned), I.stream>>>(d_values ? d_values : (const float *)t->dev,
                                                                    t->pixels(), t->c, t->cp, width, bins,
                                                                    (unsigned long long *)d_hist);
  TPUCB_CUDA(cudaGetLastError());
}

int tpucb_calib_minmax(tpucb_interp *it, const char *name, float *d_stats) {
  TPUCB_API_BEGIN
  calib_minmax_impl(it, name, d_stats, nullptr, "tpucb_calib_minmax");
  TPUCB_API_END
}

int tpucb_calib_minmax_keep(tpucb_interp *it, const char *name, float *d_stats, float *d_keep) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(d_keep, "tpucb_calib_minmax_keep: bad argument");
  calib_minmax_impl(it, name, d_stats, d_keep, "tpucb_calib_minmax_keep");
  TPUCB_API_END
}

int tpucb_calib_hist(tpucb_interp *it, const char *name, float abs_max, int bins, int64_t *d_hist) {
  TPUCB_API_BEGIN
  calib_hist_impl(it, name, nullptr, abs_max, bins, d_hist, "tpucb_calib_hist");
  TPUCB_API_END
}

int tpucb_calib_hist_kept(tpucb_interp *it, const char *name, const float *d_kept, float abs_max, int bins,
                          int64_t *d_hist) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(d_kept, "tpucb_calib_hist_kept: bad argument");
  calib_hist_impl(it, name, d_kept, abs_max, bins, d_hist, "tpucb_calib_hist_kept");
  TPUCB_API_END
}

// Fills and uploads the descriptor list of an all-tensor statistics launch (ordered on the interpreter's stream behind
// the previous launch that read the list).
static const StatDesc *stat_descs_upload(tpucb_interp *it, const char *const *names, int count, const float *const *d_values,
                                         float *const *d_keep, const float *abs_max, int bins, const char *who) {
  Interpreter &I = it->impl;
  std::vector<StatDesc> h((size_t)count);
  for (int t = 0; t < count; ++t) {
    TPUCB_CHECK(names[t], "%s: name %d is NULL", who, t);
    auto tn = I.tensor(names[t]);
    TPUCB_CHECK(tn->dtype == DT_F32 && tn->cp % 4 == 0, "%s: tensor %s is not fp32 with a channel pitch of 4n", who, names[t]);
    StatDesc &d = h[t];
    d.x = d_values && d_values[t] ? d_values[t] : (const float *)tn->dev;
    d.keep = d_keep ? d_keep[t] : nullptr;
    TPUCB_CHECK((((uintptr_t)d.x | (uintptr_t)d.keep) & 15) == 0, "%s: buffer %d is not 16-byte aligned", who, t);
    d.nvec = (unsigned long long)(tn->pixels() * tn->cp / 4);
    d.vpp = tn->cp / 4;
    d.c = tn->c;
    // width = abs_max / (bin_num - 1), in fp32 as numpy computes it (kld_calibrator.py:34)
    d.width = abs_max ? abs_max[t] / (float)(bins - 1) : 0.0f;
    d.pad_ = 0;
  }
  if (it->stat_descs_cap < count) {
    TPUCB_CUDA(cudaStreamSynchronize(I.stream));
    if (it->stat_descs) TPUCB_CUDA(cudaFree(it->stat_descs));
    it->stat_descs = nullptr;
    it->stat_descs_cap = 0;
    TPUCB_CUDA(cudaMalloc(&it->stat_descs, sizeof(StatDesc) * count));
    it->stat_descs_cap = count;
  }
  TPUCB_CUDA(cudaMemcpyAsync(it->stat_descs, h.data(), sizeof(StatDesc) * count, cudaMemcpyHostToDevice, I.stream));
  return it->stat_descs;
}

int tpucb_calib_minmax_all(tpucb_interp *it, const char *const *names, int count, float *d_stats, float *const *d_keep) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && names && d_stats && count > 0, "tpucb_calib_minmax_all: bad argument");
  Interpreter &I = it->impl;
  I.bind();
  const StatDesc *d = stat_descs_upload(it, names, count, nullptr, d_keep, nullptr, 2, "tpucb_calib_minmax_all");
  // one 1024-thread block per SM: the kernel keeps four 16-byte loads per thread in flight (about 60 registers), which
  // covers the memory latency at half occupancy
  minmax_multi_kernel<<<I.sm_count, 1024, 0, I.stream>>>(d, count, d_stats);
  TPUCB_CUDA(cudaGetLastError());
  TPUCB_API_END
}

int tpucb_calib_hist_all(tpucb_interp *it, const char *const *names, int count, const float *const *d_values,
                         const float *abs_max, int bins, int64_t *d_hist) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && names && abs_max && d_hist && count > 0, "tpucb_calib_hist_all: bad argument");
  TPUCB_CHECK(bins >= 128 && bins <= 4096, "tpucb_calib_hist_all: bins must be in [128, 4096]");
  Interpreter &I = it->impl;
  I.bind();
  const StatDesc *d = stat_descs_upload(it, names, count, d_values, nullptr, abs_max, bins, "tpucb_calib_hist_all");
  hist_multi_kernel<<<I.sm_count * 2, 1024, bins * sizeof(unsigned), I.stream>>>(d, count, bins,
                                                                               (unsigned long long *)d_hist);
  TPUCB_CUDA(cudaGetLastError());
  TPUCB_API_END
}

int tpucb_calib_kld(tpucb_interp *it, const int64_t *d_hist, const float *widths, int count, int bins,
                    float *thresholds) {
  TPUCB_API_BEGIN
  TPUCB_CHECK(it && d_hist && widths && thresholds && count > 0, "tpucb_calib_kld: bad argument");
  TPUCB_CHECK(bins % 128 == 0 && bins >= 128 && bins <= 4096, "tpucb_calib_kld: bins must be a multiple of 128 up to 4096");
  Interpreter &I = it->impl;
  I.bind();
  const int kl_num = bins / 128;
  float *d_kl = nullptr;
  TPUCB_CUDA(cudaMalloc(&d_kl, sizeof(float) * count * kl_num));
  size_t smem = (size_t)bins * (2 * sizeof(float) + sizeof(double));
  // always the limit of the largest bin count: the attribute is per function and device, shared with
  // tpucb_calib_kld_static and with other threads, so no call may lower it under another call's launch
  cudaError_t e = cudaFuncSetAttribute(kld_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kKldMaxSmem);
  if (e != cudaSuccess) {
    cudaFree(d_kl);
    TPUCB_CUDA(e);
  }
  kld_kernel<<<count * kl_num, 256, smem, I.stream>>>((const long long *)d_hist, bins, d_kl);
  std::vector<float> kl((size_t)count * kl_num);
  e = cudaMemcpyAsync(kl.data(), d_kl, kl.size() * sizeof(float), cudaMemcpyDeviceToHost, I.stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(I.stream);
  cudaFree(d_kl);
  TPUCB_CUDA(e);
  // the_min_index + threshold (calibration_math.cpp:85-98, 321-322): first strict minimum.
  for (int t = 0; t < count; ++t) {
    const float *k = kl.data() + (size_t)t * kl_num;
    int m_min = 0;
    float best = k[0];
    for (int i = 1; i < kl_num; ++i)
      if (best > k[i]) {
        best = k[i];
        m_min = i;
      }
    thresholds[t] = widths[t] * (m_min + 1) * 128;
  }
  TPUCB_API_END
}

} // extern "C"

// ------------------------------------------------------- allocation-free KLD threshold search
//
// Scratch for tpucb_calib_kld_static: the KL value of every (histogram, candidate) pair. The
// array is part of the library's device image, so each GPU that loads the library holds these
// 32 KiB until the process exits. In host code the name below is only a handle for the runtime;
// the device address is obtained per device with cudaGetSymbolAddress and that pointer is what
// the kernel receives.
static __device__ __align__(256) float g_kld_static_scratch[TPUCB_KLD_STATIC_MAX_HISTS * 32];

namespace {
constexpr int kMaxDevices = 64;
float *g_kld_static_ptr[kMaxDevices] = {nullptr};
bool g_kld_static_ready[kMaxDevices] = {false};
std::mutex g_kld_static_mutex;

// Once per device, with that device current: resolve the scratch array's device address.
float *kld_static_setup(int device) {
  std::lock_guard<std::mutex> lock(g_kld_static_mutex);
  if (!g_kld_static_ready[device]) {
    float *ptr = nullptr;
    TPUCB_CUDA(cudaGetSymbolAddress((void **)&ptr, g_kld_static_scratch));
    // the dynamic shared memory limit of the kernel (a per-function setting, not an allocation), once, at the value
    // of the largest bin count, which is also what tpucb_calib_kld sets: no call ever lowers it
    TPUCB_CUDA(cudaFuncSetAttribute(kld_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kKldMaxSmem));
    TPUCB_CHECK(ptr != nullptr, "tpucb_calib_kld_static: the scratch array has no device address");
    g_kld_static_ptr[device] = ptr;
    g_kld_static_ready[device] = true;
  }
  return g_kld_static_ptr[device];
}
} // namespace

extern "C" int tpucb_calib_kld_static(int device, void *stream, const int64_t *d_hist, const float *widths,
                                      int count, int bins, float *thresholds) {
  int previous = -1;
  bool switched = false;
  try {
    TPUCB_CHECK(d_hist && widths && thresholds, "tpucb_calib_kld_static: NULL argument");
    TPUCB_CHECK(count > 0 && count <= TPUCB_KLD_STATIC_MAX_HISTS,
                "tpucb_calib_kld_static: count %d is outside [1, %d] (the static scratch holds %d histograms' "
                "candidates; split the call or use tpucb_calib_kld)",
                count, TPUCB_KLD_STATIC_MAX_HISTS, TPUCB_KLD_STATIC_MAX_HISTS);
    TPUCB_CHECK(bins % 128 == 0 && bins >= 128 && bins <= 4096,
                "tpucb_calib_kld_static: bins must be a multiple of 128 in [128, 4096], got %d", bins);
    TPUCB_CHECK(device >= 0 && device < kMaxDevices, "tpucb_calib_kld_static: device %d out of range", device);
    TPUCB_CUDA(cudaGetDevice(&previous));
    if (previous != device) {
      TPUCB_CUDA(cudaSetDevice(device));
      switched = true;
    }
    float *d_kl = kld_static_setup(device);
    cudaStream_t st = (cudaStream_t)stream;
    const int kl_num = bins / 128;
    const size_t smem = (size_t)bins * (2 * sizeof(float) + sizeof(double));
    kld_kernel<<<count * kl_num, 256, smem, st>>>((const long long *)d_hist, bins, d_kl);
    TPUCB_CUDA(cudaGetLastError());
    // host copy of the KL values: fixed-size, on the stack
    float kl[TPUCB_KLD_STATIC_MAX_HISTS * 32];
    TPUCB_CUDA(cudaMemcpyAsync(kl, d_kl, sizeof(float) * (size_t)count * kl_num, cudaMemcpyDeviceToHost, st));
    TPUCB_CUDA(cudaStreamSynchronize(st));
    for (int t = 0; t < count; ++t) {
      const float *k = kl + (size_t)t * kl_num;
      int m_min = 0;
      float best = k[0];
      for (int i = 1; i < kl_num; ++i)
        if (best > k[i]) {
          best = k[i];
          m_min = i;
        }
      thresholds[t] = widths[t] * (m_min + 1) * 128;
    }
    if (switched) cudaSetDevice(previous);
  } catch (const std::exception &e) {
    if (switched) cudaSetDevice(previous);
    g_last_error = e.what();
    return 1;
  }
  return 0;
}
