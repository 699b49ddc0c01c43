/* C ABI of the B200 interpreter backend (libtpucb.so).
 *
 * The reference exposes this path as C++ classes, not as a C ABI:
 *   class MlirModuleInterpreter   include/tpuc/MlirModuleInterpreter.h:32-83
 *   class CPUOpKernel::invoke()   include/tpuc/Interpreter/cpukernel.h:87-159
 *   pymlir.module (pybind11)      bindings/python/pymlir.cpp:289-311
 *   kl_diversity_hist (extern C)  bindings/python/kld/calibration_math.cpp:342-344
 * Each entry point below names the member it stands in for. Host tensors cross
 * this boundary exactly as they do in the reference: float32 NCHW "containers"
 * (cpukernel.h:15-78) holding int8 / bf16 / fp32 values. Host memory passed in
 * is borrowed for the duration of the call only.
 *
 * Every function returns 0 on success and a non-zero status otherwise;
 * tpucb_last_error() returns the message of the calling thread's last failure.
 * There is no CPU fallback: without a CUDA device every compute call fails.
 */
#ifndef TPUCB_H_
#define TPUCB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tpucb_interp tpucb_interp;

const char *tpucb_last_error(void);
/* Library/ABI version, for the binding to check. */
int tpucb_version(void);

/* ---- MlirModuleInterpreter ------------------------------------------------- */

/* MlirModuleInterpreter::MlirModuleInterpreter(max_batch_size)
 * (MlirModuleInterpreter.h:35). `device` is the CUDA ordinal; the interpreter owns
 * one stream and every device tensor of the module. */
int tpucb_interp_create(int device, tpucb_interp **out);
/* The same with max_batch_size > 1 (MlirModuleInterpreter.h:35, CPUOpKernel::max_batch_size cpukernel.h:153): the
 * reference then keeps max_batch_size copies ("batch slots") of every activation (TensorData, cpukernel.h:15-78) and
 * runs its kernels on one slot at a time (set_batch_idx). Here slot b is image group b of ONE device tensor whose
 * leading dimension is max_batch_size x the module's, so a launch covers every slot. The tensor shapes, input / output
 * sizes and op shapes reported by the calls below stay the module's (one slot). Ops that may mix the leading
 * dimension with the others (matmul, permute, reduce, pad, crop, broadcast) are refused at load on such an
 * interpreter. tpucb_interp_set_tensor / get_tensor without a slot address all slots at once (max_batch_size x the
 * slot's values, slot-major). */
int tpucb_interp_create_batched(int device, int max_batch_size, tpucb_interp **out);
int tpucb_interp_max_batch_size(tpucb_interp *it, int *max_batch_size);
int tpucb_interp_destroy(tpucb_interp *it);

/* MlirModuleInterpreter::updateWeightMap (MlirModuleInterpreter.cpp:352-369): register
 * one tpu.load_weight tensor by name as fp32 values, before tpucb_interp_load_module. */
int tpucb_interp_set_weight(tpucb_interp *it, const char *name, const float *data,
                            const int64_t *shape, int rank);

/* MlirModuleInterpreter::loadModule (MlirModuleInterpreter.cpp:73-83, 118-350). The module
 * is given as text, one op per line:
 *     <op_type> name=<result> in=<operand>,<operand>,... shape=<d0>,<d1>,.. dtype=INT8|BF16|FP32 key=value ...
 * with the operand order of the TPU dialect op ("-" for an absent operand) and the
 * attribute names of the dialect's param structs. An op the backend does not implement
 * is an error here, not at run time. */
int tpucb_interp_load_module(tpucb_interp *it, const char *module_text);

/* MlirModuleInterpreter::setTensor (MlirModuleInterpreter.cpp:407-417). */
int tpucb_interp_set_tensor(tpucb_interp *it, const char *name, const float *data, size_t numel);
/* setTensor / getTensor with their bidx argument (MlirModuleInterpreter.cpp:407-427; TensorData::assign and
 * TensorData::tensor, cpukernel.h:49-67): the values of batch slot `bidx`, numel = the module's tensor size. */
int tpucb_interp_set_tensor_slot(tpucb_interp *it, const char *name, const float *data, size_t numel, int bidx);
int tpucb_interp_get_tensor_slot(tpucb_interp *it, const char *name, float *out, size_t numel, int bidx);
/* invokeTo(name, bidx) / invoke(bidx) (MlirModuleInterpreter.cpp:371-381; NULL or "" = the whole module). The
 * reference runs the kernels on slot bidx only; one launch here computes every slot, so slot bidx holds what the
 * reference would have produced and the other slots the results for whatever inputs they hold. Synchronous. */
int tpucb_interp_invoke_slot(tpucb_interp *it, const char *name, int bidx);
/* fastInvokeAllBatch(name, batch) (MlirModuleInterpreter.cpp:383-405): every op built since the last such call (the
 * "dirty" ones, cpukernel.h:152) up to `name`, for the slots 0..batch-1: ONE launch per op over all slots instead of
 * the reference's loop over the slots. Synchronous. */
int tpucb_interp_fast_invoke_all_batch(tpucb_interp *it, const char *name, int batch);
/* MlirModuleInterpreter::dump(name) / CPUOpKernel::dump (cpukernel.h:126): a text description of one op (name,
 * type, data type, shape, the line it was built from). *needed receives the required capacity. */
int tpucb_interp_dump(tpucb_interp *it, const char *name, char *out, size_t cap, size_t *needed);

/* ---- CPUOpKernel (include/tpuc/Interpreter/cpukernel.h:87-159) ------------------------------------
 * One op at a time, for an adapter that subclasses the reference's CPUOpKernel and owns a single op. The interpreter
 * handle plays the part of the (value_map_t, weight_map_t) pair the reference constructors receive: operands are looked
 * up in it by name, the result tensor is created in it and becomes visible to later ops; weights are registered with
 * tpucb_interp_set_weight beforehand. */
typedef struct tpucb_op tpucb_op;
/* CPUOpKernel::CPUOpKernel(Operation &, value_map_t &, weight_map_t &) (cpukernel.h:90): `op_line` is one line of the
 * module text of tpucb_interp_load_module. An op the backend does not implement is an error here. Ops created this
 * way also run as part of tpucb_interp_invoke, in creation order; they are not fused with their neighbours. The handle
 * belongs to the interpreter (freed by tpucb_interp_destroy, invalidated by tpucb_interp_load_module). */
int tpucb_op_create(tpucb_interp *ctx, const char *op_line, tpucb_op **out);
/* CPUOpKernel::invoke() (cpukernel.h:101): runs this op on its operands' current values, all batch slots. Synchronous. */
int tpucb_op_invoke(tpucb_op *op);
/* CPUOpKernel::set_tensor (cpukernel.h:97; implemented by the input op only, core/input.cpp:17-24) and get_tensor
 * (deep copy, cpukernel.h:130-134), for batch slot bidx. */
int tpucb_op_set_tensor(tpucb_op *op, const float *data, size_t numel, int bidx);
int tpucb_op_get_tensor(tpucb_op *op, float *out, size_t numel, int bidx);
/* get_name / get_op_type / get_data_type / get_shape and the dirty flag (cpukernel.h:103-124, 144-152) as
 * "name\ttype\tdtype\tshape\tdirty". */
int tpucb_op_info(tpucb_op *op, char *out, size_t cap, size_t *needed);

/* Pipelined setTensor for serving loops (no reference counterpart): the copy from PINNED host
 * memory runs on a second stream and overlaps a module launch that is still executing; the data
 * becomes the tensor's value for the next launch. The host buffer must stay untouched until
 * the next tpucb_interp_sync / invoke / get_tensor. */
int tpucb_interp_set_tensor_async(tpucb_interp *it, const char *name, const float *pinned, size_t numel);
/* The same for input values the caller has ALREADY quantised (no reference counterpart): int8, NCHW order, pinned.
 * One byte per value crosses the host link instead of the four of the fp32 container, which is what bounds the
 * end-to-end rate once several GPUs share a host. `name` is an INT8 tensor that is a module input or the result of
 * the tpu.quant (NONE -> INT8) op directly behind an fp32 module input; that quant op is then skipped by the launches
 * that follow, until the fp32 input is set again with tpucb_interp_set_tensor(_async). The values must be what the op
 * would have produced: sat8(round half away from zero(x * scale)) (QuantOpKernel, core/quant.cpp:22-30). */
int tpucb_interp_set_tensor_async_i8(tpucb_interp *it, const char *name, const int8_t *pinned, size_t numel);
/* Blocks until every copy started by tpucb_interp_set_tensor_async has left its host buffer (the buffers may be
 * refilled afterwards); does not wait for launches. */
int tpucb_interp_wait_uploads(tpucb_interp *it);
/* MlirModuleInterpreter::invoke / invokeTo (MlirModuleInterpreter.cpp:371-381); an empty or
 * NULL name runs the whole module. Synchronous, like the reference. */
int tpucb_interp_invoke(tpucb_interp *it);
int tpucb_interp_invoke_to(tpucb_interp *it, const char *name);
/* Asynchronous halves of invoke: enqueue on the interpreter's stream / wait and check the
 * device error word. (No reference counterpart: the CPU interpreter is synchronous.) */
int tpucb_interp_launch(tpucb_interp *it);
int tpucb_interp_sync(tpucb_interp *it);
/* MlirModuleInterpreter::getTensor (deep copy, MlirModuleInterpreter.cpp:419-427). */
int tpucb_interp_get_tensor(tpucb_interp *it, const char *name, float *out, size_t numel);
/* getTensorShape / getDataType / getAllTensorName (MlirModuleInterpreter.h:52-60). */
int tpucb_interp_get_tensor_shape(tpucb_interp *it, const char *name, int64_t *shape, int *rank);
/* writes "INT8", "BF16" or "FP32" */
int tpucb_interp_get_data_type(tpucb_interp *it, const char *name, char *out, size_t cap);
/* names separated by '\n'; *needed receives the required capacity */
int tpucb_interp_get_all_tensor_names(tpucb_interp *it, char *out, size_t cap, size_t *needed);
/* input_details / output_details (MlirModuleInterpreter.h:79-80): "name:numel" lines */
int tpucb_interp_get_details(tpucb_interp *it, int outputs, char *out, size_t cap, size_t *needed);
/* op_info of pymlir (bindings/python/pymlir.cpp:62-97): "name\ttype\tdtype\tshape" lines */
int tpucb_interp_get_op_info(tpucb_interp *it, char *out, size_t cap, size_t *needed);

/* Options: "cuda_graph" (0/1, default 1): replay the op list as one CUDA graph.
 *          "pdl" (0 off, 1 = default, 2 every kernel): programmatic dependent launch. A kernel launched with the
 *          attribute may be scheduled while its predecessor in the stream is still running: its launch and set-up
 *          (barriers, tensor memory) overlap that kernel's tail, and it waits for that kernel's results before its first
 *          global access. 1 gives the attribute to the tensor-core convolution kernels only, which measured faster than
 *          none and than all on every graph and batch tried (on the memory-bound kernels alone it costs 1-5%).
 *          "split_k" (0/1, default 1; read by the next load_module): INT8 convolutions and inner products with few
 *          tiles and 24 K blocks or more share each tile among several CTAs (exact: int32 partial sums).
 *          "fuse_activations" (0/1, default 1; read by the next load_module): run each
 *          quant(INT8->BF16) -> slope-table activation -> quant(BF16->INT8) chain as one launch
 *          that still writes all three tensors.
 *          "selftest_lost_arrival" (0 = off (default), else rounds in [1, 1024]; read by the next load_module): a
 *          self-test of the error path. Every wait inside the tensor-core kernels is bounded (1024 rounds of 1024
 *          polls); when one runs out the kernel records a code in the interpreter's device error word, drains its
 *          copies, frees its tensor memory and returns, and the next tpucb_interp_sync / invoke reports it as an
 *          error status while the interpreter stays usable. With this option the INT8 convolutions of the next
 *          module never hand their accumulator back and wait only `rounds` rounds, so that exactly this happens.
 *          "fuse_residual_add" (0/1, default 0; read by the next load_module; needs fuse_activations): an INT8
 *          two-input eltwise add whose later-produced operand is a tensor-core convolution that feeds nothing else
 *          (the last convolution of a residual block) runs in that convolution's epilogue, which reads the other
 *          operand and writes both the convolution's tensor and the sum; the add launches nothing. Same bits.
 *          Measured on INT8 ResNet-50 at batch 256: 1% fewer ms per step (the add kernels already run at the
 *          HBM rate and the epilogue is bound by its integer instructions), so it is off by default.
 *          "fp32_tensor_cores" (0/1, default 1; read by the next load_module): fp32 convolutions with a
 *          multiple of 8 input channels run on the tensor cores as three TF32 products with fp32 accumulation
 *          (about 5e-6 of a tensor's range per layer against a double-accumulated sum, 6e-5 at the end of an
 *          fp32 ResNet-50); 0 keeps every fp32 convolution on the FMA pipe (2e-6 end to end, 2.5 x slower). */
int tpucb_interp_set_option(tpucb_interp *it, const char *key, int value);
/* Per-op device time of one eager pass (CUDA events on the interpreter's stream);
 * ms[i] belongs to the i-th line of tpucb_interp_get_op_info. Returns the op count. */
int tpucb_interp_profile(tpucb_interp *it, float *ms, int cap, int *count);
/* Device time in milliseconds of `iters` back-to-back whole-module launches. */
int tpucb_interp_time_launches(tpucb_interp *it, int iters, float *ms_total);
/* Number of this library's kernels one whole-module invoke launches. */
int tpucb_interp_kernel_count(tpucb_interp *it, int *count);

/* Device pointer, byte size and channel pitch of a tensor's NHWC storage (for the
 * calibration statistics entry points below and for torch.distributed collectives). */
int tpucb_interp_tensor_device(tpucb_interp *it, const char *name, void **dev, size_t *bytes,
                               int *channels, int *channel_pitch, int *dtype);

/* Measures the dense INT8 rate of the tensor pipe on `device`: every SM issues a long chain of
 * tcgen05.mma kind::i8 (M=128, N=n_cols in {64,128,256}, K=32) on operands resident in shared memory.
 * Writes tera-ops/s (2 ops per MAC). No reference counterpart; it supplies the roofline denominator
 * of the convolution kernel, for which the driver-written peaks have no INT8 entry. */
int tpucb_measure_i8_mma_peak(int device, int n_cols, double *tops);

/* Pinned host buffers for the e2e path. */
int tpucb_host_alloc(void **ptr, size_t bytes);
/* write-combined pinned memory: faster for the device to read, slow for the host to read back; for upload buffers
 * that the host only writes */
int tpucb_host_alloc_write_combined(void **ptr, size_t bytes);
int tpucb_host_free(void *ptr);

/* ---- calibration statistics (python/cvi_toolkit/calibration/kld_calibrator.py) --------- */

/* find_min_max_abs (kld_calibrator.py:269-296): running min / max over the fp32 tensor's
 * real channels, folded into stats[0]=min, stats[1]=max (device floats, caller-initialised
 * to +inf / -inf). */
int tpucb_calib_minmax(tpucb_interp *it, const char *name, float *d_stats);
/* histogram (kld_calibrator.py:31-43): adds the tensor's |x| != 0 values to a device
 * histogram of `bins` int64 counts with width abs_max / (bins - 1). */
int tpucb_calib_hist(tpucb_interp *it, const char *name, float abs_max, int bins, int64_t *d_hist);
/* The same two with every batch's activations kept on the device between the passes, so that the
 * histogram pass needs no second forward (the reference re-runs the model per image in
 * calc_thresholds, kld_calibrator.py:298-336; a B200 holds the fp32 activations of hundreds of
 * images). tpucb_calib_minmax_keep also writes the tensor's real lanes to d_keep, a 16-byte aligned
 * device buffer of the tensor's storage size (tpucb_interp_tensor_device gives the bytes), in the
 * pass that reads them; tpucb_calib_hist_kept takes its values from such a copy (`name` gives the
 * geometry). Work is ordered on the interpreter's stream. */
int tpucb_calib_minmax_keep(tpucb_interp *it, const char *name, float *d_stats, float *d_keep);
int tpucb_calib_hist_kept(tpucb_interp *it, const char *name, const float *d_kept, float abs_max,
                          int bins, int64_t *d_hist);
/* Both statistics for a list of tensors in ONE launch each (persistent blocks that walk the list: a
 * module has some seventy tensors, most of them too small to fill the GPU for the length of a
 * launch). names [count]; d_stats [count][2] device floats as in tpucb_calib_minmax; d_keep NULL or
 * a host array of `count` device pointers as in tpucb_calib_minmax_keep; d_values NULL or a host
 * array of kept copies (a NULL entry reads the tensor itself); abs_max [count] host floats; d_hist
 * [count][bins] device counts. */
int tpucb_calib_minmax_all(tpucb_interp *it, const char *const *names, int count, float *d_stats,
                           float *const *d_keep);
int tpucb_calib_hist_all(tpucb_interp *it, const char *const *names, int count,
                         const float *const *d_values, const float *abs_max, int bins,
                         int64_t *d_hist);
/* kl_diversity_hist (calibration_math.cpp:283-344) for `count` histograms at once:
 * d_hist [count][bins] int64 device counts, widths [count] host floats, thresholds
 * [count] host floats out. */
int tpucb_calib_kld(tpucb_interp *it, const int64_t *d_hist, const float *widths, int count,
                    int bins, float *thresholds);

/* ---- threshold auto-tuner (python/cvi_toolkit/calibration/kld_calibrator.py:113-201) ------ */

/* Device-to-device copy of one tensor between two interpreters on the same GPU; the two
 * tensors must agree in type, shape and device layout. It stands in for the get_tensor ->
 * set_data round trip through numpy with which the reference's tuner would move an activation
 * between two loaded modules (bindings/python/pytuner.cpp:252-288). Returns after the copy. */
int tpucb_interp_copy_tensor(tpucb_interp *dst, const char *dst_name, tpucb_interp *src,
                             const char *src_name);
/* The two norms of SimpleTuner.run (kld_calibrator.py:184-196) for every image of the batch,
 * with both activations left on the device: sums[2i] = sum over image i of
 * (ref - scale * tgt)^2, sums[2i+1] = sum |ref| (host doubles out, `images` = the tensors'
 * batch). ref is an fp32 tensor of `ref`; tgt a tensor of the same shape of `tgt` (INT8, BF16
 * or fp32; pass scale = threshold / 127 for INT8 and 1 otherwise). The difference is formed in
 * fp32 as numpy forms it, the sums in double. */
int tpucb_tuner_distance(tpucb_interp *ref, const char *ref_name, tpucb_interp *tgt,
                         const char *tgt_name, float scale, double *sums, int images);

/* Allocation-free variant of tpucb_calib_kld. It has no counterpart in the reference; it exists
 * for hosts that must not allocate device memory while they work: a calibration service that
 * sized its device memory once at start-up (this backend keeps every activation of the module
 * resident, so the budget is usually spoken for), or a worker thread that runs the threshold
 * search while other streams are busy and cannot afford the device-wide synchronisation and the
 * late out-of-memory failure that cudaMalloc / cudaFree bring. The per-candidate KL values that
 * tpucb_calib_kld keeps in a temporary device buffer live here in a fixed array inside the
 * library's device image: TPUCB_KLD_STATIC_MAX_HISTS x 32 floats (32 KiB), held by every GPU
 * that loads the library until the process exits.
 *   - `device` is the CUDA ordinal the histograms live on, `stream` a cudaStream_t. NULL is the
 *     LEGACY default stream, which waits for, and holds up, every blocking stream of the process;
 *     pass a stream made with cudaStreamNonBlocking to stay clear of other work. d_hist [count][bins] int64 device counts, widths [count] host floats,
 *     thresholds [count] host floats out: same meaning as in tpucb_calib_kld.
 *   - count > TPUCB_KLD_STATIC_MAX_HISTS, or bins not a multiple of 128 in [128, 4096], is
 *     refused with an error; nothing is launched.
 *   - The first call on a device looks up the array's device address (once per device); make
 *     that first call before any stream capture is begun on the calling thread.
 *   - All calls share the one array, which keeps the previous call's values: the kernel
 *     overwrites every slot it later reads, so nothing needs clearing, but two calls that
 *     overlap on the same GPU (different streams or threads) race on it. Serialise them.
 *   - Calls no cudaMalloc, cudaFree or other allocating routine; returns after the results are
 *     on the host. */
#define TPUCB_KLD_STATIC_MAX_HISTS 256
int tpucb_calib_kld_static(int device, void *stream, const int64_t *d_hist, const float *widths,
                           int count, int bins, float *thresholds);

#ifdef __cplusplus
}
#endif
#endif /* TPUCB_H_ */
