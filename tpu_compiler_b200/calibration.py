"""Activation calibration on device: the statistics half of the reference's
``ActivationCalibrator`` (python/cvi_toolkit/calibration/kld_calibrator.py:204-382).

Two dependent passes over the calibration images, as in the reference: (1) running min / max /
abs-max of every op result; (2) 2048-bin |x| histograms with width abs_max / 2047; then the
KLD threshold search (bindings/python/kld/calibration_math.cpp) per tensor. The fp32 forward
and all three statistics run as CUDA kernels; the tensors never leave the device. With
``torch.distributed`` initialised, every rank calibrates on its own shard of the images and
the statistics are combined with one all-reduce(MAX) after pass 1 (abs-max, max and -min packed
into one buffer) and one all-reduce(SUM) of the int64 histograms after pass 2.

The reference runs the model a second time for the histograms (calc_thresholds,
kld_calibrator.py:298-336) because it cannot keep every activation of every image. A 180 GB GPU
can: pass 1 writes each batch's fp32 activations to a device cache in the same kernel that takes
their min / max (``keep_activations_gb``, default: up to 60% of the memory free at that time), and
pass 2 reads the histograms of the cached batches from there -- no upload, no second forward.
Batches beyond the budget are recomputed as before. The values read are the same bits either way.
"""
import ctypes as C
import datetime
import time

import numpy as np
import torch

from ._lib import check, lib


def join_ranks(backend, rank, world_size, timeout_s=60.0, init_method=None):
    """``torch.distributed.init_process_group`` with a short rendezvous limit and a plain error: a rank that never
    starts (a crashed worker, a wrong WORLD_SIZE) makes the others fail after ``timeout_s`` seconds with a message that
    says so, instead of waiting for the default half hour. Returns ``torch.distributed``."""
    import datetime as _dt
    import torch.distributed as dist
    try:
        dist.init_process_group(backend, rank=rank, world_size=world_size, init_method=init_method,
                                timeout=_dt.timedelta(seconds=timeout_s))
    except Exception as e:  # the store's own message names sockets and keys, not the cause
        raise RuntimeError("rank %d: not all %d ranks joined within %.0f s (%s: %s)"
                           % (rank, world_size, timeout_s, type(e).__name__, str(e).splitlines()[0][:120])) from e
    return dist


class ActivationCalibrator:
    def __init__(self, model, batches, histogram_bin_num=2048, input_name=None, dist=None, keep_activations_gb=None,
                 expected_batches=None):
        """model: a loaded ``tpu_compiler_b200.module`` of an fp32 graph; batches: a callable
        returning an iterator over this rank's input batches (float32 arrays of the input's
        shape) -- it is called twice, once per pass."""
        self.model = model
        self.batches = batches
        self.bin_num = int(histogram_bin_num)
        self.dist = dist
        self.input_name = input_name or model.get_input_details()[0]
        self.names = [o["name"] for o in model.op_info if o["dtype"] == "FP32"]
        self.device = torch.device("cuda", model._device) if model._device is not None else torch.device("cpu")
        self._lib = lib() if model._device is not None else None
        self.num_samples = 0
        self.keep_activations_gb = keep_activations_gb   # None: 60% of the free device memory; 0: keep nothing
        self._kept = []          # per cached batch: (uint8 device buffer, images)
        self._kept_offsets = None
        self._local_images = -1   # images this rank saw in pass 1
        self._pinned = None
        self._pinned_numel = 0
        self._pinned_next = 0
        self._reserved = []      # cache buffers allocated ahead of pass 1
        # host seconds of this rank's last pass 1 by part: copying batches into pinned memory, waiting for earlier
        # uploads to leave their buffer, enqueueing (module launch + statistics launch), the final synchronisation
        self.pass1_host_s = {"pinned_copy": 0.0, "wait_uploads": 0.0, "enqueue": 0.0, "final_sync": 0.0, "combine": 0.0}
        if self.dist is not None:
            self._check_ranks_agree()   # once, at set-up: its all-reduces are not part of a pass
        if self._lib is not None:
            # the two pinned upload buffers are part of setting up (tens of milliseconds), not of a pass
            self._alloc_pinned(int(np.prod(model.get_tensor_shape(self.input_name))))
            if expected_batches:
                # so is the activation cache when the caller says how many batches will come: a cudaMalloc of several GB
                # blocks the host for milliseconds, and for far longer while other ranks' processes allocate too
                per_batch, budget = self._keep_plan()
                for _ in range(min(int(expected_batches), budget // per_batch if per_batch else 0)):
                    try:
                        self._reserved.append(torch.empty(per_batch, dtype=torch.uint8, device=self.device))
                    except torch.OutOfMemoryError:
                        break
                torch.cuda.synchronize(self.device)

    # -- device work of the two passes (overridden by the CPU stand-in used in the gloo tests) -------
    def _local_min_max(self):
        """This rank's running (min, max) per tensor as a [T, 2] tensor, and its image count."""
        T = len(self.names)
        stats = torch.empty((T, 2), dtype=torch.float32, device=self.device)
        stats[:, 0] = float("inf")
        stats[:, 1] = float("-inf")
        torch.cuda.synchronize(self.device)
        n_img = 0
        self._kept = []
        per_batch, budget = self._keep_plan()
        self.pass1_host_s = {k: 0.0 for k in self.pass1_host_s}
        for batch in self.batches():
            self._upload(batch)
            t_enq = time.perf_counter()
            self.model.launch()
            keep = None
            if self._reserved:
                keep = self._reserved.pop()
            elif per_batch and (len(self._kept) + 1) * per_batch <= budget:
                try:
                    keep = torch.empty(per_batch, dtype=torch.uint8, device=self.device)
                    # torch may hand out a block whose last use is still queued on ITS stream; the kernels that fill
                    # this buffer run on the module's stream, which knows nothing of that work: wait for it here
                    torch.cuda.current_stream(self.device).synchronize()
                except torch.OutOfMemoryError:
                    budget = 0
            keeps = None
            if keep is not None:
                keeps = (C.c_void_p * T)(*[keep.data_ptr() + o for o in self._kept_offsets])
            check(self._lib.tpucb_calib_minmax_all(self.model._h, self._name_array(), T, C.c_void_p(stats.data_ptr()), keeps))
            if keep is not None:
                # torch allocated `keep` on its own stream and the kernels above ran on the module's: the buffer is not
                # handed back to torch before the module's stream has been synchronised (end of this pass and of pass 2)
                self._kept.append((keep, batch.shape[0]))
            n_img += batch.shape[0]
            self.pass1_host_s["enqueue"] += time.perf_counter() - t_enq
        t_sync = time.perf_counter()
        self.model.sync()
        self.pass1_host_s["final_sync"] += time.perf_counter() - t_sync
        self._local_images = n_img
        return stats, n_img

    def _name_array(self):
        if getattr(self, "_names_c", None) is None:
            self._names_c = (C.c_char_p * len(self.names))(*[n.encode() for n in self.names])
        return self._names_c

    def _keep_plan(self):
        """(bytes one batch's fp32 activations take in the cache, byte budget of the cache)."""
        if self.keep_activations_gb is not None and self.keep_activations_gb <= 0:
            return 0, 0
        offs, total = [], 0
        for name in self.names:
            offs.append(total)
            total += (self.model.tensor_device(name)["bytes"] + 255) // 256 * 256
        self._kept_offsets = offs
        if self.keep_activations_gb is None:
            free, _ = torch.cuda.mem_get_info(self.device)
            budget = int(free * 0.6)
        else:
            budget = int(self.keep_activations_gb * 2 ** 30)
        return total, budget

    def _upload(self, batch):
        """The batch becomes the input of the next launch. It is copied into one of two pinned host buffers and sent
        with set_tensor_async, so the host-side copy and the transfer of batch i + 1 run while batch i is computed."""
        if (isinstance(batch, torch.Tensor) and batch.device.type == "cpu" and batch.dtype == torch.float32 and
                batch.is_contiguous() and batch.is_pinned()):
            # already in page-locked memory (a loader with pin_memory=True): sent from where it lies; the two most
            # recent batches are kept alive until their copies have left the host
            t0 = time.perf_counter()
            self.model.set_tensor_async(self.input_name, C.c_void_p(batch.data_ptr()), batch.numel())
            self._in_flight = (getattr(self, "_in_flight", ()) + (batch,))[-2:]
            self.pass1_host_s["enqueue"] += time.perf_counter() - t0
            return
        if isinstance(batch, torch.Tensor):
            batch = batch.numpy()
        batch = np.ascontiguousarray(batch, np.float32)
        if self._pinned is None or self._pinned_numel != batch.size:
            self._alloc_pinned(batch.size)
        h = self._pinned[self._pinned_next]
        self._pinned_next ^= 1
        t0 = time.perf_counter()
        self.model.wait_uploads()   # earlier copies have left the host buffers
        t1 = time.perf_counter()
        np.copyto(np.ctypeslib.as_array(C.cast(h, C.POINTER(C.c_float)), shape=(batch.size,)), batch.reshape(-1))
        t2 = time.perf_counter()
        self.model.set_tensor_async(self.input_name, h, batch.size)
        self.pass1_host_s["wait_uploads"] += t1 - t0
        self.pass1_host_s["pinned_copy"] += t2 - t1
        self.pass1_host_s["enqueue"] += time.perf_counter() - t2

    def _alloc_pinned(self, numel):
        self._free_pinned()
        self._pinned = []
        for _ in range(2):
            h = C.c_void_p()
            check(self._lib.tpucb_host_alloc(C.byref(h), numel * 4))
            self._pinned.append(h)
        self._pinned_numel = numel
        self._pinned_next = 0

    def _free_pinned(self):
        if getattr(self, "_pinned", None):
            try:
                self.model.sync()   # no copy may still read the buffers
            except Exception:
                pass                # the module was closed first: closing it synchronised the device
            for h in self._pinned:
                self._lib.tpucb_host_free(h)
        self._pinned = None

    def __del__(self):
        try:
            self._free_pinned()
        except Exception:
            pass

    def _local_histograms(self, activations_statistics, release=True):
        """This rank's [T, bins] int64 histograms. ``release`` False keeps the activation cache for another histogram
        pass with a different bin count (run_multi)."""
        T = len(self.names)
        hist = torch.zeros((T, self.bin_num), dtype=torch.int64, device=self.device)
        torch.cuda.synchronize(self.device)
        kept = self._kept
        if release:
            self._kept = []   # this was the cache's last histogram pass
        absmax = (C.c_float * T)(*[float(activations_statistics[n][2]) for n in self.names])
        for keep, _ in kept:
            vals = (C.c_void_p * T)(*[keep.data_ptr() + o for o in self._kept_offsets])
            check(self._lib.tpucb_calib_hist_all(self.model._h, self._name_array(), T, vals, absmax, self.bin_num,
                                                 C.c_void_p(hist.data_ptr())))
        for i, batch in enumerate(self.batches() if self._needs_recompute(kept) else ()):
            if i < len(kept):
                continue   # this batch's activations were read from the cache
            self._upload(batch)
            self.model.launch()
            check(self._lib.tpucb_calib_hist_all(self.model._h, self._name_array(), T, None, absmax, self.bin_num,
                                                 C.c_void_p(hist.data_ptr())))
        self.model.sync()
        del kept
        return hist

    def _needs_recompute(self, kept):
        """False when every batch of pass 1 is in the cache (then pass 2 does not even ask for the images again)."""
        return sum(n for _, n in kept) < self._local_images

    def _check_ranks_agree(self):
        """Every rank must calibrate the same tensors in the same order, or the all-reduces below would combine
        unrelated rows (or, with different counts, fail deep inside the collective): compare a fingerprint of the
        tensor list first and fail on every rank with a message that names the mismatch."""
        import zlib
        dev = self.device if self.device.type == "cuda" else torch.device("cpu")
        mine = torch.tensor([len(self.names), zlib.crc32("\n".join(self.names).encode()), self.bin_num], dtype=torch.int64,
                            device=dev)
        lo, hi = mine.clone(), mine.clone()
        self.dist.all_reduce(lo, op=self.dist.ReduceOp.MIN)
        self.dist.all_reduce(hi, op=self.dist.ReduceOp.MAX)
        if not torch.equal(lo, hi):
            raise RuntimeError("calibration ranks disagree: this rank has %d tensors (fingerprint %d, %d bins); across "
                               "ranks the counts span %d..%d" % (len(self.names), int(mine[1]), self.bin_num,
                                                                 int(lo[0]), int(hi[0])))
        # One collective of each kind and size the passes use, on zeros: the library builds its connections and loads
        # its kernels at the first use of each (30 ms measured on two GPUs), which belongs to the set-up.
        # The same goes for the few torch kernels of the combine step (loaded at their first launch): 27 ms in all.
        T = len(self.names)
        self._combine_min_max(torch.zeros(T, 2, dtype=torch.float32, device=dev), 0)[0].cpu()
        self.dist.all_reduce(torch.zeros(T, self.bin_num, dtype=torch.int64, device=dev), op=self.dist.ReduceOp.SUM)
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)

    def _combine_min_max(self, stats, n_img):
        """[T, 2] (min, max) of this rank and its image count -> those of all ranks: one all-reduce(MAX) over
        (-min, max), one all-reduce(SUM) of the count."""
        packed = torch.stack([-stats[:, 0], stats[:, 1]], dim=1).contiguous()
        self.dist.all_reduce(packed, op=self.dist.ReduceOp.MAX)
        stats = torch.stack([-packed[:, 0], packed[:, 1]], dim=1)
        cnt = torch.tensor([n_img], dtype=torch.int64, device=stats.device)
        self.dist.all_reduce(cnt, op=self.dist.ReduceOp.SUM)
        return stats, int(cnt.item())

    # -- pass 1 ------------------------------------------------------------------
    def find_min_max_abs(self):
        stats, n_img = self._local_min_max()
        t_comb = time.perf_counter()
        if self.dist is not None:
            stats, n_img = self._combine_min_max(stats, n_img)
        self.num_samples = n_img
        host = stats.cpu().numpy()
        self.pass1_host_s["combine"] = time.perf_counter() - t_comb
        out = {}
        for t, name in enumerate(self.names):
            mn, mx = np.float32(host[t, 0]), np.float32(host[t, 1])
            ab = max(abs(mn), abs(mx))
            if ab == 0:
                mn, mx, ab = np.float32(-1e-5), np.float32(1e-5), np.float32(1e-5)
            out[name] = (mn, mx, np.float32(ab))
        return out

    # -- pass 2 ------------------------------------------------------------------
    def calc_histograms(self, activations_statistics, release=True):
        hist = self._local_histograms(activations_statistics, release=release)
        if self.dist is not None:
            self.dist.all_reduce(hist, op=self.dist.ReduceOp.SUM)
        return hist

    def find_threshold(self, hist, activations_statistics):
        T = len(self.names)
        widths = np.array([np.float32(activations_statistics[n][2]) / np.float32(self.bin_num - 1) for n in self.names],
                          np.float32)
        thr = np.zeros(T, np.float32)
        torch.cuda.synchronize(self.device)
        fp = C.POINTER(C.c_float)
        check(self._lib.tpucb_calib_kld(self.model._h, C.c_void_p(hist.data_ptr()), widths.ctypes.data_as(fp), T,
                                        self.bin_num, thr.ctypes.data_as(fp)))
        return {n: thr[t] for t, n in enumerate(self.names)}

    def run_multi(self, bin_nums):
        """Thresholds for several histogram sizes from ONE min / max pass and one set of cached activations, the way the
        reference's calc_thresholds fills its thresholds_map for every bin count from the same pass
        (kld_calibrator.py:298-336): per bin count one histogram launch per cached batch and one KLD search. Returns
        ({bin count: {name: threshold}} in the order given, statistics). Bin counts are limited to 4096 by the
        histogram kernels (shared-memory tables); the reference's larger candidates (8192 .. 32768) are not covered."""
        stats = self.find_min_max_abs()
        out = {}
        bin_nums = list(bin_nums)
        keep = self.bin_num
        for i, bins in enumerate(bin_nums):
            self.bin_num = int(bins)
            hist = self.calc_histograms(stats, release=(i == len(bin_nums) - 1))
            out[int(bins)] = self.find_threshold(hist, stats)
        self.bin_num = keep
        return out, stats

    def run(self, output_calibration_table=None):
        stats = self.find_min_max_abs()
        hist = self.calc_histograms(stats)
        thresholds = self.find_threshold(hist, stats)
        self.histograms = hist
        if output_calibration_table and (self.dist is None or self.dist.get_rank() == 0):
            with open(output_calibration_table, "w") as f:
                f.write("# genetated time: {}\n".format(datetime.datetime.now()))
                f.write("# histogram number: {}\n".format(self.bin_num))
                f.write("# sample number: {}\n###\n".format(self.num_samples))
                f.write("# op_name    threshold    min    max\n")
                for name in self.names:
                    mn, mx, _ = stats[name]
                    f.write("{} {:.7f} {:.7f} {:.7f}\n".format(name, thresholds[name], mn, mx))
        return thresholds, stats
