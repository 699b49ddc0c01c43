#!/usr/bin/env python
"""Benchmark of the interpreter hot path: INT8 ResNet-50 images/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]

A step is one pass of the whole INT8 ResNet-50 module over one batch of B synthetic images
per GPU (uniform[-1,1] fp32 3x224x224, He-normal weights quantized per channel; see
tpu_compiler_b200/graphs.py). One process per GPU; the path has no cross-image dependency, so
ranks are independent replicas on disjoint image shards (weak scaling) and the only
collective is the max-reduce of the measured time.

`value`  : images/s with the inputs already resident in HBM (K graph launches, CUDA events).
`e2e`    : images/s through the public module API with host buffers: per step one pinned
           fp32 NCHW input upload (set_tensor_async: overlaps the previous step's compute),
           one launch, one fp32 output download.
`roofline` : the tcgen05 convolution kernel (dominant kernel), per-launch CUDA-event times
           from an eager pass inside this run, against the measured dense tensor peak.
`cpu_baseline` : the reference-faithful CPU path (oracle/cpu_path.py) on this host, all threads.
Untimed for the headline, in the same line (skipped by --no-extras): `e2e_i8_input` (the end-to-end loop with input the
caller has quantised), `e2e.h2d_ceiling_gbs` (plain pinned copies of the same bytes, all ranks at once), `c1_batch1`
(the module at batch 1), `cpu_baseline_omp4`, `secondary` (MobileNet-v2 batch 32, the YOLOv4-style graph batch 8, the
3x3 op sweep; rank 0) and, at every N, `calibration` (the calibration pass on 256 images per GPU and the check that N ranks
together reproduce one rank's histograms and thresholds).
`--workload mobilenet_v2|yolov4|resnet50_bf16|conv_sweep|calibration|tuner` measure the other graphs on their own;
`--impl reference` times the CPU path of the same workload (rank 0 only under torchrun).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


PDL_OPTION = None  # --pdl: the interpreter's "pdl" option for every module of the run (None: the library's default)


def new_module(device):
    """A module on `device`, with the options given on the command line."""
    from tpu_compiler_b200 import module
    m = module(device)
    if PDL_OPTION is not None:
        m.set_option("pdl", PDL_OPTION)
    return m


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop_evt = threading.Event()

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop_evt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q,
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                f = [s.strip() for s in out.strip().split(",")]
                self.samples.append(float(f[0]))
                self.max_mhz = float(f[1])
                for n, v in zip(names, f[2:]):
                    if v.lower().startswith("active"):
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop_evt.wait(0.2)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=6)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def cpu_path_images_per_s(model_b1, images, warmup=1, threads=None):
    """Times the reference-faithful CPU path (oracle/cpu_path.py: oneDNN fp32 convolution on integer-valued
    floats, as the reference does with MKL-DNN, + the reference's own requantisation code) on `images` batch-1
    passes with `threads` host threads (default: all), after checking one image bit for bit against the oracle.
    A thread count other than the default only takes full effect when OMP_NUM_THREADS was set to it before the
    OpenMP runtimes loaded (see cpu_path_in_subprocess)."""
    import torch
    from oracle import cpu_path, graph_runner
    torch.set_num_threads(threads or os.cpu_count() or 1)
    rng = np.random.default_rng(4242)
    x = rng.uniform(-1, 1, (1, 3, 224, 224)).astype(np.float32)
    out = model_b1.outputs[0]
    ref = graph_runner.run(model_b1.text, model_b1.weights, {"data": x})[out]
    got = cpu_path.run(model_b1.text, model_b1.weights, {"data": x})[out]
    if not np.array_equal(ref, got):
        raise RuntimeError("CPU baseline path disagrees with the oracle")
    for _ in range(warmup):
        cpu_path.run(model_b1.text, model_b1.weights, {"data": x})
    t0 = time.perf_counter()
    for _ in range(images):
        x = rng.uniform(-1, 1, (1, 3, 224, 224)).astype(np.float32)
        cpu_path.run(model_b1.text, model_b1.weights, {"data": x})
    dt = time.perf_counter() - t0
    return images / dt, dt


def cpu_path_in_subprocess(threads, images):
    """The CPU arm at a fixed OpenMP thread count (the reference's regression scripts run at OMP_NUM_THREADS=4,
    regression/run_regression.sh:14): a fresh process, so that the variable is seen by every OpenMP runtime it loads."""
    env = dict(os.environ, OMP_NUM_THREADS=str(threads))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    out = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", str(images),
                          "--warmup", "1", "--cpu-threads", str(threads)], capture_output=True, text=True, env=env,
                         timeout=900)
    for line in out.stdout.splitlines():
        if line.startswith("{"):
            return json.loads(line)
    raise RuntimeError("the CPU arm printed no result: " + out.stderr[-400:])


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU path for the same workload. The reference binary needs
    MLIR/LLVM, MKL-DNN 1.0.2 and cnpy, none of which are vendored, so the arm runs the CPU oracle
    (its restatement, pinned to the reference's own arithmetic sources) with all host threads."""
    if rank != 0:
        return
    from tpu_compiler_b200 import graphs
    model = graphs.resnet50_int8(batch=1, seed=1001)
    threads = args.cpu_threads or os.cpu_count() or 1
    ips, dt = cpu_path_images_per_s(model, args.steps, warmup=max(args.warmup, 1), threads=threads)
    line = {
        "impl": "reference", "metric": "INT8 ResNet-50 images/sec", "value": ips, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "resnet50_v1_int8_224, batch %d per GPU, whole module per step" % args.batch,
                   "sample": "each step is one batch-1 image of that workload on the host CPU"},
        "cpu_baseline": {"value": ips, "unit": "images/s", "cores": threads, "kind": "port",
                         "sample": "%d batch-1 ResNet-50 INT8 forward passes: oneDNN fp32 convolution on "
                                   "integer-valued floats + the reference's own requantisation code, %d threads"
                                   % (args.steps, threads)},
        "e2e": {"value": ips, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def calibration_record(rank, world, local_rank, dist, images_per_gpu, bs, check_images=64):
    """The calibration pass (fp32 ResNet-50 forward, running min / max, 2048-bin |x| histograms, KLD threshold
    search) over `images_per_gpu` synthetic images per GPU in batches of `bs`, every rank on its own shard,
    statistics combined by all-reduce. Wall clock through the public calibrator API, host input batches included
    (uploaded per batch, once per pass), max over ranks. Then, untimed, the rank-count check: a set of
    `check_images` images calibrated by all ranks together (each on its slice, combined by the two all-reduces)
    must give the histograms and thresholds that rank 0 gets from the whole set on its own. Every rank calls this;
    the returned record is complete on rank 0."""
    import torch
    from tpu_compiler_b200 import graphs, module
    from tpu_compiler_b200.calibration import ActivationCalibrator
    n_batches = max(images_per_gpu // bs, 1)
    model = graphs.resnet50_fp32(batch=bs)
    m = new_module(local_rank)
    m.load_text(model.text, model.weights)
    rng = np.random.default_rng(7000 + rank)
    # the input batches lie in pinned host memory, as a loader with pin_memory=True delivers them: the calibrator sends
    # such a batch from where it lies (a pageable numpy batch is first copied into a pinned buffer: 3.2 ms of host time
    # per batch of 64, three times that with eight ranks sharing the host's memory; the rank-count check below feeds
    # numpy batches, so both ways run)
    data = [torch.from_numpy(np.clip(rng.standard_normal((bs, 3, 224, 224), dtype=np.float32), -3, 3)).pin_memory()
            for _ in range(n_batches)]
    # expected_batches: the device cache of the activations (one buffer per batch) is allocated with the calibrator,
    # like its pinned upload buffers and the module itself, not inside the timed passes
    cal = ActivationCalibrator(m, lambda: iter(data), dist=dist, expected_batches=n_batches)
    m.set_tensor(cal.input_name, data[0].numpy())
    for _ in range(3):
        m.invoke()
    # untimed warm-up of the statistics path on one batch (first launches of its kernels, the device staging buffers of
    # the pipelined upload), local to the rank
    warm = ActivationCalibrator(m, lambda: iter(data[:1]), dist=None)
    for _ in range(3):
        ws = warm.find_min_max_abs()
        wh = warm.calc_histograms(ws)
        warm.find_threshold(wh, ws)
    del warm
    sampler = ClockSampler(local_rank)
    sampler.start()
    if dist is not None:
        # untimed warm-up of the two collectives the pass uses, with the shapes of the pass (NCCL prepares per message
        # size; the first [T, 2] MAX of a process cost 28 ms, later ones 0.5), then the barrier that starts the timed region
        w1 = torch.zeros((len(cal.names), 2), dtype=torch.float32, device="cuda")
        w2 = torch.zeros((len(cal.names), cal.bin_num), dtype=torch.int64, device="cuda")
        w3 = torch.zeros(1, dtype=torch.int64, device="cuda")
        for _ in range(3):
            dist.all_reduce(w1, op=dist.ReduceOp.MAX)
            dist.all_reduce(w2, op=dist.ReduceOp.SUM)
            dist.all_reduce(w3, op=dist.ReduceOp.SUM)
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    stats = cal.find_min_max_abs()
    t1 = time.perf_counter()
    hist = cal.calc_histograms(stats)
    t2 = time.perf_counter()
    thr = cal.find_threshold(hist, stats)
    torch.cuda.synchronize()
    t3 = time.perf_counter()
    parts = dict(cal.pass1_host_s)
    times = [t3 - t0, t1 - t0, t2 - t1, t3 - t2, parts["pinned_copy"], parts["wait_uploads"], parts["enqueue"],
             parts["final_sync"], parts["combine"]]
    if dist is not None:
        dist.barrier()
        tt = torch.tensor(times, dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        times = [float(v) for v in tt.tolist()]
    clocks = sampler.stop()
    fwd_ms = m.time_launches(5) / 5
    del cal, hist
    m.close()
    torch.cuda.empty_cache()

    # ---- untimed: N ranks together against rank 0 alone on the same images
    cb = 8
    small = graphs.resnet50_fp32(batch=cb)
    ms = new_module(local_rank)
    ms.load_text(small.text, small.weights)
    crng = np.random.default_rng(7777)
    cdata = [np.clip(crng.standard_normal((cb, 3, 224, 224), dtype=np.float32), -3, 3) for _ in range(check_images // cb)]
    mine = cdata[rank::world]
    both = ActivationCalibrator(ms, lambda: iter(mine), dist=dist)
    thr_n, stats_n = both.run()
    hist_n = both.histograms.cpu().numpy()
    equal = None
    if rank == 0:
        alone = ActivationCalibrator(ms, lambda: iter(cdata), dist=None)
        thr_1, stats_1 = alone.run()
        hist_1 = alone.histograms.cpu().numpy()
        equal = bool(np.array_equal(hist_n, hist_1) and all(thr_n[k] == thr_1[k] for k in thr_1) and
                     all(tuple(stats_n[k]) == tuple(stats_1[k]) for k in stats_1) and both.num_samples == alone.num_samples)
        del alone
    del both
    ms.close()
    if dist is not None:
        dist.barrier()
    images = world * n_batches * bs
    return {"value": images / times[0], "unit": "images/s", "images": images, "images_per_gpu": n_batches * bs,
            "batch": bs, "tensors": len(thr), "seconds": times[0], "input_batches": "fp32, pinned host memory",
            "phases_s": {"min_max_pass": times[1], "histogram_pass": times[2], "kld_search": times[3]},
            "min_max_pass_host_s": {"pinned_copy": times[4], "wait_uploads": times[5], "enqueue": times[6],
                                    "final_sync": times[7], "combine_and_read_back": times[8]},
            "forward_ms_per_batch": fwd_ms, "clocks": clocks,
            "collectives": "all-reduce(MAX) of packed min/max, all-reduce(SUM) of int64 histograms" if world > 1 else "none",
            "equal_to_single_rank": equal,
            "equality_check": "%d images in batches of %d: histograms, min/max and thresholds of %d rank(s) together "
                              "against rank 0 alone, exact" % (check_images, cb, world)}


def run_calibration(args, rank, world, local_rank):
    """--workload calibration: one JSON line for the calibration pass (see calibration_record)."""
    import torch
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    rec = calibration_record(rank, world, local_rank, dist, args.cal_images, args.cal_batch)
    if rank == 0:
        n_batches = max(args.cal_images // args.cal_batch, 1)
        print(json.dumps({
            "metric": "fp32 ResNet-50 calibration images/sec", "value": rec["value"], "unit": "images/s",
            "n_gpus": world, "steps": n_batches, "warmup": 3, "ms_per_step": rec["seconds"] / n_batches * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "calibration: fp32 ResNet-50, %d images per GPU in batches of %d (N(0,1) clipped to "
                                   "[-3,3]), %d tensors, min/max pass + 2048-bin histogram pass + KLD search" %
                                   (rec["images_per_gpu"], rec["batch"], rec["tensors"]),
                       "parallelism": "image shards x%d, all-reduce(MAX) of min/max, all-reduce(SUM) of histograms" % world},
            "phases_s": rec["phases_s"], "min_max_pass_host_s": rec["min_max_pass_host_s"],
            "forward_ms_per_batch": rec["forward_ms_per_batch"], "thresholds": rec["tensors"],
            "equal_to_single_rank": rec["equal_to_single_rank"], "clocks": rec["clocks"]}), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_tuner(args, local_rank):
    """--workload tuner: the threshold auto-tuner (kld_calibrator.py:113-201) on the fp32 ResNet-50 over
    `--tune-images` synthetic images with three candidate tables (KLD thresholds at 2048 / 1024 / 512 bins from the
    calibrator on the same images). Wall clock of SimpleTuner.run() through the public API on one GPU: the loop is
    serial in the ops, so more GPUs would only run replicas. Candidate evaluations per second, plus how many INT8 op
    executions the run needed against the count of the reference's loop (every candidate re-runs the graph prefix)."""
    from tpu_compiler_b200 import graphs, module
    from tpu_compiler_b200 import quantize as Q
    from tpu_compiler_b200.calibration import ActivationCalibrator
    from tpu_compiler_b200.tuner import SimpleTuner
    n = args.tune_images
    model = graphs.resnet50_fp32(batch=n)
    rng = np.random.default_rng(7100)
    images = np.clip(rng.standard_normal((n, 3, 224, 224), dtype=np.float32), -3, 3)
    m = new_module(local_rank)
    m.load_text(model.text, model.weights)
    # the candidate tables: one min / max pass, the cached activations serve all three histogram sizes
    cal = ActivationCalibrator(m, lambda: iter([images]))
    multi, stats = cal.run_multi((2048, 1024, 512))
    tables = {"bins%d" % bins: {k: float(v) for k, v in thr.items()} for bins, thr in multi.items()}
    del cal
    m.close()
    ops = Q.parse_text(model.text)
    tunable = [o["name"] for o in ops if o["type"] not in ("input", "softmax", "reshape")]
    for t in tables.values():
        t.pop("prob", None)
    sampler = ClockSampler(local_rank)
    sampler.start()
    t0 = time.perf_counter()
    tuner = SimpleTuner(model.text, model.weights, tables, stats, images, device=local_rank)
    t1 = time.perf_counter()
    best = tuner.run()
    t2 = time.perf_counter()
    clocks = sampler.stop()
    evals = sum(len(d) for d in tuner.distances.values())
    # the reference's loop runs, for the k-th op and each candidate, the k quantised ops of the prefix
    index = {o["name"]: i for i, o in enumerate(o for o in ops if o["type"] != "input")}
    ref_ops = sum((index[nm] + 1) * len(tuner.distances[nm]) for nm in tuner.distances)
    moved = sum(1 for nm in tunable if best[nm] != tables["bins2048"][nm])
    tuner.close()
    print(json.dumps({
        "metric": "auto-tuner candidate evaluations/sec (fp32 ResNet-50, %d images)" % n, "value": evals / (t2 - t1),
        "unit": "evaluations/s", "n_gpus": 1, "steps": evals, "warmup": 0, "ms_per_step": (t2 - t1) / max(evals, 1) * 1e3,
        "higher_is_better": True, "scaling": "replicas only", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "tuner: fp32 ResNet-50, %d images N(0,1) clipped to [-3,3], %d ops x 3 candidate tables" %
                               (n, len(tuner.distances))},
        "seconds": {"fp32_reference_and_store": t1 - t0, "tuning_loop": t2 - t1},
        "int8_op_executions": tuner.ops_run, "int8_op_executions_reference_loop": ref_ops,
        "candidate_modules_launched": tuner.launches, "thresholds_changed": moved, "clocks": clocks}), flush=True)


# graph builder name in tpu_compiler_b200.graphs, input resolution, input value range, default batch
WORKLOADS = {
    "resnet50": {"builder": "resnet50_int8", "res": 224, "lo": -1.0, "batch": 256,
                 "metric": "INT8 ResNet-50 images/sec", "name": "resnet50_v1_int8_224"},
    "resnet50_bf16": {"builder": "resnet50_bf16", "res": 224, "lo": -1.0, "batch": 128,
                      "metric": "BF16 ResNet-50 images/sec", "name": "resnet50_v1_bf16_224"},
    "mobilenet_v2": {"builder": "mobilenet_v2_int8", "res": 224, "lo": -1.0, "batch": 128,
                     "metric": "INT8 MobileNet-v2 images/sec", "name": "mobilenet_v2_int8_224"},
    "yolov4": {"builder": "yolov4_style_int8", "res": 416, "lo": 0.0, "batch": 16,
               "metric": "INT8+BF16 YOLOv4-style images/sec", "name": "yolov4_style_int8_bf16_416"},
}


def run_conv_sweep(args, local_rank):
    """--workload conv_sweep: the single INT8 Conv2D op sweep (3x3, stride 1, pad 1; uniform int8 operands,
    per-channel multiplier / rshift requantisation with ReLU). One JSON line with the rate of every case."""
    from tpu_compiler_b200 import graphs, module
    import ctypes as C
    from tpu_compiler_b200._lib import check, lib
    peaks = measured_peaks()
    cases = [(c, hw, n, 3, c, 1) for n in (1, 8, 32) for c, hw in ((64, 56), (128, 28), (256, 14), (512, 7))]
    if args.case:
        # c,hw,n of the sweep, optionally followed by kernel size, output channels and ReLU (0/1): other layers of the
        # benchmark graphs (e.g. 64,56,256,1,256,0 = the 1x1 expand layers of ResNet-50's second stage at batch 256)
        v = [int(x) for x in args.case.split(",")]
        c, hw, n = v[:3]
        cases = [(c, hw, n, v[3] if len(v) > 3 else 3, v[4] if len(v) > 4 else c, v[5] if len(v) > 5 else 1)]
    i8_tops = C.c_double(0.0)
    check(lib().tpucb_measure_i8_mma_peak(local_rank, 128, C.byref(i8_tops)))
    rows = []
    for c, hw, n, k, co, relu in cases:
        model = graphs.single_conv_i8(n=n, c_in=c, c_out=co, hw=hw, k=k, stride=1, pad=k // 2, relu=bool(relu),
                                      seed=2000 + c + n)
        m = new_module(local_rank)
        m.load_text(model.text, model.weights)
        m.set_tensor("x", model.meta["x"])
        for _ in range(max(args.warmup, 3)):
            m.invoke()
        ms = m.time_launches(args.steps) / args.steps
        ops = 2.0 * n * hw * hw * c * co * k * k
        row = {"c": c, "hw": hw, "n": n, "us": ms * 1e3, "tops": ops / (ms * 1e-3) / 1e12}
        if (k, co, relu) != (3, c, 1):
            row.update({"k": k, "c_out": co, "relu": relu, "outputs_per_s": n * hw * hw * co / (ms * 1e-3)})
        rows.append(row)
        m.close()
    best = max(r["tops"] for r in rows)
    print(json.dumps({
        "metric": "INT8 Conv2D 3x3 op sweep", "value": best, "unit": "TOP/s (best case)", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "higher_is_better": True, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "single INT8 Conv2D op, 3x3 stride 1 pad 1, C_in = C_out = c, H = W = hw, batch n; "
                               "operands fit in L2 (back-to-back launches of one op)"},
        "cases": rows,
        "roofline": {"bound": "tensor", "achieved": best, "peak": 2.0 * peaks["bf16_tflops_sustained"], "unit": "TOP/s",
                     "frac": best / (2.0 * peaks["bf16_tflops_sustained"]), "i8_mma_peak_measured": i8_tops.value}}),
        flush=True)


def h2d_ceiling(nbytes, local_rank, barrier, max_over_ranks, world, reps=10):
    """GB/s (all ranks together) of `reps` pinned host-to-device copies of `nbytes` each per rank, CUDA events."""
    import torch
    torch.cuda.set_device(local_rank)
    host = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    dev = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for _ in range(3):
            dev.copy_(host, non_blocking=True)
        st.synchronize()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(st)
        for _ in range(reps):
            dev.copy_(host, non_blocking=True)
        b.record(st)
        b.synchronize()
    ms = max_over_ranks(a.elapsed_time(b))
    barrier()
    del host, dev
    torch.cuda.empty_cache()
    return world * nbytes * reps / (ms * 1e-3) / 1e9


def graph_replay_rate(model, local_rank, inputs, steps, warmup=5):
    """(ms per launch, kernels per launch) of a module under CUDA-graph replay, inputs resident."""
    from tpu_compiler_b200 import module
    m = new_module(local_rank)
    m.load_text(model.text, model.weights)
    for k, v in inputs.items():
        m.set_tensor(k, v)
    for _ in range(warmup):
        m.invoke()
    ms = m.time_launches(steps) / steps
    kernels = m.kernel_count()
    m.close()
    return ms, kernels


def batch1_record(local_rank, steps=200):
    """BASELINE configuration C1 as written: ResNet-50 INT8, batch 1. Graph replay with the input resident, and the
    synchronous public call sequence (set_tensor, invoke, get_tensor) per image."""
    from tpu_compiler_b200 import graphs, module
    model = graphs.resnet50_int8(batch=1, seed=1001)
    x = np.random.default_rng(4243).uniform(-1, 1, (1, 3, 224, 224)).astype(np.float32)
    m = new_module(local_rank)
    m.load_text(model.text, model.weights)
    m.set_tensor("data", x)
    for _ in range(10):
        m.invoke()
    ms = m.time_launches(steps) / steps
    t0 = time.perf_counter()
    for _ in range(steps):
        m.set_tensor("data", x)
        m.invoke()
        m.get_tensor(model.outputs[0])
    e2e_ms = (time.perf_counter() - t0) / steps * 1e3
    kernels = m.kernel_count()
    m.close()
    return {"workload": "resnet50_v1_int8_224, batch 1 (configuration C1 as written), CUDA-graph replay",
            "ms_per_launch": ms, "value": 1e3 / ms, "unit": "images/s", "kernels_per_launch": kernels,
            "e2e_ms_per_image": e2e_ms, "e2e_value": 1e3 / e2e_ms,
            "e2e_note": "set_tensor + invoke + get_tensor per image, synchronous, pageable host arrays"}


def secondary_records(local_rank, steps=20):
    """The other BASELINE configurations on one GPU (device-resident CUDA-graph replay; no CPU arm for them):
    MobileNet-v2 batch 32, the YOLOv4-style graph batch 8 at 416 x 416, and the twelve points of the 3x3 op sweep."""
    from tpu_compiler_b200 import graphs
    out = {}
    for key, builder, batch, res, lo in (("mobilenet_v2_int8_b32_224", graphs.mobilenet_v2_int8, 32, 224, -1.0),
                                         ("yolov4_style_int8_bf16_b8_416", graphs.yolov4_style_int8, 8, 416, 0.0)):
        model = builder(batch=batch, res=res, simulate=False)
        x = np.random.default_rng(5).uniform(lo, 1, (batch, 3, res, res)).astype(np.float32)
        ms, kernels = graph_replay_rate(model, local_rank, {"data": x}, steps)
        out[key] = {"value": batch / (ms * 1e-3), "unit": "images/s", "ms_per_step": ms, "batch": batch,
                    "kernels_per_step": kernels}
    sweep = []
    for n in (1, 8, 32):
        for c, hw in ((64, 56), (128, 28), (256, 14), (512, 7)):
            model = graphs.single_conv_i8(n=n, c_in=c, c_out=c, hw=hw, k=3, stride=1, pad=1, relu=True, seed=2000 + c + n)
            ms, _ = graph_replay_rate(model, local_rank, {"x": model.meta["x"]}, 50, warmup=5)
            sweep.append({"n": n, "c": c, "hw": hw, "us": ms * 1e3, "tops": 2.0 * n * hw * hw * c * c * 9 / (ms * 1e-3) / 1e12})
    out["conv_sweep_3x3"] = {"unit": "TOP/s", "note": "back-to-back launches of one op: operands stay in L2",
                             "cases": sweep}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=None, help="images per GPU per step (default: 256 for resnet50)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-images", type=int, default=100, help="images of the bounded CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-threads", type=int, default=0, help="--impl reference: host threads (default: all)")
    ap.add_argument("--no-extras", action="store_true", help="headline only: skip the batch-1 configuration, the "
                    "secondary graphs, the link ceiling and the calibration sub-record")
    ap.add_argument("--pdl", type=int, default=None, choices=(0, 1, 2),
                    help="programmatic dependent launch: 0 off, 1 the convolution kernels (the library's default), 2 every kernel")
    ap.add_argument("--case", default=None, help="conv_sweep only: one case as c,hw,n[,k[,c_out[,relu]]]")
    ap.add_argument("--cal-images", type=int, default=512, help="calibration workload: images per GPU")
    ap.add_argument("--cal-batch", type=int, default=64, help="calibration workload: images per batch (64 in the "
                    "configuration; smaller values are for profiler captures)")
    ap.add_argument("--tune-images", type=int, default=16, help="tuner workload: images held on the GPU")
    ap.add_argument("--workload", default="resnet50", choices=sorted(WORKLOADS) + ["conv_sweep", "calibration", "tuner"],
                    help="resnet50 is the headline configuration; the others are the secondary graphs "
                         "(their lines carry no cpu_baseline)")
    args = ap.parse_args()
    global PDL_OPTION
    PDL_OPTION = args.pdl
    if args.cpu_threads:
        os.environ["OMP_NUM_THREADS"] = str(args.cpu_threads)   # before any OpenMP runtime loads
    if args.workload == "conv_sweep":
        if args.impl == "ours" and int(os.environ.get("RANK", "0")) == 0:
            run_conv_sweep(args, int(os.environ.get("LOCAL_RANK", "0")))
        return
    if args.workload == "tuner":
        if args.impl == "ours" and int(os.environ.get("RANK", "0")) == 0:
            run_tuner(args, int(os.environ.get("LOCAL_RANK", "0")))
        return
    if args.workload == "calibration":
        if args.impl == "ours":
            run_calibration(args, int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
                            int(os.environ.get("LOCAL_RANK", "0")))
        return
    wl = WORKLOADS[args.workload]
    if args.batch is None:
        args.batch = wl["batch"]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if args.workload != "resnet50":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the CPU reference arm covers the resnet50 workload only"}))
            return
        run_reference(args, rank, world)
        return

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod

    from tpu_compiler_b200 import graphs, module
    from tpu_compiler_b200._lib import check, lib
    import ctypes as C

    B = args.batch
    if args.workload == "resnet50":
        model = graphs.resnet50_int8(batch=B, seed=1001)
    else:
        model = getattr(graphs, wl["builder"])(batch=B, simulate=False)
    m = new_module(local_rank)
    m.load_text(model.text, model.weights)

    # pinned host buffers: this rank's image shard and its results (every module output)
    in_numel = B * 3 * wl["res"] * wl["res"]
    shapes = {i["name"]: i["shape"] for i in m.op_info}
    L = lib()
    hin = C.c_void_p()
    check(L.tpucb_host_alloc(C.byref(hin), in_numel * 4))
    houts = []
    for name in model.outputs:
        numel = int(np.prod(shapes[name]))
        h = C.c_void_p()
        check(L.tpucb_host_alloc(C.byref(h), numel * 4))
        houts.append((name, h, numel))
    out_numel = sum(n for _, _, n in houts)
    src = np.ctypeslib.as_array(C.cast(hin, C.POINTER(C.c_float)), shape=(in_numel,))
    rng = np.random.default_rng(9000 + rank)
    src[:] = rng.uniform(wl["lo"], 1, in_numel).astype(np.float32)

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v):
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- warm-up (also instantiates the CUDA graph)
    m.set_tensor_ptr("data", hin, in_numel)
    for _ in range(max(args.warmup, 3)):
        m.invoke()

    sampler = ClockSampler(local_rank)
    sampler.start()

    # ---- device-resident: K launches, inputs already in HBM
    barrier()
    m.sync()
    ms = m.time_launches(args.steps)
    m.sync()
    barrier()
    ms = max_over_ranks(ms)
    value = world * B * args.steps / (ms * 1e-3)

    # ---- end to end through the public API with host buffers: every step uploads its own input
    # batch from pinned memory and reads its own result back; the upload of step i+1 is issued
    # (set_tensor_async, second stream) while step i is still executing.
    hin2 = C.c_void_p()
    check(L.tpucb_host_alloc(C.byref(hin2), in_numel * 4))
    src2 = np.ctypeslib.as_array(C.cast(hin2, C.POINTER(C.c_float)), shape=(in_numel,))
    src2[:] = src[::-1]
    bufs = [hin, hin2]
    # untimed warm-up of the pipelined path (allocates the two device staging buffers)
    for i in range(max(args.warmup, 3)):
        m.set_tensor_async("data", bufs[i & 1], in_numel)
        m.launch()
        for name, h, numel in houts:
            m.get_tensor_into(name, h, numel)
    barrier()
    m.sync()
    t0 = time.perf_counter()
    m.set_tensor_async("data", bufs[0], in_numel)
    for i in range(args.steps):
        m.launch()
        if i + 1 < args.steps:
            m.set_tensor_async("data", bufs[(i + 1) & 1], in_numel)
        for name, h, numel in houts:
            m.get_tensor_into(name, h, numel)
    m.sync()
    e2e_s = time.perf_counter() - t0
    barrier()
    e2e_s = max_over_ranks(e2e_s)
    e2e = world * B * args.steps / e2e_s
    clocks = sampler.stop()

    # ---- the same end-to-end loop with the input quantised by the caller: int8 instead of the fp32 container, a
    # quarter of the bytes over the host link (tpucb_interp_set_tensor_async_i8; the module's input quant op is skipped)
    e2e_i8 = None
    quant_name = next((o["name"] for o in m.op_info if o["type"] == "quant" and o["dtype"] == "INT8"), None)
    if not args.no_extras and args.workload == "resnet50" and quant_name:
        qb = []
        for k in range(2):
            h = C.c_void_p()
            check(L.tpucb_host_alloc_write_combined(C.byref(h), in_numel))
            q8 = np.random.default_rng(9100 + rank + k).integers(-128, 128, in_numel, dtype=np.int8)
            C.memmove(h, q8.ctypes.data, in_numel)
            qb.append(h)
        for i in range(3):
            m.set_tensor_async_i8(quant_name, qb[i & 1], in_numel)
            m.launch()
            for name, h, numel in houts:
                m.get_tensor_into(name, h, numel)
        barrier()
        m.sync()
        t0 = time.perf_counter()
        m.set_tensor_async_i8(quant_name, qb[0], in_numel)
        for i in range(args.steps):
            m.launch()
            if i + 1 < args.steps:
                m.set_tensor_async_i8(quant_name, qb[(i + 1) & 1], in_numel)
            for name, h, numel in houts:
                m.get_tensor_into(name, h, numel)
        m.sync()
        i8_s = max_over_ranks(time.perf_counter() - t0)
        barrier()
        e2e_i8 = {"value": world * B * args.steps / i8_s, "unit": "images/s", "h2d_bytes_per_step": in_numel,
                  "d2h_bytes_per_step": out_numel * 4,
                  "note": "input already quantised to int8 by the caller (one byte per value), uploaded with "
                          "tpucb_interp_set_tensor_async_i8 into the result of the input quant op, which is skipped"}
        m.set_tensor_ptr("data", hin, in_numel)   # the fp32 way again: the quant op runs in what follows
        m.invoke()
        for h in qb:
            check(L.tpucb_host_free(h))

    # ---- the host link's own ceiling for this step's upload: the same bytes from pinned memory with plain
    # asynchronous copies and nothing else, all ranks at once (untimed for the headline)
    h2d = None
    if not args.no_extras:
        h2d = h2d_ceiling(in_numel * 4, local_rank, barrier, max_over_ranks, world)

    line = None
    if rank == 0:
        # ---- per-kernel roofline from an eager pass with CUDA events around every op
        peaks = measured_peaks()
        m.set_option("cuda_graph", 0)
        m.invoke()
        reps = 5
        acc = np.zeros(len(m.op_info))
        for _ in range(reps):
            acc += np.array(m.profile())
        per_op_ms = acc / reps
        m.set_option("cuda_graph", 1)
        conv_ops = conv_ms = conv_bytes = 0.0
        n_conv = 0
        other_bytes = other_ms = 0.0
        for info, t in zip(m.op_info, per_op_ms):
            if info["bound"] == "tensor":
                conv_ops += info["ops"]
                conv_bytes += info["bytes"]
                conv_ms += t
                n_conv += 1
            elif info["type"] != "input":
                other_bytes += info["bytes"]
                other_ms += t
        int8_peak = 2.0 * peaks["bf16_tflops_sustained"]
        achieved = conv_ops / (conv_ms * 1e-3) / 1e12
        i8_tops = C.c_double(0.0)  # this library's own tcgen05 kind::i8 issue microbenchmark, live on this GPU
        check(L.tpucb_measure_i8_mma_peak(local_rank, 128, C.byref(i8_tops)))
        # DRAM bytes per conv launch from the committed ncu capture of one step at batch 64
        # (profiles/resnet50_int8_b64_dram_traffic.md: 10.09 MB read per launch, writes still dirty in L2 when the
        # kernel ends), scaled by the images per launch; null for the workloads that have no capture.
        # DRAM traffic per launch: not captured in this run (a profiler capture of this size is out of bounds). The read
        # side is the ncu figure of a whole step at batch 64 (10.09 MB of dram__bytes_read per tensor-core launch)
        # scaled by the images per launch; ncu attributes no write-back to these kernels (their outputs are still
        # dirty in L2 when they end), so the write side is the algorithmic output bytes.
        traffic = None
        if args.workload == "resnet50":
            out_bytes = sum(float(np.prod(i["shape"])) for i in m.op_info if i["bound"] == "tensor") / max(n_conv, 1)
            traffic = 10.09e6 * B / 64.0 + out_bytes
        if args.workload == "resnet50_bf16":
            # BF16 graph: the same pipeline with kind::f16 MMAs; the denominator is the measured bf16 rate itself
            roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                        "frac": achieved / peaks["bf16_tflops_sustained"], "traffic": None,
                        "kernel": "conv_gemm_bf16_kernel (tcgen05 kind::f16 implicit GEMM on BF16 operands, %d launches "
                                  "per step)" % n_conv,
                        "peak_source": "bf16_tflops_sustained of %s peaks" % peaks["source"],
                        "avg_launch_us": conv_ms * 1e3 / max(n_conv, 1)}
        else:
            roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
                        "frac": achieved / int8_peak,
                        "peak_burst": 2.0 * peaks["bf16_tflops"], "frac_burst": achieved / (2.0 * peaks["bf16_tflops"]),
                        "traffic": traffic,
                        "traffic_note": "per launch: DRAM reads of an ncu capture of one step at batch 64 scaled by "
                                        "batch / 64, plus the algorithmic output bytes (ncu attributes no write-back to "
                                        "the kernel); not captured in this run. Algorithmic bytes per launch: %.1f MB"
                                        % (conv_bytes / max(n_conv, 1) / 1e6),
                        "kernel": "conv_gemm_i8_act_kernel<1> / <10> and conv_stem_i8_kernel: the tcgen05 kind::i8 implicit GEMM of "
                                  "conv_gemm_i8.cuh in its ReLU and plain instantiations, %d launches per step" % n_conv,
                        "peak_source": "2 x bf16_tflops_sustained of %s peaks (no INT8 figure is measured; the 8-bit "
                                       "rate of the same tensor pipe is twice the 16-bit rate)" % peaks["source"],
                        "avg_launch_us": conv_ms * 1e3 / max(n_conv, 1),
                        "i8_mma_peak_measured": i8_tops.value,
                        "frac_of_i8_mma_peak": achieved / i8_tops.value if i8_tops.value > 0 else None,
                        "hbm_view": {"achieved_gbs": conv_bytes / (conv_ms * 1e-3) / 1e9, "peak_gbs": peaks["hbm_gbs"],
                                     "frac": conv_bytes / (conv_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}}
        mem_kernels = {"achieved_gbs": other_bytes / (other_ms * 1e-3) / 1e9 if other_ms > 0 else None,
                       "peak_gbs": peaks["hbm_gbs"], "ms_per_step": other_ms}
        cpu = None
        if not args.no_cpu_baseline and world == 1 and args.workload == "resnet50":
            model_b1 = graphs.resnet50_int8(batch=1, seed=1001)
            ips, dt = cpu_path_images_per_s(model_b1, args.cpu_images)
            cpu = {"value": ips, "unit": "images/s", "cores": os.cpu_count() or 1, "kind": "port",
                   "sample": "%d batch-1 ResNet-50 INT8 forward passes (oneDNN fp32 convolution on integer-valued "
                             "floats + the reference's own requantisation code, checked against the oracle) in %.1f s"
                             % (args.cpu_images, dt)}
        cpu4 = None
        if cpu is not None and not args.no_extras:
            try:
                r4 = cpu_path_in_subprocess(4, max(args.cpu_images // 4, 8))
                cpu4 = {"value": r4["value"], "unit": "images/s", "cores": 4, "kind": "port",
                        "sample": "the same path in a fresh process with OMP_NUM_THREADS=4, the thread count of the "
                                  "reference's regression scripts: " + r4["cpu_baseline"]["sample"]}
            except Exception as e:   # the all-threads figure above stands on its own
                cpu4 = {"unavailable": str(e)[:200]}
        act_bytes = sum(i["bytes"] for i in m.op_info)
        line = {
            "metric": wl["metric"], "value": value, "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if args.workload == "resnet50_bf16" else "int8", "data": "synthetic",
            "config": {"workload": "%s, batch %d per GPU, whole module per step" % (wl["name"], B),
                       "global_batch": B * world, "parallelism": "replicas x%d (image shards, no data-path collective)" % world,
                       "l2": "per-step working set %.0f MB exceeds the 126 MB L2" % (act_bytes / 1e6),
                       "cuda_graph": True},
            "e2e": {"value": e2e, "unit": "images/s", "h2d_bytes_per_step": in_numel * 4, "d2h_bytes_per_step": out_numel * 4,
                    "h2d_ceiling_gbs": h2d,
                    "h2d_link_frac": (e2e * in_numel * 4 / B / 1e9 / h2d) if h2d else None,
                    "h2d_note": "ceiling: the same bytes per rank as plain pinned asynchronous copies, all ranks at "
                                "once, CUDA events; link_frac = the end-to-end run's upload rate over it"},
            "e2e_i8_input": e2e_i8,
            "gpu_launches": m.kernel_count() * args.steps,
            "clocks": clocks,
            "roofline": roofline,
            "memory_bound_kernels": mem_kernels,
            "cpu_baseline": cpu,
            "cpu_baseline_omp4": cpu4,
        }
    check(L.tpucb_host_free(hin))
    check(L.tpucb_host_free(hin2))
    for _, h, _ in houts:
        check(L.tpucb_host_free(h))
    m.close()
    if not args.no_extras and args.workload == "resnet50":
        if line is not None and world == 1:
            line["c1_batch1"] = batch1_record(local_rank)
            line["secondary"] = secondary_records(local_rank)
        # the calibration half of the path (the only part with collectives), at every N: all ranks take part
        import torch
        torch.cuda.empty_cache()
        rec = calibration_record(rank, world, local_rank, dist, 256, 64)
        if line is not None:
            line["calibration"] = rec
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
