"""GPU parity of the calibration path: fp32 forward statistics (min / max / abs-max, 2048-bin
histograms) and the KLD threshold search against the reference rule run on the CPU (numpy as
in kld_calibrator.py, the oracle's restatement of calibration_math.cpp)."""
import numpy as np
import pytest

import oracle
from oracle import graph_runner
from tpu_compiler_b200 import graphs

pytestmark = pytest.mark.gpu


def small_fp32_model(batch):
    rng = np.random.default_rng(9)
    b = graphs.GraphBuilder(9, simulate=False)
    b.op("input", "data", [], (batch, 3, 24, 24), "FP32")
    b.weight("w1", rng.normal(0, 0.3, (20, 3, 3, 3))), b.weight("b1", rng.normal(0, 0.1, 20))
    b.op("conv_2d", "c1", ["data", "w1", "b1"], (batch, 20, 24, 24), "FP32", kh=3, kw=3, pt=1, pb=1, pl=1, pr=1,
         do_relu=1, with_bias=1)
    b.op("pool_max_2d", "p1", ["c1"], (batch, 20, 12, 12), "FP32", kh=2, kw=2, sh=2, sw=2)
    b.weight("w2", rng.normal(0, 0.2, (33, 20, 1, 1))), b.weight("b2", rng.normal(0, 0.1, 33))
    b.op("conv_2d", "c2", ["p1", "w2", "b2"], (batch, 33, 12, 12), "FP32", kh=1, kw=1, do_relu=0, with_bias=1)
    b.op("conv_2d", "dead", ["p1", "wz", None], (batch, 4, 12, 12), "FP32", kh=1, kw=1, do_relu=1, with_bias=0)
    b.weight("wz", np.zeros((4, 20, 1, 1)))
    return graphs.Model(b.text(), b.weights, ["data"], ["c2"])


def test_statistics_and_thresholds_match_cpu_rule():
    from tpu_compiler_b200 import module
    from tpu_compiler_b200.calibration import ActivationCalibrator
    B, nb = 4, 3
    model = small_fp32_model(B)
    rng = np.random.default_rng(77)
    data = [np.clip(rng.normal(0, 1, (B, 3, 24, 24)), -3, 3).astype(np.float32) for _ in range(nb)]
    m = module(0)
    m.load_text(model.text, model.weights)
    cal = ActivationCalibrator(m, lambda: iter(data))
    thr, stats = cal.run()
    hist_gpu = cal.histograms.cpu().numpy()

    # CPU: activations from the oracle forward, statistics exactly as kld_calibrator.py computes them.
    acts = [graph_runner.run(model.text, model.weights, {"data": d}) for d in data]
    # the GPU forward differs from the CPU forward in the last bits of fp32 (accumulation order), so
    # statistics are compared on the GPU's own activations as well: fetch them once more
    for t, name in enumerate(cal.names):
        ref_all = np.concatenate([a[name].reshape(-1) for a in acts])
        mn, mx, ab = stats[name]
        if name == "dead":
            assert (mn, mx, ab) == (np.float32(-1e-5), np.float32(1e-5), np.float32(1e-5))
            continue
        assert abs(mn - ref_all.min()) <= 1e-4 * max(1, abs(ref_all.min()))
        assert abs(mx - ref_all.max()) <= 1e-4 * max(1, abs(ref_all.max()))
    # exact check of the statistics kernels: recompute from the activations the GPU itself produced
    got_acts = {n: [] for n in cal.names}
    for d in data:
        m.set_tensor("data", d)
        m.invoke()
        for n in cal.names:
            got_acts[n].append(m.get_tensor(n).reshape(-1))
    for t, name in enumerate(cal.names):
        x = np.concatenate(got_acts[name])
        mn, mx, ab = stats[name]
        if name == "dead":
            continue
        assert mn == x.min() and mx == x.max() and ab == max(abs(x.min()), abs(x.max()))
        tt = np.abs(x)
        tt = tt[tt != 0]
        width = ab / (2048 - 1)
        ref_hist, _ = np.histogram(np.floor(tt / width + 0.5), bins=2048, range=(0, 2047))
        assert np.array_equal(hist_gpu[t], ref_hist.astype(np.int64)), name
        assert thr[name] == oracle.kld_threshold(ref_hist.astype(np.int32), float(width)), name
    m.close()


def test_kld_kernel_matches_golden(golden_dir):
    """The device KLD search reproduces the reference's own kl_diversity_hist on the golden histograms."""
    import ctypes as C
    import os
    import torch
    from tpu_compiler_b200 import module
    from tpu_compiler_b200._lib import check, lib
    g = np.load(os.path.join(golden_dir, "kld.npz"))
    model = graphs.single_conv_i8(1, 16, 16, 4, 1, 1, 0, seed=1)
    m = module(0)
    m.load_text(model.text, model.weights)
    hist = torch.tensor(g["hist"].astype(np.int64), device="cuda")
    widths = np.ascontiguousarray(g["width"], np.float32)
    thr = np.zeros(len(widths), np.float32)
    torch.cuda.synchronize()
    fp = C.POINTER(C.c_float)
    check(lib().tpucb_calib_kld(m._h, C.c_void_p(hist.data_ptr()), widths.ctypes.data_as(fp), len(widths), 2048,
                                thr.ctypes.data_as(fp)))
    assert np.array_equal(thr, g["threshold"])
    m.close()


def test_resnet50_fp32_calibration_runs_and_matches_cpu_rule_on_sampled_tensors():
    """The calibration configuration's graph (fp32 ResNet-50, N(0,1) images clipped to [-3, 3]) at a small
    image count: thresholds of a few tensors recomputed on the CPU from the GPU's own activations."""
    from tpu_compiler_b200 import module
    from tpu_compiler_b200.calibration import ActivationCalibrator
    B, nb = 4, 2
    model = graphs.resnet50_fp32(batch=B, seed=5001)
    rng = np.random.default_rng(5001)
    data = [np.clip(rng.normal(0, 1, (B, 3, 224, 224)), -3, 3).astype(np.float32) for _ in range(nb)]
    m = module(0)
    m.load_text(model.text, model.weights)
    cal = ActivationCalibrator(m, lambda: iter(data))
    thr, stats = cal.run()
    assert len(cal.names) == 74 and cal.num_samples == B * nb
    hist_gpu = cal.histograms.cpu().numpy()
    sample = ["data", "conv1", "res2a", "res3b_branch2b", "res4f", "pool5", "fc1000", "prob"]
    acts = {n: [] for n in sample}
    for d in data:
        m.set_tensor("data", d)
        m.invoke()
        for n in sample:
            acts[n].append(m.get_tensor(n).reshape(-1))
    for n in sample:
        t = cal.names.index(n)
        x = np.concatenate(acts[n])
        mn, mx, ab = stats[n]
        assert mn == x.min() and mx == x.max()
        tt = np.abs(x)
        tt = tt[tt != 0]
        width = ab / (2048 - 1)
        ref_hist, _ = np.histogram(np.floor(tt / width + 0.5), bins=2048, range=(0, 2047))
        assert np.array_equal(hist_gpu[t], ref_hist.astype(np.int64)), n
        assert thr[n] == oracle.kld_threshold(ref_hist.astype(np.int32), float(width)), n
    # the fp32 forward itself: one image against the oracle, 1e-4 of each tensor's range
    ref = graph_runner.run(model.text, model.weights, {"data": data[0]})
    m.set_tensor("data", data[0])
    m.invoke()
    for n in ("conv1", "res2a", "res4f", "fc1000", "prob"):
        got = m.get_tensor(n)
        err = np.abs(got - ref[n]).max() / (np.abs(ref[n]).max() + 1e-30)
        assert err < 1e-4, (n, err)
    m.close()


def test_kept_activations_give_the_same_histograms():
    """Pass 2 from the device cache of pass 1 (all batches, some batches, none) reads the same bits."""
    from tpu_compiler_b200 import module
    from tpu_compiler_b200.calibration import ActivationCalibrator
    model = small_fp32_model(4)
    rng = np.random.default_rng(78)
    data = [np.clip(rng.normal(0, 1, (4, 3, 24, 24)), -3, 3).astype(np.float32) for _ in range(3)]
    m = module(0)
    m.load_text(model.text, model.weights)
    calls = []

    def batches():
        calls.append(0)
        return iter(data)

    base = ActivationCalibrator(m, batches, keep_activations_gb=0)
    thr0, _ = base.run()
    h0 = base.histograms.cpu().numpy()
    assert len(calls) == 2   # nothing kept: the images are asked for twice
    per_batch, _ = ActivationCalibrator(m, batches)._keep_plan()
    for gb, expect_calls in ((None, 1), (1.5 * per_batch / 2 ** 30, 2)):
        del calls[:]
        cal = ActivationCalibrator(m, batches, keep_activations_gb=gb, expected_batches=3 if gb is None else None)
        thr, _ = cal.run()
        assert len(calls) == expect_calls
        assert np.array_equal(cal.histograms.cpu().numpy(), h0)
        assert {k: float(v) for k, v in thr.items()} == {k: float(v) for k, v in thr0.items()}
    m.close()


def test_pinned_batches_are_sent_from_where_they_lie():
    """Batches that already lie in page-locked memory (torch tensors, pin_memory) skip the calibrator's staging copy and
    give the same histograms and thresholds as the same values in numpy arrays."""
    import torch
    from tpu_compiler_b200 import module
    from tpu_compiler_b200.calibration import ActivationCalibrator
    model = small_fp32_model(4)
    rng = np.random.default_rng(79)
    data = [np.clip(rng.normal(0, 1, (4, 3, 24, 24)), -3, 3).astype(np.float32) for _ in range(5)]
    pinned = [torch.from_numpy(d).pin_memory() for d in data]
    m = module(0)
    m.load_text(model.text, model.weights)
    a = ActivationCalibrator(m, lambda: iter(data))
    thr_a, stats_a = a.run()
    b = ActivationCalibrator(m, lambda: iter(pinned), keep_activations_gb=0)   # both passes upload
    thr_b, stats_b = b.run()
    assert b.pass1_host_s["pinned_copy"] == 0.0   # no batch went through the staging buffers
    assert np.array_equal(a.histograms.cpu().numpy(), b.histograms.cpu().numpy())
    assert {k: float(v) for k, v in thr_a.items()} == {k: float(v) for k, v in thr_b.items()}
    assert {k: tuple(map(float, v)) for k, v in stats_a.items()} == {k: tuple(map(float, v)) for k, v in stats_b.items()}
    m.close()


def test_several_bin_counts_from_one_pass():
    """run_multi: the thresholds of three histogram sizes from one min / max pass and one activation cache equal
    those of three separate calibrations, and the images are asked for only once."""
    from tpu_compiler_b200 import module
    from tpu_compiler_b200.calibration import ActivationCalibrator
    model = small_fp32_model(4)
    rng = np.random.default_rng(79)
    data = [np.clip(rng.normal(0, 1, (4, 3, 24, 24)), -3, 3).astype(np.float32) for _ in range(3)]
    m = module(0)
    m.load_text(model.text, model.weights)
    calls = []

    def batches():
        calls.append(0)
        return iter(data)

    multi, stats = ActivationCalibrator(m, batches, expected_batches=3).run_multi((512, 2048, 1024))
    assert len(calls) == 1 and list(multi) == [512, 2048, 1024]
    for bins in (512, 1024, 2048):
        thr, st = ActivationCalibrator(m, lambda: iter(data), histogram_bin_num=bins).run()
        assert {k: float(v) for k, v in thr.items()} == {k: float(v) for k, v in multi[bins].items()}, bins
        assert {k: tuple(map(float, v)) for k, v in st.items()} == {k: tuple(map(float, v)) for k, v in stats.items()}
    m.close()


def _calib_rank(rank, world, port, q):
    import os
    import torch
    import torch.distributed as dist
    from tpu_compiler_b200 import module
    from tpu_compiler_b200.calibration import ActivationCalibrator
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    model = small_fp32_model(4)
    rng = np.random.default_rng(77)
    data = [np.clip(rng.normal(0, 1, (4, 3, 24, 24)), -3, 3).astype(np.float32) for _ in range(4)]
    m = module(rank)
    m.load_text(model.text, model.weights)
    cal = ActivationCalibrator(m, lambda: iter(data[rank::world]), dist=dist)
    thr, stats = cal.run()
    q.put((rank, {k: float(v) for k, v in thr.items()}, cal.histograms.cpu().numpy(), cal.num_samples))
    dist.barrier()
    m.close()
    dist.destroy_process_group()


def test_two_gpu_calibration_equals_single_gpu():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from tpu_compiler_b200 import module
    from tpu_compiler_b200.calibration import ActivationCalibrator
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_calib_rank, args=(r, 2, 29733, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    model = small_fp32_model(4)
    rng = np.random.default_rng(77)
    data = [np.clip(rng.normal(0, 1, (4, 3, 24, 24)), -3, 3).astype(np.float32) for _ in range(4)]
    m = module(0)
    m.load_text(model.text, model.weights)
    cal = ActivationCalibrator(m, lambda: iter(data))
    thr, _ = cal.run()
    hist = cal.histograms.cpu().numpy()
    for rank, thr_r, hist_r, n in results:
        assert n == 16
        assert np.array_equal(hist_r, hist)
        assert thr_r == {k: float(v) for k, v in thr.items()}
    m.close()


def test_histogram_bins_at_the_rounding_boundaries():
    """The all-tensor histogram kernel forms |x| / width from a reciprocal taken once per tensor and fused multiply-adds
    instead of one division per value. The bin index floor(|x| / width + 0.5) must still be the one an IEEE fp32
    division gives (numpy, as kld_calibrator.py:31-43 computes it): checked on the values where a quotient off by one
    unit in the last place changes the bin -- the fp32 neighbours of every (k + 0.5) * width -- for widths with awkward
    mantissas, plus random values, subnormals and values beyond abs_max."""
    import ctypes as C
    import torch
    from tpu_compiler_b200 import module
    from tpu_compiler_b200._lib import check, lib
    bins = 2048
    rng = np.random.default_rng(2024)
    abs_maxes = [np.float32(1.0), np.float32(3.0), np.float32(2047.0), np.float32(1e-5), np.float32(6.25e4),
                 np.nextafter(np.float32(2.0), np.float32(0)) * np.float32(2047), np.float32(0.3333333), np.float32(7.77e-3)]
    abs_maxes += [np.float32(v) for v in rng.uniform(0.01, 300.0, 8)]
    per = bins * 5 + 4096
    n = per + (-per) % 4
    m = module(0)
    m.load_text("input name=x shape=1,4,%d,1 dtype=FP32\n" % (n // 4), {})
    L = lib()
    names = (C.c_char_p * 1)(b"x")
    for am in abs_maxes:
        width = am / np.float32(bins - 1)
        edges = ((np.arange(bins, dtype=np.float64) + 0.5) * float(width)).astype(np.float32)
        vals = [edges]
        for _ in range(2):
            vals.append(np.nextafter(vals[-1], np.float32(np.inf)))
        lo = edges
        for _ in range(2):
            lo = np.nextafter(lo, np.float32(0))
            vals.append(lo)
        extra = rng.uniform(0, float(am) * 1.01, 4096 - 8).astype(np.float32)
        tail = np.array([0.0, 1e-42, -1e-40, float(am), -float(am), float(am) * 4, 1e38, -3e38], np.float32)
        x = np.concatenate(vals + [extra, tail, np.zeros(n - per, np.float32)])
        x[::3] *= -1
        m.set_tensor("x", x.reshape(1, 4, n // 4, 1))
        hist = torch.zeros((1, bins), dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        amax = (C.c_float * 1)(float(am))
        check(L.tpucb_calib_hist_all(m._h, names, 1, None, amax, bins, C.c_void_p(hist.data_ptr())))
        m.sync()
        t = np.abs(x)
        t = t[t != 0]
        with np.errstate(over="ignore"):
            idx = np.floor(t / width + np.float32(0.5))
        ref, _ = np.histogram(idx, bins=bins, range=(0, bins - 1))
        assert np.array_equal(hist.cpu().numpy()[0], ref.astype(np.int64)), float(am)
    m.close()
