"""The allocation-free KLD entry point (tpucb_calib_kld_static) against the regular one.

Some hosts of this library may not allocate device memory once they are running (a calibration
service with a fixed device-memory budget, a worker that must not trigger the device-wide
synchronisation of cudaMalloc / cudaFree). For them the KLD threshold search exists in a form
whose scratch lives in a fixed array inside the library. This test calls it through the C ABI
twice in a row -- the second time with different histograms, so stale scratch contents from the
first call would show -- and requires the same thresholds, bit for bit, as tpucb_calib_kld;
a second test ties it to the reference directly through the golden histograms and thresholds
that the reference's own kl_diversity_hist produced (tests/golden/kld.npz).
The file name sorts last so that a run that stops at the first failure has already run every
other test."""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _hists(seed, count, bins):
    rng = np.random.default_rng(seed)
    out, widths = [], []
    for k in range(count):
        n = int(rng.integers(20000, 200000))
        data = np.abs(rng.normal(0, 1 + 0.3 * k, n)) if k % 2 == 0 else np.abs(rng.laplace(0, 1, n))
        data = data.astype(np.float32)
        width = np.float32(data.max()) / np.float32(bins - 1)
        h, _ = np.histogram(np.floor(data[data != 0] / width + np.float32(0.5)), bins=bins, range=(0, bins - 1))
        out.append(h.astype(np.int64))
        widths.append(width)
    return np.stack(out), np.array(widths, np.float32)


def test_kld_static_matches_allocating_entry_point_twice():
    import torch
    from tpu_compiler_b200 import graphs, module
    from tpu_compiler_b200._lib import check, lib
    L = lib()
    fp = C.POINTER(C.c_float)
    model = graphs.single_conv_i8(1, 16, 16, 4, 1, 1, 0, seed=1)
    m = module(0)          # the regular entry point runs on an interpreter's stream
    m.load_text(model.text, model.weights)
    for call, (seed, count, bins) in enumerate([(11, 7, 2048), (12, 5, 2048), (13, 3, 1024)]):
        hist, widths = _hists(seed, count, bins)
        d_hist = torch.tensor(hist, device="cuda")
        torch.cuda.synchronize()
        ref = np.zeros(count, np.float32)
        check(L.tpucb_calib_kld(m._h, C.c_void_p(d_hist.data_ptr()), widths.ctypes.data_as(fp), count, bins,
                                ref.ctypes.data_as(fp)))
        got = np.zeros(count, np.float32)
        check(L.tpucb_calib_kld_static(0, None, C.c_void_p(d_hist.data_ptr()), widths.ctypes.data_as(fp), count,
                                       bins, got.ctypes.data_as(fp)))
        assert np.array_equal(got, ref), "call %d: %s vs %s" % (call, got, ref)
        assert np.all(got > 0)
    # sizes beyond the static scratch are refused with a clear message, nothing is launched
    too_many = 257
    widths = np.ones(too_many, np.float32)
    out = np.zeros(too_many, np.float32)
    d = torch.zeros((too_many, 128), dtype=torch.int64, device="cuda")
    rc = L.tpucb_calib_kld_static(0, None, C.c_void_p(d.data_ptr()), widths.ctypes.data_as(fp), too_many, 128,
                                  out.ctypes.data_as(fp))
    assert rc != 0 and b"outside [1, 256]" in L.tpucb_last_error()
    rc = L.tpucb_calib_kld_static(0, None, C.c_void_p(d.data_ptr()), widths.ctypes.data_as(fp), 4, 100,
                                  out.ctypes.data_as(fp))
    assert rc != 0 and b"multiple of 128" in L.tpucb_last_error()
    m.close()


def test_kld_static_matches_reference_golden(golden_dir):
    """The thresholds the reference's compiled kl_diversity_hist gave for the golden histograms."""
    import torch
    from tpu_compiler_b200._lib import check, lib
    g = np.load(os.path.join(golden_dir, "kld.npz"))
    hist = torch.tensor(g["hist"].astype(np.int64), device="cuda")
    widths = np.ascontiguousarray(g["width"], np.float32)
    torch.cuda.synchronize()
    fp = C.POINTER(C.c_float)
    for _ in range(2):
        got = np.zeros(len(widths), np.float32)
        check(lib().tpucb_calib_kld_static(0, None, C.c_void_p(hist.data_ptr()), widths.ctypes.data_as(fp), len(widths),
                                           2048, got.ctypes.data_as(fp)))
        assert np.array_equal(got, g["threshold"])
