"""CPU-side checks: the C-ABI library loads and exports every symbol include/tpucb.h declares,
fails loudly without a GPU, and the host-side graph builders agree with the oracle."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle
from oracle import graph_runner
from tpu_compiler_b200 import _lib, graphs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tpucb.h")).read()
    return sorted(set(re.findall(r"\b(tpucb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    names = _declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(L, n), n
    assert L.tpucb_version() >= 1


def test_no_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = _lib.lib()
    h = C.c_void_p()
    assert L.tpucb_interp_create(0, C.byref(h)) != 0
    msg = L.tpucb_last_error().decode()
    assert "no CPU fallback" in msg


def test_numpy_requant_matches_oracle():
    rng = np.random.default_rng(3)
    v = rng.integers(-2 ** 31, 2 ** 31, 5000)
    m = (rng.integers(2 ** 30, 2 ** 31 - 128, 5000) // 128) * 128
    r = rng.integers(0, 32, 5000)
    got = graphs.qdm_np(v, m, r)
    L = oracle.lib()
    exp = np.array([L.orc_qdm_i32(int(a), int(c), int(b)) for a, b, c in zip(v, m, r)])
    assert np.array_equal(got, exp)


def test_quantize_multiplier_range():
    for q in (0.9, 0.5, 0.123, 1e-3, 3e-6):
        m, r = graphs.quantize_multiplier(q)
        assert 2 ** 30 <= m < 2 ** 31 and 0 <= r <= 31
        assert float(np.float32(m)) == m
        assert abs(m / 2 ** 31 / 2 ** r - q) / q < 1e-6


def test_builder_simulation_matches_oracle_graph():
    """The scale-picking simulation inside the builder and the oracle agree on a small
    residual network, tensor by tensor (bit-exact INT8)."""
    b = graphs.GraphBuilder(11, simulate=True)
    img = np.random.default_rng(5).uniform(-1, 1, (1, 3, 20, 20))
    b.input("data", (1, 3, 20, 20), sample=img)
    x = b.quant_in("q", "data", 1.0)
    x = b.conv_i8("c1", x, 32, 3, stride=2, pad=1)
    x = b.pool_max("p1", x, 3, 2, pad=(0, 1, 0, 1))
    y = b.conv_i8("c2", x, 16, 1, pad=0)
    y = b.conv_i8("c3", y, 16, 3, pad=1)
    y = b.conv_i8("c4", y, 32, 1, pad=0, relu=False)
    x = b.eltwise_add_i8("add", [x, y])
    x = b.pool_avg_i8("gap", x)
    x = b.fc_i8("fc", x, 10)
    T = graph_runner.run(b.text(), b.weights, {"data": img.astype(np.float32)})
    for name in ("q", "c1", "p1", "c2", "c3", "c4", "add", "gap", "fc"):
        assert np.array_equal(T[name].reshape(-1), b.sim[name].astype(np.float32).reshape(-1)), name
    assert T["c3"].std() > 5  # the synthetic scales keep a live dynamic range


def test_resnet50_graph_shape():
    m = graphs.resnet50_int8(batch=1, simulate=False)
    ops = graph_runner.parse(m.text)
    assert sum(o["type"] == "conv_2d" for o in ops) == 53
    assert sum(o["type"] == "eltwise_add" for o in ops) == 16
    macs = 0
    for o in ops:
        if o["type"] == "conv_2d":
            w = m.weights[o["in"][1]]
            macs += int(np.prod(o["shape"])) * int(np.prod(w.shape[1:]))
    assert 3.8e9 < macs < 4.2e9


def _build_worker(args):
    """One process of test_concurrent_builds: points the build module at a scratch library and a fake compiler."""
    lib_path, log_path = args
    import subprocess
    import time
    from tpu_compiler_b200 import build as b
    b.LIB = lib_path

    def fake_compiler(cmd, check=True):
        out = cmd[cmd.index("-o") + 1]
        assert out != lib_path, "the compiler must not write the library in place"
        with open(out, "wb") as f:
            f.write(b"half")
            f.flush()
            time.sleep(0.3)   # a reader that opened the final path now would see a truncated file
            f.write(b"-written-library")
        with open(log_path, "a") as f:
            f.write("compiled\n")
        return subprocess.CompletedProcess(cmd, 0)

    b.build(run=fake_compiler)
    with open(lib_path, "rb") as f:
        return f.read()


def test_concurrent_builds(tmp_path):
    """Two ranks that both find the library stale: one compiles (into a temporary file, renamed over the library),
    the other waits on the lock, sees a fresh library and does not compile; neither reads a partial file."""
    import multiprocessing as mp
    lib_path, log_path = str(tmp_path / "libfake.so"), str(tmp_path / "log.txt")
    with mp.get_context("spawn").Pool(2) as pool:
        got = pool.map(_build_worker, [(lib_path, log_path)] * 2)
    assert got == [b"half-written-library"] * 2
    assert open(log_path).read().count("compiled") == 1
    assert [f for f in os.listdir(tmp_path) if f.endswith(".tmp")] == []
