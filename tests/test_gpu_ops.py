"""GPU parity: every op kernel through the C ABI (one-op modules, like the reference's
single-op backend tests under lib/Dialect/TPU/Backend/test) against the CPU oracle.
INT8 tensors must be bit-exact; BF16 within 1 ulp (they are in fact compared exactly);
fp32 within 1e-4 relative."""
import numpy as np
import pytest

import oracle
from oracle import graph_runner
from tpu_compiler_b200 import graphs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def M():
    from tpu_compiler_b200 import module
    return module


def run_both(M, model, inputs, check=None):
    m = M(0)
    m.load_text(model.text, model.weights)
    for k, v in inputs.items():
        m.set_tensor(k, v)
    m.invoke()
    ref = graph_runner.run(model.text, model.weights, inputs)
    names = check or model.outputs
    out = {}
    for n in names:
        out[n] = (m.get_tensor(n), ref[n])
    m.close()
    return out


def assert_exact(pairs):
    for n, (got, exp) in pairs.items():
        bad = np.flatnonzero(got.reshape(-1) != exp.reshape(-1))
        assert bad.size == 0, "%s: %d of %d differ, first at %d: got %s expected %s" % (
            n, bad.size, got.size, bad[0], got.reshape(-1)[bad[:5]], exp.reshape(-1)[bad[:5]])


CONV_CASES = [
    # n, cin, cout, hw, k, stride, pad, dil
    (1, 64, 64, 56, 3, 1, 1, 1),
    (1, 128, 128, 28, 3, 1, 1, 1),
    (1, 256, 256, 14, 3, 1, 1, 1),
    (1, 512, 512, 7, 3, 1, 1, 1),
    (2, 64, 256, 14, 1, 1, 0, 1),     # 1x1: tiled A path
    (1, 256, 64, 14, 1, 2, 0, 1),     # 1x1 stride 2
    (3, 32, 48, 13, 3, 2, 1, 1),      # odd size, stride 2, ragged tiles, Cout not a multiple of 32
    (1, 16, 255, 13, 1, 1, 0, 1),     # 255-channel head
    (1, 3, 64, 32, 7, 2, 3, 1),       # 3-channel 7x7/2 stem: row-window path
    (2, 3, 32, 32, 3, 1, 1, 1),       # 3-channel 3x3/1 stem: row-window path, 16-byte pixels
    (2, 3, 32, 48, 3, 2, 1, 1),       # 3-channel 3x3/2 stem (OW = 24: 8-pixel copies)
    (1, 3, 16, 13, 3, 2, 1, 1),       # stem whose width does not suit the window copies: patch path
    (1, 4, 32, 32, 5, 4, 2, 1),       # stride 4, 4 channels
    (2, 8, 32, 32, 3, 2, 1, 1),       # 8 channels, stride 2: row-window TMA path (8-byte pixels)
    (1, 12, 48, 16, 3, 1, 1, 1),      # 12 channels, stride 1: row-window TMA path (16-byte pixels)
    (1, 96, 24, 9, 3, 1, 2, 2),       # dilation 2
    (2, 144, 40, 10, 5, 1, 2, 1),     # 5x5, channels not a multiple of 64
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv2d_i8(M, case):
    n, cin, cout, hw, k, s, p, d = case
    model = graphs.single_conv_i8(n, cin, cout, hw, k, s, p, d, seed=2000 + cin + k)
    assert_exact(run_both(M, model, {"x": model.meta["x"]}))


def test_conv2d_i8_full_rshift_range_no_relu(M):
    model = graphs.single_conv_i8(1, 64, 64, 12, 3, 1, 1, relu=False, rshift_range=(0, 32), seed=77)
    assert_exact(run_both(M, model, {"x": model.meta["x"]}))


def test_conv2d_i8_batch8_sweep_point(M):
    model = graphs.single_conv_i8(8, 128, 128, 28, 3, 1, 1, seed=2101)
    assert_exact(run_both(M, model, {"x": model.meta["x"]}))


def test_conv2d_depthwise_and_grouped(M):
    for groups, c in ((96, 96), (2, 64)):
        model = graphs.single_conv_i8(2, c, c, 15, 3, 2, 1, groups=groups, seed=31 + groups)
        assert_exact(run_both(M, model, {"x": model.meta["x"]}))


def test_small_residual_network(M):
    b = graphs.GraphBuilder(11, simulate=True)
    img = np.random.default_rng(5).uniform(-1, 1, (1, 3, 20, 20))
    b.input("data", (2, 3, 20, 20), sample=img)
    x = b.quant_in("q", "data", 1.0)
    x = b.conv_i8("c1", x, 32, 3, stride=2, pad=1)
    x = b.pool_max("p1", x, 3, 2, pad=(0, 1, 0, 1))
    y = b.conv_i8("c2", x, 16, 1, pad=0)
    y = b.conv_i8("c3", y, 16, 3, pad=1)
    y = b.conv_i8("c4", y, 32, 1, pad=0, relu=False)
    x = b.eltwise_add_i8("add", [x, y])
    x = b.pool_avg_i8("gap", x)
    x = b.fc_i8("fc", x, 10)
    b.dequant("out", x, 100.0)
    model = graphs.Model(b.text(), b.weights, ["data"], ["out"])
    data = np.random.default_rng(6).uniform(-1, 1, (2, 3, 20, 20)).astype(np.float32)
    data[0] = img[0]
    pairs = run_both(M, model, {"data": data}, check=["q", "c1", "p1", "c2", "c3", "c4", "add", "gap", "fc", "out"])
    assert_exact(pairs)
