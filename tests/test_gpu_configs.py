"""GPU parity at the sizes the benchmark configurations name, not at reduced ones:

* ResNet-50 INT8 at the bench batch (256 images in one launch): sampled images against the batch-1
  module, which `test_gpu_resnet.py` compares with the CPU oracle tensor by tensor. At this size the
  persistent tile walk, the 256-pixel tiles of the narrow layers and the weight-resident mode of the
  convolution kernel take other paths than at the small batches of the other tests.
* the 3x3 op sweep at N = 32 (all four points) and N = 8 (the remaining three), and one point with
  the right shift drawn over the whole range [0, 31], against the CPU oracle;
* MobileNet-v2 at 224 x 224, batch 32, and the YOLOv4-style graph at 416 x 416, batch 8: the first and the
  last image of the batch against the CPU oracle run on those two images (the synthetic graphs'
  weights do not depend on the batch), every tensor, exact.
"""
import numpy as np
import pytest

from oracle import graph_runner
from tpu_compiler_b200 import graphs

pytestmark = pytest.mark.gpu


def test_resnet50_at_the_bench_batch():
    from tpu_compiler_b200 import module
    B = 256
    names = ["conv1", "res2c", "res4f", "res5c", "pool5", "fc1000_dequant"]
    picks = (0, 127, 255)
    rng = np.random.default_rng(20256)
    imgs = rng.uniform(-1, 1, (B, 3, 224, 224)).astype(np.float32)
    big = graphs.resnet50_int8(batch=B, seed=1001)
    m = module(0)
    m.load_text(big.text, big.weights)
    m.set_tensor("data", imgs)
    m.invoke()
    m.invoke()   # the CUDA-graph replay, as the bench runs it
    got = {}
    for n in names:
        t = m.get_tensor(n)
        got[n] = {i: t[i:i + 1].copy() for i in picks}
        del t
    m.close()
    one = graphs.resnet50_int8(batch=1, seed=1001)
    s = module(0)
    s.load_text(one.text, one.weights)
    for i in picks:
        s.set_tensor("data", imgs[i:i + 1])
        s.invoke()
        for n in names:
            assert np.array_equal(got[n][i], s.get_tensor(n)), "image %d of the batch differs at %s" % (i, n)
    s.close()


SWEEP = [(32, 64, 56), (32, 128, 28), (32, 256, 14), (32, 512, 7), (8, 64, 56), (8, 256, 14), (8, 512, 7)]


def _conv_against_oracle(model):
    from tpu_compiler_b200 import module
    m = module(0)
    m.load_text(model.text, model.weights)
    m.set_tensor("x", model.meta["x"])
    m.invoke()
    got = m.get_tensor("conv")
    m.close()
    exp = graph_runner.run(model.text, model.weights, {"x": model.meta["x"]})["conv"]
    bad = np.flatnonzero(got.reshape(-1) != exp.reshape(-1))
    assert bad.size == 0, "%d of %d values differ, first at %d" % (bad.size, got.size, bad[0] if bad.size else -1)
    return got


@pytest.mark.parametrize("n,c,hw", SWEEP)
def test_conv_sweep_point(n, c, hw):
    out = _conv_against_oracle(graphs.single_conv_i8(n, c, c, hw, 3, 1, 1, seed=2000 + c + n))
    assert 0.02 < float((out > 0).mean()) and float((out == 127).mean()) < 0.9   # neither all zero nor all saturated


@pytest.mark.parametrize("relu", [True, False])
def test_conv_sweep_point_full_rshift_range(relu):
    _conv_against_oracle(graphs.single_conv_i8(8, 128, 128, 28, 3, 1, 1, relu=relu, rshift_range=(0, 32), seed=2999))


@pytest.mark.parametrize("n,c,hw,relu", [(1, 512, 7, True), (2, 1024, 5, False), (3, 384, 9, True)])
def test_split_k_layers(n, c, hw, relu):
    """Launches with few tiles and 24 K blocks or more share each tile among several CTAs (int32 partial sums added in
    global memory, the CTA that completes a tile runs the epilogue). Exact against the oracle, equal to the unsplit
    launch, and the same again on every graph replay (the workspace is left zero)."""
    from tpu_compiler_b200 import module
    model = graphs.single_conv_i8(n, c, c, hw, 3, 1, 1, relu=relu, rshift_range=(0, 32) if not relu else (14, 17),
                                  seed=2700 + c)
    exp = graph_runner.run(model.text, model.weights, {"x": model.meta["x"]})["conv"]
    for split in (1, 0):
        m = module(0)
        m.set_option("split_k", split)
        m.load_text(model.text, model.weights)
        m.set_tensor("x", model.meta["x"])
        for _ in range(4):
            m.invoke()
            assert np.array_equal(m.get_tensor("conv"), exp), "split_k=%d" % split
        m.close()


def _first_and_last_against_oracle(builder, batch, res, lo, seed):
    from tpu_compiler_b200 import module
    rng = np.random.default_rng(seed)
    data = rng.uniform(lo, 1, (batch, 3, res, res)).astype(np.float32)
    big = builder(batch=batch, res=res)
    m = module(0)
    m.load_text(big.text, big.weights)
    m.set_tensor("data", data)
    m.invoke()
    two = builder(batch=2, res=res)
    assert set(two.weights) == set(big.weights) and all(np.array_equal(two.weights[k], big.weights[k]) for k in two.weights)
    pair = np.stack([data[0], data[batch - 1]])
    ref = graph_runner.run(two.text, two.weights, {"data": pair})
    bad = None
    for name in m.get_all_tensor_names():
        got = m.get_tensor(name)
        got = np.stack([got[0], got[batch - 1]]).reshape(-1)
        exp = ref[name].reshape(-1)
        if not np.array_equal(got, exp):
            bad = (name, int((got != exp).sum()), got.size)
            break
    outs = {n: m.get_tensor(n).shape for n in big.outputs}
    m.close()
    assert bad is None, "first mismatching op: %s (%d of %d values)" % bad
    return outs


def test_mobilenet_v2_224_batch_32():
    outs = _first_and_last_against_oracle(graphs.mobilenet_v2_int8, 32, 224, -1.0, 3032)
    assert outs == {"fc_dequant": (32, 1000)}


def test_yolov4_style_416_batch_8():
    outs = _first_and_last_against_oracle(graphs.yolov4_style_int8, 8, 416, 0.0, 4008)
    assert outs == {"head8": (8, 255, 52, 52), "head16": (8, 255, 26, 26), "head32": (8, 255, 13, 13)}
