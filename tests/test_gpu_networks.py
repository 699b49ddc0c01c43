"""GPU parity of whole MobileNet-v2 (depthwise / pointwise / residual adds) and YOLOv4-style (BF16 mish
tables between INT8 convolutions, leaky-ReLU, SPP max-pools, upsample, concat, 255-channel heads)
modules at reduced resolution, every tensor against the CPU oracle. INT8 and BF16 exactly."""
import numpy as np
import pytest

from oracle import graph_runner
from tpu_compiler_b200 import graphs

pytestmark = pytest.mark.gpu


def check_all_tensors(model, data, options=()):
    from tpu_compiler_b200 import module
    ref = graph_runner.run(model.text, model.weights, {"data": data})
    m = module(0)
    for key, value in options:
        m.set_option(key, value)
    m.load_text(model.text, model.weights)
    m.set_tensor("data", data)
    m.invoke()
    bad = None
    for name in m.get_all_tensor_names():
        got = m.get_tensor(name).reshape(-1)
        exp = ref[name].reshape(-1)
        if not np.array_equal(got, exp):
            bad = (name, int((got != exp).sum()), got.size)
            break
    m.close()
    assert bad is None, "first mismatching op: %s (%d of %d values)" % bad


def test_mobilenet_v2_every_tensor():
    model = graphs.mobilenet_v2_int8(batch=3, res=96, seed=3001)
    data = np.random.default_rng(31).uniform(-1, 1, (3, 3, 96, 96)).astype(np.float32)
    check_all_tensors(model, data)


def test_mobilenet_v2_every_tensor_with_adds_in_the_convolution_epilogue():
    """The residual adds of the inverted-residual blocks (no ReLU, project convolution without activation) fused into
    the project convolution's epilogue (option fuse_residual_add)."""
    model = graphs.mobilenet_v2_int8(batch=2, res=96, seed=3002)
    data = np.random.default_rng(32).uniform(-1, 1, (2, 3, 96, 96)).astype(np.float32)
    check_all_tensors(model, data, options=(("fuse_residual_add", 1),))


def test_yolov4_style_every_tensor():
    model = graphs.yolov4_style_int8(batch=2, res=64, width=0.25, depth=(1, 1, 2, 2, 1), seed=4001)
    data = np.random.default_rng(41).uniform(0, 1, (2, 3, 64, 64)).astype(np.float32)
    check_all_tensors(model, data)


def test_yolov4_style_every_tensor_unfused_activations():
    """With the quant -> mish -> quant chains as three separate launches (the default runs them as one)."""
    from tpu_compiler_b200 import module
    model = graphs.yolov4_style_int8(batch=2, res=64, width=0.25, depth=(1, 1, 2, 2, 1), seed=4002)
    data = np.random.default_rng(42).uniform(0, 1, (2, 3, 64, 64)).astype(np.float32)
    check_all_tensors(model, data, options=(("fuse_activations", 0),))
    counts = []
    for fuse in (1, 0):
        m = module(0)
        m.set_option("fuse_activations", fuse)
        m.load_text(model.text, model.weights)
        counts.append(m.kernel_count())
        m.close()
    ops = graph_runner.parse(model.text)
    n_mish = sum(o["type"] == "mish" for o in ops)
    n_leaky = sum(o["type"] == "leaky_relu" for o in ops)
    # a quant -> mish -> quant chain saves two launches, a leaky ReLU fused into its convolution one; chains whose
    # result feeds a few-channel convolution keep that convolution's padded-row layout and stay unfused
    saved = counts[1] - counts[0]
    assert n_mish > 0 and n_leaky > 0 and n_mish <= saved <= 2 * n_mish + n_leaky, (counts, n_mish, n_leaky)


def test_yolov4_style_full_topology_loads_and_counts():
    """The full-size graph has the op counts of the reference's YOLOv4 graph (110 conv, 23 shortcut,
    10 route, 3 max-pool, 2 upsample) and loads at 416 x 416."""
    from tpu_compiler_b200 import module
    model = graphs.yolov4_style_int8(batch=1, res=416, simulate=False)
    ops = graph_runner.parse(model.text)
    count = lambda t: sum(o["type"] == t for o in ops)  # noqa: E731
    assert (count("conv_2d"), count("eltwise_add"), count("concat"), count("pool_max_2d"), count("upsample")) == \
        (110, 23, 10, 3, 2)
    m = module(0)
    m.load_text(model.text, model.weights)
    m.set_tensor("data", np.random.default_rng(1).uniform(0, 1, (1, 3, 416, 416)).astype(np.float32))
    m.invoke()
    for name, hw in (("head8", 52), ("head16", 26), ("head32", 13)):
        assert m.get_tensor(name).shape == (1, 255, hw, hw)
    m.close()


def test_resnet50_bf16_graph():
    """An all-BF16 ResNet-50 (BF16 convolutions and inner product on the tensor cores, BF16 pooling and eltwise)
    against the oracle. A BF16 result may land one unit in the last place (0.4%) away from the CPU loop's, and such
    flips feed the next layer, so only the first layers are compared in ulps; deeper tensors and the logits are
    compared to a few percent of their range."""
    from tpu_compiler_b200 import module
    model = graphs.resnet50_bf16(batch=2)
    x = np.random.default_rng(5).uniform(-1, 1, (2, 3, 224, 224)).astype(np.float32)
    ref = graph_runner.run(model.text, model.weights, {"data": x})
    m = module(0)
    m.load_text(model.text, model.weights)
    m.set_tensor("data", x)
    m.invoke()
    got = {n: m.get_tensor(n) for n in ("data_bf16", "conv1", "pool1", "res2a", "res3d", "res5c", "fc1000_f32")}
    m.close()
    assert np.array_equal(got["data_bf16"], ref["data_bf16"])
    for n in ("conv1", "pool1"):
        g = (got[n].reshape(-1).view(np.uint32) >> 16).astype(np.int64)
        e = (ref[n].reshape(-1).view(np.uint32) >> 16).astype(np.int64)
        big = np.abs(ref[n].reshape(-1)) > 1e-2 * np.abs(ref[n]).max()
        assert np.abs(g - e)[big].max() <= 1, n
    for n, tol in (("res2a", 0.01), ("res3d", 0.02), ("res5c", 0.04), ("fc1000_f32", 0.04)):
        err = np.abs(got[n] - ref[n]).max() / np.abs(ref[n]).max()
        assert err <= tol, (n, err)
    assert (np.argmax(got["fc1000_f32"], axis=1) == np.argmax(ref["fc1000_f32"], axis=1)).all()
