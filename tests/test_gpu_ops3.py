"""GPU parity of the layout / arithmetic ops of neighbouring networks (eltwise max / min, broadcast add / sub /
mul, pad, crop, permute, reduce), each as a small module through the C ABI against the CPU oracle. INT8 results
are compared exactly, fp32 within 1e-4 relative."""
import numpy as np
import pytest

from tpu_compiler_b200 import graphs
from tests.test_gpu_ops2 import assert_close, assert_exact, i8, run_both

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(2, 32, 9, 9), (1, 19, 5, 7)])
def test_eltwise_max_min_i8(shape):
    rng = np.random.default_rng(11)
    b = graphs.GraphBuilder(11, simulate=False)
    for nm in ("a", "b", "c"):
        b.op("input", nm, [], shape, "INT8")
    b.weight("r", [5]), b.weight("m", [37, -21, 64])
    b.op("eltwise_max", "mx", ["a", "b", "c", None, None, "r", "m"], shape, "INT8", do_relu=0)
    b.op("eltwise_max", "mx_relu", ["a", "b", None, None, "r", "m"], shape, "INT8", do_relu=1)
    b.op("eltwise_min", "mn", ["a", "b", "c", None, None, "r", "m"], shape, "INT8", do_relu=0)
    ins = {nm: i8(rng, shape) for nm in ("a", "b", "c")}
    assert_exact(run_both(b.text(), b.weights, ins, ["mx", "mx_relu", "mn"]))


@pytest.mark.parametrize("shape_b", [(1, 24, 1, 1), (2, 1, 6, 5), (2, 24, 6, 5), (1, 1, 1, 5)])
def test_broadcast_i8(shape_b):
    rng = np.random.default_rng(12)
    shape_a = (2, 24, 6, 5)
    b = graphs.GraphBuilder(12, simulate=False)
    b.op("input", "a", [], shape_a, "INT8")
    b.op("input", "b", [], shape_b, "INT8")
    b.weight("r", [6]), b.weight("m", [41, 29])
    mq, rq = graphs.quantize_multiplier(0.0079)
    b.weight("rq", [rq]), b.weight("mq", [mq])
    b.op("broadcast_add", "add", ["a", "b", None, None, "r", "m"], shape_a, "INT8", do_relu=0)
    b.op("broadcast_sub", "sub", ["a", "b", None, None, "r", "m"], shape_a, "INT8", do_relu=1)
    b.op("broadcast_mul", "mul", ["a", "b", None, None, "rq", "mq"], shape_a, "INT8", do_relu=0)
    ins = {"a": i8(rng, shape_a), "b": i8(rng, shape_b)}
    assert_exact(run_both(b.text(), b.weights, ins, ["add", "sub", "mul"]))


def test_broadcast_fp32_and_lower_rank():
    rng = np.random.default_rng(13)
    b = graphs.GraphBuilder(13, simulate=False)
    b.op("input", "a", [], (3, 10, 4, 4), "FP32")
    b.op("input", "v", [], (4,), "FP32")          # rank 1, aligned to the last dimension
    b.op("broadcast_mul", "mul", ["a", "v"], (3, 10, 4, 4), "FP32", do_relu=1)
    b.op("broadcast_add", "add", ["a", "v"], (3, 10, 4, 4), "FP32")
    ins = {"a": rng.normal(0, 1, (3, 10, 4, 4)).astype(np.float32), "v": rng.normal(0, 1, (4,)).astype(np.float32)}
    assert_close(run_both(b.text(), b.weights, ins, ["mul", "add"]), rtol=1e-6)


@pytest.mark.parametrize("dtype", ["INT8", "FP32"])
def test_pad_crop_permute(dtype):
    rng = np.random.default_rng(14)
    shape = (2, 20, 7, 9)
    b = graphs.GraphBuilder(14, simulate=False)
    b.op("input", "x", [], shape, dtype)
    b.op("pad", "pad_c", ["x"], (2, 23, 10, 12), dtype, pads="0,1,2,3,0,2,1,0", mode="constant", const_val="0")
    b.op("pad", "pad_cut", ["x"], (1, 20, 6, 11), dtype, pads="-1,0,0,2,0,0,-1,0")
    b.op("pad", "pad_e", ["x"], (2, 20, 10, 13), dtype, pads="0,0,1,3,0,0,2,1", mode="edge")
    b.op("crop", "crop", ["x"], (1, 8, 5, 4), dtype, crop_offset="1,3,2,1")
    b.op("crop", "crop_step", ["x"], (2, 5, 3, 4), dtype, crop_offset="0,2,1,0", steps="1,3,2,2")
    b.op("permute", "nhwc", ["x"], (2, 7, 9, 20), dtype, order="0,2,3,1")
    b.op("permute", "swap", ["x"], (20, 2, 9, 7), dtype, order="1,0,3,2")
    x = i8(rng, shape) if dtype == "INT8" else rng.normal(0, 1, shape).astype(np.float32)
    assert_exact(run_both(b.text(), b.weights, {"x": x},
                          ["pad_c", "pad_cut", "pad_e", "crop", "crop_step", "nhwc", "swap"]))


def test_reduce_i8_and_fp32():
    rng = np.random.default_rng(15)
    shape = (2, 18, 7, 7)
    b = graphs.GraphBuilder(15, simulate=False)
    b.op("input", "x", [], shape, "INT8")
    b.op("input", "f", [], shape, "FP32")
    # INT8 mean over H x W: the 1/49 lives in the multiplier / rshift pair (non-QDM)
    b.weight("r", [13]), b.weight("m", [167])
    b.op("reduce_mean", "mean_hw", ["x", None, None, "r", "m"], (2, 18), "INT8", axes="2,3")
    b.op("reduce_max", "max_hw", ["x", None, None, None, None], (2, 18), "INT8", axes="2,3")
    b.op("reduce_min", "min_c", ["x", None, None, None, None], (2, 7, 7), "INT8", axes="1")
    b.op("reduce_mean", "fmean", ["f"], (2, 18), "FP32", axes="2,3")
    b.op("reduce_sum", "fsum_c", ["f"], (2, 7, 7), "FP32", axes="1")
    b.op("reduce_max", "fmax_w", ["f"], (2, 18, 7), "FP32", axes="3")
    ins = {"x": i8(rng, shape), "f": rng.normal(0, 2, shape).astype(np.float32)}
    out = run_both(b.text(), b.weights, ins, ["mean_hw", "max_hw", "min_c", "fmean", "fsum_c", "fmax_w"])
    assert_exact({k: out[k] for k in ("mean_hw", "max_hw", "min_c", "fmax_w")})
    assert_close({k: out[k] for k in ("fmean", "fsum_c")}, rtol=1e-5)


@pytest.mark.parametrize("cfg", [dict(ic=16, oc=24, hw=7, k=4, s=2, p=1, g=1), dict(ic=32, oc=32, hw=5, k=3, s=2, p=0, g=1),
                                 dict(ic=64, oc=64, hw=6, k=2, s=2, p=0, g=4), dict(ic=8, oc=40, hw=9, k=3, s=1, p=1, g=1)])
def test_deconv_i8(cfg):
    """Transposed convolution (upsampling layers of segmentation / detection necks)."""
    rng = np.random.default_rng(16)
    ic, oc, hw, k, s, p, g = (cfg[x] for x in ("ic", "oc", "hw", "k", "s", "p", "g"))
    oh = (hw - 1) * s - 2 * p + k
    b = graphs.GraphBuilder(16, simulate=False)
    b.op("input", "x", [], (2, ic, hw, hw), "INT8")
    b.weight("w", rng.integers(-127, 128, (oc, ic // g, k, k)))
    b.weight("bias", rng.integers(-2 ** 14, 2 ** 14, oc))
    b.weight("rs", rng.integers(9, 13, oc))
    b.weight("mu", np.float32((rng.integers(2 ** 30, 2 ** 31 - 128, oc) // 128) * 128))
    b.op("deconv_2d", "y", ["x", "w", "bias", None, None, "rs", "mu"], (2, oc, oh, oh), "INT8", kh=k, kw=k, sh=s, sw=s,
         pt=p, pb=p, pl=p, pr=p, dh=1, dw=1, g=g, do_relu=1, with_bias=1)
    assert_exact(run_both(b.text(), b.weights, {"x": i8(rng, (2, ic, hw, hw))}, ["y"]))
