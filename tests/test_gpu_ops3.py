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


def _bf16(x):
    return (np.asarray(x, np.float32).view(np.uint32) & 0xffff0000).view(np.float32)


def assert_bf16_ulp(pairs, max_ulp=1):
    """BF16 tensors within `max_ulp` units in the last place (the tolerance the interpreter path allows for BF16;
    the tensor core accumulates in another order than the CPU loop)."""
    for n, (got, exp) in pairs.items():
        g = (got.reshape(-1).view(np.uint32) >> 16).astype(np.int64)
        e = (exp.reshape(-1).view(np.uint32) >> 16).astype(np.int64)
        key = lambda b: np.where(b & 0x8000, 0x8000 - (b & 0x7fff), 0x8000 + b)  # noqa: E731  monotone in the value
        d = np.abs(key(g) - key(e))
        # results next to zero: compare against the tensor's scale instead of ulps of a tiny number
        tiny = np.abs(exp.reshape(-1)) < 1e-3 * (np.abs(exp).max() + 1e-30)
        bad = np.flatnonzero((d > max_ulp) & ~tiny)
        assert bad.size == 0, "%s: %d of %d differ by more than %d ulp, e.g. idx %d got %r expected %r" % (
            n, bad.size, g.size, max_ulp, bad[0], got.reshape(-1)[bad[0]], exp.reshape(-1)[bad[0]])
        assert np.abs(got.reshape(-1)[tiny] - exp.reshape(-1)[tiny]).max(initial=0) <= 4e-3 * (np.abs(exp).max() + 1e-30)


@pytest.mark.parametrize("cfg", [dict(ic=32, oc=64, hw=12, k=1, s=1, p=0, relu=1), dict(ic=64, oc=128, hw=14, k=3, s=1, p=1, relu=1),
                                 dict(ic=16, oc=256, hw=9, k=3, s=2, p=1, relu=0), dict(ic=128, oc=24, hw=7, k=1, s=1, p=0, relu=0),
                                 dict(ic=3, oc=64, hw=30, k=7, s=2, p=3, relu=1), dict(ic=4, oc=32, hw=11, k=3, s=1, p=1, relu=0)])
def test_conv_bf16(cfg):
    """BF16 convolution on the tensor cores (BF16 operands, fp32 accumulation) against the fp32-loop oracle."""
    rng = np.random.default_rng(17)
    ic, oc, hw, k, s, p = (cfg[x] for x in ("ic", "oc", "hw", "k", "s", "p"))
    oh = (hw + 2 * p - k) // s + 1
    b = graphs.GraphBuilder(17, simulate=False)
    b.op("input", "x", [], (3, ic, hw, hw), "BF16")
    b.weight("w", _bf16(rng.normal(0, (2.0 / (ic * k * k)) ** 0.5, (oc, ic, k, k))))
    b.weight("bias", rng.normal(0, 0.1, oc).astype(np.float32))
    b.op("conv_2d", "y", ["x", "w", "bias"], (3, oc, oh, oh), "BF16", kh=k, kw=k, sh=s, sw=s, pt=p, pb=p, pl=p, pr=p,
         dh=1, dw=1, g=1, do_relu=cfg["relu"], with_bias=1)
    x = _bf16(rng.normal(0, 1, (3, ic, hw, hw)))
    assert_bf16_ulp(run_both(b.text(), b.weights, {"x": x}, ["y"]))


@pytest.mark.gpu
@pytest.mark.parametrize("cfg", [dict(ic=32, oc=32, g=32, hw=14, k=3, s=1, p=1, relu=1), dict(ic=48, oc=48, g=48, hw=15, k=3, s=2, p=1, relu=0),
                                 dict(ic=32, oc=64, g=4, hw=10, k=3, s=1, p=1, relu=1), dict(ic=24, oc=24, g=24, hw=9, k=5, s=1, p=2, relu=0),
                                 dict(ic=16, oc=40, g=2, hw=8, k=1, s=1, p=0, relu=1)])
def test_conv_bf16_grouped_and_depthwise(cfg):
    """Grouped and depthwise BF16 convolutions (the direct kernel, fp32 accumulation) against the fp32-loop oracle."""
    rng = np.random.default_rng(19)
    ic, oc, g, hw, k, s, p = (cfg[x] for x in ("ic", "oc", "g", "hw", "k", "s", "p"))
    oh = (hw + 2 * p - k) // s + 1
    b = graphs.GraphBuilder(19, simulate=False)
    b.op("input", "x", [], (2, ic, hw, hw), "BF16")
    b.weight("w", _bf16(rng.normal(0, (2.0 / (ic // g * k * k)) ** 0.5, (oc, ic // g, k, k))))
    b.weight("bias", rng.normal(0, 0.1, oc).astype(np.float32))
    b.op("conv_2d", "y", ["x", "w", "bias"], (2, oc, oh, oh), "BF16", kh=k, kw=k, sh=s, sw=s, pt=p, pb=p, pl=p, pr=p,
         dh=1, dw=1, g=g, do_relu=cfg["relu"], with_bias=1)
    x = _bf16(rng.normal(0, 1, (2, ic, hw, hw)))
    assert_bf16_ulp(run_both(b.text(), b.weights, {"x": x}, ["y"]))


@pytest.mark.gpu
def test_relu_and_leaky_relu_bf16():
    """BF16 ReLU and leaky ReLU (x > 0 ? x : x * slope in fp32, one BF16 rounding), also right behind a BF16 convolution
    (which must not take the INT8 fusion path)."""
    rng = np.random.default_rng(25)
    b = graphs.GraphBuilder(25, simulate=False)
    b.op("input", "x", [], (2, 40, 8, 8), "BF16")
    b.op("relu", "r", ["x"], (2, 40, 8, 8), "BF16")
    b.op("leaky_relu", "l", ["x"], (2, 40, 8, 8), "BF16", negative_slope=0.1)
    b.weight("w", _bf16(rng.normal(0, 0.2, (16, 40, 1, 1))))
    b.weight("bias", rng.normal(0, 0.1, 16).astype(np.float32))
    b.op("conv_2d", "c", ["x", "w", "bias"], (2, 16, 8, 8), "BF16", kh=1, kw=1, sh=1, sw=1, pt=0, pb=0, pl=0, pr=0,
         dh=1, dw=1, g=1, do_relu=0, with_bias=1)
    b.op("leaky_relu", "cl", ["c"], (2, 16, 8, 8), "BF16", negative_slope=0.125)
    x = rng.normal(0, 1, (2, 40, 8, 8)).astype(np.float32)
    x.reshape(-1)[:4] = [0.0, -0.0, 1e-30, -1e-30]
    x = _bf16(x)
    out = run_both(b.text(), b.weights, {"x": x}, ["r", "l", "c", "cl"])
    assert_exact({k: out[k] for k in ("r", "l")})
    assert_bf16_ulp({k: out[k] for k in ("c", "cl")})


@pytest.mark.gpu
def test_concat_upsample_pixelshuffle_bf16():
    """The data-movement ops of BF16 graphs: plain copies of two-byte values (vector path and byte path of the concat)."""
    rng = np.random.default_rng(24)
    b = graphs.GraphBuilder(24, simulate=False)
    b.op("input", "a", [], (2, 24, 6, 6), "BF16")
    b.op("input", "b", [], (2, 255, 6, 6), "BF16")
    b.op("input", "c", [], (2, 16, 6, 6), "BF16")
    b.op("concat", "cat", ["a", "b", "c"], (2, 295, 6, 6), "BF16", axis=1, do_relu=0)
    b.op("concat", "cat_vec", ["a", "c"], (2, 40, 6, 6), "BF16", axis=1, do_relu=0)
    b.op("upsample", "up", ["a"], (2, 24, 12, 18), "BF16", scale_h=2, scale_w=3)
    b.op("pixelshuffle", "ps", ["c"], (2, 4, 12, 12), "BF16", upscale_factor=2, mode="CRD")
    ins = {k: _bf16(rng.normal(0, 1, shp)) for k, shp in (("a", (2, 24, 6, 6)), ("b", (2, 255, 6, 6)), ("c", (2, 16, 6, 6)))}
    assert_exact(run_both(b.text(), b.weights, ins, ["cat", "cat_vec", "up", "ps"]))


@pytest.mark.gpu
@pytest.mark.parametrize("cfg", [dict(ic=16, oc=32, g=1, hw=7, k=2, s=2, p=0, relu=0), dict(ic=24, oc=16, g=1, hw=6, k=4, s=2, p=1, relu=1),
                                 dict(ic=32, oc=32, g=32, hw=5, k=3, s=2, p=1, relu=0), dict(ic=8, oc=24, g=2, hw=9, k=3, s=1, p=1, relu=1)])
def test_deconv_bf16(cfg):
    """BF16 deconvolution (the direct kernel over the zero-inserted input with the flipped filter) against the scatter
    form of the oracle."""
    rng = np.random.default_rng(23)
    ic, oc, g, hw, k, s, p = (cfg[x] for x in ("ic", "oc", "g", "hw", "k", "s", "p"))
    oh = (hw - 1) * s + k - 2 * p
    b = graphs.GraphBuilder(23, simulate=False)
    b.op("input", "x", [], (2, ic, hw, hw), "BF16")
    b.weight("w", _bf16(rng.normal(0, (2.0 / (ic // g * k * k)) ** 0.5, (oc, ic // g, k, k))))
    b.weight("bias", rng.normal(0, 0.1, oc).astype(np.float32))
    b.op("deconv_2d", "y", ["x", "w", "bias"], (2, oc, oh, oh), "BF16", kh=k, kw=k, sh=s, sw=s, pt=p, pb=p, pl=p, pr=p,
         dh=1, dw=1, g=g, do_relu=cfg["relu"], with_bias=1)
    x = _bf16(rng.normal(0, 1, (2, ic, hw, hw)))
    assert_bf16_ulp(run_both(b.text(), b.weights, {"x": x}, ["y"]))


@pytest.mark.gpu
@pytest.mark.parametrize("cfg", [dict(m=4, c=512, hw=1, n=1000, relu=0), dict(m=2, c=64, hw=7, n=40, relu=1)])
def test_fc_bf16(cfg):
    """BF16 inner product on the tensor cores against the fp32-loop oracle (result rounded to BF16)."""
    rng = np.random.default_rng(23)
    m, c, hw, n = cfg["m"], cfg["c"], cfg["hw"], cfg["n"]
    k = c * hw * hw
    b = graphs.GraphBuilder(23, simulate=False)
    b.op("input", "x", [], (m, c, hw, hw), "BF16")
    b.weight("w", _bf16(rng.normal(0, (2.0 / k) ** 0.5, (n, k))))
    b.weight("bias", rng.normal(0, 0.1, n).astype(np.float32))
    b.op("fully_connected", "y", ["x", "w", "bias"], (m, n, 1, 1), "BF16", do_relu=cfg["relu"])
    x = _bf16(rng.normal(0, 1, (m, c, hw, hw)))
    assert_bf16_ulp(run_both(b.text(), b.weights, {"x": x}, ["y"]))


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 32, 9, 9), (1, 24, 5, 7)])
def test_eltwise_and_pool_bf16(shape):
    """BF16 eltwise add (with coefficients) / mul and pooling: fp32 arithmetic in the reference's order, one BF16
    rounding of the result. The reference's fp32 container keeps the unrounded average; a BF16 tensor holds its rounding."""
    rng = np.random.default_rng(29)
    b = graphs.GraphBuilder(29, simulate=False)
    for nm in ("a", "b", "c"):
        b.op("input", nm, [], shape, "BF16")
    b.op("eltwise_add", "add", ["a", "b", "c"], shape, "BF16", do_relu=1, coeff="1.0,-0.5,0.75")
    b.op("eltwise_mul", "mul", ["a", "b"], shape, "BF16", do_relu=0)
    n, c, h, w = shape
    oh, ow = (h + 2 - 3) // 2 + 1, (w + 2 - 3) // 2 + 1
    b.op("pool_max_2d", "pmax", ["a"], (n, c, oh, ow), "BF16", kh=3, kw=3, sh=2, sw=2, pt=1, pb=1, pl=1, pr=1)
    b.op("pool_avg_2d", "pavg", ["b"], (n, c, oh, ow), "BF16", kh=3, kw=3, sh=2, sw=2, pt=1, pb=1, pl=1, pr=1, count_include_pad=0)
    b.op("pool_avg_2d", "gap", ["c"], (n, c, 1, 1), "BF16", kh=h, kw=w, sh=1, sw=1, pt=0, pb=0, pl=0, pr=0, count_include_pad=1)
    feeds = {nm: _bf16(rng.normal(0, 2, shape)) for nm in ("a", "b", "c")}
    res = run_both(b.text(), b.weights, feeds, ["add", "mul", "pmax", "pavg", "gap"])
    from oracle import bf16_round
    for nm in ("pavg", "gap"):
        res[nm] = (res[nm][0], bf16_round(res[nm][1]))
    assert_exact(res)


@pytest.mark.parametrize("cfg", [dict(a=(2, 3, 20, 40), b=(2, 3, 40, 24), o=(2, 3, 20, 24)),
                                 dict(a=(5, 33, 17), b=(5, 17, 9), o=(5, 33, 9)),
                                 dict(a=(37, 50), b=(50, 21), o=(37, 21)),
                                 dict(a=(2, 20, 3, 40), b=(2, 40, 3, 24), o=(2, 20, 3, 24), lt=1, rt=1, ot=1),
                                 dict(a=(20, 3, 40), b=(3, 40, 24), o=(3, 20, 24), lt=1)])
@pytest.mark.parametrize("dtype", ["INT8", "BF16", "FP32"])
def test_matmul(cfg, dtype):
    """Batched product of two activations, with the storage orders of the three transposes."""
    rng = np.random.default_rng(31)
    b = graphs.GraphBuilder(31, simulate=False)
    b.op("input", "a", [], cfg["a"], dtype)
    b.op("input", "b", [], cfg["b"], dtype)
    ins = ["a", "b"]
    if dtype == "INT8":
        b.weight("rs", np.array([9.0], np.float32))
        b.weight("mu", np.array([1518500250.0], np.float32))
        ins += ["-", "-", "rs", "mu"]
    b.op("matmul", "y", ins, cfg["o"], dtype, do_relu=0, left_transpose=cfg.get("lt", 0), right_transpose=cfg.get("rt", 0),
         output_transpose=cfg.get("ot", 0))
    b.op("matmul", "yr", ins, cfg["o"], dtype, do_relu=1, left_transpose=cfg.get("lt", 0), right_transpose=cfg.get("rt", 0),
         output_transpose=cfg.get("ot", 0))
    if dtype == "INT8":
        feeds = {"a": i8(rng, cfg["a"]), "b": i8(rng, cfg["b"])}
        assert_exact(run_both(b.text(), b.weights, feeds, ["y", "yr"]))
    elif dtype == "BF16":
        feeds = {"a": _bf16(rng.normal(0, 1, cfg["a"])), "b": _bf16(rng.normal(0, 1, cfg["b"]))}
        assert_bf16_ulp(run_both(b.text(), b.weights, feeds, ["y", "yr"]))
    else:
        feeds = {"a": rng.normal(0, 1, cfg["a"]).astype(np.float32), "b": rng.normal(0, 1, cfg["b"]).astype(np.float32)}
        assert_close(run_both(b.text(), b.weights, feeds, ["y", "yr"]))


@pytest.mark.parametrize("cfg", [dict(shape=(3, 21, 2, 2), sd=3.0), dict(shape=(2, 1000, 1, 1), sd=2.0), dict(shape=(1, 80, 3, 3), sd=8.0)])
@pytest.mark.parametrize("do_log", [0, 1])
def test_softmax_bf16(cfg, do_log):
    """BF16 softmax through the exp slope table and the reciprocal / log exponent-mantissa tables: bit-exact,
    the fp32 sum is taken in the reference's channel order."""
    import oracle as O
    rng = np.random.default_rng(37)
    b = graphs.GraphBuilder(37, simulate=False)
    b.op("input", "x", [], cfg["shape"], "BF16")
    eb, es = O.lut_slope_tables("exp")
    re_, rm = O.lut_log_tables() if do_log else O.lut_pow_tables(-1.0)
    for nm, t in (("eb", eb), ("es", es), ("re", re_), ("rm", rm)):
        b.weight(nm, t)
    b.op("softmax", "y", ["x", "eb", "es", "re", "rm"], cfg["shape"], "BF16", axis=1, do_log=do_log)
    x = O.bf16_round(rng.normal(0, cfg["sd"], cfg["shape"]))
    assert_exact(run_both(b.text(), b.weights, {"x": x}, ["y"]))


@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("rshift_range", [(0, 4), (8, 30), (28, 32)])
def test_conv_i8_requant_forms(relu, rshift_range):
    """Both forms of the tensor-core requantisation against the oracle: shifts up to 29 take the multiply-high
    form, a layer with a larger shift the 64-bit multiply-add form; small shifts saturate most outputs."""
    model = graphs.single_conv_i8(n=2, c_in=64, c_out=160, hw=12, k=3, pad=1, relu=relu, seed=4100 + rshift_range[0],
                                  rshift_range=rshift_range)
    assert_exact(run_both(model.text, model.weights, model.meta, ["conv"]))


@pytest.mark.parametrize("cfg", [dict(ic=64, oc=64, hw=14, k=1, s=1, p=0, relu=1), dict(ic=32, oc=160, hw=13, k=3, s=1, p=1, relu=1),
                                 dict(ic=128, oc=40, hw=12, k=3, s=2, p=1, relu=0), dict(ic=8, oc=256, hw=9, k=1, s=1, p=0, relu=0),
                                 dict(ic=3, oc=64, hw=30, k=7, s=2, p=3, relu=1), dict(ic=4, oc=24, hw=9, k=3, s=1, p=1, relu=0)])
def test_conv_fp32_tensor_core(cfg):
    """fp32 convolution as three TF32 products on the tensor cores against the double-accumulated oracle. The bound
    (2e-5 of the tensor's range; measured 1e-6 to 5e-6, the tensor core truncates its partial sums) is far below what
    one TF32 product would reach (5e-4), so a missing correction term fails."""
    rng = np.random.default_rng(41)
    ic, oc, hw, k, s, p = (cfg[x] for x in ("ic", "oc", "hw", "k", "s", "p"))
    oh = (hw + 2 * p - k) // s + 1
    b = graphs.GraphBuilder(41, simulate=False)
    b.op("input", "x", [], (3, ic, hw, hw), "FP32")
    b.weight("w", rng.normal(0, (2.0 / (ic * k * k)) ** 0.5, (oc, ic, k, k)).astype(np.float32))
    b.weight("bias", rng.normal(0, 0.1, oc).astype(np.float32))
    b.op("conv_2d", "y", ["x", "w", "bias"], (3, oc, oh, oh), "FP32", kh=k, kw=k, sh=s, sw=s, pt=p, pb=p, pl=p, pr=p,
         dh=1, dw=1, g=1, do_relu=cfg["relu"], with_bias=1)
    x = rng.normal(0, 1, (3, ic, hw, hw)).astype(np.float32)
    assert_close(run_both(b.text(), b.weights, {"x": x}, ["y"]), rtol=2e-5)


def test_conv_fp32_fma_path_with_option_off():
    """`fp32_tensor_cores` = 0 keeps fp32 convolutions on the FMA pipe: same graph, tighter agreement (fp32 sums in
    another order only) and one launch instead of the split + tensor-core pair."""
    from tpu_compiler_b200 import module
    from oracle import graph_runner
    rng = np.random.default_rng(43)
    b = graphs.GraphBuilder(43, simulate=False)
    b.op("input", "x", [], (2, 64, 10, 10), "FP32")
    b.weight("w", rng.normal(0, 0.06, (96, 64, 3, 3)).astype(np.float32))
    b.weight("bias", rng.normal(0, 0.1, 96).astype(np.float32))
    b.op("conv_2d", "y", ["x", "w", "bias"], (2, 96, 10, 10), "FP32", kh=3, kw=3, sh=1, sw=1, pt=1, pb=1, pl=1, pr=1,
         dh=1, dw=1, g=1, do_relu=1, with_bias=1)
    x = rng.normal(0, 1, (2, 64, 10, 10)).astype(np.float32)
    ref = graph_runner.run(b.text(), b.weights, {"x": x})["y"]
    counts = {}
    for opt in (0, 1):
        m = module(0)
        m.set_option("fp32_tensor_cores", opt)
        m.load_text(b.text(), b.weights)
        m.set_tensor("x", x)
        m.invoke()
        err = np.abs(m.get_tensor("y") - ref).max() / np.abs(ref).max()
        counts[opt] = m.kernel_count()
        m.close()
        assert err <= (2e-5 if opt else 2e-6), (opt, err)
    assert counts[1] == counts[0] + 1


def test_batchnorm_and_reduce_l2_fp32():
    """BatchNormOpKernel (core/batchnorm.cpp:20-68) and ReduceL2 (core/reduce.cpp:91-103), fp32 as in the reference."""
    rng = np.random.default_rng(88)
    shape = (3, 21, 6, 5)
    b = graphs.GraphBuilder(88, simulate=False)
    b.op("input", "f", [], shape, "FP32")
    b.weight("mean", rng.normal(0, 1, 21)), b.weight("var", rng.uniform(0.05, 3, 21)), b.weight("sc", [0.9])
    b.op("batchnorm", "bn", ["f", "mean", "var", "sc"], shape, "FP32", variance_epsilon=1e-5)
    b.op("reduce_l2", "l2_c", ["bn"], (3, 6, 5), "FP32", axes="1", coeff=0.5)
    b.op("reduce_l2", "l2_hw", ["f"], (3, 21), "FP32", axes="2,3", coeff=0.5)
    out = run_both(b.text(), b.weights, {"f": rng.normal(0, 2, shape).astype(np.float32)}, ["bn", "l2_c", "l2_hw"])
    assert_close(out, rtol=1e-6)


@pytest.mark.parametrize("relu", [0, 1])
def test_fc_batched_i8(relu):
    """FullyConnected with a rank-3 filter: one product per batch index, each with its own bias row and its own
    (rshift, multiplier) pair (core/fullyconnected.cpp:59-88)."""
    rng = np.random.default_rng(61 + relu)
    B, m, k, n = 3, 20, 37, 11
    b = graphs.GraphBuilder(61, simulate=False)
    b.op("input", "x", [], (B, m, k), "INT8")
    b.weight("w", rng.integers(-127, 128, (B, n, k)))
    b.weight("bias", rng.integers(-2 ** 12, 2 ** 12, (B, n)))
    b.weight("rs", [5, 7, 6])
    b.weight("mu", np.float32((rng.integers(2 ** 30, 2 ** 31 - 128, B) // 128) * 128))
    b.op("fully_connected", "y", ["x", "w", "bias", None, None, "rs", "mu"], (B, m, n), "INT8", do_relu=relu)
    assert_exact(run_both(b.text(), b.weights, {"x": i8(rng, (B, m, k))}, ["y"]))
