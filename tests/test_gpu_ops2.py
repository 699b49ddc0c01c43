"""GPU parity of the HBM-bound op kernels and the fp32 ops, each as a one- or two-op module
through the C ABI against the CPU oracle. INT8 and BF16 results are compared exactly (the
BF16 tolerance of 1 ulp is not needed), fp32 within 1e-4 relative."""
import numpy as np
import pytest

import oracle
from oracle import graph_runner
from tpu_compiler_b200 import graphs

pytestmark = pytest.mark.gpu


def run_both(model_text, weights, inputs, names):
    from tpu_compiler_b200 import module
    m = module(0)
    m.load_text(model_text, weights)
    for k, v in inputs.items():
        m.set_tensor(k, v)
    m.invoke()
    ref = graph_runner.run(model_text, weights, inputs)
    out = {n: (m.get_tensor(n), ref[n]) for n in names}
    m.close()
    return out


def assert_exact(pairs):
    for n, (got, exp) in pairs.items():
        g, e = got.reshape(-1), exp.reshape(-1)
        bad = np.flatnonzero(g.view(np.uint32) != e.view(np.uint32))
        bad = bad[(g[bad] != e[bad])]  # +0 / -0 are the same value
        assert bad.size == 0, "%s: %d of %d differ, e.g. idx %d got %r expected %r" % (
            n, bad.size, g.size, bad[0], g[bad[0]], e[bad[0]])


def assert_close(pairs, rtol=1e-4):
    for n, (got, exp) in pairs.items():
        scale = np.abs(exp).max() + 1e-30
        err = np.abs(got - exp).max() / scale
        assert err <= rtol, "%s: max error %.3g relative to the tensor's range" % (n, err)


def i8(rng, shape):
    return rng.integers(-128, 128, shape).astype(np.float32)


def bf16(x):
    return (np.asarray(x, np.float32).view(np.uint32) & 0xffff0000).view(np.float32)


@pytest.mark.parametrize("shape", [(2, 32, 9, 9), (1, 255, 13, 13), (3, 24, 5, 7)])
def test_eltwise_add_mul_i8(shape):
    rng = np.random.default_rng(1)
    b = graphs.GraphBuilder(1, simulate=False)
    for nm in ("a", "b", "c"):
        b.op("input", nm, [], shape, "INT8")
    b.weight("add_r", [7]), b.weight("add_m", [45, -30, 101])
    b.op("eltwise_add", "add", ["a", "b", "c", None, None, "add_r", "add_m"], shape, "INT8", do_relu=0)
    b.op("eltwise_add", "add_relu", ["a", "b", None, None, "add_r", "add_m"], shape, "INT8", do_relu=1)
    mq, rq = graphs.quantize_multiplier(0.0123)
    b.weight("mul_r", [rq]), b.weight("mul_m", [mq])
    b.op("eltwise_mul", "mul", ["a", "b", None, None, "mul_r", "mul_m"], shape, "INT8", do_relu=0)
    b.op("eltwise_mul", "mul_relu", ["a", "c", None, None, "mul_r", "mul_m"], shape, "INT8", do_relu=1)
    ins = {k: i8(rng, shape) for k in ("a", "b", "c")}
    assert_exact(run_both(b.text(), b.weights, ins, ["add", "add_relu", "mul", "mul_relu"]))


@pytest.mark.parametrize("case", [
    # n, c, h, w, k, s, pt, pl, oh, ow
    (2, 64, 12, 12, 3, 2, 0, 0, 6, 6),       # ceil-mode style: bottom/right pad implied by the output size
    (1, 48, 13, 13, 5, 1, 2, 2, 13, 13),     # SPP-style stride-1 window
    (2, 33, 9, 9, 2, 2, 0, 0, 4, 4),         # channels not a multiple of 16
])
def test_pool_i8(case):
    n, c, h, w, k, s, pt, pl, oh, ow = case
    rng = np.random.default_rng(2)
    b = graphs.GraphBuilder(2, simulate=False)
    b.op("input", "x", [], (n, c, h, w), "INT8")
    b.op("pool_max_2d", "mx", ["x"], (n, c, oh, ow), "INT8", kh=k, kw=k, sh=s, sw=s, pt=pt, pb=0, pl=pl, pr=0)
    b.weight("av_r", [9]), b.weight("av_m", [int(512 / (k * k))])
    b.op("pool_avg_2d", "av", ["x", None, None, "av_r", "av_m"], (n, c, oh, ow), "INT8", kh=k, kw=k, sh=s, sw=s,
         pt=pt, pb=0, pl=pl, pr=0, count_include_pad=1)
    assert_exact(run_both(b.text(), b.weights, {"x": i8(rng, (n, c, h, w))}, ["mx", "av"]))


def test_global_avg_pool_and_fc_i8():
    rng = np.random.default_rng(3)
    b = graphs.GraphBuilder(3, simulate=False)
    b.op("input", "x", [], (4, 96, 7, 7), "INT8")
    b.weight("av_r", [11]), b.weight("av_m", [41])
    b.op("pool_avg_2d", "gap", ["x", None, None, "av_r", "av_m"], (4, 96, 1, 1), "INT8", kh=7, kw=7, sh=7, sw=7,
         count_include_pad=1)
    w = rng.integers(-127, 128, (37, 96)).astype(np.float32)
    mq, rq = graphs.quantize_multiplier(0.004)
    b.weight("fw", w), b.weight("fb", rng.integers(-3000, 3000, 37)), b.weight("fr", [rq]), b.weight("fm", [mq])
    b.op("fully_connected", "fc", ["gap", "fw", "fb", None, None, "fr", "fm"], (4, 37), "INT8", do_relu=0)
    b.op("fully_connected", "fc_relu", ["gap", "fw", "fb", None, None, "fr", "fm"], (4, 37), "INT8", do_relu=1)
    # fully-connected straight on a spatial tensor (NCHW flattening order)
    w2 = rng.integers(-127, 128, (20, 96 * 49)).astype(np.float32)
    mq2, rq2 = graphs.quantize_multiplier(0.0004)
    b.weight("gw", w2), b.weight("gb", rng.integers(-3000, 3000, 20)), b.weight("gr", [rq2]), b.weight("gm", [mq2])
    b.op("fully_connected", "fc_sp", ["x", "gw", "gb", None, None, "gr", "gm"], (4, 20), "INT8", do_relu=0)
    assert_exact(run_both(b.text(), b.weights, {"x": i8(rng, (4, 96, 7, 7))}, ["gap", "fc", "fc_relu", "fc_sp"]))


def test_concat_upsample_pixelshuffle_i8():
    rng = np.random.default_rng(4)
    b = graphs.GraphBuilder(4, simulate=False)
    b.op("input", "a", [], (2, 24, 6, 6), "INT8")
    b.op("input", "b", [], (2, 255, 6, 6), "INT8")
    b.op("input", "c", [], (2, 16, 6, 6), "INT8")
    b.weight("cr", [0, 5, 3]), b.weight("cm", [1, 23, 9])
    b.op("concat", "cat", ["a", "b", "c", None, None, "cr", "cm"], (2, 295, 6, 6), "INT8", axis=1, do_relu=0)
    b.op("concat", "cat_plain", ["a", "c"], (2, 40, 6, 6), "INT8", axis=1, do_relu=1)
    b.op("upsample", "up", ["a"], (2, 24, 12, 18), "INT8", scale_h=2, scale_w=3)
    b.op("pixelshuffle", "ps_crd", ["c"], (2, 4, 12, 12), "INT8", upscale_factor=2, mode="CRD")
    b.op("pixelshuffle", "ps_dcr", ["c"], (2, 4, 12, 12), "INT8", upscale_factor=2, mode="DCR")
    ins = {"a": i8(rng, (2, 24, 6, 6)), "b": i8(rng, (2, 255, 6, 6)), "c": i8(rng, (2, 16, 6, 6))}
    assert_exact(run_both(b.text(), b.weights, ins, ["cat", "cat_plain", "up", "ps_crd", "ps_dcr"]))


def test_relu_leaky_lut_i8():
    rng = np.random.default_rng(5)
    shape = (2, 40, 8, 8)
    b = graphs.GraphBuilder(5, simulate=False)
    b.op("input", "x", [], shape, "INT8")
    b.op("relu", "r", ["x"], shape, "INT8")
    for nm, v in (("rp", [4]), ("mp", [13]), ("rn", [7]), ("mn", [12]), ("mp0", [0])):
        b.weight(nm, v)
    b.op("leaky_relu", "lk", ["x", None, None, None, None, "rp", "mp", "rn", "mn"], shape, "INT8", negative_slope=0.1)
    b.op("leaky_relu", "lk_nopos", ["x", None, None, None, None, "rp", "mp0", "rn", "mn"], shape, "INT8",
         negative_slope=0.1)
    table = rng.integers(-128, 128, 256).astype(np.float32)
    b.weight("tab", np.tile(table, 4)), b.weight("tab2", np.zeros(1024))
    b.op("sigmoid", "lut", ["x", "tab", "tab2"], shape, "INT8")
    assert_exact(run_both(b.text(), b.weights, {"x": i8(rng, shape)}, ["r", "lk", "lk_nopos", "lut"]))


def test_quant_family():
    rng = np.random.default_rng(6)
    shape = (2, 19, 7, 5)
    b = graphs.GraphBuilder(6, simulate=False)
    b.op("input", "f", [], shape, "FP32")
    b.op("quant", "f_i8_host", ["f"], shape, "INT8", **{"from": "NONE", "to": "INT8", "scale": repr(128 / 2.7)})
    b.op("quant", "f_bf16", ["f"], shape, "BF16", **{"from": "NONE", "to": "BF16", "scale": "1.0"})
    b.op("quant", "i8_f32", ["f_i8_host"], shape, "FP32", **{"from": "INT8", "to": "NONE", "scale": repr(2.7 / 128)})
    b.op("quant", "i8_bf16", ["f_i8_host"], shape, "BF16", **{"from": "INT8", "to": "BF16", "scale": repr(2.7 / 128)})
    b.op("quant", "bf16_i8", ["i8_bf16"], shape, "INT8", **{"from": "BF16", "to": "INT8", "scale": repr(128 / 1.9)})
    # fp32 -> int8 away from the graph input takes the TPU (bf16) rounding path
    b.op("quant", "f32_i8_tpu", ["i8_f32"], shape, "INT8", **{"from": "NONE", "to": "INT8", "scale": repr(128 / 3.3)})
    x = rng.normal(0, 1.2, shape).astype(np.float32)
    x.reshape(-1)[:8] = [0.5 * 2.7 / 128, -0.5 * 2.7 / 128, 1.5 * 2.7 / 128, 2.5 * 2.7 / 128, 100, -100, 0, -0.0]
    assert_exact(run_both(b.text(), b.weights, {"f": x},
                          ["f_i8_host", "f_bf16", "i8_f32", "i8_bf16", "bf16_i8", "f32_i8_tpu"]))


def test_quant_bf16_overflow_and_wide_channels():
    """int8 -> bf16 products that round past max-finite become +0x7f7f for either sign (F32ToBF16), and the
    16-value vector path covers a 255-channel tensor's padding lane."""
    rng = np.random.default_rng(66)
    shape = (1, 255, 6, 6)
    b = graphs.GraphBuilder(66, simulate=False)
    b.op("input", "x", [], shape, "INT8")
    b.op("quant", "big", ["x"], shape, "BF16", **{"from": "INT8", "to": "BF16", "scale": "3.0e36"})
    # (BF16 -> INT8 of magnitudes past int32 is an undefined float-to-int cast in the reference: not compared)
    b.op("quant", "small", ["x"], shape, "BF16", **{"from": "INT8", "to": "BF16", "scale": repr(1.0 / 3)})
    b.op("quant", "small_i8", ["small"], shape, "INT8", **{"from": "BF16", "to": "INT8", "scale": "2.5"})
    assert_exact(run_both(b.text(), b.weights, {"x": i8(rng, shape)}, ["big", "small", "small_i8"]))


@pytest.mark.parametrize("kind", ["sigmoid", "mish", "exp", "tanh"])
def test_lut_bf16_slope(kind):
    rng = np.random.default_rng(7)
    shape = (2, 24, 9, 9)
    base, slope = oracle.lut_slope_tables(kind)
    b = graphs.GraphBuilder(7, simulate=False)
    b.op("input", "x", [], shape, "BF16")
    # the reference replicates each 256-entry table per TPU lane ([1, lanes, 32, 8]); only the first 256 are read
    b.weight("t0", np.tile(base, 8)), b.weight("t1", np.tile(slope, 8))
    b.op(kind, "y", ["x", "t0", "t1"], shape, "BF16")
    x = bf16(rng.normal(0, 5, shape))
    x.reshape(-1)[:6] = bf16([0.0, 20.0, -20.0, 127.9, -128.5, 7.96875])
    assert_exact(run_both(b.text(), b.weights, {"x": x}, ["y"]))


def test_lut_bf16_reciprocal():
    rng = np.random.default_rng(8)
    shape = (1, 16, 10, 10)
    e, m = oracle.lut_pow_tables(-1.0)
    b = graphs.GraphBuilder(8, simulate=False)
    b.op("input", "x", [], shape, "BF16")
    b.weight("t0", e), b.weight("t1", m)
    b.op("reciprocal", "y", ["x", "t0", "t1"], shape, "BF16")
    x = bf16(np.concatenate([rng.uniform(1e-3, 1e3, 1200), -rng.uniform(1e-3, 1e3, 400)]).reshape(shape))
    x.reshape(-1)[:4] = [0.0, 1.0, 2.0, 0.5]
    assert_exact(run_both(b.text(), b.weights, {"x": x}, ["y"]))


def test_fp32_ops():
    rng = np.random.default_rng(9)
    b = graphs.GraphBuilder(9, simulate=False)
    b.op("input", "x", [], (2, 3, 20, 20), "FP32")
    w1 = rng.normal(0, 0.2, (24, 3, 7, 7)).astype(np.float32)
    b.weight("w1", w1), b.weight("b1", rng.normal(0, 0.1, 24))
    b.op("conv_2d", "c1", ["x", "w1", "b1"], (2, 24, 10, 10), "FP32", kh=7, kw=7, sh=2, sw=2, pt=3, pb=3, pl=3, pr=3,
         do_relu=1, with_bias=1)
    b.op("pool_max_2d", "p1", ["c1"], (2, 24, 5, 5), "FP32", kh=3, kw=3, sh=2, sw=2, pt=0, pb=1, pl=0, pr=1)
    w2 = rng.normal(0, 0.1, (70, 24, 3, 3)).astype(np.float32)
    b.weight("w2", w2)
    b.op("conv_2d", "c2", ["p1", "w2", None], (2, 70, 5, 5), "FP32", kh=3, kw=3, sh=1, sw=1, pt=1, pb=1, pl=1, pr=1,
         do_relu=0, with_bias=0)
    w3 = rng.normal(0, 0.1, (70, 24, 1, 1)).astype(np.float32)
    b.weight("w3", w3), b.weight("b3", rng.normal(0, 0.1, 70))
    b.op("conv_2d", "c3", ["p1", "w3", "b3"], (2, 70, 5, 5), "FP32", kh=1, kw=1, do_relu=0, with_bias=1)
    b.op("eltwise_add", "add", ["c2", "c3"], (2, 70, 5, 5), "FP32", do_relu=1)
    b.weight("sc", rng.normal(1, 0.1, 70)), b.weight("sb", rng.normal(0, 0.1, 70))
    b.op("scale", "scl", ["add", "sc", "sb"], (2, 70, 5, 5), "FP32")
    b.op("pool_avg_2d", "gap", ["scl"], (2, 70, 1, 1), "FP32", kh=5, kw=5, sh=5, sw=5, count_include_pad=1)
    b.weight("fw", rng.normal(0, 0.1, (11, 70))), b.weight("fb", rng.normal(0, 0.1, 11))
    b.op("fully_connected", "fc", ["gap", "fw", "fb"], (2, 11), "FP32", do_relu=0)
    b.op("softmax", "prob", ["fc"], (2, 11), "FP32", axis=1)
    x = rng.normal(0, 1, (2, 3, 20, 20)).astype(np.float32)
    assert_close(run_both(b.text(), b.weights, {"x": x}, ["c1", "p1", "c2", "c3", "add", "scl", "gap", "fc", "prob"]))


def test_generic_mlir_graph_runs(tmp_path):
    """A graph in the reference's generic .mlir form, weights in the npz it names, loaded with load_mlir."""
    from tests.test_mlir_text import MLIR, tiny_weights
    from tpu_compiler_b200 import mlir_text, module
    (tmp_path / "tiny.mlir").write_text(MLIR)
    np.savez(tmp_path / "tiny_net_1a2b3c4d.npz", **tiny_weights())
    m = module(0)
    m.load_mlir(str(tmp_path / "tiny.mlir"))
    x = np.random.default_rng(3).normal(0, 1, (2, 3, 16, 16)).astype(np.float32)
    out = m.run(x)
    text, _ = mlir_text.convert(MLIR)
    ref = graph_runner.run(text, tiny_weights(), {"image": x})
    assert_close({"prob": (out["prob"], ref["prob"]), "stem": (m.get_tensor("stem"), ref["stem"])})
    assert m.get_weight_file_path().endswith("tiny_net_1a2b3c4d.npz")
    m.close()
