"""The reader of the reference's generic-form TPU-dialect .mlir text (format test, CPU): a small
hand-written graph in that form converts to the module text the oracle and the backend both run."""
import numpy as np

from oracle import graph_runner
from tpu_compiler_b200 import mlir_text

MLIR = """
module {
  func @tpu_func(%arg0: tensor<2x3x16x16xf32>) -> tensor<2x10xf32> {
    %0 = "tpu.weight_file"() {filename = "tiny_net_1a2b3c4d.npz"} : () -> memref<10xf32>
    %1 = "tpu.input"(%arg0) {name = "image", quant = {mode = "NONE", param_type = "NONE", threshold = 0.000000e+00 : f32}} : (tensor<2x3x16x16xf32>) -> tensor<2x3x16x16xf32>
    %2 = "tpu.load_weight"(%0) {name = "stem.weight", storage = "NONE"} : (memref<10xf32>) -> tensor<8x3x3x3xf32>
    %3 = "tpu.load_weight"(%0) {name = "stem.bias", storage = "NONE"} : (memref<10xf32>) -> tensor<8xf32>
    %4 = "tpu.none"() : () -> none
    %5 = "tpu.conv_2d"(%1, %2, %3, %4, %4, %4, %4) {name = "stem", param = {dilation_h = 1 : i32, dilation_w = 1 : i32, do_relu = true, group = 1 : i32, ins = [], is_dw = false, pad_value = 0 : i32, padding = "SAME", padding_b = 1 : i32, padding_l = 1 : i32, padding_r = 1 : i32, padding_t = 1 : i32, stride_h = 2 : i32, stride_w = 2 : i32, with_bias = true}, quant = {mode = "NONE", param_type = "NONE", threshold = 0.000000e+00 : f32}} : (tensor<2x3x16x16xf32>, tensor<8x3x3x3xf32>, tensor<8xf32>, none, none, none, none) -> tensor<2x8x8x8xf32>
    %6 = "tpu.pool_avg_2d"(%5, %4, %4, %4, %4) {name = "gap", param = {count_include_pad = true, do_relu = false, kernel_h = 8 : i32, kernel_w = 8 : i32, pad_value = 0 : i32, padding_b = 0 : i32, padding_l = 0 : i32, padding_r = 0 : i32, padding_t = 0 : i32, stride_h = 8 : i32, stride_w = 8 : i32}, quant = {mode = "NONE", param_type = "NONE", threshold = 0.000000e+00 : f32}} : (tensor<2x8x8x8xf32>, none, none, none, none) -> tensor<2x8x1x1xf32>
    %7 = "tpu.reshape"(%6) {name = "flat"} : (tensor<2x8x1x1xf32>) -> tensor<2x8xf32>
    %8 = "tpu.load_weight"(%0) {name = "head.weight", storage = "NONE"} : (memref<10xf32>) -> tensor<10x8xf32>
    %9 = "tpu.load_weight"(%0) {name = "head.bias", storage = "NONE"} : (memref<10xf32>) -> tensor<10xf32>
    %10 = "tpu.fully_connected"(%7, %8, %9, %4, %4, %4, %4) {name = "head", quant = {mode = "NONE", param_type = "NONE", threshold = 0.000000e+00 : f32}} : (tensor<2x8xf32>, tensor<10x8xf32>, tensor<10xf32>, none, none, none, none) -> tensor<2x10xf32>
    %11 = "tpu.softmax"(%10) {axis = 1 : i32, name = "prob", quant = {mode = "NONE", param_type = "NONE", threshold = 0.000000e+00 : f32}} : (tensor<2x10xf32>) -> tensor<2x10xf32>
    return %11 : tensor<2x10xf32>
  }
}
"""


def tiny_weights():
    rng = np.random.default_rng(12)
    return {"stem.weight": rng.normal(0, 0.3, (8, 3, 3, 3)).astype(np.float32),
            "stem.bias": rng.normal(0, 0.1, 8).astype(np.float32),
            "head.weight": rng.normal(0, 0.3, (10, 8)).astype(np.float32),
            "head.bias": rng.normal(0, 0.1, 10).astype(np.float32)}


def test_convert_generic_form():
    text, wf = mlir_text.convert(MLIR)
    assert wf == "tiny_net_1a2b3c4d.npz"
    ops = graph_runner.parse(text)
    assert [o["type"] for o in ops] == ["input", "conv_2d", "pool_avg_2d", "reshape", "fully_connected", "softmax"]
    conv = ops[1]
    assert conv["in"] == ["image", "stem.weight", "stem.bias", "-", "-", "-", "-"]
    assert conv["shape"] == [2, 8, 8, 8] and conv["dtype"] == "FP32"
    a = conv["attrs"]
    assert (a["kh"], a["kw"], a["sh"], a["sw"], a["pt"], a["pl"], a["do_relu"], a["with_bias"]) == \
        ("3", "3", "2", "2", "1", "1", "1", "1")
    assert ops[2]["attrs"]["kh"] == "8" and ops[2]["attrs"]["count_include_pad"] == "1"
    assert ops[3]["shape"] == [2, 8] and ops[5]["attrs"]["axis"] == "1"
    # and the oracle runs it
    x = np.random.default_rng(3).normal(0, 1, (2, 3, 16, 16)).astype(np.float32)
    out = graph_runner.run(text, tiny_weights(), {"image": x})
    assert out["prob"].shape == (2, 10) and abs(out["prob"].sum() - 2.0) < 1e-4


def test_attr_parser_nested():
    d = mlir_text._AttrParser('{axis = 1 : i32, name = "c", q = {mode = "INT8", t = 1.500000e+00 : f32}, o = [ 1 : i32, 0 : i32 ], f = false}').dict()
    assert d == {"axis": 1, "name": "c", "q": {"mode": "INT8", "t": 1.5}, "o": [1, 0], "f": False}


def test_reference_backend_fixtures_parse():
    """Format test on the reference's own single-op graphs (lib/Dialect/TPU/Backend/test/*.mlir), read as text where
    a checkout is reachable: every file converts, and the ones made only of ops this backend implements are
    counted (those are the graphs the command line can run)."""
    import glob
    import os
    import pytest
    from .conftest import reference_dir
    ref = reference_dir()
    if ref is None:
        pytest.skip("no reference checkout reachable")
    files = sorted(glob.glob(os.path.join(ref, "lib", "Dialect", "TPU", "Backend", "test", "*.mlir")))
    assert len(files) >= 30
    implemented = {"input", "quant", "conv_2d", "deconv_2d", "fully_connected", "pool_max_2d", "pool_avg_2d", "eltwise_add",
                   "eltwise_mul", "eltwise_max", "eltwise_min", "broadcast_add", "broadcast_sub", "broadcast_mul", "pad",
                   "crop", "permute", "reduce_mean", "reduce_sum", "reduce_max", "reduce_min", "reduce_l2", "matmul",
                   "concat", "upsample", "pixelshuffle", "relu", "leaky_relu", "sigmoid", "mish", "exp", "tanh",
                   "reciprocal", "scale", "batchnorm", "softmax", "reshape"}
    runnable = 0
    for f in files:
        with open(f) as fh:
            text, _ = mlir_text.convert(fh.read())
        ops = graph_runner.parse(text)
        assert ops and ops[0]["type"] == "input", f
        assert all(o["shape"] for o in ops), f
        runnable += all(o["type"] in implemented for o in ops)
    assert runnable >= 19
