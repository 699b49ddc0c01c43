"""CPU checks of the oracle restatements of the layout / arithmetic ops of neighbouring networks against numpy's
slicing, padding and transposition, and of the INT8 arithmetic against its definition written out in integers."""
import numpy as np

import oracle as O


def _rs(v, r):  # (v + 2^(r-1)) >> r, saturated: applyRShiftAndSaturateInt8 on integers
    v = np.asarray(v, np.int64)
    q = v if r == 0 else (v + (1 << (r - 1))) >> r
    return np.clip(q, -128, 127).astype(np.float32)


def test_layout_ops_match_numpy():
    x = np.arange(2 * 3 * 4 * 5, dtype=np.float32).reshape(2, 3, 4, 5)
    assert np.array_equal(O.permute(x, [0, 2, 3, 1]), x.transpose(0, 2, 3, 1))
    assert np.array_equal(O.permute(x, [1, 0, 3, 2]), x.transpose(1, 0, 3, 2))
    assert np.array_equal(O.pad(x, [0, 0, 1, 2, 0, 0, 3, 1]), np.pad(x, ((0, 0), (0, 0), (1, 3), (2, 1))))
    assert np.array_equal(O.pad(x, [0, 1, 0, 0, 1, 0, 0, 0]), np.pad(x, ((0, 1), (1, 0), (0, 0), (0, 0))))
    assert np.array_equal(O.pad(x, [0, 0, 1, 2, 0, 0, 3, 1], "edge"), np.pad(x, ((0, 0), (0, 0), (1, 3), (2, 1)), mode="edge"))
    assert np.array_equal(O.pad(x, [0, 0, -1, 0, 0, -1, 0, -2]), x[:, :2, 1:, :3])
    assert np.array_equal(O.crop(x, [1, 2, 2, 2], [1, 1, 0, 1], [1, 1, 2, 2]), x[1:2, 1:3, 0:4:2, 1:5:2])
    assert np.array_equal(O.crop(x, [2, 1, 3, 4], [0, 2, 1, 0]), x[:, 2:3, 1:4, 0:4])


def test_reduce_matches_numpy_and_int8_rule():
    rng = np.random.default_rng(3)
    f = rng.normal(0, 1, (2, 5, 4, 3)).astype(np.float32)
    assert np.array_equal(O.reduce(f, [2, 3], "max", is_int8=False), f.max(axis=(2, 3)))
    assert np.array_equal(O.reduce(f, [1], "min", is_int8=False), f.min(axis=1))
    assert np.allclose(O.reduce(f, [1], "mean", is_int8=False), f.mean(axis=1), rtol=1e-6)
    assert np.allclose(O.reduce(f, [2, 3], "sum", is_int8=False), f.sum(axis=(2, 3)), rtol=1e-6)
    x = rng.integers(-128, 128, (2, 6, 7, 7)).astype(np.float32)
    got = O.reduce(x, [2, 3], "mean", is_int8=True, multiplier=167, rshift=13)
    exp = np.clip(np.floor(x.sum(axis=(2, 3)) * 167 / 2.0 ** 13 + 0.5), -128, 127)
    assert np.array_equal(got, exp.astype(np.float32))


def test_eltwise_maxmin_and_broadcast_int8_rules():
    rng = np.random.default_rng(4)
    a = rng.integers(-128, 128, (2, 4, 3, 5)).astype(np.float32)
    b = rng.integers(-128, 128, (2, 4, 3, 5)).astype(np.float32)
    m, r = [37, -21], 5
    ia, ib = a.astype(np.int64) * m[0], b.astype(np.int64) * m[1]
    assert np.array_equal(O.eltwise_maxmin_i8([a, b], m, r), _rs(np.maximum(ia, ib), r))
    assert np.array_equal(O.eltwise_maxmin_i8([a, b], m, r, do_relu=True), _rs(np.maximum(np.maximum(ia, ib), 0), r))
    assert np.array_equal(O.eltwise_maxmin_i8([a, b], m, r, is_min=True), _rs(np.minimum(ia, ib), r))
    c = rng.integers(-128, 128, (1, 4, 1, 1)).astype(np.float32)
    ic = c.astype(np.int64) * m[1]
    assert np.array_equal(O.broadcast(a, c, "add", multiplier=m, rshift=r), _rs(ia + ic, r))
    assert np.array_equal(O.broadcast(a, c, "sub", multiplier=m, rshift=r, do_relu=True), _rs(np.maximum(ia - ic, 0), r))
    v = rng.normal(0, 1, (5,)).astype(np.float32)
    assert np.array_equal(O.broadcast(a, v, "mul", is_int8=False), a * v)


def test_deconv_scatter_equals_conv_on_inserted_zeros():
    rng = np.random.default_rng(5)
    n, ic, oc, ih, iw, kh, kw, sh, sw, pt, pl = 2, 6, 8, 5, 4, 3, 4, 2, 3, 1, 2
    x = rng.integers(-128, 128, (n, ic, ih, iw)).astype(np.float32)
    w = rng.integers(-127, 128, (oc, ic, kh, kw)).astype(np.float32)
    bias = rng.integers(-1000, 1000, oc).astype(np.float32)
    mult = np.full(oc, 1.5e9, np.float32)
    rsh = np.full(oc, 9, np.float32)
    oh = (ih - 1) * sh - 2 * pt + kh
    ow = (iw - 1) * sw - 2 * pl + kw
    d = O.deconv2d_i8(x, w, bias, rsh, mult, (oh, ow), (sh, sw), (pt, pl))
    c = O.conv2d(x, w[:, :, ::-1, ::-1].copy(), bias, rsh, mult, (oh, ow), stride=(1, 1), pad=(kh - 1 - pt, kw - 1 - pl),
                 ins=(sh - 1, sw - 1))
    assert np.array_equal(d, c)


def test_softmax_bf16_golden():
    """BF16 softmax (and the log tables / "log" lookup under it) against vectors stepped over the reference's own
    compiled BF16 and table primitives (tests/golden/make_golden.py: make_softmax_bf16)."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "softmax_bf16.npz"))
    le, lm = O.lut_log_tables()
    assert np.array_equal(le.view(np.uint32), g["log_exp"].view(np.uint32))
    assert np.array_equal(lm.view(np.uint32), g["log_mant"].view(np.uint32))
    eb, es = O.lut_slope_tables("exp")
    assert np.array_equal(eb.view(np.uint32), g["exp_base"].view(np.uint32))
    assert np.array_equal(es.view(np.uint32), g["exp_slope"].view(np.uint32))
    for ci in range(3):
        for do_log in (0, 1):
            t = (g["log_exp"], g["log_mant"]) if do_log else (g["rec_exp"], g["rec_mant"])
            y = O.softmax_bf16(g["x%d" % ci], g["exp_base"], g["exp_slope"], t[0], t[1], axis=1, do_log=bool(do_log))
            assert np.array_equal(y.view(np.uint32), g["y%d_log%d" % (ci, do_log)].view(np.uint32)), (ci, do_log)


def test_matmul_oracle_against_numpy():
    """The matmul restatement against numpy in every storage order (exact in INT8 below 2^24)."""
    rng = np.random.default_rng(5)
    a = rng.integers(-128, 128, (2, 3, 7, 11)).astype(np.float32)
    b = rng.integers(-128, 128, (2, 3, 11, 5)).astype(np.float32)
    exp = np.einsum("xymk,xykn->xymn", a, b)
    y = O.matmul(a, b, (2, 3, 7, 5), mode="FP32")
    assert np.array_equal(y, exp)
    # transposed storage: left [bh, M, bl, K], right [bh, K, bl, N], out [bh, M, bl, N]
    at, bt = a.transpose(0, 2, 1, 3).copy(), b.transpose(0, 2, 1, 3).copy()
    yt = O.matmul(at, bt, (2, 7, 3, 5), mode="FP32", ltrans=True, rtrans=True, otrans=True)
    assert np.array_equal(yt, exp.transpose(0, 2, 1, 3))
    q = O.matmul(a, b, (2, 3, 7, 5), mode="INT8", rshift=9.0, multiplier=float(2 ** 30), do_relu=True)
    hi = np.floor((np.maximum(exp, 0).astype(np.int64) * 2 ** 30 + 2 ** 30) / 2.0 ** 31).astype(np.int64)
    ref = np.clip((hi + 256) >> 9, -128, 127)
    assert np.array_equal(q, ref.astype(np.float32))


def test_batchnorm_and_reduce_l2_against_numpy():
    """core/batchnorm.cpp:20-68 and the REDUCE_L2 case of core/reduce.cpp:91-103 written out with numpy in the
    reference's operation order and types."""
    rng = np.random.default_rng(8)
    x = rng.normal(0, 2, (2, 5, 3, 4)).astype(np.float32)
    mean, var = rng.normal(0, 1, 5).astype(np.float32), rng.uniform(0.1, 2, 5).astype(np.float32)
    scale0, eps = np.float32(0.8), np.float32(1e-5)
    sf = np.float32(1) / scale0
    m = (mean * sf).reshape(1, 5, 1, 1)
    d = np.sqrt(var * sf + eps).astype(np.float32).reshape(1, 5, 1, 1)
    assert np.array_equal(O.batchnorm_f32(x, mean, var, float(scale0), float(eps)), (x - m) / d)
    got = O.reduce_l2_f32(x, [1], 0.5)
    s = np.zeros((2, 3, 4), np.float32)
    for c in range(5):
        s = (s.astype(np.float64) + x[:, c].astype(np.float64) ** 2).astype(np.float32)
    assert np.allclose(got, np.sqrt(s), rtol=2e-7) and got.shape == (2, 3, 4)
