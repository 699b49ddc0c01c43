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
