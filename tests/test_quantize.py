"""Host-side INT8 quantisation (tpu_compiler_b200/quantize.py) against golden vectors made by the
reference's own QuantizationArithmetic.cpp (tests/golden/make_golden.py weight_quant), and the
threshold overwrite rules of ImportCalibrationTable.cpp on small graphs. CPU only."""
import os

import numpy as np

from tpu_compiler_b200 import quantize as Q

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "weight_quant.npz"))


def test_conv_weight_quantiser_matches_reference():
    ci = 0
    while "conv%d_w" % ci in G:
        w, b, (ty, tx) = G["conv%d_w" % ci], G["conv%d_b" % ci], G["conv%d_t" % ci]
        nf, nb, r, m = Q.quantize_conv_weights(w, b if b.size else None, ty, tx)
        np.testing.assert_array_equal(r, G["conv%d_r" % ci])
        np.testing.assert_array_equal(m, G["conv%d_m" % ci])
        np.testing.assert_array_equal(nf, G["conv%d_nf" % ci])
        if b.size:
            np.testing.assert_array_equal(nb, G["conv%d_nb" % ci])
        ci += 1
    assert ci >= 6


def test_fc_weight_quantiser_matches_reference():
    ci = 0
    while "fc%d_w" % ci in G:
        w, b, (ty, tx) = G["fc%d_w" % ci], G["fc%d_b" % ci], G["fc%d_t" % ci]
        nf, nb, r, m = Q.quantize_fc_weights(w, b if b.size else None, ty, tx)
        np.testing.assert_array_equal(r, G["fc%d_r" % ci])
        np.testing.assert_array_equal(m, G["fc%d_m" % ci])
        np.testing.assert_array_equal(nf, G["fc%d_nf" % ci])
        if b.size:
            np.testing.assert_array_equal(nb, G["fc%d_nb" % ci])
        ci += 1
    assert ci >= 3


def test_no_weight_rescale_matches_reference():
    for q, r, m in zip(G["rescale_qscale"], G["rescale_rshift"], G["rescale_mult"]):
        n = int(np.count_nonzero(q))
        rr, mm = Q.rescale_from_qscale(list(q[:n]))
        assert int(rr[0]) == int(r)
        np.testing.assert_array_equal(mm, m[:n])


TEXT = """
input name=data shape=2,3,8,8 dtype=FP32
conv_2d name=c1 in=data,c1_f,c1_b shape=2,4,8,8 dtype=FP32 kh=3 kw=3 sh=1 sw=1 pt=1 pb=1 pl=1 pr=1 dh=1 dw=1 g=1 do_relu=1 with_bias=1
pool_max_2d name=p1 in=c1 shape=2,4,4,4 dtype=FP32 kh=2 kw=2 sh=2 sw=2 pt=0 pb=0 pl=0 pr=0
conv_2d name=c2 in=p1,c2_f,c2_b shape=2,4,4,4 dtype=FP32 kh=1 kw=1 sh=1 sw=1 pt=0 pb=0 pl=0 pr=0 dh=1 dw=1 g=1 do_relu=0 with_bias=1
pool_max_2d name=p2 in=c2 shape=2,4,2,2 dtype=FP32 kh=2 kw=2 sh=2 sw=2 pt=0 pb=0 pl=0 pr=0
eltwise_add name=add in=p1,c2 shape=2,4,4,4 dtype=FP32 do_relu=1
"""


def test_threshold_overwrite_rules():
    ops = Q.parse_text(TEXT)
    thr = Q.import_thresholds(ops, {"data": 1.0, "c1": 2.0, "p1": 3.0, "c2": 4.0, "p2": 5.0, "add": 6.0})
    # c1 has one use (p1): it takes p1's threshold backwards; c2 has two uses: p2 takes c2's forwards
    assert float(thr["c1"]) == 3.0 and float(thr["p1"]) == 3.0
    assert float(thr["c2"]) == 4.0 and float(thr["p2"]) == 4.0
    assert float(thr["data"]) == 1.0 and float(thr["add"]) == 6.0


def test_quantize_module_text():
    rng = np.random.default_rng(5)
    w = {"c1_f": rng.normal(0, 0.3, (4, 3, 3, 3)), "c1_b": rng.normal(0, 0.1, 4),
         "c2_f": rng.normal(0, 0.3, (4, 4, 1, 1)), "c2_b": rng.normal(0, 0.1, 4)}
    table = {"data": 1.0, "c1": 2.0, "p1": 3.0, "c2": 4.0, "p2": 5.0, "add": 6.0}
    text, qw = Q.quantize_module(TEXT, w, table)
    ops = {o["name"]: o for o in Q.parse_text(text)}
    assert ops["data_quant_i8"]["attrs"]["scale"] == repr(128.0)
    assert ops["c1"]["in"][0] == "data_quant_i8" and ops["c1"]["dtype"] == "INT8"
    assert ops["add"]["in"] == ["p1", "c2", None, None, "add_rshift", "add_multiplier"]
    # the add rescales 3.0 -> 6.0 and 4.0 -> 6.0: multipliers 0.5 and 0.667 at one common shift
    r, m = int(qw["add_rshift"][0]), qw["add_multiplier"]
    assert abs(m[0] / 2 ** r - 0.5) < 0.01 and abs(m[1] / 2 ** r - 2 / 3) < 0.01 and m.max() <= 127
    text2, _ = Q.quantize_module(TEXT, w, table, upto="c2")
    assert [o["name"] for o in Q.parse_text(text2)][-1] == "c2"
