"""GPU parity of the threshold auto-tuner (tpu_compiler_b200/tuner.py) against the reference's loop
run as written (kld_calibrator.py:156-201): per op and candidate, re-quantise the WHOLE module,
run it on the CPU oracle from the input up to the op, take the numpy distance. The incremental
device tuner must reach the same distances and pick the same thresholds; the INT8 tensors it
keeps must be the oracle's bit for bit."""
import numpy as np
import pytest

from oracle import graph_runner
from tpu_compiler_b200 import quantize as Q

pytestmark = pytest.mark.gpu

N = 4


def small_fp32_net(rng):
    w = {}

    def conv(name, src, ic, oc, k, hw, relu, pad):
        w[name + "_f"] = rng.normal(0, np.sqrt(2.0 / (ic * k * k)), (oc, ic, k, k)).astype(np.float32)
        w[name + "_b"] = rng.normal(0, 0.1, oc).astype(np.float32)
        return ("conv_2d name=%s in=%s,%s_f,%s_b shape=%d,%d,%d,%d dtype=FP32 kh=%d kw=%d sh=1 sw=1 pt=%d pb=%d pl=%d pr=%d "
                "dh=1 dw=1 g=1 do_relu=%d with_bias=1" % (name, src, name, name, N, oc, hw, hw, k, k, pad, pad, pad, pad, relu))

    lines = ["input name=data shape=%d,3,16,16 dtype=FP32" % N,
             conv("c1", "data", 3, 16, 3, 16, 1, 1),
             "pool_max_2d name=p1 in=c1 shape=%d,16,8,8 dtype=FP32 kh=2 kw=2 sh=2 sw=2 pt=0 pb=0 pl=0 pr=0" % N,
             conv("c2a", "p1", 16, 16, 1, 8, 1, 0),
             conv("c2b", "c2a", 16, 32, 3, 8, 0, 1),
             conv("sc", "p1", 16, 32, 1, 8, 0, 0),
             "eltwise_add name=add in=sc,c2b shape=%d,32,8,8 dtype=FP32 do_relu=1" % N,
             "pool_avg_2d name=gap in=add shape=%d,32,1,1 dtype=FP32 kh=8 kw=8 sh=8 sw=8 count_include_pad=1" % N]
    w["fc_f"] = rng.normal(0, 0.2, (10, 32)).astype(np.float32)
    w["fc_b"] = rng.normal(0, 0.1, 10).astype(np.float32)
    lines.append("fully_connected name=fc in=gap,fc_f,fc_b shape=%d,10 dtype=FP32 do_relu=0" % N)
    return "\n".join(lines) + "\n", w


def reference_order_tuner(text, weights, cand_map, images, ref_act):
    """SimpleTuner.run as the reference writes it, on the CPU oracle."""
    ops = Q.parse_text(text)
    cands = {}
    for _, m in cand_map.items():
        for op, t in m.items():
            cands.setdefault(op, []).append(t)
    table = {k: v[0] for k, v in cands.items()}
    dists = {}
    for op in ops:
        name = op["name"]
        if op["type"] == "input":
            continue
        best, minimum = cands[name][0], float("inf")
        dists[name] = {}
        for t in cands[name]:
            if t <= 1e-6:
                continue
            trial = dict(table)
            trial[name] = t
            # the trial table reaches the quantiser through a text file (kld_calibrator.py:98-108, 175-177)
            trial = {k: np.float32("{:.7f}".format(v)) for k, v in trial.items()}
            qtext, qw = Q.quantize_module(text, weights, trial, upto=name)
            allw = dict(weights)
            allw.update(qw)
            out = graph_runner.run(qtext, allw, {"data": images})[name]
            distance = 0.0
            for i in range(images.shape[0]):
                target = out[i].astype(np.float32) * (t / 127.0)
                ref = ref_act[name][i]
                diff = ref.flatten() - target.flatten()
                distance += np.linalg.norm(diff) / np.linalg.norm(ref.flatten(), ord=1)
            dists[name][t] = float(distance)
            if distance < minimum:
                best, minimum = t, distance
        table[name] = best
    return table, dists


@pytest.mark.parametrize("image_scale", [1.0, 0.02])  # 0.02: every threshold below 1, where the table text rounds
def test_tuner_matches_reference_order_loop(image_scale):
    from tpu_compiler_b200.tuner import SimpleTuner
    rng = np.random.default_rng(77)
    text, weights = small_fp32_net(rng)
    images = (rng.normal(0, 1, (N, 3, 16, 16)).clip(-3, 3) * image_scale).astype(np.float32)
    if image_scale != 1.0:
        weights = {k: (v * image_scale if k.endswith("_b") else v) for k, v in weights.items()}
    fp32 = graph_runner.run(text, weights, {"data": images})
    absmax = {k: float(np.abs(v).max()) for k, v in fp32.items()}
    # three candidate tables; the order differs per op so that "first" is not always the largest
    factors = [(1.0, 0.6, 0.35), (0.6, 1.0, 0.35), (0.35, 0.6, 1.0)]
    names = [o["name"] for o in Q.parse_text(text)]
    cand_map = {"t%d" % k: {n: absmax[n] * factors[i % 3][k] for i, n in enumerate(names)} for k in range(3)}
    cand_map["t2"]["c2a"] = 0.0  # a candidate the loop must skip

    tuner = SimpleTuner(text, weights, cand_map, None, images)
    try:
        ref_act = {n: tuner.ref_fp32_activation(n) for n in names}
        for n in names:  # the resident fp32 activations are the oracle's within the fp32 tolerance
            rngv = max(absmax[n], 1e-6)
            assert np.abs(ref_act[n] - fp32[n]).max() <= 1e-4 * rngv, n
        got = tuner.run()
        exp_table, exp_d = reference_order_tuner(text, weights, cand_map, images, ref_act)
        for n in names[1:]:
            assert set(tuner.distances[n]) == set(exp_d[n]), n
            for t, d in exp_d[n].items():
                assert abs(tuner.distances[n][t] - d) <= 1e-5 * abs(d) + 1e-12, (n, t, tuner.distances[n][t], d)
            assert got[n] == exp_table[n], n
        # the INT8 tensors kept on the device are those of the whole-graph quantisation under the final table
        qtext, qw = Q.quantize_module(text, weights, {k: np.float32("{:.7f}".format(v)) for k, v in got.items()})
        allw = dict(weights)
        allw.update(qw)
        oracle_q = graph_runner.run(qtext, allw, {"data": images})
        for n in names[1:]:
            np.testing.assert_array_equal(tuner.store.get_tensor(n), oracle_q[n], err_msg=n)
        # far fewer op executions than re-running every prefix: 8 ops x 3 candidates would be 108 prefix ops
        assert tuner.launches == len(names) - 1
        assert tuner.ops_run <= 3 * (len(names) - 1) + 3
    finally:
        tuner.close()


def test_distance_entry_point_against_numpy():
    from tpu_compiler_b200 import module
    rng = np.random.default_rng(5)
    for c, hw in ((5, 7), (16, 4), (35, 3)):
        a = rng.normal(0, 2, (3, c, hw, hw)).astype(np.float32)
        q = rng.integers(-128, 128, (3, c, hw, hw)).astype(np.float32)
        m1, m2 = module(0), module(0)
        m1.load_text("input name=x shape=3,%d,%d,%d dtype=FP32\n" % (c, hw, hw), {})
        m2.load_text("input name=y shape=3,%d,%d,%d dtype=INT8\ninput name=z shape=3,%d,%d,%d dtype=FP32\n"
                     % (c, hw, hw, c, hw, hw), {})
        m1.set_tensor("x", a)
        m2.set_tensor("y", q)
        m2.set_tensor("z", q * np.float32(0.5))
        scale = np.float32(3.3 / 127.0)
        for name, s in (("y", scale), ("z", np.float32(1.0))):
            sums = m2.tuner_distance(name, m1, "x", s)
            tv = q if name == "y" else q * np.float32(0.5)
            for i in range(3):
                diff = a[i].flatten() - (tv[i].flatten() * s)
                assert abs(sums[i, 0] - float(np.sum(diff.astype(np.float64) ** 2))) <= 1e-9 * sums[i, 0]
                assert abs(sums[i, 1] - float(np.abs(a[i].astype(np.float64)).sum())) <= 1e-9 * sums[i, 1]
        m3 = module(0)
        m3.load_text("input name=y2 shape=3,%d,%d,%d dtype=INT8\n" % (c, hw, hw), {})
        m3.copy_tensor_from("y2", m2, "y")
        np.testing.assert_array_equal(m3.get_tensor("y2"), q)
        with pytest.raises(RuntimeError):
            m3.copy_tensor_from("y2", m2, "z")
        for m in (m1, m2, m3):
            m.close()
