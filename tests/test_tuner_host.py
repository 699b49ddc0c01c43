"""Host logic of the incremental tuner (which ops a candidate re-runs, candidate sharing, the store
of INT8 activations) with the device module replaced by a stand-in over the CPU oracle: the result
must equal the reference's loop run as written (whole-module re-quantisation per candidate)."""
import numpy as np
import pytest

from oracle import graph_runner
from tpu_compiler_b200 import quantize as Q
from tpu_compiler_b200.tuner import SimpleTuner, ThresholdTable

from .test_gpu_tuner import N, reference_order_tuner, small_fp32_net


class OracleModule:
    """The slice of the ``module`` interface the tuner uses, computed by the CPU oracle."""

    def __init__(self, device=0):
        self.T, self.inputs = {}, {}

    def set_option(self, key, value):
        pass

    def load_text(self, text, weights):
        self.text, self.weights = text, dict(weights)
        self.ops = Q.parse_text(text)

    def set_tensor(self, name, array):
        self.inputs[name] = np.asarray(array, np.float32)
        self.T[name] = self.inputs[name]

    def copy_tensor_from(self, name, other, other_name):
        self.set_tensor(name, other.T[other_name])

    def invoke(self):
        self.T.update(graph_runner.run(self.text, self.weights, self.inputs))

    def sync(self):
        pass

    def get_tensor(self, name):
        return self.T[name]

    def get_data_type(self, name):
        return {o["name"]: o["dtype"] for o in self.ops}[name]

    def tuner_distance(self, name, ref, ref_name, scale):
        a, q = ref.T[ref_name], self.T[name]
        out = np.zeros((a.shape[0], 2))
        for i in range(a.shape[0]):
            diff = a[i].flatten() - q[i].flatten().astype(np.float32) * np.float32(scale)
            out[i] = (np.sum(diff.astype(np.float64) ** 2), np.abs(a[i].astype(np.float64)).sum())
        return out

    def close(self):
        pass


@pytest.mark.parametrize("image_scale", [1.0, 0.02])  # 0.02: every threshold below 1, where the table text rounds
def test_incremental_tuner_equals_reference_order_loop(image_scale):
    rng = np.random.default_rng(77)
    text, weights = small_fp32_net(rng)
    images = (rng.normal(0, 1, (N, 3, 16, 16)).clip(-3, 3) * image_scale).astype(np.float32)
    if image_scale != 1.0:
        weights = {k: (v * image_scale if k.endswith("_b") else v) for k, v in weights.items()}
    fp32 = graph_runner.run(text, weights, {"data": images})
    absmax = {k: float(np.abs(v).max()) for k, v in fp32.items()}
    factors = [(1.0, 0.6, 0.35), (0.6, 1.0, 0.35), (0.35, 0.6, 1.0)]
    names = [o["name"] for o in Q.parse_text(text)]
    cand_map = {"t%d" % k: {n: absmax[n] * factors[i % 3][k] for i, n in enumerate(names)} for k in range(3)}
    cand_map["t2"]["c2a"] = 0.0
    tuner = SimpleTuner(text, weights, cand_map, None, images, module_cls=OracleModule)
    got = tuner.run()
    exp_table, exp_d = reference_order_tuner(text, weights, cand_map, images, fp32)
    for n in names[1:]:
        assert set(tuner.distances[n]) == set(exp_d[n]), n
        for t, d in exp_d[n].items():
            assert abs(tuner.distances[n][t] - d) <= 1e-6 * abs(d), (n, t)
        assert got[n] == exp_table[n], n
    # c1's threshold is overwritten by its max pool's, so its three candidates share one copy
    assert tuner.launches == len(names) - 1
    assert tuner.ops_run < 3 * (len(names) - 1) + 3
    if image_scale != 1.0:
        assert max(got.values()) < 1.0 and any(np.float32("{:.7f}".format(v)) != np.float32(v) for v in got.values())
    qtext, qw = Q.quantize_module(text, weights, {k: np.float32("{:.7f}".format(v)) for k, v in got.items()})
    allw = dict(weights)
    allw.update(qw)
    oracle_q = graph_runner.run(qtext, allw, {"data": images})
    for n in names[1:]:
        np.testing.assert_array_equal(tuner.store.get_tensor(n), oracle_q[n], err_msg=n)


def test_threshold_table_file_format(tmp_path):
    t = ThresholdTable({"a": {"x": 1.5, "y": 2.0}, "b": {"x": 1.0, "y": 2.5}}, {"x": (-1.0, 2.0, 2.0), "y": (0.0, 3.0, 3.0)})
    assert t.candidate_thresholds("x") == [1.5, 1.0] and t.thresholds_map == {"x": 1.5, "y": 2.0}
    p = tmp_path / "table.txt"
    t.update_to(str(p), "y", 2.5)
    assert p.read_text().splitlines() == ["x 1.5000000 -1.0000000 2.0000000", "y 2.5000000 0.0000000 3.0000000"]
    t.update("y", 2.5)
    assert t.thresholds_map["y"] == 2.5
