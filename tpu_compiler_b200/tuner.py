"""Threshold auto-tuner: ``ThresholdTable`` and ``SimpleTuner`` of the reference's
python/cvi_toolkit/calibration/kld_calibrator.py:75-201, with every activation left on the GPU.

The reference loop, per op and per candidate threshold, writes a table, re-quantises the whole
fp32 module, runs the INT8 graph from the input up to the op on every image, copies the op's
output to numpy and takes ``sum_i ||ref_i - q_i * threshold / 127||_2 / ||ref_i||_1`` against the
fp32 activations of a first run. The best candidate is kept before the next op is tuned.

Here the same decisions come out of far less work:

* the fp32 activations of all images stay resident in one fp32 module (batch = image count);
* the INT8 activations under the thresholds chosen so far stay resident in a "store" module, so
  tuning an op re-runs only the ops whose quantisation parameters the candidate changes (the op
  itself; also its producer when the threshold travels backwards through a max pool) instead of
  the whole prefix of the graph;
* all candidates of an op are quantised into ONE small module (a copy of the changed ops per
  candidate, reading shared inputs), launched once; candidates that lead to the same effective
  parameters share one copy;
* both norms are taken on the device (``tpucb_tuner_distance``); 16 bytes per image come back.

Which ops a candidate changes is decided by comparing quantisation signatures (own threshold and
operand thresholds after the reference's overwrite rules), and every threshold reaches the
quantiser as the reference's does, through the ``'{:.7f}'`` text of a trial table
(``through_table_text``), so the INT8 tensors are exactly those of the reference's whole-graph
re-quantisation.
"""
import numpy as np

from . import quantize as Q
from .interpreter import module

SKIP_TYPES = ("input", "softmax", "reshape")


def through_table_text(threshold):
    """The value the reference's quantiser sees for a threshold: every trial table goes through a text file
    (``update_to`` writes ``'{:.7f}'``, kld_calibrator.py:98-108) that ImportCalibrationTable.cpp:274-290 parses back
    into a float. Below 1 that round trip changes most float32 values."""
    return np.float32("{:.7f}".format(float(threshold)))


class ThresholdTable:
    """kld_calibrator.py:75-111. ``candidate_threshold_map``: {key: {op name: threshold}}, one entry
    per candidate table (e.g. per histogram setting); the first entry is the starting point."""

    def __init__(self, candidate_threshold_map, activations_statistics=None):
        self.candidate_threshold_map = self.transform_threshold_map(candidate_threshold_map)
        self.activations_statistics = activations_statistics or {}
        self.thresholds_map = {k: v[0] for k, v in self.candidate_threshold_map.items()}

    @staticmethod
    def transform_threshold_map(candidate_threshold_map):
        out = {}
        for _, m in candidate_threshold_map.items():
            for op, threshold in m.items():
                out.setdefault(op, []).append(threshold)
        return out

    def table_with(self, target_op, new_threshold):
        """The table a quantiser reads for this trial: every entry as it comes back from the text file. The
        unrounded candidate stays the caller's (distance scale, returned best threshold), as in the reference."""
        t = {k: through_table_text(v) for k, v in self.thresholds_map.items()}
        t[target_op] = through_table_text(new_threshold)
        return t

    def update_to(self, dest_table, target_op, new_threshold):
        trial = dict(self.thresholds_map)
        trial[target_op] = new_threshold
        with open(dest_table, "w") as f:
            for k, v in trial.items():
                mn, mx = (self.activations_statistics.get(k) or (0.0, 0.0, 0.0))[:2]
                f.write("{} {:.7f} {:.7f} {:.7f}\n".format(k, v, mn, mx))

    def update(self, target_op, best_threshold):
        self.thresholds_map[target_op] = best_threshold

    def candidate_thresholds(self, target_op):
        return self.candidate_threshold_map[target_op]


def distance_from_sums(sums):
    """sum over images of ||diff||_2 / ||ref||_1 from the per-image (sum diff^2, sum |ref|)."""
    with np.errstate(divide="ignore", invalid="ignore"):
        return float(np.sum(np.sqrt(sums[:, 0]) / sums[:, 1]))


class SimpleTuner:
    """kld_calibrator.py:113-201. ``text`` / ``weights``: the fp32 module with batch = number of
    images; ``images``: {input name: float32 array [images, ...]} (or one array for a single
    input)."""

    def __init__(self, text, weights, thresholds_map, activations_statistics, images, device=0, log=None,
                 module_cls=module):
        self.text, self.weights, self.device = text, weights, device
        self._module = module_cls  # the pymlir-shaped class that runs module text (tests substitute a CPU stand-in)
        self.ops = Q.parse_text(text)
        self.by_name = {op["name"]: op for op in self.ops}
        self.threshold_table = ThresholdTable(thresholds_map, activations_statistics)
        self.log = log or (lambda s: None)
        self.inputs = [op["name"] for op in self.ops if op["type"] == "input"]
        if not isinstance(images, dict):
            images = {self.inputs[0]: images}
        self.image_num = int(self.by_name[self.inputs[0]]["shape"][0])
        self.distances = {}   # op -> {threshold: distance}, filled by run()
        self.launches = 0     # candidate modules launched
        self.ops_run = 0      # INT8 op instances executed over all candidates
        self._pre_run(images)

    # ---- fp32 reference activations, resident --------------------------------------------------
    def _pre_run(self, images):
        self.ref = self._module(self.device)
        self.ref.load_text(self.text, self.weights)
        for name in self.inputs:
            self.ref.set_tensor(name, np.ascontiguousarray(images[name], np.float32))
        self.ref.invoke()
        self.ref.sync()
        # every INT8 activation under the thresholds chosen so far, as input ops of a module that computes nothing
        lines = []
        for op in self.ops:
            if op["type"] in ("input", "softmax"):
                continue
            lines.append(Q.format_op({"type": "input", "name": op["name"], "in": [], "shape": op["shape"],
                                      "dtype": "INT8", "attrs": {}}))
        self.store = self._module(self.device)
        self.store.load_text("\n".join(lines) + "\n", {})
        self.sig = {}  # op name -> signature its stored tensor was computed with

    def ref_fp32_activation(self, name):
        return self.ref.get_tensor(name)

    # ---- which ops a table changes ---------------------------------------------------------------
    def _ancestors(self, target):
        need, order = {target}, []
        for op in reversed(self.ops):
            if op["name"] in need:
                order.append(op)
                need.update(Q.activation_operands(op, self.by_name))
        return list(reversed(order))

    def _recompute_set(self, target, thr):
        """Ancestors-or-self of ``target`` (program order, inputs and softmax excluded) whose stored
        INT8 tensor is not the one the effective thresholds ``thr`` give, with their signatures."""
        out = {}
        for op in self._ancestors(target):
            if op["type"] in ("input", "softmax"):
                continue
            s = Q.quant_param_signature(op, thr, self.by_name)
            acts = Q.activation_operands(op, self.by_name)
            if op["name"] == target or self.sig.get(op["name"]) != s or any(a in out for a in acts):
                out[op["name"]] = s
        return out

    @staticmethod
    def _move(dst, dst_name, src, src_name):
        """Device-to-device when the two tensors share a device layout; a few-channel tensor that a
        stem convolution wants with padded rows is staged through the host instead."""
        try:
            dst.copy_tensor_from(dst_name, src, src_name)
        except RuntimeError as e:
            if "device layout" not in str(e):
                raise
            dst.set_tensor(dst_name, src.get_tensor(src_name))

    # ---- one op ------------------------------------------------------------------------------------
    def _tune_op(self, name, candidates):
        table = self.threshold_table
        variants, plan = [], {}  # variants: distinct (recompute set, effective thresholds); plan: candidate -> variant
        usable = [t for t in candidates if t > 1e-6]  # the reference skips the others (kld_calibrator.py:173-174)
        for t in usable or candidates[:1]:
            thr = Q.import_thresholds(self.ops, table.table_with(name, t))
            rs = self._recompute_set(name, thr)
            key = tuple(sorted(rs.items()))
            for vi, v in enumerate(variants):
                if v["key"] == key:
                    plan[t] = vi
                    break
            else:
                variants.append({"key": key, "rs": rs, "thr": thr})
                plan[t] = len(variants) - 1
        # one module for all variants
        ops_out, w_out, declared = [], {}, set()
        w64 = {}  # float64 filter copies shared by this op's candidates
        from_ref, from_store = [], []
        for vi, v in enumerate(variants):
            sfx = "__%d" % vi
            rename = {a: a + sfx for a in v["rs"]}
            for a in v["rs"]:
                op = self.by_name[a]
                for src in Q.activation_operands(op, self.by_name):
                    if src in v["rs"]:
                        continue
                    sop = self.by_name[src]
                    if sop["type"] == "input":
                        if src not in declared:
                            ops_out.append(dict(sop))
                            declared.add(src)
                            from_ref.append(src)
                        qn = src + "_quant_i8" + sfx
                        if qn not in declared:
                            ops_out.append(Q.input_quant_op(sop, v["thr"], out_name=qn))
                            declared.add(qn)
                        rename[src] = qn
                    elif src not in declared:
                        ops_out.append({"type": "input", "name": src, "in": [], "shape": sop["shape"], "dtype": "INT8",
                                        "attrs": {}})
                        declared.add(src)
                        from_store.append(src)
                new_ops, w = Q.quantize_op(op, v["thr"], self.weights, self.by_name, rename, out_name=a + sfx,
                                           cache=w64)
                ops_out += new_ops
                w_out.update(w)
                self.ops_run += 1
        sub = self._module(self.device)
        try:
            sub.set_option("cuda_graph", 0)
            sub.load_text("\n".join(Q.format_op(o) for o in ops_out) + "\n", w_out)
            for src in from_ref:
                self._move(sub, src, self.ref, src)
            for src in from_store:
                self._move(sub, src, self.store, src)
            sub.invoke()
            self.launches += 1
            is_int8 = sub.get_data_type(name + "__0") == "INT8"
            dist = {}
            for t in usable:
                vi = plan[t]
                scale = np.float32(t / 127.0) if is_int8 else np.float32(1.0)
                dist[t] = distance_from_sums(sub.tuner_distance(name + "__%d" % vi, self.ref, name, scale))
            best, minimum = candidates[0], float("inf")
            for t in candidates:
                if t in dist and dist[t] < minimum:
                    best, minimum = t, dist[t]
            kept = plan.get(best, 0)
            v = variants[kept]
            sfx = "__%d" % kept
            for a, s in v["rs"].items():
                self.store.copy_tensor_from(a, sub, a + sfx)
                self.sig[a] = s
        finally:
            sub.close()
        self.distances[name] = dist
        return best

    def run(self):
        for op in self.ops:
            name = op["name"]
            if op["type"] in SKIP_TYPES or name not in self.threshold_table.candidate_threshold_map:
                continue
            candidates = list(self.threshold_table.candidate_thresholds(name))
            best = self._tune_op(name, candidates)
            self.log("{} => threshold: {}".format(name, best))
            self.threshold_table.update(name, best)
        return self.threshold_table.thresholds_map

    def close(self):
        for m in (getattr(self, "ref", None), getattr(self, "store", None)):
            if m is not None:
                m.close()
