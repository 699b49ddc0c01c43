"""fp32 module text + calibration thresholds -> INT8 module text, on the host.

This is the part of the reference's ``tpuc-opt --import-calibration-table --tpu-quant`` pipeline
that the auto-tuner re-runs for every candidate threshold (bindings/python/pytuner.cpp:139-170):

* ``import_thresholds``  lib/Dialect/TPU/Quantization/ImportCalibrationTable.cpp:317-395
  (table lookup, backward overwrite for pool_max / relu / leaky_relu / crop with a single-use
  producer, forward overwrite for the ops that never rescale);
* ``quantize_conv_weights``  quantizeWeightInt8Multiplier, QuantizationArithmetic.cpp:741-818;
* ``quantize_fc_weights``    quantizeWeightInt8ForFC, QuantizationArithmetic.cpp:630-690;
* ``rescale_no_weight``      quantizeInt8RescaleNoWeightOps, QuantizeInt8.cpp:669-854
  (eltwise_add, pool_avg_2d);
* the tpu.quant op after an fp32 producer, scale 128 / threshold  Quantization.cpp:180-186.

Every float / double choice of the C++ is kept (see the comments at each step) so that the
quantised weights, multipliers and shifts are the reference's bit for bit. Covered op set: input,
conv_2d (groups = 1 or depthwise), fully_connected, eltwise_add, pool_max_2d, pool_avg_2d,
reshape, relu, leaky_relu-free graphs; a softmax stays fp32 behind a dequantising tpu.quant
(TpuConvertSoftmaxToSoftmaxCpu). Anything else raises.
"""
import math

import numpy as np

f32 = np.float32

BACKWARD_OPS = ("leaky_relu", "relu", "crop", "pool_max_2d")
FORWARD_OPS = ("abs", "copy", "crop", "leaky_relu", "relu", "pad", "pixelshuffle", "permute", "pool_max_2d",
               "reorg", "reverse", "reduce_max", "reduce_min", "shuffle_channel", "swap_channel", "tile", "upsample")
NO_THRESHOLD = ("reshape",)


def parse_text(text):
    """Module text -> list of op dicts {type, name, in, shape, dtype, attrs} in program order."""
    ops = []
    for line in text.splitlines():
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        toks = line.split()
        op = {"type": toks[0], "name": None, "in": [], "shape": [], "dtype": "FP32", "attrs": {}}
        for t in toks[1:]:
            k, v = t.split("=", 1)
            if k == "name":
                op["name"] = v
            elif k == "in":
                op["in"] = [None if s == "-" else s for s in v.split(",")]
            elif k == "shape":
                op["shape"] = [int(d) for d in v.split(",")]
            elif k == "dtype":
                op["dtype"] = v
            else:
                op["attrs"][k] = v
        ops.append(op)
    return ops


def format_op(op):
    parts = [op["type"], "name=" + op["name"]]
    if op["in"]:
        parts.append("in=" + ",".join(i if i else "-" for i in op["in"]))
    parts.append("shape=" + ",".join(str(int(d)) for d in op["shape"]))
    parts.append("dtype=" + op["dtype"])
    for k, v in op["attrs"].items():
        parts.append("%s=%s" % (k, v))
    return " ".join(parts)


def activation_operands(op, names):
    """The operands of ``op`` that are results of other ops (not weights, not absent)."""
    return [i for i in op["in"] if i is not None and i in names]


# ---------------------------------------------------------------------------------------------
# thresholds
# ---------------------------------------------------------------------------------------------
def import_thresholds(ops, table):
    """Effective threshold of every op result after the reference's overwrite rules.

    ``table`` maps op name -> threshold (the first column of a calibration table). Ops missing
    from the table keep no threshold of their own (the reference warns); reshape never has one and
    resolves to its operand's."""
    by_name = {op["name"]: op for op in ops}
    uses = {}
    for op in ops:
        for i in activation_operands(op, by_name):
            uses[i] = uses.get(i, 0) + 1
    thr = {}
    for op in ops:
        if op["type"] in NO_THRESHOLD:
            continue
        if op["name"] in table:
            thr[op["name"]] = f32(table[op["name"]])

    def producer(op):
        acts = activation_operands(op, by_name)
        if not acts:
            return None
        p = by_name[acts[0]]
        while p["type"] in NO_THRESHOLD:
            p = by_name[activation_operands(p, by_name)[0]]
        return p

    # backward: the op does not rescale, so its single-use producer takes the op's threshold
    changed = True
    while changed:
        changed = False
        for op in ops:
            if op["type"] not in BACKWARD_OPS or op["name"] not in thr:
                continue
            p = producer(op)
            if p is None or p["name"] not in thr:
                continue
            if thr[p["name"]] == thr[op["name"]] or uses.get(p["name"], 0) != 1:
                continue
            thr[p["name"]] = thr[op["name"]]
            changed = True
    # forward: whatever is left takes the producer's threshold
    for op in ops:
        if op["type"] not in FORWARD_OPS:
            continue
        p = producer(op)
        if p is None or p["name"] not in thr:
            continue
        thr[op["name"]] = thr[p["name"]]
    # reshape: alias of its operand
    for op in ops:
        if op["type"] in NO_THRESHOLD:
            p = producer(op)
            if p is not None and p["name"] in thr:
                thr[op["name"]] = thr[p["name"]]
    return thr


# ---------------------------------------------------------------------------------------------
# QuantizationArithmetic.cpp restated with numpy, keeping the C++ float / double types
# ---------------------------------------------------------------------------------------------
def qscale_for_filter(max_filter, threshold_y, threshold_x):
    """findQScaleForFilter (:154-164): every operand is a float, so the quotient is formed in
    fp32 and only then widened to double."""
    ty = f32(threshold_y)
    if ty <= 0:
        ty = f32(0.00001)
    num = np.asarray(max_filter, f32) * f32(threshold_x)
    den = f32(127.0) * ty
    return (num / den).astype(np.float64)


def qscale_for_bias_i32(max_bias, threshold_y):
    """findQScaleForBiasI32 (:174-182): float numerator over a double denominator."""
    ty = f32(threshold_y)
    if ty <= 0:
        ty = f32(0.00001)
    num = (np.asarray(max_bias, f32) * f32(127.0)).astype(np.float64)
    return num / (float(0x7FFFFFFF) * 0.99 * float(ty))


def quantize_multiplier_qdm(qscale):
    """findRShiftAndMultiplierFromQScale with qdm = true (:239-262) over QuantizeMultiplier
    (:188-222): returns (multiplier, rshift) with multiplier in [2^30, 2^31) or 0."""
    q = float(qscale)
    if q >= 1:
        q = 0.999999
    if q == 0.0:
        return 0, 0
    m, shift = math.frexp(q)
    q_fixed = int(math.floor(m * float(1 << 31) + 0.5))  # std::round of a positive value
    if q_fixed == (1 << 31):
        q_fixed //= 2
        shift += 1
    if shift < -31:
        shift = 0
        q_fixed = 0
    rshift = -shift
    assert rshift >= 0
    return q_fixed, rshift


def rshift_for_qscale_i8(qscale, max_multiplier=127):
    """findRShiftAndMultiplierFromQScale with qdm = false (:263-289): the shift that puts
    qscale * 2^rshift into (max/2, max]."""
    q = float(qscale)
    if q > max_multiplier:
        return 0
    for rshift in range(63):
        if q * float(1 << (rshift + 1)) >= float(max_multiplier):
            return rshift
    return 0


def multiplier_i8(qscale, rshift):
    """findMultiplierI8FromQScaleAndRShift (:296-298): truncation through uint32 to int8."""
    v = int(float(qscale) * float(1 << rshift)) & 0xFFFFFFFF
    v &= 0xFF
    return v - 256 if v >= 128 else v


def _saturate_int8(q_f):
    # saturateInt8 (:301-334): floor(f + 0.5) with the sum formed in double
    q = np.floor(q_f.astype(np.float64) + 0.5)
    return np.clip(q, -128, 127)


def _saturate_int32(q_f):
    # saturateInt32 (:367-397): INT_MAX / INT_MIN become floats in the comparisons
    q = np.floor(q_f.astype(np.float64) + 0.5)
    q = np.where(q_f > f32(2147483647), 2147483647.0, q)
    q = np.where(q_f < f32(-2147483648), -2147483648.0, q)
    return q


def _filter_factor(threshold_y, threshold_x, rshift, multiplier):
    # quantizeFilterRShiftAndMultiplier (:442-453): (double)(tx / ty as floats) * 2^(rshift+31) / multiplier
    ratio = float(f32(threshold_x) / f32(threshold_y))
    return 0.0 if multiplier == 0 else ratio * float(1 << (int(rshift) + 31)) / float(multiplier)


def _bias_factor(threshold_y, rshift, multiplier):
    # quantizeBiasRShiftAndMultiplier (:459-478)
    ratio = float(f32(128.0) / f32(threshold_y))
    return 0.0 if multiplier == 0 else ratio * float(1 << (int(rshift) + 31)) / float(multiplier)


def quantize_multiplier_qdm_array(qscale):
    """quantize_multiplier_qdm over a float64 array: (multipliers int64, rshifts int64)."""
    q = np.asarray(qscale, np.float64).copy()
    q[q >= 1] = 0.999999
    m, shift = np.frexp(q)
    shift = shift.astype(np.int64)
    q_fixed = np.floor(m * float(1 << 31) + 0.5).astype(np.int64)
    over = q_fixed == (1 << 31)
    q_fixed[over] //= 2
    shift[over] += 1
    small = (shift < -31) | (q == 0.0)
    shift[small] = 0
    q_fixed[small] = 0
    assert (shift <= 0).all()
    return q_fixed, -shift


def quantize_conv_weights(filt, bias, threshold_y, threshold_x, flat64=None):
    """quantizeWeightInt8Multiplier (:741-818) without a filter threshold. ``filt`` is
    [oc, ...] fp32, ``bias`` [oc] fp32 or None. Returns (new_filter, new_bias, rshift, multiplier)
    as fp32 arrays the way the reference stores them (the multiplier rounded to fp32)."""
    filt = np.ascontiguousarray(filt, f32)
    oc = filt.shape[0]
    flat = filt.reshape(oc, -1)
    max_filter = np.abs(flat).max(axis=1).astype(f32)
    q = qscale_for_filter(max_filter, threshold_y, threshold_x)
    q[q >= 1] = 0.999999
    if bias is not None:
        bias = np.asarray(bias, f32).reshape(oc)
        qb = qscale_for_bias_i32(np.abs(bias), threshold_y)
        take = (qb > q) & ~(qb >= 1)  # a bias scale of 1 or more is ignored ("prevent for auto tuning")
        q = np.where(take, qb, q)
    m, r = quantize_multiplier_qdm_array(q)
    mult = m.astype(f32)  # stored in a float tensor: rounded to 24 bits
    rshift = r.astype(f32)
    m_used = mult.astype(np.float64)  # what the weight scaling then reads back
    live = m_used != 0
    safe = np.where(live, m_used, 1.0)
    # quantizeFilterRShiftAndMultiplier (:442-453): (double)(tx / ty as floats) * 2^(rshift+31) / multiplier
    fac = np.where(live, np.ldexp(float(f32(threshold_x) / f32(threshold_y)), (r + 31).astype(np.int32)) / safe, 0.0)
    # (float)(w * factor) then floor(f + 0.5) in double and the clamp (saturateInt8), with few temporaries; ``flat64`` is
    # the [oc, isz] float64 copy of the filter when the caller quantises the same filter for several thresholds
    x = (flat.astype(np.float64) if flat64 is None else flat64) * fac[:, None]
    np.copyto(x, x.astype(f32))
    x += 0.5
    np.floor(x, out=x)
    np.clip(x, -128, 127, out=x)
    new_f = x.astype(f32)
    new_b = None
    if bias is not None:
        # quantizeBiasRShiftAndMultiplier (:459-478)
        bfac = np.where(live, np.ldexp(float(f32(128.0) / f32(threshold_y)), (r + 31).astype(np.int32)) / safe, 0.0)
        new_b = _saturate_int32((bias.astype(np.float64) * bfac).astype(f32)).astype(f32)
    return new_f.reshape(filt.shape), new_b, rshift, mult


def quantize_fc_weights(filt, bias, threshold_y, threshold_x):
    """quantizeWeightInt8ForFC (:630-690) with batch = 1: one (multiplier, rshift) for the layer."""
    filt = np.ascontiguousarray(filt, f32)
    max_filter = f32(np.abs(filt).max())
    q = float(qscale_for_filter(max_filter, threshold_y, threshold_x))
    if bias is not None:
        qb = qscale_for_bias_i32(np.abs(np.asarray(bias, f32)), threshold_y)
        if qb.size and qb.max() > q:
            q = float(qb.max())
    m, r = quantize_multiplier_qdm(q)
    mult = f32(m)
    m_used = int(mult)
    fac = _filter_factor(threshold_y, threshold_x, r, m_used)
    new_f = _saturate_int8((filt.astype(np.float64) * fac).astype(f32)).astype(f32)
    new_b = None
    if bias is not None:
        bf = _bias_factor(threshold_y, r, m_used)
        new_b = _saturate_int32((np.asarray(bias, f32).astype(np.float64) * bf).astype(f32)).astype(f32)
    return new_f, new_b, np.array([r], f32), np.array([mult], f32)


def rescale_from_qscale(qscale):
    """The shift and the int8 multipliers for a list of fp32 input scales (QuantizeInt8.cpp:787-815)."""
    max_q = max(abs(float(f32(q))) for q in qscale)
    r = rshift_for_qscale_i8(max_q)
    return np.array([r], f32), np.array([multiplier_i8(float(f32(q)), r) for q in qscale], f32)


def rescale_no_weight(thresholds_x, threshold_y, divide_by=1):
    """quantizeInt8RescaleNoWeightOps (:727-833): one shift for the op, one int8 multiplier per
    input. ``divide_by`` is kh * kw of an average pool."""
    qscale = [f32(tx) / f32(threshold_y) for tx in thresholds_x]
    if divide_by != 1:
        qscale[0] = f32(qscale[0] / f32(divide_by))
    return rescale_from_qscale(qscale)


# ---------------------------------------------------------------------------------------------
# op and graph level
# ---------------------------------------------------------------------------------------------
QUANTIZABLE = ("conv_2d", "fully_connected", "eltwise_add", "pool_avg_2d", "pool_max_2d")


def _resolve(name, by_name):
    """Follows reshape aliases back to the op that owns a threshold (getPreviousOpThreshold)."""
    op = by_name[name]
    while op["type"] in NO_THRESHOLD:
        op = by_name[activation_operands(op, by_name)[0]]
    return op["name"]


def quant_param_signature(op, thr, by_name):
    """What the quantised form of ``op`` depends on besides its fp32 weights: its own threshold
    and its operands' thresholds. Two tables that give an op the same signature give it the
    same INT8 kernel."""
    acts = activation_operands(op, by_name)
    own = thr.get(op["name"])
    return (None if own is None else float(own),) + tuple(float(thr[_resolve(a, by_name)]) for a in acts)


def quantize_op(op, thr, weights, by_name, rename=None, out_name=None, cache=None):
    """INT8 form of one fp32 op. ``rename`` maps operand names of the fp32 graph to the names
    they carry in the module being written; ``out_name`` renames the result (and the weights made
    for it); ``cache``: see the conv_2d branch. Returns (list of op dicts, dict of new weights)."""
    rename = rename or {}
    name = out_name or op["name"]
    t = op["type"]
    acts = activation_operands(op, by_name)
    ins = [rename.get(i, i) if i in by_name else i for i in op["in"]]
    new = {"type": t, "name": name, "in": list(ins), "shape": list(op["shape"]), "dtype": "INT8",
           "attrs": dict(op["attrs"])}
    w = {}
    if t in ("pool_max_2d", "reshape"):
        return [new], w
    ty = thr[op["name"]]
    txs = [thr[_resolve(a, by_name)] for a in acts]
    if t == "conv_2d":
        bias = weights[op["in"][2]] if len(op["in"]) > 2 and op["in"][2] else None
        flat64 = None
        if cache is not None:
            # the float64 copy of the filter is shared by the candidates of one op (``cache``: a dict the caller owns)
            key = op["in"][1]
            if key not in cache:
                wf = np.ascontiguousarray(weights[key], f32)
                cache[key] = wf.reshape(wf.shape[0], -1).astype(np.float64)
            flat64 = cache[key]
        nf, nb, r, m = quantize_conv_weights(weights[op["in"][1]], bias, ty, txs[0], flat64=flat64)
        w[name + "_filter_q"] = nf
        new["in"] = [ins[0], name + "_filter_q", None, None, None, name + "_rshift", name + "_multiplier"]
        if nb is not None:
            w[name + "_bias_q"] = nb
            new["in"][2] = name + "_bias_q"
        w[name + "_rshift"], w[name + "_multiplier"] = r, m
    elif t == "fully_connected":
        bias = weights[op["in"][2]] if len(op["in"]) > 2 and op["in"][2] else None
        nf, nb, r, m = quantize_fc_weights(weights[op["in"][1]], bias, ty, txs[0])
        w[name + "_filter_q"] = nf
        new["in"] = [ins[0], name + "_filter_q", None, None, None, name + "_rshift", name + "_multiplier"]
        if nb is not None:
            w[name + "_bias_q"] = nb
            new["in"][2] = name + "_bias_q"
        w[name + "_rshift"], w[name + "_multiplier"] = r, m
    elif t == "eltwise_add":
        n_in = len(acts)
        r, m = rescale_no_weight(txs, ty)
        w[name + "_rshift"], w[name + "_multiplier"] = r, m
        new["in"] = ins[:n_in] + [None, None, name + "_rshift", name + "_multiplier"]
    elif t == "pool_avg_2d":
        kh, kw = int(op["attrs"].get("kh", 1)), int(op["attrs"].get("kw", 1))
        r, m = rescale_no_weight(txs, ty, divide_by=kh * (kw if kw else 1))
        w[name + "_rshift"], w[name + "_multiplier"] = r, m
        new["in"] = [ins[0], None, None, name + "_rshift", name + "_multiplier"]
        new["attrs"]["count_include_pad"] = 1  # the TPU only averages this way (QuantizeInt8.cpp:757-774)
    else:
        raise NotImplementedError("quantize: op type %s (%s) is not covered" % (t, op["name"]))
    return [new], w


def input_quant_op(op, thr, out_name=None):
    """tpu.quant NONE -> INT8 behind an fp32 input: scale = 128 / threshold as a float
    (Quantization.cpp:180-186)."""
    scale = f32(128) / f32(thr[op["name"]])
    return {"type": "quant", "name": out_name or op["name"] + "_quant_i8", "in": [op["name"]],
            "shape": list(op["shape"]), "dtype": "INT8",
            "attrs": {"from": "NONE", "to": "INT8", "scale": repr(float(scale))}}


def quantize_module(text, weights, table, upto=None):
    """Whole-graph INT8 quantisation: (module text, weights) of the INT8 graph whose results keep
    the fp32 graph's op names, truncated after ``upto`` when given (the tuner's build(op_name))."""
    ops = parse_text(text)
    by_name = {op["name"]: op for op in ops}
    thr = import_thresholds(ops, table)
    out_ops, out_w, rename = [], {}, {}
    for op in ops:
        if op["type"] == "input":
            out_ops.append(dict(op))
            q = input_quant_op(op, thr)
            out_ops.append(q)
            rename[op["name"]] = q["name"]
        elif op["type"] == "softmax":
            src = activation_operands(op, by_name)[0]
            dq = {"type": "quant", "name": src + "_dequant", "in": [rename.get(src, src)], "shape": list(by_name[src]["shape"]),
                  "dtype": "FP32", "attrs": {"from": "INT8", "to": "NONE",
                                             "scale": repr(float(f32(thr[_resolve(src, by_name)]) / f32(128)))}}
            sm = dict(op)
            sm["in"] = [dq["name"]]
            out_ops += [dq, sm]
        else:
            new_ops, w = quantize_op(op, thr, weights, by_name, rename)
            out_ops += new_ops
            out_w.update(w)
        if upto is not None and op["name"] == upto:
            break
    return "\n".join(format_op(o) for o in out_ops) + "\n", out_w
