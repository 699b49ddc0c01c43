"""The reference-faithful CPU path for timing (TEST INFRASTRUCTURE / CPU BASELINE ONLY).

The reference interpreter performs INT8 convolution as an fp32 MKL-DNN convolution on
integer-valued floats followed by its own requantisation pass (core/conv.cpp:80-104). MKL-DNN
v1.0.2 is not vendored, so this path uses its direct successor, oneDNN, through torch's CPU
convolution for the contraction -- the same trick, exact while partial sums stay below 2^24 --
and the reference's OWN requantisation code (QuantizationArithmetic.cpp compiled unmodified into
oracle/_ref) where that build is present, else the oracle's restatement. Every other op runs
through the oracle. Results are checked bit for bit against the oracle before any timing counts.
"""
import ctypes as C

import numpy as np
import torch
import torch.nn.functional as F

import oracle as O
from oracle import graph_runner

_f = C.POINTER(C.c_float)


def _p(a):
    return a.ctypes.data_as(_f)


def _requant(acc, bias, rshift, mult, relu):
    n, oc = acc.shape[:2]
    isz = int(np.prod(acc.shape[2:]))
    acc = np.ascontiguousarray(acc, np.float32)
    out = np.empty_like(acc)
    R = O.ref()
    bias = np.ascontiguousarray(bias if bias is not None else np.zeros(oc), np.float32)
    rs = np.ascontiguousarray(rshift, np.float32)
    mu = np.ascontiguousarray(mult, np.float32)
    if R is not None:
        R.ref_requant_per_channel(_p(out), _p(acc), _p(bias), int(relu), C.c_int64(n), C.c_int64(oc), C.c_int64(isz),
                                  _p(rs), _p(mu))
        return out
    v = acc.astype(np.int64) + bias.astype(np.int64).reshape(1, oc, *([1] * (acc.ndim - 2)))
    L = O.lib()
    flat = v.reshape(n, oc, -1)
    res = np.empty(flat.shape, np.float32)
    for c in range(oc):
        res[:, c] = [L.orc_qdm_i32(int(x), int(rs[c]), int(mu[c])) for x in flat[:, c].reshape(-1)]
    res = res.reshape(acc.shape)
    return np.maximum(res, 0) if relu else res


def run(text, weights, inputs, keep_all=False):
    """Runs an INT8 classification module (input, quant, conv_2d, pooling, eltwise_add, fully_connected)."""
    T, prod = {}, {}
    wt = {}
    out_name = None
    for op in graph_runner.parse(text):
        t, name, a, ins = op["type"], op["name"], op["attrs"], op["in"]
        gi = lambda k, d=0: int(a.get(k, d))  # noqa: E731
        if t == "conv_2d" and op["dtype"] == "INT8":
            x = torch.from_numpy(T[ins[0]])
            if ins[1] not in wt:
                wt[ins[1]] = torch.from_numpy(np.ascontiguousarray(weights[ins[1]], np.float32))
            pt, pl = gi("pt"), gi("pl")
            oh, ow = op["shape"][2], op["shape"][3]
            kh, kw, sh, sw, dh, dw = gi("kh", 1), gi("kw", 1), gi("sh", 1), gi("sw", 1), gi("dh", 1), gi("dw", 1)
            pb = max((oh - 1) * sh + (kh - 1) * dh + 1 - x.shape[2] - pt, 0)
            pr = max((ow - 1) * sw + (kw - 1) * dw + 1 - x.shape[3] - pl, 0)
            if pt or pl or pb or pr:
                x = F.pad(x, (pl, pr, pt, pb))
            acc = F.conv2d(x, wt[ins[1]], None, (sh, sw), 0, (dh, dw), gi("g", 1))[:, :, :oh, :ow].numpy()
            bias = weights[ins[2]] if ins[2] != "-" else None
            out = _requant(acc, bias, weights[ins[5]], weights[ins[6]], bool(gi("do_relu")))
        else:
            out = _oracle_op(op, T, prod, weights, inputs)
        T[name] = np.asarray(out, np.float32).reshape(op["shape"])
        prod[name] = t
        out_name = name
    return T if keep_all else {out_name: T[out_name]}


def _oracle_op(op, T, prod, weights, inputs):
    """One op through the oracle's graph runner (state injected)."""
    line = _line(op)
    # build a tiny module: declared inputs for the operands that are tensors, then the op
    ops = []
    feed = {}
    for n in op["in"]:
        if n in T:
            ops.append("input name=%s shape=%s dtype=FP32" % (n, ",".join(str(d) for d in T[n].shape)))
            feed[n] = T[n]
    if op["type"] == "input":
        return np.asarray(inputs[op["name"]], np.float32)
    text = "\n".join(ops + [line]) + "\n"
    if op["type"] == "quant" and prod.get(op["in"][0]) != "input":
        # the one-op module above would make the operand look like a graph input, which selects the
        # host rounding rule of QuantOpKernel; away from the input the TPU rule applies
        kind_map = {("NONE", "INT8"): "f32_i8", ("INT8", "NONE"): "i8_f32", ("UINT8", "NONE"): "i8_f32",
                    ("INT8", "BF16"): "i8_bf16", ("BF16", "INT8"): "bf16_i8", ("NONE", "BF16"): "f32_bf16"}
        a = op["attrs"]
        return O.quant(T[op["in"][0]], float(a.get("scale", 1.0)), kind_map[(a.get("from", "NONE"), a.get("to", "NONE"))])
    return graph_runner.run(text, weights, feed)[op["name"]]


def _line(op):
    parts = [op["type"], "name=" + op["name"]]
    if op["in"]:
        parts.append("in=" + ",".join(op["in"]))
    parts.append("shape=" + ",".join(str(d) for d in op["shape"]))
    parts.append("dtype=" + op["dtype"])
    parts += ["%s=%s" % kv for kv in op["attrs"].items()]
    return " ".join(parts)
