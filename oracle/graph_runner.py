"""Run a module text on the CPU oracle, op by op, keeping every tensor
(the reference's ``--dump-all-tensor`` idea, tools/tpuc-interpreter/tpuc-interpreter.cpp:155-176).
TEST INFRASTRUCTURE ONLY."""
import numpy as np

import oracle as O


def parse(text):
    ops = []
    for line in text.splitlines():
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        toks = line.split()
        op = {"type": toks[0], "in": [], "attrs": {}, "dtype": "FP32", "shape": []}
        for t in toks[1:]:
            k, v = t.split("=", 1)
            if k == "name":
                op["name"] = v
            elif k == "in":
                op["in"] = v.split(",")
            elif k == "shape":
                op["shape"] = [int(d) for d in v.split(",")]
            elif k == "dtype":
                op["dtype"] = v
            else:
                op["attrs"][k] = v
        ops.append(op)
    return ops


def _i(a, k, d=0):
    return int(a.get(k, d))


def run(text, weights, inputs, upto=None):
    """inputs: {name: float32 NCHW array}. Returns {name: float32 array} for every op result."""
    T = {}
    prod = {}
    for op in parse(text):
        t, name, a, ins = op["type"], op["name"], op["attrs"], op["in"]
        W = lambda i: weights[ins[i]] if i < len(ins) and ins[i] != "-" and ins[i] in weights else None  # noqa: E731
        X = lambda i: T[ins[i]]  # noqa: E731
        if t == "input":
            out = np.asarray(inputs[name], np.float32).reshape(op["shape"])
        elif t == "quant":
            frm, to = a.get("from", "NONE"), a.get("to", "NONE")
            scale = float(a.get("scale", 1.0))
            if frm == "NONE" and to == "INT8":
                kind = "f32_i8_host" if prod[ins[0]] == "input" else "f32_i8"
            elif frm in ("INT8", "UINT8") and to == "NONE":
                kind = "i8_f32"
            elif frm in ("INT8", "UINT8") and to == "BF16":
                kind = "i8_bf16"
            elif frm == "BF16" and to == "INT8":
                kind = "bf16_i8"
            elif frm == "NONE" and to == "BF16":
                kind = "f32_bf16"
            else:
                kind = None
            out = X(0).copy() if kind is None else O.quant(X(0), scale, kind)
        elif t == "conv_2d":
            mode = op["dtype"]
            out = O.conv2d(X(0), W(1), W(2), W(5), W(6), (op["shape"][2], op["shape"][3]),
                           stride=(_i(a, "sh", 1), _i(a, "sw", 1)), pad=(_i(a, "pt"), _i(a, "pl")),
                           dilation=(_i(a, "dh", 1), _i(a, "dw", 1)), groups=_i(a, "g", 1),
                           ins=(_i(a, "ins_h"), _i(a, "ins_w")), do_relu=bool(_i(a, "do_relu")), mode=mode)
        elif t == "deconv_2d" and op["dtype"] != "INT8":
            out = O.deconv2d_f(X(0), W(1), W(2),
                               (op["shape"][2], op["shape"][3]), stride=(_i(a, "sh", 1), _i(a, "sw", 1)),
                               pad=(_i(a, "pt"), _i(a, "pl")), dilation=(_i(a, "dh", 1), _i(a, "dw", 1)),
                               groups=_i(a, "g", 1), do_relu=bool(_i(a, "do_relu")), to_bf16=(op["dtype"] == "BF16"))
        elif t == "deconv_2d":
            out = O.deconv2d_i8(X(0), W(1), W(2), W(5), W(6), (op["shape"][2], op["shape"][3]),
                                stride=(_i(a, "sh", 1), _i(a, "sw", 1)), pad=(_i(a, "pt"), _i(a, "pl")),
                                dilation=(_i(a, "dh", 1), _i(a, "dw", 1)), groups=_i(a, "g", 1),
                                do_relu=bool(_i(a, "do_relu")))
        elif t == "fully_connected":
            x = X(0)
            if W(1).ndim >= 3:   # batched: one product per leading filter index (core/fullyconnected.cpp:59-88)
                out = O.fc(x, W(1), W(2), W(5), W(6), do_relu=bool(_i(a, "do_relu")), mode=op["dtype"])
            else:
                out = O.fc(x.reshape(x.shape[0], -1), W(1), W(2), W(5), W(6), do_relu=bool(_i(a, "do_relu")),
                           mode=op["dtype"])
        elif t in ("pool_max_2d", "pool_avg_2d"):
            is_i8 = op["dtype"] == "INT8"
            rs = float(W(3)[0]) if (t == "pool_avg_2d" and is_i8) else 0.0
            mu = float(W(4)[0]) if (t == "pool_avg_2d" and is_i8) else 0.0
            out = O.pool(X(0), (_i(a, "kh", 1), _i(a, "kw", 1)), (_i(a, "sh", 1), _i(a, "sw", 1)),
                         (_i(a, "pt"), _i(a, "pl")), (op["shape"][2], op["shape"][3]),
                         method="max" if t == "pool_max_2d" else "avg", is_int8=is_i8,
                         count_include_pad=bool(_i(a, "count_include_pad")), rshift=rs, multiplier=mu)
        elif t in ("eltwise_add", "eltwise_mul"):
            xs = [T[n] for n in ins if n in T]
            nin = len(xs)
            if op["dtype"] == "INT8":
                rs, mu = W(nin + 2), W(nin + 3)
                if t == "eltwise_add":
                    out = O.eltwise_add_i8(xs, mu, float(rs[0]), bool(_i(a, "do_relu")))
                else:
                    out = O.eltwise_mul_i8(xs, float(mu[0]), float(rs[0]), bool(_i(a, "do_relu")))
            elif t == "eltwise_mul":
                # fp32 product (core/eltwise.cpp:320-333); BF16 rounds the result
                out = O.eltwise_mul_i8(xs, 0.0, 0.0, bool(_i(a, "do_relu")))
                if op["dtype"] == "BF16":
                    out = O.bf16_round(out)
            else:
                coeff = [float(c) for c in a["coeff"].split(",")] if "coeff" in a else None
                out = O.eltwise_add_f32(xs, coeff, bool(_i(a, "do_relu")), to_bf16=(op["dtype"] == "BF16"))
        elif t in ("eltwise_max", "eltwise_min"):
            n_in = sum(1 for nm in ins if nm in T)
            out = O.eltwise_maxmin_i8([T[nm] for nm in ins[:n_in]], W(n_in + 3), float(W(n_in + 2)[0]),
                                      bool(_i(a, "do_relu")), is_min=(t == "eltwise_min"))
        elif t in ("broadcast_add", "broadcast_sub", "broadcast_mul"):
            is_i8 = op["dtype"] == "INT8"
            out = O.broadcast(X(0), X(1), t.split("_")[1], is_int8=is_i8, multiplier=W(5) if is_i8 else None,
                              rshift=float(W(4)[0]) if is_i8 else 0.0, do_relu=bool(_i(a, "do_relu")))
            out = out.reshape(op["shape"])
        elif t == "pad":
            out = O.pad(X(0), [int(v) for v in a["pads"].split(",")], a.get("mode", "constant"))
        elif t == "crop":
            steps = [int(v) for v in a["steps"].split(",")] if "steps" in a else None
            out = O.crop(X(0), op["shape"], [int(v) for v in a["crop_offset"].split(",")], steps)
        elif t == "permute":
            out = O.permute(X(0), [int(v) for v in a["order"].split(",")])
        elif t in ("reduce_mean", "reduce_sum", "reduce_max", "reduce_min"):
            is_i8 = op["dtype"] == "INT8"
            mu = float(W(4)[0]) if (is_i8 and W(4) is not None) else 1.0
            rs = float(W(3)[0]) if (is_i8 and W(3) is not None) else 0.0
            out = O.reduce(X(0), [int(v) for v in a["axes"].split(",")], t.split("_")[1], is_int8=is_i8,
                           multiplier=mu, rshift=rs).reshape(op["shape"])
        elif t == "matmul":
            is_i8 = op["dtype"] == "INT8"
            out = O.matmul(X(0), X(1), op["shape"], mode=op["dtype"], rshift=float(W(4)[0]) if is_i8 else 0.0,
                           multiplier=float(W(5)[0]) if is_i8 else 0.0, do_relu=bool(_i(a, "do_relu")),
                           ltrans=bool(_i(a, "left_transpose")), rtrans=bool(_i(a, "right_transpose")),
                           otrans=bool(_i(a, "output_transpose")))
        elif t == "concat":
            xs = [T[n] for n in ins if n in T]
            nin = len(xs)
            rs, mu = W(nin + 2), W(nin + 3)
            out = O.concat_c(xs, mu, rs, bool(_i(a, "do_relu")))
        elif t == "upsample":
            out = O.upsample(X(0), _i(a, "scale_h", 1), _i(a, "scale_w", 1))
        elif t == "pixelshuffle":
            out = O.pixelshuffle(X(0), _i(a, "upscale_factor", 1), a.get("mode", "CRD") == "DCR")
        elif t == "relu":
            out = O.relu(X(0))
        elif t == "leaky_relu" and op["dtype"] != "INT8":
            out = O.leaky_relu_f(X(0), float(a.get("negative_slope", 0.0)), to_bf16=(op["dtype"] == "BF16"))
        elif t == "leaky_relu":
            out = O.leaky_relu_i8(X(0), float(W(5)[0]), float(W(6)[0]), float(W(7)[0]), float(W(8)[0]))
        elif t in ("sigmoid", "mish", "exp", "tanh"):
            if op["dtype"] == "INT8":
                out = O.lut_i8(X(0), W(1))
            else:
                out = O.lut_bf16_slope(t, X(0), W(1)[:256], W(2)[:256])
        elif t == "reciprocal":
            out = O.lut_bf16_mantissa(X(0), W(1)[:256], W(2)[:256])
        elif t == "scale":
            out = O.scale_f32(X(0), W(1), W(2))
        elif t == "batchnorm":
            out = O.batchnorm_f32(X(0), W(1), W(2), float(W(3).reshape(-1)[0]), float(a.get("variance_epsilon", 1e-5)))
        elif t == "reduce_l2":
            out = O.reduce_l2_f32(X(0), [int(v) for v in a["axes"].split(",")], float(a.get("coeff", 0.5)))
        elif t == "softmax":
            if op["dtype"] == "BF16":
                out = O.softmax_bf16(X(0), W(1), W(2), W(3), W(4), axis=_i(a, "axis", 1), do_log=bool(_i(a, "do_log")))
            else:
                out = O.softmax_f32(X(0), 1)
        elif t == "reshape":
            out = X(0).reshape(op["shape"])
        else:
            raise NotImplementedError(t)
        T[name] = np.asarray(out, np.float32).reshape(op["shape"])
        prod[name] = t
        if upto is not None and name == upto:
            break
    return T
