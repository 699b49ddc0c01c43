"""Module text + synthetic weights for the benchmark networks.

The reference obtains quantized graphs from its own compiler passes
(lib/Dialect/TPU/Quantization/QuantizeInt8.cpp) fed by trained models and a
calibration table; neither the models nor the datasets are available, so the
graphs here have the same op sequence, operand layout and quantization
parameter forms (per-channel int32 multiplier in [2^30, 2^31) rounded to an
fp32-representable value plus rshift for conv/fc, int8 multipliers plus one
rshift for eltwise add / avg-pool / concat / leaky-ReLU, 256-entry tables for
the lookup activations) with seeded random He-normal weights. Per-layer scales
are chosen from a short host-side simulation of the first image so that every
layer keeps a realistic int8 dynamic range instead of saturating or dying.

The module text format is the one ``tpucb_interp_load_module`` parses: one op
per line, operands in the TPU dialect's operand order.
"""
import math

import numpy as np

try:  # torch is only used as a fast exact integer conv on the host while choosing scales
    import torch
    import torch.nn.functional as F
except Exception:  # pragma: no cover
    torch = None


# ----------------------------------------------------------------------------- requant (numpy)
def qdm_np(v, mult, rshift):
    """QDM requant on int64 arrays (QuantizationArithmetic.cpp:487-539)."""
    v = v.astype(np.int64)
    ab = v * np.int64(mult) if np.isscalar(mult) else v * mult.astype(np.int64)
    nudge = np.where(ab >= 0, np.int64(1 << 30), np.int64(1 - (1 << 30)))
    x = ab + nudge
    fl = x >> 31
    fl = fl + ((x < 0) & ((x & 0x7fffffff) != 0))
    hi = fl.astype(np.int32).astype(np.int64)
    r = np.asarray(rshift, dtype=np.int64)
    mask = (np.int64(1) << r) - 1
    rem = hi & mask
    thr = (mask >> 1) + (hi < 0)
    q = (hi >> r) + (rem > thr)
    q = np.where((hi == 0) | (r == 0), hi, q)
    return np.clip(q, -128, 127)


def rshift_round_np(v, rshift):
    v = v.astype(np.int64)
    if rshift == 0:
        return np.clip(v, -128, 127)
    return np.clip((v + (1 << (rshift - 1))) >> rshift, -128, 127)


def quantize_multiplier(qscale):
    """QuantizeMultiplier + findRShiftAndMultiplierFromQScale(qdm=true)
    (QuantizationArithmetic.cpp:188-259), then rounded to the nearest fp32-representable
    value because the interpreter stores multipliers in float tensors."""
    qscale = min(float(qscale), 0.999999)
    if qscale <= 0:
        return 0.0, 0.0
    q, shift = math.frexp(qscale)
    m = int(round(q * (1 << 31)))
    if m == (1 << 31):
        m //= 2
        shift += 1
    rshift = -shift
    if rshift > 31:
        return 0.0, 0.0
    m = float(np.float32(m))
    if m >= 2 ** 31:
        m = float(2 ** 31 - 128)
    return m, float(max(rshift, 0))


class Model:
    def __init__(self, text, weights, inputs, outputs, meta=None):
        self.text, self.weights, self.inputs, self.outputs = text, weights, inputs, outputs
        self.meta = meta or {}


class GraphBuilder:
    def __init__(self, seed, simulate=True):
        self.rng = np.random.default_rng(seed)
        self.lines = []
        self.weights = {}
        self.shapes = {}
        self.dtypes = {}
        self.sim = {} if simulate else None  # name -> float64 NCHW array of the first image
        self.simulate = simulate

    # ---- plumbing
    def op(self, type_, name, ins, shape, dtype, **attrs):
        parts = [type_, "name=" + name]
        if ins:
            parts.append("in=" + ",".join(i if i else "-" for i in ins))
        parts.append("shape=" + ",".join(str(int(d)) for d in shape))
        parts.append("dtype=" + dtype)
        for k, v in attrs.items():
            parts.append("%s=%s" % (k, v))
        self.lines.append(" ".join(parts))
        self.shapes[name] = tuple(int(d) for d in shape)
        self.dtypes[name] = dtype
        return name

    def weight(self, name, arr):
        self.weights[name] = np.ascontiguousarray(arr, dtype=np.float32)
        return name

    def text(self):
        return "\n".join(self.lines) + "\n"

    # ---- ops
    def input(self, name, shape, sample=None):
        self.op("input", name, [], shape, "FP32")
        if self.simulate:
            self.sim[name] = sample
        return name

    def quant_in(self, name, src, threshold=1.0):
        """tpu.quant NONE->INT8 right after the input op: scale = 128 / threshold."""
        scale = 128.0 / threshold
        self.op("quant", name, [src], self.shapes[src], "INT8", **{"from": "NONE", "to": "INT8", "scale": repr(scale)})
        if self.simulate:
            x = self.sim[src].astype(np.float32) * np.float32(scale)
            r = np.where(x >= 0, np.floor(x + np.float32(0.5)), np.ceil(x - np.float32(0.5)))
            self.sim[name] = np.clip(r, -128, 127).astype(np.float64)
        return name

    def dequant(self, name, src, threshold, to="NONE"):
        dt = "FP32" if to == "NONE" else "BF16"
        self.op("quant", name, [src], self.shapes[src], dt, **{"from": "INT8", "to": to, "scale": repr(threshold / 128.0)})
        return name

    def _conv_acc(self, x, w, stride, pad, dil, groups):
        xt = torch.from_numpy(x)
        wt = torch.from_numpy(w.astype(np.float64))
        pt, pb, pl, pr = pad
        xt = F.pad(xt, (pl, pr, pt, pb))
        return F.conv2d(xt, wt, None, stride, 0, dil, groups).numpy()

    def conv_i8(self, name, src, oc, k, stride=1, pad=None, relu=True, groups=1, dilation=1, target_std=28.0,
                with_bias=True):
        n, ic, ih, iw = self.shapes[src]
        kh = kw = k
        if pad is None:
            pad = (k - 1) * dilation // 2
        pads = (pad, pad, pad, pad) if np.isscalar(pad) else tuple(pad)
        pt, pb, pl, pr = pads
        oh = (ih + pt + pb - dilation * (kh - 1) - 1) // stride + 1
        ow = (iw + pl + pr - dilation * (kw - 1) - 1) // stride + 1
        icg = ic // groups
        fan_in = icg * kh * kw
        w = self.rng.normal(0.0, math.sqrt(2.0 / fan_in), (oc, icg, kh, kw))
        wmax = np.abs(w).reshape(oc, -1).max(axis=1)
        wq = np.clip(np.floor(w * (127.0 / wmax)[:, None, None, None] + 0.5), -128, 127)
        bias = np.zeros(oc)
        mult = np.zeros(oc, np.float32)
        rsh = np.zeros(oc, np.float32)
        if self.simulate:
            acc = self._conv_acc(self.sim[src][:1], wq, stride, pads, dilation, groups)
            std_c = acc.reshape(oc, -1).std(axis=1) if acc[0, 0].size > 1 else np.abs(acc.reshape(oc, -1)).mean(axis=1)
            layer_std = max(float(np.sqrt((acc ** 2).mean())), 1.0)
            std_c = np.maximum(std_c, 0.25 * layer_std)
            if with_bias:
                bias = np.round(self.rng.normal(0.0, 0.3, oc) * std_c)
            for c in range(oc):
                mult[c], rsh[c] = quantize_multiplier(target_std / std_c[c])
            q = qdm_np((acc + bias[None, :, None, None]).astype(np.int64), mult.astype(np.int64)[None, :, None, None],
                       rsh.astype(np.int64)[None, :, None, None])
            if relu:
                q = np.maximum(q, 0)
            self.sim[name] = q.astype(np.float64)
        else:
            if with_bias:
                bias = np.round(self.rng.normal(0.0, 2000.0, oc))
            for c in range(oc):
                mult[c], rsh[c] = quantize_multiplier(1.0 / (math.sqrt(fan_in) * 40.0))
        f = self.weight(name + "_filter", wq)
        b = self.weight(name + "_bias", bias) if with_bias else None
        r = self.weight(name + "_rshift", rsh)
        m = self.weight(name + "_multiplier", mult)
        self.op("conv_2d", name, [src, f, b, None, None, r, m], (n, oc, oh, ow), "INT8", kh=kh, kw=kw, sh=stride,
                sw=stride, pt=pt, pb=pb, pl=pl, pr=pr, dh=dilation, dw=dilation, g=groups, do_relu=int(relu),
                with_bias=int(with_bias))
        return name

    def pool_max(self, name, src, k, stride, pad=(0, 0, 0, 0)):
        n, c, ih, iw = self.shapes[src]
        pt, pb, pl, pr = pad
        oh = (ih + pt + pb - k) // stride + 1
        ow = (iw + pl + pr - k) // stride + 1
        self.op("pool_max_2d", name, [src], (n, c, oh, ow), self.dtypes[src], kh=k, kw=k, sh=stride, sw=stride, pt=pt,
                pb=pb, pl=pl, pr=pr)
        if self.simulate:
            xt = torch.from_numpy(self.sim[src][:1])
            xt = F.pad(xt, (pl, pr, pt, pb), value=-1e9)
            self.sim[name] = F.max_pool2d(xt, k, stride).numpy()
        return name

    def pool_avg_i8(self, name, src, k=None):
        """Global (or k x k, stride k) average pool, INT8: window sum * M >> r with the 1/(kh*kw)
        folded into (M, r) (QuantizeInt8.cpp:669-730)."""
        n, c, ih, iw = self.shapes[src]
        kh, kw = (ih, iw) if k is None else (k, k)
        oh, ow = ih // kh, iw // kw
        qscale = 1.0 / (kh * kw)
        rshift = 0
        while qscale * (1 << (rshift + 1)) <= 127 and rshift < 15:
            rshift += 1
        mult = int(qscale * (1 << rshift))
        r = self.weight(name + "_rshift", [rshift])
        m = self.weight(name + "_multiplier", [mult])
        self.op("pool_avg_2d", name, [src, None, None, r, m], (n, c, oh, ow), "INT8", kh=kh, kw=kw, sh=kh, sw=kw, pt=0,
                pb=0, pl=0, pr=0, count_include_pad=1)
        if self.simulate:
            x = self.sim[src][:1]
            s = x.reshape(1, c, oh, kh, ow, kw).sum(axis=(3, 5))
            self.sim[name] = rshift_round_np((s * mult).astype(np.int64), rshift).astype(np.float64)
        return name

    def eltwise_add_i8(self, name, srcs, relu=True):
        shape = self.shapes[srcs[0]]
        nin = len(srcs)
        # equal-weight sum rescaled by 1/sqrt(nin)-ish so the range stays put: M = 45, r = 6 (0.70)
        mults = [45] * nin
        rshift = 6
        r = self.weight(name + "_rshift", [rshift])
        m = self.weight(name + "_multiplier", mults)
        self.op("eltwise_add", name, list(srcs) + [None, None, r, m], shape, "INT8", do_relu=int(relu))
        if self.simulate:
            acc = sum(self.sim[s][:1] * mu for s, mu in zip(srcs, mults))
            if relu:
                acc = np.maximum(acc, 0)
            self.sim[name] = rshift_round_np(acc.astype(np.int64), rshift).astype(np.float64)
        return name

    def fc_i8(self, name, src, out_features, relu=False, target_std=28.0):
        shape = self.shapes[src]
        m = shape[0]
        k = int(np.prod(shape[1:]))
        w = self.rng.normal(0.0, math.sqrt(2.0 / k), (out_features, k))
        wq = np.clip(np.floor(w * (127.0 / np.abs(w).max()) + 0.5), -128, 127)
        bias = np.zeros(out_features)
        mult, rsh = quantize_multiplier(1.0 / (math.sqrt(k) * 40.0))
        if self.simulate:
            x = self.sim[src][:1].reshape(1, k)
            acc = x @ wq.T
            std = max(float(acc.std()), 1.0)
            bias = np.round(self.rng.normal(0.0, 0.3 * std, out_features))
            mult, rsh = quantize_multiplier(target_std / std)
            v = acc + bias[None]
            if relu:
                v = np.maximum(v, 0)
            self.sim[name] = qdm_np(v.astype(np.int64), int(mult), int(rsh)).astype(np.float64)
        f = self.weight(name + "_filter", wq)
        b = self.weight(name + "_bias", bias)
        r = self.weight(name + "_rshift", [rsh])
        mu = self.weight(name + "_multiplier", [mult])
        self.op("fully_connected", name, [src, f, b, None, None, r, mu], (m, out_features), "INT8", do_relu=int(relu))
        return name

    def reshape(self, name, src, shape):
        self.op("reshape", name, [src], shape, self.dtypes[src])
        if self.simulate:
            self.sim[name] = self.sim[src][:1].reshape((1,) + tuple(shape[1:]))
        return name


# ----------------------------------------------------------------------------- networks
def resnet50_int8(batch=1, seed=1001, simulate=True, image=None):
    """ResNet-50 v1 (Caffe layout: stride on the first 1x1 of a stage, 3x3 max-pool with
    ceil-mode padding), INT8, input [batch,3,224,224] fp32 in [-1,1] quantized with threshold 1.0."""
    b = GraphBuilder(seed, simulate)
    if image is None:
        image = np.random.default_rng(seed + 17).uniform(-1, 1, (1, 3, 224, 224))
    b.input("data", (batch, 3, 224, 224), sample=np.asarray(image, np.float64)[:1])
    x = b.quant_in("data_quant", "data", 1.0)
    x = b.conv_i8("conv1", x, 64, 7, stride=2, pad=3)
    x = b.pool_max("pool1", x, 3, 2, pad=(0, 1, 0, 1))
    stages = [(64, 256, 3, 1), (128, 512, 4, 2), (256, 1024, 6, 2), (512, 2048, 3, 2)]
    for si, (mid, out, blocks, stride) in enumerate(stages):
        for bi in range(blocks):
            p = "res%d%s" % (si + 2, "abcdef"[bi])
            s = stride if bi == 0 else 1
            if bi == 0:
                short = b.conv_i8(p + "_branch1", x, out, 1, stride=s, pad=0, relu=False)
            else:
                short = x
            y = b.conv_i8(p + "_branch2a", x, mid, 1, stride=s, pad=0)
            y = b.conv_i8(p + "_branch2b", y, mid, 3, stride=1, pad=1)
            y = b.conv_i8(p + "_branch2c", y, out, 1, stride=1, pad=0, relu=False)
            x = b.eltwise_add_i8(p, [short, y], relu=True)
    x = b.pool_avg_i8("pool5", x)
    x = b.fc_i8("fc1000", x, 1000)
    b.dequant("fc1000_dequant", x, 28.0 * 4)
    return Model(b.text(), b.weights, ["data"], ["fc1000_dequant"], {"sim": b.sim, "batch": batch})


def single_conv_i8(n, c_in, c_out, hw, k=3, stride=1, pad=1, dilation=1, groups=1, relu=True, seed=2000,
                   rshift_range=(14, 17), with_bias=True):
    """One INT8 Conv2D op with uniform random int8 operands (the op-sweep configuration)."""
    rng = np.random.default_rng(seed)
    b = GraphBuilder(seed, simulate=False)
    b.op("input", "x", [], (n, c_in, hw, hw), "INT8")
    oh = (hw + 2 * pad - dilation * (k - 1) - 1) // stride + 1
    icg = c_in // groups
    w = rng.integers(-127, 128, (c_out, icg, k, k))
    bias = rng.integers(-2 ** 16, 2 ** 16 + 1, c_out)
    mult = np.float32((rng.integers(2 ** 30, 2 ** 31 - 128, c_out) // 128) * 128)
    rsh = rng.integers(rshift_range[0], rshift_range[1], c_out)
    f = b.weight("conv_filter", w)
    bi = b.weight("conv_bias", bias) if with_bias else None
    r = b.weight("conv_rshift", rsh)
    m = b.weight("conv_multiplier", mult)
    b.op("conv_2d", "conv", ["x", f, bi, None, None, r, m], (n, c_out, oh, oh), "INT8", kh=k, kw=k, sh=stride,
         sw=stride, pt=pad, pb=pad, pl=pad, pr=pad, dh=dilation, dw=dilation, g=groups, do_relu=int(relu),
         with_bias=int(with_bias))
    x = rng.integers(-128, 128, (n, c_in, hw, hw)).astype(np.float32)
    return Model(b.text(), b.weights, ["x"], ["conv"], {"x": x})


# ----------------------------------------------------------------------------- fp32 (calibration)
def resnet50_fp32(batch=1, seed=5001):
    """fp32 ResNet-50 v1 with batch-norm folded into the convolution bias (what the reference's
    --convert-bn-to-scale --canonicalize --fuse-relu pipeline leaves), He-normal weights. This is
    the graph the calibration pass runs."""
    rng = np.random.default_rng(seed)
    b = GraphBuilder(seed, simulate=False)

    def conv(name, src, oc, k, stride=1, pad=0, relu=True):
        n, ic, ih, iw = b.shapes[src]
        oh = (ih + 2 * pad - k) // stride + 1
        ow = (iw + 2 * pad - k) // stride + 1
        w = rng.normal(0.0, math.sqrt(2.0 / (ic * k * k)), (oc, ic, k, k))
        f = b.weight(name + "_filter", w)
        bi = b.weight(name + "_bias", rng.normal(0.0, 0.05, oc))
        b.op("conv_2d", name, [src, f, bi], (n, oc, oh, ow), "FP32", kh=k, kw=k, sh=stride, sw=stride, pt=pad, pb=pad,
             pl=pad, pr=pad, dh=1, dw=1, g=1, do_relu=int(relu), with_bias=1)
        return name

    b.op("input", "data", [], (batch, 3, 224, 224), "FP32")
    x = conv("conv1", "data", 64, 7, 2, 3)
    b.op("pool_max_2d", "pool1", [x], (batch, 64, 56, 56), "FP32", kh=3, kw=3, sh=2, sw=2, pt=0, pb=1, pl=0, pr=1)
    x = "pool1"
    stages = [(64, 256, 3, 1), (128, 512, 4, 2), (256, 1024, 6, 2), (512, 2048, 3, 2)]
    for si, (mid, out, blocks, stride) in enumerate(stages):
        for bi_ in range(blocks):
            p = "res%d%s" % (si + 2, "abcdef"[bi_])
            s = stride if bi_ == 0 else 1
            short = conv(p + "_branch1", x, out, 1, s, 0, relu=False) if bi_ == 0 else x
            y = conv(p + "_branch2a", x, mid, 1, s, 0)
            y = conv(p + "_branch2b", y, mid, 3, 1, 1)
            y = conv(p + "_branch2c", y, out, 1, 1, 0, relu=False)
            b.op("eltwise_add", p, [short, y], b.shapes[y], "FP32", do_relu=1)
            x = p
    n, c, h, w = b.shapes[x]
    b.op("pool_avg_2d", "pool5", [x], (n, c, 1, 1), "FP32", kh=h, kw=w, sh=h, sw=w, count_include_pad=1)
    fw = b.weight("fc1000_filter", rng.normal(0.0, math.sqrt(2.0 / c), (1000, c)))
    fb = b.weight("fc1000_bias", rng.normal(0.0, 0.05, 1000))
    b.op("fully_connected", "fc1000", ["pool5", fw, fb], (n, 1000), "FP32", do_relu=0)
    b.op("softmax", "prob", ["fc1000"], (n, 1000), "FP32", axis=1)
    return Model(b.text(), b.weights, ["data"], ["prob"], {"batch": batch})
