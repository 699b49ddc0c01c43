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


def resnet50_bf16(batch=1, seed=6001, simulate=False):
    """ResNet-50 v1 as an all-BF16 graph (the reference's BF16 quantisation of the fp32 graph: BF16 weights, fp32
    bias, every tensor rounded to BF16): fp32 input -> quant NONE->BF16 -> BF16 convolutions / pooling / eltwise /
    inner product -> quant BF16->NONE."""
    rng = np.random.default_rng(seed)
    b = GraphBuilder(seed, simulate=False)

    def conv(name, src, oc, k, stride=1, pad=0, relu=True):
        n, ic, ih, iw = b.shapes[src]
        oh = (ih + 2 * pad - k) // stride + 1
        ow = (iw + 2 * pad - k) // stride + 1
        f = b.weight(name + "_filter", _bf16_np(rng.normal(0.0, math.sqrt(2.0 / (ic * k * k)), (oc, ic, k, k))))
        bi = b.weight(name + "_bias", rng.normal(0.0, 0.05, oc))
        b.op("conv_2d", name, [src, f, bi], (n, oc, oh, ow), "BF16", kh=k, kw=k, sh=stride, sw=stride, pt=pad, pb=pad,
             pl=pad, pr=pad, dh=1, dw=1, g=1, do_relu=int(relu), with_bias=1)
        return name

    b.op("input", "data", [], (batch, 3, 224, 224), "FP32")
    b.op("quant", "data_bf16", ["data"], (batch, 3, 224, 224), "BF16", **{"from": "NONE", "to": "BF16", "scale": 1.0,
                                                                        "zero_point": 0})
    x = conv("conv1", "data_bf16", 64, 7, 2, 3)
    b.op("pool_max_2d", "pool1", [x], (batch, 64, 56, 56), "BF16", kh=3, kw=3, sh=2, sw=2, pt=0, pb=1, pl=0, pr=1)
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
            b.op("eltwise_add", p, [short, y], b.shapes[y], "BF16", do_relu=1)
            x = p
    n, c, h, w = b.shapes[x]
    b.op("pool_avg_2d", "pool5", [x], (n, c, 1, 1), "BF16", kh=h, kw=w, sh=h, sw=w, count_include_pad=1)
    fw = b.weight("fc1000_filter", _bf16_np(rng.normal(0.0, math.sqrt(2.0 / c), (1000, c))))
    fb = b.weight("fc1000_bias", rng.normal(0.0, 0.05, 1000))
    b.op("fully_connected", "fc1000", ["pool5", fw, fb], (n, 1000), "BF16", do_relu=0)
    b.op("quant", "fc1000_f32", ["fc1000"], (n, 1000), "FP32", **{"from": "BF16", "to": "NONE", "scale": 1.0, "zero_point": 0})
    return Model(b.text(), b.weights, ["data"], ["fc1000_f32"], {"batch": batch})


# ----------------------------------------------------------------------------- BF16 tables (numpy)
def _bf16_np(x):
    """F32ToBF16 with rounding (QuantizationArithmetic.cpp:873-910) on arrays."""
    x = np.asarray(x, np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    u = u + 0x7fff + ((u >> 16) & 1)
    h = (u >> 16) & 0xffff
    h = np.where((h & 0x7f80) == 0x7f80, 0x7f7f, h)
    return (h.astype(np.uint32) << 16).view(np.float32)


def _act_fn(kind):
    if kind == "sigmoid":
        return (lambda x: (1 / (1 + np.exp(-x.astype(np.float32)))).astype(np.float32)), 12
    if kind == "mish":
        def f(x):
            x = x.astype(np.float32)
            sp = np.log(np.exp(x) + np.float32(1)).astype(np.float32)
            return (x.astype(np.float64) * np.tanh(sp.astype(np.float64))).astype(np.float32)
        return f, 8
    if kind == "exp":
        return (lambda x: np.exp(x.astype(np.float32)).astype(np.float32)), 15
    raise ValueError(kind)


def lut_slope_tables(kind):
    """base / slope tables of bf16_gen_base_slope_table (core/lut_func.cpp:32-134); 256 entries
    each, which the reference then replicates per TPU lane."""
    f, R = _act_fn(kind)
    hw, half = 256, 128
    interval = np.float32(int(2 * R)) / np.float32(hw)
    i = np.arange(half, dtype=np.float32)
    base = np.zeros(256, np.float32)
    base[:half] = _bf16_np(f(np.float32(0) + i * interval))
    base[half:] = _bf16_np(f(np.float32(-R) + i * interval))
    scale = np.float32(hw) / np.float32(2 * R)
    slope = np.zeros(256, np.float32)

    def same(a, b):
        return (a.view(np.uint32) >> 16) == (b.view(np.uint32) >> 16)
    x0, x1 = base[:half - 1], base[1:half]
    slope[:half - 1] = np.where(same(x0, x1), 0, _bf16_np(x1 - x0))
    e = np.float32(R)
    slope[half - 1] = _bf16_np(np.float32((f(np.array([3 * e]))[0] - f(np.array([e]))[0]) / (2 * e * scale)))
    x0, x1 = base[half + 1:], base[half:-1]
    slope[half + 1:] = np.where(same(x0, x1), 0, _bf16_np(x0 - x1))
    s = np.float32(-R)
    slope[half] = _bf16_np(np.float32((f(np.array([3 * s]))[0] - f(np.array([s]))[0]) / (abs(2 * s) * scale)))
    return base, slope


def _more_builder_ops():
    """Ops needed by the MobileNet-v2 and YOLOv4-style graphs."""

    def lut_bf16(self, name, src, kind, thr_in, thr_out):
        """An activation run as a BF16 lookup table on an INT8 tensor: int8 -> bf16 dequant
        (scale thr_in/128), table, bf16 -> int8 quant (scale 128/thr_out), the op sequence
        insertQuantOp produces around a BF16 op (Quantization.cpp:180-206)."""
        shape = self.shapes[src]
        base, slope = lut_slope_tables(kind)
        t0 = self.weight(name + "_table0", np.tile(base, 4))
        t1 = self.weight(name + "_table1", np.tile(slope, 4))
        d = self.op("quant", src + "_dequant_bf16", [src], shape, "BF16",
                    **{"from": "INT8", "to": "BF16", "scale": repr(thr_in / 128.0)})
        a = self.op(kind, name, [d, t0, t1], shape, "BF16")
        q = self.op("quant", name + "_quant_i8", [a], shape, "INT8",
                    **{"from": "BF16", "to": "INT8", "scale": repr(128.0 / thr_out)})
        if self.simulate:
            f, _ = _act_fn(kind)
            x = self.sim[src].astype(np.float32) * np.float32(thr_in / 128.0)
            y = f(np.clip(x, -30, 30))
            self.sim[q] = np.clip(np.round(y * (128.0 / thr_out)), -128, 127).astype(np.float64)
        return q

    def leaky_relu_i8(self, name, src, slope=0.1):
        shape = self.shapes[src]
        # positive side passes through (multiplier 0 = no rescale), negative side x * slope:
        # slope ~= M / 2^r with an int8 multiplier (QuantizeInt8.cpp:349-432)
        rn = 7
        mn = int(round(slope * (1 << rn)))
        names = [self.weight(name + s, [v]) for s, v in (("_rshift_pos", 0), ("_multiplier_pos", 0),
                                                         ("_rshift_neg", rn), ("_multiplier_neg", mn))]
        self.op("leaky_relu", name, [src, None, None, None, None] + names, shape, "INT8", negative_slope=slope)
        if self.simulate:
            x = self.sim[src]
            neg = rshift_round_np((x * mn).astype(np.int64), rn)
            self.sim[name] = np.where(x > 0, x, neg).astype(np.float64)
        return name

    def concat_i8(self, name, srcs):
        n, _, h, w = self.shapes[srcs[0]]
        c = sum(self.shapes[s][1] for s in srcs)
        r = self.weight(name + "_rshift", [0] * len(srcs))
        m = self.weight(name + "_multiplier", [1] * len(srcs))
        self.op("concat", name, list(srcs) + [None, None, r, m], (n, c, h, w), "INT8", axis=1, do_relu=0)
        if self.simulate:
            self.sim[name] = np.concatenate([self.sim[s][:1] for s in srcs], axis=1)
        return name

    def upsample(self, name, src, scale=2):
        n, c, h, w = self.shapes[src]
        self.op("upsample", name, [src], (n, c, h * scale, w * scale), self.dtypes[src], scale_h=scale, scale_w=scale)
        if self.simulate:
            self.sim[name] = self.sim[src][:1].repeat(scale, axis=2).repeat(scale, axis=3)
        return name

    def eltwise_add_plain(self, name, srcs):
        return self.eltwise_add_i8(name, srcs, relu=False)

    for fn in (lut_bf16, leaky_relu_i8, concat_i8, upsample, eltwise_add_plain):
        setattr(GraphBuilder, fn.__name__, fn)


_more_builder_ops()


def mobilenet_v2_int8(batch=32, seed=3001, res=224, width=1.0, simulate=True, classes=1000):
    """MobileNet-v2 (expansion 6, 3x3 depthwise + 1x1 pointwise), INT8. ReLU6 is the saturation of the
    int8 range with a fused ReLU: the reference deletes the clip and moves its threshold onto the producer
    (Quantization.cpp:322-345)."""
    b = GraphBuilder(seed, simulate)
    image = np.random.default_rng(seed + 17).uniform(-1, 1, (1, 3, res, res))
    b.input("data", (batch, 3, res, res), sample=image)
    x = b.quant_in("data_quant", "data", 1.0)

    def ch(c):
        return max(8, int(c * width + 4) // 8 * 8)

    x = b.conv_i8("conv1", x, ch(32), 3, stride=2, pad=1, target_std=40.0)
    cin = ch(32)
    cfg = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]
    bi = 0
    for t, c, n, s in cfg:
        for i in range(n):
            bi += 1
            p = "block%d" % bi
            stride = s if i == 0 else 1
            y = x
            if t != 1:
                y = b.conv_i8(p + "_expand", y, cin * t, 1, pad=0, target_std=40.0)
            y = b.conv_i8(p + "_dw", y, cin * t, 3, stride=stride, pad=1, groups=cin * t, target_std=40.0)
            y = b.conv_i8(p + "_project", y, ch(c), 1, pad=0, relu=False)
            if stride == 1 and cin == ch(c):
                y = b.eltwise_add_i8(p + "_add", [x, y], relu=False)
            x, cin = y, ch(c)
    x = b.conv_i8("conv_last", x, ch(1280) if width > 1 else 1280, 1, pad=0, target_std=40.0)
    x = b.pool_avg_i8("pool", x)
    x = b.fc_i8("fc", x, classes)
    b.dequant("fc_dequant", x, 28.0 * 4)
    return Model(b.text(), b.weights, ["data"], ["fc_dequant"], {"sim": b.sim, "batch": batch})


def yolov4_style_int8(batch=8, seed=4001, res=416, width=1.0, depth=(1, 2, 8, 8, 4), simulate=True, heads=255):
    """YOLOv4-style network: CSPDarknet-53 backbone with mish as BF16 lookup tables, SPP, PANet neck with
    INT8 leaky-ReLU, 2x nearest upsampling, concats and three int8 heads at strides 8 / 16 / 32."""
    b = GraphBuilder(seed, simulate)
    image = np.random.default_rng(seed + 17).uniform(0, 1, (1, 3, res, res))
    b.input("data", (batch, 3, res, res), sample=image)
    x = b.quant_in("data_quant", "data", 1.0)
    TH = 28.0 * 4  # activation threshold bookkeeping of the synthetic graph: int8 value * TH / 128

    def ch(c):
        return max(16, int(c * width) // 16 * 16)

    def conv_mish(name, src, oc, k, stride=1):
        y = b.conv_i8(name, src, oc, k, stride=stride, pad=k // 2, relu=False, target_std=40.0)
        return b.lut_bf16(name + "_mish", y, "mish", 4.0, 4.0)

    def conv_leaky(name, src, oc, k, stride=1):
        y = b.conv_i8(name, src, oc, k, stride=stride, pad=k // 2, relu=False)
        return b.leaky_relu_i8(name + "_leaky", y)

    x = conv_mish("conv0", x, ch(32), 3)
    feats = []
    c = ch(32)
    for si, nblk in enumerate(depth):
        oc = ch(64 * (2 ** si))
        p = "s%d" % si
        x = conv_mish(p + "_down", x, oc, 3, stride=2)
        half = oc if si == 0 else oc // 2
        r1 = conv_mish(p + "_route1", x, half, 1)
        r2 = conv_mish(p + "_route2", x, half, 1)
        y = r2
        for k in range(nblk):
            z = conv_mish("%s_b%d_1" % (p, k), y, half if si else oc // 2, 1)
            z = conv_mish("%s_b%d_2" % (p, k), z, half, 3)
            y = b.eltwise_add_plain("%s_b%d_add" % (p, k), [y, z])
        y = conv_mish(p + "_post", y, half, 1)
        x = b.concat_i8(p + "_cat", [y, r1])
        x = conv_mish(p + "_merge", x, oc, 1)
        c = oc
        if si >= 2:
            feats.append(x)
    f8, f16, f32 = feats
    # SPP
    x = conv_leaky("spp_pre1", f32, c // 2, 1)
    x = conv_leaky("spp_pre2", x, c, 3)
    x = conv_leaky("spp_pre3", x, c // 2, 1)
    pools = [b.pool_max("spp_pool%d" % k, x, k, 1, pad=(k // 2, k // 2, k // 2, k // 2)) for k in (5, 9, 13)]
    x = b.concat_i8("spp_cat", pools[::-1] + [x])
    x = conv_leaky("spp_post1", x, c // 2, 1)
    x = conv_leaky("spp_post2", x, c, 3)
    p32 = conv_leaky("spp_post3", x, c // 2, 1)
    # top-down
    def merge_up(name, top, lateral, oc):
        u = conv_leaky(name + "_up_conv", top, oc, 1)
        u = b.upsample(name + "_up", u, 2)
        l = conv_leaky(name + "_lat", lateral, oc, 1)
        y = b.concat_i8(name + "_cat", [l, u])
        for k in range(2):
            y = conv_leaky("%s_c%d_1" % (name, k), y, oc, 1)
            y = conv_leaky("%s_c%d_3" % (name, k), y, oc * 2, 3)
        return conv_leaky(name + "_out", y, oc, 1)
    p16 = merge_up("pan16", p32, f16, c // 4)
    p8 = merge_up("pan8", p16, f8, c // 8)
    # heads + bottom-up
    h8 = conv_leaky("head8_conv", p8, c // 4, 3)
    b.conv_i8("head8", h8, heads, 1, pad=0, relu=False)

    def merge_down(name, low, high, oc):
        d = conv_leaky(name + "_down", low, oc, 3, stride=2)
        y = b.concat_i8(name + "_cat", [d, high])
        for k in range(2):
            y = conv_leaky("%s_c%d_1" % (name, k), y, oc, 1)
            y = conv_leaky("%s_c%d_3" % (name, k), y, oc * 2, 3)
        return conv_leaky(name + "_out", y, oc, 1)
    n16 = merge_down("pan16d", p8, p16, c // 4)
    h16 = conv_leaky("head16_conv", n16, c // 2, 3)
    b.conv_i8("head16", h16, heads, 1, pad=0, relu=False)
    n32 = merge_down("pan32d", n16, p32, c // 2)
    h32 = conv_leaky("head32_conv", n32, c, 3)
    b.conv_i8("head32", h32, heads, 1, pad=0, relu=False)
    return Model(b.text(), b.weights, ["data"], ["head8", "head16", "head32"], {"sim": b.sim, "batch": batch})
