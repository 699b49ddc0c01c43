"""Reader for the generic-form TPU-dialect ``.mlir`` text the reference's tools write and its
interpreter loads (the form of lib/Dialect/TPU/Backend/test/*.mlir): converts it to the one-op-per-line
module text of ``tpucb_interp_load_module``. Weights stay in the ``.npz`` named by ``tpu.weight_file``
(npz of fp32 arrays keyed by the ``name`` of each ``tpu.load_weight``, include/tpuc/Support/TensorFile.h).

Only the syntax the reference emits is handled: one op per line,
``%id = "tpu.op"(%operands) {attributes} : (types) -> type``.
"""
import re

_OP_RE = re.compile(r'^\s*(%[\w.]+)\s*=\s*"tpu\.([\w.]+)"\((.*?)\)\s*(\{.*\})?\s*:\s*\((.*?)\)\s*->\s*(.+?)\s*$')
_TENSOR_RE = re.compile(r"tensor<([0-9x]+)x(\w+)>")


class _AttrParser:
    """Parses ``{a = 1 : i32, b = {c = "x"}, d = [1 : i32, 2 : i32], e = true}``."""

    def __init__(self, text):
        self.s, self.i = text, 0

    def _ws(self):
        while self.i < len(self.s) and self.s[self.i] in " \t\n":
            self.i += 1

    def value(self):
        self._ws()
        c = self.s[self.i]
        if c == "{":
            return self.dict()
        if c == "[":
            self.i += 1
            out = []
            while True:
                self._ws()
                if self.s[self.i] == "]":
                    self.i += 1
                    return out
                out.append(self.value())
                self._ws()
                if self.s[self.i] == ",":
                    self.i += 1
        if c == '"':
            j = self.s.index('"', self.i + 1)
            v = self.s[self.i + 1:j]
            self.i = j + 1
            return v
        m = re.match(r"[-+0-9.eE]+|true|false|\w+", self.s[self.i:])
        tok = m.group(0)
        self.i += len(tok)
        self._ws()
        if self.i < len(self.s) and self.s[self.i] == ":":  # type suffix ": i32"
            self.i += 1
            self._ws()
            self.i += len(re.match(r"[\w<>x]+", self.s[self.i:]).group(0))
        if tok == "true":
            return True
        if tok == "false":
            return False
        try:
            return int(tok)
        except ValueError:
            try:
                return float(tok)
            except ValueError:
                return tok

    def dict(self):
        self._ws()
        assert self.s[self.i] == "{"
        self.i += 1
        out = {}
        while True:
            self._ws()
            if self.s[self.i] == "}":
                self.i += 1
                return out
            m = re.match(r"[\w.]+", self.s[self.i:])
            key = m.group(0)
            self.i += len(key)
            self._ws()
            assert self.s[self.i] == "=", self.s[self.i:self.i + 20]
            self.i += 1
            out[key] = self.value()
            self._ws()
            if self.s[self.i] == ",":
                self.i += 1


def _shape(type_text):
    m = _TENSOR_RE.search(type_text)
    if not m:
        return None
    return [int(d) for d in m.group(1).split("x")]


_MODE_DTYPE = {"NONE": "FP32", "INT8": "INT8", "UINT8": "INT8", "BF16": "BF16"}

_CONV_KEYS = (("stride_h", "sh"), ("stride_w", "sw"), ("padding_t", "pt"), ("padding_b", "pb"), ("padding_l", "pl"),
              ("padding_r", "pr"), ("dilation_h", "dh"), ("dilation_w", "dw"), ("group", "g"))
_POOL_KEYS = (("kernel_h", "kh"), ("kernel_w", "kw"), ("stride_h", "sh"), ("stride_w", "sw"), ("padding_t", "pt"),
              ("padding_b", "pb"), ("padding_l", "pl"), ("padding_r", "pr"))


def convert(mlir_text):
    """Returns (module_text, weight_file_name_or_None). Ops this backend does not implement are still
    emitted (the loader rejects them by name)."""
    values = {}   # SSA id -> tensor / weight name, "-" for none
    shapes = {}   # name -> shape
    weight_shapes = {}
    lines = []
    weight_file = None
    for raw in mlir_text.splitlines():
        m = _OP_RE.match(raw)
        if not m:
            continue
        ssa, op, operands, attrs_text, _in_types, out_type = m.groups()
        attrs = _AttrParser(attrs_text).dict() if attrs_text else {}
        opnds = [o.strip() for o in operands.split(",") if o.strip()]
        if op == "weight_file":
            weight_file = attrs.get("filename")
            continue
        if op == "none":
            values[ssa] = "-"
            continue
        if op == "load_weight":
            values[ssa] = attrs["name"]
            weight_shapes[attrs["name"]] = _shape(out_type)
            continue
        name = attrs.get("name", ssa.lstrip("%"))
        values[ssa] = name
        shape = _shape(out_type) or []
        shapes[name] = shape
        ins = [values.get(o, o) for o in opnds if not o.startswith("%arg")]
        quant = attrs.get("quant", {}) if isinstance(attrs.get("quant"), dict) else {}
        dtype = _MODE_DTYPE.get(quant.get("mode", "NONE"), "FP32")
        kv = {}
        if op == "input":
            ins = []
        elif op == "quant":
            kv = {"from": attrs.get("from", "NONE"), "to": attrs.get("to", "NONE"), "scale": repr(float(attrs.get("scale", 1.0))),
                  "zero_point": int(attrs.get("zero_point", 0))}
            dtype = _MODE_DTYPE.get(kv["to"], "FP32")
        elif op in ("conv_2d", "deconv_2d"):
            p = attrs.get("param", {})
            w = weight_shapes.get(ins[1]) if len(ins) > 1 else None
            kv = {dst: int(p.get(src, 1 if dst in ("sh", "sw", "dh", "dw", "g") else 0)) for src, dst in _CONV_KEYS}
            if w:
                kv["kh"], kv["kw"] = w[-2], w[-1]
            kv["do_relu"] = int(bool(p.get("do_relu", False)))
            kv["with_bias"] = int(bool(p.get("with_bias", False)))
            ins_attr = p.get("ins", [])
            if ins_attr:
                kv["ins_w"], kv["ins_h"] = int(ins_attr[0]), int(ins_attr[-1])
        elif op in ("pool_avg_2d", "pool_max_2d"):
            p = attrs.get("param", {})
            kv = {dst: int(p.get(src, 0)) for src, dst in _POOL_KEYS}
            kv["count_include_pad"] = int(bool(p.get("count_include_pad", False)))
            kv["do_relu"] = int(bool(p.get("do_relu", False)))
        elif op == "fully_connected":
            kv = {"do_relu": int(bool(attrs.get("do_relu", False)))}
            if len(shape) == 3 and shape[1] == 1:      # [batch, 1, n] of the reference's matmul form
                pass
        elif op in ("eltwise_add", "eltwise_mul", "eltwise_max", "eltwise_min"):
            kv = {"do_relu": int(bool(attrs.get("do_relu", False)))}
            if "coeff" in attrs:
                kv["coeff"] = ",".join(repr(float(c)) for c in attrs["coeff"])
        elif op == "concat":
            kv = {"axis": int(attrs.get("axis", 1)), "do_relu": int(bool(attrs.get("do_relu", False)))}
        elif op == "upsample":
            kv = {"scale_h": int(attrs.get("scale_h", 1)), "scale_w": int(attrs.get("scale_w", 1))}
        elif op == "pixelshuffle":
            kv = {"upscale_factor": int(attrs.get("upscale_factor", 1)), "mode": attrs.get("mode", "CRD")}
        elif op == "leaky_relu":
            kv = {"negative_slope": repr(float(attrs.get("negative_slope", 0.0)))}
        elif op == "softmax":
            kv = {"axis": int(attrs.get("axis", 1)), "do_log": int(bool(attrs.get("do_log", False)))}
        elif op in ("eltwise_max", "eltwise_min"):
            kv = {"do_relu": int(bool(attrs.get("do_relu", False)))}
        elif op in ("broadcast_add", "broadcast_sub", "broadcast_mul"):
            kv = {"do_relu": int(bool(attrs.get("do_relu", False))), "align_right": int(bool(attrs.get("align_right", True)))}
        elif op == "pad":
            kv = {"pads": ",".join(str(int(v)) for v in attrs.get("pads", [])), "mode": attrs.get("mode", "constant"),
                  "const_val": repr(float(attrs.get("const_val", 0.0)))}
        elif op == "crop":
            kv = {"crop_offset": ",".join(str(int(v)) for v in attrs.get("crop_offset", []))}
            if attrs.get("steps"):
                kv["steps"] = ",".join(str(int(v)) for v in attrs["steps"])
        elif op == "permute":
            kv = {"order": ",".join(str(int(v)) for v in attrs.get("order", []))}
        elif op in ("reduce_mean", "reduce_sum", "reduce_max", "reduce_min"):
            kv = {"axes": ",".join(str(int(v)) for v in attrs.get("axes", []))}
        elif op == "matmul":
            kv = {k: int(bool(attrs.get(k, False))) for k in ("do_relu", "left_transpose", "right_transpose", "output_transpose")}
        if op == "reshape":
            dtype = None  # alias: inherits the operand's type
        parts = [op, "name=" + name]
        if ins:
            parts.append("in=" + ",".join(ins))
        parts.append("shape=" + ",".join(str(d) for d in shape))
        parts.append("dtype=" + (dtype or "FP32"))
        parts += ["%s=%s" % (k, v) for k, v in kv.items()]
        lines.append(" ".join(parts))
    return "\n".join(lines) + "\n", weight_file
