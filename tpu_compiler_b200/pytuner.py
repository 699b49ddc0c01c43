"""``tuner``: the method set of the reference's ``pytuner.tuner`` (bindings/python/pytuner.cpp:290-310) over this
backend, so that a calibration script written against the reference binding (the loop of ``SimpleTuner.run``,
python/cvi_toolkit/calibration/kld_calibrator.py:156-201) drives the B200 path unchanged:

    t = tuner(n_images)          # one batch slot per calibration image
    t.load(fp32_module); t.build(); t.set_data(x, i) ...; t.invoke(); t.get_all_tensors(i)
    per op and candidate:  t.load(fp32_module); t.quantize(table_file); t.build(op); t.invoke(op)
                           t.get_tensor_type(op); t.get_tensor(op, i)

``load`` reads an fp32 module (this package's one-op-per-line text with its ``.npz``, or the reference's
generic-form ``.mlir``); ``quantize`` stands in for the reference's ``--import-calibration-table --tpu-quant`` passes
(``quantize.quantize_module``, the reference's weight quantisers bit for bit); ``build(target_op)`` loads the module
up to that op into an interpreter with ``batch`` slots; ``invoke`` is fastInvokeAllBatch: ONE launch over all slots.
Input data given with ``set_data`` survives ``load`` / ``quantize`` / ``build``, as it does in the reference, whose
interpreter keeps the input op's tensor while its signature is unchanged.
"""
import os
import re

import numpy as np

from . import quantize as Q
from .interpreter import module


def read_calibration_table(path):
    """{op name: threshold} from a calibration table: ``name threshold`` or ``name threshold min max`` lines, ``#``
    comments (ImportCalibrationTable.cpp:262-313; ``weight`` / ``bitwidth`` lines carry no activation threshold)."""
    table = {}
    num = r"[-0-9.e]+"
    old = re.compile(r"^(\S+)\s+(%s)$" % num)
    new = re.compile(r"^(\S+)\s+(%s)\s+%s\s+%s$" % (num, num, num))
    with open(path) as f:
        for raw in f:
            line = raw.rstrip("\r\n")
            if not line or line.startswith("#") or line.startswith("weight ") or line.startswith("bitwidth "):
                continue
            m = old.match(line) or new.match(line)
            if not m:
                raise ValueError("calibration table line does not match the required format: %r" % line)
            table[m.group(1)] = np.float32(m.group(2))
    return table


class tuner:
    version = "tpu_compiler_b200"

    def __init__(self, batch=1, device=0, module_cls=module):
        self.batch = int(batch)
        self._device = device
        self._module_cls = module_cls
        self._m = None
        self._fp32_text = self._text = None
        self._fp32_weights, self._weights = {}, {}
        self._table = None
        self._data = {}      # input name -> {bidx: array}
        self._inputs = []

    # ---- module -------------------------------------------------------------------------------------------------
    def load(self, mlir_file):
        """load module from fp32 mlir file"""
        with open(mlir_file) as f:
            text = f.read()
        weights = None
        if '"tpu.' in text:
            from . import mlir_text
            text, wf = mlir_text.convert(text)
            if wf:
                weights = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(mlir_file)), wf)))
        else:
            wf = mlir_file + ".npz"
            for line in text.splitlines():
                if line.startswith("# weight_file:"):
                    wf = os.path.join(os.path.dirname(os.path.abspath(mlir_file)), line.split(":", 1)[1].strip())
            if os.path.exists(wf):
                weights = dict(np.load(wf))
        self.load_text(text, weights or {})

    def load_text(self, text, weights):
        """``load`` for a module already in memory (module text + fp32 weight arrays)."""
        self._fp32_text, self._fp32_weights = text, dict(weights)
        self._text, self._weights, self._table = text, dict(weights), None
        self._inputs = [op["name"] for op in Q.parse_text(text) if op["type"] == "input"]

    def quantize(self, calib_table, mix_table=""):
        """quantization with calib_table and mix_table"""
        if mix_table:
            raise NotImplementedError("mixed-precision layer tables are not supported: every quantisable op becomes INT8")
        self._table = read_calibration_table(calib_table) if isinstance(calib_table, str) else dict(calib_table)
        self._text = None  # produced by build(), which knows the target op

    def build(self, target_op=""):
        """rebuild interpreter to target layer if set"""
        if self._fp32_text is None:
            raise RuntimeError("load a module first")
        if self._table is not None:
            text, qw = Q.quantize_module(self._fp32_text, self._fp32_weights, self._table, upto=target_op or None)
            weights = dict(self._fp32_weights)
            weights.update(qw)
        else:
            text, weights = self._fp32_text, self._fp32_weights
            if target_op:
                keep = []
                for op in Q.parse_text(text):
                    keep.append(Q.format_op(op))
                    if op["name"] == target_op:
                        break
                text = "\n".join(keep) + "\n"
        if self._m is not None:
            self._m.close()
        self._m = self._module_cls(self._device, max_batch_size=self.batch)
        self._m.load_text(text, weights)
        self._text, self._weights = text, weights
        for name, slots in self._data.items():
            for bidx, arr in slots.items():
                self._m.set_tensor(name, arr, bidx)

    # ---- data ---------------------------------------------------------------------------------------------------
    def set_data(self, *args):
        """set_data(array, bidx) or set_data(name, array, bidx) (bindings/python/pytuner.cpp:205-239)."""
        if len(args) == 2:
            name, (array, bidx) = "", args
        else:
            name, array, bidx = args
        if not name:
            name = self._inputs[0]
        if name not in self._inputs:
            raise RuntimeError("cannot find input tensor with name: %s" % name)
        arr = np.ascontiguousarray(array, np.float32)
        need = dict(self._m.input_sizes())[name] if self._m is not None else arr.size
        if arr.size != need:
            raise RuntimeError("input tensor size not same, needed is %d, get %d" % (need, arr.size))
        self._data.setdefault(name, {})[int(bidx)] = arr
        if self._m is not None:
            self._m.set_tensor(name, arr, int(bidx))

    def invoke(self, target_op=""):
        """run forward to target layer if set"""
        self._m.fast_invoke_all_batch(target_op, self.batch)

    # ---- results ------------------------------------------------------------------------------------------------
    def get_tensor(self, name, bidx):
        return self._m.get_tensor(name, int(bidx))

    def get_tensor_type(self, name):
        return self._m.get_data_type(name)

    def get_all_tensors(self, bidx):
        """{name: values of batch slot bidx as a 1-D array}, as the reference returns them."""
        return {n: self._m.get_tensor(n, int(bidx)).reshape(-1) for n in self._m.get_all_tensor_names()}

    def get_output_details(self):
        return self._m.get_output_details()

    def op_info(self):
        """[{name, type, quant}] of the loaded module (the module text when it has not been built yet)."""
        if self._m is not None:
            ops = [(o["name"], o["type"], o["dtype"]) for o in self._m.op_info]
        else:
            ops = [(o["name"], o["type"], o["dtype"]) for o in Q.parse_text(self._text or self._fp32_text)]
        return [{"name": n, "type": "tpu." + t, "quant": "NONE" if d == "FP32" else d} for n, t, d in ops]

    def close(self):
        if self._m is not None:
            self._m.close()
            self._m = None
