"""``module``: the pymlir.module method set (bindings/python/pymlir.cpp:289-311) over the
C ABI of libtpucb.so. Tensors cross as float32 numpy arrays in the logical (NCHW) shape,
exactly as they do with the reference binding."""
import ctypes as C
import os

import numpy as np

from ._lib import check, lib

_f = C.POINTER(C.c_float)


def _text(fn, *prefix):
    need = C.c_size_t(0)
    check(fn(*prefix, None, 0, C.byref(need)))
    buf = C.create_string_buffer(need.value + 1)
    check(fn(*prefix, buf, need.value + 1, C.byref(need)))
    return buf.value.decode()


class op_kernel:
    """One op owned by itself: the CPUOpKernel surface (include/tpuc/Interpreter/cpukernel.h:87-159) over
    tpucb_op_*. Made by ``module.create_op``; the module is the value / weight map it looks its operands up in."""

    def __init__(self, owner, handle):
        self._m, self._h = owner, handle

    def _info(self):
        name, typ, dt, shape, dirty = _text(self._m._lib.tpucb_op_info, self._h).split("\t")
        return name, typ, dt, [int(v) for v in shape.split(",") if v], dirty == "1"

    name = property(lambda self: self._info()[0])
    op_type = property(lambda self: self._info()[1])
    datatype = property(lambda self: self._info()[2])
    shape = property(lambda self: self._info()[3])
    dirty = property(lambda self: self._info()[4])

    def invoke(self):
        check(self._m._lib.tpucb_op_invoke(self._h))

    def set_tensor(self, array, bidx=0):
        a = np.ascontiguousarray(array, dtype=np.float32)
        check(self._m._lib.tpucb_op_set_tensor(self._h, a.ctypes.data_as(_f), a.size, int(bidx)))

    def get_tensor(self, bidx=0):
        out = np.empty(self.shape, np.float32)
        check(self._m._lib.tpucb_op_get_tensor(self._h, out.ctypes.data_as(_f), out.size, int(bidx)))
        return out


class module:
    def __init__(self, device=0, max_batch_size=1):
        """``max_batch_size``: the constructor argument of MlirModuleInterpreter (MlirModuleInterpreter.h:35): that many
        batch slots per tensor, addressed by the ``bidx`` arguments below."""
        self._h = C.c_void_p()
        self._device = device
        self._lib = lib()
        self.max_batch_size = int(max_batch_size)
        if self.max_batch_size == 1:
            check(self._lib.tpucb_interp_create(int(device), C.byref(self._h)))
        else:
            check(self._lib.tpucb_interp_create_batched(int(device), self.max_batch_size, C.byref(self._h)))
        self._weight_file = None
        self.op_info = []

    def __del__(self):
        try:
            if self._h:
                self._lib.tpucb_interp_destroy(self._h)
                self._h = C.c_void_p()
        except Exception:
            pass

    close = __del__

    # ---- loading ---------------------------------------------------------------
    def load(self, mlir_file, weights=None):
        """pymlir.module.load: ``mlir_file`` is a module text file; its weights come from the
        ``.npz`` written next to it (``<file>.npz``, or the path on a ``# weight_file:`` line)."""
        with open(mlir_file) as f:
            text = f.read()
        if weights is None:
            wf = mlir_file + ".npz"
            for line in text.splitlines():
                if line.startswith("# weight_file:"):
                    wf = os.path.join(os.path.dirname(mlir_file), line.split(":", 1)[1].strip())
            self._weight_file = wf
            weights = dict(np.load(wf))
        self.load_text(text, weights)

    def load_mlir(self, mlir_file, weights=None):
        """Loads a generic-form TPU-dialect ``.mlir`` as the reference writes it; weights come from
        the ``.npz`` its ``tpu.weight_file`` op names (looked up next to the file) unless given."""
        from . import mlir_text
        with open(mlir_file) as f:
            text, wf = mlir_text.convert(f.read())
        if weights is None:
            weights = {}
            if wf:
                self._weight_file = os.path.join(os.path.dirname(os.path.abspath(mlir_file)), wf)
                weights = dict(np.load(self._weight_file))
        self.load_text(text, weights)

    def set_weights(self, weights):
        """updateWeightMap: registers fp32 weight arrays by name (before load_text / create_op)."""
        for name, arr in weights.items():
            a = np.ascontiguousarray(arr, dtype=np.float32)
            shape = (C.c_int64 * max(a.ndim, 1))(*(a.shape if a.ndim else (1,)))
            check(self._lib.tpucb_interp_set_weight(self._h, name.encode(), a.ctypes.data_as(_f), shape,
                                                    max(a.ndim, 1)))

    def create_op(self, op_line):
        """One op from one line of module text (its operands must exist already): an ``op_kernel``."""
        h = C.c_void_p()
        check(self._lib.tpucb_op_create(self._h, op_line.encode(), C.byref(h)))
        self._refresh_op_info()
        return op_kernel(self, h)

    def load_text(self, text, weights):
        self.set_weights(weights)
        check(self._lib.tpucb_interp_load_module(self._h, text.encode()))
        self._refresh_op_info()

    def _refresh_op_info(self):
        self.op_info = []
        for line in _text(self._lib.tpucb_interp_get_op_info, self._h).splitlines():
            name, typ, dt, shape, ops, nbytes, bound = line.split("\t")
            self.op_info.append({"name": name, "type": typ, "dtype": dt,
                                 "shape": [int(s) for s in shape.split(",") if s],
                                 "ops": float(ops), "bytes": float(nbytes), "bound": bound})

    def get_weight_file_path(self):
        return self._weight_file

    # ---- tensors ---------------------------------------------------------------
    def set_tensor(self, name, array, bidx=None):
        """``bidx`` None: the whole tensor (with max_batch_size > 1: all slots, slot-major); else one batch slot."""
        a = np.ascontiguousarray(array, dtype=np.float32)
        if bidx is None:
            check(self._lib.tpucb_interp_set_tensor(self._h, name.encode(), a.ctypes.data_as(_f), a.size))
        else:
            check(self._lib.tpucb_interp_set_tensor_slot(self._h, name.encode(), a.ctypes.data_as(_f), a.size, int(bidx)))

    def set_tensor_ptr(self, name, host_ptr, numel):
        """Same as set_tensor, from a raw (e.g. pinned) host pointer."""
        check(self._lib.tpucb_interp_set_tensor(self._h, name.encode(), C.cast(host_ptr, _f), numel))

    def set_tensor_async(self, name, host_ptr, numel):
        """Pipelined set_tensor from PINNED host memory: the copy overlaps the launch in flight."""
        check(self._lib.tpucb_interp_set_tensor_async(self._h, name.encode(), C.cast(host_ptr, _f), numel))

    def set_tensor_async_i8(self, name, host_ptr, numel):
        """Pipelined upload of already quantised int8 values (NCHW, pinned) into an INT8 input tensor or into the
        result of the quant op right behind an fp32 input (that op is then skipped): a quarter of the bytes."""
        check(self._lib.tpucb_interp_set_tensor_async_i8(self._h, name.encode(), C.cast(host_ptr, C.c_void_p), numel))

    def wait_uploads(self):
        """Blocks until every set_tensor_async copy has left its pinned host buffer."""
        check(self._lib.tpucb_interp_wait_uploads(self._h))

    def get_tensor_shape(self, name):
        shape = (C.c_int64 * 8)()
        rank = C.c_int(0)
        check(self._lib.tpucb_interp_get_tensor_shape(self._h, name.encode(), shape, C.byref(rank)))
        return [int(shape[i]) for i in range(rank.value)]

    def get_tensor(self, name, bidx=None):
        shape = self.get_tensor_shape(name)
        if bidx is None:
            if self.max_batch_size > 1:
                shape = [shape[0] * self.max_batch_size] + shape[1:]
            out = np.empty(shape, np.float32)
            check(self._lib.tpucb_interp_get_tensor(self._h, name.encode(), out.ctypes.data_as(_f), out.size))
        else:
            out = np.empty(shape, np.float32)
            check(self._lib.tpucb_interp_get_tensor_slot(self._h, name.encode(), out.ctypes.data_as(_f), out.size, int(bidx)))
        return out

    def get_tensor_into(self, name, host_ptr, numel):
        check(self._lib.tpucb_interp_get_tensor(self._h, name.encode(), C.cast(host_ptr, _f), numel))

    def get_data_type(self, name):
        buf = C.create_string_buffer(16)
        check(self._lib.tpucb_interp_get_data_type(self._h, name.encode(), buf, 16))
        return buf.value.decode()

    def get_all_tensor_names(self):
        return [n for n in _text(self._lib.tpucb_interp_get_all_tensor_names, self._h).splitlines() if n]

    def get_all_tensor(self, bidx=None):
        return {n: self.get_tensor(n, bidx) for n in self.get_all_tensor_names()}

    def _details(self, outputs, sizes=False):
        out = []
        for line in _text(self._lib.tpucb_interp_get_details, self._h, int(outputs)).splitlines():
            if line:
                n, sz = line.rsplit(":", 1)
                out.append((n, int(sz)) if sizes else n)
        return out

    def input_sizes(self):
        """input_details of the reference: (name, element count of one batch slot) in module order."""
        return self._details(False, sizes=True)

    def dump(self, name):
        """MlirModuleInterpreter::dump: a text description of one op."""
        return _text(self._lib.tpucb_interp_dump, self._h, name.encode())

    def get_input_details(self):
        return self._details(False)

    def get_output_details(self):
        return self._details(True)

    # ---- execution -------------------------------------------------------------
    def invoke(self, bidx=None):
        if bidx is None:
            check(self._lib.tpucb_interp_invoke(self._h))
        else:
            check(self._lib.tpucb_interp_invoke_slot(self._h, None, int(bidx)))

    def invoke_to(self, name, bidx=None):
        if bidx is None:
            check(self._lib.tpucb_interp_invoke_to(self._h, name.encode()))
        else:
            check(self._lib.tpucb_interp_invoke_slot(self._h, name.encode(), int(bidx)))

    def fast_invoke_all_batch(self, name="", batch=None):
        """fastInvokeAllBatch: the ops built since the last such call, up to ``name``, over all batch slots at once."""
        check(self._lib.tpucb_interp_fast_invoke_all_batch(self._h, name.encode() if name else None,
                                                           int(batch or self.max_batch_size)))

    def launch(self):
        check(self._lib.tpucb_interp_launch(self._h))

    def sync(self):
        check(self._lib.tpucb_interp_sync(self._h))

    def run(self, input, target_op=""):
        """pymlir.module.run (bindings/python/pymlir.cpp:215-266): ``input`` holds the values of all inputs one after
        the other in module order; runs the module (up to ``target_op`` when given) and returns the outputs (or that
        op's tensor) as a dict."""
        flat = np.ascontiguousarray(input, dtype=np.float32).reshape(-1)
        ins = self.input_sizes()
        scale = self.max_batch_size
        need = sum(sz for _, sz in ins) * scale
        if flat.size != need:
            raise RuntimeError("input data size %d not same with all input needed size %d" % (flat.size, need))
        at = 0
        for name, sz in ins:
            self.set_tensor(name, flat[at:at + sz * scale])
            at += sz * scale
        if target_op:
            self.invoke_to(target_op)
            return {target_op: self.get_tensor(target_op)}
        self.invoke()
        return {n: self.get_tensor(n) for n in self.get_output_details()}

    # ---- measurement helpers ------------------------------------------------------
    def set_option(self, key, value):
        check(self._lib.tpucb_interp_set_option(self._h, key.encode(), int(value)))

    def profile(self):
        n = len(self.op_info)
        ms = (C.c_float * max(n, 1))()
        cnt = C.c_int(0)
        check(self._lib.tpucb_interp_profile(self._h, ms, n, C.byref(cnt)))
        return [float(ms[i]) for i in range(cnt.value)]

    def time_launches(self, iters):
        ms = C.c_float(0)
        check(self._lib.tpucb_interp_time_launches(self._h, int(iters), C.byref(ms)))
        return float(ms.value)

    def kernel_count(self):
        c = C.c_int(0)
        check(self._lib.tpucb_interp_kernel_count(self._h, C.byref(c)))
        return int(c.value)

    def tensor_device(self, name):
        dev, nbytes = C.c_void_p(), C.c_size_t()
        c, cp, dt = C.c_int(), C.c_int(), C.c_int()
        check(self._lib.tpucb_interp_tensor_device(self._h, name.encode(), C.byref(dev), C.byref(nbytes), C.byref(c),
                                                   C.byref(cp), C.byref(dt)))
        return {"ptr": dev.value, "bytes": nbytes.value, "channels": c.value, "pitch": cp.value, "dtype": dt.value}

    # ---- tuner helpers ---------------------------------------------------------------
    def copy_tensor_from(self, name, other, other_name):
        """Device-to-device copy of ``other_name`` of module ``other`` into this module's ``name``
        (same GPU, same type, shape and device layout)."""
        check(self._lib.tpucb_interp_copy_tensor(self._h, name.encode(), other._h, other_name.encode()))

    def tuner_distance(self, name, ref, ref_name, scale):
        """Per image of the batch: (sum (ref - scale * this)^2, sum |ref|) between this module's
        ``name`` and the fp32 tensor ``ref_name`` of module ``ref``, both left on the device.
        Returns a float64 array [images, 2]."""
        n = self.get_tensor_shape(name)[0]
        out = np.zeros((n, 2), np.float64)
        check(self._lib.tpucb_tuner_distance(ref._h, ref_name.encode(), self._h, name.encode(), float(scale),
                                             out.ctypes.data_as(C.POINTER(C.c_double)), n))
        return out
