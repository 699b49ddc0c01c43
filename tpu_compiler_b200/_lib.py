"""ctypes binding of libtpucb.so (the C ABI declared in include/tpucb.h).

The library is the product: there is no Python or CPU fallback. If it is missing
it is built in-tree with nvcc; if that fails the import error says so.
"""
import ctypes as C
import os

from . import build as _build

_lib = None


class TpucbError(RuntimeError):
    pass


def _declare(lib):
    vp, cp, sz = C.c_void_p, C.c_char_p, C.c_size_t
    fp = C.POINTER(C.c_float)
    i64p = C.POINTER(C.c_int64)
    ip = C.POINTER(C.c_int)
    szp = C.POINTER(C.c_size_t)
    lib.tpucb_last_error.restype = cp
    lib.tpucb_last_error.argtypes = []
    sigs = {
        "tpucb_version": [],
        "tpucb_interp_create": [C.c_int, C.POINTER(vp)],
        "tpucb_interp_create_batched": [C.c_int, C.c_int, C.POINTER(vp)],
        "tpucb_interp_max_batch_size": [vp, ip],
        "tpucb_interp_destroy": [vp],
        "tpucb_interp_set_tensor_slot": [vp, cp, fp, sz, C.c_int],
        "tpucb_interp_get_tensor_slot": [vp, cp, fp, sz, C.c_int],
        "tpucb_interp_invoke_slot": [vp, cp, C.c_int],
        "tpucb_interp_fast_invoke_all_batch": [vp, cp, C.c_int],
        "tpucb_interp_dump": [vp, cp, cp, sz, szp],
        "tpucb_op_create": [vp, cp, C.POINTER(vp)],
        "tpucb_op_invoke": [vp],
        "tpucb_op_set_tensor": [vp, fp, sz, C.c_int],
        "tpucb_op_get_tensor": [vp, fp, sz, C.c_int],
        "tpucb_op_info": [vp, cp, sz, szp],
        "tpucb_interp_set_weight": [vp, cp, fp, i64p, C.c_int],
        "tpucb_interp_load_module": [vp, cp],
        "tpucb_interp_set_tensor": [vp, cp, fp, sz],
        "tpucb_interp_set_tensor_async": [vp, cp, fp, sz],
        "tpucb_interp_set_tensor_async_i8": [vp, cp, vp, sz],
        "tpucb_interp_wait_uploads": [vp],
        "tpucb_interp_invoke": [vp],
        "tpucb_interp_invoke_to": [vp, cp],
        "tpucb_interp_launch": [vp],
        "tpucb_interp_sync": [vp],
        "tpucb_interp_get_tensor": [vp, cp, fp, sz],
        "tpucb_interp_get_tensor_shape": [vp, cp, i64p, ip],
        "tpucb_interp_get_data_type": [vp, cp, cp, sz],
        "tpucb_interp_get_all_tensor_names": [vp, cp, sz, szp],
        "tpucb_interp_get_details": [vp, C.c_int, cp, sz, szp],
        "tpucb_interp_get_op_info": [vp, cp, sz, szp],
        "tpucb_interp_set_option": [vp, cp, C.c_int],
        "tpucb_interp_profile": [vp, fp, C.c_int, ip],
        "tpucb_interp_time_launches": [vp, C.c_int, fp],
        "tpucb_interp_kernel_count": [vp, ip],
        "tpucb_interp_tensor_device": [vp, cp, C.POINTER(vp), szp, ip, ip, ip],
        "tpucb_measure_i8_mma_peak": [C.c_int, C.c_int, C.POINTER(C.c_double)],
        "tpucb_host_alloc": [C.POINTER(vp), sz],
        "tpucb_host_alloc_write_combined": [C.POINTER(vp), sz],
        "tpucb_host_free": [vp],
        "tpucb_calib_minmax": [vp, cp, vp],
        "tpucb_calib_hist": [vp, cp, C.c_float, C.c_int, vp],
        "tpucb_calib_minmax_keep": [vp, cp, vp, vp],
        "tpucb_calib_hist_kept": [vp, cp, vp, C.c_float, C.c_int, vp],
        "tpucb_calib_minmax_all": [vp, C.POINTER(cp), C.c_int, vp, C.POINTER(vp)],
        "tpucb_calib_hist_all": [vp, C.POINTER(cp), C.c_int, C.POINTER(vp), fp, C.c_int, vp],
        "tpucb_calib_kld": [vp, vp, fp, C.c_int, C.c_int, fp],
        "tpucb_interp_copy_tensor": [vp, cp, vp, cp],
        "tpucb_tuner_distance": [vp, cp, vp, cp, C.c_float, C.POINTER(C.c_double), C.c_int],
        "tpucb_calib_kld_static": [C.c_int, vp, vp, fp, C.c_int, C.c_int, fp],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = args
    return sigs


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB
        if not os.path.exists(path) or _build.stale():
            try:
                path = _build.build()
            except Exception as e:  # no nvcc: use the prebuilt file if there is one
                if not os.path.exists(path):
                    raise ImportError("libtpucb.so is missing and could not be built: %s" % e)
        _lib = C.CDLL(path)
        _declare(_lib)
    return _lib


def check(status):
    if status != 0:
        raise TpucbError(lib().tpucb_last_error().decode("utf-8", "replace"))
