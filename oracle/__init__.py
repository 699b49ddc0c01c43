"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only tests, ``__graft_entry__.smoke`` and the CPU-baseline leg of ``bench.py``
import this package. Every tensor follows the reference interpreter's
container convention: float32 NCHW arrays whose values are int8 / bf16 / fp32.
"""
import ctypes as C
import os

import numpy as np

from . import build_oracle as _b

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None
_ref = None

_f = C.POINTER(C.c_float)


def _p(a):
    return None if a is None else a.ctypes.data_as(_f)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(_b.build_oracle())
        _lib.orc_bf16.restype = C.c_float
        _lib.orc_bf16.argtypes = [C.c_float, C.c_int]
        _lib.orc_f32_to_bf16.restype = C.c_uint16
        _lib.orc_f32_to_bf16.argtypes = [C.c_float, C.c_int]
        _lib.orc_f32_to_int8.argtypes = [C.c_float, C.c_int]
        _lib.orc_qdm_i32.argtypes = [C.c_int32, C.c_uint32, C.c_uint32]
        _lib.orc_qdm_f32.argtypes = [C.c_float, C.c_uint32, C.c_uint32]
        _lib.orc_mul_rshift_f32.argtypes = [C.c_float, C.c_uint32, C.c_uint32]
        _lib.orc_rshift_f32.argtypes = [C.c_float, C.c_uint32]
        _lib.orc_kld_threshold.restype = C.c_float
        _lib.orc_kld_threshold.argtypes = [C.c_void_p, C.c_float, C.c_longlong, C.c_void_p]
    return _lib


def ref():
    """The reference's own arithmetic, compiled unmodified (None if unavailable)."""
    global _ref
    if _ref is None:
        path = _b.build_ref()
        if path is None:
            return None
        _ref = C.CDLL(path)
        _ref.ref_bf16.restype = C.c_float
        _ref.ref_bf16.argtypes = [C.c_float, C.c_int]
        _ref.ref_f32_to_bf16.restype = C.c_uint16
        _ref.ref_f32_to_bf16.argtypes = [C.c_float, C.c_int]
        _ref.ref_f32_to_int8.argtypes = [C.c_float, C.c_int]
        _ref.ref_qdm_i32.argtypes = [C.c_int32, C.c_uint32, C.c_uint32]
        _ref.ref_qdm_f32.argtypes = [C.c_float, C.c_uint32, C.c_uint32]
        _ref.ref_mul_rshift_f32.argtypes = [C.c_float, C.c_uint32, C.c_uint32]
        _ref.ref_rshift_f32.argtypes = [C.c_float, C.c_uint32]
        _ref.kl_diversity_hist.restype = C.c_float
        _ref.kl_diversity_hist.argtypes = [C.c_void_p, C.c_float, C.c_longlong]
    return _ref


# --------------------------------------------------------------------------- ops
def conv2d(x, w, bias, rshift, multiplier, out_hw, stride=(1, 1), pad=(0, 0), dilation=(1, 1),
           groups=1, ins=(0, 0), do_relu=False, mode="INT8"):
    """core/conv.cpp Conv2DOpKernel::invoke. x [n,ic,ih,iw], w [oc,ic/g,kh,kw]; pad=(top,left)."""
    x, w = _f32(x), _f32(w)
    n, ic, ih, iw = x.shape
    oc, _, kh, kw = w.shape
    oh, ow = out_hw
    out = np.empty((n, oc, oh, ow), np.float32)
    bias, rshift, multiplier = _f32(bias), _f32(rshift), _f32(multiplier)
    m = {"INT8": 0, "FP32": 1, "BF16": 2}[mode]
    lib().orc_conv2d(_p(x), _p(w), _p(bias), _p(rshift), _p(multiplier), _p(out), n, ic, ih, iw, oc,
                     oh, ow, groups, kh, kw, stride[0], stride[1], pad[0], pad[1], dilation[0],
                     dilation[1], ins[0], ins[1], int(do_relu), m)
    return out


def deconv2d_i8(x, w, bias, rshift, multiplier, out_hw, stride=(1, 1), pad=(0, 0), dilation=(1, 1), groups=1,
                do_relu=False):
    """core/deconv.cpp DeConv2DOpKernel::invoke, INT8. x [n,ic,ih,iw], w [oc,ic/g,kh,kw] (oihw / goihw)."""
    x, w = _f32(x), _f32(w)
    n, ic, ih, iw = x.shape
    oc, _, kh, kw = w.shape
    oh, ow = out_hw
    out = np.empty((n, oc, oh, ow), np.float32)
    bias = _f32(bias) if bias is not None else None
    rshift, multiplier = _f32(rshift), _f32(multiplier)
    lib().orc_deconv2d_i8(_p(x), _p(w), _p(bias) if bias is not None else None, _p(rshift), _p(multiplier), _p(out),
                          n, ic, ih, iw, oc, oh, ow, groups, kh, kw, stride[0], stride[1], pad[0], pad[1],
                          dilation[0], dilation[1], int(do_relu))
    return out


def deconv2d_f(x, w, bias, out_hw, stride=(1, 1), pad=(0, 0), dilation=(1, 1), groups=1, do_relu=False, to_bf16=False):
    """core/deconv.cpp DeConv2DOpKernel::invoke, fp32 and BF16 graphs. x [n,ic,ih,iw], w [oc,ic/g,kh,kw]."""
    x, w = _f32(x), _f32(w)
    n, ic, ih, iw = x.shape
    oc, _, kh, kw = w.shape
    oh, ow = out_hw
    out = np.empty((n, oc, oh, ow), np.float32)
    bias = _f32(bias) if bias is not None else None
    lib().orc_deconv2d_f(_p(x), _p(w), _p(bias) if bias is not None else None, _p(out), n, ic, ih, iw, oc, oh, ow, groups,
                         kh, kw, stride[0], stride[1], pad[0], pad[1], dilation[0], dilation[1], int(do_relu),
                         int(to_bf16))
    return out


def fc(x, w, bias, rshift, multiplier, do_relu=False, mode="INT8"):
    """core/fullyconnected.cpp. x [batch?, m, k] or [m,k]; w [n,k]."""
    x, w = _f32(x), _f32(w)
    m, k = x.shape[-2], x.shape[-1]
    n = w.shape[-2]
    batch = int(np.prod(x.shape[:-2])) if x.ndim > 2 else 1
    out = np.empty(x.shape[:-1] + (n,), np.float32)
    bias, rshift, multiplier = _f32(bias), _f32(rshift), _f32(multiplier)
    md = {"INT8": 0, "FP32": 1, "BF16": 2}[mode]
    lib().orc_fc(_p(x), _p(w), _p(bias), _p(rshift), _p(multiplier), _p(out), batch, m, k, n,
                 int(do_relu), md)
    return out


def pool(x, kernel, stride, pad, out_hw, method="max", is_int8=True, count_include_pad=True,
         rshift=0.0, multiplier=0.0):
    """core/pooling.cpp. pad=(top,left); bottom/right pads are implied by out_hw."""
    x = _f32(x)
    n, c, ih, iw = x.shape
    oh, ow = out_hw
    out = np.empty((n, c, oh, ow), np.float32)
    lib().orc_pool(_p(x), _p(out), n, c, ih, iw, oh, ow, kernel[0], kernel[1], stride[0], stride[1],
                   pad[0], pad[1], 0 if method == "max" else 1, int(is_int8), int(count_include_pad),
                   C.c_float(rshift), C.c_float(multiplier))
    return out


def _ptr_array(arrs):
    arrs = [_f32(a) for a in arrs]
    pa = (_f * len(arrs))(*[_p(a) for a in arrs])
    return arrs, pa


def eltwise_add_i8(inputs, multiplier, rshift, do_relu=False):
    arrs, pa = _ptr_array(inputs)
    out = np.empty_like(arrs[0])
    m = _f32(multiplier)
    lib().orc_eltwise_add_i8(pa, len(arrs), _p(m), C.c_float(rshift), int(do_relu), _p(out),
                             C.c_size_t(out.size))
    return out


def eltwise_add_f32(inputs, coeff=None, do_relu=False, to_bf16=False):
    arrs, pa = _ptr_array(inputs)
    out = np.empty_like(arrs[0])
    c = _f32(coeff)
    lib().orc_eltwise_add_f32(pa, len(arrs), _p(c), int(do_relu), int(to_bf16), _p(out),
                              C.c_size_t(out.size))
    return out


def eltwise_mul_i8(inputs, multiplier, rshift, do_relu=False):
    arrs, pa = _ptr_array(inputs)
    out = np.empty_like(arrs[0])
    lib().orc_eltwise_mul_i8(pa, len(arrs), C.c_float(multiplier), C.c_float(rshift), int(do_relu),
                             _p(out), C.c_size_t(out.size))
    return out


def eltwise_maxmin_i8(inputs, multiplier, rshift, do_relu=False, is_min=False):
    arrs, pa = _ptr_array(inputs)
    out = np.empty_like(arrs[0])
    m = _f32(multiplier)
    lib().orc_eltwise_maxmin_i8(pa, len(arrs), _p(m), C.c_float(rshift), int(do_relu), int(is_min), _p(out),
                                C.c_size_t(out.size))
    return out


def _shape4(a, align_right=True):
    s = list(a.shape)
    return ([1] * (4 - len(s)) + s) if align_right else (s + [1] * (4 - len(s)))


def broadcast(a, b, op, is_int8=True, multiplier=None, rshift=0.0, do_relu=False):
    """op: "add" | "sub" | "mul"; shapes are aligned to 4-D on the right (the reference's default)."""
    a, b = _f32(a), _f32(b)
    sa, sb = _shape4(a), _shape4(b)
    so = [max(x, y) for x, y in zip(sa, sb)]
    out = np.empty(so, np.float32)
    m = _f32(multiplier if multiplier is not None else [1, 1])
    lib().orc_broadcast(_p(a), (C.c_int * 4)(*sa), _p(b), (C.c_int * 4)(*sb), {"add": 0, "sub": 1, "mul": 2}[op],
                        int(is_int8), _p(m), C.c_float(rshift), int(do_relu), _p(out))
    return out


def pad(x, pads, mode="constant"):
    x = _f32(x)
    s = list(x.shape)
    so = [s[i] + pads[i] + pads[i + 4] for i in range(4)]
    out = np.empty(so, np.float32)
    lib().orc_pad(_p(x), (C.c_int * 4)(*s), (C.c_int * 8)(*pads), 1 if mode == "edge" else 0, _p(out))
    return out


def crop(x, out_shape, offsets, steps=None):
    x = _f32(x)
    steps = list(steps) if steps else [1, 1, 1, 1]
    out = np.empty(list(out_shape), np.float32)
    lib().orc_crop(_p(x), (C.c_int * 4)(*x.shape), (C.c_int * 4)(*out_shape), (C.c_int * 4)(*offsets),
                   (C.c_int * 4)(*steps), _p(out))
    return out


def permute(x, order):
    x = _f32(x)
    out = np.empty([x.shape[o] for o in order], np.float32)
    lib().orc_permute(_p(x), (C.c_int * 4)(*x.shape), (C.c_int * 4)(*order), _p(out))
    return out


def reduce(x, axes, kind, is_int8=True, multiplier=1.0, rshift=0.0):
    """kind: "mean" | "sum" | "max" | "min" over consecutive axes; the reduced axes are dropped."""
    x = _f32(x)
    a0, a1 = axes[0], axes[-1] + 1
    outer = int(np.prod(x.shape[:a0], dtype=np.int64))
    axis = int(np.prod(x.shape[a0:a1], dtype=np.int64))
    inner = int(np.prod(x.shape[a1:], dtype=np.int64))
    out = np.empty(list(x.shape[:a0]) + list(x.shape[a1:]), np.float32)
    lib().orc_reduce(_p(x), outer, axis, inner, {"mean": 0, "sum": 1, "max": 2, "min": 3}[kind], int(is_int8),
                     C.c_float(multiplier), C.c_float(rshift), _p(out))
    return out


def matmul_dims(a_shape, out_shape, ltrans=False, rtrans=False, otrans=False):
    """(batch_high, batch_low, M, K, N) as parseMatMulParam derives them (TPUOperationSupport.cpp:615-655)."""
    axis = len(out_shape) - 1
    bh = bl = 1
    if ltrans or rtrans or otrans:
        k, n = a_shape[axis], out_shape[axis]
        if ltrans:
            bl, m = a_shape[axis - 1], a_shape[axis - 2]
        else:
            bl, m = a_shape[axis - 2], a_shape[axis - 1]
        if axis == 3:
            bh = a_shape[0]
        return bh, bl, m, k, n
    for d in a_shape[:axis - 1]:
        bh *= d
    return bh, 1, a_shape[axis - 1], a_shape[axis], out_shape[axis]


def matmul(a, b, out_shape, mode="INT8", rshift=0.0, multiplier=0.0, do_relu=False, ltrans=False, rtrans=False,
           otrans=False):
    """core/matmul.cpp: two activations, batched; see matmul_dims for the dimension rule."""
    a, b = _f32(a), _f32(b)
    bh, bl, m, k, n = matmul_dims(a.shape, out_shape, ltrans, rtrans, otrans)
    out = np.empty(out_shape, np.float32)
    assert a.size == bh * bl * m * k and b.size == bh * bl * k * n and out.size == bh * bl * m * n
    lib().orc_matmul(_p(a), _p(b), _p(out), bh, bl, m, k, n, int(ltrans), int(rtrans), int(otrans), int(do_relu),
                     {"INT8": 0, "FP32": 1, "BF16": 2}[mode], C.c_float(rshift), C.c_float(multiplier))
    return out


def concat_c(inputs, multiplier=None, rshift=None, do_relu=False):
    arrs, pa = _ptr_array(inputs)
    n, _, h, w = arrs[0].shape
    cs = np.array([a.shape[1] for a in arrs], np.int32)
    out = np.empty((n, int(cs.sum()), h, w), np.float32)
    need = multiplier is not None
    m, r = _f32(multiplier), _f32(rshift)
    lib().orc_concat_c(pa, len(arrs), cs.ctypes.data_as(C.POINTER(C.c_int)), n, h * w, _p(m), _p(r),
                       int(need), int(do_relu), _p(out))
    return out


def upsample(x, scale_h, scale_w):
    x = _f32(x)
    n, c, h, w = x.shape
    out = np.empty((n, c, h * scale_h, w * scale_w), np.float32)
    lib().orc_upsample(_p(x), _p(out), n, c, h, w, scale_h, scale_w)
    return out


def pixelshuffle(x, r, dcr_mode=False):
    x = _f32(x)
    n, c, h, w = x.shape
    out = np.empty((n, c // (r * r), h * r, w * r), np.float32)
    lib().orc_pixelshuffle(_p(x), _p(out), n, c, h, w, r, int(dcr_mode))
    return out


QUANT_KINDS = {"f32_i8_host": 0, "f32_i8": 1, "i8_f32": 2, "i8_bf16": 3, "bf16_i8": 4, "f32_bf16": 5}


def quant(x, scale, kind, zero_point=0):
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_quant(_p(x), _p(out), C.c_size_t(x.size), C.c_float(scale), int(zero_point),
                    QUANT_KINDS[kind])
    return out


def bf16_round(x):
    """F32ToBF16 with rounding over an array (QuantizationArithmetic.cpp:873-910): add 0x7fff plus the lowest kept
    bit, keep the high half; a result whose exponent is all ones becomes 0x7f7f."""
    u = _f32(x).view(np.uint32).astype(np.uint64)
    u = (u + 0x7fff + ((u >> 16) & 1)) & 0xffffffff
    h = (u >> 16).astype(np.uint32)
    h = np.where((h & 0x7f80) == 0x7f80, np.uint32(0x7f7f), h)
    return (h << 16).astype(np.uint32).view(np.float32).reshape(np.shape(x))


def leaky_relu_i8(x, rshift_pos, mult_pos, rshift_neg, mult_neg):
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_leaky_relu_i8(_p(x), _p(out), C.c_size_t(x.size), C.c_float(rshift_pos),
                            C.c_float(mult_pos), C.c_float(rshift_neg), C.c_float(mult_neg))
    return out


def relu(x):
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_relu(_p(x), _p(out), C.c_size_t(x.size))
    return out


def leaky_relu_f(x, negative_slope, to_bf16=False):
    """LeakyReluOpKernel::invoke, fp32 and BF16 (core/activation.cpp:129-131, 150-152; core/internal.cpp:20-25):
    x > 0 ? x : x * slope in fp32, then for BF16 one rounding."""
    x = _f32(x)
    out = np.where(x > 0, x, (x * np.float32(negative_slope)).astype(np.float32)).astype(np.float32)
    return bf16_round(out) if to_bf16 else out


LUT_KINDS = {"sigmoid": 0, "mish": 1, "exp": 2, "tanh": 3}


def lut_slope_tables(kind, p0=1.0, p1=0.0):
    base, slope = np.zeros(256, np.float32), np.zeros(256, np.float32)
    lib().orc_lut_gen_slope_tables(LUT_KINDS[kind], C.c_float(p0), C.c_float(p1), _p(base), _p(slope))
    return base, slope


def lut_bf16_slope(kind, x, base, slope):
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_lut_bf16_slope(LUT_KINDS[kind], _p(x), _p(out), C.c_size_t(x.size), _p(_f32(base)),
                             _p(_f32(slope)))
    return out


def lut_pow_tables(coeff):
    e, m = np.zeros(256, np.float32), np.zeros(256, np.float32)
    lib().orc_lut_gen_pow_tables(C.c_float(coeff), _p(e), _p(m))
    return e, m


def lut_bf16_mantissa(x, exp_table, mant_table):
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_lut_bf16_mantissa(_p(x), _p(out), C.c_size_t(x.size), _p(_f32(exp_table)),
                                _p(_f32(mant_table)))
    return out


def lut_log_tables():
    e, m = np.zeros(256, np.float32), np.zeros(256, np.float32)
    lib().orc_lut_gen_log_tables(_p(e), _p(m))
    return e, m


def lut_bf16_mantissa_log(x, exp_table, mant_table):
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_lut_bf16_mantissa_log(_p(x), _p(out), C.c_size_t(x.size), _p(_f32(exp_table)),
                                    _p(_f32(mant_table)))
    return out


def softmax_bf16(x, exp_table, exp_slope, rec_table, rec_mant, axis=1, do_log=False):
    """core/softmax.cpp:88-151; the last two tables are the reciprocal (pow -1) pair, or the log pair with do_log."""
    x = _f32(x)
    out = np.empty_like(x)
    outer = int(np.prod(x.shape[:axis]))
    inner = int(np.prod(x.shape[axis + 1:]))
    lib().orc_softmax_bf16(_p(x), _p(out), outer, x.shape[axis], inner, int(do_log), _p(_f32(exp_table)),
                           _p(_f32(exp_slope)), _p(_f32(rec_table)), _p(_f32(rec_mant)))
    return out


def lut_i8(x, table):
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_lut_i8(_p(x), _p(out), C.c_size_t(x.size), _p(_f32(table)))
    return out


def batchnorm_f32(x, mean, variance, scale0, eps):
    """BatchNormOpKernel, fp32 (core/batchnorm.cpp:20-68)."""
    x = _f32(x)
    n, c = x.shape[0], x.shape[1]
    out = np.empty_like(x)
    lib().orc_batchnorm_f32(_p(x), _p(_f32(mean)), _p(_f32(variance)), C.c_float(scale0), C.c_float(eps), _p(out), n, c,
                            x.size // (n * c))
    return out


def reduce_l2_f32(x, axes, coeff):
    """ReduceL2 over consecutive axes, fp32 (core/reduce.cpp:91-103); the reduced axes are dropped."""
    x = _f32(x)
    outer = int(np.prod(x.shape[:axes[0]], dtype=np.int64))
    axis = int(np.prod(x.shape[axes[0]:axes[-1] + 1], dtype=np.int64))
    inner = int(np.prod(x.shape[axes[-1] + 1:], dtype=np.int64))
    out = np.empty(outer * inner, np.float32)
    lib().orc_reduce_l2_f32(_p(x), outer, axis, inner, C.c_float(coeff), _p(out))
    return out.reshape(x.shape[:axes[0]] + x.shape[axes[-1] + 1:])


def scale_f32(x, scale, bias=None):
    x = _f32(x)
    out = np.empty_like(x)
    n, c = x.shape[:2]
    lib().orc_scale_f32(_p(x), _p(_f32(scale)), _p(_f32(bias)), _p(out), n, c, x.size // (n * c))
    return out


def softmax_f32(x, axis=1):
    x = _f32(x)
    out = np.empty_like(x)
    outer = int(np.prod(x.shape[:axis]))
    inner = int(np.prod(x.shape[axis + 1:]))
    lib().orc_softmax_f32(_p(x), _p(out), outer, x.shape[axis], inner)
    return out


def histogram(x, abs_max, bins=2048):
    x = _f32(x).ravel()
    hist = np.zeros(bins, np.int64)
    lib().orc_histogram(_p(x), C.c_size_t(x.size), C.c_float(abs_max), bins,
                        hist.ctypes.data_as(C.c_void_p))
    return hist


def kld_threshold(hist, width, bins=2048, return_kl=False):
    h = np.ascontiguousarray(hist, dtype=np.int32)
    kl = np.zeros(bins // 128, np.float32)
    t = lib().orc_kld_threshold(h.ctypes.data_as(C.c_void_p), C.c_float(width), bins,
                                kl.ctypes.data_as(C.c_void_p))
    return (t, kl) if return_kl else t
