"""ctypes loader for the plain-C oracle (oracle/fp8_oracle.c) and the toolkit-converter pin.

TEST INFRASTRUCTURE: used by tests/ and the smoke check only.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(HERE, "_build", "libfp8_oracle.so")
_REF = os.path.join(HERE, "_ref", "libref_fp8_cvt.so")


def build():
    subprocess.run(["make", "-s", "-C", HERE], check=True)


def _load(path):
    if not os.path.exists(path):
        build()
    return ctypes.CDLL(path)


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        _lib = _load(_LIB)
        _lib.fp8_oracle_cvt.restype = ctypes.c_uint8
        _lib.fp8_oracle_cvt.argtypes = [ctypes.c_float, ctypes.c_int]
        _lib.fp8_oracle_to_f32.restype = ctypes.c_float
        _lib.fp8_oracle_to_f32.argtypes = [ctypes.c_uint8, ctypes.c_int]
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def cvt_array(x_f32, fmt):
    """float32 array -> fp8 bytes with the C oracle's converter."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    out = np.empty(x.size, dtype=np.uint8)
    lib().fp8_oracle_cvt_array(_p(x), _p(out), ctypes.c_int64(x.size), ctypes.c_int(fmt))
    return out.reshape(x.shape)


def quantize(in_bf16_u16, scale, fmt, amax0=0.0):
    x = np.ascontiguousarray(in_bf16_u16, dtype=np.uint16)
    out = np.empty(x.size, dtype=np.uint8)
    am = ctypes.c_float(amax0)
    lib().fp8_oracle_quantize(_p(x), _p(out), ctypes.c_int64(x.size), ctypes.c_float(scale), ctypes.c_int(fmt),
                              ctypes.byref(am))
    return out.reshape(x.shape), am.value


def pad_cast_transpose(in_bf16_u16, scale, fmt, padded_rows, gelu_in=None, amax0=0.0):
    x = np.ascontiguousarray(in_bf16_u16, dtype=np.uint16)
    rows, cols = x.shape
    gi = np.ascontiguousarray(gelu_in, dtype=np.uint16) if gelu_in is not None else None
    out = np.empty((rows, cols), dtype=np.uint8)
    out_t = np.empty((cols, padded_rows), dtype=np.uint8)
    am = ctypes.c_float(amax0)
    lib().fp8_oracle_pad_cast_transpose(_p(x), _p(gi), _p(out), _p(out_t), ctypes.c_int64(rows), ctypes.c_int64(cols),
                                        ctypes.c_int64(padded_rows), ctypes.c_float(scale), ctypes.c_int(fmt),
                                        ctypes.byref(am))
    return out, out_t, am.value


def pad_transpose(in_u8, padded_rows):
    x = np.ascontiguousarray(in_u8, dtype=np.uint8)
    rows, cols = x.shape
    out_t = np.empty((cols, padded_rows), dtype=np.uint8)
    lib().fp8_oracle_pad_transpose(_p(x), _p(out_t), ctypes.c_int64(rows), ctypes.c_int64(cols),
                                   ctypes.c_int64(padded_rows))
    return out_t


def scale_mul(x_bf16_u16, s1, s2):
    x = np.ascontiguousarray(x_bf16_u16, dtype=np.uint16).copy()
    lib().fp8_oracle_scale_mul(_p(x), ctypes.c_int64(x.size), ctypes.c_float(s1), ctypes.c_float(s2))
    return x


def gemm_nt(a_u8, a_fmt, b_u8, b_fmt, alpha):
    a = np.ascontiguousarray(a_u8, dtype=np.uint8)
    b = np.ascontiguousarray(b_u8, dtype=np.uint8)
    m, k = a.shape
    n = b.shape[0]
    c = np.empty((m, n), dtype=np.uint16)
    lib().fp8_oracle_gemm_nt(_p(a), ctypes.c_int(a_fmt), _p(b), ctypes.c_int(b_fmt), _p(c), ctypes.c_int64(m),
                             ctypes.c_int64(n), ctypes.c_int64(k), ctypes.c_float(alpha))
    return c


def toolkit_cvt(x_f32, fmt):
    """The CUDA toolkit's host-side __nv_fp8_* constructor (what the reference's kernels call)."""
    global _ref
    if _ref is None:
        _ref = _load(_REF)
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    out = np.empty(x.size, dtype=np.uint8)
    _ref.ref_fp8_cvt_array(_p(x), _p(out), ctypes.c_int64(x.size), ctypes.c_int(fmt))
    return out.reshape(x.shape)
