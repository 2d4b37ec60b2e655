"""ctypes access to oracle/c/liboracle_c.so, the plain-C restatement of the two benchmark-critical reference goldens.
TEST INFRASTRUCTURE ONLY (tests and the benchmark's CPU-baseline leg); the product never imports this module."""
import ctypes
import os
import subprocess

import numpy as np

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "c")
_PATH = os.path.join(_DIR, "liboracle_c.so")
_lib = None


def lib(build=True):
    global _lib
    if _lib is None:
        if not os.path.exists(_PATH) and build:
            subprocess.run(["make", "-s", "-C", _DIR], check=True)
        L = ctypes.CDLL(_PATH)
        P, I64, I = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        L.oracle_qmm_int8_kc.argtypes = [P, P, I64, I64, I64, P, P, P, P, P, I]
        L.oracle_qmm_int8_kc.restype = None
        L.oracle_wq_w4a16_group.argtypes = [P, P, P, P, I64, I64, I64, I64, I64, I64, P, I]
        L.oracle_wq_w4a16_group.restype = None
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def qmm_int8_kc(x1, x2, s2, s1=None, bias=None, threads=1, want_acc=False):
    """x1 (m,k) int8, x2 (k,n) int8, s2 (n,) f32, s1 (m,) f32 | None, bias (n,) int32 | None -> bf16 bits (m,n) uint16."""
    x1 = np.ascontiguousarray(x1, np.int8)
    x2 = np.ascontiguousarray(x2, np.int8)
    s2 = np.ascontiguousarray(s2, np.float32)
    s1 = None if s1 is None else np.ascontiguousarray(s1, np.float32)
    bias = None if bias is None else np.ascontiguousarray(bias, np.int32)
    m, k = x1.shape
    n = x2.shape[1]
    out = np.empty((m, n), np.uint16)
    acc = np.empty((m, n), np.int32) if want_acc else None
    lib().oracle_qmm_int8_kc(_ptr(x1), _ptr(x2), m, k, n, _ptr(s2), _ptr(s1), _ptr(bias), _ptr(out), _ptr(acc), int(threads))
    return (out, acc) if want_acc else out


def wq_w4a16_group(x_bits, words, scale_bits, offset_bits, group, col_begin=0, col_end=None, threads=1):
    """x_bits (m,k) uint16 (bf16 bits), words (k,n/8) int32, scale/offset bits (k/group, n) uint16 -> y bits (m,n) uint16
    with columns [col_begin, col_end) filled."""
    x_bits = np.ascontiguousarray(x_bits, np.uint16)
    words = np.ascontiguousarray(words, np.int32)
    scale_bits = np.ascontiguousarray(scale_bits, np.uint16)
    offset_bits = None if offset_bits is None else np.ascontiguousarray(offset_bits, np.uint16)
    m, k = x_bits.shape
    n = words.shape[1] * 8
    col_end = n if col_end is None else col_end
    y = np.zeros((m, n), np.uint16)
    lib().oracle_wq_w4a16_group(_ptr(x_bits), _ptr(words), _ptr(scale_bits), _ptr(offset_bits), m, k, n, int(group),
                                int(col_begin), int(col_end), _ptr(y), int(threads))
    return y
