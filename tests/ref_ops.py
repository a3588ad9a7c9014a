"""Test helper: run one ggml operator on a ggml backend device through oracle/op_harness.cpp.

Device "CPU" is the reference's own CPU backend (the oracle); "B200_0" is the plugin under test.
"""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")
PLUGIN = os.path.join(ROOT, "whisper.cpp_b200", "libggml-b200.so")

OPS = dict(MUL_MAT=1, MUL_MAT_CONV=2, FLASH_ATTN=3, NORM=4, ADD=5, MUL=6, SCALE=7, GELU=8, CPY_F16=9, CONT_T=10,
           GET_ROWS=11, IM2COL=12, SOFT_MAX=13, CONCAT=14, KQ_NOFA=15, KQV_NOFA=16, CPY_F16_T=17, ROUNDTRIP=18, MM_TWICE=19)
F32, F16, Q5_0, Q8_0 = 0, 1, 6, 8
BLOCK = {Q5_0: 22, Q8_0: 34}

_lib = None
_n_dev = None


def have_ref():
    return os.path.exists(os.path.join(REF, "libop_harness.so"))


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(os.path.join(REF, "libop_harness.so"), mode=C.RTLD_GLOBAL)
        _lib.oph_run.restype = C.c_int64
        _lib.oph_run.argtypes = [C.c_char_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int]
        _lib.oph_quantize.restype = C.c_int64
        _lib.oph_quantize.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]
        _lib.oph_dequantize.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        _lib.oph_cpu_from_float.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        _lib.oph_load_backend.argtypes = [C.c_char_p]
        _lib.oph_try_alloc.argtypes = [C.c_char_p, C.c_int64]
        _lib.oph_unsupported_status.argtypes = [C.c_char_p]
    return _lib


def load_plugin():
    global _n_dev
    if _n_dev is None:
        _n_dev = lib().oph_load_backend(PLUGIN.encode())
    return _n_dev


def quantize(wtype, w):
    """reference ggml_quantize_chunk: f32 [rows, k] -> uint8 [rows, k/32, block]."""
    w = np.ascontiguousarray(w, np.float32)
    rows, k = w.shape
    out = np.empty((rows, k // 32, BLOCK[wtype]), np.uint8)
    n = lib().oph_quantize(wtype, w.ctypes.data, out.ctypes.data, rows, k)
    assert n == out.size
    return out


def dequantize(wtype, blocks):
    blocks = np.ascontiguousarray(blocks, np.uint8)
    n = blocks.size // BLOCK[wtype] * 32
    out = np.empty(n, np.float32)
    assert lib().oph_dequantize(wtype, blocks.ctypes.data, out.ctypes.data, n) == 0
    return out


def cpu_quantize_row_q8_0(x):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.size // 32 * 34, np.uint8)
    assert lib().oph_cpu_from_float(Q8_0, x.ctypes.data, out.ctypes.data, x.size) == 0
    return out.reshape(-1, 34)


def run(dev, op, p, f=(), inputs=(), out_shape=None, out_dtype=np.float32, threads=8):
    pa = (C.c_int64 * 16)(*list(p) + [0] * (16 - len(p)))
    fa = (C.c_float * 8)(*list(f) + [0.0] * (8 - len(f)))
    keep = [np.ascontiguousarray(a) if a is not None else None for a in inputs]
    ia = (C.c_void_p * 4)(*[(a.ctypes.data if a is not None else None) for a in keep] + [None] * (4 - len(keep)))
    out = np.empty(out_shape, out_dtype)
    n = lib().oph_run(dev.encode(), OPS[op], pa, fa, ia, out.ctypes.data, out.nbytes, threads)
    if n != out.nbytes:
        raise RuntimeError(f"oph_run({dev}, {op}) returned {n}, expected {out.nbytes}")
    return out
