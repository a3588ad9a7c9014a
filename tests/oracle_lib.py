"""ctypes wrapper of oracle/liboracle.so (the CPU restatement; test infrastructure only)."""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(os.path.join(ROOT, "oracle", "liboracle.so"))
        _lib.orc_log_mel.restype = C.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def dequantize(wtype, blocks):
    blocks = np.ascontiguousarray(blocks, np.uint8)
    k = blocks.size // (22 if wtype == 6 else 34) * 32
    y = np.empty(k, np.float32)
    (lib().orc_dequantize_q5_0 if wtype == 6 else lib().orc_dequantize_q8_0)(_p(blocks), _p(y), C.c_int64(k))
    return y


def quantize_row_q8_0(x):
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    qs, d = np.empty(x.size, np.int8), np.empty(x.size // 32, np.float32)
    lib().orc_quantize_row_q8_0(_p(x), _p(qs), _p(d), C.c_int64(x.size))
    return qs, d


def mul_mat_q(wtype, w_blocks, M, K, x):
    x = np.ascontiguousarray(x, np.float32)
    w_blocks = np.ascontiguousarray(w_blocks, np.uint8)
    N = x.shape[0]
    dst = np.empty((N, M), np.float32)
    lib().orc_mul_mat_q(C.c_int(wtype), _p(w_blocks), C.c_int64(M), C.c_int64(K), _p(x), C.c_int64(N), _p(dst))
    return dst


def mul_mat_f16(w16, x):
    w16 = np.ascontiguousarray(w16, np.float16)
    x = np.ascontiguousarray(x, np.float32)
    M, K = w16.shape
    N = x.shape[0]
    dst = np.empty((N, M), np.float32)
    lib().orc_mul_mat_f16(_p(w16), C.c_int64(M), C.c_int64(K), _p(x), C.c_int64(N), _p(dst))
    return dst


def norm(x, eps=1e-5):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty_like(x)
    lib().orc_norm(_p(x), _p(y), C.c_int64(x.shape[-1]), C.c_int64(x.size // x.shape[-1]), C.c_float(eps))
    return y


def gelu(x):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty_like(x)
    lib().orc_gelu(_p(x), _p(y), C.c_int64(x.size))
    return y


def flash_attn(q, k, v, mask, scale):
    """q [n_q, H, 64] f32; k, v [n_kv, H, 64] f16; mask [>=n_q, n_kv] f16 or None -> [n_q, H, 64]."""
    q = np.ascontiguousarray(q, np.float32)
    k, v = np.ascontiguousarray(k, np.float16), np.ascontiguousarray(v, np.float16)
    n_q, H, _ = q.shape
    n_kv = k.shape[0]
    if mask is not None:
        mask = np.ascontiguousarray(mask, np.float16)
    dst = np.empty_like(q)
    lib().orc_flash_attn(_p(q), _p(k), _p(v), _p(mask), _p(dst), C.c_int64(n_q), C.c_int64(n_kv), C.c_int64(H), C.c_float(scale))
    return dst


def soft_max(x, mask, scale, ne01):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty_like(x)
    m32 = np.ascontiguousarray(mask, np.float32) if mask is not None and mask.dtype == np.float32 else None
    m16 = np.ascontiguousarray(mask, np.float16) if mask is not None and mask.dtype == np.float16 else None
    ne0 = x.shape[-1]
    lib().orc_soft_max(_p(x), _p(m32), _p(m16), _p(y), C.c_int64(ne0), C.c_int64(x.size // ne0), C.c_int64(ne01), C.c_float(scale))
    return y


def im2col_1d(x, KW, stride, pad=1, dil=1):
    x = np.ascontiguousarray(x, np.float32)
    IC, IW = x.shape
    OW = (IW + 2 * pad - dil * (KW - 1) - 1) // stride + 1
    dst = np.empty((OW, IC * KW), np.float16)
    lib().orc_im2col_1d(_p(x), C.c_int64(IW), C.c_int64(IC), C.c_int64(KW), C.c_int64(OW), C.c_int(stride), C.c_int(pad), C.c_int(dil), _p(dst))
    return dst


def log_mel(pcm, filters):
    pcm = np.ascontiguousarray(pcm, np.float32)
    filters = np.ascontiguousarray(filters, np.float32)
    n_mel = filters.shape[0]
    n_len = (pcm.size + 480000 + 400 - 400) // 160
    mel = np.empty((n_mel, n_len), np.float32)
    r = lib().orc_log_mel(_p(pcm), C.c_int64(pcm.size), _p(filters), C.c_int(n_mel), _p(mel), C.c_int64(mel.size))
    assert r == n_len
    return mel
