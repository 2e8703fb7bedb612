"""ctypes access to oracle/oracle_c.c (CPU baseline + second-opinion checker).  Test tooling only."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build_c

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build_c.build())
        _lib.oc_num_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def num_threads() -> int:
    return int(lib().oc_num_threads())


def permute(x: np.ndarray, out_strides) -> np.ndarray:
    x = np.ascontiguousarray(x)
    out = np.empty(x.size, dtype=x.dtype)
    shape = (C.c_int64 * x.ndim)(*x.shape)
    st = (C.c_int64 * x.ndim)(*out_strides)
    lib().oc_permute(_p(x), _p(out), C.c_int(x.dtype.itemsize), C.c_int(x.ndim), shape, st)
    return out


def affine_relu_nchw_nhwc(x_bits: np.ndarray, s: np.ndarray, b: np.ndarray) -> np.ndarray:
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    n, c, h, w = x_bits.shape
    y = np.empty((n, h, w, c), dtype=np.uint16)
    s = np.ascontiguousarray(s, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    lib().oc_affine_relu_nchw_nhwc(_p(x_bits), _p(s), _p(b), _p(y), C.c_int64(n), C.c_int64(c), C.c_int64(h), C.c_int64(w))
    return y


def gemm_bf16(a_bits: np.ndarray, b_bits: np.ndarray, mask_bits=None, m_begin: int = 0, m_end=None) -> np.ndarray:
    a_bits = np.ascontiguousarray(a_bits, dtype=np.uint16)
    b_bits = np.ascontiguousarray(b_bits, dtype=np.uint16)
    m, k = a_bits.shape
    k2, n = b_bits.shape
    assert k == k2
    m_end = m if m_end is None else m_end
    out = np.empty((m_end - m_begin, n), dtype=np.float32)
    mp = _p(np.ascontiguousarray(mask_bits, dtype=np.uint16)) if mask_bits is not None else C.c_void_p(0)
    lib().oc_gemm_bf16(_p(a_bits), mp, _p(b_bits), _p(out), C.c_int64(m), C.c_int64(n), C.c_int64(k),
                       C.c_int64(m_begin), C.c_int64(m_end))
    return out


def c3_epilogue(acc: np.ndarray, mask_bits, y_bits, b1_bits, b2_bits, inv_n: float, m_begin: int = 0, m_total=None):
    acc = np.ascontiguousarray(acc, dtype=np.float32)
    rows, n = acc.shape
    m_total = rows + m_begin if m_total is None else m_total
    gt = np.zeros((m_total, n), dtype=np.uint16)
    gz1 = np.zeros((m_total, n), dtype=np.uint16)
    loss = np.zeros(1, dtype=np.float64)
    db2 = np.zeros(n, dtype=np.float64)
    db1 = np.zeros(n, dtype=np.float64)
    args = [np.ascontiguousarray(v, dtype=np.uint16) for v in (mask_bits, y_bits, b1_bits, b2_bits)]
    lib().oc_c3_epilogue(_p(acc), _p(args[0]), _p(args[1]), _p(args[2]), _p(args[3]), _p(gt), _p(gz1), _p(loss), _p(db2),
                         _p(db1), C.c_int64(n), C.c_int64(m_begin), C.c_int64(m_begin + rows), C.c_float(inv_n))
    return float(loss[0]), db2, db1, gt[m_begin:m_begin + rows], gz1[m_begin:m_begin + rows]
