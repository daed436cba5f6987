"""numpy front end of cdr_oracle.c (TEST INFRASTRUCTURE ONLY).

bf16 arrays travel as ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes
from functools import lru_cache

import numpy as np

from .build import build

_i64 = ctypes.c_int64
_p = ctypes.c_void_p


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    l = ctypes.CDLL(str(build()))
    sig = {
        "oracle_mul_add_f32": [_p, _p, _p, _p, _i64],
        "oracle_addcdiv_f32": [_p, _p, _p, ctypes.c_float, _p, _i64],
        "oracle_relu_f32": [_p, _p, _i64],
        "oracle_add_i32": [_p, _p, _p, _i64],
        "oracle_mul_add_bf16": [_p, _p, _p, _p, _i64],
        "oracle_mean_relu_mul_add_bf16": [_p, _p, _p, _p, _i64, _i64],
        "oracle_row_sum_f32": [_p, _p, _i64, _i64, ctypes.c_int],
        "oracle_softmax_f32": [_p, _p, _i64, _i64],
        "oracle_online_softmax_f32": [_p, _p, _i64, _i64],
        "oracle_softmax_backward_jacobian_f32": [_p, _p, _p, _i64, _i64],
        "oracle_softmax_backward_f32": [_p, _p, _p, _i64, _i64],
        "oracle_linear_bf16": [_p, _p, _p, _p, _i64, _i64, _i64, ctypes.c_int],
        "oracle_matmul_i32": [_p, _p, _p, _i64, _i64, _i64],
        "oracle_attention_f32": [_p, _p, _p, _p, _i64, _i64, _i64, ctypes.c_double, ctypes.c_int],
        "oracle_attention_bf16": [_p, _p, _p, _p, _i64, _i64, _i64, ctypes.c_double, ctypes.c_int],
    }
    for name, argtypes in sig.items():
        fn = getattr(l, name)
        fn.argtypes = argtypes
        fn.restype = None
    return l


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a, a.ctypes.data


def mul_add_f32(a, b, c):
    a, pa = _c(a, np.float32); b, pb = _c(b, np.float32); c, pc = _c(c, np.float32)
    out = np.empty_like(a)
    lib().oracle_mul_add_f32(pa, pb, pc, out.ctypes.data, a.size)
    return out


def addcdiv_f32(a, b, c, value=1.0):
    a, pa = _c(a, np.float32); b, pb = _c(b, np.float32); c, pc = _c(c, np.float32)
    out = np.empty_like(a)
    lib().oracle_addcdiv_f32(pa, pb, pc, value, out.ctypes.data, a.size)
    return out


def relu_f32(x):
    x, px = _c(x, np.float32)
    out = np.empty_like(x)
    lib().oracle_relu_f32(px, out.ctypes.data, x.size)
    return out


def add_i32(a, b):
    a, pa = _c(a, np.int32); b, pb = _c(b, np.int32)
    out = np.empty_like(a)
    lib().oracle_add_i32(pa, pb, out.ctypes.data, a.size)
    return out


def mul_add_bf16(a, b, c):
    a, pa = _c(a, np.uint16); b, pb = _c(b, np.uint16); c, pc = _c(c, np.uint16)
    out = np.empty_like(a)
    lib().oracle_mul_add_bf16(pa, pb, pc, out.ctypes.data, a.size)
    return out


def mean_relu_mul_add_bf16(x, w, b):
    x, px = _c(x, np.uint16); w, pw = _c(w, np.uint16); b, pb = _c(b, np.uint16)
    rows, cols = x.shape
    out = np.empty(rows, dtype=np.float32)
    lib().oracle_mean_relu_mul_add_bf16(px, pw, pb, out.ctypes.data, rows, cols)
    return out


def row_sum_f32(x, mean=False):
    x, px = _c(x, np.float32)
    rows, cols = x.shape
    out = np.empty(rows, dtype=np.float32)
    lib().oracle_row_sum_f32(px, out.ctypes.data, rows, cols, int(mean))
    return out


def softmax_f32(x, online=False):
    x, px = _c(x, np.float32)
    m, n = x.shape
    out = np.empty_like(x)
    (lib().oracle_online_softmax_f32 if online else lib().oracle_softmax_f32)(px, out.ctypes.data, m, n)
    return out


def softmax_backward_f32(y, dy, jacobian=False):
    y, py = _c(y, np.float32); dy, pdy = _c(dy, np.float32)
    m, n = y.shape
    out = np.empty_like(y)
    fn = lib().oracle_softmax_backward_jacobian_f32 if jacobian else lib().oracle_softmax_backward_f32
    fn(py, pdy, out.ctypes.data, m, n)
    return out


def linear_bf16(x, w, bias=None, relu=False):
    x, px = _c(x, np.uint16); w, pw = _c(w, np.uint16)
    M, K = x.shape
    N = w.shape[0]
    pb = None
    if bias is not None:
        bias, pb = _c(bias, np.uint16)
    out = np.empty((M, N), dtype=np.uint16)
    lib().oracle_linear_bf16(px, pw, pb, out.ctypes.data, M, N, K, int(relu))
    return out


def matmul_i32(lhs, rhs):
    lhs, pl = _c(lhs, np.int32); rhs, pr = _c(rhs, np.int32)
    M, K = lhs.shape
    N = rhs.shape[1]
    out = np.zeros((M, N), dtype=np.int32)
    lib().oracle_matmul_i32(pl, pr, out.ctypes.data, M, N, K)
    return out


def attention_f32(q, k, v, scale, causal):
    q, pq = _c(q, np.float32); k, pk = _c(k, np.float32); v, pv = _c(v, np.float32)
    seq, dim = q.shape[-2:]
    bh = q.size // (seq * dim)
    out = np.empty_like(q)
    lib().oracle_attention_f32(pq, pk, pv, out.ctypes.data, bh, seq, dim, float(scale), int(causal))
    return out


def attention_bf16(q, k, v, scale, causal):
    q, pq = _c(q, np.uint16); k, pk = _c(k, np.uint16); v, pv = _c(v, np.uint16)
    seq, dim = q.shape[-2:]
    bh = q.size // (seq * dim)
    out = np.empty_like(q)
    lib().oracle_attention_bf16(pq, pk, pv, out.ctypes.data, bh, seq, dim, float(scale), int(causal))
    return out
