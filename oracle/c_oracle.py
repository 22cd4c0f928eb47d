"""ctypes front-end of the C oracle (oracle/kbn_oracle.c).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libkbn_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "kbn_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libkbn_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


_i64 = ctypes.c_int64


def quant_1x128(x_bf16_bits: np.ndarray, eps: float = 1e-10, ue8m0: bool = True, colmajor: bool = False):
    """x: uint16 [M,K] bf16 bit patterns -> (uint8 [M,K], float32 [M,G] (strides (1,M) if colmajor))."""
    x = np.ascontiguousarray(x_bf16_bits, dtype=np.uint16)
    m, k = x.shape
    g = (k + 127) // 128
    q = np.empty((m, k), np.uint8)
    s = np.empty((g, m) if colmajor else (m, g), np.float32)
    srow, sgrp = (1, m) if colmajor else (g, 1)
    lib().kbo_quant_1x128(_p(x), _i64(m), _i64(k), _i64(k), _p(q), _i64(k), _p(s), _i64(srow), _i64(sgrp),
                          ctypes.c_float(eps), ctypes.c_int(int(ue8m0)))
    return q, (s.T if colmajor else s)


def silu_mul_quant_1x128(x_bf16_bits: np.ndarray, eps: float = 1e-10, ue8m0: bool = True):
    """x: uint16 [M, 2*N2] -> (uint8 [M,N2], float32 [M, N2/128] with strides (1, M))."""
    x = np.ascontiguousarray(x_bf16_bits, dtype=np.uint16)
    m, n = x.shape
    n2 = n // 2
    g = n2 // 128
    q = np.empty((m, n2), np.uint8)
    s = np.empty((g, m), np.float32)
    lib().kbo_silu_mul_quant_1x128(_p(x), _i64(m), _i64(n2), _i64(n), _p(q), _i64(n2), _p(s), _i64(1), _i64(m),
                                   ctypes.c_float(eps), ctypes.c_int(int(ue8m0)))
    return q, s.T


def silu_bf16_table() -> np.ndarray:
    out = np.empty(65536, np.uint16)
    lib().kbo_silu_bf16_table(_p(out))
    return out


def block_quant_128x128(w_bf16_bits: np.ndarray, eps: float = 1e-10, ue8m0: bool = True):
    w = np.ascontiguousarray(w_bf16_bits, dtype=np.uint16)
    r, c = w.shape
    q = np.empty((r, c), np.uint8)
    s = np.empty(((r + 127) // 128, (c + 127) // 128), np.float32)
    lib().kbo_block_quant_128x128(_p(w), _i64(r), _i64(c), _p(q), _p(s), ctypes.c_float(eps), ctypes.c_int(int(ue8m0)))
    return q, s


def gemm_nt_dequant(a_q: np.ndarray, sa: np.ndarray, w_q: np.ndarray, sw: np.ndarray) -> np.ndarray:
    """Returns uint16 [M,N] bf16 bit patterns."""
    a_q = np.ascontiguousarray(a_q, np.uint8)
    w_q = np.ascontiguousarray(w_q, np.uint8)
    sa = np.ascontiguousarray(sa, np.float32)
    sw = np.ascontiguousarray(sw, np.float32)
    m, k = a_q.shape
    n = w_q.shape[0]
    c = np.empty((m, n), np.uint16)
    lib().kbo_gemm_nt_dequant(_p(a_q), _p(sa), _i64(sa.shape[1]), _i64(1), _p(w_q), _p(sw), _i64(sw.shape[1]), _i64(1),
                              _p(c), _i64(n), _i64(m), _i64(n), _i64(k))
    return c


def grouped_gemm_nt(a_q, sa, b_q, sb, row_expert, c_init: np.ndarray | None = None) -> np.ndarray:
    a_q = np.ascontiguousarray(a_q, np.uint8)
    b_q = np.ascontiguousarray(b_q, np.uint8)
    sa = np.ascontiguousarray(sa, np.float32)
    sb = np.ascontiguousarray(sb, np.float32)
    row_expert = np.ascontiguousarray(row_expert, np.int32)
    m, k = a_q.shape
    n = b_q.shape[1]
    c = np.zeros((m, n), np.uint16) if c_init is None else np.ascontiguousarray(c_init, np.uint16).copy()
    lib().kbo_grouped_gemm_nt(_p(a_q), _p(sa), _i64(sa.shape[1]), _i64(1), _p(b_q), _p(sb), _p(c), _i64(n),
                              _p(row_expert), _i64(m), _i64(n), _i64(k))
    return c
