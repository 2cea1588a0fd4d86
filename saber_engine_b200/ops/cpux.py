"""ctypes front of the host twin (`csrc/cpu/cpux.cpp`): W4A8 GEMM and routed-expert chain on the CPU."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import native as N


def _sig():
    L = N.lib()
    L.saber_cpux_gemm_w4a8.argtypes = [C.c_void_p] * 5 + [C.c_int] * 4
    L.saber_cpux_quant_rows.argtypes = [C.c_void_p] * 3 + [C.c_int] * 2
    L.saber_cpux_expert_chain.argtypes = [C.c_void_p] * 6 + [C.c_int] * 4
    L.saber_cpux_has_avx2.restype = C.c_int
    return L


def pack_nibbles(q: np.ndarray) -> np.ndarray:
    """int8 values in [-8, 7], [N, K] -> uint8 [N, K/2], low nibble = even element."""
    u = (q.astype(np.int16) & 0xF).astype(np.uint8)
    return (u[:, 0::2] | (u[:, 1::2] << 4)).copy()


def gemm_w4a8(a_q: np.ndarray, a_scale: np.ndarray, w_nib: np.ndarray, w_scale: np.ndarray, simd: bool = True):
    L = _sig()
    M, K = a_q.shape
    Nn = w_nib.shape[0]
    out = np.empty((M, Nn), dtype=np.float32)
    a_q, a_scale = np.ascontiguousarray(a_q, np.int8), np.ascontiguousarray(a_scale, np.float32)
    w_nib, w_scale = np.ascontiguousarray(w_nib, np.uint8), np.ascontiguousarray(w_scale, np.float32)
    L.saber_cpux_gemm_w4a8(a_q.ctypes.data, a_scale.ctypes.data, w_nib.ctypes.data, w_scale.ctypes.data,
                           out.ctypes.data, M, Nn, K, int(simd))
    return out


def quant_rows(x: np.ndarray):
    L = _sig()
    x = np.ascontiguousarray(x, np.float32)
    M, K = x.shape
    q, s = np.empty((M, K), np.int8), np.empty(M, np.float32)
    L.saber_cpux_quant_rows(x.ctypes.data, q.ctypes.data, s.ctypes.data, M, K)
    return q, s


def expert_chain(x, w_gu, s_gu, w_down, s_down, simd: bool = True):
    L = _sig()
    x = np.ascontiguousarray(x, np.float32)
    M, H = x.shape
    I = w_down.shape[1] * 2
    out = np.empty((M, H), np.float32)
    args = [np.ascontiguousarray(w_gu, np.uint8), np.ascontiguousarray(s_gu, np.float32),
            np.ascontiguousarray(w_down, np.uint8), np.ascontiguousarray(s_down, np.float32)]
    L.saber_cpux_expert_chain(x.ctypes.data, *[a.ctypes.data for a in args], out.ctypes.data, M, H, I, int(simd))
    return out


def has_avx2() -> bool:
    return bool(_sig().saber_cpux_has_avx2())
