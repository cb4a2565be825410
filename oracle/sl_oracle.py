"""ctypes binding of the CPU oracle (oracle/sl_oracle.c). TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this module; the product
package never does. The library is built by ``make -C oracle`` (or :func:`build`).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsl_oracle.so")

Q4_0, Q8_0, Q4_K, Q6_K = 2, 8, 12, 14
FORMATS = {"q4_0": Q4_0, "q8_0": Q8_0, "q4_k": Q4_K, "q6_k": Q6_K}

_lib = None


def build(force: bool = False) -> str:
    """Compiles the oracle with gcc when the shared library is missing or older than its source."""
    src = os.path.join(HERE, "sl_oracle.c")
    hdr = os.path.join(HERE, "sl_oracle.h")
    stale = (not os.path.exists(LIB_PATH)) or any(
        os.path.getmtime(p) > os.path.getmtime(LIB_PATH) for p in (src, hdr))
    if force or stale:
        subprocess.check_call(["make", "-C", HERE, "-B", "libsl_oracle.so"], stdout=subprocess.DEVNULL)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = C.CDLL(LIB_PATH)
        vp, i64, i32 = C.c_void_p, C.c_int64, C.c_int
        L.slo_block_size.argtypes = [i32]
        L.slo_block_bytes.argtypes = [i32]
        L.slo_h2f.argtypes = [C.c_uint16]
        L.slo_h2f.restype = C.c_float
        L.slo_dequantize_row.argtypes = [i32, vp, i64, vp]
        L.slo_quantize_row.argtypes = [vp, i64, vp, vp, vp]
        L.slo_quantize_row.restype = None
        L.slo_decode_row.argtypes = [i32, vp, i64, vp, vp, vp]
        L.slo_dot_scalar.argtypes = [vp, vp, vp, vp, vp, vp, i64]
        L.slo_dot_scalar.restype = C.c_float
        L.slo_block_dots.argtypes = [vp, vp, i64, vp]
        L.slo_block_dots.restype = None
        L.slo_matmul_intdot.argtypes = [i32, vp, i64, i64, vp, i64, vp, vp, vp, i32, i32]
        L.slo_matmul_f64.argtypes = [i32, vp, i64, i64, vp, i64, vp, i32]
        L.slo_fast_tier_name.restype = C.c_char_p
        L.slo_matmul_intdot_pooled.argtypes = [i32, vp, i64, i64, vp, i64, vp, i32, i32]
        L.slo_matmul_gemm.argtypes = [i32, vp, i64, i64, vp, i64, vp, i32]
        L.slo_matmul_run.argtypes = [i32, vp, i64, i64, vp, i64, vp, i32]
        L.slo_gemm_tile_name.restype = C.c_char_p
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def block_size(fmt: int) -> int:
    return lib().slo_block_size(fmt)


def block_bytes(fmt: int) -> int:
    return lib().slo_block_bytes(fmt)


def row_bytes(fmt: int, k: int) -> int:
    return k // block_size(fmt) * block_bytes(fmt)


def dequantize(fmt: int, blocks: np.ndarray, n: int, k: int) -> np.ndarray:
    """Raw ggml blocks of an [n, k] weight -> f32 [n, k]."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    rb = row_bytes(fmt, k)
    assert blocks.size == n * rb
    out = np.empty((n, k), np.float32)
    for r in range(n):
        rc = lib().slo_dequantize_row(fmt, blocks.ctypes.data + r * rb, k, out[r].ctypes.data)
        assert rc == 0
    return out


def quantize(x: np.ndarray):
    """f32 [m, k] -> (q int8 [m, k], d f32 [m, k/32], gs f32 [m, k/16])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    assert k % 32 == 0
    q = np.empty((m, k), np.int8)
    d = np.empty((m, k // 32), np.float32)
    gs = np.empty((m, k // 16), np.float32)
    for t in range(m):
        lib().slo_quantize_row(x[t].ctypes.data, k, q[t].ctypes.data, d[t].ctypes.data, gs[t].ctypes.data)
    return q, d, gs


def decode(fmt: int, blocks: np.ndarray, n: int, k: int):
    """Raw blocks -> (u uint8 [n, k], a f32 [n, k/16], b f32 [n, k/16])."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    rb = row_bytes(fmt, k)
    assert blocks.size == n * rb
    u = np.empty((n, k), np.uint8)
    a = np.empty((n, k // 16), np.float32)
    b = np.empty((n, k // 16), np.float32)
    for r in range(n):
        rc = lib().slo_decode_row(fmt, blocks.ctypes.data + r * rb, k, u[r].ctypes.data, a[r].ctypes.data,
                                  b[r].ctypes.data)
        assert rc == 0
    return u, a, b


def matmul_intdot(fmt: int, blocks: np.ndarray, n: int, k: int, x: np.ndarray, *, threads: int = 1,
                  tier: int = 0, want_f64: bool = False, want_s32: bool = False):
    """The integer-dot MatMul. Returns (y f32 [m, n], y64 or None, s32 [m, n, k/32] or None)."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32)
    m = x.shape[0]
    assert x.shape[1] == k and blocks.size == n * row_bytes(fmt, k)
    y = np.zeros((m, n), np.float32)
    y64 = np.zeros((m, n), np.float64) if want_f64 else None
    s32 = np.zeros((m, n, k // 32), np.int32) if want_s32 else None
    rc = lib().slo_matmul_intdot(fmt, _p(blocks), n, k, _p(x), m, _p(y), _p(y64), _p(s32), threads, tier)
    assert rc == 0
    return y, y64, s32


def matmul_f64(fmt: int, blocks: np.ndarray, n: int, k: int, x: np.ndarray, *, threads: int = 1) -> np.ndarray:
    """Dequantized weight times unquantized activations, in double."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32)
    m = x.shape[0]
    y64 = np.zeros((m, n), np.float64)
    rc = lib().slo_matmul_f64(fmt, _p(blocks), n, k, _p(x), m, _p(y64), threads)
    assert rc == 0
    return y64


def matmul_intdot_pooled(fmt: int, blocks: np.ndarray, n: int, k: int, x: np.ndarray, *, threads: int = 1,
                         tier: int = 1) -> np.ndarray:
    """The integer-dot MatMul with the reference's chunking on its spinning worker pool (MatMulOp.cs:174-213)."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32)
    m = x.shape[0]
    assert x.shape[1] == k and blocks.size == n * row_bytes(fmt, k)
    y = np.zeros((m, n), np.float32)
    assert lib().slo_matmul_intdot_pooled(fmt, _p(blocks), n, k, _p(x), m, _p(y), threads, tier) == 0
    return y


def matmul_gemm(fmt: int, blocks: np.ndarray, n: int, k: int, x: np.ndarray, *, threads: int = 1) -> np.ndarray:
    """The f32 GEMM path the reference's CPU provider takes from 32 rows (MatMulOp.cs:218-369, Gemm.cs:210-330)."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32)
    m = x.shape[0]
    assert x.shape[1] == k and blocks.size == n * row_bytes(fmt, k)
    y = np.zeros((m, n), np.float32)
    assert lib().slo_matmul_gemm(fmt, _p(blocks), n, k, _p(x), m, _p(y), threads) == 0
    return y


def matmul_run(fmt: int, blocks: np.ndarray, n: int, k: int, x: np.ndarray, *, threads: int = 1) -> np.ndarray:
    """MatMulOp.Run's dispatch (MatMulOp.cs:125-160): the f32 GEMM from 32 rows, integer dots below."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32)
    m = x.shape[0]
    y = np.zeros((m, n), np.float32)
    assert lib().slo_matmul_run(fmt, _p(blocks), n, k, _p(x), m, _p(y), threads) == 0
    return y


def gemm_tile_name() -> str:
    return lib().slo_gemm_tile_name().decode()


def fast_tier_name() -> str:
    return lib().slo_fast_tier_name().decode()
