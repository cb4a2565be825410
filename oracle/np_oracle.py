"""Vectorised numpy restatement of the same arithmetic as oracle/sl_oracle.c. TEST INFRASTRUCTURE ONLY.

A second, independently written statement of the reference's rules (paths relative to the Sharplight tree):
src/Sharplight.Cpu/Quant.cs:371-405,504-545,585-618 (decode), src/Sharplight.Cpu/IntDot.cs:92-126 (activation
quantization), src/Sharplight.Cpu/IntDot.Decode.cs:70-99,125-148,189-223 (unsigned codes). The tests hold the two
restatements against each other and against the ggml golden fixtures.
"""
from __future__ import annotations

import numpy as np

Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL = 2, 6, 8, 12, 13, 14, 20
BLOCK = {Q4_0: (32, 18), Q5_0: (32, 22), Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210), IQ4_NL: (32, 18)}
# IQ4_NL's non-linear codebook (src/Sharplight.Cpu/Quant.cs:409)
IQ4NL_VALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.int32)


def _f16(b: np.ndarray) -> np.ndarray:
    """Two little-endian bytes (last axis of size 2) -> f32."""
    return np.ascontiguousarray(b).view("<f2")[..., 0].astype(np.float32)


def _fma(a, b, c):
    """fma in f32 for small-integer a: the product and sum are exact in double, one final rounding."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


def scale_min(s: np.ndarray):
    """12 scale bytes [..., 12] -> (sc [..., 8], m [..., 8]) 6-bit values."""
    s = s.astype(np.int32)
    sc = np.empty(s.shape[:-1] + (8,), np.int32)
    m = np.empty_like(sc)
    sc[..., :4] = s[..., 0:4] & 63
    m[..., :4] = s[..., 4:8] & 63
    sc[..., 4:] = (s[..., 8:12] & 15) | ((s[..., 0:4] >> 6) << 4)
    m[..., 4:] = (s[..., 8:12] >> 4) | ((s[..., 4:8] >> 6) << 4)
    return sc, m


def codes(fmt: int, blocks: np.ndarray, n: int, k: int):
    """Raw blocks -> (u int32 [n, k] unsigned codes, a f32 [n, k/16], b f32 [n, k/16])."""
    bs, bb = BLOCK[fmt]
    nb = k // bs
    blk = np.ascontiguousarray(blocks, np.uint8).reshape(n, nb, bb)
    if fmt == Q8_0:
        d = _f16(blk[..., 0:2])
        u = (blk[..., 2:34] ^ 0x80).astype(np.int32).reshape(n, k)
        a = np.repeat(d, 2, axis=1)
        b = np.float32(-128.0) * a
    elif fmt == Q4_0:
        d = _f16(blk[..., 0:2])
        qs = blk[..., 2:18].astype(np.int32)
        u = np.concatenate([qs & 15, qs >> 4], axis=-1).reshape(n, k)
        a = np.repeat(d, 2, axis=1)
        b = np.float32(-8.0) * a
    elif fmt == Q5_0:
        # { f16 d; u32 qh; u8 qs[16] }: bit j of qh is the fifth bit of value j (IntDot.Decode.cs:101-123)
        d = _f16(blk[..., 0:2])
        qh = np.ascontiguousarray(blk[..., 2:6]).view("<u4")[..., 0].astype(np.int64)
        hi = ((qh[..., None] >> np.arange(32)) & 1).astype(np.int32) << 4
        qs = blk[..., 6:22].astype(np.int32)
        u = (np.concatenate([qs & 15, qs >> 4], axis=-1) | hi).reshape(n, k)
        a = np.repeat(d, 2, axis=1)
        b = np.float32(-16.0) * a
    elif fmt == IQ4_NL:
        # { f16 d; u8 qs[16] }: u = codebook value + 128 (IntDot.Decode.cs:225-238)
        d = _f16(blk[..., 0:2])
        qs = blk[..., 2:18].astype(np.int32)
        u = (IQ4NL_VALUES[np.concatenate([qs & 15, qs >> 4], axis=-1)] + 128).reshape(n, k)
        a = np.repeat(d, 2, axis=1)
        b = np.float32(-128.0) * a
    elif fmt == Q4_K:
        d = _f16(blk[..., 0:2])
        dmin = _f16(blk[..., 2:4])
        sc, m = scale_min(blk[..., 4:16])
        qs = blk[..., 16:144].astype(np.int32).reshape(n, nb, 4, 32)
        u = np.concatenate([qs & 15, qs >> 4], axis=-1).reshape(n, k)
        a8 = d[..., None] * sc.astype(np.float32)
        b8 = -dmin[..., None] * m.astype(np.float32)
        a = np.repeat(a8.reshape(n, nb * 8), 2, axis=1)
        b = np.repeat(b8.reshape(n, nb * 8), 2, axis=1)
    elif fmt == Q5_K:
        # Q4_K plus a fifth bit: bit 2j / 2j + 1 of qh[l] for value l of the low- / high-nibble sub-block of chunk j
        d = _f16(blk[..., 0:2])
        dmin = _f16(blk[..., 2:4])
        sc, m = scale_min(blk[..., 4:16])
        qh = blk[..., 16:48].astype(np.int32)[:, :, None, :]                       # [n, nb, 1, 32]
        qs = blk[..., 48:176].astype(np.int32).reshape(n, nb, 4, 32)
        sh = (2 * np.arange(4))[None, None, :, None]
        lo = (qs & 15) | (((qh >> sh) & 1) << 4)
        hi = (qs >> 4) | (((qh >> (sh + 1)) & 1) << 4)
        u = np.concatenate([lo, hi], axis=-1).reshape(n, k)
        a8 = d[..., None] * sc.astype(np.float32)
        b8 = -dmin[..., None] * m.astype(np.float32)
        a = np.repeat(a8.reshape(n, nb * 8), 2, axis=1)
        b = np.repeat(b8.reshape(n, nb * 8), 2, axis=1)
    elif fmt == Q6_K:
        ql = blk[..., 0:128].astype(np.int32).reshape(n, nb, 2, 64)
        qh = blk[..., 128:192].astype(np.int32).reshape(n, nb, 2, 32)
        sc = blk[..., 192:208].view(np.int8).astype(np.float32)
        d = _f16(blk[..., 208:210])
        la, lb = ql[..., :32], ql[..., 32:]
        v1 = (la & 15) | ((qh & 3) << 4)
        v2 = (lb & 15) | (((qh >> 2) & 3) << 4)
        v3 = (la >> 4) | (((qh >> 4) & 3) << 4)
        v4 = (lb >> 4) | (((qh >> 6) & 3) << 4)
        u = np.concatenate([v1, v2, v3, v4], axis=-1).reshape(n, k)
        a = (d[..., None] * sc).reshape(n, nb * 16).astype(np.float32)
        b = np.float32(-32.0) * a
    else:
        raise ValueError(fmt)
    return u, a.astype(np.float32), b.astype(np.float32)


def dequantize(fmt: int, blocks: np.ndarray, n: int, k: int) -> np.ndarray:
    """w = fma(code, a, b) per value with the reference's signed code for Q8_0 (offset 0)."""
    u, a, b = codes(fmt, blocks, n, k)
    a16 = np.repeat(a, 16, axis=1)
    if fmt == Q8_0 or fmt == IQ4_NL:   # a plain product of the signed code and d
        return _fma((u - 128).astype(np.float32), a16, np.zeros_like(a16))
    return _fma(u.astype(np.float32), a16, np.repeat(b, 16, axis=1))


def quantize(x: np.ndarray):
    """f32 [m, k] -> (q int8, d [m, k/32], gs [m, k/16]) by the scalar rule, all in f32 arithmetic."""
    x = np.ascontiguousarray(x, np.float32)
    m, k = x.shape
    xb = x.reshape(m, k // 32, 32)
    amax = np.abs(xb).max(axis=-1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    v = (xb * inv[..., None]).astype(np.float32)
    r = np.trunc((v + np.copysign(np.float32(0.5), v)).astype(np.float32)).astype(np.int32)
    q = r.astype(np.int8).reshape(m, k)
    s16 = r.reshape(m, k // 16, 16).sum(axis=-1)
    gs = (np.repeat(d, 2, axis=1) * s16.astype(np.float32)).astype(np.float32)
    return q, d, gs


def block_dots(u: np.ndarray, q: np.ndarray) -> np.ndarray:
    """u int [n, k], q int8 [m, k] -> int32 [m, n, k/32] exact dots per 32-value block."""
    n, k = u.shape
    m = q.shape[0]
    ub = u.astype(np.int64).reshape(n, k // 32, 32)
    qb = q.astype(np.int64).reshape(m, k // 32, 32)
    return np.einsum("nbi,mbi->mnb", ub, qb).astype(np.int32)


def matmul_intdot_f64(fmt: int, blocks: np.ndarray, n: int, k: int, x: np.ndarray) -> np.ndarray:
    """Sum of the integer-dot terms a*d*s + b*(d*sum q) per 16 values, in double."""
    u, a, b = codes(fmt, blocks, n, k)
    q, d, _ = quantize(x)
    m = q.shape[0]
    ug = u.astype(np.int64).reshape(n, k // 16, 16)
    qg = q.astype(np.int64).reshape(m, k // 16, 16)
    s = np.einsum("ngi,mgi->mng", ug, qg).astype(np.float64)
    sq = qg.sum(axis=-1).astype(np.float64)
    d16 = np.repeat(d, 2, axis=1).astype(np.float64)
    return (s * a.astype(np.float64)[None] * d16[:, None, :]).sum(-1) + \
        (b.astype(np.float64)[None] * (d16 * sq)[:, None, :]).sum(-1)


# ---- the operations on either side of the MatMul that the CUDA path fuses with the activation quantization ---------------

def rms_norm(x: np.ndarray, weight, eps: float) -> np.ndarray:
    """RmsNorm as the reference's CPU row op computes it (src/Sharplight.Cpu/RowOp.cs:63-76, Simd.cs:464-483):
    scale = 1 / sqrt(sum(x^2) / n + eps); y = (x * scale) * w, every step in f32. The reference's sum of squares runs
    in an ISA-dependent order (Simd.cs:274-310); here it is accumulated in f64 and rounded once, which every such order
    matches to a few ulp."""
    x = np.asarray(x, np.float32)
    n = x.shape[-1]
    sumsq = np.sum(x.astype(np.float64) ** 2, axis=-1, keepdims=True).astype(np.float32)
    scale = (np.float32(1.0) / np.sqrt(sumsq / np.float32(n) + np.float32(eps))).astype(np.float32)
    y = (x * scale).astype(np.float32)
    if weight is not None:
        y = (y * np.asarray(weight, np.float32)).astype(np.float32)
    return y


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """silu(gate) * up with silu(v) = v / (1 + exp(-v)) (src/Sharplight.Cpu/ScalarMath.cs:552-577), in f32."""
    g = np.asarray(gate, np.float32)
    with np.errstate(over="ignore"):
        s = (g / (np.float32(1.0) + np.exp(-g).astype(np.float32))).astype(np.float32)
    return (s * np.asarray(up, np.float32)).astype(np.float32)


def argmax_first(y: np.ndarray) -> np.ndarray:
    """Index of the first maximum per row as the reference's sequential scan finds it (src/Sharplight.Cpu/RowOp.cs:174-189):
    best = 0; x[i] > x[best] replaces it -- so NaN never beats a number, and a row that starts with NaN answers 0."""
    y = np.asarray(y, np.float32)
    out = np.zeros(y.shape[0], np.int32)
    for r in range(y.shape[0]):
        row = y[r]
        if row.size == 0 or np.isnan(row[0]):
            continue
        masked = np.where(np.isnan(row), -np.inf, row)
        out[r] = int(np.argmax(masked))      # numpy's argmax is the first maximum too
    return out
