"""Seeded synthetic weights and activations with the shapes and value distributions of the benchmark configurations.

No model file or dataset is involved: raw ggml blocks are generated directly (block layouts:
src/Sharplight.Core/Tensors/DataType.cs:102,110,116,120 of the Sharplight tree) from a counter-based generator.
"""
from __future__ import annotations

import numpy as np

BLOCK = {"Q4_0": (32, 18), "Q8_0": (32, 34), "Q4_K": (256, 144), "Q6_K": (256, 210), "Q5_0": (32, 22), "IQ4_NL": (32, 18),
         "Q5_K": (256, 176)}


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def _f16_bytes(values: np.ndarray) -> np.ndarray:
    return values.astype(np.float16).view(np.uint8).reshape(values.shape + (2,))


def weight_blocks(type_name: str, n: int, k: int, seed: int, scale_sigma: float | None = None) -> np.ndarray:
    """Raw blocks of an [n, k] weight as a flat uint8 array.

    Q8_0: codes uniform in [-127, 127], d = |N(0, 0.02)| / 127.   Q4_0: nibbles uniform, d = |N(0, 0.02)| / 8.
    Q4_K: 6-bit scales / mins uniform (12 uniform bytes), d, dmin = |N(0, 0.01)|, nibbles uniform.
    Q6_K: ql / qh uniform bits, int8 sub-block scales uniform, d = |N(0, 0.01)|.
    Q5_K: like Q4_K plus 32 uniform bytes of fifth bits.
    Q5_0: nibbles and the 32 high bits uniform, d = |N(0, 0.02)| / 16.   IQ4_NL: nibbles uniform, d = |N(0, 0.02)| / 127.
    """
    bs, bb = BLOCK[type_name]
    assert k % bs == 0
    nb = n * (k // bs)
    g = _rng(seed)
    out = np.empty((nb, bb), np.uint8)
    if type_name == "Q8_0":
        sigma = 0.02 if scale_sigma is None else scale_sigma
        out[:, 0:2] = _f16_bytes(np.abs(g.normal(0.0, sigma, nb)) / 127.0)
        out[:, 2:34] = g.integers(-127, 128, (nb, 32), dtype=np.int8).view(np.uint8)
    elif type_name == "Q4_0":
        sigma = 0.02 if scale_sigma is None else scale_sigma
        out[:, 0:2] = _f16_bytes(np.abs(g.normal(0.0, sigma, nb)) / 8.0)
        out[:, 2:18] = g.integers(0, 256, (nb, 16), dtype=np.uint8)
    elif type_name == "Q5_0":
        sigma = 0.02 if scale_sigma is None else scale_sigma
        out[:, 0:2] = _f16_bytes(np.abs(g.normal(0.0, sigma, nb)) / 16.0)
        out[:, 2:22] = g.integers(0, 256, (nb, 20), dtype=np.uint8)
    elif type_name == "IQ4_NL":
        sigma = 0.02 if scale_sigma is None else scale_sigma
        out[:, 0:2] = _f16_bytes(np.abs(g.normal(0.0, sigma, nb)) / 127.0)
        out[:, 2:18] = g.integers(0, 256, (nb, 16), dtype=np.uint8)
    elif type_name == "Q4_K":
        sigma = 0.01 if scale_sigma is None else scale_sigma
        out[:, 0:2] = _f16_bytes(np.abs(g.normal(0.0, sigma, nb)))
        out[:, 2:4] = _f16_bytes(np.abs(g.normal(0.0, sigma, nb)))
        out[:, 4:144] = g.integers(0, 256, (nb, 140), dtype=np.uint8)
    elif type_name == "Q5_K":
        sigma = 0.01 if scale_sigma is None else scale_sigma
        out[:, 0:2] = _f16_bytes(np.abs(g.normal(0.0, sigma, nb)))
        out[:, 2:4] = _f16_bytes(np.abs(g.normal(0.0, sigma, nb)))
        out[:, 4:176] = g.integers(0, 256, (nb, 172), dtype=np.uint8)
    elif type_name == "Q6_K":
        sigma = 0.01 if scale_sigma is None else scale_sigma
        out[:, 0:208] = g.integers(0, 256, (nb, 208), dtype=np.uint8)
        out[:, 208:210] = _f16_bytes(np.abs(g.normal(0.0, sigma, nb)))
    else:
        raise ValueError(type_name)
    return out.reshape(-1)


def activations(m: int, k: int, seed: int) -> np.ndarray:
    """f32 [m, k] ~ N(0, 1)."""
    return _rng(seed).standard_normal((m, k), dtype=np.float32)


def exact_int8_activations(m: int, k: int, seed: int) -> np.ndarray:
    """Activations the 8-bit quantizer represents exactly (the idea of Rnd.ExactInt8,
    tests/Sharplight.Vulkan.Tests/Rnd.cs:24-36): integers in [-127, 127] times a power of two per block, with one
    +-127 in every block so the block scale is that power of two."""
    g = _rng(seed)
    q = g.integers(-127, 128, (m, k // 32, 32)).astype(np.float32)
    q[:, :, 0] = np.where(g.integers(0, 2, (m, k // 32)) == 0, -127.0, 127.0)
    e = -(4 + (np.arange(k // 32) % 5)).astype(np.float32)
    return (q * np.exp2(e)[None, :, None]).reshape(m, k).astype(np.float32)


def weight_bytes(type_name: str, n: int, k: int) -> int:
    bs, bb = BLOCK[type_name]
    return n * (k // bs) * bb
