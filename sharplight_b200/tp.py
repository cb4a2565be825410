"""Tensor-parallel sharding of quantized weights, one process per GPU.

The reference has no tensor parallelism (its multi-device story is layer placement,
src/Sharplight.Core/Runtime/PlacementPlanner.cs:7-13 of the Sharplight tree); this module is the new functionality the
70B configuration needs. The split is the usual one for a decoder layer:

  column split (over N) for q / k / v / gate / up: rank r keeps rows [r*N/tp, (r+1)*N/tp) of the row-major block array,
  a contiguous byte range;
  row split (over K) for o / down: rank r keeps the K range [r*K/tp, (r+1)*K/tp) of every row, cut on block boundaries
  (32 values for Q8_0 / Q4_0, 256 for Q4_K / Q6_K), so no block is re-quantized and 8-bit activation blocks never straddle a
  shard: every per-block int32 dot is the same integer at every tensor-parallel degree, only the order of the final
  f32 sum changes. The partial outputs of a row-split MatMul are summed by an all-reduce.

Everything here is host logic on numpy arrays of raw ggml blocks; it runs (and is tested) without a GPU.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np

BLOCK = {"Q4_0": (32, 18), "Q8_0": (32, 34), "Q4_K": (256, 144), "Q6_K": (256, 210), "Q5_0": (32, 22), "IQ4_NL": (32, 18),
         "Q5_K": (256, 176)}


def shard_range(total: int, rank: int, tp: int, align: int = 1) -> Tuple[int, int]:
    """[begin, end) of rank's share of `total` items, in units of `align`, remainders to the first ranks."""
    if total % align:
        raise ValueError(f"{total} is not a multiple of {align}")
    units = total // align
    base, extra = divmod(units, tp)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin * align, end * align


def column_shard(blocks: np.ndarray, type_name: str, n: int, k: int, rank: int, tp: int, align: int = 1):
    """Rows [n0, n1) of an [n, k] weight: (blocks, n1 - n0, k). `align`: keep whole heads together (e.g. 128)."""
    bs, bb = BLOCK[type_name]
    row_bytes = k // bs * bb
    n0, n1 = shard_range(n, rank, tp, align)
    flat = np.ascontiguousarray(blocks, np.uint8).reshape(n, row_bytes)
    return flat[n0:n1].reshape(-1), n1 - n0, k


def row_shard(blocks: np.ndarray, type_name: str, n: int, k: int, rank: int, tp: int):
    """The K range [k0, k1) of every row of an [n, k] weight: (blocks, n, k1 - k0, k0)."""
    bs, bb = BLOCK[type_name]
    k0, k1 = shard_range(k, rank, tp, bs)
    flat = np.ascontiguousarray(blocks, np.uint8).reshape(n, k // bs, bb)
    return flat[:, k0 // bs:k1 // bs].reshape(-1), n, k1 - k0, k0


# Llama-3-70B-shaped decoder layer: (name, N, K, split, input). Inputs: x = hidden state (replicated), a = attention
# output (sharded over heads), h = SiLU(gate) * up (sharded over the FFN dimension).
LLAMA70B = {"hidden": 8192, "ffn": 28672, "heads": 64, "kv_heads": 8, "head_dim": 128, "layers": 80}
LLAMA8B = {"hidden": 4096, "ffn": 14336, "heads": 32, "kv_heads": 8, "head_dim": 128, "layers": 32}


def layer_matmuls(arch: dict):
    h, f = arch["hidden"], arch["ffn"]
    kv = arch["kv_heads"] * arch["head_dim"]
    return [("q", h, h, "column", "x_attn"), ("k", kv, h, "column", "x_attn"), ("v", kv, h, "column", "x_attn"),
            ("o", h, h, "row", "x_o"),
            ("gate", f, h, "column", "x_ffn"), ("up", f, h, "column", "x_ffn"),
            ("down", h, f, "row", "x_down")]


def shard_shape(n: int, k: int, split: str, rank: int, tp: int, type_name: str = "Q4_K", head_dim: int = 128):
    """(n_local, k_local) of rank's shard."""
    if split == "column":
        n0, n1 = shard_range(n, rank, tp, head_dim if n % (head_dim * tp) == 0 else 1)
        return n1 - n0, k
    k0, k1 = shard_range(k, rank, tp, BLOCK[type_name][0])
    return n, k1 - k0


def layer_weight_bytes(arch: dict, type_name: str = "Q4_K") -> int:
    bs, bb = BLOCK[type_name]
    return sum(n * (k // bs) * bb for _, n, k, _, _ in layer_matmuls(arch))


# The same layer with the MatMuls that share an input stacked along N, the way a runtime stores them: one MatMul for
# q / k / v and one for gate / up. A stacked weight is column-split part by part (rank r keeps its rows of q, its rows of
# k and its rows of v), so its local rows are exactly the local rows of the separate MatMuls, in the same order.
def fused_layer_matmuls(arch: dict):
    """(name, [N of every stacked part], K, split, input) per MatMul of a layer."""
    h, f = arch["hidden"], arch["ffn"]
    kv = arch["kv_heads"] * arch["head_dim"]
    return [("qkv", [h, kv, kv], h, "column", "x_attn"), ("o", [h], h, "row", "x_o"),
            ("gate_up", [f, f], h, "column", "x_ffn"), ("down", [h], f, "row", "x_down")]


def fused_shard_shape(parts, k: int, split: str, rank: int, tp: int, type_name: str = "Q4_K", head_dim: int = 128):
    """(n_local, k_local) of rank's shard of a stacked weight."""
    shapes = [shard_shape(n, k, split, rank, tp, type_name, head_dim) for n in parts]
    return sum(s[0] for s in shapes), shapes[0][1]


def fused_column_shard(blocks: np.ndarray, type_name: str, parts, k: int, rank: int, tp: int, align: int = 1):
    """Rank's rows of every part of a stacked [sum(parts), k] weight, concatenated: (blocks, n_local, k)."""
    bs, bb = BLOCK[type_name]
    row_bytes = k // bs * bb
    flat = np.ascontiguousarray(blocks, np.uint8).reshape(sum(parts), row_bytes)
    out, base = [], 0
    for n in parts:
        n0, n1 = shard_range(n, rank, tp, align if n % (align * tp) == 0 else 1)
        out.append(flat[base + n0:base + n1])
        base += n
    cat = np.concatenate(out, axis=0)
    return cat.reshape(-1), cat.shape[0], k
