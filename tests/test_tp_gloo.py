"""Tensor-parallel sharding on CPU: two gloo ranks, the oracle as the per-rank MatMul (no GPU).

Column-split shards concatenate to the full output; row-split shards sum (all-reduce) to it; per-block int32 dots of
a row-split shard are the same integers as the matching K range of the unsharded dots.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import FMT_OF, max_rel_error, sl_oracle
from sharplight_b200 import synth, tp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, type_name, n, k, m, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fmt = FMT_OF[type_name]
        blocks = synth.weight_blocks(type_name, n, k, seed=9)
        x = synth.activations(m, k, seed=10)
        full, _, full_s32 = sl_oracle.matmul_intdot(fmt, blocks, n, k, x, want_s32=True)

        # column split: each rank owns a slice of the outputs
        cb, cn, ck = tp.column_shard(blocks, type_name, n, k, rank, world)
        ycol, _, _ = sl_oracle.matmul_intdot(fmt, cb, cn, ck, x)
        n0, n1 = tp.shard_range(n, rank, world)
        assert np.array_equal(ycol, full[:, n0:n1])             # rows are independent: bit-identical
        gathered = [torch.zeros(m, tp.shard_range(n, r, world)[1] - tp.shard_range(n, r, world)[0]) for r in range(world)]
        dist.all_gather(gathered, torch.from_numpy(ycol)) if n % world == 0 else None

        # row split: each rank owns a K range of every row; partial outputs are all-reduced
        rb, rn, rk, k0 = tp.row_shard(blocks, type_name, n, k, rank, world)
        ypart, _, s32 = sl_oracle.matmul_intdot(fmt, rb, rn, rk, x[:, k0:k0 + rk], want_s32=True)
        assert np.array_equal(s32, full_s32[:, :, k0 // 32:(k0 + rk) // 32])   # same integers at every TP degree
        t = torch.from_numpy(ypart.copy())
        dist.all_reduce(t)
        err = max_rel_error(t.numpy(), full)
        if rank == 0:
            ok_gather = True
            if n % world == 0:
                ok_gather = bool(np.array_equal(torch.cat(gathered, dim=1).numpy(), full))
            out.put((err, ok_gather))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("type_name,n,k", [("Q4_K", 64, 1024), ("Q8_0", 48, 1568 - 32), ("Q4_0", 37, 512), ("Q6_K", 32, 768)])
def test_two_rank_sharding(type_name, n, k):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, type_name, n, k, 3, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err, ok_gather = out.get(timeout=10)
    assert err <= 1e-3 and ok_gather


def test_shard_ranges_cover_everything():
    for total, tpn, align in [(8192, 8, 128), (28672, 8, 256), (1024, 8, 128), (14336, 3, 256), (37, 2, 1)]:
        spans = [tp.shard_range(total, r, tpn, align) for r in range(tpn)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all((e - b) % align == 0 for b, e in spans)
    with pytest.raises(ValueError):
        tp.shard_range(100, 0, 2, 32)
    assert tp.layer_weight_bytes(tp.LLAMA70B) * 80 == 38503710720      # the 70B stack of the benchmark configuration
    assert tp.layer_weight_bytes(tp.LLAMA8B) == 122683392
    assert tp.shard_shape(28672, 8192, "column", 3, 8) == (3584, 8192)
    assert tp.shard_shape(8192, 28672, "row", 3, 8) == (8192, 3584)
    assert tp.shard_shape(1024, 8192, "column", 0, 8) == (128, 8192)


def test_stacked_column_split_equals_separate_splits():
    """A stacked q/k/v weight split part by part holds exactly the rows the separate MatMuls would hold."""
    parts, k, world = [64, 16, 16], 512, 2
    blocks = synth.weight_blocks("Q4_K", sum(parts), k, seed=21)
    x = synth.activations(2, k, seed=22)
    fmt = FMT_OF["Q4_K"]
    full, _, _ = sl_oracle.matmul_intdot(fmt, blocks, sum(parts), k, x)
    row_bytes = k // 256 * 144
    flat = blocks.reshape(sum(parts), row_bytes)
    for rank in range(world):
        sb, sn, sk = tp.fused_column_shard(blocks, "Q4_K", parts, k, rank, world, align=8)
        assert (sn, sk) == tp.fused_shard_shape(parts, k, "column", rank, world, "Q4_K", head_dim=8)
        y, _, _ = sl_oracle.matmul_intdot(fmt, sb, sn, sk, x)
        base, cols = 0, []
        for n in parts:
            n0, n1 = tp.shard_range(n, rank, world, 8)
            cols.append(full[:, base + n0:base + n1])
            separate, _, _ = tp.column_shard(flat[base:base + n].reshape(-1), "Q4_K", n, k, rank, world, align=8)
            assert separate.tobytes() in sb.tobytes()
            base += n
        assert np.array_equal(y, np.concatenate(cols, axis=1))
    names = [m[0] for m in tp.fused_layer_matmuls(tp.LLAMA70B)]
    assert names == ["qkv", "o", "gate_up", "down"]
    assert sum(sum(p) * k_ for _, p, k_, _, _ in tp.fused_layer_matmuls(tp.LLAMA70B)) == \
        sum(n * k_ for _, n, k_, _, _ in tp.layer_matmuls(tp.LLAMA70B))
