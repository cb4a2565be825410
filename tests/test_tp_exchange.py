"""The in-kernel all-reduce of a row-split MatMul (slc_tp_exchange, slc_matmul_run_quantized_allreduce).

One GPU: a group of one rank runs the whole exchange machinery (stores into its own receive area, arrival words, wait,
sum, counters, slot alternation) and must give the bits of the plain MatMul. Two GPUs (skipped with fewer): two
processes, each with its K range of the weight, sum through each other's memory; the total must match the oracle on
the unsharded weight, the NCCL all-reduce of the plain partial outputs, and be bit-identical on both ranks; and a
peer that never arrives must end in a timeout status, not a hang.
"""
import ctypes as C
import os
import socket

import numpy as np
import pytest

from helpers import FMT_OF, MAX_REL, max_rel_error, sl_oracle
from sharplight_b200 import MatMulOp, NotSupportedError, InvalidOperationError, SharedActivation, TpExchange, synth, tp
from sharplight_b200 import native as N

pytestmark = pytest.mark.gpu


def _dev(lib, device, host: np.ndarray):
    p = C.c_void_p()
    assert lib.slc_buffer_alloc(device.handle, host.nbytes, C.byref(p)) == N.OK
    assert lib.slc_buffer_upload(device.handle, p, host.ctypes.data_as(C.c_void_p), host.nbytes) == N.OK
    return p


def _read(lib, device, p, shape):
    out = np.empty(shape, np.float32)
    assert lib.slc_device_sync(device.handle) == N.OK
    assert lib.slc_buffer_download(device.handle, out.ctypes.data_as(C.c_void_p), p, out.nbytes) == N.OK
    return out


@pytest.mark.parametrize("type_name,n,k", [("Q4_K", 200, 2048), ("Q8_0", 100, 1568), ("Q4_0", 72, 512), ("Q6_K", 64, 1024)])
def test_group_of_one_gives_the_plain_result(cuda_device, type_name, n, k):
    lib = N.load()
    w = cuda_device.upload_weight(type_name, (n, k), synth.weight_blocks(type_name, n, k, seed=31))
    op = MatMulOp(cuda_device, w, 64)
    act = SharedActivation(cuda_device, 64, k)
    ex = TpExchange(cuda_device, 0, 1, 64, n)
    try:
        for call, rows in enumerate((1, 2, 4, 8, 17, 64, 3, 1)):      # both kernel families, both slots, several epochs
            x = synth.activations(rows, k, seed=40 + call)
            xd = _dev(lib, cuda_device, x)
            y0 = _dev(lib, cuda_device, np.full((rows, n), np.nan, np.float32))
            y1 = _dev(lib, cuda_device, np.full((rows, n), np.nan, np.float32))
            act.quantize(xd.value, N.F32, rows, k)
            act.matmul(op, y0.value, n)
            ex.matmul(op, act, y1.value, n)
            plain, summed = _read(lib, cuda_device, y0, (rows, n)), _read(lib, cuda_device, y1, (rows, n))
            if rows <= 2:
                assert np.array_equal(plain.view(np.uint32), summed.view(np.uint32)), (rows, op.last_kernel())
            else:
                # from 3 rows the plain launch may cut K in chunks between CTAs (few weight rows): another order of the
                # same f32 sums
                assert np.max(np.abs(plain - summed)) <= 1e-5 * np.max(np.abs(plain)), (rows, op.last_kernel())
            # the same from rows that have not been quantized yet (slc_matmul_run_allreduce)
            y2 = _dev(lib, cuda_device, np.full((rows, n), np.nan, np.float32))
            ex.run(op, xd.value, N.F32, rows, k, y2.value, n)
            assert np.array_equal(summed.view(np.uint32), _read(lib, cuda_device, y2, (rows, n)).view(np.uint32)), rows
            lib.slc_buffer_free(cuda_device.handle, y2)
            for p in (xd, y0, y1):
                lib.slc_buffer_free(cuda_device.handle, p)
        assert cuda_device.last_status() == 0
    finally:
        ex.dispose(); act.dispose(); op.dispose(); w.dispose()


def test_exchange_limits(cuda_device):
    lib = N.load()
    n, k = 64, 512
    w = cuda_device.upload_weight("Q8_0", (n, k), synth.weight_blocks("Q8_0", n, k, seed=1))
    op = MatMulOp(cuda_device, w, 128)
    act = SharedActivation(cuda_device, 128, k)
    xd = _dev(lib, cuda_device, synth.activations(128, k, seed=2))
    yd = _dev(lib, cuda_device, np.zeros((128, n), np.float32))
    ex = TpExchange(cuda_device, 0, 1, 64, n)
    lonely = TpExchange(cuda_device, 0, 2, 8, n)          # a group of two that nobody connected
    narrow = TpExchange(cuda_device, 0, 1, 64, 32)        # created for fewer output columns
    try:
        act.quantize(xd.value, N.F32, 128, k)
        with pytest.raises(NotSupportedError):
            ex.matmul(op, act, yd.value, n)               # 128 rows: beyond the exchange
        act.quantize(xd.value, N.F32, 4, k)
        with pytest.raises(InvalidOperationError):
            lonely.matmul(op, act, yd.value, n)
        with pytest.raises(ValueError):
            narrow.matmul(op, act, yd.value, n)
        with pytest.raises(ValueError):
            TpExchange(cuda_device, 2, 2, 8, n)           # rank outside the group
        with pytest.raises(ValueError):
            TpExchange(cuda_device, 0, 1, 65, n)          # more rows than an exchange carries
        assert cuda_device.last_status() == 0
    finally:
        for e in (ex, lonely, narrow):
            e.dispose()
        act.dispose(); op.dispose(); w.dispose()
        lib.slc_buffer_free(cuda_device.handle, xd)
        lib.slc_buffer_free(cuda_device.handle, yd)


# ---- two GPUs ----------------------------------------------------------------------------------------------------

def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_gpu_worker(rank, world, port, out):
    import torch
    import torch.distributed as dist
    from sharplight_b200 import CudaExecutionProvider, TpComm
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    provider = CudaExecutionProvider()
    device = provider.open_device([d for d in provider.get_devices() if d.index == rank][0])
    failures = []
    try:
        stream = torch.cuda.Stream()
        torch.cuda.set_stream(stream)
        sp = stream.cuda_stream
        for type_name, n, k in (("Q4_K", 520, 4096), ("Q8_0", 136, 1024), ("Q5_K", 136, 2048), ("Q5_0", 72, 1024)):
            fmt = FMT_OF[type_name]
            blocks = synth.weight_blocks(type_name, n, k, seed=61)
            sb, sn, sk, k0 = tp.row_shard(blocks, type_name, n, k, rank, world)
            w = device.upload_weight(type_name, (sn, sk), sb)
            op = MatMulOp(device, w, 64)
            act = SharedActivation(device, 64, sk)
            ex = TpExchange(device, rank, world, 64, n)
            ex.connect_group(dist)
            dist.barrier()
            for call, rows in enumerate((1, 4, 8, 33, 64, 2)):
                x_full = synth.activations(rows, k, seed=70 + call)
                ref, _, _ = sl_oracle.matmul_intdot(fmt, blocks, n, k, x_full)
                x = torch.from_numpy(np.ascontiguousarray(x_full[:, k0:k0 + sk])).cuda()
                y_part = torch.full((rows, n), float("nan"), device="cuda")
                y_sum = torch.full((rows, n), float("nan"), device="cuda")
                torch.cuda.synchronize()
                act.quantize(x.data_ptr(), N.F32, rows, sk, sp)
                act.matmul(op, y_part.data_ptr(), n, sp)
                ex.matmul(op, act, y_sum.data_ptr(), n, sp)
                stream.synchronize()
                dist.all_reduce(y_part)                           # the collective-library way, for comparison
                mine = y_sum.cpu().numpy()
                if max_rel_error(mine, ref) > MAX_REL:
                    failures.append(f"{type_name} rows={rows}: differs from the oracle by {max_rel_error(mine, ref):.2e}")
                # (the plain launch may sum K in chunks between CTAs, the exchanging one does not: f32 rounding apart)
                if max_rel_error(mine, y_part.cpu().numpy()) > 1e-4:
                    failures.append(f"{type_name} rows={rows}: differs from the NCCL all-reduce")
                both = [torch.empty_like(y_sum) for _ in range(world)]
                dist.all_gather(both, y_sum)
                if not all(torch.equal(both[0], b) for b in both[1:]):
                    failures.append(f"{type_name} rows={rows}: the ranks hold different sums")
            status = device.last_status()
            if status != 0:
                failures.append(f"{type_name}: device status {status}")
            dist.barrier()
            torch.cuda.synchronize()
            if type_name == "Q4_K":
                # the library's own NCCL communicator takes the sums above in_kernel_rows and above the exchange's bound
                comm = TpComm.for_group(device, dist)
                comm.set_chunking(1024)          # two ranks are below the default policy's group size
                ex.set_comm(comm, 16)
                op_big = MatMulOp(device, w, 1280)
                act_big = SharedActivation(device, 1280, sk)
                # (1100 rows: the prefill path, rows in four chunks whose all-reduces run beside the next chunk's GEMM)
                for call, rows in enumerate((8, 17, 64, 200, 1100)):
                    x_full = synth.activations(rows, k, seed=170 + call)
                    ref, _, _ = sl_oracle.matmul_intdot(fmt, blocks, n, k, x_full)
                    x = torch.from_numpy(np.ascontiguousarray(x_full[:, k0:k0 + sk])).cuda()
                    y_sum = torch.full((rows, n + 8), float("nan"), device="cuda")      # a row stride wider than n
                    torch.cuda.synchronize()
                    act_big.quantize(x.data_ptr(), N.F32, rows, sk, sp)
                    ex.matmul(op_big, act_big, y_sum.data_ptr(), n + 8, sp)
                    stream.synchronize()
                    mine = y_sum[:, :n].cpu().numpy()
                    if max_rel_error(mine, ref) > MAX_REL:
                        failures.append(f"comm rows={rows}: differs from the oracle by {max_rel_error(mine, ref):.2e}")
                    if not bool(torch.isnan(y_sum[:, n:]).all()):
                        failures.append(f"comm rows={rows}: wrote beyond n")
                    launches = op_big.last_kernel()[1]
                    if (rows > 16) != (launches >= 2):
                        failures.append(f"comm rows={rows}: {launches} launches (the sum went the wrong way)")
                    both = [torch.empty_like(y_sum) for _ in range(world)]
                    dist.all_gather(both, y_sum.nan_to_num())
                    if not all(torch.equal(both[0], b) for b in both[1:]):
                        failures.append(f"comm rows={rows}: the ranks hold different sums")
                ex.set_comm(None, 16)
                torch.cuda.synchronize()
                dist.barrier()
                act_big.dispose(); op_big.dispose(); comm.dispose()
            if type_name == "Q8_0":
                # A peer that never shows up: rank 1 sits this exchange out (it has nothing in flight), rank 0's
                # kernel gives up after the limit, reports through the status word and leaves the context usable.
                ex.set_wait_ms(200)
                if rank == 0:
                    x = torch.from_numpy(np.ascontiguousarray(synth.activations(1, k, seed=99)[:, k0:k0 + sk])).cuda()
                    y_sum = torch.zeros((1, n), device="cuda")
                    act.quantize(x.data_ptr(), N.F32, 1, sk, sp)
                    ex.matmul(op, act, y_sum.data_ptr(), n, sp)
                    stream.synchronize()
                    status = device.last_status()
                    if status != N.ERR_TIMEOUT:
                        failures.append(f"abandoned exchange: status {status}, expected {N.ERR_TIMEOUT}")
                    act.matmul(op, y_sum.data_ptr(), n, sp)          # the device still works
                    stream.synchronize()
                    if device.last_status() != 0 or not bool(torch.isfinite(y_sum).all()):
                        failures.append("the device did not recover after the abandoned exchange")
                dist.barrier()
                torch.cuda.synchronize()
            ex.dispose(); act.dispose(); op.dispose(); w.dispose()
        out.put((rank, failures))
    except Exception as exc:  # the parent reports it
        out.put((rank, [f"exception: {exc!r}"]))
    finally:
        dist.destroy_process_group()


def test_two_gpus_sum_through_peer_memory():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_two_gpu_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(60)
    for rank, failures in results:
        assert not failures, (rank, failures)
