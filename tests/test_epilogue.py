"""slc_matmul_run_quantized_epilogue: bias and residual added inside the MatMul's launch. The fused store must give the
bits of the plain MatMul followed by the two f32 additions, in every kernel family, also when the residual is y itself
and when the output is summed over a (one-rank) tensor-parallel group."""
import ctypes as C

import numpy as np
import pytest

from sharplight_b200 import MatMulOp, SharedActivation, TpExchange, synth
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


@pytest.mark.parametrize("type_name,n,k,rows", [("Q4_K", 200, 1024, 1), ("Q8_0", 100, 1568, 2), ("Q6_K", 72, 512, 8),
                                                ("Q4_0", 40, 512, 33), ("Q4_0", 300, 512, 130), ("Q4_K", 136, 256, 200)])
def test_fused_additions_equal_separate_additions(cuda_device, type_name, n, k, rows):
    lib = N.load()
    rng = np.random.Generator(np.random.Philox(77))
    w = cuda_device.upload_weight(type_name, (n, k), synth.weight_blocks(type_name, n, k, seed=3))
    op = MatMulOp(cuda_device, w, rows)
    act = SharedActivation(cuda_device, rows, k)
    ex = TpExchange(cuda_device, 0, 1, 64, n)
    x = synth.activations(rows, k, seed=4)
    bias = rng.standard_normal(n).astype(np.float32)
    res = rng.standard_normal((rows, n + 5)).astype(np.float32)           # a residual with its own row stride
    xd, bd, rd = _dev(lib, cuda_device, x), _dev(lib, cuda_device, bias), _dev(lib, cuda_device, res)
    ys = [_dev(lib, cuda_device, np.full((rows, n), np.nan, np.float32)) for _ in range(5)]
    try:
        act.quantize(xd.value, N.F32, rows, k)
        act.matmul(op, ys[0].value, n)
        act.matmul_epilogue(op, ys[1].value, n, bias_ptr=bd.value)
        act.matmul_epilogue(op, ys[2].value, n, bias_ptr=bd.value, residual_ptr=rd.value, residual_stride=n + 5)
        plain = _read(lib, cuda_device, ys[0], (rows, n))
        with_bias = plain + bias[None, :]
        assert np.array_equal(_read(lib, cuda_device, ys[1], (rows, n)).view(np.uint32), with_bias.view(np.uint32))
        both = with_bias + res[:, :n]
        assert np.array_equal(_read(lib, cuda_device, ys[2], (rows, n)).view(np.uint32), both.view(np.uint32))
        # residual in place: y += act . W^T
        start = rng.standard_normal((rows, n)).astype(np.float32)
        assert lib.slc_buffer_upload(cuda_device.handle, ys[3], start.ctypes.data_as(C.c_void_p), start.nbytes) == N.OK
        act.matmul_epilogue(op, ys[3].value, n, residual_ptr=ys[3].value, residual_stride=n)
        assert np.array_equal(_read(lib, cuda_device, ys[3], (rows, n)).view(np.uint32), (plain + start).view(np.uint32))
        if rows <= 64:      # with the sum over a tensor-parallel group (one rank) in front of the additions
            act.matmul_epilogue(op, ys[4].value, n, bias_ptr=bd.value, residual_ptr=rd.value, residual_stride=n + 5, exchange=ex)
            assert np.array_equal(_read(lib, cuda_device, ys[4], (rows, n)).view(np.uint32), both.view(np.uint32))
        assert cuda_device.last_status() == 0
    finally:
        for p in [xd, bd, rd] + ys:
            lib.slc_buffer_free(cuda_device.handle, p)
        ex.dispose(); act.dispose(); op.dispose(); w.dispose()


@pytest.mark.parametrize("type_name,n,k", [("Q4_K", 200, 1024), ("Q8_0", 100, 1568), ("Q6_K", 72, 512), ("Q4_0", 136, 512)])
def test_dual_gate_up(cuda_device, type_name, n, k):
    """slc_matmul_create_dual: y = silu(x . gate^T) * (x . up^T). One dual mat-vec launch up to two rows, the two MatMuls
    and the element-wise tail above; both against the oracle's two MatMuls followed by the same f32 arithmetic."""
    from helpers import FMT_OF, MAX_REL, max_rel_error, sl_oracle
    fmt = FMT_OF[type_name]
    gate_b, up_b = synth.weight_blocks(type_name, n, k, seed=21), synth.weight_blocks(type_name, n, k, seed=22)
    gate, up = cuda_device.upload_weight(type_name, (n, k), gate_b), cuda_device.upload_weight(type_name, (n, k), up_b)
    op = MatMulOp(cuda_device, gate, 100, up=up)
    try:
        for rows, launches in ((1, 2), (2, 2), (8, 4), (100, 4)):
            x = synth.activations(rows, k, seed=30 + rows) * np.float32(3.0)
            y = op.run(x)
            g, _, _ = sl_oracle.matmul_intdot(fmt, gate_b, n, k, x)
            u, _, _ = sl_oracle.matmul_intdot(fmt, up_b, n, k, x)
            with np.errstate(over="ignore"):
                ref = (g / (np.float32(1) + np.exp(-g))).astype(np.float32) * u
            assert y.shape == (rows, n) and max_rel_error(y, ref) <= MAX_REL, (rows, op.last_kernel())
            got = op.last_kernel()[1]                       # quantization included
            assert got == launches if rows <= 2 else got >= launches
        with pytest.raises(Exception):
            op.block_dots(synth.activations(1, k, seed=1))   # no block-dot export for a pair
        other = cuda_device.upload_weight(type_name, (n + 16, k), synth.weight_blocks(type_name, n + 16, k, seed=23))
        with pytest.raises(ValueError):
            MatMulOp(cuda_device, gate, 4, up=other)
        other.dispose()
        assert cuda_device.last_status() == 0
    finally:
        op.dispose(); gate.dispose(); up.dispose()


@pytest.mark.parametrize("rows", [1, 8, 130])
def test_q5_k_epilogue_counts_bias_and_residual_once(cuda_device, rows):
    """A Q5_K weight is two Q4_K weights on the device, the second product added onto the first: bias and residual belong
    to the first pass only. (The order of the f32 additions differs from plain + bias + residual, hence a tolerance.)"""
    lib = N.load()
    n, k = 136, 512
    rng = np.random.Generator(np.random.Philox(78))
    w = cuda_device.upload_weight("Q5_K", (n, k), synth.weight_blocks("Q5_K", n, k, seed=5))
    op = MatMulOp(cuda_device, w, rows)
    act = SharedActivation(cuda_device, rows, k)
    ex = TpExchange(cuda_device, 0, 1, 64, n)
    x = synth.activations(rows, k, seed=6)
    bias = rng.standard_normal(n).astype(np.float32)
    res = rng.standard_normal((rows, n + 5)).astype(np.float32)
    xd, bd, rd = _dev(lib, cuda_device, x), _dev(lib, cuda_device, bias), _dev(lib, cuda_device, res)
    ys = [_dev(lib, cuda_device, np.full((rows, n), np.nan, np.float32)) for _ in range(3)]
    try:
        act.quantize(xd.value, N.F32, rows, k)
        act.matmul(op, ys[0].value, n)
        act.matmul_epilogue(op, ys[1].value, n, bias_ptr=bd.value, residual_ptr=rd.value, residual_stride=n + 5)
        plain = _read(lib, cuda_device, ys[0], (rows, n))
        want = plain + bias[None, :] + res[:, :n]
        got = _read(lib, cuda_device, ys[1], (rows, n))
        assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(1.0, np.abs(want)))
        if rows <= 64:
            act.matmul_epilogue(op, ys[2].value, n, bias_ptr=bd.value, residual_ptr=rd.value, residual_stride=n + 5, exchange=ex)
            got = _read(lib, cuda_device, ys[2], (rows, n))
            assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(1.0, np.abs(want)))
        assert cuda_device.last_status() == 0
    finally:
        for p in [xd, bd, rd] + ys:
            lib.slc_buffer_free(cuda_device.handle, p)
        ex.dispose(); act.dispose(); op.dispose(); w.dispose()
