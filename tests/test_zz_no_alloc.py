"""slc_matmul_run_static, the entry point for hosts that must not allocate device memory while they run (a serving
loop with a fixed memory budget, a framework that owns the allocator): it keeps the quantized activations in a fixed
array inside the library instead of allocated planes. Collected last on purpose: a failure here leaves every other
test already run.

Checked through the C ABI: two calls in a row (the second with different activations, so stale scratch contents would
show) give exactly what the ordinary entry point gives; sizes beyond the scratch are refused with a clear error.
"""
import ctypes as C

import numpy as np
import pytest

from sharplight_b200 import MatMulOp, synth
from sharplight_b200 import native as N

pytestmark = pytest.mark.gpu


def _dev_buffer(lib, device, host: np.ndarray):
    p = C.c_void_p()
    assert lib.slc_buffer_alloc(device.handle, host.nbytes, C.byref(p)) == N.OK
    assert lib.slc_buffer_upload(device.handle, p, host.ctypes.data_as(C.c_void_p), host.nbytes) == N.OK
    return p


@pytest.mark.parametrize("type_name,n,k", [("Q4_K", 200, 4096), ("Q8_0", 96, 1568), ("Q6_K", 64, 1024)])
def test_static_scratch_matches_allocating_entry_point(cuda_device, type_name, n, k):
    lib = N.load()
    blocks = synth.weight_blocks(type_name, n, k, seed=71)
    w = cuda_device.upload_weight(type_name, (n, k), blocks)
    op = MatMulOp(cuda_device, w, 4)
    op.set_kernel(N.KERNEL_MMVQ)          # the dp4a family, which the static entry point always uses
    try:
        for call, rows in enumerate((4, 1)):                      # two calls in a row on the shared scratch
            x = synth.activations(rows, k, seed=80 + call) * np.float32(1 + 3 * call)
            expected = op.run(x)                                  # the existing entry point
            xd = _dev_buffer(lib, cuda_device, x)
            y = np.full((rows, n), np.nan, np.float32)
            yd = _dev_buffer(lib, cuda_device, y)
            rc = lib.slc_matmul_run_static(w.handle, xd, N.F32, rows, k, yd, n, None)
            assert rc == N.OK, lib.slc_static_last_error()
            assert lib.slc_device_sync(cuda_device.handle) == N.OK
            assert lib.slc_buffer_download(cuda_device.handle, y.ctypes.data_as(C.c_void_p), yd, y.nbytes) == N.OK
            lib.slc_buffer_free(cuda_device.handle, xd)
            lib.slc_buffer_free(cuda_device.handle, yd)
            assert np.array_equal(y.view(np.uint32), expected.view(np.uint32))   # same kernels, same bits
        assert cuda_device.last_status() == 0
    finally:
        op.dispose()
        w.dispose()


@pytest.mark.parametrize("n,k,rows", [(48, 28672, 4), (32, 32768, 4), (40, 256, 3), (40, 32, 4)])
def test_static_scratch_long_and_short_k(cuda_device, n, k, rows):
    """Four rows at a K where the kernel's shared memory holds fewer rows per launch (the rows then go in two launches on
    the same scratch), and at a K of one super-tile or less (a one-warp CTA then owns two outputs per thread)."""
    lib = N.load()
    type_name = "Q4_K" if k % 256 == 0 else "Q8_0"
    blocks = synth.weight_blocks(type_name, n, k, seed=k)
    w = cuda_device.upload_weight(type_name, (n, k), blocks)
    op = MatMulOp(cuda_device, w, 4)
    op.set_kernel(N.KERNEL_MMVQ)
    try:
        x = synth.activations(rows, k, seed=91)
        expected = op.run(x)
        xd = _dev_buffer(lib, cuda_device, x)
        y = np.full((rows, n), np.nan, np.float32)
        yd = _dev_buffer(lib, cuda_device, y)
        rc = lib.slc_matmul_run_static(w.handle, xd, N.F32, rows, k, yd, n, None)
        assert rc == N.OK, lib.slc_static_last_error()
        assert lib.slc_device_sync(cuda_device.handle) == N.OK
        assert lib.slc_buffer_download(cuda_device.handle, y.ctypes.data_as(C.c_void_p), yd, y.nbytes) == N.OK
        lib.slc_buffer_free(cuda_device.handle, xd)
        lib.slc_buffer_free(cuda_device.handle, yd)
        assert np.array_equal(y.view(np.uint32), expected.view(np.uint32))
    finally:
        op.dispose()
        w.dispose()


def test_static_scratch_rejects_what_does_not_fit(cuda_device):
    lib = N.load()
    w = cuda_device.upload_weight("Q8_0", (16, 256), synth.weight_blocks("Q8_0", 16, 256, 1))
    big = cuda_device.upload_weight("Q4_0", (16, 32768 + 256), synth.weight_blocks("Q4_0", 16, 32768 + 256, 2))
    x = np.zeros((8, 32768 + 256), np.float32)
    xd = _dev_buffer(lib, cuda_device, x)
    y = np.zeros((8, 16), np.float32)
    yd = _dev_buffer(lib, cuda_device, y)
    try:
        assert lib.slc_matmul_run_static(w.handle, xd, N.F32, 5, 256, yd, 16, None) == N.ERR_UNSUPPORTED
        assert b"4 activation rows" in lib.slc_static_last_error()
        assert lib.slc_matmul_run_static(big.handle, xd, N.F32, 1, 32768 + 256, yd, 16, None) == N.ERR_UNSUPPORTED
        assert b"32768" in lib.slc_static_last_error()
        assert lib.slc_matmul_run_static(w.handle, None, N.F32, 1, 256, yd, 16, None) == N.ERR_INVALID_ARGUMENT
        assert lib.slc_matmul_run_static(w.handle, xd, N.F32, 0, 256, yd, 16, None) == N.OK      # nothing to do
    finally:
        lib.slc_buffer_free(cuda_device.handle, xd)
        lib.slc_buffer_free(cuda_device.handle, yd)
        w.dispose()
        big.dispose()
