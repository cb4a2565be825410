"""The kernels that produce the MatMul's 8-bit activations in the same pass as the operation in front of it (RmsNorm,
silu(gate) * up), and the arg-max behind the lm_head. Parity chain: the f32 values against the oracle's restatement of
the reference's row ops (tolerance: the reference's own sum order depends on the ISA); the quantized planes bit for bit
against the plain quantizer applied to those same f32 values (the plain quantizer is checked bit for bit against the
oracle's elsewhere); the MatMul result from the fused planes against the oracle's MatMul of the oracle's norm."""
import numpy as np
import pytest

from helpers import FMT_OF, np_oracle, relative_rms, sl_oracle
from sharplight_b200 import MatMulOp, SharedActivation, synth
from sharplight_b200 import native as N


def test_oracle_row_ops_known_answers():
    x = np.array([[3.0, -4.0, 0.0, 0.0]], np.float32)
    y = np_oracle.rms_norm(x, np.array([1, 2, 1, 1], np.float32), 0.0)
    assert np.allclose(y, [[3 / 2.5, -8 / 2.5, 0, 0]], rtol=1e-6)          # rms = sqrt(25 / 4) = 2.5
    assert np.allclose(np_oracle.silu_mul(np.array([0.0, 1.0, -1.0]), np.array([2.0, 2.0, 2.0])),
                       [0.0, 2 / (1 + np.exp(-1.0)), -2 / (1 + np.exp(1.0))], rtol=1e-6)
    rows = np.array([[1, 5, 5, 2], [np.nan, 9, 1, 1], [1, np.nan, 3, 3], [-np.inf, -np.inf, -np.inf, -np.inf]], np.float32)
    assert np_oracle.argmax_first(rows).tolist() == [1, 0, 2, 0]


# The chain checks compare results whose 8-bit codes come from f32 values that differ in the last bits (the norm's sum
# order): a value on a rounding boundary may take the neighbouring code, which moves single outputs by more than the
# MatMul's own tolerance. They are therefore held to the reference's measure for quantized MatMuls, relative RMS
# (tests/Sharplight.Cpu.Tests/QuantTests.cs: MatMulWithIntDotMatchesReference), at a tenth of its bound (one flipped code among 4096 values moves a row by about 4e-4 of its magnitude).
CHAIN_RMS = 1e-3


def _torch():
    import torch
    return torch


@pytest.mark.gpu
@pytest.mark.parametrize("rows,k,dtype", [(1, 4096, "f32"), (5, 1568, "f32"), (33, 8192, "f32"), (8, 4096, "bf16"), (70, 256, "f32")])
def test_rmsnorm_quantize(cuda_device, rows, k, dtype):
    torch = _torch()
    n = 96
    x = synth.activations(rows, k, seed=rows + k)
    w = (1.0 + 0.1 * np.random.Generator(np.random.Philox(k)).standard_normal(k)).astype(np.float32)
    eps = 1e-5
    if dtype == "bf16":
        xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
        x = xt.float().cpu().numpy()
    else:
        xt = torch.from_numpy(x).cuda()
    wt = torch.from_numpy(w).cuda()
    blocks = synth.weight_blocks("Q4_K" if k % 256 == 0 else "Q8_0", n, k, seed=7)
    type_name = "Q4_K" if k % 256 == 0 else "Q8_0"
    weight = cuda_device.upload_weight(type_name, (n, k), blocks)
    op = MatMulOp(cuda_device, weight, rows)
    fused, plain = SharedActivation(cuda_device, rows, k), SharedActivation(cuda_device, rows, k)
    try:
        y_norm = torch.full((rows, k), float("nan"), device="cuda")
        fused.quantize_rmsnorm(xt.data_ptr(), N.BF16 if dtype == "bf16" else N.F32, rows, k, wt.data_ptr(), eps, y_norm.data_ptr(), k)
        ya = torch.empty((rows, n), device="cuda")
        fused.matmul(op, ya.data_ptr(), n)
        # 1. the f32 values against the oracle's norm
        ref_norm = np_oracle.rms_norm(x, w, eps)
        got_norm = y_norm.cpu().numpy()
        assert np.max(np.abs(got_norm - ref_norm)) <= 4e-6 * np.max(np.abs(ref_norm))
        # 2. the planes bit for bit: the plain quantizer on the kernel's own f32 values gives the same MatMul result
        plain.quantize(y_norm.data_ptr(), N.F32, rows, k)
        yb = torch.empty((rows, n), device="cuda")
        plain.matmul(op, yb.data_ptr(), n)
        torch.cuda.synchronize()
        assert torch.equal(ya, yb)
        # 3. the whole chain against the oracle (its MatMul of its norm)
        ref, _, _ = sl_oracle.matmul_intdot(FMT_OF[type_name], blocks, n, k, ref_norm, threads=4)
        assert relative_rms(ya.cpu().numpy(), ref) <= CHAIN_RMS
        # without the f32 output and without a weight vector
        fused.quantize_rmsnorm(xt.data_ptr(), N.BF16 if dtype == "bf16" else N.F32, rows, k, 0, eps)
        fused.matmul(op, ya.data_ptr(), n)
        ref, _, _ = sl_oracle.matmul_intdot(FMT_OF[type_name], blocks, n, k, np_oracle.rms_norm(x, None, eps), threads=4)
        torch.cuda.synchronize()
        assert relative_rms(ya.cpu().numpy(), ref) <= CHAIN_RMS
        assert cuda_device.last_status() == 0
    finally:
        fused.dispose(); plain.dispose(); op.dispose(); weight.dispose()


@pytest.mark.gpu
@pytest.mark.parametrize("rows,k", [(1, 14336), (4, 3584), (33, 1024), (64, 28672)])
def test_silu_mul_quantize(cuda_device, rows, k):
    torch = _torch()
    n = 80
    gu = synth.activations(rows, 2 * k, seed=3 * rows + k) * 3.0       # gate and up as the halves of one stacked output
    gut = torch.from_numpy(gu).cuda()
    blocks = synth.weight_blocks("Q4_K", n, k, seed=11)
    weight = cuda_device.upload_weight("Q4_K", (n, k), blocks)
    op = MatMulOp(cuda_device, weight, rows)
    fused, plain = SharedActivation(cuda_device, rows, k), SharedActivation(cuda_device, rows, k)
    try:
        h = torch.full((rows, k), float("nan"), device="cuda")
        fused.quantize_silu_mul(gut.data_ptr(), 2 * k, gut.data_ptr() + 4 * k, 2 * k, rows, h.data_ptr(), k)
        ya = torch.empty((rows, n), device="cuda")
        fused.matmul(op, ya.data_ptr(), n)
        ref_h = np_oracle.silu_mul(gu[:, :k], gu[:, k:])
        got_h = h.cpu().numpy()
        assert np.max(np.abs(got_h - ref_h)) <= 2e-6 * np.max(np.abs(ref_h))     # expf against the host's exp
        plain.quantize(h.data_ptr(), N.F32, rows, k)
        yb = torch.empty((rows, n), device="cuda")
        plain.matmul(op, yb.data_ptr(), n)
        torch.cuda.synchronize()
        assert torch.equal(ya, yb)
        ref, _, _ = sl_oracle.matmul_intdot(FMT_OF["Q4_K"], blocks, n, k, ref_h, threads=4)
        assert relative_rms(ya.cpu().numpy(), ref) <= CHAIN_RMS
        assert cuda_device.last_status() == 0
    finally:
        fused.dispose(); plain.dispose(); op.dispose(); weight.dispose()


@pytest.mark.gpu
def test_argmax_rows(cuda_device):
    torch = _torch()
    rng = np.random.Generator(np.random.Philox(5))
    for rows, n, stride in ((1, 7, 7), (32, 128256, 128256), (5, 1000, 1024), (3, 1025, 1025)):
        y = rng.standard_normal((rows, stride)).astype(np.float32)
        y[:, n:] = 1e9                                   # beyond n: must not be looked at
        if rows >= 3:
            y[0, 5] = y[0, 900 % n] = 50.0               # a tie: the first one wins
            y[1, 0] = np.nan                             # leading NaN: the scan answers 0
            y[2, 3] = np.nan; y[2, 4] = 60.0             # NaN elsewhere never wins
        yt = torch.from_numpy(y).cuda()
        out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        cuda_device.argmax_rows(yt.data_ptr(), rows, n, stride, out.data_ptr())
        torch.cuda.synchronize()
        assert out.cpu().numpy().tolist() == np_oracle.argmax_first(y[:, :n]).tolist()
    # behind a MatMul: the index of the largest logit per sequence
    n, k, rows = 5000, 1024, 9
    blocks = synth.weight_blocks("Q6_K", n, k, seed=2)
    x = synth.activations(rows, k, seed=3)
    w = cuda_device.upload_weight("Q6_K", (n, k), blocks)
    op = MatMulOp(cuda_device, w, rows)
    act = SharedActivation(cuda_device, rows, k)
    try:
        xt = torch.from_numpy(x).cuda()
        logits = torch.empty((rows, n), device="cuda")
        idx = torch.empty((rows,), dtype=torch.int32, device="cuda")
        act.quantize(xt.data_ptr(), N.F32, rows, k)
        act.matmul(op, logits.data_ptr(), n)
        cuda_device.argmax_rows(logits.data_ptr(), rows, n, n, idx.data_ptr())
        torch.cuda.synchronize()
        assert idx.cpu().numpy().tolist() == np_oracle.argmax_first(logits.cpu().numpy()).tolist()
    finally:
        act.dispose(); op.dispose(); w.dispose()


@pytest.mark.gpu
def test_producer_argument_checks(cuda_device):
    torch = _torch()
    act = SharedActivation(cuda_device, 4, 256)
    x = torch.zeros((4, 256), device="cuda")
    try:
        with pytest.raises(Exception):
            act.quantize_rmsnorm(x.data_ptr(), N.F32, 5, 256, 0, 1e-5)                # rows beyond the bound
        with pytest.raises(Exception):
            act.quantize_rmsnorm(x.data_ptr(), N.F32, 2, 128, 0, 1e-5)                # stride < K
        with pytest.raises(Exception):
            act.quantize_silu_mul(x.data_ptr(), 256, 0, 256, 2)                       # null up
        act.quantize_rmsnorm(x.data_ptr(), N.F32, 0, 256, 0, 1e-5)                    # zero rows: nothing happens
        with pytest.raises(Exception):
            cuda_device.argmax_rows(x.data_ptr(), 2, 256, 128, x.data_ptr())          # stride < n
    finally:
        act.dispose()
