"""Parity of the CUDA path with the CPU oracle, through the C ABI (needs a B200).

Bars: activation codes, scales and group sums bit-identical; per-block int32 dots bit-identical; fp32 outputs within
max relative error 1e-3 of the oracle's integer-dot result on the same inputs (helpers.max_rel_error states the
floor used for outputs that cancel to nothing). Shapes follow the reference's own tests
(tests/Sharplight.Cpu.Tests/QuantTests.cs:119-128, tests/Sharplight.Vulkan.Tests/MatMulTests.cs:7-48, MmqTests.cs:21-98,
SkinnyGemmTests.cs:29-39 of the Sharplight tree).
"""
import ctypes as C

import numpy as np
import pytest

from helpers import FMT_OF, MAX_REL, max_rel_error, relative_rms, sl_oracle
from sharplight_b200 import (ArgumentError, CompileOptions, GraphSegment, InvalidOperationError, MatMulNode, MatMulOp,
                             NotSupportedError, ObjectDisposedError, SharedActivation, WeightInfo, synth)
from sharplight_b200 import native as N
from sharplight_b200.provider import bf16_bits_to_f32, to_bf16_bits
from test_oracle import quantize_kat

pytestmark = pytest.mark.gpu

TYPES = ["Q8_0", "Q4_0", "Q4_K", "Q6_K"]


def check_matmul(device, type_name, n, k, rows, *, seed=1, kernel=N.KERNEL_AUTO, dots=True, blocks=None, x=None,
                 max_rows=None):
    fmt = FMT_OF[type_name]
    blocks = synth.weight_blocks(type_name, n, k, seed) if blocks is None else blocks
    x = synth.activations(rows, k, seed + 1000) if x is None else x
    w = device.upload_weight(type_name, (n, k), blocks)
    op = MatMulOp(device, w, max_rows or max(rows, 1))
    try:
        if kernel != N.KERNEL_AUTO:
            op.set_kernel(kernel)
        y = op.run(x)
        ref, ref64, s32 = sl_oracle.matmul_intdot(fmt, blocks, n, k, x, threads=8, want_f64=True, want_s32=dots)
        assert y.shape == ref.shape
        assert max_rel_error(y, ref) <= MAX_REL, (type_name, n, k, rows, op.last_kernel())
        assert max_rel_error(y, ref64) <= MAX_REL
        if dots and rows > 0 and n > 0:
            got = op.block_dots(x)
            assert np.array_equal(got, s32), (type_name, n, k, rows, op.last_kernel())
        return y, op.last_kernel()
    finally:
        op.dispose()
        w.dispose()


# ---- activation quantization ------------------------------------------------------------------------------------

def test_quantize_known_answers_bit_exact(cuda_device):
    x = quantize_kat()
    q, d, gs = cuda_device.debug_quantize(x)
    rq, rd, rgs = sl_oracle.quantize(x)
    assert np.array_equal(q, rq)
    assert np.array_equal(d.view(np.uint32), rd.view(np.uint32))
    assert np.array_equal(gs.view(np.uint32), rgs.view(np.uint32))


@pytest.mark.parametrize("rows,k", [(1, 32), (3, 1568), (8, 4096), (33, 1024), (70, 256)])
def test_quantize_random_bit_exact(cuda_device, rows, k):
    g = np.random.Generator(np.random.Philox(rows * 7919 + k))
    x = (g.standard_normal((rows, k)) * np.exp(g.uniform(-6, 6, (rows, 1)))).astype(np.float32)
    x[0, :32] = 0.0
    x[-1, -32:] = np.float32(-3.0)           # constant block: every code -127
    x[rows // 2, ::7] *= np.float32(1e4)
    q, d, gs = cuda_device.debug_quantize(x)
    rq, rd, rgs = sl_oracle.quantize(x)
    assert np.array_equal(q, rq)
    assert np.array_equal(d.view(np.uint32), rd.view(np.uint32))
    assert np.array_equal(gs.view(np.uint32), rgs.view(np.uint32))


def test_quantize_bf16_input(cuda_device):
    x = synth.activations(5, 512, 77)
    bits = to_bf16_bits(x)
    q, d, gs = cuda_device.debug_quantize(bits, N.BF16)
    rq, rd, rgs = sl_oracle.quantize(bf16_bits_to_f32(bits))
    assert np.array_equal(q, rq) and np.array_equal(d, rd) and np.array_equal(gs, rgs)


# ---- weights ----------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("type_name", TYPES)
@pytest.mark.parametrize("n,k", [(1, 256), (7, 512), (37, 1280), (16, 256), (4112, 512)])
def test_weight_layout_round_trip(cuda_device, type_name, n, k):
    """The device layout is a permutation of the raw blocks: download(upload(blocks)) == blocks."""
    blocks = synth.weight_blocks(type_name, n, k, seed=n + k)
    w = cuda_device.upload_weight(type_name, (n, k), blocks)
    try:
        assert np.array_equal(w.download(), blocks)
        assert w.device_bytes >= blocks.size
    finally:
        w.dispose()


@pytest.mark.parametrize("type_name,k", [("Q8_0", 1568), ("Q4_0", 1568), ("Q8_0", 32), ("Q4_0", 96)])
def test_weight_round_trip_k_not_multiple_of_256(cuda_device, type_name, k):
    blocks = synth.weight_blocks(type_name, 5, k, seed=k)
    w = cuda_device.upload_weight(type_name, (5, k), blocks)
    try:
        assert np.array_equal(w.download(), blocks)
    finally:
        w.dispose()


def test_upload_rejects_bad_shapes(cuda_device):
    with pytest.raises(ArgumentError):
        cuda_device.upload_weight("Q4_K", (4, 288), np.zeros(4 * 162, np.uint8))      # K % 256 != 0
    with pytest.raises(ArgumentError):
        cuda_device.upload_weight("Q8_0", (4, 64), np.zeros(10, np.uint8))            # byte count
    with pytest.raises(NotSupportedError):
        cuda_device.upload_weight("Q5_1", (4, 256), np.zeros(4 * 8 * 24, np.uint8))   # a format without kernels
    # Q5_K is split into two Q4_K weights, one of them with 16 d as its f16 scale: a d whose sixteenfold is no f16 is refused
    huge = synth.weight_blocks("Q5_K", 4, 256, seed=1).reshape(4, 176)
    huge[2, 0:2] = np.array([0xFF, 0x7B], np.uint8)                                   # d = 65504
    with pytest.raises(NotSupportedError):
        cuda_device.upload_weight("Q5_K", (4, 256), huge.reshape(-1))
    assert cuda_device.last_status() == 0


# ---- the operator ---------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("type_name", TYPES)
@pytest.mark.parametrize("rows", [1, 2, 3, 4, 5, 8, 9, 16, 17, 20, 33, 40, 64, 65, 100])
def test_matmul_row_counts(cuda_device, type_name, rows):
    """MatMulTests.WeightFormat: K = 512, N = 96 over the row counts that cross every kernel boundary."""
    check_matmul(cuda_device, type_name, 96, 512, rows, seed=rows)


@pytest.mark.parametrize("type_name", TYPES)
@pytest.mark.parametrize("n,k", [(7, 1536), (7, 2560), (7, 1024), (37, 768), (4112, 512), (1, 256), (16, 4096)])
def test_matmul_shapes(cuda_device, type_name, n, k):
    """QuantTests.MatMulWithIntDotMatchesReference shapes (N = 7), odd N, and SkinnyGemmTests' N = 4112."""
    for rows in (1, 3, 16, 40):
        check_matmul(cuda_device, type_name, n, k, rows, seed=n + rows, dots=(n * rows <= 4112 * 3))


@pytest.mark.parametrize("type_name", ["Q8_0", "Q4_0"])
@pytest.mark.parametrize("k", [32, 96, 1568])
def test_matmul_k_multiple_of_32_only(cuda_device, type_name, k):
    for rows in (1, 3, 12):
        check_matmul(cuda_device, type_name, 7, k, rows, seed=k)


@pytest.mark.parametrize("type_name", TYPES)
@pytest.mark.parametrize("kernel,rows", [(N.KERNEL_MMVQ, 1), (N.KERNEL_MMVQ, 7), (N.KERNEL_MMVQ, 19), (N.KERNEL_SKINNY, 1),
                                         (N.KERNEL_SKINNY, 2), (N.KERNEL_SKINNY, 24), (N.KERNEL_SKINNY, 130)])
def test_each_kernel_family_at_any_row_count(cuda_device, type_name, kernel, rows):
    _, (used, launches) = check_matmul(cuda_device, type_name, 100, 1024, rows, seed=rows, kernel=kernel)
    assert used == kernel and launches >= 1


@pytest.mark.parametrize("tid", [2, 8, 12, 14])
def test_golden_fixture_rows_as_weights(cuda_device, golden, tid):
    """The ggml-quantized (and the random-byte) fixture records as weights: device output vs the oracle, and vs the
    double product of ggml's own decoded floats with exactly representable activations (MatMulTests.
    IntDotExactActivations, MmqTests: atol 2e-3, rtol 1e-3)."""
    from helpers import TYPE_OF
    for kind in ("ggml", "random"):
        name = f"ext_{tid}_{kind}"
        _, rows, cols = (int(v) for v in golden[name + "_shape"])
        blocks = golden[name + "_blocks"]
        expected = golden[name + "_expected"].reshape(rows, cols)
        if not np.all(np.isfinite(expected)):
            # random bytes can decode to inf / nan scales: keep the rows whose floats are finite
            keep = np.all(np.isfinite(expected), axis=1)
            if not keep.any():
                continue
            bb = blocks.size // rows
            blocks = blocks.reshape(rows, bb)[keep].reshape(-1)
            expected = expected[keep]
            rows = int(keep.sum())
        for t in (1, 5, 20):
            x = synth.exact_int8_activations(t, cols, seed=tid * 10 + t)
            y, _ = check_matmul(cuda_device, TYPE_OF[tid], rows, cols, t, blocks=blocks, x=x)
            ref = x.astype(np.float64) @ expected.astype(np.float64).T
            scale = max(1.0, float(np.abs(ref).max()))
            assert np.all(np.abs(y - ref) <= 2e-3 * scale + 1e-3 * np.abs(ref))


@pytest.mark.parametrize("type_name", TYPES)
def test_row_invariance(cuda_device, type_name):
    """RowInvarianceTests (tests/Sharplight.Cpu.Tests/RowInvarianceTests.cs:11-57): with the row-invariant flag a
    2-4 row step equals single-row steps bit for bit."""
    n, k = 200, 1024
    blocks = synth.weight_blocks(type_name, n, k, 5)
    w = cuda_device.upload_weight(type_name, (n, k), blocks)
    op = MatMulOp(cuda_device, w, 8, row_invariant=True)
    try:
        x = synth.activations(8, k, 6)
        single = np.concatenate([op.run(x[i:i + 1]) for i in range(8)])
        for rows in (2, 3, 4, 8):
            multi = op.run(x[:rows])
            assert np.array_equal(multi.view(np.uint32), single[:rows].view(np.uint32))
    finally:
        op.dispose()
        w.dispose()


def test_int8_exact_activations_match_float_product(cuda_device):
    """With activations the quantizer represents exactly, the integer-dot result equals the product with the
    dequantized weight up to f32 rounding (MmqTests.cs:71-78: atol 2e-3, rtol 1e-3)."""
    for type_name in TYPES:
        n, k = 96, 1024
        blocks = synth.weight_blocks(type_name, n, k, 21)
        for rows in (2, 65):
            x = synth.exact_int8_activations(rows, k, 22)
            y, _ = check_matmul(cuda_device, type_name, n, k, rows, blocks=blocks, x=x, dots=False)
            exact = sl_oracle.matmul_f64(FMT_OF[type_name], blocks, n, k, x, threads=8)
            assert np.all(np.abs(y - exact) <= 2e-3 + 1e-3 * np.abs(exact))


def test_bf16_activations(cuda_device):
    n, k, rows = 64, 512, 6
    blocks = synth.weight_blocks("Q4_0", n, k, 31)
    bits = to_bf16_bits(synth.activations(rows, k, 32))
    w = cuda_device.upload_weight("Q4_0", (n, k), blocks)
    op = MatMulOp(cuda_device, w, rows)
    try:
        y = op.run(bits, N.BF16)
        ref, _, _ = sl_oracle.matmul_intdot(2, blocks, n, k, bf16_bits_to_f32(bits))
        assert max_rel_error(y, ref) <= MAX_REL
    finally:
        op.dispose()
        w.dispose()


def test_edge_cases_and_errors(cuda_device):
    blocks = synth.weight_blocks("Q8_0", 8, 64, 1)
    w = cuda_device.upload_weight("Q8_0", (8, 64), blocks)
    op = MatMulOp(cuda_device, w, 4)
    assert op.run(np.zeros((0, 64), np.float32)).shape == (0, 8)          # empty input is a no-op
    with pytest.raises(InvalidOperationError):
        op.run(np.zeros((5, 64), np.float32))                             # rows beyond the compiled bound
    with pytest.raises(ArgumentError):
        op.run(np.zeros((1, 32), np.float32))                             # wrong K
    y = op.run(np.zeros((2, 64), np.float32))
    assert not y.any()                                                    # all-zero activations: zero scales
    op.dispose()
    with pytest.raises(ObjectDisposedError):
        op.run(np.zeros((1, 64), np.float32))
    w.dispose()
    empty = cuda_device.upload_weight("Q4_K", (0, 256), np.zeros(0, np.uint8))   # a weight with no rows
    op = MatMulOp(cuda_device, empty, 2)
    assert op.run(np.ones((2, 256), np.float32)).shape == (2, 0)
    op.dispose()
    empty.dispose()
    assert cuda_device.last_status() == 0


def test_segment_contract(cuda_device):
    """ICompiledSegment behaviour (src/Sharplight.Cpu/CpuCompiledSegment.cs:96-124,149,189)."""
    k, n1, n2 = 512, 48, 80
    w1 = WeightInfo("Q4_K", (n1, k), synth.weight_blocks("Q4_K", n1, k, 1))
    w2 = WeightInfo("Q8_0", (n2, k), synth.weight_blocks("Q8_0", n2, k, 2))
    seg = GraphSegment([MatMulNode("gate", "x", w1, "g"), MatMulNode("up", "x", w2, "u")], ["x"], ["g", "u"])
    compiled = cuda_device.compile(seg, CompileOptions(max_rows=8))
    assert compiled.device_memory_bytes > 0
    with pytest.raises(InvalidOperationError):
        compiled.get_output("g")                                          # before Execute
    with pytest.raises(ArgumentError):
        compiled.set_input("nope", np.zeros((1, k), np.float32))
    with pytest.raises(ArgumentError):
        compiled.set_input("x", np.zeros((9, k), np.float32))             # beyond the compiled capacity
    x = synth.activations(8, k, 3)
    compiled.set_input("x", x)
    with pytest.raises(InvalidOperationError):
        compiled.execute({"T": 9})
    compiled.execute({"T": 5})
    g = compiled.get_output("g")
    ref, _, _ = sl_oracle.matmul_intdot(12, w1.blocks, n1, k, x[:5])
    assert g.shape == (5, n1) and max_rel_error(g, ref) <= MAX_REL
    ref2, _, _ = sl_oracle.matmul_intdot(8, w2.blocks, n2, k, x[:5])
    assert max_rel_error(compiled.get_output("u"), ref2) <= MAX_REL
    compiled.dispose()
    with pytest.raises(ObjectDisposedError):
        compiled.execute({"T": 1})
    with pytest.raises(NotSupportedError):
        cuda_device.compile(GraphSegment([MatMulNode("m", "x", WeightInfo("Q5_1", (4, 256), np.zeros(768, np.uint8)),
                                                     "y")], ["x"], ["y"]), CompileOptions())


def test_segment_replays_a_captured_step(cuda_device):
    """From the third Execute with the same row counts the step is a captured graph (outputs copied on a side stream):
    every call, before and after the capture, must return what a fresh MatMul of that call's input gives; a different
    row count in between gets its own steps; a chained node (y of one MatMul feeding the next) stays on the device."""
    k, n1, n2 = 512, 64, 96
    w1 = WeightInfo("Q4_K", (n1, k), synth.weight_blocks("Q4_K", n1, k, 4))
    w2 = WeightInfo("Q8_0", (n2, k), synth.weight_blocks("Q8_0", n2, k, 5))
    w3 = WeightInfo("Q8_0", (32, n2), synth.weight_blocks("Q8_0", 32, n2, 6))
    seg = GraphSegment([MatMulNode("a", "x", w1, "ya"), MatMulNode("b", "x", w2, "yb"), MatMulNode("c", "yb", w3, "yc")],
                       ["x"], ["ya", "yc"])
    compiled = cuda_device.compile(seg, CompileOptions(max_rows=4))
    eager = cuda_device.compile(seg, CompileOptions(max_rows=4, capture_steps=False))
    try:
        for call, rows in enumerate((1, 1, 1, 1, 3, 1, 3, 3, 3, 1)):
            x = synth.activations(rows, k, 50 + call) * np.float32(1 + call)
            for c in (compiled, eager):
                c.set_input("x", x)
                c.execute({"T": rows})
            ya, yc = compiled.get_output("ya"), compiled.get_output("yc")
            assert ya.shape == (rows, n1) and yc.shape == (rows, 32)
            assert np.array_equal(ya, eager.get_output("ya")) and np.array_equal(yc, eager.get_output("yc")), call
            ref, _, _ = sl_oracle.matmul_intdot(12, w1.blocks, n1, k, x)
            assert max_rel_error(ya, ref) <= MAX_REL
        assert cuda_device.last_status() == 0
    finally:
        compiled.dispose()
        eager.dispose()


def test_segment_forwards_an_output_on_the_device(cuda_device):
    """IDeviceForwardingSegment.TryForwardFrom: the second segment reads the first one's output in device memory; the
    value is neither downloaded nor uploaded, and the result equals the two MatMuls chained through the host."""
    k, n1, n2 = 512, 256, 48
    w1 = WeightInfo("Q4_K", (n1, k), synth.weight_blocks("Q4_K", n1, k, 7))
    w2 = WeightInfo("Q4_K", (n2, n1), synth.weight_blocks("Q4_K", n2, n1, 8))
    first = cuda_device.compile(GraphSegment([MatMulNode("a", "x", w1, "h")], ["x"], ["h"]), CompileOptions(max_rows=4))
    second = cuda_device.compile(GraphSegment([MatMulNode("b", "h", w2, "y")], ["h"], ["y"]), CompileOptions(max_rows=4))
    host_a = cuda_device.compile(GraphSegment([MatMulNode("a", "x", w1, "h")], ["x"], ["h"]), CompileOptions(max_rows=4))
    host_b = cuda_device.compile(GraphSegment([MatMulNode("b", "h", w2, "y")], ["h"], ["y"]), CompileOptions(max_rows=4))
    other = cuda_device.compile(GraphSegment([MatMulNode("c", "x", w1, "z")], ["x"], ["z"]), CompileOptions(max_rows=4))
    try:
        assert not second.try_forward_from("h", other)        # that segment has no output of this name
        assert not second.try_forward_from("y", first)        # not an input of this segment
        assert second.try_forward_from("h", first)
        first.keep_on_device("h")
        with pytest.raises(InvalidOperationError):
            second.set_input("h", np.zeros((1, n1), np.float32))
        for call, rows in enumerate((1, 1, 1, 1, 3, 3, 3, 3)):    # long enough for both segments to switch to their graphs
            x = synth.activations(rows, k, 60 + call)
            first.set_input("x", x)
            first.execute({"T": rows})
            second.execute({"T": rows})
            host_a.set_input("x", x)
            host_a.execute({"T": rows})
            host_b.set_input("h", host_a.get_output("h"))
            host_b.execute({"T": rows})
            assert np.array_equal(second.get_output("y"), host_b.get_output("y")), call
        with pytest.raises(InvalidOperationError):
            first.get_output("h")
        assert cuda_device.last_status() == 0
    finally:
        for seg in (second, first, host_a, host_b, other):
            seg.dispose()


# ---- the benchmark configurations at full size ------------------------------------------------------------------

def test_config1_q8_0_qwen_up_proj(cuda_device):
    check_matmul(cuda_device, "Q8_0", 3072, 1024, 1, seed=101)


@pytest.mark.parametrize("rows", [1, 4, 16, 64])
def test_config2_q4_k_llama8b_ffn(cuda_device, rows):
    check_matmul(cuda_device, "Q4_K", 14336, 4096, rows, seed=102, dots=(rows <= 4))


def test_intdot_stays_close_to_exact_product_at_full_size(cuda_device):
    """Size-independent property at the benchmark shape: 8-bit activations cost < 1e-2 relative RMS."""
    n, k, rows = 14336, 4096, 4
    blocks = synth.weight_blocks("Q4_K", n, k, 102)
    x = synth.activations(rows, k, 103)
    w = cuda_device.upload_weight("Q4_K", (n, k), blocks)
    op = MatMulOp(cuda_device, w, rows)
    try:
        y = op.run(x)
        exact = sl_oracle.matmul_f64(12, blocks, n, k, x, threads=8)
        assert relative_rms(y, exact) < 1e-2
        # linearity in the weight rows: permuting rows of W permutes columns of y
        perm = np.random.Generator(np.random.Philox(9)).permutation(n)
        wp = cuda_device.upload_weight("Q4_K", (n, k), blocks.reshape(n, -1)[perm].reshape(-1))
        opp = MatMulOp(cuda_device, wp, rows)
        assert np.array_equal(opp.run(x), y[:, perm])
        opp.dispose()
        wp.dispose()
    finally:
        op.dispose()
        w.dispose()


# ---- prefill: the tensor-core GEMM ------------------------------------------------------------------------------

@pytest.mark.parametrize("type_name", ["Q4_0", "Q8_0", "Q4_K", "Q6_K"])
@pytest.mark.parametrize("rows,n,k", [(65, 96, 512), (200, 100, 512), (300, 520, 512), (129, 128, 256), (1000, 3000, 256)])
def test_mmq_shapes(cuda_device, type_name, rows, n, k):
    """MmqTests (tests/Sharplight.Vulkan.Tests/MmqTests.cs:21-98): (T, N) in {(65, 96), (200, 100), (300, 520)} at
    K = 512 and the large grid T = 1000, N = 3000, K = 256; here every block dot is also compared bit for bit."""
    _, (used, launches) = check_matmul(cuda_device, type_name, n, k, rows, seed=rows + n, kernel=N.KERNEL_MMQ,
                                       dots=(rows * n <= 300 * 520))
    assert used == N.KERNEL_MMQ and launches >= 1


@pytest.mark.parametrize("type_name", ["Q4_0", "Q8_0", "Q4_K", "Q6_K"])
def test_mmq_exact_int8_activations(cuda_device, type_name):
    """MmqTests' exact-activation case (K = 1024): atol 2e-3, rtol 1e-3 against the product with the dequantized weight."""
    n, k, rows = 520, 1024, 300
    blocks = synth.weight_blocks(type_name, n, k, 41)
    x = synth.exact_int8_activations(rows, k, 42)
    y, _ = check_matmul(cuda_device, type_name, n, k, rows, blocks=blocks, x=x, dots=False, kernel=N.KERNEL_MMQ)
    exact = sl_oracle.matmul_f64(FMT_OF[type_name], blocks, n, k, x, threads=8)
    assert np.all(np.abs(y - exact) <= 2e-3 + 1e-3 * np.abs(exact))


def test_config3_q4_0_prefill_bf16(cuda_device):
    """benchmark configuration 3 at full size: Q4_0 [4096, 4096], bf16 activations [2048, 4096]. The oracle checks a sample of
    the token rows (rows are independent), every weight row; the block dots of a second, smaller sample bit for bit."""
    n, k, rows = 4096, 4096, 2048
    blocks = synth.weight_blocks("Q4_0", n, k, 103)
    bits = to_bf16_bits(synth.activations(rows, k, 104))
    w = cuda_device.upload_weight("Q4_0", (n, k), blocks)
    op = MatMulOp(cuda_device, w, rows)
    try:
        y = op.run(bits, N.BF16)
        assert op.last_kernel()[0] == N.KERNEL_MMQ
        sample = np.random.Generator(np.random.Philox(5)).choice(rows, 24, replace=False)
        xs = bf16_bits_to_f32(bits[sample])
        ref, ref64, _ = sl_oracle.matmul_intdot(2, blocks, n, k, xs, threads=8, want_f64=True)
        assert max_rel_error(y[sample], ref) <= MAX_REL
        assert max_rel_error(y[sample], ref64) <= MAX_REL
    finally:
        op.dispose()
        w.dispose()


def _check_sampled_rows(device, type_name, n, k, rows, seed, sample_n):
    """Full-size weight on the GPU; the oracle recomputes a sample of the weight rows (rows of W are independent)."""
    fmt = FMT_OF[type_name]
    blocks = synth.weight_blocks(type_name, n, k, seed)
    x = synth.activations(rows, k, seed + 1)
    w = device.upload_weight(type_name, (n, k), blocks)
    op = MatMulOp(device, w, rows)
    try:
        y = op.run(x)
        pick = np.sort(np.random.Generator(np.random.Philox(seed)).choice(n, sample_n, replace=False))
        row_bytes = blocks.size // n
        sub = np.ascontiguousarray(blocks.reshape(n, row_bytes)[pick]).reshape(-1)
        ref, ref64, _ = sl_oracle.matmul_intdot(fmt, sub, sample_n, k, x, threads=8, want_f64=True)
        assert max_rel_error(y[:, pick], ref) <= MAX_REL, (type_name, n, k, rows, op.last_kernel())
        assert max_rel_error(y[:, pick], ref64) <= MAX_REL
        assert device.last_status() == 0
        return op.last_kernel()[0]
    finally:
        op.dispose()
        w.dispose()


def test_config4_q6_k_lm_head_batch32(cuda_device):
    """benchmark configuration 4's largest MatMul at full size: the Q6_K lm_head [128256, 4096] for a batch of 32 sequences."""
    assert _check_sampled_rows(cuda_device, "Q6_K", 128256, 4096, 32, 201, 512) == N.KERNEL_SKINNY


@pytest.mark.parametrize("n,k,rows", [(8192, 28672, 1), (8192, 28672, 64), (10240, 8192, 8), (57344, 8192, 1),
                                      (8192, 3584, 1), (1280, 8192, 64)])
def test_config5_llama70b_shapes(cuda_device, n, k, rows):
    """benchmark configuration 5: the Q4_K MatMuls of a Llama-3-70B-shaped layer at full size, whole (down [8192, 28672],
    stacked qkv [10240, 8192], stacked gate_up [57344, 8192]) and as 8-way tensor-parallel shards."""
    _check_sampled_rows(cuda_device, "Q4_K", n, k, rows, 300 + rows, 256)


# ---- short K with 3 and 4 rows on the dp4a family (a CTA of one warp owns two output values per thread) ----------------

@pytest.mark.parametrize("type_name,k", [("Q8_0", 32), ("Q4_0", 64), ("Q8_0", 256), ("Q4_K", 256), ("Q6_K", 256)])
@pytest.mark.parametrize("rows", [3, 4, 7])
def test_mmvq_short_k_three_and_four_rows(cuda_device, type_name, k, rows):
    check_matmul(cuda_device, type_name, 40, k, rows, seed=rows + k, kernel=N.KERNEL_MMVQ)


@pytest.mark.parametrize("rows", [3, 4, 8])
def test_row_invariant_short_k(cuda_device, rows):
    blocks = synth.weight_blocks("Q4_K", 48, 256, seed=3)
    x = synth.activations(rows, 256, seed=4)
    w = cuda_device.upload_weight("Q4_K", (48, 256), blocks)
    op = MatMulOp(cuda_device, w, 8, row_invariant=True)
    try:
        y = op.run(x)
        singles = np.concatenate([op.run(x[i:i + 1]) for i in range(rows)], axis=0)
        assert np.array_equal(y.view(np.uint32), singles.view(np.uint32))
        ref, _, _ = sl_oracle.matmul_intdot(FMT_OF["Q4_K"], blocks, 48, 256, x, threads=4, want_f64=False, want_s32=False)
        assert max_rel_error(y, ref) <= MAX_REL
    finally:
        op.dispose()
        w.dispose()


# ---- the tcgen05 tile kernel (selectable family): stream-K over persistent CTAs, every token-tile width ---------------------

@pytest.mark.parametrize("type_name,n,k,rows", [
    ("Q4_0", 128, 256, 16), ("Q4_0", 96, 512, 5), ("Q8_0", 96, 512, 3), ("Q4_K", 96, 512, 8), ("Q4_K", 130, 1024, 17),
    ("Q4_K", 300, 2048, 33), ("Q8_0", 7, 1568, 12), ("Q4_0", 7, 96, 3), ("Q4_K", 1000, 3072, 64), ("Q4_K", 384, 1024, 65),
    ("Q4_0", 640, 2048, 130), ("Q8_0", 256, 1024, 300), ("Q4_K", 4112, 512, 40), ("Q4_K", 1000, 2816, 256),
    ("Q8_0", 2500, 1024, 31), ("Q4_0", 19000, 256, 9), ("Q6_K", 128, 256, 65), ("Q6_K", 1000, 2816, 300),
    ("Q6_K", 7, 512, 70), ("Q6_K", 520, 1024, 129)])
def test_tile_kernel_shapes(cuda_device, type_name, n, k, rows):
    """Ragged N and K, every token-tile width (16, 32, 64, 128), tiles split between CTAs and tiles owned by one CTA,
    more tiles than CTAs and fewer; y against the oracle and the int32 block dots bit for bit."""
    _, kern = check_matmul(cuda_device, type_name, n, k, rows, seed=n + k + rows, kernel=N.KERNEL_TILE)
    assert kern[0] == N.KERNEL_TILE
    assert cuda_device.last_status() == 0


def test_tile_kernel_falls_back_where_it_does_not_serve(cuda_device):
    # Q6_K is served at the 128-token tile only: up to 64 rows the forced family falls back to the automatic choice
    _, kern = check_matmul(cuda_device, "Q6_K", 64, 256, 8, kernel=N.KERNEL_TILE)
    assert kern[0] != N.KERNEL_TILE
    # and so do fewer than 3 rows of any format
    _, kern = check_matmul(cuda_device, "Q4_K", 64, 512, 2, kernel=N.KERNEL_TILE, max_rows=8)
    assert kern[0] != N.KERNEL_TILE


def test_q6_k_prefill_takes_the_gemm(cuda_device):
    """More than 64 rows of a Q6_K weight: two half-masked tensor-core instructions per block instead of 64-row chunks of
    the skinny kernel (the reference's GEMM serves Q6_K the same way, src/Sharplight.Shaders/Kernels/mmq.slang:235-239);
    ragged N and K, block dots bit for bit, then a full-size case against a sample of the weight rows."""
    _, kern = check_matmul(cuda_device, "Q6_K", 640, 1024, 200, seed=9)
    assert kern[0] == N.KERNEL_MMQ
    _, kern = check_matmul(cuda_device, "Q6_K", 1000, 2816, 300, seed=10)
    assert kern[0] == N.KERNEL_MMQ
    _, kern = check_matmul(cuda_device, "Q6_K", 7, 512, 70, seed=11)
    assert kern[0] == N.KERNEL_MMQ
    assert _check_sampled_rows(cuda_device, "Q6_K", 4096, 4096, 2048, 210, 32) == N.KERNEL_MMQ
    assert _check_sampled_rows(cuda_device, "Q6_K", 32064, 4096, 300, 211, 48) == N.KERNEL_MMQ


@pytest.mark.parametrize("rows", [16, 64])
def test_tile_kernel_config2_full_size(cuda_device, rows):
    fmt, n, k = FMT_OF["Q4_K"], 14336, 4096
    blocks = synth.weight_blocks("Q4_K", n, k, 77)
    x = synth.activations(rows, k, 78 + rows)
    w = cuda_device.upload_weight("Q4_K", (n, k), blocks)
    op = MatMulOp(cuda_device, w, rows)
    try:
        op.set_kernel(N.KERNEL_TILE)
        y = op.run(x)
        ref, ref64, _ = sl_oracle.matmul_intdot(fmt, blocks, n, k, x, threads=8, want_f64=True)
        assert max_rel_error(y, ref) <= MAX_REL and max_rel_error(y, ref64) <= MAX_REL
        assert op.last_kernel()[0] == N.KERNEL_TILE and cuda_device.last_status() == 0
    finally:
        op.dispose()
        w.dispose()


# ---- prefill GEMM at full size: int32 block dots of config 3, and the 70B-shaped Q4_K MatMuls at 2048 rows -----------------

@pytest.mark.parametrize("kernel", [N.KERNEL_AUTO, N.KERNEL_TILE])
def test_config3_block_dots_sample_full_size(cuda_device, kernel):
    """Q4_0 [4096, 4096] x [2048, 4096]: the GEMM exports every int32 block dot of the full-size problem (4.3 GB); a sample of
    token rows is compared bit for bit with the oracle's."""
    n, k, rows = 4096, 4096, 2048
    blocks = synth.weight_blocks("Q4_0", n, k, 103)
    x = synth.activations(rows, k, 105)
    w = cuda_device.upload_weight("Q4_0", (n, k), blocks)
    op = MatMulOp(cuda_device, w, rows)
    try:
        if kernel != N.KERNEL_AUTO:
            op.set_kernel(kernel)
        got = op.block_dots(x)
        assert op.last_kernel()[0] == (N.KERNEL_MMQ if kernel == N.KERNEL_AUTO else kernel)
        sample = np.sort(np.random.Generator(np.random.Philox(9)).choice(rows, 12, replace=False))
        _, _, s32 = sl_oracle.matmul_intdot(2, blocks, n, k, x[sample], threads=8, want_f64=False, want_s32=True)
        assert np.array_equal(got[sample], s32)
        assert cuda_device.last_status() == 0
    finally:
        op.dispose()
        w.dispose()


@pytest.mark.parametrize("kernel", [N.KERNEL_AUTO, N.KERNEL_TILE])
@pytest.mark.parametrize("n,k", [(8192, 8192), (1280, 8192), (8192, 3584)])
def test_q4_k_gemm_70b_shapes_at_2048_rows(cuda_device, n, k, kernel):
    """The Q4_K MatMuls of the 70B-shaped stack in prefill: attention output [8192, 8192], and the 8-way tensor-parallel
    shards of stacked qkv [1280, 8192] and down [8192, 3584], 2048 token rows; a sample of weight rows against the oracle."""
    fmt, rows, sample_n = FMT_OF["Q4_K"], 2048, 48
    blocks = synth.weight_blocks("Q4_K", n, k, 400 + n % 97)
    x = synth.activations(rows, k, 401)
    w = cuda_device.upload_weight("Q4_K", (n, k), blocks)
    op = MatMulOp(cuda_device, w, rows)
    try:
        if kernel != N.KERNEL_AUTO:
            op.set_kernel(kernel)
        y = op.run(x)
        assert op.last_kernel()[0] == (N.KERNEL_MMQ if kernel == N.KERNEL_AUTO else kernel)
        pick = np.sort(np.random.Generator(np.random.Philox(n + k)).choice(n, sample_n, replace=False))
        sub = np.ascontiguousarray(blocks.reshape(n, blocks.size // n)[pick]).reshape(-1)
        ref, ref64, _ = sl_oracle.matmul_intdot(fmt, sub, sample_n, k, x, threads=8, want_f64=True)
        assert max_rel_error(y[:, pick], ref) <= MAX_REL
        assert max_rel_error(y[:, pick], ref64) <= MAX_REL
        assert cuda_device.last_status() == 0
    finally:
        op.dispose()
        w.dispose()


# ---- K chunks in the skinny kernel (few weight rows, long K) -----------------------------------------------------------

@pytest.mark.parametrize("type_name,n,k,rows", [("Q4_K", 64, 8192, 8), ("Q4_K", 200, 2816, 5), ("Q8_0", 40, 8448, 16),
                                                ("Q4_0", 1000, 4096, 33), ("Q6_K", 130, 4352, 64), ("Q4_K", 4096, 14336, 32)])
def test_skinny_k_chunks(cuda_device, type_name, n, k, rows):
    """Row tiles alone would fill less than the machine: the launch splits K between CTAs (2 to 8 chunks, uneven and empty
    last chunks included); the sum over chunks must not change the result beyond rounding, the block dots not at all."""
    dots = n * k * rows <= 1 << 28
    _, kern = check_matmul(cuda_device, type_name, n, k, rows, seed=n + rows, kernel=N.KERNEL_SKINNY, dots=dots)
    assert kern[0] == N.KERNEL_SKINNY and cuda_device.last_status() == 0
    # twice in a row: the arrival counters are back at zero
    check_matmul(cuda_device, type_name, n, k, rows, seed=n + rows + 1, kernel=N.KERNEL_SKINNY, dots=False)


# ---- f32 activations kept: the dequant-fused f32 mat-vec ---------------------------------------------------------------

@pytest.mark.parametrize("type_name", TYPES)
@pytest.mark.parametrize("n,k,rows", [(40, 256, 1), (100, 1024, 3), (33, 4096, 4), (7, 2560, 9), (4112, 512, 2)])
def test_f32_activation_matvec(cuda_device, type_name, n, k, rows):
    """An op that keeps f32 activation math against the exact product of the dequantized weight (the oracle's f64
    MatMul), at the tolerance the reference holds its f32 paths to (atol 2e-3, rtol 1e-4,
    tests/Sharplight.Cpu.Tests/QuantTests.cs:257-265) -- far tighter than 8-bit activations could meet."""
    blocks = synth.weight_blocks(type_name, n, k, seed=n + k)
    x = synth.activations(rows, k, seed=rows + k)
    w = cuda_device.upload_weight(type_name, (n, k), blocks)
    op = MatMulOp(cuda_device, w, rows, f32_activations=True)
    try:
        y = op.run(x)
        exact = sl_oracle.matmul_f64(FMT_OF[type_name], blocks, n, k, x, threads=4)
        assert np.all(np.abs(y - exact) <= 2e-3 + 1e-4 * np.abs(exact)), float(np.max(np.abs(y - exact)))
        assert op.last_kernel()[0] == N.KERNEL_F32
        bits = to_bf16_bits(x)
        yb = op.run(bits, N.BF16)
        exact_b = sl_oracle.matmul_f64(FMT_OF[type_name], blocks, n, k, bf16_bits_to_f32(bits), threads=4)
        assert np.all(np.abs(yb - exact_b) <= 2e-3 + 1e-4 * np.abs(exact_b))
        # such an op takes no quantized activations
        act = SharedActivation(cuda_device, rows, k)
        try:
            with pytest.raises(Exception):
                act.matmul(op, 0, n)
        finally:
            act.dispose()
    finally:
        op.dispose()
        w.dispose()


def test_f32_activation_node_in_a_segment(cuda_device):
    """A segment with one node that keeps f32 activations and one that does not, reading the same input."""
    from sharplight_b200 import CompileOptions, GraphSegment, MatMulNode, WeightInfo
    n, k, rows = 64, 1024, 3
    b1, b2 = synth.weight_blocks("Q4_K", n, k, 1), synth.weight_blocks("Q8_0", n, k, 2)
    x = synth.activations(rows, k, 3)
    nodes = [MatMulNode("a", "x", WeightInfo("Q4_K", (n, k), b1), "ya", f32_activations=True),
             MatMulNode("b", "x", WeightInfo("Q8_0", (n, k), b2), "yb")]
    seg = cuda_device.compile(GraphSegment(nodes, ["x"], ["ya", "yb"]), CompileOptions(max_rows=4))
    try:
        for _ in range(4):      # direct launches, then the captured graph
            seg.set_input("x", x)
            seg.execute({"T": rows})
            ya, yb = seg.get_output("ya"), seg.get_output("yb")
            exact = sl_oracle.matmul_f64(FMT_OF["Q4_K"], b1, n, k, x, threads=4)
            assert np.all(np.abs(ya - exact) <= 2e-3 + 1e-4 * np.abs(exact))
            ref, _, _ = sl_oracle.matmul_intdot(FMT_OF["Q8_0"], b2, n, k, x, threads=4)
            assert max_rel_error(yb, ref) <= MAX_REL
    finally:
        seg.dispose()


# ---- view nodes in front of a MatMul: Slice and Reshape are a pointer and a stride, Permute is gathered first -------------

def test_views_in_front_of_matmuls(cuda_device):
    from sharplight_b200 import ViewNode
    rows = 5
    x = synth.activations(rows, 3074, 11)          # sliced at an odd column: rows that start at any element
    z = synth.activations(rows, 1024, 12)
    w1 = synth.weight_blocks("Q4_K", 48, 2048, 1)
    w2 = synth.weight_blocks("Q8_0", 40, 1024, 2)
    w3 = synth.weight_blocks("Q6_K", 24, 1024, 3)
    nodes = [ViewNode("v1", "x", "xs", "slice", 3074, start=1025, length=2048),
             MatMulNode("m1", "xs", WeightInfo("Q4_K", (48, 2048), w1), "y1"),
             ViewNode("v2", "z", "zr", "reshape", 1024, split=4),
             ViewNode("v3", "z", "zp", "permute", 1024, a=4, b=256),
             MatMulNode("m2", "zp", WeightInfo("Q8_0", (40, 1024), w2), "y2"),
             MatMulNode("m3", "z", WeightInfo("Q6_K", (24, 1024), w3), "y3")]
    w4 = synth.weight_blocks("Q4_0", 16, 256, 4)
    nodes.append(MatMulNode("m4", "zr", WeightInfo("Q4_0", (16, 256), w4), "y4"))      # [4 T, 256] rows out of [T, 1024]
    seg = cuda_device.compile(GraphSegment(nodes, ["x", "z"], ["y1", "y2", "y3", "y4"]), CompileOptions(max_rows=8))
    try:
        for _ in range(4):          # direct launches, then the captured graph
            seg.set_input("x", x)
            seg.set_input("z", z)
            seg.execute({"T": rows})
            ref, _, _ = sl_oracle.matmul_intdot(FMT_OF["Q4_K"], w1, 48, 2048, np.ascontiguousarray(x[:, 1025:3073]), threads=4)
            assert max_rel_error(seg.get_output("y1"), ref) <= MAX_REL
            zp = np.ascontiguousarray(z.reshape(rows, 4, 256).transpose(0, 2, 1).reshape(rows, 1024))
            ref, _, _ = sl_oracle.matmul_intdot(FMT_OF["Q8_0"], w2, 40, 1024, zp, threads=4)
            assert max_rel_error(seg.get_output("y2"), ref) <= MAX_REL
            ref, _, _ = sl_oracle.matmul_intdot(FMT_OF["Q6_K"], w3, 24, 1024, z, threads=4)
            assert max_rel_error(seg.get_output("y3"), ref) <= MAX_REL
            ref, _, _ = sl_oracle.matmul_intdot(FMT_OF["Q4_0"], w4, 16, 256, z.reshape(rows * 4, 256), threads=4)
            y4 = seg.get_output("y4")
            assert y4.shape == (rows * 4, 16) and max_rel_error(y4, ref) <= MAX_REL
    finally:
        seg.dispose()
    with pytest.raises(Exception):
        cuda_device.compile(GraphSegment([ViewNode("v", "x", "xs", "slice", 1024, start=1000, length=100)], ["x"], []),
                            CompileOptions(max_rows=2))


# ---- the device layout as an artefact ---------------------------------------------------------------------------------

@pytest.mark.parametrize("type_name,n,k", [("Q4_K", 100, 1024), ("Q8_0", 37, 1568), ("Q6_K", 4112, 512), ("Q4_0", 7, 96)])
def test_weight_layout_artefact_round_trip(cuda_device, type_name, n, k):
    """Export the re-laid-out records, import them on the device without the raw blocks: the same weight (raw blocks
    come back byte for byte) and the same MatMul bits; a damaged or foreign artefact is refused."""
    blocks = synth.weight_blocks(type_name, n, k, seed=n)
    x = synth.activations(5, k, seed=k)
    w = cuda_device.upload_weight(type_name, (n, k), blocks)
    art = w.export_layout()
    w2 = cuda_device.import_weight_layout(art)
    op, op2 = MatMulOp(cuda_device, w, 5), MatMulOp(cuda_device, w2, 5)
    try:
        assert (w2.n, w2.k, w2.format) == (n, k, FMT_OF[type_name])
        assert np.array_equal(w2.download(), blocks)
        assert np.array_equal(op.run(x).view(np.uint32), op2.run(x).view(np.uint32))
        bad = art.copy(); bad[0] ^= 0xFF
        with pytest.raises(Exception):
            cuda_device.import_weight_layout(bad)
        with pytest.raises(Exception):
            cuda_device.import_weight_layout(art[:-16])
        newer = art.copy(); newer[4] = 99
        with pytest.raises(NotSupportedError):
            cuda_device.import_weight_layout(newer)
    finally:
        op.dispose(); op2.dispose(); w.dispose(); w2.dispose()


# ---- deferred quantization: the mat-vec quantizes short rows itself ------------------------------------------------------

@pytest.mark.parametrize("type_name", TYPES + ["Q5_K", "Q5_0"])
@pytest.mark.parametrize("n,k,rows", [(64, 1024, 1), (200, 3584, 2), (48, 512, 4), (100, 4096, 1), (40, 8192, 1), (64, 1024, 8),
                                      (33, 1568, 3)])
def test_deferred_quantization_bit_identical(cuda_device, type_name, n, k, rows):
    """slc_activation_set_rows + MatMul against slc_activation_quantize + the same MatMul: the same bits whether the
    mat-vec quantized the rows inside its own kernel (K <= 2048, up to 4 rows per launch), or the quantizer ran at the
    first use (longer K, more rows, other kernel families); a second MatMul on the same rows included."""
    import torch
    if k % N.BLOCK[FMT_OF[type_name]][0] != 0:
        pytest.skip("K is not a multiple of this format's block size")
    blocks = synth.weight_blocks(type_name, n, k, seed=n + k)
    x = torch.from_numpy(synth.activations(rows, k + 5, seed=k)[:, 2:2 + k].copy()).cuda()     # (a contiguous copy)
    xs = torch.from_numpy(synth.activations(rows, k + 8, seed=k)).cuda()                        # rows 8 elements wider than K
    w = cuda_device.upload_weight(type_name, (n, k), blocks)
    op = MatMulOp(cuda_device, w, rows)
    a0, a1 = SharedActivation(cuda_device, rows, k), SharedActivation(cuda_device, rows, k)
    try:
        for src, stride in ((x, k), (xs, k + 8)):
            y0 = torch.empty((rows, n), device="cuda"); y1 = torch.empty((rows, n), device="cuda"); y2 = torch.empty((rows, n), device="cuda")
            a0.quantize(src.data_ptr(), N.F32, rows, stride)
            a0.matmul(op, y0.data_ptr(), n)
            a1.set_rows(src.data_ptr(), N.F32, rows, stride)
            a1.matmul(op, y1.data_ptr(), n)
            fused = op.last_kernel()[0] == N.KERNEL_MMVQ and k <= 2048 and type_name != "Q5_K"   # (two passes: quantized once)
            assert op.last_kernel()[1] == ((rows + 3) // 4 if fused else op.last_kernel()[1])
            a1.matmul(op, y2.data_ptr(), n)
            torch.cuda.synchronize()
            assert torch.equal(y0, y1) and torch.equal(y0, y2), (type_name, n, k, rows)
        assert cuda_device.last_status() == 0
    finally:
        a0.dispose(); a1.dispose(); op.dispose(); w.dispose()


# ---- formats rewritten at upload as Q8_0 device records: Q5_0, IQ4_NL ---------------------------------------------------

CONVERTED = ["Q5_0", "IQ4_NL"]


@pytest.mark.parametrize("type_name", CONVERTED)
@pytest.mark.parametrize("n,k,rows", [(48, 256, 1), (100, 1568, 3), (7, 96, 4), (300, 1024, 16), (520, 512, 64), (100, 512, 200),
                                      (1000, 768, 129)])
def test_converted_formats_every_kernel_family(cuda_device, type_name, n, k, rows):
    """Q5_0 and IQ4_NL weights (src/Sharplight.Cpu/IntDot.Decode.cs:101-123, 225-238) through the mat-vec, the skinny
    kernel and the GEMM: y against the oracle's integer-dot MatMul of the uploaded format, and the int32 block dots -- in the
    reference's unsigned-code convention for that format -- bit for bit."""
    _, kern = check_matmul(cuda_device, type_name, n, k, rows, seed=n + k + rows)
    assert kern[0] == (N.KERNEL_MMVQ if rows <= 2 else N.KERNEL_MMQ if rows > 64 else kern[0])
    assert cuda_device.last_status() == 0


@pytest.mark.parametrize("type_name", CONVERTED)
def test_converted_formats_f32_activations_and_shape(cuda_device, type_name):
    """The f32-activation mat-vec on a converted weight against the exact product of the dequantized weight (atol 2e-3,
    rtol 1e-4); the handle reports the uploaded format and refuses a download."""
    n, k, rows = 100, 1024, 3
    blocks = synth.weight_blocks(type_name, n, k, seed=77)
    x = synth.activations(rows, k, seed=78)
    w = cuda_device.upload_weight(type_name, (n, k), blocks)
    op = MatMulOp(cuda_device, w, rows, f32_activations=True)
    try:
        y = op.run(x)
        exact = sl_oracle.matmul_f64(FMT_OF[type_name], blocks, n, k, x, threads=4)
        assert np.all(np.abs(y - exact) <= 2e-3 + 1e-4 * np.abs(exact)), float(np.max(np.abs(y - exact)))
        fmt = C.c_int32(0)
        assert N.load().slc_weight_shape(w.handle, C.byref(fmt), None, None, None) == N.OK
        assert fmt.value == FMT_OF[type_name]
        with pytest.raises(Exception):
            w.download()
    finally:
        op.dispose()
        w.dispose()


@pytest.mark.parametrize("type_name", CONVERTED)
def test_converted_formats_kslice_and_layout_artefact(cuda_device, type_name):
    """The K-slice upload of a row-split shard and the layout artefact of a converted weight: both give the results of a
    plain upload of the same blocks, bit for bit, block dots included (the artefact remembers the uploaded format)."""
    n, k, rows = 64, 1024, 5
    blocks = synth.weight_blocks(type_name, n, k, seed=5)
    x = synth.activations(rows, k, seed=6)
    bs, bb = N.BLOCK[FMT_OF[type_name]]
    k0, k1 = 256, 768
    sliced = np.ascontiguousarray(blocks.reshape(n, k // bs, bb)[:, k0 // bs:k1 // bs]).reshape(-1)
    wh = C.c_void_p()
    assert N.load().slc_weight_upload_kslice(cuda_device.handle, FMT_OF[type_name], n, k, blocks.ctypes.data_as(C.c_void_p),
                                             blocks.size, k0, k1, C.byref(wh)) == N.OK
    from sharplight_b200.provider import DeviceWeight
    ws = DeviceWeight(cuda_device, FMT_OF[type_name], n, k1 - k0, wh.value)
    wr = cuda_device.upload_weight(type_name, (n, k1 - k0), sliced)
    wa = cuda_device.import_weight_layout(wr.export_layout())
    ops = [MatMulOp(cuda_device, w, rows) for w in (ws, wr, wa)]
    try:
        xs = np.ascontiguousarray(x[:, k0:k1])
        ys = [op.run(xs) for op in ops]
        assert np.array_equal(ys[0].view(np.uint32), ys[1].view(np.uint32))
        assert np.array_equal(ys[2].view(np.uint32), ys[1].view(np.uint32))
        _, _, s32 = sl_oracle.matmul_intdot(FMT_OF[type_name], sliced, n, k1 - k0, xs, threads=4, want_s32=True)
        for op in ops:
            assert np.array_equal(op.block_dots(xs), s32)
    finally:
        for op in ops:
            op.dispose()
        for w in (ws, wr, wa):
            w.dispose()


# ---- Q5_K: split at upload into two Q4_K weights (nibbles; fifth bits with d' = 16 d), the second product added ----------

@pytest.mark.parametrize("n,k,rows", [(48, 256, 1), (100, 1536, 3), (7, 512, 4), (300, 1024, 16), (520, 512, 64), (100, 512, 200),
                                      (1000, 768, 129), (4112, 512, 2), (64, 14336, 32), (40, 28672, 2), (24, 65536, 1),
                                      (24, 98304, 2)])
def test_q5_k_every_kernel_family(cuda_device, n, k, rows):
    """Q5_K (src/Sharplight.Cpu/IntDot.Decode.cs:150-176) through the mat-vec, the skinny kernel (K chunks included) and
    the GEMM: y against the oracle's integer-dot MatMul of the Q5_K blocks, the int32 block dots of the 5-bit codes bit for
    bit (dots of the nibbles + 16 x dots of the fifth bits)."""
    _, kern = check_matmul(cuda_device, "Q5_K", n, k, rows, seed=n + k + rows)
    assert kern[0] == (N.KERNEL_MMVQ if rows <= 2 else N.KERNEL_MMQ if rows > 64 else kern[0])
    assert cuda_device.last_status() == 0


def test_q5_k_other_entry_points(cuda_device):
    """The f32-activation mat-vec, an epilogue (bias and residual stay counted once), a K-slice shard, the no-allocation
    entry point and the refusals (download, layout artefact, dual MatMul) on a Q5_K weight."""
    n, k, rows = 96, 1024, 3
    fmt = FMT_OF["Q5_K"]
    blocks = synth.weight_blocks("Q5_K", n, k, seed=31)
    x = synth.activations(rows, k, seed=32)
    w = cuda_device.upload_weight("Q5_K", (n, k), blocks)
    opf = MatMulOp(cuda_device, w, rows, f32_activations=True)
    op = MatMulOp(cuda_device, w, rows)
    try:
        exact = sl_oracle.matmul_f64(fmt, blocks, n, k, x, threads=4)
        yf = opf.run(x)
        assert np.all(np.abs(yf - exact) <= 2e-3 + 1e-4 * np.abs(exact)), float(np.max(np.abs(yf - exact)))
        ref, _, _ = sl_oracle.matmul_intdot(fmt, blocks, n, k, x, threads=4)
        y = op.run(x)
        assert max_rel_error(y, ref) <= MAX_REL
        # the no-allocation entry point gives the same rows
        import torch
        xd = torch.from_numpy(x).cuda()
        yd = torch.zeros((rows, n), device="cuda", dtype=torch.float32)
        assert N.load().slc_matmul_run_static(w.handle, C.c_void_p(xd.data_ptr()), N.F32, rows, k, C.c_void_p(yd.data_ptr()), n,
                                              None) == N.OK
        torch.cuda.synchronize()
        assert max_rel_error(yd.cpu().numpy(), ref) <= MAX_REL
        # K-slice shard == upload of the sliced blocks
        k0, k1 = 256, 768
        sliced = np.ascontiguousarray(blocks.reshape(n, k // 256, 176)[:, k0 // 256:k1 // 256]).reshape(-1)
        wh = C.c_void_p()
        assert N.load().slc_weight_upload_kslice(cuda_device.handle, fmt, n, k, blocks.ctypes.data_as(C.c_void_p), blocks.size,
                                                 k0, k1, C.byref(wh)) == N.OK
        from sharplight_b200.provider import DeviceWeight
        ws = DeviceWeight(cuda_device, fmt, n, k1 - k0, wh.value)
        wr = cuda_device.upload_weight("Q5_K", (n, k1 - k0), sliced)
        a, b = MatMulOp(cuda_device, ws, rows), MatMulOp(cuda_device, wr, rows)
        try:
            xs = np.ascontiguousarray(x[:, k0:k1])
            assert np.array_equal(a.run(xs).view(np.uint32), b.run(xs).view(np.uint32))
        finally:
            a.dispose(); b.dispose(); ws.dispose(); wr.dispose()
        with pytest.raises(Exception):
            w.download()
        with pytest.raises(Exception):
            w.export_layout()
    finally:
        op.dispose()
        opf.dispose()
        w.dispose()
