"""The CPU oracle against the reference's golden vectors and known-answer cases (no GPU).

Mirrors tests/Sharplight.Cpu.Tests/GgmlDequantTests.cs:155-183, IntDotTests.cs:46-185 and QuantTests.cs:119-128,
208-266 of the Sharplight tree.
"""
import numpy as np
import pytest

from helpers import FMT_OF, TYPE_OF, np_oracle, relative_rms, same_floats, sl_oracle
from sharplight_b200 import synth

RECORDS = ([f"ext_{t}_{kind}" for t in (2, 6, 8, 12, 13, 14, 20) for kind in ("ggml", "random")] +
           [f"src_{t}" for t in (2, 6, 8, 12, 13, 14)])


def _record(golden, name):
    tid, rows, cols = (int(v) for v in golden[name + "_shape"])
    return tid, rows, cols, golden[name + "_blocks"], golden[name + "_expected"].reshape(rows, cols)


@pytest.mark.parametrize("name", RECORDS)
def test_dequantize_matches_ggml(golden, name):
    """GgmlDequantTests.MatchesGgmlDecoder: the reference allows 1e-5 for these FMA-fused types; the oracle's values are
    equal to ggml's (only the sign of zero may differ), and the two restatements agree bit for bit."""
    tid, rows, cols, blocks, expected = _record(golden, name)
    got = sl_oracle.dequantize(tid, blocks, rows, cols)
    assert same_floats(got, expected)
    got_np = np_oracle.dequantize(tid, blocks, rows, cols)
    assert same_floats(got_np, expected)
    finite = np.isfinite(expected)
    assert np.array_equal(got.view(np.uint32)[finite], got_np.view(np.uint32)[finite])


@pytest.mark.parametrize("name", [r for r in RECORDS if not r.endswith("random")])
def test_decode_matches_dequantize(golden, name):
    """IntDotTests.DecodeMatchesDequantize: a*u + b reproduces ggml's values within 1e-6*|e| + 1e-7, small-code
    formats stay below 128."""
    tid, rows, cols, blocks, expected = _record(golden, name)
    u, a, b = sl_oracle.decode(tid, blocks, rows, cols)
    if tid not in (8, 20):
        assert u.max() < 128
    actual = np.repeat(a, 16, axis=1) * u.astype(np.float32) + np.repeat(b, 16, axis=1)
    assert np.all(np.abs(expected - actual) <= 1e-6 * np.abs(expected) + 1e-7)
    u2, a2, b2 = np_oracle.codes(tid, blocks, rows, cols)
    assert np.array_equal(u, u2.astype(np.uint8))
    assert np.array_equal(a.view(np.uint32), a2.view(np.uint32))
    assert np.array_equal(b.view(np.uint32), b2.view(np.uint32))


def quantize_kat():
    """The input of IntDotTests.QuantizeMatchesReference: K = 288, block 1 all zero, block 2 exact halves after
    scaling, a 1e-30 and a -1e30 outlier."""
    x = synth.activations(1, 288, 3)[0] * 4.0
    x[32:64] = 0.0
    x[64:96] = (np.arange(64, 96) - 80) * 0.5
    x[100] = 1e-30
    x[130] = -1e30
    return x.astype(np.float32)[None, :]


def test_quantize_known_answers():
    x = quantize_kat()
    q, d, gs = sl_oracle.quantize(x)
    q2, d2, gs2 = np_oracle.quantize(x)
    assert np.array_equal(q, q2)
    assert np.array_equal(d.view(np.uint32), d2.view(np.uint32))
    assert np.array_equal(gs.view(np.uint32), gs2.view(np.uint32))
    # all-zero block: zero scale, zero codes
    assert d[0, 1] == 0 and not q[0, 32:64].any() and not gs[0, 2:4].any()
    # exact halves: amax = 8 -> x * (127 / 8) lands on k + 0.5 for odd multiples; half away from zero
    assert d[0, 2] == np.float32(8.0) / np.float32(127.0)
    assert q[0, 64] == -127 and q[0, 80] == 0
    v = (x[0, 64:96] * (np.float32(1.0) / d[0, 2])).astype(np.float32)
    expect = np.trunc(v + np.copysign(np.float32(0.5), v)).astype(np.int8)
    assert np.array_equal(q[0, 64:96], expect)
    assert q[0, 81] == 8 and q[0, 79] == -8           # 7.9375 -> 8: halves round away from zero
    # outliers: the block holding -1e30 quantizes everything else to zero, the outlier to -127
    blk = 130 // 32
    assert q[0, 130] == -127 and np.count_nonzero(q[0, blk * 32:(blk + 1) * 32]) == 1
    assert q[0, 100] == 0
    # group sums are d * sum16(q)
    s16 = q.astype(np.int32).reshape(1, -1, 16).sum(-1)
    assert np.array_equal(gs, (np.repeat(d, 2, axis=1) * s16.astype(np.float32)).astype(np.float32))
    assert np.abs(q.astype(np.int32)).max() <= 127


@pytest.mark.parametrize("small", [True, False])
def test_scalar_dot_matches_double_reference(small):
    """IntDotTests.ScalarDotMatchesDoubleReference: within 1e-5 of the magnitude."""
    k = 1024
    g = np.random.Generator(np.random.Philox(5 + small))
    u = g.integers(0, 128 if small else 256, k).astype(np.uint8)
    a = (g.standard_normal(k // 16) * 0.01).astype(np.float32)
    b = (g.standard_normal(k // 16) * 0.5).astype(np.float32)
    x = (g.standard_normal((1, k)) * 2).astype(np.float32)
    q, d, gs = sl_oracle.quantize(x)
    L = sl_oracle.lib()
    got = L.slo_dot_scalar(u.ctypes.data, a.ctypes.data, b.ctypes.data, q.ctypes.data, d.ctypes.data, gs.ctypes.data, k)
    w = np.repeat(a, 16).astype(np.float64) * u + np.repeat(b, 16)
    xv = np.repeat(d[0], 32).astype(np.float64) * q[0]
    assert abs(got - np.sum(w * xv)) <= 1e-5 * np.sum(np.abs(w * xv))


def _raw_constant(fmt, n, k, code):
    """Q8_0 blocks whose unsigned codes all equal `code` (IntDotTests.TierMatchesScalar's saturation cases)."""
    nb = n * k // 32
    blk = np.zeros((nb, 34), np.uint8)
    blk[:, 0:2] = np.array([0.01], np.float16).view(np.uint8)
    blk[:, 2:] = np.uint8(code ^ 0x80)
    return blk.reshape(-1)


@pytest.mark.parametrize("code,act", [(255, 1.0), (255, -1.0), (128, -1.0), (127, 1.0)])
def test_fast_tier_matches_scalar_on_extremes(code, act):
    n, k = 3, 512
    w = _raw_constant(8, n, k, code)
    x = np.full((2, k), act, np.float32)
    y0, y64, _ = sl_oracle.matmul_intdot(8, w, n, k, x, tier=0, want_f64=True)
    y1, _, _ = sl_oracle.matmul_intdot(8, w, n, k, x, tier=1, threads=2)
    mag = 0.01 * max(abs(code - 128), 1) * k * abs(act) + 0.01 * 128 * k
    assert np.all(np.abs(y0 - y1) <= 2e-6 * mag + 1e-6)
    assert np.all(np.abs(y0 - y64) <= 1e-5 * mag)


@pytest.mark.parametrize("type_name", ["Q8_0", "Q4_0", "Q4_K", "Q6_K"])
@pytest.mark.parametrize("k", [256, 512 + 256, 4096])
def test_fast_tier_matches_scalar(type_name, k):
    """Every tier sums the same integers; only the f32 order differs (2e-6 of the magnitude, as the reference)."""
    n, m = 5, 3
    w = synth.weight_blocks(type_name, n, k, seed=k)
    x = synth.activations(m, k, seed=k + 1)
    fmt = FMT_OF[type_name]
    y0, y64, s0 = sl_oracle.matmul_intdot(fmt, w, n, k, x, tier=0, want_f64=True, want_s32=True)
    y1, _, s1 = sl_oracle.matmul_intdot(fmt, w, n, k, x, tier=1, threads=3, want_s32=True)
    assert np.array_equal(s0, s1)
    u, a, b = sl_oracle.decode(fmt, w, n, k)
    q, d, _ = sl_oracle.quantize(x)
    mag = np.einsum("nk,mk->mn", np.abs(np.repeat(a, 16, 1) * u) + np.abs(np.repeat(b, 16, 1)),
                    np.abs(np.repeat(d, 32, 1) * q))
    assert np.all(np.abs(y0 - y1) <= 2e-6 * mag + 1e-6)
    assert np.all(np.abs(y0 - y64) <= 1e-5 * mag)
    assert np.array_equal(s0, np_oracle.block_dots(u, q))
    assert np.allclose(y64, np_oracle.matmul_intdot_f64(fmt, w, n, k, x), rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("type_name", ["Q8_0", "Q4_0", "Q4_K", "Q6_K"])
@pytest.mark.parametrize("k", [1536 + 32, 2560, 1024])
def test_intdot_matmul_close_to_exact_product(type_name, k):
    """QuantTests.MatMulWithIntDotMatchesReference: N = 7, T in {1, 3, 16}: the 8-bit-activation result stays within
    1e-2 relative RMS of the exact product with the dequantized weight."""
    if type_name in ("Q4_K", "Q6_K") and k % 256:
        k = 1536
    n = 7
    fmt = FMT_OF[type_name]
    w = synth.weight_blocks(type_name, n, k, seed=11)
    ys, exacts = [], []
    for t in (1, 3, 16):
        x = synth.activations(t, k, seed=100 + t)
        y, _, _ = sl_oracle.matmul_intdot(fmt, w, n, k, x)
        exact = sl_oracle.matmul_f64(fmt, w, n, k, x)
        # seven outputs of uniformly random codes are a noisy sample: 2.5e-2 per call, 1e-2 over the pooled rows
        assert relative_rms(y, exact) < 2.5e-2
        ys.append(y)
        exacts.append(exact)
    assert relative_rms(np.concatenate(ys), np.concatenate(exacts)) < 1e-2


def test_golden_rows_through_the_intdot_path(golden):
    """The ggml-quantized fixture rows as weights: integer-dot output vs the double product of ggml's own floats
    (GgmlDequantTests.MatMulMatchesDequantizedProduct uses T in {1, 5})."""
    for tid in (2, 8, 12, 14):
        _, rows, cols, blocks, expected = _record(golden, f"ext_{tid}_ggml")
        for t in (1, 5):
            x = synth.exact_int8_activations(t, cols, seed=tid + t)
            y, y64, _ = sl_oracle.matmul_intdot(tid, blocks, rows, cols, x, want_f64=True)
            ref = x.astype(np.float64) @ expected.astype(np.float64).T
            assert np.all(np.abs(y64 - ref) <= 2e-3 + 1e-4 * np.abs(ref)), TYPE_OF[tid]
            assert np.all(np.abs(y - ref) <= 2e-3 + 1e-4 * np.abs(ref)), TYPE_OF[tid]


def test_empty_and_bad_shapes():
    assert sl_oracle.lib().slo_dequantize_row(12, None, 100, None) == -1   # K not a multiple of 256
    assert sl_oracle.lib().slo_decode_row(99, None, 32, None, None, None) == -1
    y, _, _ = sl_oracle.matmul_intdot(8, np.zeros(0, np.uint8), 0, 32, np.zeros((2, 32), np.float32))
    assert y.shape == (2, 0)


# ---- the reference's CPU drivers: chunked integer dots on the worker pool, f32 GEMM from 32 rows ---------------------

@pytest.mark.parametrize("fmt_name", ["Q8_0", "Q4_0", "Q4_K", "Q6_K"])
def test_pooled_intdot_equals_the_plain_driver(fmt_name):
    """Chunking and the worker pool change who computes a row, not what is computed."""
    from sharplight_b200 import synth
    fmt = {"Q4_0": 2, "Q8_0": 8, "Q4_K": 12, "Q6_K": 14}[fmt_name]
    n, k, m = 203, 1024, 5
    blocks = synth.weight_blocks(fmt_name, n, k, 11)
    x = synth.activations(m, k, 12)
    plain, _, _ = sl_oracle.matmul_intdot(fmt, blocks, n, k, x, threads=3, tier=1)
    for threads in (1, 4, 7):
        pooled = sl_oracle.matmul_intdot_pooled(fmt, blocks, n, k, x, threads=threads)
        assert np.array_equal(plain.view(np.uint32), pooled.view(np.uint32))


@pytest.mark.parametrize("fmt_name", ["Q8_0", "Q4_0", "Q4_K", "Q6_K"])
@pytest.mark.parametrize("n,k,m", [(37, 512, 32), (70, 768, 45), (33, 256, 64)])
def test_gemm_path_matches_the_exact_product(fmt_name, n, k, m):
    """MatMulOp.RunGemm restated: within atol 2e-3 / rtol 1e-4 of the double-precision product of the dequantized weight
    with the f32 activations (the tolerance of the reference's float MatMul tests, tests/Sharplight.Cpu.Tests/QuantTests.cs:257-265
    compare the integer-dot result with the same product at 1e-2 relative RMS), and identical for every thread count."""
    from sharplight_b200 import synth
    fmt = {"Q4_0": 2, "Q8_0": 8, "Q4_K": 12, "Q6_K": 14}[fmt_name]
    blocks = synth.weight_blocks(fmt_name, n, k, n + k)
    x = synth.activations(m, k, m)
    exact = sl_oracle.matmul_f64(fmt, blocks, n, k, x, threads=4)
    y1 = sl_oracle.matmul_gemm(fmt, blocks, n, k, x, threads=1)
    assert np.all(np.abs(y1 - exact) <= 2e-3 + 1e-4 * np.abs(exact))
    for threads in (3, 8):
        assert np.array_equal(y1.view(np.uint32), sl_oracle.matmul_gemm(fmt, blocks, n, k, x, threads=threads).view(np.uint32))
    # the sequential fused multiply-add chain over k, spelled out for a few outputs
    w = sl_oracle.dequantize(fmt, blocks, n, k)
    for (t, r) in [(0, 0), (m - 1, n - 1), (m // 2, n // 3)]:
        acc = np.float32(0)
        for i in range(k):
            acc = np.float32(np.float64(x[t, i]) * np.float64(w[r, i]) + np.float64(acc))   # exact product, one rounding
        assert acc == y1[t, r]


def test_run_dispatch_switches_at_32_rows():
    from sharplight_b200 import synth
    n, k = 48, 512
    blocks = synth.weight_blocks("Q4_K", n, k, 5)
    x = synth.activations(40, k, 6)
    assert np.array_equal(sl_oracle.matmul_run(12, blocks, n, k, x[:31], threads=4),
                          sl_oracle.matmul_intdot_pooled(12, blocks, n, k, x[:31], threads=4))
    assert np.array_equal(sl_oracle.matmul_run(12, blocks, n, k, x[:32], threads=4),
                          sl_oracle.matmul_gemm(12, blocks, n, k, x[:32], threads=4))
