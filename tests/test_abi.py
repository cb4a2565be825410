"""The C-ABI boundary and the host logic that need no GPU: the library loads, exports exactly what the header
declares, reports errors by code, and the provider stays quiet on a machine without a device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from sharplight_b200 import native as N
from sharplight_b200 import provider as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            names += re.findall(r"SLC_API\s+[\w\s\*]+?\b(slc_\w+)\s*\(", text)
    return names


def test_library_exports_every_declared_symbol():
    lib = N.load()
    declared = header_symbols()
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    assert set(declared) == set(N.SIGNATURES), "binding and header disagree"


def test_abi_version_and_strings():
    lib = N.load()
    assert lib.slc_abi_version() == N.ABI_VERSION
    assert b"sharplight" in lib.slc_version_string()
    for code in range(0, -9, -1):
        assert lib.slc_error_string(code)
    assert lib.slc_error_string(-100) == b"unknown error"


def test_argument_checks_need_no_device():
    lib = N.load()
    assert lib.slc_device_count(None) == N.ERR_INVALID_ARGUMENT
    assert lib.slc_device_open(0, None) == N.ERR_INVALID_ARGUMENT
    h = C.c_void_p()
    assert lib.slc_weight_upload(None, N.FMT_Q8_0, 1, 32, None, 34, C.byref(h)) == N.ERR_INVALID_ARGUMENT
    assert lib.slc_matmul_create(None, None, 1, 0, C.byref(h)) == N.ERR_INVALID_ARGUMENT
    assert lib.slc_matmul_run(None, None, 0, 1, 32, 0, None, 1, 0, None) == N.ERR_INVALID_ARGUMENT
    assert lib.slc_last_error_message()
    # destroying nothing is allowed
    lib.slc_weight_free(None)
    lib.slc_matmul_destroy(None)
    lib.slc_activation_destroy(None)
    lib.slc_device_close(None)


def _has_gpu():
    c = C.c_int32(0)
    return N.load().slc_device_count(C.byref(c)) == N.OK and c.value > 0


def test_provider_without_device_reports_unavailable():
    """CheckAvailability never throws and GetDevices is empty when the provider cannot run
    (ExecutionProviderCatalog.cs:28-47 of the Sharplight tree); there is no CPU fallback behind it."""
    prov = P.CudaExecutionProvider()
    a = prov.check_availability()
    if _has_gpu():
        pytest.skip("a CUDA device is present")
    assert a.available is False and a.reason
    assert prov.get_devices() == []
    fake = P.DeviceInfo("cuda", 0, "none", "DiscreteGpu", 0, "NVIDIA", "", b"", P.FEATURES, 0)
    with pytest.raises(P.NotSupportedError):
        prov.open_device(fake)
    with pytest.raises(P.ArgumentError):
        prov.open_device(P.DeviceInfo("cpu", 0, "x", "Cpu", 0, "", "", b"", frozenset(), 0))
    c = C.c_int32(7)
    assert N.load().slc_device_count(C.byref(c)) == N.ERR_NO_DEVICE and c.value == 0
    h = C.c_void_p()
    assert N.load().slc_device_open(0, C.byref(h)) == N.ERR_NO_DEVICE and not h.value


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(N, "_lib", None)
    monkeypatch.setattr(N, "LIB_PATH", "/nonexistent/libsharplight_cuda.so")
    with pytest.raises(FileNotFoundError):
        N.load()
    assert P.CudaExecutionProvider().check_availability().available is False


def _bare_device(disabled=(), allow_reduced_precision=False):
    d = object.__new__(P.CudaDevice)
    d.enabled_features = frozenset(P.FEATURES - frozenset(disabled))
    d.allow_reduced_precision = allow_reduced_precision
    return d


def test_supports_mirrors_the_quantized_matmul_check():
    """CpuOpSupport.CheckQuantizedMatMul (src/Sharplight.Cpu/CpuOpSupport.Linear.cs:21-53): format, K alignment."""
    d = _bare_device()
    blocks = np.zeros(34, np.uint8)
    ok = P.MatMulNode("m", "x", P.WeightInfo("Q8_0", (1, 32), blocks), "y")
    assert d.supports(ok).supported
    assert not d.supports(P.MatMulNode("m", "x", P.WeightInfo("Q4_1", (1, 256), blocks), "y")).supported
    bad_k = d.supports(P.MatMulNode("m", "x", P.WeightInfo("Q4_K", (1, 288), blocks), "y"))
    assert not bad_k.supported and "multiple" in bad_k.reason
    assert not d.supports(P.MatMulNode("m", "x", P.WeightInfo("Q8_0", (1, 32), blocks), "y", x_dtype="f16")).supported
    assert not d.supports("Softmax").supported
    assert not _bare_device(["int_dot"]).supports(ok).supported


def test_supports_honours_the_f32_activation_opt_out():
    """A MatMul node may opt out of 8-bit activations (src/Sharplight.Core/Graph/StandardOps.cs:130-135); the reference
    then keeps f32 activations unless reduced precision is allowed (src/Sharplight.Shaders/Lowering/
    GraphLowerer.IntDot.cs:61-62, src/Sharplight.Cpu/CpuCompiledSegment.LowerLinear.cs:39). Such a node is taken for the
    dequant-fused f32 mat-vec (never silently quantized), as long as one f32 activation row fits that kernel's shared
    memory; beyond that it is refused and goes to the placement fallback."""
    blocks = np.zeros(34, np.uint8)
    node = P.MatMulNode("m", "x", P.WeightInfo("Q8_0", (1, 32), blocks), "y", f32_activations=True)
    assert _bare_device().supports(node).supported
    long_k = P.MatMulNode("m", "x", P.WeightInfo("Q8_0", (1, 65536), None), "y", f32_activations=True)
    no = _bare_device().supports(long_k)
    assert not no.supported and "f32 activations" in no.reason
    assert _bare_device(allow_reduced_precision=True).supports(long_k).supported


def test_bf16_helpers_round_trip():
    x = np.array([0.0, 1.0, -2.5, 3.1415927, 1e-3, 65504.0], np.float32)
    b = P.to_bf16_bits(x)
    back = P.bf16_bits_to_f32(b)
    assert np.all(np.abs(back - x) <= np.abs(x) * 2.0 ** -8)
    assert np.array_equal(P.to_bf16_bits(back), b)


def test_managed_pinvoke_list_covers_the_header():
    """Every export of include/sharplight_cuda.h has its [LibraryImport] in the managed provider's NativeMethods.cs (the
    C# sources are not compiled in this image: this at least keeps the list complete and free of stale names)."""
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = open(os.path.join(root, "include", "sharplight_cuda.h")).read()
    managed = open(os.path.join(root, "sharplight_b200", "Sharplight.Cuda", "Native", "NativeMethods.cs")).read()
    exported = set(re.findall(r"SLC_API\s+[\w\s\*]+?\b(slc_[a-z0-9_]+)\s*\(", header))
    imported = set(re.findall(r"static partial [\w\*]+ (slc_[a-z0-9_]+)\(", managed))
    assert exported and exported == imported, (sorted(exported - imported), sorted(imported - exported))


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` (the restated reference CPU path on the host cores) runs without a GPU and prints one
    JSON line with the keys the measurement contract names, on the same metric, unit and workload as the GPU arm."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and line["metric"] == "quant MatMul weight GB/s" and line["unit"] == "GB/s"
    assert line["higher_is_better"] is True and line["value"] > 0 and line["n_gpus"] == 1
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1 and line["cpu_baseline"]["sample"]
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "70B" in line["config"]["workload"]
