"""Host side of the CUDA execution provider, mirroring the reference's provider contract for the MatMul path.

The managed provider (Sharplight.Cuda) is C#; this module is the same surface in Python over the same C ABI, so the
parity tests read like the reference's own: ``CudaExecutionProvider`` (IExecutionProvider,
src/Sharplight.Core/Runtime/IExecutionProvider.cs:25-74 of the Sharplight tree), ``CudaDevice`` (IComputeDevice,
IComputeDevice.cs:6-67), ``CudaSegment`` (ICompiledSegment, ICompiledSegment.cs:6-25) and ``MatMulOp`` (the CPU
provider's operator, src/Sharplight.Cpu/MatMulOp.cs:88-160). Names, argument meaning and error behaviour follow the
reference; .NET exception types map to the classes below.

Everything computes on the GPU through libsharplight_cuda.so. Nothing here falls back to the CPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import native as N


class ArgumentError(ValueError):
    """System.ArgumentException."""


class InvalidOperationError(RuntimeError):
    """System.InvalidOperationException."""


class ObjectDisposedError(InvalidOperationError):
    """System.ObjectDisposedException."""


class NotSupportedError(NotImplementedError):
    """System.NotSupportedException."""


class InsufficientMemoryError(MemoryError):
    """System.InsufficientMemoryException."""


_EXC = {N.ERR_INVALID_ARGUMENT: ArgumentError, N.ERR_OUT_OF_MEMORY: InsufficientMemoryError,
        N.ERR_UNSUPPORTED: NotSupportedError, N.ERR_INVALID_STATE: InvalidOperationError,
        N.ERR_NO_DEVICE: NotSupportedError}


def _check_graph(code: int) -> None:
    """Result check for the stream / graph group, which reports through slc_graph_last_error."""
    if code < 0:
        raise N.NativeError(code, N.load().slc_graph_last_error().decode() or "stream / graph call failed")


def _check(code: int) -> None:
    """Native result -> the exception the managed wrapper throws."""
    if code >= 0:
        return
    lib = N.load()
    detail = lib.slc_last_error_message().decode() or lib.slc_error_string(code).decode()
    raise _EXC.get(code, N.NativeError)(detail) if code in _EXC else N.NativeError(code, detail)


DATA_TYPES = {"Q4_0": N.FMT_Q4_0, "Q8_0": N.FMT_Q8_0, "Q4_K": N.FMT_Q4_K, "Q6_K": N.FMT_Q6_K, "Q5_0": N.FMT_Q5_0,
              "IQ4_NL": N.FMT_IQ4_NL, "Q5_K": N.FMT_Q5_K}

# DeviceFeatures names the device reports (src/Sharplight.Core/Runtime/DeviceFeatures.cs:28,54)
FEATURES = frozenset({"int_dot", "matrix_int8", "subgroup_ops", "fp16", "bf16"})


@dataclass(frozen=True)
class ProviderAvailability:
    available: bool
    reason: str = ""


@dataclass(frozen=True)
class DeviceInfo:
    """The fields of src/Sharplight.Core/Runtime/DeviceInfo.cs:4-50 this provider fills."""
    provider: str
    index: int
    name: str
    kind: str
    total_memory: int
    vendor: str
    driver: str
    uuid: bytes
    features: frozenset
    concurrent_workgroups: int
    sm_count: int = 0
    compute_capability: tuple = (0, 0)


@dataclass(frozen=True)
class OpSupport:
    supported: bool
    reason: str = ""

    @staticmethod
    def yes() -> "OpSupport":
        return OpSupport(True)

    @staticmethod
    def no(reason: str) -> "OpSupport":
        return OpSupport(False, reason)


@dataclass
class WeightInfo:
    """A static weight as the importer describes it: type name, shape [N, K], raw ggml blocks."""
    type: str
    shape: Sequence[int]
    blocks: Optional[np.ndarray]
    resident: Optional["DeviceWeight"] = None   # already on the device (a weight shared between segments): not uploaded again


@dataclass
class MatMulNode:
    """StandardOps.MatMul (src/Sharplight.Core/Graph/StandardOps.cs:144-163): y = x . W^T."""
    name: str
    x: str                     # input value name, f32 or bf16 [T, K]
    weight: WeightInfo
    y: str                     # output value name, f32 [T, N]
    x_dtype: str = "f32"
    f32_activations: bool = False   # StandardOps.cs:130-135: the node opts out of 8-bit activations
    allreduce: bool = False         # tensor parallelism: the node is row-split, its output is summed over the ranks


@dataclass
class ViewNode:
    """A node of OpCategory.View in front of a MatMul (Reshape, Slice, Permute: src/Sharplight.Core/Graph/StandardOps.cs:61,68,89).
    The placement planner does not ask providers about such nodes, they stay on their group's device
    (src/Sharplight.Core/Runtime/PlacementPlanner.cs:238), so the segment has to take them. x is a [T, x_cols] value.
      kind "slice":   y = x[:, start : start + length]                      -- a pointer and a row stride, nothing moves
      kind "reshape": y = x seen as [T * split, x_cols / split]             -- the same bytes, more and shorter rows
      kind "permute": y[t] = x[t] seen as [a, b] and transposed to [b, a]   -- rows are no longer runs of memory: gathered
                      into a dense buffer first, as the reference's lowering densifies such an input
                      (src/Sharplight.Shaders/Lowering/GraphLowerer.MatMul.cs:117-126)"""
    name: str
    x: str
    y: str
    kind: str
    x_cols: int
    dtype: str = "f32"
    start: int = 0
    length: int = 0
    split: int = 1
    a: int = 0
    b: int = 0


@dataclass
class GraphSegment:
    nodes: List[object]          # MatMulNode and ViewNode, in execution order
    inputs: List[str]
    outputs: List[str]


@dataclass
class CompileOptions:
    """The knobs of src/Sharplight.Core/Runtime/CompileOptions.cs:4-60 the MatMul path reads."""
    max_rows: int = 1                       # bound of the symbolic row count T
    disabled_features: frozenset = frozenset()
    allow_reduced_precision: bool = False
    row_invariant_rows: int = 0
    capture_steps: bool = True              # replay Execute as a captured CUDA graph from the third call per row count
    exchange: Optional["TpExchange"] = None  # tensor parallelism: the receive area through which allreduce nodes sum


class CudaExecutionProvider:
    """IExecutionProvider "cuda". Cheap to construct; touches the driver only in check_availability / get_devices."""

    name = "cuda"
    portable_code_format = None   # kernels are compiled ahead of time into the shared library

    def __init__(self):
        self._disposed = False

    def check_availability(self) -> ProviderAvailability:
        """Never raises (the catalog wraps providers the same way, ExecutionProviderCatalog.cs:28-47)."""
        try:
            lib = N.load()
            count = C.c_int32(0)
            rc = lib.slc_device_count(C.byref(count))
            if rc != N.OK:
                return ProviderAvailability(False, lib.slc_last_error_message().decode())
            for i in range(count.value):
                info = N.DeviceInfoStruct()
                if lib.slc_device_info_get(i, C.byref(info)) == N.OK and info.supported:
                    return ProviderAvailability(True)
            return ProviderAvailability(False, "no compute-capability 10.0 device")
        except Exception as e:  # library missing, ABI mismatch
            return ProviderAvailability(False, str(e))

    def get_devices(self) -> List[DeviceInfo]:
        if not self.check_availability().available:
            return []
        lib = N.load()
        count = C.c_int32(0)
        _check(lib.slc_device_count(C.byref(count)))
        out = []
        for i in range(count.value):
            s = N.DeviceInfoStruct()
            _check(lib.slc_device_info_get(i, C.byref(s)))
            if not s.supported:
                continue
            out.append(DeviceInfo("cuda", i, s.name.decode(), "DiscreteGpu", s.total_memory, "NVIDIA",
                                  s.driver.decode(), bytes(s.uuid), FEATURES, s.concurrent_workgroups,
                                  s.sm_count, (s.cc_major, s.cc_minor)))
        return out

    def open_device(self, device: DeviceInfo, options: Optional[dict] = None) -> "CudaDevice":
        if self._disposed:
            raise ObjectDisposedError("CudaExecutionProvider")
        if device.provider != self.name:
            raise ArgumentError(f"device belongs to provider '{device.provider}'")
        if not self.check_availability().available:
            raise NotSupportedError("the CUDA provider is unavailable")
        return CudaDevice(device, options or {})

    def can_compile_for(self, profile) -> bool:
        return False

    def dispose(self) -> None:
        self._disposed = True


class DeviceWeight:
    """A weight resident on the device (slc_weight)."""

    def __init__(self, device: "CudaDevice", fmt: int, n: int, k: int, handle: int):
        self.device, self.format, self.n, self.k, self._h = device, fmt, n, k, C.c_void_p(handle)

    @property
    def handle(self):
        if self._h is None:
            raise ObjectDisposedError("DeviceWeight")
        return self._h

    @property
    def device_bytes(self) -> int:
        b = C.c_int64(0)
        _check(N.load().slc_weight_shape(self.handle, None, None, None, C.byref(b)))
        return b.value

    def download(self) -> np.ndarray:
        bs, bb = N.BLOCK[self.format]
        out = np.empty(self.n * (self.k // bs) * bb, np.uint8)
        _check(N.load().slc_weight_download(self.handle, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def export_layout(self) -> np.ndarray:
        """The device layout as an artefact (header + re-laid-out records) for CudaDevice.import_weight_layout."""
        b = C.c_int64(0)
        _check(N.load().slc_weight_layout_bytes(self.handle, C.byref(b)))
        out = np.empty(b.value, np.uint8)
        _check(N.load().slc_weight_export_layout(self.handle, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def dispose(self) -> None:
        if self._h is not None:
            N.load().slc_weight_free(self._h)
            self._h = None


class CudaDevice:
    """IComputeDevice over one opened GPU (slc_device). Safe to share between threads."""

    def __init__(self, info: DeviceInfo, options: dict):
        self.info = info
        self.options = options
        self.allow_reduced_precision = bool(options.get("allow_reduced_precision", False))
        h = C.c_void_p()
        _check(N.load().slc_device_open(info.index, C.byref(h)))
        self._h = h
        disabled = frozenset(options.get("disabled_features", ()))
        self.enabled_features = frozenset(info.features - disabled)

    @property
    def handle(self):
        if self._h is None:
            raise ObjectDisposedError("CudaDevice")
        return self._h

    @property
    def available_memory(self) -> int:
        free = C.c_int64(0)
        _check(N.load().slc_device_memory(self.handle, C.byref(free), None))
        return free.value

    @property
    def stream(self) -> int:
        """The device's own cudaStream_t."""
        return N.load().slc_device_stream(self.handle) or 0

    def synchronize(self) -> None:
        _check(N.load().slc_device_sync(self.handle))

    def argmax_rows(self, y_device_ptr: int, rows: int, n: int, y_stride: int, out_index_ptr: int, stream: int = 0) -> None:
        """out[t] = index of the first maximum of row t (slc_argmax_rows): the sampling head behind the lm_head."""
        _check(N.load().slc_argmax_rows(self.handle, C.c_void_p(y_device_ptr), rows, n, y_stride, C.c_void_p(out_index_ptr),
                                        C.c_void_p(stream) if stream else None))

    def matmul_id(self, weight: "DeviceWeight", experts: int, x_device_ptr: int, x_dtype: int, x_stride: int, ids_device_ptr: int,
                  tokens: int, slots: int, per_slot: bool, y_device_ptr: int, y_stride: int, stream: int = 0) -> None:
        """MatMulId (slc_matmul_id_run): y[t, s] = W[ids[t, s]] . x[t (, s)] with the experts' matrices uploaded as one
        [experts * N, K] weight; device pointers, asynchronous on the stream."""
        _check(N.load().slc_matmul_id_run(weight.handle, experts, C.c_void_p(x_device_ptr), x_dtype, x_stride,
                                          C.c_void_p(ids_device_ptr), tokens, slots, 1 if per_slot else 0,
                                          C.c_void_p(y_device_ptr), y_stride, C.c_void_p(stream) if stream else None))

    def last_status(self) -> int:
        v = C.c_int32(0)
        _check(N.load().slc_last_status(self.handle, C.byref(v)))
        return v.value

    def supports(self, node) -> OpSupport:
        """Yes only for MatMul with a static Q8_0 / Q4_0 / Q4_K / Q6_K / Q5_0 / Q5_K / IQ4_NL weight whose K is a multiple of the block size
        and activations that may be quantized to 8 bits (mirrors CpuOpSupport.CheckQuantizedMatMul,
        src/Sharplight.Cpu/CpuOpSupport.Linear.cs:21-53); everything else goes to the placement fallback."""
        if not isinstance(node, MatMulNode):
            return OpSupport.no("only MatMul runs on the CUDA provider")
        fmt = DATA_TYPES.get(node.weight.type)
        if fmt is None:
            return OpSupport.no(f"weight type {node.weight.type} has no CUDA kernel")
        if len(node.weight.shape) != 2:
            return OpSupport.no("weight must be [N, K]")
        if node.weight.shape[1] % N.BLOCK[fmt][0] != 0:
            return OpSupport.no(f"K={node.weight.shape[1]} is not a multiple of the {node.weight.type} block size")
        if node.x_dtype not in ("f32", "bf16"):
            return OpSupport.no("activations must be f32 or bf16")
        if "int_dot" not in self.enabled_features:
            return OpSupport.no("int_dot is disabled and this provider has no float path")
        # a node may opt out of 8-bit activations (StandardOps.cs:130-135); the reference then runs its f32-activation
        # path unless reduced precision is allowed (GraphLowerer.IntDot.cs:61-62, CpuCompiledSegment.LowerLinear.cs:39).
        # Here such a node runs the dequant-fused f32 mat-vec (never silently quantized), which keeps one activation row
        # of K f32 values in shared memory: K beyond that goes to the placement fallback.
        if node.f32_activations and not self.allow_reduced_precision and node.weight.shape[1] > F32_ACTIVATIONS_MAX_K:
            return OpSupport.no(f"f32 activations requested and K={node.weight.shape[1]} exceeds the f32 mat-vec's {F32_ACTIVATIONS_MAX_K}")
        return OpSupport.yes()

    def _supports_ignoring_f32(self, node: "MatMulNode") -> bool:
        import dataclasses
        return self.supports(dataclasses.replace(node, f32_activations=False)).supported

    def upload_weight(self, type_name: str, shape: Sequence[int], blocks, k_slice=None) -> DeviceWeight:
        fmt = DATA_TYPES.get(type_name)
        if fmt is None:
            raise NotSupportedError(f"weight type {type_name}")
        n, k = int(shape[0]), int(shape[1])
        blocks = np.ascontiguousarray(blocks, np.uint8).reshape(-1)
        h = C.c_void_p()
        ptr = blocks.ctypes.data_as(C.c_void_p)
        if k_slice is None:
            _check(N.load().slc_weight_upload(self.handle, fmt, n, k, ptr, blocks.size, C.byref(h)))
        else:
            k0, k1 = k_slice
            _check(N.load().slc_weight_upload_kslice(self.handle, fmt, n, k, ptr, blocks.size, k0, k1, C.byref(h)))
            k = k1 - k0
        return DeviceWeight(self, fmt, n, k, h.value)

    def import_weight_layout(self, artefact) -> DeviceWeight:
        """Uploads an artefact written by DeviceWeight.export_layout: no raw blocks, no re-layout pass."""
        artefact = np.ascontiguousarray(artefact, np.uint8).reshape(-1)
        h = C.c_void_p()
        _check(N.load().slc_weight_import_layout(self.handle, artefact.ctypes.data_as(C.c_void_p), artefact.size, C.byref(h)))
        fmt, n, k = C.c_int32(0), C.c_int64(0), C.c_int64(0)
        _check(N.load().slc_weight_shape(h, C.byref(fmt), C.byref(n), C.byref(k), None))
        return DeviceWeight(self, fmt.value, n.value, k.value, h.value)

    def compile(self, segment: GraphSegment, options: CompileOptions) -> "CudaSegment":
        for node in segment.nodes:
            if isinstance(node, ViewNode):
                continue
            s = self.supports(node)
            if not s.supported and not (isinstance(node, MatMulNode) and node.f32_activations and options.allow_reduced_precision
                                        and self._supports_ignoring_f32(node)):
                raise NotSupportedError(f"{node.name}: {s.reason}")
        return CudaSegment(self, segment, options)

    def debug_quantize(self, x: np.ndarray, dtype: int = N.F32):
        """(q, d, gs) of the device quantizer for host rows x [rows, k]."""
        rows, k = x.shape
        x = np.ascontiguousarray(x)
        q = np.empty((rows, k), np.int8)
        d = np.empty((rows, k // 32), np.float32)
        gs = np.empty((rows, k // 16), np.float32)
        _check(N.load().slc_debug_quantize(self.handle, x.ctypes.data_as(C.c_void_p), dtype, rows, k,
                                           q.ctypes.data_as(C.c_void_p), d.ctypes.data_as(C.c_void_p),
                                           gs.ctypes.data_as(C.c_void_p)))
        return q, d, gs

    def dispose(self) -> None:
        if self._h is not None:
            N.load().slc_device_close(self._h)
            self._h = None


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns (uint16), round to nearest even."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


F32_ACTIVATIONS_MAX_K = 49152   # one f32 activation row in 200 KB of shared memory (matvec_f32.cu), less the reduction area


class MatMulOp:
    """y = x . W^T for activation rows x and a quantized weight W [N, K] (src/Sharplight.Cpu/MatMulOp.cs:88-160),
    on the integer-dot path at every row count."""

    def __init__(self, device: CudaDevice, weight: DeviceWeight, max_rows: int, *, row_invariant: bool = False,
                 up: Optional[DeviceWeight] = None, f32_activations: bool = False):
        """``up``: a second weight of the same shape; the op then computes silu(x . weight^T) * (x . up^T), the gated
        FFN's gate / up pair as one MatMul (slc_matmul_create_dual). ``f32_activations``: the activations are never
        quantized; ``run`` / ``run_pointers`` use the dequant-fused f32 mat-vec (SLC_MATMUL_F32_ACTIVATIONS)."""
        self.device, self.weight, self.max_rows, self.up = device, weight, max_rows, up
        h = C.c_void_p()
        flags = (N.MATMUL_ROW_INVARIANT if row_invariant else N.MATMUL_DEFAULT) | (N.MATMUL_F32_ACTIVATIONS if f32_activations else 0)
        if up is None:
            _check(N.load().slc_matmul_create(device.handle, weight.handle, max_rows, flags, C.byref(h)))
        else:
            _check(N.load().slc_matmul_create_dual(device.handle, weight.handle, up.handle, max_rows, flags, C.byref(h)))
        self._h = h

    @property
    def handle(self):
        if self._h is None:
            raise ObjectDisposedError("MatMulOp")
        return self._h

    def set_kernel(self, kernel: int) -> None:
        _check(N.load().slc_matmul_set_kernel(self.handle, kernel))

    def last_kernel(self):
        k, l = C.c_int32(0), C.c_int32(0)
        _check(N.load().slc_matmul_last_kernel(self.handle, C.byref(k), C.byref(l)))
        return k.value, l.value

    def run(self, x: np.ndarray, dtype: int = N.F32) -> np.ndarray:
        """Host rows in, host rows out (copies inside the call)."""
        if x.ndim != 2 or x.shape[1] != self.weight.k:
            raise ArgumentError(f"x must be [rows, {self.weight.k}]")
        rows = x.shape[0]
        x = np.ascontiguousarray(x)
        y = np.zeros((rows, self.weight.n), np.float32)
        _check(N.load().slc_matmul_run(self.handle, x.ctypes.data_as(C.c_void_p), dtype, rows, self.weight.k, 0,
                                       y.ctypes.data_as(C.c_void_p), max(self.weight.n, 1), 0, None))
        return y

    def run_pointers(self, x_ptr: int, dtype: int, rows: int, x_stride: int, x_is_device: bool, y_ptr: int,
                     y_stride: int, y_is_device: bool, stream: int = 0) -> None:
        """The raw entry point: host or device pointers, caller-owned stream (0 = the device's own)."""
        _check(N.load().slc_matmul_run(self.handle, C.c_void_p(x_ptr), dtype, rows, x_stride, int(x_is_device),
                                       C.c_void_p(y_ptr), y_stride, int(y_is_device),
                                       C.c_void_p(stream) if stream else None))

    def block_dots(self, x: np.ndarray, dtype: int = N.F32) -> np.ndarray:
        """int32 [rows, N, K/32]: the unsigned-code block dots the kernels computed for host rows x."""
        rows = x.shape[0]
        x = np.ascontiguousarray(x)
        s32 = np.zeros((rows, self.weight.n, self.weight.k // 32), np.int32)
        _check(N.load().slc_debug_block_dots(self.handle, x.ctypes.data_as(C.c_void_p), dtype, rows,
                                             s32.ctypes.data_as(C.c_void_p)))
        return s32

    def dispose(self) -> None:
        if self._h is not None:
            N.load().slc_matmul_destroy(self._h)
            self._h = None


class SharedActivation:
    """One 8-bit copy of x serving several MatMuls (slc_activation)."""

    def __init__(self, device: CudaDevice, max_rows: int, k: int):
        self.device, self.max_rows, self.k = device, max_rows, k
        h = C.c_void_p()
        _check(N.load().slc_activation_create(device.handle, max_rows, k, C.byref(h)))
        self._h = h

    @property
    def handle(self):
        if self._h is None:
            raise ObjectDisposedError("SharedActivation")
        return self._h

    def quantize(self, x_device_ptr: int, dtype: int, rows: int, x_stride: int, stream: int = 0) -> None:
        _check(N.load().slc_activation_quantize(self.handle, C.c_void_p(x_device_ptr), dtype, rows, x_stride,
                                                C.c_void_p(stream) if stream else None))

    def set_rows(self, x_device_ptr: int, dtype: int, rows: int, x_stride: int, stream: int = 0) -> None:
        """Deferred quantization (slc_activation_set_rows): the first MatMul that reads the rows quantizes them -- inside
        its own kernel when it is a mat-vec over a short K, through the quantizer otherwise."""
        _check(N.load().slc_activation_set_rows(self.handle, C.c_void_p(x_device_ptr), dtype, rows, x_stride,
                                                C.c_void_p(stream) if stream else None))

    def quantize_rmsnorm(self, x_device_ptr: int, dtype: int, rows: int, x_stride: int, weight_ptr: int, eps: float,
                         y_device_ptr: int = 0, y_stride: int = 0, stream: int = 0) -> None:
        """RmsNorm and quantization in one pass (slc_activation_quantize_rmsnorm); y (optional) also gets the f32 values."""
        _check(N.load().slc_activation_quantize_rmsnorm(
            self.handle, C.c_void_p(x_device_ptr), dtype, rows, x_stride, C.c_void_p(weight_ptr) if weight_ptr else None,
            C.c_float(eps), C.c_void_p(y_device_ptr) if y_device_ptr else None, y_stride, C.c_void_p(stream) if stream else None))

    def quantize_silu_mul(self, gate_ptr: int, gate_stride: int, up_ptr: int, up_stride: int, rows: int,
                          y_device_ptr: int = 0, y_stride: int = 0, stream: int = 0) -> None:
        """silu(gate) * up and quantization in one pass (slc_activation_quantize_silu_mul)."""
        _check(N.load().slc_activation_quantize_silu_mul(
            self.handle, C.c_void_p(gate_ptr), gate_stride, C.c_void_p(up_ptr), up_stride, rows,
            C.c_void_p(y_device_ptr) if y_device_ptr else None, y_stride, C.c_void_p(stream) if stream else None))

    def matmul(self, op: MatMulOp, y_device_ptr: int, y_stride: int, stream: int = 0) -> None:
        _check(N.load().slc_matmul_run_quantized(op.handle, self.handle, C.c_void_p(y_device_ptr), y_stride,
                                                 C.c_void_p(stream) if stream else None))

    def matmul_epilogue(self, op: MatMulOp, y_device_ptr: int, y_stride: int, *, bias_ptr: int = 0, residual_ptr: int = 0,
                        residual_stride: int = 0, stream: int = 0, exchange: "TpExchange" = None) -> None:
        """y = (act . W^T + bias) + residual in the MatMul's own launch (slc_matmul_run_quantized_epilogue)."""
        _check(N.load().slc_matmul_run_quantized_epilogue(
            op.handle, self.handle, exchange.handle if exchange is not None else None,
            C.c_void_p(bias_ptr) if bias_ptr else None, C.c_void_p(residual_ptr) if residual_ptr else None,
            residual_stride, C.c_void_p(y_device_ptr), y_stride, C.c_void_p(stream) if stream else None))

    def dispose(self) -> None:
        if self._h is not None:
            N.load().slc_activation_destroy(self._h)
            self._h = None


class TpComm:
    """The collective-library communicator of a tensor-parallel group (slc_tp_comm: NCCL, loaded by the native library
    at run time). Rank 0 makes the id, the host hands it to every rank, all ranks create at the same time."""

    def __init__(self, device: CudaDevice, rank: int, world: int, unique_id: bytes):
        if len(unique_id) != N.TP_COMM_ID_BYTES:
            raise ArgumentError("unique_id must be the 128 bytes of TpComm.unique_id()")
        self.device, self.rank, self.world = device, rank, world
        h = C.c_void_p()
        buf = (C.c_uint8 * N.TP_COMM_ID_BYTES).from_buffer_copy(unique_id)
        _check(N.load().slc_tp_comm_create(device.handle, rank, world, buf, C.byref(h)))
        self._h = h

    def set_chunking(self, min_rows: int) -> None:
        """Prefill sums in chunks beside the GEMM from ``min_rows`` rows whatever the group size; 0: the default policy."""
        _check(N.load().slc_tp_comm_set_chunking(self.handle, min_rows))

    @staticmethod
    def unique_id() -> bytes:
        buf = (C.c_uint8 * N.TP_COMM_ID_BYTES)()
        _check(N.load().slc_tp_comm_unique_id(buf))
        return bytes(buf)

    @classmethod
    def for_group(cls, device: CudaDevice, dist) -> "TpComm":
        """Creates the communicator over an initialised torch.distributed group (the id travels by broadcast)."""
        box = [cls.unique_id() if dist.get_rank() == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return cls(device, dist.get_rank(), dist.get_world_size(), box[0])

    @property
    def handle(self):
        if self._h is None:
            raise ObjectDisposedError("TpComm")
        return self._h

    def dispose(self) -> None:
        if self._h is not None:
            N.load().slc_tp_comm_destroy(self._h)
            self._h = None


class TpExchange:
    """The receive area through which a row-split MatMul's kernel sums its output over the ranks of a tensor-parallel
    group (slc_tp_exchange). One per rank; ``handle_bytes`` of every rank, in rank order, go to ``connect``."""

    def __init__(self, device: CudaDevice, rank: int, world: int, max_rows: int, n: int):
        self.device, self.rank, self.world, self.max_rows, self.n = device, rank, world, max_rows, n
        h = C.c_void_p()
        buf = (C.c_uint8 * N.TP_HANDLE_BYTES)()
        _check(N.load().slc_tp_exchange_create(device.handle, rank, world, max_rows, n, C.byref(h), buf))
        self._h = h
        self.handle_bytes = bytes(buf)

    @property
    def handle(self):
        if self._h is None:
            raise ObjectDisposedError("TpExchange")
        return self._h

    def connect(self, handles: Sequence[bytes]) -> None:
        if len(handles) != self.world or any(len(b) != N.TP_HANDLE_BYTES for b in handles):
            raise ArgumentError("connect needs one 64-byte handle per rank, in rank order")
        blob = (C.c_uint8 * (N.TP_HANDLE_BYTES * self.world)).from_buffer_copy(b"".join(handles))
        _check(N.load().slc_tp_exchange_connect(self.handle, blob))

    def set_wait_ms(self, milliseconds: int) -> None:
        """How long a kernel waits for its peers before it raises the device status to ERR_TIMEOUT."""
        _check(N.load().slc_tp_exchange_set_wait_ms(self.handle, milliseconds))

    def set_comm(self, comm: Optional["TpComm"], in_kernel_rows: int = 16) -> None:
        """Calls with more than ``in_kernel_rows`` rows (or more than this exchange's max_rows) are summed by the
        communicator's all-reduce instead of inside the MatMul kernel; None detaches."""
        _check(N.load().slc_tp_exchange_set_comm(self.handle, comm.handle if comm is not None else None, in_kernel_rows))

    def connect_group(self, dist) -> None:
        """Exchanges the handles over an initialised torch.distributed group and connects."""
        handles = [None] * self.world
        dist.all_gather_object(handles, self.handle_bytes)
        self.connect(handles)

    def matmul(self, op: MatMulOp, act: "SharedActivation", y_device_ptr: int, y_stride: int, stream: int = 0) -> None:
        """y = sum over ranks of act . W^T (every rank calls it with its shard)."""
        _check(N.load().slc_matmul_run_quantized_allreduce(op.handle, act.handle, self.handle, C.c_void_p(y_device_ptr),
                                                           y_stride, C.c_void_p(stream) if stream else None))

    def run(self, op: MatMulOp, x_device_ptr: int, dtype: int, rows: int, x_stride: int, y_device_ptr: int,
            y_stride: int, stream: int = 0) -> None:
        """y = sum over ranks of x . W^T with x not yet quantized (slc_matmul_run_allreduce)."""
        _check(N.load().slc_matmul_run_allreduce(op.handle, self.handle, C.c_void_p(x_device_ptr), dtype, rows, x_stride,
                                                 C.c_void_p(y_device_ptr), y_stride, C.c_void_p(stream) if stream else None))

    def dispose(self) -> None:
        if self._h is not None:
            N.load().slc_tp_exchange_destroy(self._h)
            self._h = None


class _Pinned:
    """Page-locked host staging exposed as a numpy array."""

    def __init__(self, nbytes: int):
        p = C.c_void_p()
        _check(N.load().slc_host_alloc(max(nbytes, 16), C.byref(p)))
        self.ptr, self.nbytes = p, nbytes
        self.array = np.ctypeslib.as_array((C.c_uint8 * max(nbytes, 16)).from_address(p.value))

    def free(self):
        if self.ptr is not None:
            self.array = None
            N.load().slc_host_free(self.ptr)
            self.ptr = None


class CudaSegment:
    """ICompiledSegment for a list of MatMul nodes. Weights are uploaded at compile time; SetInput copies the host
    bytes (into page-locked staging, then to the device); Execute quantizes every distinct input once and runs all
    nodes that read it from that one 8-bit copy (as the reference's lowering shares it,
    src/Sharplight.Shaders/Lowering/GraphLowerer.IntDot.cs:38-43), then starts the copy of the outputs back to the
    host -- all asynchronous; GetOutput waits for the device once and reads the staged result. Error behaviour follows
    the CPU segment (src/Sharplight.Cpu/CpuCompiledSegment.cs:96-124,149,189). A node's input may also be the output
    of an earlier node of the segment (it then stays on the device)."""

    def __init__(self, device: CudaDevice, segment: GraphSegment, options: CompileOptions):
        self.device, self.segment, self.options = device, segment, options
        self._disposed = False
        self._executed = False
        self._synced = False
        self._rows: Dict[str, int] = {}
        self._ops: Dict[str, MatMulOp] = {}
        self._weights: List[DeviceWeight] = []
        self._f32_nodes: set = set()   # nodes that keep f32 activation math (never quantized)
        lib = N.load()
        mr = options.max_rows
        row_inv = options.row_invariant_rows > 0
        # value name -> (columns, element bytes)
        self._shape: Dict[str, tuple] = {}
        self._reduce = {node.name for node in segment.nodes if isinstance(node, MatMulNode) and node.allreduce}
        if self._reduce and options.exchange is None:
            raise ArgumentError("a segment with allreduce nodes needs CompileOptions.exchange")
        # views: value -> (the value whose buffer it lives in, element offset, row stride in elements, rows per T)
        self._alias: Dict[str, tuple] = {}
        self._row_mult: Dict[str, int] = {}
        for node in segment.nodes:
            if isinstance(node, ViewNode):
                self._lower_view(node)
                continue
            w = node.weight.resident
            if w is None:
                w = device.upload_weight(node.weight.type, node.weight.shape, node.weight.blocks)
                self._weights.append(w)
            f32 = node.f32_activations and not (device.allow_reduced_precision or options.allow_reduced_precision)
            mult = self._row_mult.get(node.x, 1)
            self._ops[node.name] = MatMulOp(device, w, mr * mult, row_invariant=row_inv and not f32, f32_activations=f32)
            if f32:
                self._f32_nodes.add(node.name)
            esz = 2 if node.x_dtype == "bf16" else 4
            if node.x in self._shape and self._shape[node.x] != (w.k, esz):
                raise ArgumentError(f"{node.name}: input '{node.x}' is [T, {self._shape[node.x][0]}], the weight wants K={w.k}")
            self._shape.setdefault(node.x, (w.k, esz))
            self._shape[node.y] = (w.n, 4)
            self._row_mult[node.y] = mult
        for v in segment.outputs:
            if v in self._alias:
                raise NotSupportedError(f"output '{v}' is a view of another value: read that value instead")
        # device buffers for every value that owns its bytes; page-locked staging for inputs and outputs
        self._dev: Dict[str, C.c_void_p] = {}
        for name, (cols, esz) in self._shape.items():
            if name in self._alias:
                continue
            p = C.c_void_p()
            _check(lib.slc_buffer_alloc(device.handle, mr * self._row_mult.get(name, 1) * cols * esz, C.byref(p)))
            self._dev[name] = p
        self._in_stage = {v: _Pinned(mr * self._shape[v][0] * self._shape[v][1]) for v in segment.inputs}
        self._out_offset, off = {}, 0
        for v in segment.outputs:
            self._out_offset[v] = off
            off += mr * self._row_mult.get(v, 1) * self._shape[v][0] * 4
        self._out_stage = _Pinned(off)
        self._acts = {v: SharedActivation(device, mr * self._row_mult.get(v, 1), self._shape[v][0])
                      for v in {n.x for n in segment.nodes if isinstance(n, MatMulNode) and n.name not in self._f32_nodes}}
        # output copies travel on a second stream beside the kernels; per row-count signature: None -> issued once
        # from the host, 1 -> issued twice (every kernel configured), then the captured graph
        self._copy_stream = C.c_void_p()
        _check_graph(lib.slc_stream_create(device.handle, C.byref(self._copy_stream)))
        self._graphs: Dict[tuple, object] = {}
        self._last_signature, self._last_graph = None, None
        self._forward: Dict[str, "CudaSegment"] = {}   # input value -> the segment whose output it is read from
        self._device_only: set = set()                 # outputs nobody reads on the host: not copied back

    def _lower_view(self, node: "ViewNode") -> None:
        esz = 2 if node.dtype == "bf16" else 4
        if node.x in self._shape and self._shape[node.x] != (node.x_cols, esz):
            raise ArgumentError(f"{node.name}: '{node.x}' is [T, {self._shape[node.x][0]}], not [T, {node.x_cols}]")
        self._shape.setdefault(node.x, (node.x_cols, esz))
        self._row_mult.setdefault(node.x, 1)
        root, off, stride, mult = self._alias.get(node.x, (node.x, 0, node.x_cols, self._row_mult[node.x]))
        if node.kind == "slice":
            if node.start < 0 or node.length < 1 or node.start + node.length > node.x_cols:
                raise ArgumentError(f"{node.name}: slice [{node.start}, {node.start + node.length}) of {node.x_cols} columns")
            self._alias[node.y] = (root, off + node.start, stride, mult)
            self._shape[node.y] = (node.length, esz)
            self._row_mult[node.y] = mult
        elif node.kind == "reshape":
            if node.split < 1 or node.x_cols % node.split != 0:
                raise ArgumentError(f"{node.name}: {node.x_cols} columns do not split in {node.split} rows")
            if stride != node.x_cols:
                raise NotSupportedError(f"{node.name}: a row-splitting reshape of a column slice (rows are not contiguous)")
            cols = node.x_cols // node.split
            self._alias[node.y] = (root, off, cols, mult * node.split)
            self._shape[node.y] = (cols, esz)
            self._row_mult[node.y] = mult * node.split
        elif node.kind == "permute":
            if node.a < 1 or node.b < 1 or node.a * node.b != node.x_cols:
                raise ArgumentError(f"{node.name}: [{node.a}, {node.b}] is not {node.x_cols} columns")
            self._shape[node.y] = (node.x_cols, esz)      # a buffer of its own, filled by the gather
            self._row_mult[node.y] = mult
        else:
            raise NotSupportedError(f"{node.name}: view kind '{node.kind}'")

    def _where(self, value: str):
        """(device address, row stride in elements) of a value: its own buffer, or the place inside another one."""
        if value in self._alias:
            root, off, stride, _ = self._alias[value]
            return self._dev[root].value + off * self._shape[value][1], stride
        return self._dev[value].value, self._shape[value][0]

    @property
    def device_memory_bytes(self) -> int:
        return sum(w.device_bytes for w in self._weights) + \
            sum(self.options.max_rows * self._row_mult.get(n, 1) * c * e for n, (c, e) in self._shape.items() if n not in self._alias)

    def _live(self):
        if self._disposed:
            raise ObjectDisposedError("CudaSegment")

    def try_forward_from(self, value: str, producer) -> bool:
        """IDeviceForwardingSegment.TryForwardFrom (src/Sharplight.Core/Runtime/IDeviceForwardingSegment.cs:10-21):
        from now on input ``value`` is read straight from ``producer``'s output of the same name in device memory.
        False when that output is not reachable from here (another provider or device, another shape)."""
        self._live()
        if not isinstance(producer, CudaSegment) or producer._disposed or producer.device is not self.device:
            return False
        if value not in self.segment.inputs or value not in producer.segment.outputs:
            return False
        if producer._shape[value] != self._shape[value] or producer.options.max_rows > self.options.max_rows:
            return False
        if value not in self._forward:
            N.load().slc_buffer_free(self.device.handle, self._dev[value])
        self._dev[value] = producer._dev[value]
        self._forward[value] = producer
        self._graphs_clear()
        return True

    def keep_on_device(self, value: str) -> None:
        """No host consumer reads output ``value`` (a later segment takes it by try_forward_from): skip its copy back."""
        self._live()
        if value not in self._out_offset:
            raise ArgumentError(f"'{value}' is not an output of this segment")
        self._device_only.add(value)
        self._graphs_clear()

    def _graphs_clear(self) -> None:
        self.device.synchronize()
        for g in self._graphs.values():
            if not isinstance(g, int):
                N.load().slc_graph_destroy(g)
        self._graphs.clear()
        self._last_signature, self._last_graph = None, None

    def set_input(self, value: str, data: np.ndarray) -> None:
        self._live()
        if value not in self.segment.inputs:
            raise ArgumentError(f"'{value}' is not an input of this segment")
        if value in self._forward:
            raise InvalidOperationError(f"input '{value}' is forwarded from another segment's output")
        cols, esz = self._shape[value]
        data = np.ascontiguousarray(data)
        if data.ndim != 2 or data.shape[1] != cols or data.dtype.itemsize != esz:
            raise ArgumentError(f"input '{value}' must be [T, {cols}] of {esz}-byte elements")
        if data.shape[0] > self.options.max_rows:
            raise ArgumentError(f"input '{value}' holds more rows than the compiled capacity")
        nbytes = data.nbytes
        stage = self._in_stage[value]
        stage.array[:nbytes] = data.reshape(-1).view(np.uint8)
        _check(N.load().slc_buffer_copy_async(self.device.handle, self._dev[value], stage.ptr, nbytes, 0, None))
        self._rows[value] = data.shape[0]

    def execute(self, symbols: Optional[Dict[str, int]] = None) -> None:
        self._live()
        t = (symbols or {}).get("T")
        if t is not None and t > self.options.max_rows:
            raise InvalidOperationError(f"T={t} exceeds the compiled bound {self.options.max_rows}")
        lib = N.load()
        rows_of: Dict[str, int] = dict(self._rows)
        for value, producer in self._forward.items():
            if not producer._executed:
                raise InvalidOperationError(f"the segment that produces '{value}' has not executed")
            rows_of[value] = producer._out_rows[value]
        # the same row counts as the last call, already captured: one launch, no planning
        signature = (t, tuple(rows_of.items()))
        if signature == self._last_signature:
            self._out_rows = self._last_out_rows
            _check_graph(lib.slc_graph_launch(self._last_graph, None))
            self._executed, self._synced = True, False
            return
        # the step as a list of launches (host logic only), then issued directly or through its captured graph
        plan, quantized = [], set()
        for node in self.segment.nodes:
            if node.x not in rows_of:
                raise InvalidOperationError(f"input '{node.x}' was never set")
            if isinstance(node, ViewNode):
                rows_of[node.y] = rows_of[node.x] * (node.split if node.kind == "reshape" else 1)
                if node.kind == "permute":
                    plan.append(("densify", node, rows_of[node.x] if t is None else min(t * self._row_mult[node.x], rows_of[node.x])))
                    quantized.discard(node.y)
                continue
            mult = self._row_mult.get(node.x, 1)
            rows = rows_of[node.x] if t is None else min(t * mult, rows_of[node.x])
            if node.name in self._f32_nodes:
                plan.append(("matmul_f32", node, rows))
            else:
                if node.x not in quantized:
                    plan.append(("quantize", node, rows))
                    quantized.add(node.x)
                plan.append(("matmul", node, rows))
            rows_of[node.y] = rows
            quantized.discard(node.y)
        self._out_rows = {v: rows_of[v] for v in self.segment.outputs}
        key = tuple(sorted(self._out_rows.items())) + tuple(sorted((v, rows_of[v]) for v in self.segment.inputs))
        state = self._graphs.get(key)
        if not self.options.capture_steps or (state is None and len(self._graphs) >= 32):
            self._issue(plan)
        elif state is None or state == 1:
            self._issue(plan)
            self._graphs[key] = 1 if state is None else 2
        elif state == 2:
            _check_graph(lib.slc_graph_begin(self.device.handle, None))
            try:
                self._issue(plan)
            finally:
                g = C.c_void_p()
                code = lib.slc_graph_end(self.device.handle, None, C.byref(g))
            _check_graph(code)
            self._graphs[key] = g
            _check_graph(lib.slc_graph_launch(g, None))
        else:
            _check_graph(lib.slc_graph_launch(state, None))
            self._last_signature, self._last_graph, self._last_out_rows = signature, state, dict(self._out_rows)
        self._executed, self._synced = True, False

    def _issue(self, plan) -> None:
        """The step's launches on the device's stream; every output leaves on the copy stream as soon as the kernel
        that produced it is queued, and the copy stream is joined back at the end."""
        lib = N.load()
        outputs = set(self.segment.outputs)
        copied = False
        for kind, node, rows in plan:
            if kind == "densify":
                src, stride = self._where(node.x)
                _check(lib.slc_buffer_densify(self.device.handle, self._dev[node.y], C.c_void_p(src), rows, node.b, node.a,
                                              stride, 1, node.b, self._shape[node.y][1], None))
                continue
            if kind == "quantize":
                dtype = N.BF16 if node.x_dtype == "bf16" else N.F32
                src, stride = self._where(node.x)
                self._acts[node.x].quantize(src, dtype, rows, stride, 0)
                continue
            if kind == "matmul_f32":
                if node.name in self._reduce:
                    raise NotSupportedError("an f32-activation MatMul does not sum over ranks")
                dtype = N.BF16 if node.x_dtype == "bf16" else N.F32
                src, stride = self._where(node.x)
                self._ops[node.name].run_pointers(src, dtype, rows, stride, True,
                                                  self._dev[node.y].value, self._shape[node.y][0], True, 0)
            elif node.name in self._reduce:
                self.options.exchange.matmul(self._ops[node.name], self._acts[node.x], self._dev[node.y].value,
                                             self._shape[node.y][0], 0)
            else:
                self._acts[node.x].matmul(self._ops[node.name], self._dev[node.y].value, self._shape[node.y][0], 0)
            if node.y in outputs and node.y not in self._device_only:
                nbytes = rows * self._shape[node.y][0] * 4
                dst = C.c_void_p(self._out_stage.ptr.value + self._out_offset[node.y])
                _check_graph(lib.slc_stream_wait(self.device.handle, self._copy_stream, None))
                _check(lib.slc_buffer_copy_async(self.device.handle, dst, self._dev[node.y], nbytes, 1, self._copy_stream))
                copied = True
        if copied:
            _check_graph(lib.slc_stream_wait(self.device.handle, None, self._copy_stream))

    def get_output(self, value: str, copy: bool = True) -> np.ndarray:
        self._live()
        if not self._executed:
            raise InvalidOperationError("GetOutput before Execute")
        if value not in self._out_offset:
            raise ArgumentError(f"'{value}' is not an output of this segment")
        if value in self._device_only:
            raise InvalidOperationError(f"output '{value}' stays on the device (keep_on_device)")
        if not self._synced:
            self.device.synchronize()
            self._synced = True
        rows, cols = self._out_rows[value], self._shape[value][0]
        off = self._out_offset[value]
        out = self._out_stage.array[off:off + rows * cols * 4].view(np.float32).reshape(rows, cols)
        return out.copy() if copy else out

    def reset_state(self) -> None:
        self._live()   # MatMul keeps no state

    def dispose(self) -> None:
        if self._disposed:
            return
        self._graphs_clear()
        N.load().slc_stream_destroy(self.device.handle, self._copy_stream)
        for op in self._ops.values():
            op.dispose()
        for a in self._acts.values():
            a.dispose()
        for w in self._weights:
            w.dispose()
        for name, p in self._dev.items():
            if name not in self._forward:    # a forwarded input's buffer belongs to the producing segment
                N.load().slc_buffer_free(self.device.handle, p)
        for st in self._in_stage.values():
            st.free()
        self._out_stage.free()
        self._disposed = True
