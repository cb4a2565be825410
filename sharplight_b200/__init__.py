"""sharplight_b200: B200-native (sm_100a) quantized MatMul for Sharplight -- the CUDA execution provider's host side
over the C ABI of libsharplight_cuda.so. Build the library with ``python -m sharplight_b200.build``."""
from .provider import (ArgumentError, CompileOptions, CudaDevice, CudaExecutionProvider, CudaSegment, DeviceInfo,
                       DeviceWeight, GraphSegment, InvalidOperationError, MatMulNode, MatMulOp, NotSupportedError,
                       ObjectDisposedError, OpSupport, SharedActivation, TpComm, TpExchange, ViewNode, WeightInfo)

__all__ = ["ArgumentError", "CompileOptions", "CudaDevice", "CudaExecutionProvider", "CudaSegment", "DeviceInfo",
           "DeviceWeight", "GraphSegment", "InvalidOperationError", "MatMulNode", "MatMulOp", "NotSupportedError",
           "ObjectDisposedError", "OpSupport", "SharedActivation", "TpComm", "TpExchange", "ViewNode", "WeightInfo"]
