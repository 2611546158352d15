"""ingot_b200: the decode hot path of ingot (fused dequantise-and-dot GEMV over
GGUF block-quantised weights, expert-routed GEMV, routing and combine, the
prefill dequant-GEMM) as hand-written sm_100a CUDA behind a C ABI
(include/ingot_cuda.h, libingot_cuda.so).

`Gpu`, `Buffer`, `Command`, `Weight`, `Tensor`, `Matrix` mirror the reference's
Rust interface; importing them loads the shared library and fails loudly when
it has not been built (`python -m ingot_b200.build`).
"""
from .gpu import (BF16, F16, F32, Q4_0, Q4_K, Q6_K, Q8_0, X_DIGITS, X_PACKED, X_PACKED_HI, Buffer, Command, DeviceError, DeviceTimeout, Gpu,
                  Graph, IngotError, InvalidData, Matrix, Tensor, Weight)
from .synth import geometry, stride_of

__all__ = ["Gpu", "Buffer", "Command", "Graph", "Weight", "Tensor", "Matrix", "IngotError", "InvalidData",
           "DeviceError", "DeviceTimeout", "geometry", "stride_of", "F32", "F16", "BF16", "Q4_0", "Q8_0",
           "Q4_K", "Q6_K", "X_PACKED", "X_DIGITS", "X_PACKED_HI"]
