"""B200-native (sm_100a) implementation of one hot path of the DeepSeek-V4.1 A100 runtime: the packed-FP4 MoE expert
chain (router top-k, gate/up projection, SiLU*mul, down projection, routing-weighted combine, FP8 shared expert) and the
block-scaled FP8 dense GEMV/GEMM around it.

Module names and function signatures mirror the reference's Python call surface (`quant`, `kernels`, `moe_kernels`,
`fused`, `fused2`, `cukern`, `w8`, `ep`) so a caller of that runtime can switch imports; every operator launches
hand-written CUDA through the C-ABI of csrc/libb200moe.so on the current torch stream.  There is no Triton, no CPU path.
"""
from . import _lib  # noqa: F401

__all__ = ["quant", "kernels", "moe_kernels", "fused", "fused2", "cukern", "w8", "ep", "moe", "synth"]
