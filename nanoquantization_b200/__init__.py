"""B200-native AWQ W4A16 linear: the reference's WQLinear_GEMM API over sm_100a CUDA."""
from .layers.gemm import WQLinear_GEMM, awq_dequantize, awq_gemm, pack_int4, unpack_int4  # noqa: F401

__all__ = ["WQLinear_GEMM", "awq_dequantize", "awq_gemm", "pack_int4", "unpack_int4"]
