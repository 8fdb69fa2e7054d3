from .gemm import WQLinear_GEMM, awq_dequantize, awq_gemm, pack_int4, unpack_int4  # noqa: F401
