"""B200-native AWQ W4A16 linear: the reference's WQLinear_GEMM API over sm_100a CUDA."""
from .layers.gemm import WQLinear_GEMM, awq_dequantize, awq_gemm, pack_int4, unpack_int4  # noqa: F401

from .layers.parallel import (ColumnParallelWQLinear, MergedColumnParallelWQLinear, RowParallelWQLinear,  # noqa: F401
                              column_shard_bounds, row_shard_bounds, shard_columns, shard_rows)

__all__ = ["ColumnParallelWQLinear", "MergedColumnParallelWQLinear", "RowParallelWQLinear", "shard_columns", "shard_rows",
           "WQLinear_GEMM", "awq_dequantize", "awq_gemm", "pack_int4", "unpack_int4"]
