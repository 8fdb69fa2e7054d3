from .gemm import WQLinear_GEMM, awq_dequantize, awq_gemm, pack_int4, unpack_int4  # noqa: F401
from .parallel import (ColumnParallelWQLinear, MergedColumnParallelWQLinear, RowParallelWQLinear,  # noqa: F401
                       column_shard_bounds, row_shard_bounds, shard_columns, shard_rows)
