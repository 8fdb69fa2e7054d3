from .qwen3_quantized import (Qwen3Config, Qwen3QuantizedAttention, Qwen3QuantizedBlock, Qwen3QuantizedForCausalLM,  # noqa: F401
                              Qwen3QuantizedMLP, Qwen3QuantizedModel, RMSNorm, RotaryCache, QWEN3_SHAPES)
