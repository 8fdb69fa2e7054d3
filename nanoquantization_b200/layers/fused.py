"""Fused elementwise steps of a Qwen3 block (one CUDA launch each), bound through the C ABI.
They produce what the reference's RMSNorm / RoPE modules and ``F.silu(y1) * y2`` produce
(nanoquantization/layers/norm.py:18-32, layers/rope.py:24-45, models/qwen3_quantized.py:150)."""
from __future__ import annotations

import torch

from .. import _lib


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, eps: float):
    """``h = x (+ residual)``; returns ``(RMSNorm(h) * weight, h)``.  ``h`` is written over ``residual``
    when one is given (the residual stream is updated in place), else it is ``x`` itself."""
    dev = _lib.require_cuda(x, weight)
    T, H = x.shape
    x = x if x.is_contiguous() else x.contiguous()
    out = torch.empty_like(x)
    if residual is None:
        res_ptr, res_out, new_res = None, None, x
    else:
        res_ptr, res_out, new_res = residual.data_ptr(), residual.data_ptr(), residual
    _lib.check(_lib.load().nqb200_add_rmsnorm(x.data_ptr(), res_ptr, weight.data_ptr(), out.data_ptr(), res_out, T, H,
                                              float(eps), _lib.dtype_code(x.dtype), _lib.stream_ptr()))
    return out, new_res


def qknorm_rope_(qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, cos_sin: torch.Tensor,
                 positions: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int, eps: float,
                 kv_target=None) -> torch.Tensor:
    """In place on ``qkv [T, (Hq + 2 Hkv) * D]``: per-head RMSNorm of q and k, then rotary embedding.
    ``kv_target = (k_cache, v_cache, slots)``: also store the rotated k and v of token t in row
    ``slots[t]`` of the caches (each ``[..., Hkv, D]`` contiguous, any leading shape)."""
    _lib.require_cuda(qkv, q_weight, k_weight, cos_sin, positions)
    assert qkv.is_contiguous() and positions.dtype == torch.int64 and cos_sin.dtype == torch.float32
    T = qkv.shape[0]
    if kv_target is not None:
        k_cache, v_cache, slots = kv_target
        _lib.require_cuda(k_cache, v_cache, slots)
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and slots.dtype == torch.int64 and slots.numel() == T
        assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype and k_cache.shape[-2:] == (num_kv_heads, head_dim)
        _lib.check(_lib.load().nqb200_qknorm_rope_kv(qkv.data_ptr(), q_weight.data_ptr(), k_weight.data_ptr(), cos_sin.data_ptr(),
                                                     positions.data_ptr(), slots.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                                     T, num_q_heads, num_kv_heads, head_dim, qkv.shape[1], float(eps),
                                                     _lib.dtype_code(qkv.dtype), _lib.stream_ptr()))
        return qkv
    _lib.check(_lib.load().nqb200_qknorm_rope(qkv.data_ptr(), q_weight.data_ptr(), k_weight.data_ptr(), cos_sin.data_ptr(),
                                              positions.data_ptr(), T, num_q_heads, num_kv_heads, head_dim, qkv.shape[1],
                                              float(eps), _lib.dtype_code(qkv.dtype), _lib.stream_ptr()))
    return qkv


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate_up[:, :I]) * gate_up[:, I:]``."""
    _lib.require_cuda(gate_up)
    assert gate_up.is_contiguous()
    T, two_i = gate_up.shape
    out = torch.empty(T, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
    _lib.check(_lib.load().nqb200_silu_mul(gate_up.data_ptr(), out.data_ptr(), T, two_i // 2,
                                           _lib.dtype_code(gate_up.dtype), _lib.stream_ptr()))
    return out
