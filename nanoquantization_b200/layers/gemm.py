"""AWQ W4A16 linear on B200: the module and function API of the reference's
``nanoquantization/layers/gemm.py`` over hand-written sm_100a kernels.

Same names, arguments, buffer names, dtypes and shapes as the reference, so a
caller switches by changing one import and reference checkpoints load
unchanged:

  * ``WQLinear_GEMM``      -- gemm.py:382-567
  * ``awq_gemm``           -- gemm.py:329-379
  * ``awq_dequantize``     -- gemm.py:126-180

The forward has no CPU path and no PyTorch fallback; it raises if the CUDA
library is missing or the tensors are not on a B200.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn as nn

from .. import _lib

# group sizes the reference accepts (gemm.py:7), besides group_size == in_features
AWQ_SUPPORTED_GROUP_SIZES = [-1, 32, 64, 128]
AWQ_TRITON_SUPPORTED_GROUP_SIZES = AWQ_SUPPORTED_GROUP_SIZES  # the reference's name for the same list

AWQ_PACK_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)  # nibble j of a word holds column AWQ_PACK_ORDER[j] (gemm.py:504-513)
_PACK_NUM = 8


def _contig(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


def unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    """``[R, C/8]`` int32 words -> ``[R, C]`` uint8 values 0..15 in natural column
    order; the shift/mask step of gemm.py:64-69 as a kernel of its own."""
    assert packed.dtype == torch.int32 and packed.dim() == 2
    dev = _lib.require_cuda(packed)
    _lib.require_b200(dev)
    packed = _contig(packed)
    out = torch.empty(packed.shape[0], packed.shape[1] * _PACK_NUM, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().nqb200_unpack_int4(packed.data_ptr(), out.data_ptr(), packed.shape[0],
                                                  packed.shape[1], _lib.stream_ptr()))
    return out


def awq_dequantize(
    qweight: torch.Tensor,
    qscales: torch.Tensor,
    qzeros: torch.Tensor,
    block_size_x: int = 32,
    block_size_y: int = 32,
) -> torch.Tensor:
    """Dense ``[in_features, out_features]`` weight in ``qscales.dtype``.

    Arguments and checks as gemm.py:126-152; the two block sizes were Triton
    tuning knobs and are accepted and ignored.
    """
    K = qweight.shape[0]
    M = qscales.shape[1]
    group_size = qweight.shape[0] // qscales.shape[0]

    assert K > 0 and M > 0
    assert qzeros.shape[0] == K // group_size and qzeros.shape[1] == M // 8
    assert qweight.shape[1] == M // 8
    assert group_size <= K
    assert group_size in AWQ_SUPPORTED_GROUP_SIZES or group_size == K

    dev = _lib.require_cuda(qweight, qscales, qzeros)
    _lib.require_b200(dev)
    code = _lib.dtype_code(qscales.dtype)
    qweight, qscales, qzeros = _contig(qweight), _contig(qscales), _contig(qzeros)
    result = torch.empty(K, M, dtype=qscales.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().nqb200_dequant(qweight.data_ptr(), qscales.data_ptr(), qzeros.data_ptr(),
                                              result.data_ptr(), K, M, group_size, code, _lib.stream_ptr()))
    return result


_ws_bytes_cache: dict[tuple, int] = {}


def _w4a16(x: torch.Tensor, qweight: torch.Tensor, qscales: torch.Tensor, qzeros: torch.Tensor,
           bias: torch.Tensor | None, out: torch.Tensor | None = None, silu_mul: bool = False, peer=None,
           norm=None, residual: torch.Tensor | None = None):
    """One fused call: out = x @ ((q - z) * s) (+ bias), any M.  ``out`` may name a preallocated
    contiguous ``[M, N]`` tensor of the output dtype (e.g. a slot of a peer-mapped buffer).
    ``silu_mul``: the matrix is a merged gate|up projection and the result is
    ``silu(y[:, :N/2]) * y[:, N/2:]`` (``[M, N/2]``); the caller has checked that the library
    supports it for this shape.  ``peer = (buffers, rank, world, slot_offset, slot_bytes)``: the
    linear is a row-parallel shard and the result is the sum over the ranks, reduced over peer
    memory by the kernel that finishes the GEMM (again only where the library supports it).
    ``norm = (ssq, weight, eps)``: ``x`` is a residual stream and the input is its RMSNorm, computed
    on the fly from per-tile sums of squares ``ssq [M, tiles]``.  ``residual``: the result is
    ``(16-bit(y) + residual, ssq_out)``, the new residual stream and its per-tile sums of squares."""
    M, K = x.shape
    N = qweight.shape[1] * 8
    group_size = K // qscales.shape[0]
    dev = _lib.require_cuda(x, qweight, qscales, qzeros)
    _lib.require_b200(dev)
    dtype = qscales.dtype
    code = _lib.dtype_code(dtype)
    if x.dtype != dtype:  # the reference casts x to the output dtype (gemm.py:259)
        x = x.to(dtype)
    x, qweight, qscales, qzeros = _contig(x), _contig(qweight), _contig(qscales), _contig(qzeros)
    bias_ptr, bias_code = None, 0
    if bias is not None:
        bias = _contig(bias)
        bias_ptr, bias_code = bias.data_ptr(), _lib.dtype_code(bias.dtype)
    n_out = N // 2 if silu_mul else N
    if out is None:
        out = torch.empty(M, n_out, dtype=dtype, device=dev)
    else:
        assert out.shape == (M, n_out) and out.dtype == dtype and out.is_contiguous()
    if M == 0:
        return out
    lib = _lib.load()
    entry = lib.nqb200_gemm_gate_up_silu if silu_mul else lib.nqb200_gemm
    tail = (_lib.stream_ptr(),)
    ssq_out = None
    if norm is not None or residual is not None:
        f = _lib.DecodeFusion()
        f.silu_mul = int(silu_mul)
        if norm is not None:
            ssq, nweight, eps = norm
            assert ssq.dtype == torch.float32 and ssq.is_contiguous() and ssq.shape[0] == M and nweight.dtype == dtype
            f.norm_ssq, f.norm_tiles, f.norm_weight, f.norm_eps = ssq.data_ptr(), ssq.shape[1], nweight.data_ptr(), float(eps)
        if residual is not None:
            assert residual.shape == (M, N) and residual.dtype == dtype and residual.is_contiguous()
            tile = lib.nqb200_decode_tile_columns()
            ssq_out = torch.empty(M, (N + tile - 1) // tile, dtype=torch.float32, device=dev)
            f.residual_in, f.ssq_out = residual.data_ptr(), ssq_out.data_ptr()
        entry = lib.nqb200_gemm_decode_fused
        tail = (ctypes.byref(f),) + (tuple(peer) if peer is not None else (None, 0, 0, 0, 0)) + tail
    elif peer is not None:
        assert not silu_mul
        entry, tail = lib.nqb200_gemm_allreduce, tuple(peer) + tail
    key = (M, N, K, group_size, code)
    nbytes = _ws_bytes_cache.get(key)
    if nbytes is None:
        nbytes = _ws_bytes_cache[key] = lib.nqb200_gemm_workspace_bytes(M, N, K, group_size, code)
    other_device = dev.index is not None and dev.index != torch.cuda.current_device()
    if other_device:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        ws = _lib.workspace(dev, nbytes)
        status = entry(x.data_ptr(), qweight.data_ptr(), qscales.data_ptr(), qzeros.data_ptr(),
                       bias_ptr, bias_code, out.data_ptr(), M, N, K, group_size, code,
                       ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, *tail)
    finally:
        if other_device:
            torch.cuda.set_device(prev)
    if status:
        _lib.check(status)
    return (out, ssq_out) if ssq_out is not None else out


def awq_gemm(
    x: torch.Tensor,
    qweight: torch.Tensor,
    qscales: torch.Tensor,
    qzeros: torch.Tensor,
    split_k_iters: int,
    block_size_m: int = 32,
    block_size_n: int = 32,
    block_size_k: int = 32,
) -> torch.Tensor:
    """Fused dequantise + GEMM, result ``[M, N]`` in ``qscales.dtype``.

    Arguments and checks as gemm.py:329-354.  ``split_k_iters`` must still be a
    power of two, but the kernel chooses its own K split; the block sizes are
    accepted and ignored.
    """
    M, K = x.shape
    N = qweight.shape[1] * 8
    group_size = qweight.shape[0] // qscales.shape[0]

    assert qweight.shape[0] == K and qweight.shape[1] == N // 8
    assert qscales.shape[0] == K // group_size and qscales.shape[1] == N
    assert qzeros.shape[0] == K // group_size and qzeros.shape[1] == N // 8
    assert split_k_iters & (split_k_iters - 1) == 0
    assert group_size in AWQ_SUPPORTED_GROUP_SIZES or group_size == K

    return _w4a16(x, qweight, qscales, qzeros, None)


def pack_int4(values: torch.Tensor) -> torch.Tensor:
    """``[R, C]`` integers -> ``[R, C/8]`` int32 in AWQ order: word i of a row is
    the OR of ``values[:, 8*i + order[j]] << 4*j`` (gemm.py:501-520), int32
    arithmetic, no clamp."""
    v = values.to(torch.int32)
    rows, cols = v.shape
    v = v.view(rows, cols // _PACK_NUM, _PACK_NUM)
    word = torch.zeros(rows, cols // _PACK_NUM, dtype=torch.int32, device=v.device)
    for j, e in enumerate(AWQ_PACK_ORDER):
        word |= v[:, :, e] << (4 * j)
    return word


class WQLinear_GEMM(nn.Module):
    """4-bit AWQ linear layer; buffers and behaviour as gemm.py:382-567.

    Buffers: ``qweight`` int32 ``[K, N/8]``, ``qscales`` ``output_dtype``
    ``[K/g, N]``, ``qzeros`` int32 ``[K/g, N/8]`` and, with ``bias=True``,
    ``bias`` bfloat16 ``[N]``.
    """

    def __init__(
        self,
        w_bits: int,
        group_size: int,
        in_features: int,
        out_features: int,
        device: str | torch.device = "cpu",
        bias: bool = False,
        output_dtype: torch.dtype = torch.bfloat16,
    ):
        super().__init__()
        if w_bits not in [4]:
            raise ValueError("Only 4-bit quantization is supported")

        self.w_bits = w_bits
        self.group_size = group_size
        self.in_features = in_features
        self.out_features = out_features
        self.device = device

        assert in_features % group_size == 0, "in_features must be divisible by group_size"
        assert out_features % (32 // self.w_bits) == 0, "out_features must be divisible by (32 // self.w_bits)"

        pack = 32 // self.w_bits
        groups = in_features // group_size
        self.register_buffer("qweight", torch.zeros(in_features, out_features // pack, dtype=torch.int32, device=device))
        self.register_buffer("qscales", torch.zeros(groups, out_features, dtype=output_dtype, device=device))
        self.register_buffer("qzeros", torch.zeros(groups, out_features // pack, dtype=torch.int32, device=device))
        if bias:
            # the reference keeps the bias in bfloat16 whatever the output dtype (gemm.py:435-443)
            self.register_buffer("bias", torch.zeros(out_features, dtype=torch.bfloat16, device=device))
        else:
            self.bias = None

    @classmethod
    def from_linear(
        cls,
        linear_layer: nn.Linear,
        w_bits: int,
        group_size: int,
        scales: torch.Tensor,
        zeros: torch.Tensor,
        output_dtype: torch.dtype = torch.bfloat16,
    ) -> "WQLinear_GEMM":
        """Quantise and pack an ``nn.Linear`` (weight ``[N, K]``) given per-group
        ``scales`` and ``zeros`` of shape ``[K/g, N]``; results equal the
        reference packer's (gemm.py:447-550) word for word, without its
        per-column Python loops."""
        awq_linear = cls(w_bits, group_size, linear_layer.in_features, linear_layer.out_features,
                         linear_layer.weight.device, linear_layer.bias is not None, output_dtype)
        awq_linear.qscales = scales.clone().to(output_dtype)
        if linear_layer.bias is not None:
            awq_linear.bias = linear_layer.bias.clone().to(output_dtype)

        # intweight[k, n] = round(W[n, k] / scales[k // g, n] + zeros[k // g, n]), no clamp
        s_full = scales.repeat_interleave(group_size, dim=0).t()
        z_full = zeros.repeat_interleave(group_size, dim=0).t()
        intweight = torch.round(linear_layer.weight / s_full + z_full).to(torch.int32).t().contiguous()
        awq_linear.qweight = pack_int4(intweight)
        awq_linear.qzeros = pack_int4(zeros.to(torch.int32))
        return awq_linear

    @classmethod
    def from_float(cls, linear_layer: nn.Linear, w_bits: int, group_size: int,
                   output_dtype: torch.dtype = torch.bfloat16) -> "WQLinear_GEMM":
        """Quantise (asymmetric, per group) and pack a CUDA ``nn.Linear`` in one kernel.

        Equal, word for word, to what the reference's quantizer does per layer
        (awq/quantizer.py:150-170): ``pseudo_quantize`` of the weight
        (utils/quantization.py:20-41), then ``from_linear`` on the fake-quantised
        weight with the transposed scales and zero-points."""
        if w_bits != 4:
            raise ValueError("Only 4-bit quantization is supported")
        w = linear_layer.weight.data
        dev = _lib.require_cuda(w)
        _lib.require_b200(dev)
        wcode = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[w.dtype]
        q = cls(w_bits, group_size, linear_layer.in_features, linear_layer.out_features, dev,
                linear_layer.bias is not None, output_dtype)
        if linear_layer.bias is not None:
            q.bias = linear_layer.bias.clone().to(output_dtype)
        w = _contig(w)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().nqb200_quantize_pack(w.data_ptr(), wcode, q.qweight.data_ptr(), q.qscales.data_ptr(),
                                                        q.qzeros.data_ptr(), linear_layer.out_features,
                                                        linear_layer.in_features, group_size,
                                                        _lib.dtype_code(output_dtype), _lib.stream_ptr()))
        return q

    @torch.no_grad()
    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """``[..., K] -> [..., N]``.  The reference switches kernels at 256 tokens
        (gemm.py:558-564); here one library call picks the kernel by M, and the
        bias add (gemm.py:565-566) is fused into it."""
        out_shape = x.shape[:-1] + (self.out_features,)
        x = x.reshape(-1, x.shape[-1])
        out = _w4a16(x, self.qweight, self.qscales, self.qzeros, self.bias, out)
        return out.reshape(out_shape)

    @torch.no_grad()
    def forward_silu_mul(self, x: torch.Tensor) -> torch.Tensor:
        """For a merged gate|up projection: ``silu(y[..., :N/2]) * y[..., N/2:]`` with ``y = forward(x)``,
        bit-identical to running the three steps one after the other.  For decode-sized inputs the
        activation runs inside the kernel that finishes the GEMM; otherwise as a launch of its own."""
        from . import fused
        x2 = x.reshape(-1, x.shape[-1])
        M, K = x2.shape
        lib = _lib.load()
        if x2.is_cuda and M > 0 and lib.nqb200_gemm_gate_up_silu_supported(M, self.out_features, K, self.group_size,
                                                                             _lib.dtype_code(self.qscales.dtype)):
            out = _w4a16(x2, self.qweight, self.qscales, self.qzeros, self.bias, None, silu_mul=True)
        else:
            out = fused.silu_mul(_w4a16(x2, self.qweight, self.qscales, self.qzeros, self.bias, None))
        return out.reshape(x.shape[:-1] + (self.out_features // 2,))

    def fused_supported(self, M: int, *, norm: bool = False, residual: bool = False, silu_mul: bool = False,
                        world: int = 0, slot_bytes: int = 0) -> bool:
        """Whether ``forward_fused`` takes ``M`` tokens with this combination (decode sizes only)."""
        flags = (_lib.FUSE_RMSNORM if norm else 0) | (_lib.FUSE_RESIDUAL if residual else 0) | \
                (_lib.FUSE_SILU_MUL if silu_mul else 0) | (_lib.FUSE_ALLREDUCE if world > 1 else 0)
        return bool(_lib.load().nqb200_gemm_decode_fused_supported(M, self.out_features, self.in_features, self.group_size,
                                                                   _lib.dtype_code(self.qscales.dtype), flags, world, slot_bytes))

    @torch.no_grad()
    def forward_fused(self, x: torch.Tensor, *, norm=None, residual: torch.Tensor | None = None, silu_mul: bool = False,
                      peer=None):
        """The linear with its neighbours in a Qwen3 block, for ``x [M, K]`` where ``fused_supported`` says so:
        ``norm = (ssq, weight, eps)`` makes the input ``RMSNorm(x) * weight`` (``ssq``: per-tile sums of squares of
        ``x``, as returned by the call that produced it); ``residual`` makes the result
        ``(y + residual, ssq)``; ``silu_mul`` as ``forward_silu_mul``; ``peer`` as ``PeerAllReduce`` passes it."""
        return _w4a16(x, self.qweight, self.qscales, self.qzeros, self.bias, None, silu_mul=silu_mul, peer=peer,
                      norm=norm, residual=residual)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}, w_bits={self.w_bits}, group_size={self.group_size}")
