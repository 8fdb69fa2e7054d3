"""Tensor-parallel AWQ linears over the packed checkpoint layout.

The reference has no distributed code; these classes are what a tensor-parallel
engine puts around ``WQLinear_GEMM``.  Sharding never unpacks anything:

* column-parallel (q, k, v, gate, up): rank r keeps output columns
  ``[r*N/tp, (r+1)*N/tp)``, i.e. ``qweight[:, n0/8:n1/8]``, ``qscales[:, n0:n1]``,
  ``qzeros[:, n0/8:n1/8]``.  A packed word holds 8 adjacent columns, so shard
  boundaries must be multiples of 8 columns.  No collective.
* row-parallel (o, down): rank r keeps input rows ``[r*K/tp, (r+1)*K/tp)``, i.e.
  ``qweight[k0:k1]``, ``qscales[k0/g:k1/g]``, ``qzeros[k0/g:k1/g]``.  Boundaries
  must be multiples of the group size.  The partial products are summed with an
  all-reduce; a bias is added on rank 0 only.
* merged column-parallel (qkv, gate_up): several matrices that read the same
  input are sharded separately and the rank's shards concatenated along N, so
  one kernel launch serves all of them.

Each class IS a ``WQLinear_GEMM`` holding the rank's shard (same buffer names, so a
checkpoint's keys address it unchanged); ``.shard`` names the same object.  A
row-parallel linear all-reduces through ``torch.distributed`` (NCCL over NVLink) or,
once a ``PeerAllReduce`` is attached with ``attach_comm``, through the peer-memory
kernels (inside the GEMM's own finishing kernel for decode-sized inputs).
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from .gemm import WQLinear_GEMM

_PACK = 8


def column_shard_bounds(out_features: int, tp_size: int, tp_rank: int) -> tuple[int, int]:
    if out_features % tp_size != 0 or (out_features // tp_size) % _PACK != 0:
        raise ValueError(f"out_features={out_features} cannot be split into {tp_size} column shards of whole packed words")
    per = out_features // tp_size
    return tp_rank * per, (tp_rank + 1) * per


def row_shard_bounds(in_features: int, group_size: int, tp_size: int, tp_rank: int) -> tuple[int, int]:
    if in_features % tp_size != 0 or (in_features // tp_size) % group_size != 0:
        raise ValueError(f"in_features={in_features} cannot be split into {tp_size} row shards on group-{group_size} boundaries")
    per = in_features // tp_size
    return tp_rank * per, (tp_rank + 1) * per


def shard_columns(qweight: torch.Tensor, qscales: torch.Tensor, qzeros: torch.Tensor, tp_size: int, tp_rank: int):
    """The column shard of rank ``tp_rank``: slices of the packed tensors, nothing is unpacked."""
    n0, n1 = column_shard_bounds(qscales.shape[1], tp_size, tp_rank)
    return (qweight[:, n0 // _PACK:n1 // _PACK].contiguous(), qscales[:, n0:n1].contiguous(),
            qzeros[:, n0 // _PACK:n1 // _PACK].contiguous())


def shard_rows(qweight: torch.Tensor, qscales: torch.Tensor, qzeros: torch.Tensor, group_size: int, tp_size: int,
               tp_rank: int):
    """The row shard of rank ``tp_rank``; scales and zero-points split on group boundaries."""
    k0, k1 = row_shard_bounds(qweight.shape[0], group_size, tp_size, tp_rank)
    return (qweight[k0:k1].contiguous(), qscales[k0 // group_size:k1 // group_size].contiguous(),
            qzeros[k0 // group_size:k1 // group_size].contiguous())


class ColumnParallelWQLinear(WQLinear_GEMM):
    """Output columns split across ranks; ``forward`` returns this rank's columns
    (or all of them with ``gather_output=True``)."""

    def __init__(self, w_bits: int, group_size: int, in_features: int, out_features: int, tp_size: int, tp_rank: int,
                 device="cpu", bias: bool = False, output_dtype: torch.dtype = torch.bfloat16,
                 gather_output: bool = False, process_group=None):
        n0, n1 = column_shard_bounds(out_features, tp_size, tp_rank)
        super().__init__(w_bits, group_size, in_features, n1 - n0, device, bias, output_dtype)
        self.tp_size, self.tp_rank, self.group = tp_size, tp_rank, process_group
        self.full_in_features, self.full_out_features, self.gather_output = in_features, out_features, gather_output

    @property
    def shard(self) -> WQLinear_GEMM:
        return self

    def load_full(self, qweight, qscales, qzeros, bias=None) -> None:
        """Copy this rank's slice out of the un-sharded checkpoint tensors."""
        qw, qs, qz = shard_columns(qweight, qscales, qzeros, self.tp_size, self.tp_rank)
        self.qweight.copy_(qw); self.qscales.copy_(qs); self.qzeros.copy_(qz)
        if bias is not None and self.bias is not None:
            n0, n1 = column_shard_bounds(self.full_out_features, self.tp_size, self.tp_rank)
            self.bias.copy_(bias[n0:n1])

    @torch.no_grad()
    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        y = WQLinear_GEMM.forward(self, x, out)
        if self.gather_output and self.tp_size > 1:
            parts = [torch.empty_like(y) for _ in range(self.tp_size)]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            y = torch.cat(parts, dim=-1)
        return y


class MergedColumnParallelWQLinear(WQLinear_GEMM):
    """Several column-parallel matrices with a common input (q/k/v or gate/up) as one
    launch: each is sharded on its own, the rank's shards are concatenated along N.
    ``forward`` returns the concatenation; ``split`` cuts it back."""

    def __init__(self, w_bits: int, group_size: int, in_features: int, output_sizes: Sequence[int], tp_size: int,
                 tp_rank: int, device="cpu", output_dtype: torch.dtype = torch.bfloat16):
        shard_sizes = []
        for n in output_sizes:
            n0, n1 = column_shard_bounds(n, tp_size, tp_rank)
            shard_sizes.append(n1 - n0)
        super().__init__(w_bits, group_size, in_features, sum(shard_sizes), device, False, output_dtype)
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self.output_sizes, self.shard_sizes = list(output_sizes), shard_sizes

    @property
    def shard(self) -> WQLinear_GEMM:
        return self

    @classmethod
    def from_shards(cls, parts: Sequence[ColumnParallelWQLinear]) -> "MergedColumnParallelWQLinear":
        """Concatenate the shards that ``parts`` already hold (packing is local to 8-column words, so
        this is a plain ``cat`` along N)."""
        p0 = parts[0]
        m = cls(p0.w_bits, p0.group_size, p0.in_features, [p.full_out_features for p in parts], p0.tp_size, p0.tp_rank,
                "meta", p0.qscales.dtype)
        m.device = p0.qweight.device
        m.qweight = torch.cat([p.qweight for p in parts], dim=1).contiguous()
        m.qscales = torch.cat([p.qscales for p in parts], dim=1).contiguous()
        m.qzeros = torch.cat([p.qzeros for p in parts], dim=1).contiguous()
        return m

    def load_full(self, parts: Sequence[tuple[torch.Tensor, torch.Tensor, torch.Tensor]]) -> None:
        """``parts[i] = (qweight, qscales, qzeros)`` of matrix i, un-sharded."""
        assert len(parts) == len(self.output_sizes)
        shards = [shard_columns(qw, qs, qz, self.tp_size, self.tp_rank) for (qw, qs, qz) in parts]
        self.qweight.copy_(torch.cat([s[0] for s in shards], dim=1))
        self.qscales.copy_(torch.cat([s[1] for s in shards], dim=1))
        self.qzeros.copy_(torch.cat([s[2] for s in shards], dim=1))

    def split(self, y: torch.Tensor):
        return torch.split(y, self.shard_sizes, dim=-1)


class RowParallelWQLinear(WQLinear_GEMM):
    """Input rows split across ranks on group boundaries; ``forward`` takes this
    rank's slice of the input features and returns the all-reduced output."""

    def __init__(self, w_bits: int, group_size: int, in_features: int, out_features: int, tp_size: int, tp_rank: int,
                 device="cpu", bias: bool = False, output_dtype: torch.dtype = torch.bfloat16,
                 reduce_output: bool = True, process_group=None):
        k0, k1 = row_shard_bounds(in_features, group_size, tp_size, tp_rank)
        # the bias is added once: on rank 0
        super().__init__(w_bits, group_size, k1 - k0, out_features, device, bias and tp_rank == 0, output_dtype)
        self.tp_size, self.tp_rank, self.group = tp_size, tp_rank, process_group
        self.full_in_features, self.full_out_features = in_features, out_features
        self.reduce_output = reduce_output
        self.comm = None  # a PeerAllReduce, see attach_comm

    @property
    def shard(self) -> WQLinear_GEMM:
        return self

    def attach_comm(self, comm) -> None:
        """Route the all-reduce through ``comm`` (a ``PeerAllReduce``): reduced over peer memory by the kernel
        that finishes the GEMM where the library supports the shape, by the stand-alone peer kernels for
        larger messages, by NCCL beyond the communicator's slot size.  ``None`` goes back to NCCL."""
        self.comm = comm

    def load_full(self, qweight, qscales, qzeros, bias=None) -> None:
        qw, qs, qz = shard_rows(qweight, qscales, qzeros, self.group_size, self.tp_size, self.tp_rank)
        self.qweight.copy_(qw); self.qscales.copy_(qs); self.qzeros.copy_(qz)
        if bias is not None and self.bias is not None:
            self.bias.copy_(bias)

    def input_slice(self, x_full: torch.Tensor) -> torch.Tensor:
        k0, k1 = row_shard_bounds(self.full_in_features, self.group_size, self.tp_size, self.tp_rank)
        return x_full[..., k0:k1]

    @torch.no_grad()
    def forward_local(self, x_shard: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """This rank's partial product, not reduced."""
        return WQLinear_GEMM.forward(self, x_shard, out)

    @torch.no_grad()
    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        if not self.reduce_output or self.tp_size == 1:
            return self.forward_local(x_shard)
        if self.comm is not None:
            lead = x_shard.shape[:-1]
            y = self.comm.linear_all_reduce(self, x_shard.reshape(-1, x_shard.shape[-1]))
            return y.reshape(lead + (self.out_features,))
        y = self.forward_local(x_shard)
        dist.all_reduce(y, group=self.group)
        return y

    def residual_fusable(self, M: int) -> bool:
        """Whether ``forward_residual`` runs in the linear's own two launches for ``M`` tokens."""
        if self.tp_size == 1:
            return self.fused_supported(M, residual=True)
        return self.comm is not None and self.comm.fused_residual_supported(self, M)

    @torch.no_grad()
    def forward_residual(self, x_shard: torch.Tensor, residual: torch.Tensor):
        """``(all_reduce(linear(x)) + residual, its per-tile sums of squares)`` where ``residual_fusable``."""
        if self.tp_size > 1:
            return self.comm.linear_all_reduce_residual(self, x_shard, residual)
        return self.forward_fused(x_shard, residual=residual)
