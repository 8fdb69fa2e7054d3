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

Collectives go through ``torch.distributed`` (NCCL over NVLink on GPUs).
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


class ColumnParallelWQLinear(nn.Module):
    """Output columns split across ranks; ``forward`` returns this rank's columns
    (or all of them with ``gather_output=True``)."""

    def __init__(self, w_bits: int, group_size: int, in_features: int, out_features: int, tp_size: int, tp_rank: int,
                 device="cpu", bias: bool = False, output_dtype: torch.dtype = torch.bfloat16,
                 gather_output: bool = False, process_group=None):
        super().__init__()
        n0, n1 = column_shard_bounds(out_features, tp_size, tp_rank)
        self.tp_size, self.tp_rank, self.group = tp_size, tp_rank, process_group
        self.in_features, self.out_features, self.gather_output = in_features, out_features, gather_output
        self.shard = WQLinear_GEMM(w_bits, group_size, in_features, n1 - n0, device, bias, output_dtype)

    def load_full(self, qweight, qscales, qzeros, bias=None) -> None:
        """Copy this rank's slice out of the un-sharded checkpoint tensors."""
        qw, qs, qz = shard_columns(qweight, qscales, qzeros, self.tp_size, self.tp_rank)
        self.shard.qweight.copy_(qw); self.shard.qscales.copy_(qs); self.shard.qzeros.copy_(qz)
        if bias is not None and self.shard.bias is not None:
            n0, n1 = column_shard_bounds(self.out_features, self.tp_size, self.tp_rank)
            self.shard.bias.copy_(bias[n0:n1])

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.shard(x)
        if self.gather_output and self.tp_size > 1:
            parts = [torch.empty_like(y) for _ in range(self.tp_size)]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            y = torch.cat(parts, dim=-1)
        return y


class MergedColumnParallelWQLinear(nn.Module):
    """Several column-parallel matrices with a common input (q/k/v or gate/up) as one
    launch: each is sharded on its own, the rank's shards are concatenated along N.
    ``forward`` returns the concatenation; ``split`` cuts it back."""

    def __init__(self, w_bits: int, group_size: int, in_features: int, output_sizes: Sequence[int], tp_size: int,
                 tp_rank: int, device="cpu", output_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self.output_sizes = list(output_sizes)
        self.shard_sizes = []
        for n in self.output_sizes:
            n0, n1 = column_shard_bounds(n, tp_size, tp_rank)
            self.shard_sizes.append(n1 - n0)
        self.shard = WQLinear_GEMM(w_bits, group_size, in_features, sum(self.shard_sizes), device, False, output_dtype)

    def load_full(self, parts: Sequence[tuple[torch.Tensor, torch.Tensor, torch.Tensor]]) -> None:
        """``parts[i] = (qweight, qscales, qzeros)`` of matrix i, un-sharded."""
        assert len(parts) == len(self.output_sizes)
        shards = [shard_columns(qw, qs, qz, self.tp_size, self.tp_rank) for (qw, qs, qz) in parts]
        self.shard.qweight.copy_(torch.cat([s[0] for s in shards], dim=1))
        self.shard.qscales.copy_(torch.cat([s[1] for s in shards], dim=1))
        self.shard.qzeros.copy_(torch.cat([s[2] for s in shards], dim=1))

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.shard(x)

    def split(self, y: torch.Tensor):
        return torch.split(y, self.shard_sizes, dim=-1)


class RowParallelWQLinear(nn.Module):
    """Input rows split across ranks on group boundaries; ``forward`` takes this
    rank's slice of the input features and returns the all-reduced output."""

    def __init__(self, w_bits: int, group_size: int, in_features: int, out_features: int, tp_size: int, tp_rank: int,
                 device="cpu", bias: bool = False, output_dtype: torch.dtype = torch.bfloat16,
                 reduce_output: bool = True, process_group=None):
        super().__init__()
        k0, k1 = row_shard_bounds(in_features, group_size, tp_size, tp_rank)
        self.tp_size, self.tp_rank, self.group = tp_size, tp_rank, process_group
        self.in_features, self.out_features, self.group_size = in_features, out_features, group_size
        self.reduce_output = reduce_output
        # the bias is added once: on rank 0
        self.shard = WQLinear_GEMM(w_bits, group_size, k1 - k0, out_features, device, bias and tp_rank == 0, output_dtype)

    def load_full(self, qweight, qscales, qzeros, bias=None) -> None:
        qw, qs, qz = shard_rows(qweight, qscales, qzeros, self.group_size, self.tp_size, self.tp_rank)
        self.shard.qweight.copy_(qw); self.shard.qscales.copy_(qs); self.shard.qzeros.copy_(qz)
        if bias is not None and self.shard.bias is not None:
            self.shard.bias.copy_(bias)

    def input_slice(self, x_full: torch.Tensor) -> torch.Tensor:
        k0, k1 = row_shard_bounds(self.in_features, self.group_size, self.tp_size, self.tp_rank)
        return x_full[..., k0:k1]

    @torch.no_grad()
    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        y = self.shard(x_shard)
        if self.reduce_output and self.tp_size > 1:
            dist.all_reduce(y, group=self.group)
        return y
