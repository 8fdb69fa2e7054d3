"""Quantised Qwen3 on the B200 W4A16 linears: the caller of the hot path.

Module tree, constructor arguments and parameter / buffer names follow the
reference's ``nanoquantization/models/qwen3_quantized.py`` (attention :10-102,
MLP :105-152, block :155-215, model :218-273, causal LM :276-341), so a
reference checkpoint's keys (``model.layers.{i}.self_attn.q_proj.qweight`` ...)
load by name.  Differences, all additive:

* ``tp_size`` / ``tp_rank``: every linear is one of the tensor-parallel classes of
  ``layers/parallel.py`` holding this rank's shard (q/k/v/gate/up column-parallel
  by whole heads, o/down row-parallel on group boundaries); the row-parallel
  classes do the all-reduce (NCCL, or peer memory once ``attach_peer_comm``);
* besides the reference's full-sequence ``forward(x, position_ids)`` (causal
  SDPA, no cache) there is ``forward_tokens`` for a serving engine: flattened
  tokens, attention delegated to a callable that owns the paged KV cache;
* ``fuse_projections()`` concatenates the packed q/k/v and gate/up tensors
  along N (packing is local to 8-column words, so this is a plain ``cat``) so
  that each pair or triple costs one launch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..layers import fused
from ..layers.gemm import WQLinear_GEMM  # noqa: F401  (the class every projection derives from)
from ..layers.parallel import ColumnParallelWQLinear, MergedColumnParallelWQLinear, RowParallelWQLinear


@dataclass
class Qwen3Config:
    num_hidden_layers: int
    vocab_size: int
    hidden_size: int
    total_num_heads: int
    total_num_kv_heads: int
    max_position_embeddings: int
    intermediate_size: int
    w_bits: int = 4
    group_size: int = 128
    head_dim: Optional[int] = 128
    tie_word_embeddings: bool = False
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-6


# the architectures the benchmark configurations name
QWEN3_SHAPES = {
    "qwen3-0.6b": dict(num_hidden_layers=28, hidden_size=1024, total_num_heads=16, total_num_kv_heads=8, intermediate_size=3072),
    "qwen3-8b": dict(num_hidden_layers=36, hidden_size=4096, total_num_heads=32, total_num_kv_heads=8, intermediate_size=12288),
    "qwen3-32b": dict(num_hidden_layers=64, hidden_size=5120, total_num_heads=64, total_num_kv_heads=8, intermediate_size=25600),
}


class RMSNorm(nn.Module):
    """fp32 ``x * rsqrt(mean(x^2) + eps)``, cast back, times weight (reference layers/norm.py:18-32)."""

    def __init__(self, norm_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.norm_size, self.eps = norm_size, eps
        self.weight = nn.Parameter(torch.ones(norm_size))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + self.eps)
        return xf.to(x.dtype) * self.weight


class RotaryCache(nn.Module):
    """Half-split rotary embedding with a ``[max_pos, 1, head_dim]`` cos|sin table
    (reference layers/rope.py:5-45)."""

    def __init__(self, head_dim: int, max_position_embeddings: int, base: float = 10000):
        super().__init__()
        inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
        ang = torch.outer(torch.arange(max_position_embeddings, dtype=torch.float32), inv)
        self.register_buffer("cos_sin_cache", torch.cat([ang.cos(), ang.sin()], dim=-1).unsqueeze(1), persistent=False)

    @staticmethod
    def _rotate(x, cos, sin):
        a, b = x.float().chunk(2, dim=-1)
        return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1).to(x.dtype)

    def forward(self, q: torch.Tensor, k: torch.Tensor, position_ids: torch.Tensor):
        cos, sin = self.cos_sin_cache[position_ids].chunk(2, dim=-1)
        return self._rotate(q, cos, sin), self._rotate(k, cos, sin)


class Qwen3QuantizedAttention(nn.Module):
    def __init__(self, hidden_size, total_num_heads, total_num_kv_heads, max_position_embeddings, w_bits=4,
                 group_size=128, head_dim=None, rope_theta=10000, rms_norm_eps=1e-6, *, tp_size=1, tp_rank=0,
                 tp_group=None, device="cpu", dtype=torch.bfloat16):
        super().__init__()
        assert total_num_heads % tp_size == 0 and total_num_kv_heads % tp_size == 0
        self.head_dim = head_dim or hidden_size // total_num_heads
        self.hidden_size = hidden_size
        self.num_heads, self.num_kv_heads = total_num_heads // tp_size, total_num_kv_heads // tp_size
        self.tp_size, self.tp_group = tp_size, tp_group
        self.rope = RotaryCache(self.head_dim, max_position_embeddings, rope_theta)
        col = lambda n: ColumnParallelWQLinear(w_bits, group_size, hidden_size, n, tp_size, tp_rank, device, False, dtype,  # noqa: E731
                                               process_group=tp_group)
        self.q_proj = col(total_num_heads * self.head_dim)
        self.k_proj = col(total_num_kv_heads * self.head_dim)
        self.v_proj = col(total_num_kv_heads * self.head_dim)
        self.o_proj = RowParallelWQLinear(w_bits, group_size, total_num_heads * self.head_dim, hidden_size, tp_size, tp_rank,
                                          device, False, dtype, process_group=tp_group)
        self.q_norm = RMSNorm(self.head_dim, rms_norm_eps)
        self.k_norm = RMSNorm(self.head_dim, rms_norm_eps)
        self.qkv_proj = None

    def fuse_projections(self):
        self.qkv_proj = MergedColumnParallelWQLinear.from_shards([self.q_proj, self.k_proj, self.v_proj])
        self.q_proj = self.k_proj = self.v_proj = None

    def _qkv(self, x):
        if self.qkv_proj is not None:
            nq, nk = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
            return self.qkv_proj(x).split([nq, nk, nk], dim=-1)
        return self.q_proj(x), self.k_proj(x), self.v_proj(x)

    def forward(self, x: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
        """Full-sequence causal attention without a cache, as the reference (:66-102)."""
        bs = x.shape[0]
        if position_ids.dim() == 1:
            position_ids = position_ids.unsqueeze(0)
        q, k, v = self._qkv(x)
        q = self.q_norm(q.view(bs, -1, self.num_heads, self.head_dim))
        k = self.k_norm(k.view(bs, -1, self.num_kv_heads, self.head_dim))
        v = v.view(bs, -1, self.num_kv_heads, self.head_dim)
        q, k = self.rope(q, k, position_ids)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                           enable_gqa=self.num_heads != self.num_kv_heads)
        o = o.transpose(1, 2).reshape(bs, -1, self.num_heads * self.head_dim)
        return self.o_proj(o)

    def fusable(self, T: int) -> bool:
        """Whether ``forward_tokens`` can take the input norm into q/k/v and the residual add into o_proj for T tokens."""
        if self.qkv_proj is None or not self.qkv_proj.qweight.is_cuda or not self.qkv_proj.fused_supported(T, norm=True):
            return False
        return self.o_proj.residual_fusable(T)

    def forward_tokens(self, x: torch.Tensor, positions: torch.Tensor, attend: Callable, norm=None,
                       residual: Optional[torch.Tensor] = None):
        """``x`` is ``[T, hidden]``; ``attend(q, k, v)`` stores k, v in its cache and returns ``[T, Hq, D]``
        (called with ``stored=True`` when this method already stored them through ``attend.kv_target``).
        One launch for q/k/v (when fused), one for QK-norm + rotary embedding."""
        T = x.shape[0]
        nq, nk = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        if norm is not None:  # x is the residual stream; its RMSNorm is taken inside the linear
            qkv = self.qkv_proj.forward_fused(x, norm=norm)
        elif self.qkv_proj is not None:
            qkv = self.qkv_proj(x)
        else:
            qkv = torch.cat([self.q_proj(x), self.k_proj(x), self.v_proj(x)], dim=-1)
        stored = False
        if self.head_dim == 128:
            # an attend() that exposes its cache (k_cache, v_cache, slots) gets k and v stored by this launch
            kv_target = getattr(attend, "kv_target", None)
            fused.qknorm_rope_(qkv, self.q_norm.weight, self.k_norm.weight, self.rope.cos_sin_cache, positions,
                               self.num_heads, self.num_kv_heads, self.head_dim, self.q_norm.eps, kv_target)
            stored = kv_target is not None
            q = qkv[:, :nq].view(T, self.num_heads, self.head_dim)
            k = qkv[:, nq:nq + nk].view(T, self.num_kv_heads, self.head_dim)
        else:
            q = self.q_norm(qkv[:, :nq].reshape(T, self.num_heads, self.head_dim))
            k = self.k_norm(qkv[:, nq:nq + nk].reshape(T, self.num_kv_heads, self.head_dim))
            q, k = self.rope(q, k, positions)
        v = qkv[:, nq + nk:].view(T, self.num_kv_heads, self.head_dim)
        o = (attend(q, k, v, stored=True) if stored else attend(q, k, v)).reshape(T, nq)
        if residual is not None:  # (new residual stream, its per-tile sums of squares) from o_proj's own launches
            return self.o_proj.forward_residual(o, residual)
        return self.o_proj(o)


class Qwen3QuantizedMLP(nn.Module):
    def __init__(self, hidden_size, intermediate_size, w_bits=4, group_size=128, *, tp_size=1, tp_rank=0, tp_group=None,
                 device="cpu", dtype=torch.bfloat16):
        super().__init__()
        assert intermediate_size % tp_size == 0 and (intermediate_size // tp_size) % group_size == 0
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size // tp_size
        self.tp_size, self.tp_group = tp_size, tp_group
        col = lambda: ColumnParallelWQLinear(w_bits, group_size, hidden_size, intermediate_size, tp_size, tp_rank, device,  # noqa: E731
                                             False, dtype, process_group=tp_group)
        self.up_proj = col()
        self.gate_proj = col()
        self.down_proj = RowParallelWQLinear(w_bits, group_size, intermediate_size, hidden_size, tp_size, tp_rank, device,
                                             False, dtype, process_group=tp_group)
        self.gate_up_proj = None

    def fuse_projections(self):
        self.gate_up_proj = MergedColumnParallelWQLinear.from_shards([self.gate_proj, self.up_proj])
        self.gate_proj = self.up_proj = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.gate_up_proj is not None:
            y1, y2 = self.gate_up_proj(x).chunk(2, dim=-1)
        else:
            y1, y2 = self.gate_proj(x), self.up_proj(x)
        return self.down_proj(F.silu(y1) * y2)

    def fusable(self, T: int) -> bool:
        if (self.gate_up_proj is None or not self.gate_up_proj.qweight.is_cuda
                or not self.gate_up_proj.fused_supported(T, norm=True, silu_mul=True)):
            return False
        return self.down_proj.residual_fusable(T)

    def forward_tokens(self, x: torch.Tensor, norm=None, residual: Optional[torch.Tensor] = None):
        if self.gate_up_proj is None:
            return self.forward(x)
        if residual is not None:  # as in the attention: norm inside gate_up, residual add inside down_proj
            y = self.gate_up_proj.forward_fused(x, norm=norm, silu_mul=True)
            return self.down_proj.forward_residual(y, residual)
        return self.down_proj(self.gate_up_proj.forward_silu_mul(x))


class Qwen3QuantizedBlock(nn.Module):
    def __init__(self, hidden_size, total_num_heads, total_num_kv_heads, max_position_embeddings, intermediate_size,
                 w_bits=4, group_size=128, head_dim=None, rope_theta=10000, rms_norm_eps=1e-6, **kw):
        super().__init__()
        self.self_attn = Qwen3QuantizedAttention(hidden_size, total_num_heads, total_num_kv_heads, max_position_embeddings,
                                                 w_bits, group_size, head_dim, rope_theta, rms_norm_eps, **kw)
        self.mlp = Qwen3QuantizedMLP(hidden_size, intermediate_size, w_bits, group_size, **kw)
        self.input_layernorm = RMSNorm(hidden_size, rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(hidden_size, rms_norm_eps)
        self._fusable: dict[int, bool] = {}  # per token count: can the norms and residual adds go into the linears?

    def forward(self, x, position_ids):
        x = x + self.self_attn(self.input_layernorm(x), position_ids)
        return x + self.mlp(self.post_attention_layernorm(x))

    def forward_tokens(self, x, residual, positions, attend, ssq=None):
        """State between sub-layers: either ``x`` is a sub-layer output still to be added to ``residual`` (``ssq``
        None), or ``x`` is None, ``residual`` is already the updated stream and ``ssq`` holds its per-tile sums of
        squares.  The second form is what the decode-sized linears produce and consume themselves (norm taken
        inside q/k/v and gate/up, residual add inside o_proj and down_proj): no launch for the norms.
        Returns the same triple."""
        T = residual.shape[0] if x is None else x.shape[0]
        fuse = self._fusable.get(T)
        if fuse is None:
            fuse = self._fusable[T] = bool(T <= 16 and self.self_attn.fusable(T) and self.mlp.fusable(T))
        if not fuse:
            if x is None:  # a fused layer ahead of an unfused one does not happen (same shapes), but stay correct
                h = fused.add_rmsnorm(residual, None, self.input_layernorm.weight, self.input_layernorm.eps)[0]
            else:
                h, residual = fused.add_rmsnorm(x, residual, self.input_layernorm.weight, self.input_layernorm.eps)
            a = self.self_attn.forward_tokens(h, positions, attend)
            h, residual = fused.add_rmsnorm(a, residual, self.post_attention_layernorm.weight, self.post_attention_layernorm.eps)
            return self.mlp.forward_tokens(h), residual, None
        if ssq is None:
            h, residual = fused.add_rmsnorm(x, residual, self.input_layernorm.weight, self.input_layernorm.eps)
            residual, ssq = self.self_attn.forward_tokens(h, positions, attend, None, residual)
        else:
            residual, ssq = self.self_attn.forward_tokens(residual, positions, attend,
                                                          (ssq, self.input_layernorm.weight, self.input_layernorm.eps), residual)
        residual, ssq = self.mlp.forward_tokens(residual, (ssq, self.post_attention_layernorm.weight,
                                                           self.post_attention_layernorm.eps), residual)
        return None, residual, ssq


class Qwen3QuantizedModel(nn.Module):
    def __init__(self, num_hidden_layers, vocab_size, hidden_size, total_num_heads, total_num_kv_heads,
                 max_position_embeddings, intermediate_size, w_bits=4, group_size=128, head_dim=None, rope_theta=10000,
                 rms_norm_eps=1e-6, **kw):
        super().__init__()
        self.layers = nn.ModuleList([
            Qwen3QuantizedBlock(hidden_size, total_num_heads, total_num_kv_heads, max_position_embeddings,
                                intermediate_size, w_bits, group_size, head_dim, rope_theta, rms_norm_eps, **kw)
            for _ in range(num_hidden_layers)])
        self.norm = RMSNorm(hidden_size, rms_norm_eps)
        self.embed_tokens = nn.Embedding(vocab_size, hidden_size, device=kw.get("device", "cpu"),
                                         dtype=kw.get("dtype", torch.bfloat16))

    def forward(self, x, position_ids):
        x = self.embed_tokens(x)
        for layer in self.layers:
            x = layer(x, position_ids)
        return self.norm(x)

    def forward_tokens(self, token_ids, positions, attend_for_layer: Callable[[int], Callable]):
        x, residual, ssq = self.embed_tokens(token_ids), None, None
        for i, layer in enumerate(self.layers):
            x, residual, ssq = layer.forward_tokens(x, residual, positions, attend_for_layer(i), ssq)
        if x is None:  # the last linear already added its output to the residual stream
            return fused.add_rmsnorm(residual, None, self.norm.weight, self.norm.eps)[0]
        return fused.add_rmsnorm(x, residual, self.norm.weight, self.norm.eps)[0]


class Qwen3QuantizedForCausalLM(nn.Module):
    def __init__(self, num_hidden_layers, vocab_size, hidden_size, total_num_heads, total_num_kv_heads,
                 max_position_embeddings, intermediate_size, w_bits=4, group_size=128, head_dim=None,
                 tie_word_embeddings=False, rope_theta=10000, rms_norm_eps=1e-6, *, tp_size=1, tp_rank=0, tp_group=None,
                 device="cpu", dtype=torch.bfloat16):
        super().__init__()
        kw = dict(tp_size=tp_size, tp_rank=tp_rank, tp_group=tp_group, device=device, dtype=dtype)
        self.tp_size, self.tp_rank, self.tp_group = tp_size, tp_rank, tp_group
        self.tp_comm = None  # a PeerAllReduce, attached by attach_peer_comm()
        self.model = Qwen3QuantizedModel(num_hidden_layers, vocab_size, hidden_size, total_num_heads, total_num_kv_heads,
                                         max_position_embeddings, intermediate_size, w_bits, group_size, head_dim,
                                         rope_theta, rms_norm_eps, **kw)
        # vocabulary-parallel head: this rank scores rows [v0, v1) of the vocabulary
        assert vocab_size % tp_size == 0
        self.vocab_size, self.vocab_shard = vocab_size, vocab_size // tp_size
        self.lm_head = nn.Linear(hidden_size, self.vocab_shard, device=device, dtype=dtype)
        if tie_word_embeddings and tp_size == 1:
            self.lm_head.weight.data = self.model.embed_tokens.weight.data
        self.to(device)
        for m in self.modules():  # norms and embeddings in the model dtype, like the reference's default-dtype construction
            if isinstance(m, RMSNorm):
                m.weight.data = m.weight.data.to(dtype)

    @classmethod
    def from_config(cls, cfg: Qwen3Config, **kw) -> "Qwen3QuantizedForCausalLM":
        return cls(cfg.num_hidden_layers, cfg.vocab_size, cfg.hidden_size, cfg.total_num_heads, cfg.total_num_kv_heads,
                   cfg.max_position_embeddings, cfg.intermediate_size, cfg.w_bits, cfg.group_size, cfg.head_dim,
                   cfg.tie_word_embeddings, cfg.rope_theta, cfg.rms_norm_eps, **kw)

    def attach_peer_comm(self, comm) -> None:
        """Route the all-reduces after o_proj and down_proj through a ``PeerAllReduce``."""
        self.tp_comm = comm
        for layer in self.model.layers:
            layer.self_attn.o_proj.attach_comm(comm)
            layer.mlp.down_proj.attach_comm(comm)
            layer._fusable.clear()

    def fuse_projections(self) -> None:
        for layer in self.model.layers:
            layer.self_attn.fuse_projections()
            layer.mlp.fuse_projections()
            layer._fusable.clear()

    def forward(self, x, position_ids):
        return self.model(x, position_ids)

    def compute_loss(self, x, labels):
        pos = torch.arange(x.shape[1], dtype=torch.int32, device=x.device).unsqueeze(0)
        logits = self.lm_head(self.model(x, pos))
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.view(-1))

    @torch.no_grad()
    def greedy_tokens(self, hidden: torch.Tensor) -> torch.Tensor:
        """Arg-max over the whole vocabulary from this rank's slice of the head: local max and
        index, then one small all-gather."""
        logits = self.lm_head(hidden).float()
        val, idx = logits.max(dim=-1)
        idx = idx + self.tp_rank * self.vocab_shard
        if self.tp_size == 1:
            return idx
        pair = torch.stack([val, idx.to(val.dtype)], dim=-1).contiguous()
        allp = [torch.empty_like(pair) for _ in range(self.tp_size)]
        dist.all_gather(allp, pair, group=self.tp_group)
        allp = torch.stack(allp)                       # [tp, B, 2]
        best = allp[..., 0].argmax(dim=0)              # [B]
        return allp[best, torch.arange(pair.shape[0], device=pair.device), 1].to(torch.long)
