"""A small serving engine around the quantised model: paged KV cache, block
manager, continuous-batching scheduler, model runner with CUDA-graph decode.

The reference has none of this (its only execution is a full-sequence forward
for a loss, models/qwen3_quantized.py:326-341); it exists so that the W4A16
linears can be measured where they are used: prefill of batched prompts and
greedy decode steps over a KV cache.  Attention is not the subject here: at
prefill it is PyTorch's scaled_dot_product_attention per prompt; at decode it is
flash_attn's paged-KV kernel when that library loads on this GPU, else
scaled_dot_product_attention over the gathered pages of each sequence.

Layout: per layer two tensors ``[num_blocks, block_size, kv_heads, head_dim]``;
a sequence owns a list of blocks; ``slot = block * block_size + offset``.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence as Seq

import torch
import torch.nn.functional as F


@dataclass
class Sequence:
    seq_id: int
    prompt: list[int]
    max_new_tokens: int
    output: list[int] = field(default_factory=list)
    blocks: list[int] = field(default_factory=list)
    prefilled: bool = False
    carried: list[int] = field(default_factory=list)  # tokens generated before a preemption (now part of the prompt)

    def __len__(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def finished(self) -> bool:
        return len(self.output) >= self.max_new_tokens


class BlockManager:
    """Free-list allocator of KV-cache blocks."""

    def __init__(self, num_blocks: int, block_size: int):
        self.block_size = block_size
        self.free = deque(range(num_blocks))

    def blocks_needed(self, n_tokens: int) -> int:
        return -(-n_tokens // self.block_size)

    def can_allocate(self, n_tokens: int) -> bool:
        return self.blocks_needed(n_tokens) <= len(self.free)

    def ensure(self, seq: Sequence, n_tokens: int) -> bool:
        """Grow ``seq`` to hold ``n_tokens``; False (and no change) if the pool is exhausted."""
        need = self.blocks_needed(n_tokens) - len(seq.blocks)
        if need > len(self.free):
            return False
        for _ in range(max(need, 0)):
            seq.blocks.append(self.free.popleft())
        return True

    def release(self, seq: Sequence) -> None:
        self.free.extend(seq.blocks)
        seq.blocks = []


class PagedKVCache:
    def __init__(self, num_layers, num_blocks, block_size, kv_heads, head_dim, dtype, device):
        shape = (num_blocks, block_size, kv_heads, head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.block_size = block_size

    def write(self, layer: int, slots: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        self.k[layer].view(-1, *k.shape[1:]).index_copy_(0, slots, k)
        self.v[layer].view(-1, *v.shape[1:]).index_copy_(0, slots, v)


class Scheduler:
    """Prefill has priority: waiting prompts are admitted while blocks and the token budget last;
    otherwise every running sequence decodes one token.  A sequence that cannot grow is preempted
    (its blocks are released and it returns to the waiting queue to be prefilled again)."""

    def __init__(self, blocks: BlockManager, max_batch: int, max_prefill_tokens: int):
        self.blocks, self.max_batch, self.max_prefill_tokens = blocks, max_batch, max_prefill_tokens
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []

    def add(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    def step(self) -> tuple[str, list[Sequence]]:
        batch, tokens = [], 0
        while self.waiting and len(self.running) + len(batch) < self.max_batch:
            s = self.waiting[0]
            n = len(s)
            if tokens + n > self.max_prefill_tokens and batch:
                break
            if not self.blocks.ensure(s, n + 1):
                break
            self.waiting.popleft()
            batch.append(s)
            tokens += n
        if batch:
            return "prefill", batch
        ready = []
        i = 0
        while i < len(self.running):
            s = self.running[i]
            if self.blocks.ensure(s, len(s) + 1):
                ready.append(s)
                i += 1
                continue
            # no block left for s to grow into: preempt the youngest running sequence and try again
            victim = self.running.pop()
            self.blocks.release(victim)
            if victim in ready:
                ready.remove(victim)
            victim.carried += victim.output
            victim.max_new_tokens -= len(victim.output)
            victim.prompt, victim.output, victim.prefilled = victim.prompt + victim.output, [], False
            self.waiting.appendleft(victim)
        return "decode", ready

    def finish_step(self, kind: str, batch: list[Sequence]) -> list[Sequence]:
        done = []
        if kind == "prefill":
            self.running.extend(batch)
        for s in batch:
            if s.finished:
                done.append(s)
                self.running.remove(s)
                self.blocks.release(s)
        return done


class LLMEngine:
    def __init__(self, model, num_blocks: int, block_size: int = 256, max_batch: int = 64,
                 max_prefill_tokens: int = 16384, use_cuda_graph: bool = True):
        self.model = model
        attn = model.model.layers[0].self_attn
        self.device = model.lm_head.weight.device
        self.dtype = model.lm_head.weight.dtype
        self.kv_heads, self.q_heads, self.head_dim = attn.num_kv_heads, attn.num_heads, attn.head_dim
        self.block_size = block_size
        # one block more than the allocator hands out: padding rows of a bucketed decode batch write there
        self.cache = PagedKVCache(len(model.model.layers), num_blocks + 1, block_size, self.kv_heads, self.head_dim,
                                  self.dtype, self.device)
        self.scratch_block = num_blocks
        self.blocks = BlockManager(num_blocks, block_size)
        self.scheduler = Scheduler(self.blocks, max_batch, max_prefill_tokens)
        self.use_cuda_graph = use_cuda_graph
        self.paged_attention = self._probe_flash_attn() if block_size % 256 == 0 else None
        self._graphs: dict[tuple[int, int], tuple] = {}
        self._warm_stream = None  # one side stream for every graph warm-up (scratch buffers are kept per stream)
        self._next_id = 0
        self.max_tokens_per_sequence = num_blocks * block_size

    # ------------------------------------------------------------------ attention
    def _probe_flash_attn(self):
        """flash_attn's paged decode kernel if this build of it runs on this GPU, else None (the
        fallback gathers the pages and calls scaled_dot_product_attention)."""
        try:
            from flash_attn import flash_attn_with_kvcache
            q = torch.zeros(1, 1, self.q_heads, self.head_dim, dtype=self.dtype, device=self.device)
            bt = torch.zeros(1, 1, dtype=torch.int32, device=self.device)
            ln = torch.ones(1, dtype=torch.int32, device=self.device)
            flash_attn_with_kvcache(q, self.cache.k[0], self.cache.v[0], cache_seqlens=ln, block_table=bt, causal=True)
            torch.cuda.synchronize()
            return flash_attn_with_kvcache
        except Exception:  # not built for this architecture, or not importable
            return None

    def _prefill_attend(self, layer: int, slots: torch.Tensor, lens: list[int]) -> Callable:
        def attend(q, k, v, stored=False):
            if not stored:
                self.cache.write(layer, slots, k, v)
            outs, o = [], 0
            for n in lens:
                qs, ks, vs = (t[o:o + n].transpose(0, 1).unsqueeze(0) for t in (q, k, v))
                outs.append(F.scaled_dot_product_attention(qs, ks, vs, is_causal=True,
                                                           enable_gqa=self.q_heads != self.kv_heads)[0].transpose(0, 1))
                o += n
            return torch.cat(outs, dim=0)
        attend.kv_target = (self.cache.k[layer], self.cache.v[layer], slots)
        return attend

    def _decode_attend(self, layer: int, slots: torch.Tensor, block_tables: torch.Tensor, ctx_lens: torch.Tensor,
                       max_blocks: int, ctx_i32=None, bt_i32=None) -> Callable:
        def attend(q, k, v, stored=False):
            if not stored:
                self.cache.write(layer, slots, k, v)
            B = q.shape[0]
            if self.paged_attention is not None:
                return self.paged_attention(q.unsqueeze(1), self.cache.k[layer], self.cache.v[layer],
                                            cache_seqlens=ctx_i32, block_table=bt_i32, causal=True).squeeze(1)
            kk = self.cache.k[layer][block_tables[:, :max_blocks]].reshape(B, -1, self.kv_heads, self.head_dim)
            vv = self.cache.v[layer][block_tables[:, :max_blocks]].reshape(B, -1, self.kv_heads, self.head_dim)
            S = kk.shape[1]
            mask = torch.arange(S, device=q.device)[None, :] < ctx_lens[:, None]          # [B, S]
            o = F.scaled_dot_product_attention(q.unsqueeze(2), kk.transpose(1, 2), vv.transpose(1, 2),
                                               attn_mask=mask[:, None, None, :], enable_gqa=self.q_heads != self.kv_heads)
            return o.squeeze(2)
        attend.kv_target = (self.cache.k[layer], self.cache.v[layer], slots)
        return attend

    # --------------------------------------------------------------------- steps
    @torch.no_grad()
    def _prefill(self, batch: list[Sequence]) -> torch.Tensor:
        toks, pos, slots, lens = [], [], [], []
        for s in batch:
            n = len(s)
            ids = s.prompt + s.output
            toks += ids
            pos += list(range(n))
            slots += [s.blocks[i // self.block_size] * self.block_size + i % self.block_size for i in range(n)]
            lens.append(n)
        dev = self.device
        toks_t = torch.tensor(toks, dtype=torch.long, device=dev)
        pos_t = torch.tensor(pos, dtype=torch.long, device=dev)
        slots_t = torch.tensor(slots, dtype=torch.long, device=dev)
        h = self.model.model.forward_tokens(toks_t, pos_t, lambda i: self._prefill_attend(i, slots_t, lens))
        last = torch.tensor([sum(lens[:i + 1]) - 1 for i in range(len(lens))], dtype=torch.long, device=dev)
        return self.model.greedy_tokens(h[last])

    def _decode_inputs(self, batch: list[Sequence], max_blocks: int, rows: Optional[int] = None):
        """Host tensors of one decode step.  ``rows`` > len(batch) pads the batch: a padding row is token 0 at
        position 0 of a one-token sequence that lives in the scratch block."""
        B = len(batch)
        rows = B if rows is None else rows
        pad = rows - B
        toks = torch.tensor([(s.output or s.prompt)[-1] for s in batch] + [0] * pad, dtype=torch.long)
        pos = torch.tensor([len(s) - 1 for s in batch] + [0] * pad, dtype=torch.long)
        slots = torch.tensor([s.blocks[(len(s) - 1) // self.block_size] * self.block_size + (len(s) - 1) % self.block_size
                              for s in batch] + [self.scratch_block * self.block_size] * pad, dtype=torch.long)
        bt = torch.zeros(rows, max_blocks, dtype=torch.long)
        for i, s in enumerate(batch):
            bt[i, :len(s.blocks)] = torch.tensor(s.blocks, dtype=torch.long)
        bt[B:, 0] = self.scratch_block
        ctx = torch.tensor([len(s) for s in batch] + [1] * pad, dtype=torch.long)
        return toks, pos, slots, bt, ctx

    def _decode_forward(self, toks, pos, slots, bt, ctx, max_blocks):
        ctx_i32, bt_i32 = None, None
        if self.paged_attention is not None:  # once per step, not once per layer
            ctx_i32, bt_i32 = ctx.to(torch.int32), bt[:, :max_blocks].to(torch.int32).contiguous()
        h = self.model.model.forward_tokens(
            toks, pos, lambda i: self._decode_attend(i, slots, bt, ctx, max_blocks, ctx_i32, bt_i32))
        return self.model.greedy_tokens(h)

    @torch.no_grad()
    def _decode(self, batch: list[Sequence]) -> torch.Tensor:
        B = len(batch)
        max_blocks = max(len(s.blocks) for s in batch)
        if not self.use_cuda_graph:
            host = self._decode_inputs(batch, max_blocks)
            return self._decode_forward(*(t.to(self.device) for t in host), max_blocks)
        # one graph per (batch bucket, block-table width): batches are padded up to a power of two, so that
        # continuous batching replays a few dozen graphs.  The block table keeps its exact width: the
        # attention kernel sizes its KV splits by it (a table padded from 9 to 16 blocks cost 18 % of a step)
        rows = 1 << (B - 1).bit_length()
        host = self._decode_inputs(batch, max_blocks, rows)
        key = (rows, max_blocks)
        if key not in self._graphs:
            static = [t.to(self.device) for t in host]
            if self._warm_stream is None:
                self._warm_stream = torch.cuda.Stream()
            side = self._warm_stream
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._decode_forward(*static, max_blocks)      # warm up outside the capture
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self._decode_forward(*static, max_blocks)
            self._graphs[key] = (graph, static, out)
        graph, static, out = self._graphs[key]
        for dst, src in zip(static, host):
            dst.copy_(src, non_blocking=True)
        graph.replay()
        return out[:B]

    # ----------------------------------------------------------------------- API
    def add_request(self, prompt: Seq[int], max_new_tokens: int) -> int:
        if len(prompt) + 1 > self.max_tokens_per_sequence:
            raise ValueError(f"a prompt of {len(prompt)} tokens can never be admitted: the KV cache holds "
                             f"{self.max_tokens_per_sequence} tokens in all")
        sid = self._next_id
        self._next_id += 1
        self.scheduler.add(Sequence(sid, list(prompt), max_new_tokens))
        return sid

    def step(self) -> list[Sequence]:
        kind, batch = self.scheduler.step()
        if not batch:
            if self.scheduler.waiting and not self.scheduler.running:
                raise RuntimeError("the head of the waiting queue cannot be admitted although nothing is running "
                                   "(the KV cache is too small for it)")
            return []
        new = (self._prefill(batch) if kind == "prefill" else self._decode(batch)).tolist()
        self._check_device_status()
        for s, t in zip(batch, new):
            s.output.append(int(t))
            s.prefilled = True
        return self.scheduler.finish_step(kind, batch)

    def _check_device_status(self) -> None:
        """After the step's results reached the host: raise if a bounded device-side wait gave up during it
        (a peer that never arrived at an all-reduce, a pipeline barrier inside a GEMM).  Such a kernel
        returns without writing its output, so the step's tokens would be garbage."""
        from .. import _lib
        comm = getattr(self.model, "tp_comm", None)
        if comm is not None:
            comm.check()
        if self.device.type == "cuda":
            _lib.check_workspaces()

    def generate(self, prompts: Seq[Seq[int]], max_new_tokens) -> list[list[int]]:
        if isinstance(max_new_tokens, int):
            max_new_tokens = [max_new_tokens] * len(prompts)
        ids = [self.add_request(p, n) for p, n in zip(prompts, max_new_tokens)]
        results: dict[int, list[int]] = {}
        while self.scheduler.waiting or self.scheduler.running:
            for s in self.step():
                results[s.seq_id] = s.carried + s.output
        return [results[i] for i in ids]
