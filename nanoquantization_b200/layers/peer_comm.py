"""One-shot all-reduce over NVLink peer memory for tensor-parallel decode.

``PeerAllReduce`` owns a cudaMalloc'd buffer per rank that every peer maps through CUDA IPC.  A
row-parallel linear writes its partial ``[M, N]`` result straight into a slot of that buffer
(``WQLinear_GEMM.forward(x, out=slot)``) and ``reduce`` launches one kernel per rank that waits
for all ranks, adds the peers' slots in rank order and writes the sum to an ordinary tensor.
For decode-sized inputs ``linear_all_reduce`` does both in the GEMM itself: the kernel that adds the
GEMM's split-K partial sums stores the rank's result into every peer's slot and reduces over the
ranks (``nqb200_gemm_allreduce``).  Messages larger than a slot take the two-shot kernel (``large_bytes``: the
rank's partial result in one large slot, reduce-scatter and all-gather over peer memory in one launch) or, beyond
that, NCCL.  The reference has no counterpart.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _lib


class _DevicePtr:
    """Lets torch wrap a raw device pointer (``__cuda_array_interface__``) without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _local(linear, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """The rank's own partial product: the plain module forward, also for a row-parallel class
    (whose ``forward`` would reduce again)."""
    from .gemm import WQLinear_GEMM
    return WQLinear_GEMM.forward(linear, x, out)


class PeerAllReduce:
    def __init__(self, group=None, slot_bytes: int = 1 << 20, num_slots: int = 8, fused: bool = True,
                 max_message_bytes: int = 1 << 20, wait_limit_s: float = 1.0, large_bytes: int = 0):
        assert num_slots >= 3 and large_bytes % 256 == 0
        self.fused = fused  # reduce inside the GEMM's finishing kernel where the library supports it
        # larger messages go through NCCL (the one-shot kernel moves world x the message over NVLink per rank)
        self.max_message_bytes = max_message_bytes
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.slot_bytes, self.num_slots, self._next = slot_bytes, num_slots, 0
        # behind the small slots: one slot for a large partial result and two, used alternately, for the reduced slices
        self.large_bytes, self._large_base, self._large_next = large_bytes, slot_bytes * num_slots, 0
        lib = _lib.load()
        self.device = torch.device("cuda", torch.cuda.current_device())
        own = ctypes.c_void_p()
        _lib.check(lib.nqb200_comm_alloc(ctypes.byref(own), slot_bytes * num_slots + 3 * large_bytes))
        self._own = own.value
        handle = ctypes.create_string_buffer(64)
        _lib.check(lib.nqb200_comm_export(self._own, handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self._ptrs = (ctypes.c_void_p * self.world)()
        self._imported = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self._ptrs[r] = self._own
            else:
                p = ctypes.c_void_p()
                _lib.check(lib.nqb200_comm_import(ctypes.create_string_buffer(h, 64), ctypes.byref(p)))
                self._ptrs[r] = p.value
                self._imported.append(p.value)
        _lib.check(lib.nqb200_comm_set_wait_limit(self._own, int(wait_limit_s * 1e9)))
        self._data_off = lib.nqb200_comm_data_offset()
        self._bytes = torch.as_tensor(_DevicePtr(self._own + self._data_off, slot_bytes * num_slots + 3 * large_bytes), device=self.device)
        dist.barrier(group=group)

    def fits(self, M: int, N: int) -> bool:
        return M * N * 2 <= min(self.slot_bytes, self.max_message_bytes) and (M * N) % 8 == 0

    def next_slot(self, M: int, N: int, dtype: torch.dtype) -> tuple[torch.Tensor, int]:
        """A ``[M, N]`` view of the next slot of this rank's buffer and its byte offset."""
        off = self._next * self.slot_bytes
        self._next = (self._next + 1) % self.num_slots
        return self._bytes[off:off + M * N * 2].view(dtype).view(M, N), off

    def reduce(self, slot_offset: int, M: int, N: int, dtype: torch.dtype, bias: torch.Tensor | None = None) -> torch.Tensor:
        out = torch.empty(M, N, dtype=dtype, device=self.device)
        _lib.check(_lib.load().nqb200_peer_allreduce(
            self._ptrs, self.rank, self.world, slot_offset, out.data_ptr(),
            bias.data_ptr() if bias is not None else None, _lib.dtype_code(bias.dtype) if bias is not None else 0,
            M, N, _lib.dtype_code(dtype), _lib.stream_ptr()))
        return out

    def fused_residual_supported(self, linear, M: int) -> bool:
        return self.fused and self.world > 1 and linear.fused_supported(M, residual=True, world=self.world, slot_bytes=self.slot_bytes)

    def linear_all_reduce_residual(self, linear, x: torch.Tensor, residual: torch.Tensor):
        """``(all_reduce(linear(x)) + residual, per-tile sums of squares of that)`` in the linear's own two launches
        (where ``fused_residual_supported``)."""
        off = self._next * self.slot_bytes
        self._next = (self._next + 1) % self.num_slots
        return linear.forward_fused(x, residual=residual, peer=(self._ptrs, self.rank, self.world, off, self.slot_bytes))

    def linear_all_reduce(self, linear, x: torch.Tensor) -> torch.Tensor:
        """``all_reduce(linear(x))`` with the partial result written straight into peer-visible memory."""
        M, N = x.shape[0], linear.out_features
        if self.world == 1:
            return _local(linear, x)
        if not self.fits(M, N):
            if self.fits_large(M, N):
                return self.linear_all_reduce_large(linear, x)
            y = _local(linear, x)
            dist.all_reduce(y, group=self.group)
            return y
        dtype = linear.qscales.dtype
        if self.fused and _lib.load().nqb200_gemm_allreduce_supported(M, N, x.shape[1], linear.group_size, _lib.dtype_code(dtype),
                                                                      self.world, self.slot_bytes):
            # the kernel that finishes the GEMM also reduces over the ranks
            from .gemm import _w4a16
            off = self._next * self.slot_bytes
            self._next = (self._next + 1) % self.num_slots
            return _w4a16(x, linear.qweight, linear.qscales, linear.qzeros, linear.bias, None,
                          peer=(self._ptrs, self.rank, self.world, off, self.slot_bytes))
        slot, off = self.next_slot(M, N, linear.qscales.dtype)
        _local(linear, x, slot)
        return self.reduce(off, M, N, linear.qscales.dtype)

    def fits_large(self, M: int, N: int) -> bool:
        return 0 < M * N * 2 <= self.large_bytes and (M * N) % 8 == 0

    def linear_all_reduce_large(self, linear, x: torch.Tensor) -> torch.Tensor:
        """``all_reduce(linear(x))`` for a prefill-sized result: the GEMM writes into the large slot, one
        two-shot kernel per rank reduces over peer memory (``nqb200_peer_allreduce_large``)."""
        M, N = x.shape[0], linear.out_features
        dtype = linear.qscales.dtype
        base = self._large_base
        _local(linear, x, self._bytes[base:base + M * N * 2].view(dtype).view(M, N))
        res = base + (1 + self._large_next) * self.large_bytes
        self._large_next ^= 1
        out = torch.empty(M, N, dtype=dtype, device=self.device)
        _lib.check(_lib.load().nqb200_peer_allreduce_large(self._ptrs, self.rank, self.world, base, res, out.data_ptr(), None, 0,
                                                           M, N, _lib.dtype_code(dtype), _lib.stream_ptr()))
        return out

    def status(self) -> int:
        """0, or the code a bounded wait recorded when it gave up (waits for the current stream; the
        record is cleared).  After a give-up the kernel has not written its output."""
        return int(_lib.load().nqb200_comm_status(self._own, _lib.stream_ptr()))

    def check(self) -> None:
        """Raise if a wait for a peer ran out since the last check."""
        _lib.check(self.status())

    def close(self) -> None:
        lib = _lib.load()
        torch.cuda.synchronize()
        for p in self._imported:
            lib.nqb200_comm_unimport(p)
        self._imported = []
        if self._own:
            lib.nqb200_comm_free(self._own)
            self._own = None
