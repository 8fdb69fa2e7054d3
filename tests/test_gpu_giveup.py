"""The give-up path of bounded device-side waits, exercised without faulting anything.

A rank's all-reduce kernel waits for its peers' flags with a time limit; when the limit runs out
it records NQB200_ERR_WAIT_TIMEOUT in the rank's buffer and returns (it writes no output).  Here
one process plays rank 0 of a two-rank all-reduce on one GPU and nobody plays rank 1: the flag is
simply never set, the wait runs out after the 50 ms set for the test, and the CUDA context stays
usable.  Nothing traps, asserts or loops without limit.
"""
import ctypes

import pytest
import torch

from nanoquantization_b200 import _lib
from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TIMEOUT = 8  # NQB200_ERR_WAIT_TIMEOUT


def _alloc(lib, nbytes):
    p = ctypes.c_void_p()
    assert lib.nqb200_comm_alloc(ctypes.byref(p), nbytes) == 0
    return p.value


def _as_tensor(ptr, nbytes):
    class _P:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
    return torch.as_tensor(_P(), device=DEV)


def test_peer_allreduce_wait_runs_out_and_the_context_survives():
    torch.cuda.set_device(0)
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    a, b = _alloc(lib, 1 << 16), _alloc(lib, 1 << 16)
    try:
        assert lib.nqb200_comm_set_wait_limit(a, 50_000_000) == 0
        ptrs = (ctypes.c_void_p * 2)(a, b)
        out = torch.full((4, 64), -3.0, dtype=torch.float16, device=DEV)
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        assert lib.nqb200_peer_allreduce(ptrs, 0, 2, 0, out.data_ptr(), None, 0, 4, 64, _lib.F16, stream) == 0
        t1.record()
        assert lib.nqb200_comm_status(a, stream) == TIMEOUT
        assert 30.0 <= t0.elapsed_time(t1) <= 2000.0          # it waited for the limit, not for ever
        assert bool((out == -3.0).all())                        # and wrote nothing
        assert lib.nqb200_comm_status(a, stream) == 0           # the record is cleared once read
        assert b"timed out" in lib.nqb200_status_string(TIMEOUT)

        # the same through the GEMM whose finishing kernel does the all-reduce
        K, N, M = 2048, 512, 2
        if lib.nqb200_gemm_allreduce_supported(M, N, K, 128, _lib.F16, 2, 1 << 14):
            c = O.make_case(K, N, M, seed=3)
            d = {k: c[k].to(DEV) for k in ("x", "qweight", "qscales", "qzeros")}
            nbytes = lib.nqb200_gemm_workspace_bytes(M, N, K, 128, _lib.F16)
            ws = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
            y = torch.full((M, N), -3.0, dtype=torch.float16, device=DEV)
            assert lib.nqb200_gemm_allreduce(d["x"].data_ptr(), d["qweight"].data_ptr(), d["qscales"].data_ptr(),
                                             d["qzeros"].data_ptr(), None, 0, y.data_ptr(), M, N, K, 128, _lib.F16,
                                             ws.data_ptr(), ws.numel(), ptrs, 0, 2, 0, 1 << 14, stream) == 0
            assert lib.nqb200_comm_status(a, stream) == TIMEOUT
            assert bool((y == -3.0).all())
            assert lib.nqb200_workspace_status(ws.data_ptr(), ws.numel(), stream) == 0   # the GEMM's own waits were fine

        # the context is intact: a one-rank call on a fresh buffer returns the slot's contents
        c1 = _alloc(lib, 1 << 16)
        try:
            data = torch.randn(4, 64, generator=torch.Generator().manual_seed(1)).to(torch.float16).to(DEV)
            off = lib.nqb200_comm_data_offset()
            _as_tensor(c1 + off, 4 * 64 * 2).view(torch.float16).view(4, 64).copy_(data)
            one = (ctypes.c_void_p * 1)(c1)
            assert lib.nqb200_peer_allreduce(one, 0, 1, 0, out.data_ptr(), None, 0, 4, 64, _lib.F16, stream) == 0
            assert lib.nqb200_comm_status(c1, stream) == 0
            assert torch.equal(out, data)
        finally:
            lib.nqb200_comm_free(c1)
    finally:
        torch.cuda.synchronize()
        lib.nqb200_comm_free(a)
        lib.nqb200_comm_free(b)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_second_device_in_one_process():
    """The per-device kernel attributes (large dynamic shared memory) are set on every device a
    process uses, not only on the first."""
    import nanoquantization_b200 as nq
    for M in (4, 300):
        c = O.make_case(1024, 512, M, seed=M)
        ref = O.w4a16_ref(c["x"], c["qweight"], c["qscales"], c["qzeros"])
        for dev in ("cuda:0", "cuda:1"):
            y = nq.awq_gemm(c["x"].to(dev), c["qweight"].to(dev), c["qscales"].to(dev), c["qzeros"].to(dev), 8)
            assert O.rel_err(y, ref) <= 2e-3, (dev, M)
    lib = _lib.load()
    c = O.make_case(1024, 512, 4, seed=9)
    with torch.cuda.device(1):
        d = {k: c[k].to("cuda:1") for k in ("x", "qweight", "qscales", "qzeros")}
        out = torch.empty(4, 512, dtype=torch.float16, device="cuda:1")
        assert lib.nqb200_gemm_decode_noalloc(d["x"].data_ptr(), d["qweight"].data_ptr(), d["qscales"].data_ptr(),
                                              d["qzeros"].data_ptr(), None, 0, out.data_ptr(), 4, 512, 1024, 128, _lib.F16,
                                              torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
    assert O.rel_err(out, O.w4a16_ref(c["x"], c["qweight"], c["qscales"], c["qzeros"])) <= 2e-3


def test_two_shot_allreduce_one_rank_and_give_up():
    """The large-message kernel: with one rank it copies the slot (both shots degenerate); with a second
    rank that nobody plays its first barrier runs out, it records the time-out and writes nothing."""
    torch.cuda.set_device(0)
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    M, N = 300, 512
    nbytes = M * N * 2
    big = 1 << 20
    a, b = _alloc(lib, 3 * big), _alloc(lib, 3 * big)
    try:
        off = lib.nqb200_comm_data_offset()
        data = torch.randn(M, N, generator=torch.Generator().manual_seed(2)).to(torch.float16).to(DEV)
        _as_tensor(a + off, nbytes).view(torch.float16).view(M, N).copy_(data)
        out = torch.full((M, N), -3.0, dtype=torch.float16, device=DEV)
        one = (ctypes.c_void_p * 1)(a)
        for k in range(3):   # result slots alternate
            assert lib.nqb200_peer_allreduce_large(one, 0, 1, 0, (1 + k % 2) * big, out.data_ptr(), None, 0, M, N, _lib.F16, stream) == 0
            assert lib.nqb200_comm_status(a, stream) == 0
            assert torch.equal(out, data)
        assert lib.nqb200_comm_set_wait_limit(a, 50_000_000) == 0
        two = (ctypes.c_void_p * 2)(a, b)
        out.fill_(-3.0)
        assert lib.nqb200_peer_allreduce_large(two, 0, 2, 0, big, out.data_ptr(), None, 0, M, N, _lib.F16, stream) == 0
        assert lib.nqb200_comm_status(a, stream) == TIMEOUT
        assert bool((out == -3.0).all())
        assert lib.nqb200_comm_status(a, stream) == 0
        # bad arguments are statuses
        assert lib.nqb200_peer_allreduce_large(two, 0, 2, 8, big, out.data_ptr(), None, 0, M, N, _lib.F16, stream) != 0
        assert lib.nqb200_peer_allreduce_large(two, 2, 2, 0, big, out.data_ptr(), None, 0, M, N, _lib.F16, stream) != 0
    finally:
        torch.cuda.synchronize()
        lib.nqb200_comm_free(a)
        lib.nqb200_comm_free(b)
