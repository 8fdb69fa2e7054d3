"""The allocation-free decode entry point, called through the C ABI.

It serves hosts that cannot give the library a scratch buffer because they may
not allocate device memory at all (an engine that has committed all of HBM to
its own pools, a plugin interface without an allocator).  The scratch is a
fixed array inside the library; this test checks that the entry point gives the
same bits as nqb200_gemm with caller-provided scratch, twice in a row (the
second call meets the first call's leftovers in the shared array), and that it
rejects sizes beyond its stated limits.  Collected last on purpose.
"""
import pytest
import torch

from nanoquantization_b200 import _lib
from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_noalloc(c, M, N, K, g, out, bias=None):
    lib = _lib.load()
    code = _lib.dtype_code(c["qscales"].dtype)
    return lib.nqb200_gemm_decode_noalloc(
        c["x"].data_ptr(), c["qweight"].data_ptr(), c["qscales"].data_ptr(), c["qzeros"].data_ptr(),
        bias.data_ptr() if bias is not None else None, _lib.dtype_code(bias.dtype) if bias is not None else 0,
        out.data_ptr(), M, N, K, g, code, torch.cuda.current_stream().cuda_stream)


def _call_regular(c, M, N, K, g, out, bias=None):
    lib = _lib.load()
    code = _lib.dtype_code(c["qscales"].dtype)
    nbytes = lib.nqb200_gemm_workspace_bytes(M, N, K, g, code)
    ws = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device=DEV)
    st = lib.nqb200_gemm(
        c["x"].data_ptr(), c["qweight"].data_ptr(), c["qscales"].data_ptr(), c["qzeros"].data_ptr(),
        bias.data_ptr() if bias is not None else None, _lib.dtype_code(bias.dtype) if bias is not None else 0,
        out.data_ptr(), M, N, K, g, code, ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return st


@pytest.mark.parametrize("K,N,M,dtype,with_bias", [
    (4096, 4096, 1, torch.float16, False),
    (1024, 3072, 8, torch.float16, True),
    (5120, 3200, 4, torch.bfloat16, False),
    (2048, 1024, 12, torch.float16, False),
    (5120, 3200, 16, torch.float16, True),
])
def test_noalloc_matches_regular_entry_point_twice(K, N, M, dtype, with_bias):
    torch.cuda.set_device(0)
    g = 128
    host = O.make_case(K, N, M, group_size=g, dtype=dtype, seed=77, bias=with_bias)
    c = {k: host[k].to(DEV) for k in ("x", "qweight", "qscales", "qzeros")}
    bias = host["bias"].to(DEV) if with_bias else None
    ref = torch.empty(M, N, dtype=dtype, device=DEV)
    assert _call_regular(c, M, N, K, g, ref, bias) == 0
    free_before = torch.cuda.mem_get_info()[0]
    for attempt in range(2):
        out = torch.full((M, N), float("nan"), dtype=dtype, device=DEV)
        assert _call_noalloc(c, M, N, K, g, out, bias) == 0
        torch.cuda.synchronize()
        # same kernel, same fixed summation order: identical bits, as the header promises
        assert torch.equal(out, ref), f"call {attempt}"
    assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20)  # nothing was taken from the device
    exact = O.w4a16_ref(host["x"], host["qweight"], host["qscales"], host["qzeros"], host["bias"])
    assert O.rel_err(out, exact) <= 1e-2


def test_noalloc_rejects_sizes_beyond_its_limits():
    lib = _lib.load()
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    p = buf.data_ptr()
    s = torch.cuda.current_stream().cuda_stream
    too_large = 9
    assert lib.nqb200_gemm_decode_noalloc(p, p, p, p, None, 0, p, 17, 4096, 4096, 128, 0, s) == too_large  # tokens
    assert lib.nqb200_gemm_decode_noalloc(p, p, p, p, None, 0, p, 4, 4096, 4096, 64, 0, s) == too_large    # group size
    assert lib.nqb200_gemm_decode_noalloc(p, p, p, p, None, 0, p, 4, 4104, 4096, 128, 0, s) == too_large   # N % 32
    assert lib.nqb200_gemm_decode_noalloc(p, p, p, p, None, 0, p, 4, 4100, 4096, 128, 0, s) == 1           # N % 8
    assert b"exceeds" in lib.nqb200_status_string(too_large)
    assert lib.nqb200_gemm_decode_noalloc(p, p, p, p, None, 0, p, 0, 4096, 4096, 128, 0, s) == 0           # empty
