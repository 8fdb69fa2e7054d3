"""The C-ABI library loads without a GPU and exports every function the header declares."""
import ctypes
import os
import re

from nanoquantization_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = []
    inc = os.path.join(ROOT, "include")
    for f in sorted(os.listdir(inc)):
        if f.endswith(".h"):
            src = open(os.path.join(inc, f)).read()
            src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
            names += re.findall(r"\b(nqb200_[a-z0-9_]+)\s*\(", src)
    return sorted(set(names))


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.load()
    declared = _declared()
    assert len(declared) >= 8
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == declared


def test_host_only_entry_points():
    lib = _lib.load()
    assert lib.nqb200_version() >= 100
    for code in range(0, 12):
        assert lib.nqb200_status_string(code)
    # bad arguments are reported as statuses, never as a crash
    assert lib.nqb200_gemm(None, None, None, None, None, 0, None, 1, 7, 128, 128, 0, None, 0, None) == 1
    assert lib.nqb200_gemm(None, None, None, None, None, 0, None, 1, 8, 128, 128, 5, None, 0, None) == 2
    assert lib.nqb200_gemm(None, None, None, None, None, 0, None, 1, 8, 128, 128, 0, None, 0, None) == 4
    assert lib.nqb200_gemm(None, None, None, None, None, 0, None, 0, 8, 128, 128, 0, None, 0, None) == 0
    assert lib.nqb200_dequant(None, None, None, None, 100, 8, 64, 0, None) == 1
    assert lib.nqb200_unpack_int4(None, None, 0, 0, None) == 0
    buf = ctypes.create_string_buffer(64)
    mis = ctypes.addressof(buf) | 8
    assert lib.nqb200_unpack_int4(mis, mis, 1, 1, None) == 3
    assert lib.nqb200_gemm_workspace_bytes(1, 4096, 4096, 128, 0) > 0
    assert lib.nqb200_gemm_kernel_name(1, 4096, 4096, 128, 0) in (b"decode_stream",)
    assert lib.nqb200_gemm_kernel_name(16, 4096, 4096, 128, 0) == b"decode_stream"
    assert lib.nqb200_gemm_kernel_name(1, 24, 100, 100, 0) == b"generic"
    # K split across CTAs: a second kernel adds the partial sums
    assert lib.nqb200_gemm_launch_count(1, 4096, 4096, 128, 0) == 2
    assert lib.nqb200_gemm_launch_count(1, 512, 128, 128, 0) == 1
    assert lib.nqb200_gemm_launch_count(4096, 4096, 4096, 128, 0) == 1
    assert lib.nqb200_gemm_launch_count(0, 4096, 4096, 128, 0) == 0
    # which decode fusions a shape takes (host-side decision, no GPU needed)
    from nanoquantization_b200._lib import FUSE_ALLREDUCE, FUSE_RESIDUAL, FUSE_RMSNORM, FUSE_SILU_MUL
    sup = lib.nqb200_gemm_decode_fused_supported
    assert sup(1, 4096, 4096, 128, 0, FUSE_RMSNORM, 0, 0) == 1
    assert sup(16, 4096, 12288, 128, 0, FUSE_RESIDUAL, 0, 0) == 1
    assert sup(4, 24576, 4096, 128, 0, FUSE_RMSNORM | FUSE_SILU_MUL, 0, 0) == 1
    assert sup(4, 24576, 4096, 128, 0, FUSE_SILU_MUL | FUSE_RESIDUAL, 0, 0) == 0      # not together
    assert sup(17, 4096, 4096, 128, 0, FUSE_RMSNORM, 0, 0) == 0                        # decode sizes only
    assert sup(1, 512, 128, 128, 0, FUSE_RESIDUAL, 0, 0) == 0                          # one CTA covers the tile's whole K
    assert sup(4, 4096, 2048, 128, 0, FUSE_RESIDUAL | FUSE_ALLREDUCE, 2, 1 << 20) == 1
    assert sup(4, 4096, 2048, 128, 0, FUSE_RESIDUAL | FUSE_ALLREDUCE, 2, 1 << 10) == 0  # slot too small for world * M * N * 2 bytes
    assert lib.nqb200_gemm_gate_up_silu_supported(1, 6400, 5120, 128, 0) == 0           # I = 3200 is not tile-aligned
    assert lib.nqb200_gemm_allreduce_supported(4, 4096, 2048, 128, 0, 9, 1 << 20) == 0   # more ranks than the buffer layout holds


def test_prefill_dispatch_is_a_host_side_decision():
    """Which tcgen05 kernel a shape takes, how it is dealt and how much scratch it needs are decided on the
    host: the benchmark sweep's points and the edges of the rule, without a GPU."""
    lib = _lib.load()
    name, launches, ws = lib.nqb200_gemm_kernel_name, lib.nqb200_gemm_launch_count, lib.nqb200_gemm_workspace_bytes
    shapes = ((4096, 4096), (4096, 12288), (12288, 4096), (5120, 25600), (25600, 5120))
    for K, N in shapes:
        assert name(128, N, K, 128, 0) == b"prefill_tcgen05"           # up to 128 tokens: one CTA per tile
        for M in (1024, 4096):
            assert name(M, N, K, 128, 0) == b"prefill_tcgen05_pair", (M, K, N)
    # whole tiles where the last wave costs less than stream-K: one launch, scratch = counters only
    assert launches(4096, 25600, 5120, 128, 0) == 1 and ws(4096, 25600, 5120, 128, 0) == ws(1024, 4096, 4096, 128, 0)
    assert launches(4096, 5120, 25600, 128, 0) == 1
    # 80 tiles of a long K on 74 clusters: stream-K, a second kernel and two fp32 segments of 256 x 256 per cluster
    assert launches(1024, 5120, 25600, 128, 0) == 2
    assert ws(1024, 5120, 25600, 128, 0) - ws(4096, 25600, 5120, 128, 0) == 2 * 74 * 256 * 256 * 4
    # small layers stay with the single-CTA kernel however many tokens
    assert name(256, 4096, 4096, 128, 0) == b"prefill_tcgen05"
    assert name(192, 4096, 12288, 128, 1) == b"prefill_tcgen05"
    # what the two-CTA kernel does not take: other group sizes, N not a multiple of 32
    assert name(4096, 4096, 4096, 64, 0) != b"prefill_tcgen05_pair"
    assert name(4096, 4112, 4096, 128, 0) != b"prefill_tcgen05_pair"


def test_library_is_not_older_than_its_sources():
    from nanoquantization_b200.csrc import build
    assert not build._stale(), "libnqb200.so is older than csrc/: rebuild with python -m nanoquantization_b200.csrc.build"
