"""Parity of the CUDA path (through the C ABI) with the CPU oracle and with the
vectors produced by the reference.  Integer work is bit-exact; the GEMM is
checked with max|y - y_ref| / max|y_ref| <= 1e-2 (the stated fp16
accumulation-order tolerance) against fp32 dequantise-then-matmul."""
import numpy as np
import pytest
import torch

import nanoquantization_b200 as nq
from nanoquantization_b200 import _lib
from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-2       # the tolerance the path is specified to
TIGHT = 2e-3     # what a correct kernel achieves here (one 16-bit rounding of the output)
DEV = "cuda:0"


def _tags(npz, suffix):
    return sorted({k[: -len(suffix)] for k in npz.files if k.endswith(suffix)})


def _bits(t):
    return t.detach().cpu().view(torch.int16).numpy().view(np.uint16)


def test_library_is_loaded_and_device_supported():
    lib = _lib.load()
    assert lib.nqb200_device_supported(0) == 1


# ------------------------------------------------------------------ unpack
def test_unpack_bit_exact_golden(golden):
    z = golden("pack_vectors.npz")
    for t in _tags(z, ".iw"):
        for words, vals in ((z[t + ".qweight"], z[t + ".iw"]), (z[t + ".qzeros"], z[t + ".iz"])):
            got = nq.unpack_int4(torch.from_numpy(words).to(DEV)).cpu().numpy()
            assert np.array_equal(got, vals), t


@pytest.mark.parametrize("rows,cols", [(1, 8), (3, 40), (4096, 4096), (200, 25600)])
def test_unpack_bit_exact_random(rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    words = rng.integers(0, 2 ** 32, size=(rows, cols // 8), dtype=np.uint64).astype(np.uint32).view(np.int32)
    got = nq.unpack_int4(torch.from_numpy(words).to(DEV)).cpu().numpy()
    assert np.array_equal(got, O.unpack_int4(words))


def test_unpack_empty():
    assert nq.unpack_int4(torch.zeros(0, 4, dtype=torch.int32, device=DEV)).shape == (0, 32)


# ----------------------------------------------------------------- dequant
def test_dequant_bit_exact_vs_reference_kernel_vectors(golden):
    for name in ("from_linear_vectors.npz", "kernel_vectors.npz"):
        z = golden(name)
        for t in _tags(z, ".dequant"):
            W = nq.awq_dequantize(torch.from_numpy(z[t + ".qweight"]).to(DEV), torch.from_numpy(z[t + ".qscales"]).to(DEV),
                                  torch.from_numpy(z[t + ".qzeros"]).to(DEV))
            assert W.dtype == torch.float16 and tuple(W.shape) == z[t + ".dequant"].shape
            assert np.array_equal(_bits(W), z[t + ".dequant"].view(np.uint16)), t


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("K,N,g", [(1024, 3072, 128), (128, 8, 128), (256, 136, 128), (3200, 3200, 128),
                                   (96, 64, 32), (192, 264, 64), (200, 24, 200)])
def test_dequant_bit_exact_vs_oracle(dtype, K, N, g):
    c = O.make_case(K, N, 1, group_size=g, dtype=dtype, seed=K + N)
    W = nq.awq_dequantize(c["qweight"].to(DEV), c["qscales"].to(DEV), c["qzeros"].to(DEV))
    ref = O.dequantize(c["qweight"], c["qscales"], c["qzeros"])
    assert W.dtype == dtype
    assert np.array_equal(_bits(W), _bits(ref))


# -------------------------------------------------------------------- gemm
def _run_case(K, N, M, g=128, dtype=torch.float16, seed=0, bias=False, tol=TIGHT):
    c = O.make_case(K, N, M, group_size=g, dtype=dtype, seed=seed, bias=bias)
    m = nq.WQLinear_GEMM(4, g, K, N, DEV, bias, dtype)
    m.qweight.copy_(c["qweight"]); m.qscales.copy_(c["qscales"]); m.qzeros.copy_(c["qzeros"])
    if bias:
        m.bias.copy_(c["bias"])
    # The output sits between sentinel rows that no kernel may touch (a write past either end of
    # the result would show there; compute-sanitizer is not available where these tests run).
    SENT = -7.25
    buf = torch.full((M + 2, N), SENT, dtype=dtype, device=DEV)
    y = m(c["x"].to(DEV), out=buf[1:M + 1])
    torch.cuda.synchronize()
    assert y.dtype == dtype and tuple(y.shape) == (M, N) and y.data_ptr() == buf[1].data_ptr()
    assert bool((buf[0] == SENT).all()) and bool((buf[M + 1] == SENT).all()), "a kernel wrote outside its output"
    ref = O.w4a16_ref(c["x"], c["qweight"], c["qscales"], c["qzeros"], c["bias"])
    err = O.rel_err(y, ref)
    bound = tol if dtype == torch.float16 else max(tol, 8e-3)  # bf16 output rounding is 2^-8 relative
    assert err <= bound <= TOL, f"rel err {err:.3e} (K={K} N={N} M={M} g={g} {dtype})"
    return y, ref


def test_gemm_vs_reference_kernel_vectors(golden):
    for name in ("from_linear_vectors.npz", "kernel_vectors.npz"):
        z = golden(name)
        for t in _tags(z, ".gemm"):
            x = torch.from_numpy(z[t + ".x"])
            qs = torch.from_numpy(z[t + ".qscales"])
            y = nq.awq_gemm(x.to(DEV), torch.from_numpy(z[t + ".qweight"]).to(DEV), qs.to(DEV),
                            torch.from_numpy(z[t + ".qzeros"]).to(DEV), 8)
            ref32 = O.w4a16_ref(x, z[t + ".qweight"], qs, z[t + ".qzeros"])
            assert O.rel_err(y, ref32) <= TIGHT, t
            # and against what the reference's own kernel produced for these inputs
            assert O.rel_err(y, torch.from_numpy(z[t + ".gemm"])) <= TOL, t
            assert y.dtype == torch.float16


def test_gemm_config1_reference_runnable_case():
    # Qwen3-0.6B gate_proj: K=1024, N=3072, M=16, fp16
    _run_case(1024, 3072, 16)


@pytest.mark.parametrize("M", [1, 2, 4, 7, 8, 9, 16, 17, 33, 128])
def test_gemm_token_counts(M):
    _run_case(512, 1024, M, seed=M)


@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 12288), (12288, 4096), (5120, 25600), (25600, 5120)])
@pytest.mark.parametrize("M", [1, 16])
def test_gemm_sweep_shapes_decode(K, N, M):
    _run_case(K, N, M, seed=K // 128 + M)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("K,N,g,M", [
    (128, 128, 128, 1),       # one group, one k/v head per rank at TP=8
    (512, 128, 128, 3),
    (3200, 5120, 128, 5),     # 25 groups: Qwen3-32B down_proj shard at TP=8
    (5120, 3200, 128, 16),    # N = 3200, not a multiple of 256
    (256, 144, 128, 4),       # N % 32 != 0 -> 64-bit loads
    (256, 136, 128, 2),       # N % 16 != 0 -> fallback kernel
    (96, 64, 32, 8),
    (192, 256, 64, 12),
    (1024, 2048, 32, 8),      # the reference unit test's shape
    (200, 24, 200, 3),        # group == K, not a multiple of 16 -> fallback kernel
    (4096, 64, 4096, 2),      # group == K
])
def test_gemm_edge_shapes(dtype, K, N, g, M):
    _run_case(K, N, M, g=g, dtype=dtype, seed=K + N + M)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M", [1, 16, 40])
def test_gemm_bias(dtype, M):
    _run_case(1024, 512, M, dtype=dtype, bias=True, seed=9)


def test_gemm_leading_dims_and_empty():
    c = O.make_case(256, 128, 6, seed=4)
    m = nq.WQLinear_GEMM(4, 128, 256, 128, DEV, False, torch.float16)
    m.qweight.copy_(c["qweight"]); m.qscales.copy_(c["qscales"]); m.qzeros.copy_(c["qzeros"])
    y = m(c["x"].to(DEV).view(2, 3, 256))
    assert tuple(y.shape) == (2, 3, 128)
    assert O.rel_err(y.view(6, 128), O.w4a16_ref(c["x"], c["qweight"], c["qscales"], c["qzeros"])) <= TIGHT
    assert tuple(m(torch.zeros(0, 256, dtype=torch.float16, device=DEV)).shape) == (0, 128)


def test_gemm_is_deterministic_and_restores_workspace():
    c = O.make_case(4096, 4096, 4, seed=21)
    args = [c["x"].to(DEV), c["qweight"].to(DEV), c["qscales"].to(DEV), c["qzeros"].to(DEV), 8]
    y1 = nq.awq_gemm(*args)
    y2 = nq.awq_gemm(*args)
    y3 = nq.awq_gemm(*args)
    assert torch.equal(y1, y2) and torch.equal(y1, y3)
    torch.cuda.synchronize()
    nbytes = _lib.load().nqb200_gemm_workspace_bytes(4, 4096, 4096, 128, 0)
    assert nbytes > (1 << 16)
    for ws in _lib._workspaces.values():
        assert int(ws[: 1 << 16].view(torch.int32).abs().sum()) == 0  # arrival counters (first 64 KiB) back at zero


def test_no_device_wait_gave_up():
    _lib.check_workspaces()


def test_gemm_x_is_cast_to_output_dtype():
    c = O.make_case(256, 128, 3, seed=2)
    y = nq.awq_gemm(c["x"].float().to(DEV), c["qweight"].to(DEV), c["qscales"].to(DEV), c["qzeros"].to(DEV), 8)
    assert y.dtype == torch.float16
    assert O.rel_err(y, O.w4a16_ref(c["x"], c["qweight"], c["qscales"], c["qzeros"])) <= TIGHT


def test_gemm_outlier_activations_and_extreme_nibbles():
    # large-mean activations stress the zero-point / sum(x) correction; all-15 weights with all-0
    # zero-points and the reverse stress the nibble paths
    K, N, M = 1024, 256, 8
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(M, K, generator=g) * 0.5 + 6.0).to(torch.float16)
    x[:, 7] = 300.0
    for wv, zv in ((15, 0), (0, 15), (8, 8)):
        qw = torch.from_numpy(O.pack_int4(np.full((K, N), wv)))
        qz = torch.from_numpy(O.pack_int4(np.full((K // 128, N), zv)))
        s = (torch.rand(K // 128, N, generator=g) * 9e-3 + 1e-3).to(torch.float16)
        y = nq.awq_gemm(x.to(DEV), qw.to(DEV), s.to(DEV), qz.to(DEV), 8)
        ref = O.w4a16_ref(x, qw, s, qz)
        if wv == zv:
            # exact answer is 0; what remains is fp32 cancellation against s*z*sum|x|
            assert float(y.float().abs().max()) <= 1e-4 * 1e-2 * 8 * float(x.float().abs().sum(1).max())
        else:
            assert O.rel_err(y, ref) <= TIGHT, (wv, zv)


@pytest.mark.parametrize("M", [256, 1024])
def test_gemm_prefill_sizes_sampled_rows(M):
    # full-size prefill shape; the oracle is evaluated on a sample of rows to stay fast
    K, N = 4096, 4096
    c = O.make_case(K, N, M, seed=M)
    y = nq.awq_gemm(c["x"].to(DEV), c["qweight"].to(DEV), c["qscales"].to(DEV), c["qzeros"].to(DEV), 8)
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:48]
    ref = O.w4a16_ref(c["x"][rows], c["qweight"], c["qscales"], c["qzeros"])
    assert O.rel_err(y[rows.to(DEV)], ref) <= TIGHT


# The whole benchmark sweep: every (K, N) shape at every token count the decode-shape test above does
# not already take, against the oracle.  One seeded case per shape and dtype is built once (the oracle's
# dense weight too) and reused for all token counts; above 40 tokens the oracle answers for a seeded
# sample of 40 rows, which still covers every output column, every K split and every token tile position
# modulo 128 that the sample hits.
SWEEP_SHAPES = [(4096, 4096), (4096, 12288), (12288, 4096), (5120, 25600), (25600, 5120)]
_sweep_cache = {}


def _sweep_case(K, N, dtype):
    key = (K, N, dtype)
    if key not in _sweep_cache:
        _sweep_cache.clear()  # one shape at a time: the dense oracle weight is up to 262 MB
        # uniform 32-bit words are uniform nibbles: the benchmark's int4 weights and zero-points
        # uniform in [0, 15], without the oracle packer's pass over 131 M elements
        g = torch.Generator().manual_seed(K // 128 + N // 128)
        c = {"qweight": torch.randint(-2 ** 31, 2 ** 31, (K, N // 8), generator=g, dtype=torch.int64).to(torch.int32),
             "qzeros": torch.randint(-2 ** 31, 2 ** 31, (K // 128, N // 8), generator=g, dtype=torch.int64).to(torch.int32),
             "qscales": (torch.rand(K // 128, N, generator=g) * 9e-3 + 1e-3).to(dtype),
             "x": torch.randn(4096, K, generator=g).to(dtype)}
        dev = {k: c[k].to(DEV) for k in ("x", "qweight", "qscales", "qzeros")}
        _sweep_cache[key] = (c, dev, O.dequantize(c["qweight"], c["qscales"], c["qzeros"]))
    return _sweep_cache[key]


@pytest.mark.parametrize("M", [4, 128, 1024, 4096])
@pytest.mark.parametrize("K,N,dtype", [(K, N, torch.float16) for K, N in SWEEP_SHAPES] +
                         [(5120, 25600, torch.bfloat16), (25600, 5120, torch.bfloat16)])
def test_gemm_sweep_every_point_vs_oracle(K, N, dtype, M):
    c, dev, W = _sweep_case(K, N, dtype)
    y = nq.awq_gemm(dev["x"][:M].contiguous(), dev["qweight"], dev["qscales"], dev["qzeros"], 8)
    torch.cuda.synchronize()
    assert y.dtype == dtype and tuple(y.shape) == (M, N)
    rows = torch.arange(M) if M <= 40 else torch.randperm(M, generator=torch.Generator().manual_seed(M + K))[:40]
    ref = c["x"][rows].float() @ W.float()
    err = O.rel_err(y[rows.to(DEV)], ref)
    bound = TIGHT if dtype == torch.float16 else 8e-3
    assert err <= bound <= TOL, f"rel err {err:.3e} (K={K} N={N} M={M} {dtype})"
    assert bool(torch.isfinite(y.float()).all())
    _lib.check_workspaces()  # no bounded wait gave up


# The two-CTA tcgen05 kernel at ragged sizes: token counts that end inside a 256-token tile, a column count whose
# last 256-column tile holds 32 columns (the second CTA of the pair then has none), whole-tile dealing and stream-K
# with its second kernel, with and without bias.  The case list pins which kernel and how many launches the
# dispatch picks, so that a change of the rule cannot silently take these paths out of the test.
@pytest.mark.parametrize("M,K,N,dtype,bias,launches", [
    (777, 4096, 12288, torch.float16, True, 1),
    (192, 4096, 12288, torch.float16, True, 1),      # a single token tile of 192: MMA N = 192, 96 tokens per CTA
    (130, 4096, 12288, torch.bfloat16, False, 1),    # 130 tokens in a tile of 160
    (1000, 1024, 25632, torch.float16, False, 1),
    (1000, 1024, 25632, torch.bfloat16, True, 1),
    (1100, 25600, 5152, torch.float16, True, 2),
    (2048, 25600, 5120, torch.bfloat16, True, 2),
    (700, 5120, 25600, torch.bfloat16, False, 1),
])
def test_gemm_pair_kernel_ragged(M, K, N, dtype, bias, launches):
    lib = _lib.load()
    code = 0 if dtype == torch.float16 else 1
    assert lib.nqb200_gemm_kernel_name(M, N, K, 128, code) == b"prefill_tcgen05_pair"
    assert lib.nqb200_gemm_launch_count(M, N, K, 128, code) == launches
    g = torch.Generator().manual_seed(M + N)
    qw = torch.randint(-2 ** 31, 2 ** 31, (K, N // 8), generator=g, dtype=torch.int64).to(torch.int32)
    qz = torch.randint(-2 ** 31, 2 ** 31, (K // 128, N // 8), generator=g, dtype=torch.int64).to(torch.int32)
    sc = (torch.rand(K // 128, N, generator=g) * 9e-3 + 1e-3).to(dtype)
    x = torch.randn(M, K, generator=g).to(dtype)
    b = torch.randn(N, generator=g).to(dtype) if bias else None
    # sentinel rows around the output: a store that runs past M tokens would change them
    m = nq.WQLinear_GEMM(4, 128, K, N, DEV, bias, dtype)
    m.qweight.copy_(qw); m.qscales.copy_(sc); m.qzeros.copy_(qz)
    if bias:
        m.bias.copy_(b)
    buf = torch.full((M + 2, N), -7.25, dtype=dtype, device=DEV)
    y = m(x.to(DEV), out=buf[1:M + 1])
    torch.cuda.synchronize()
    assert bool((buf[0] == -7.25).all()) and bool((buf[M + 1] == -7.25).all())
    rows = torch.cat([torch.tensor([0, min(255, M - 1), min(256, M - 1), M - 1]), torch.randperm(M, generator=g)[:28]])
    W = O.dequantize(qw, sc, qz)
    ref = x[rows].float() @ W.float()
    if b is not None:
        ref = ref + b.float()
    err = O.rel_err(y[rows.to(DEV)], ref)
    assert err <= (TIGHT if dtype == torch.float16 else 8e-3), f"rel err {err:.3e}"
    assert bool(torch.isfinite(y.float()).all())
    _lib.check_workspaces()


def test_gemm_linearity_property_full_size():
    # size-independent property at a full benchmark shape: y(2x) == 2*y(x) exactly in fp16
    c = O.make_case(5120, 25600, 4, seed=3)
    qw, s, qz = c["qweight"].to(DEV), c["qscales"].to(DEV), c["qzeros"].to(DEV)
    x = c["x"].to(DEV)
    y1 = nq.awq_gemm(x, qw, s, qz, 8)
    y2 = nq.awq_gemm(x * 2, qw, s, qz, 8)
    # exact wherever y1 is a normal fp16 number; a subnormal y1 has already lost bits that 2*y keeps
    normal = y1.abs() >= 2.0 ** -14
    assert torch.equal(y2[normal], (y1 * 2)[normal])
    assert float((y2.float() - 2 * y1.float()).abs().max()) <= 2.0 ** -23
    assert float(normal.float().mean()) > 0.99


# ------------------------------------------------------- quantise + pack on the GPU
@pytest.mark.parametrize("wdtype,odtype", [(torch.float16, torch.float16), (torch.bfloat16, torch.bfloat16),
                                           (torch.float32, torch.float16)])
@pytest.mark.parametrize("K,N,g", [(1024, 2048, 32), (512, 136, 128), (256, 64, 64)])
def test_quantize_pack_bit_exact_vs_reference_pipeline(wdtype, odtype, K, N, g):
    # the reference's per-layer recipe on the CPU: pseudo_quantize, then from_linear on the
    # fake-quantised weight with transposed scales / zero-points
    w = torch.randn(N, K, generator=torch.Generator().manual_seed(K + N)).to(wdtype)
    w[3, :g] = 0.25                                            # a constant group: range below the 1e-5 clamp
    wq, s, z = O.pseudo_quantize(w.clone(), g, 4)
    qw_ref, qs_ref, qz_ref = O.from_linear_ref(wq, s.t().contiguous(), z.t().contiguous(), g, odtype)
    lin = torch.nn.Linear(K, N, bias=False, device=DEV, dtype=wdtype)
    lin.weight.data.copy_(w)
    m = nq.WQLinear_GEMM.from_float(lin, 4, g, odtype)
    torch.cuda.synchronize()
    assert np.array_equal(m.qzeros.cpu().numpy(), qz_ref.numpy())
    assert np.array_equal(_bits(m.qscales), _bits(qs_ref))
    assert np.array_equal(m.qweight.cpu().numpy(), qw_ref.numpy())
