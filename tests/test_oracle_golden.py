"""The CPU oracle against vectors produced by the reference itself
(tests/golden/make_golden.py): packer output, Triton-interpreter dequantize and
split-K GEMM.  No GPU, no reference checkout needed."""
import numpy as np
import torch

from oracle import awq_oracle as O


def _tags(npz, suffix):
    return sorted({k[: -len(suffix)] for k in npz.files if k.endswith(suffix)})


def test_known_word():
    # worked example: elements [12,15,5,0,3,11,3,7] pack to 0x7b0f335c
    w = O.pack_int4(np.array([[12, 15, 5, 0, 3, 11, 3, 7]]))
    assert (int(w[0, 0]) & 0xFFFFFFFF) == 0x7B0F335C
    assert O.unpack_int4(w).tolist() == [[12, 15, 5, 0, 3, 11, 3, 7]]


def test_pack_unpack_bit_exact_vs_reference_packer(golden):
    z = golden("pack_vectors.npz")
    tags = _tags(z, ".iw")
    assert len(tags) >= 8
    for t in tags:
        iw, iz = z[t + ".iw"], z[t + ".iz"]
        qw, qz = z[t + ".qweight"], z[t + ".qzeros"]
        assert qw.dtype == np.int32
        assert np.array_equal(O.pack_int4(iw), qw), t
        assert np.array_equal(O.pack_int4(iz), qz), t
        assert np.array_equal(O.unpack_int4(qw), iw), t
        assert np.array_equal(O.unpack_int4(qz), iz), t
    assert (z["all15.qweight"] < 0).all()  # the sign bit is in use


def test_from_linear_vs_reference(golden):
    z = golden("from_linear_vectors.npz")
    for t in _tags(z, ".weight_fq"):
        g = int(t.split("_g")[1])
        w = torch.from_numpy(z[t + ".weight_fq"])
        s = torch.from_numpy(z[t + ".scales"])
        zz = torch.from_numpy(z[t + ".zeros"])
        qw, qs, qz = O.from_linear_ref(w, s, zz, g, torch.float16)
        assert np.array_equal(qw.numpy(), z[t + ".qweight"]), t
        assert np.array_equal(qz.numpy(), z[t + ".qzeros"]), t
        assert np.array_equal(qs.numpy().view(np.uint16), z[t + ".qscales"].view(np.uint16)), t
        # the reference unit test's own bound: dequant ~ fake-quantised weight, atol 1e-2
        W = O.dequantize(qw, qs, qz)
        assert torch.allclose(W, w.t().contiguous(), atol=1e-2)


def test_dequantize_bit_exact_vs_reference_kernel(golden):
    for name in ("from_linear_vectors.npz", "kernel_vectors.npz"):
        z = golden(name)
        for t in _tags(z, ".dequant"):
            W = O.dequantize(z[t + ".qweight"], torch.from_numpy(z[t + ".qscales"]), z[t + ".qzeros"])
            assert W.dtype == torch.float16
            assert np.array_equal(W.numpy().view(np.uint16), z[t + ".dequant"].view(np.uint16)), t


def test_gemm_vs_reference_kernel(golden):
    for name in ("from_linear_vectors.npz", "kernel_vectors.npz"):
        z = golden(name)
        for t in _tags(z, ".gemm"):
            x = torch.from_numpy(z[t + ".x"])
            s = torch.from_numpy(z[t + ".qscales"])
            y_ref_kernel = torch.from_numpy(z[t + ".gemm"])
            y32 = O.w4a16_ref(x, z[t + ".qweight"], s, z[t + ".qzeros"])
            # tolerance: max|y - y_ref| / max|y_ref| <= 1e-2 (fp16 accumulation order)
            assert O.rel_err(y_ref_kernel, y32) <= 1e-2, t
            # with the reference's own rounding points the agreement is ~1 fp16 ulp
            ysk = O.w4a16_splitk_ref(x, z[t + ".qweight"], s, z[t + ".qzeros"], 8)
            assert ysk.dtype == torch.float16
            assert O.rel_err(ysk, y_ref_kernel.float()) <= 2e-3, t


def test_bf16_dequant_single_rounding():
    c = O.make_case(256, 64, 1, dtype=torch.bfloat16, seed=3)
    W = O.dequantize(c["qweight"], c["qscales"], c["qzeros"])
    assert W.dtype == torch.bfloat16
    diff = c["iw"].astype(np.int32) - np.repeat(c["iz"].astype(np.int32), 128, 0)
    exact = torch.from_numpy(diff).float() * c["qscales"].float().repeat_interleave(128, 0)
    assert torch.equal(W, exact.to(torch.bfloat16))


def test_make_case_is_seeded():
    a, b = O.make_case(128, 64, 2, seed=5), O.make_case(128, 64, 2, seed=5)
    assert torch.equal(a["qweight"], b["qweight"]) and torch.equal(a["x"], b["x"])
    assert np.array_equal(O.unpack_int4(a["qweight"].numpy()), a["iw"])


def test_threaded_dequantize_equals_the_numpy_one():
    # the multi-threaded torch form that the benchmark's CPU baseline times
    for (K, N, g, dtype, seed) in ((256, 136, 128, torch.float16, 1), (192, 264, 64, torch.bfloat16, 2), (1024, 3072, 128, torch.float16, 3)):
        c = O.make_case(K, N, 1, group_size=g, dtype=dtype, seed=seed)
        a = O.dequantize(c["qweight"], c["qscales"], c["qzeros"])
        b = O.dequantize_threaded(c["qweight"], c["qscales"], c["qzeros"])
        assert a.dtype == b.dtype and torch.equal(a, b)
    words = torch.full((128, 4), -1, dtype=torch.int32)          # all-15 nibbles: the sign bit is in use
    zeros = torch.zeros(1, 4, dtype=torch.int32)
    s = torch.full((1, 32), 0.5, dtype=torch.float16)
    assert torch.equal(O.dequantize_threaded(words, s, zeros), O.dequantize(words, s, zeros))
