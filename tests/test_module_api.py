"""Host-side mirror of the reference module API (no GPU): constructor, buffers,
errors, packer parity against vectors made by the reference packer."""
import numpy as np
import pytest
import torch
import torch.nn as nn

import nanoquantization_b200 as nq
from nanoquantization_b200.layers import gemm as G


def test_constructor_buffers_and_defaults():
    m = nq.WQLinear_GEMM(4, 128, 1024, 3072)
    assert m.qweight.shape == (1024, 384) and m.qweight.dtype == torch.int32
    assert m.qscales.shape == (8, 3072) and m.qscales.dtype == torch.bfloat16  # reference default dtype
    assert m.qzeros.shape == (8, 384) and m.qzeros.dtype == torch.int32
    assert m.bias is None
    assert list(m.state_dict().keys()) == ["qweight", "qscales", "qzeros"]
    assert len(list(m.parameters())) == 0
    mb = nq.WQLinear_GEMM(4, 128, 256, 64, "cpu", True, torch.float16)
    assert mb.bias.dtype == torch.bfloat16 and mb.qscales.dtype == torch.float16
    assert list(mb.state_dict().keys()) == ["qweight", "qscales", "qzeros", "bias"]


def test_constructor_errors():
    with pytest.raises(ValueError):
        nq.WQLinear_GEMM(8, 128, 256, 64)
    with pytest.raises(AssertionError):
        nq.WQLinear_GEMM(4, 128, 200, 64)
    with pytest.raises(AssertionError):
        nq.WQLinear_GEMM(4, 128, 256, 60)


def test_forward_has_no_cpu_path():
    m = nq.WQLinear_GEMM(4, 128, 256, 64, output_dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        m(torch.zeros(2, 256, dtype=torch.float16))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        nq.awq_dequantize(m.qweight, m.qscales, m.qzeros)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        nq.awq_gemm(torch.zeros(2, 256, dtype=torch.float16), m.qweight, m.qscales, m.qzeros, 8)


def test_function_argument_checks_match_reference():
    m = nq.WQLinear_GEMM(4, 128, 256, 64, output_dtype=torch.float16)
    x = torch.zeros(2, 256, dtype=torch.float16)
    with pytest.raises(AssertionError):
        nq.awq_gemm(x, m.qweight, m.qscales, m.qzeros, 6)  # not a power of two
    with pytest.raises(AssertionError):
        nq.awq_gemm(x[:, :128], m.qweight, m.qscales, m.qzeros, 8)  # K mismatch
    with pytest.raises(AssertionError):
        nq.awq_dequantize(m.qweight, m.qscales, m.qzeros[:, :4])
    with pytest.raises(AssertionError):  # group size 16 is not in the supported list
        nq.awq_dequantize(m.qweight, torch.zeros(16, 64, dtype=torch.float16), torch.zeros(16, 8, dtype=torch.int32))


def test_pack_int4_bit_exact_vs_reference_packer(golden):
    z = golden("pack_vectors.npz")
    tags = sorted({k[:-3] for k in z.files if k.endswith(".iw")})
    for t in tags:
        assert np.array_equal(nq.pack_int4(torch.from_numpy(z[t + ".iw"].astype(np.int32))).numpy(), z[t + ".qweight"]), t
        assert np.array_equal(nq.pack_int4(torch.from_numpy(z[t + ".iz"].astype(np.int32))).numpy(), z[t + ".qzeros"]), t


def test_from_linear_bit_exact_vs_reference(golden):
    z = golden("from_linear_vectors.npz")
    tags = sorted({k[:-10] for k in z.files if k.endswith(".weight_fq")})
    assert tags
    for t in tags:
        K, N, g = (int(p[1:]) for p in t.split("_"))
        lin = nn.Linear(K, N, bias=False).to(torch.float16)
        lin.weight.data = torch.from_numpy(z[t + ".weight_fq"])
        m = nq.WQLinear_GEMM.from_linear(lin, 4, g, torch.from_numpy(z[t + ".scales"]),
                                         torch.from_numpy(z[t + ".zeros"]), output_dtype=torch.float16)
        assert np.array_equal(m.qweight.numpy(), z[t + ".qweight"]), t
        assert np.array_equal(m.qzeros.numpy(), z[t + ".qzeros"]), t
        assert np.array_equal(m.qscales.numpy().view(np.uint16), z[t + ".qscales"].view(np.uint16)), t
        assert m.qweight.dtype == torch.int32 and m.bias is None


def test_from_linear_with_bias_and_state_dict_roundtrip():
    torch.manual_seed(0)
    lin = nn.Linear(128, 16, bias=True)
    s = torch.full((1, 16), 0.01)
    zp = torch.full((1, 16), 8.0)
    m = nq.WQLinear_GEMM.from_linear(lin, 4, 128, s, zp, output_dtype=torch.float16)
    assert m.bias is not None and m.bias.dtype == torch.float16  # from_linear casts the bias (gemm.py:476)
    m2 = nq.WQLinear_GEMM(4, 128, 128, 16, bias=True, output_dtype=torch.float16)
    m2.load_state_dict(m.state_dict())
    assert torch.equal(m2.qweight, m.qweight) and torch.equal(m2.qzeros, m.qzeros)
    assert G.AWQ_TRITON_SUPPORTED_GROUP_SIZES == [-1, 32, 64, 128]
