"""The plain-C restatement (oracle/awq_oracle.c) against the Python oracle."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import awq_oracle as O

ORACLE_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle")


@pytest.fixture(scope="module")
def clib():
    subprocess.check_call(["make", "-s", "-C", ORACLE_DIR])
    return ctypes.CDLL(os.path.join(ORACLE_DIR, "libawq_oracle.so"))


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("K,N,g,M", [(256, 64, 128, 3), (96, 24, 32, 1), (128, 8, 128, 5)])
def test_c_oracle_matches_python(clib, dtype, K, N, g, M):
    c = O.make_case(K, N, M, group_size=g, dtype=dtype, seed=11, bias=True)
    qw = c["qweight"].numpy()
    qz = c["qzeros"].numpy()
    sc = c["qscales"].view(torch.int16).numpy().view(np.uint16)
    code = 0 if dtype == torch.float16 else 1

    un = np.empty((K, N), dtype=np.uint8)
    clib.awq_oracle_unpack_int4(_p(qw), _p(un), ctypes.c_int64(K), ctypes.c_int64(N // 8))
    assert np.array_equal(un, c["iw"])

    W = np.empty((K, N), dtype=np.uint16)
    clib.awq_oracle_dequant(_p(qw), _p(sc), _p(qz), _p(W), ctypes.c_int64(K), ctypes.c_int64(N),
                            ctypes.c_int64(g), ctypes.c_int(code))
    Wpy = O.dequantize(qw, c["qscales"], qz).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(W, Wpy)

    x = c["x"].view(torch.int16).numpy().view(np.uint16)
    b = c["bias"].view(torch.int16).numpy().view(np.uint16)
    y = np.empty((M, N), dtype=np.float32)
    scratch = np.empty((K, N), dtype=np.uint16)
    clib.awq_oracle_gemm_f32(_p(x), _p(qw), _p(sc), _p(qz), _p(b), ctypes.c_int(1), _p(y),
                             ctypes.c_int64(M), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int64(g),
                             ctypes.c_int(code), _p(scratch))
    ypy = O.w4a16_ref(c["x"], qw, c["qscales"], qz, c["bias"])
    assert O.rel_err(torch.from_numpy(y), ypy) < 1e-5
