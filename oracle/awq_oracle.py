"""CPU oracle for the AWQ W4A16 linear path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU, the arithmetic of the reference's
``nanoquantization/layers/gemm.py``.  It exists to check the CUDA kernels; it
is not a fallback.  Only the test-suite, the smoke check and the CPU-baseline
leg of the benchmark may import it; the shipped package never does.

Parity status: PINNED.  ``tests/golden/`` holds vectors produced by running
the reference's own packer (``WQLinear_GEMM.from_linear``) and its two Triton
kernels under ``TRITON_INTERPRET=1`` (fp16); ``tests/test_oracle_golden.py``
checks every function here against them.  The M >= 256 branch of the reference
calls ``torch.matmul`` (cuBLAS), whose summation order is not pinned by any
reference test; for that branch the fp32 dequantize-then-matmul answer computed
here is the reference answer.

Integer work is done in numpy, dtype-sensitive floating point in torch (CPU),
because numpy has no bfloat16.
"""
from __future__ import annotations

import numpy as np
import torch

# gemm.py:504-513 -- nibble j of a packed word holds element AWQ_ORDER[j].
AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)
# gemm.py:64-69, 245-249 -- element e of a word sits at bit AWQ_SHIFTS[e].
AWQ_SHIFTS = (0, 16, 4, 20, 8, 24, 12, 28)
PACK = 8  # 32 // w_bits, gemm.py:501


def pack_int4(values) -> np.ndarray:
    """Pack ``[R, C]`` integers into ``[R, C/8]`` int32 words in AWQ order.

    Follows gemm.py:501-520 (weights) and gemm.py:523-548 (zero-points):
    ``word |= values[:, 8*i + order[j]] << (4*j)`` in int32 arithmetic, with no
    clamp, so the top nibble lands in the sign bit.
    """
    v = np.asarray(values).astype(np.int64)
    rows, cols = v.shape
    assert cols % PACK == 0
    v = v.reshape(rows, cols // PACK, PACK)
    word = np.zeros((rows, cols // PACK), dtype=np.int64)
    for j, e in enumerate(AWQ_ORDER):
        word |= v[:, :, e] << (4 * j)
    # wrap to the int32 bit pattern exactly as the in-place int32 OR does
    return (word & 0xFFFFFFFF).astype(np.uint32).view(np.int32)


def unpack_int4(words) -> np.ndarray:
    """Unpack ``[R, C/8]`` int32 words into ``[R, C]`` uint8 values 0..15.

    Follows the kernels' shift table, gemm.py:64-69 and gemm.py:301-302:
    ``(word >> shift[e]) & 0xF``.
    """
    w = np.ascontiguousarray(np.asarray(words)).view(np.uint32)
    rows, cw = w.shape
    out = np.empty((rows, cw, PACK), dtype=np.uint8)
    for e, sh in enumerate(AWQ_SHIFTS):
        out[:, :, e] = (w >> np.uint32(sh)) & np.uint32(0xF)
    return out.reshape(rows, cw * PACK)


def _as_np_i32(t) -> np.ndarray:
    if isinstance(t, torch.Tensor):
        return t.detach().cpu().contiguous().numpy()
    return np.asarray(t)


def dequantize(qweight, qscales: torch.Tensor, qzeros) -> torch.Tensor:
    """Dense ``W[K, N] = dtype(q - z) * s`` in ``qscales.dtype``.

    Follows gemm.py:112 and gemm.py:303-304: the integer difference is taken
    first, promoted to the scale dtype (exact, |q - z| <= 15) and multiplied
    once, i.e. one rounding per element.
    """
    q = unpack_int4(_as_np_i32(qweight)).astype(np.int32)
    z = unpack_int4(_as_np_i32(qzeros)).astype(np.int32)
    K = q.shape[0]
    G = z.shape[0]
    assert K % G == 0
    g = K // G
    diff = q - np.repeat(z, g, axis=0)
    s = qscales.detach().cpu()
    d = torch.from_numpy(diff).to(s.dtype)
    return d * s.repeat_interleave(g, dim=0)


def dequantize_threaded(qweight: torch.Tensor, qscales: torch.Tensor, qzeros: torch.Tensor) -> torch.Tensor:
    """``dequantize`` with torch CPU ops only, so that it runs on all host threads (numpy's shifts
    and masks run on one).  Same arithmetic and citations: shift table gemm.py:64-69, integer
    difference first and one multiply in the scale dtype gemm.py:112, 303-304.  This is the form the
    benchmark's CPU baseline times; ``tests/test_oracle_golden.py`` checks it equals ``dequantize``."""
    sh = torch.tensor(AWQ_SHIFTS, dtype=torch.int32)
    q = ((qweight.unsqueeze(-1) >> sh) & 0xF).reshape(qweight.shape[0], -1)       # arithmetic shift, then mask: bits 0..3
    z = ((qzeros.unsqueeze(-1) >> sh) & 0xF).reshape(qzeros.shape[0], -1)
    g = q.shape[0] // z.shape[0]
    diff = (q.view(z.shape[0], g, -1) - z.unsqueeze(1)).to(qscales.dtype)
    return (diff * qscales.unsqueeze(1)).reshape(q.shape[0], -1)


def w4a16_ref(x: torch.Tensor, qweight, qscales: torch.Tensor, qzeros,
              bias: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 answer of the linear: ``x.float() @ dequantize(...).float() (+ bias)``.

    The weight is rounded to the scale dtype exactly as the reference does
    (gemm.py:304, gemm.py:560) and the contraction is done in fp32.  Bias add
    follows gemm.py:565-566.  Returned in fp32 so the caller chooses how to
    compare.
    """
    W = dequantize(qweight, qscales, qzeros).float()
    x2 = x.detach().cpu().reshape(-1, x.shape[-1]).float()
    y = x2 @ W
    if bias is not None:
        y = y + bias.detach().cpu().float()
    return y.reshape(*x.shape[:-1], W.shape[1])


def w4a16_splitk_ref(x: torch.Tensor, qweight, qscales: torch.Tensor, qzeros,
                     split_k_iters: int = 8, block_k: int = 32) -> torch.Tensor:
    """The small-M branch with the reference's own rounding points.

    gemm.py:255-326 gives K-split ``p`` the rows ``32*(8*i + p) .. +31``, keeps
    an fp32 accumulator, rounds each split's partial to the output dtype
    (gemm.py:324) and sums the partials with ``Tensor.sum(0)`` (gemm.py:378).
    Returned in ``qscales.dtype``.
    """
    W = dequantize(qweight, qscales, qzeros)
    dt = W.dtype
    K = W.shape[0]
    xf = x.detach().cpu().reshape(-1, K).to(dt).float()
    Wf = W.float()
    parts = []
    for p in range(split_k_iters):
        rows = [r for blk in range(p * block_k, K, block_k * split_k_iters)
                for r in range(blk, min(blk + block_k, K))]
        idx = torch.tensor(rows, dtype=torch.long)
        parts.append((xf[:, idx] @ Wf[idx]).to(dt))
    return torch.stack(parts).sum(dim=0)


def quantize_to_int(weight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                    group_size: int) -> np.ndarray:
    """``intweight[k, n] = round(W[n, k] / scales[k//g, n] + zeros[k//g, n])``.

    Follows gemm.py:478-491 (round-half-even, no clamp).  ``weight`` is
    ``[N, K]`` as in ``nn.Linear``; ``scales``/``zeros`` are ``[K/g, N]``.
    """
    w = weight.detach().cpu()
    s = scales.detach().cpu().repeat_interleave(group_size, dim=0).t()
    z = zeros.detach().cpu().repeat_interleave(group_size, dim=0).t()
    iw = torch.round(w / s + z).to(torch.int32)
    return iw.t().contiguous().numpy()


def from_linear_ref(weight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                    group_size: int, output_dtype: torch.dtype):
    """The whole packer: returns ``(qweight, qscales, qzeros)`` as torch CPU tensors.

    Follows gemm.py:447-550.
    """
    iw = quantize_to_int(weight, scales, zeros, group_size)
    qweight = torch.from_numpy(pack_int4(iw))
    qzeros = torch.from_numpy(pack_int4(zeros.detach().cpu().to(torch.int32).numpy()))
    qscales = scales.detach().cpu().clone().to(output_dtype)
    return qweight, qscales, qzeros


def pseudo_quantize(w: torch.Tensor, group_size: int, w_bits: int = 4):
    """Asymmetric group-wise fake quantisation, as in the reference's test fixture.

    Follows nanoquantization/utils/quantization.py:20-41 and
    nanoquantization/awq/tests/dequantization_kernel.py:12-48.  Returns the
    fake-quantised weight, ``scales [N, K/g]`` and ``zeros [N, K/g]``.
    """
    shape = w.shape
    x = w.reshape(-1, group_size)
    mx = x.amax(dim=-1, keepdim=True)
    mn = x.amin(dim=-1, keepdim=True)
    qmax = 2 ** w_bits - 1
    scales = (mx - mn).clamp(min=1e-5) / qmax
    zeros = (-torch.round(mn / scales)).clamp(min=0, max=qmax)
    xq = (torch.round(x / scales) + zeros).clamp(min=0, max=qmax)
    xdq = (xq - zeros) * scales
    return xdq.reshape(shape), scales.view(shape[0], -1), zeros.view(shape[0], -1)


# --------------------------------------------------------------------------
# Seeded synthetic inputs with the benchmark's distributions.
# --------------------------------------------------------------------------

def make_case(K: int, N: int, M: int, group_size: int = 128,
              dtype: torch.dtype = torch.float16, seed: int = 0, bias: bool = False):
    """int4 weights / zero-points uniform in [0, 15], scales uniform in
    [1e-3, 1e-2], activations N(0, 1); one generator per tensor."""
    def gen(k):
        g = torch.Generator(device="cpu")
        g.manual_seed(seed * 1000 + k)
        return g
    iw = torch.randint(0, 16, (K, N), generator=gen(1), dtype=torch.int32)
    iz = torch.randint(0, 16, (K // group_size, N), generator=gen(2), dtype=torch.int32)
    scales = (torch.rand(K // group_size, N, generator=gen(3)) * 9e-3 + 1e-3).to(dtype)
    x = torch.randn(M, K, generator=gen(4)).to(dtype)
    out = {
        "iw": iw.numpy().astype(np.uint8),
        "iz": iz.numpy().astype(np.uint8),
        "qweight": torch.from_numpy(pack_int4(iw.numpy())),
        "qzeros": torch.from_numpy(pack_int4(iz.numpy())),
        "qscales": scales,
        "x": x,
        "bias": None,
    }
    if bias:
        out["bias"] = torch.randn(N, generator=gen(5)).to(torch.bfloat16)
    return out


def rel_err(y: torch.Tensor, y_ref: torch.Tensor) -> float:
    """The headline tolerance metric: ``max|y - y_ref| / max|y_ref|``."""
    y = y.detach().cpu().float()
    y_ref = y_ref.detach().cpu().float()
    return float((y - y_ref).abs().max() / y_ref.abs().max().clamp(min=1e-30))
