"""Generate the golden vectors in this directory from the reference itself.

Run once, in a container that has the reference checked out (pass its path as
the first argument or in NANOQ_REFERENCE); the resulting ``*.npz`` files are
committed and are what the test-suite reads.  Nothing at test time needs the
reference.

What is run:
  * the reference packer ``WQLinear_GEMM.from_linear`` (gemm.py:447-550) on CPU;
  * the reference Triton kernels ``awq_dequantize`` (gemm.py:126-180) and
    ``awq_gemm`` (gemm.py:329-379) under ``TRITON_INTERPRET=1`` on CPU tensors,
    fp16 only (the interpreter truncates bf16 instead of rounding) and only for
    shapes with N % 256 == 0 and K % 32 == 0 (the dequantize kernel's load mask
    is transposed at ragged edges, gemm.py:27-31).

Usage:  python tests/golden/make_golden.py /path/to/reference
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
ref_path = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NANOQ_REFERENCE")
if not ref_path:
    raise SystemExit("give the path of the reference checkout")
sys.path.insert(0, ref_path)

import numpy as np  # noqa: E402
import torch  # noqa: E402
from nanoquantization.layers.gemm import WQLinear_GEMM, awq_dequantize, awq_gemm  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def pack_with_reference(iw, iz, g):
    """Integers in, packed words out, through the reference packer: a weight of
    ``iw - iz`` with unit scales quantises back to exactly ``iw``."""
    K, N = iw.shape
    lin = torch.nn.Linear(K, N, bias=False)
    lin.weight.data = (iw - iz.repeat_interleave(g, 0)).t().float().contiguous()
    m = WQLinear_GEMM.from_linear(lin, 4, g, torch.ones(K // g, N), iz.float(),
                                  output_dtype=torch.float16)
    return m.qweight.numpy(), m.qzeros.numpy()


def pack_cases():
    out = {}
    shapes = [(128, 8, 128), (128, 136, 128), (256, 256, 128), (96, 64, 32),
              (384, 1024, 128), (64, 24, 64)]
    for i, (K, N, g) in enumerate(shapes):
        iw = torch.randint(0, 16, (K, N), generator=gen(100 + i), dtype=torch.int32)
        iz = torch.randint(0, 16, (K // g, N), generator=gen(200 + i), dtype=torch.int32)
        qw, qz = pack_with_reference(iw, iz, g)
        tag = f"K{K}_N{N}_g{g}"
        out[f"{tag}.iw"] = iw.numpy().astype(np.uint8)
        out[f"{tag}.iz"] = iz.numpy().astype(np.uint8)
        out[f"{tag}.qweight"] = qw
        out[f"{tag}.qzeros"] = qz
    # extremes: all 15 (sign bit set in every word) and all 0
    for name, val in (("all15", 15), ("all0", 0)):
        iw = torch.full((128, 16), val, dtype=torch.int32)
        iz = torch.full((1, 16), val, dtype=torch.int32)
        qw, qz = pack_with_reference(iw, iz, 128)
        out[f"{name}.iw"] = iw.numpy().astype(np.uint8)
        out[f"{name}.iz"] = iz.numpy().astype(np.uint8)
        out[f"{name}.qweight"] = qw
        out[f"{name}.qzeros"] = qz
    np.savez_compressed(os.path.join(HERE, "pack_vectors.npz"), **out)
    print("pack_vectors.npz", len(out), "arrays")


def pseudo_quantize_tensor(x, group_size, w_bits):
    # the recipe of the reference's own fixture, awq/tests/dequantization_kernel.py:12-48
    shape = x.shape
    x = x.view(-1, group_size)
    mx = x.amax(dim=-1, keepdim=True)
    mn = x.amin(dim=-1, keepdim=True)
    qmax = 2 ** w_bits - 1
    scales = (mx - mn).clamp(min=1e-5) / qmax
    zeros = (-torch.round(mn / scales)).clamp(min=0, max=qmax)
    x = (torch.round(x / scales) + zeros).clamp(min=0, max=qmax)
    x = (x - zeros) * scales
    return x.reshape(shape), scales.view(shape[0], -1), zeros.view(shape[0], -1)


def from_linear_cases():
    """The reference unit test's fixture recipe with fixed seeds: fp16 weight ->
    pseudo-quantise -> from_linear."""
    out = {}
    for i, (K, N, g) in enumerate([(256, 256, 32), (256, 512, 128)]):
        w = torch.randn(N, K, generator=gen(300 + i)).to(torch.float16)
        wq, s, z = pseudo_quantize_tensor(w.clone(), g, 4)
        s = s.t().contiguous()
        z = z.t().contiguous()
        lin = torch.nn.Linear(K, N, bias=False).to(torch.float16)
        lin.weight.data = wq
        m = WQLinear_GEMM.from_linear(lin, 4, g, s, z, output_dtype=torch.float16)
        tag = f"K{K}_N{N}_g{g}"
        out[f"{tag}.weight_fq"] = wq.numpy()
        out[f"{tag}.scales"] = s.numpy()
        out[f"{tag}.zeros"] = z.numpy()
        out[f"{tag}.qweight"] = m.qweight.numpy()
        out[f"{tag}.qzeros"] = m.qzeros.numpy()
        out[f"{tag}.qscales"] = m.qscales.numpy()
        # the reference's dequantize kernel on that module (interpreter, fp16)
        W = awq_dequantize(m.qweight, m.qscales, m.qzeros)
        out[f"{tag}.dequant"] = W.numpy()
        x = torch.randn(8, K, generator=gen(400 + i)).to(torch.float16)
        y = awq_gemm(x, m.qweight, m.qscales, m.qzeros, split_k_iters=8)
        out[f"{tag}.x"] = x.numpy()
        out[f"{tag}.gemm"] = y.numpy()
    np.savez_compressed(os.path.join(HERE, "from_linear_vectors.npz"), **out)
    print("from_linear_vectors.npz", len(out), "arrays")


def kernel_cases():
    """Benchmark-distribution inputs through the reference kernels (fp16)."""
    out = {}
    for i, (K, N, g, M) in enumerate([(256, 256, 128, 1), (512, 256, 128, 16),
                                      (256, 512, 64, 5)]):
        iw = torch.randint(0, 16, (K, N), generator=gen(500 + i), dtype=torch.int32)
        iz = torch.randint(0, 16, (K // g, N), generator=gen(600 + i), dtype=torch.int32)
        qw, qz = pack_with_reference(iw, iz, g)
        s = (torch.rand(K // g, N, generator=gen(700 + i)) * 9e-3 + 1e-3).to(torch.float16)
        x = torch.randn(M, K, generator=gen(800 + i)).to(torch.float16)
        qw_t, qz_t = torch.from_numpy(qw), torch.from_numpy(qz)
        W = awq_dequantize(qw_t, s, qz_t)
        y = awq_gemm(x, qw_t, s, qz_t, split_k_iters=8)
        tag = f"K{K}_N{N}_g{g}_M{M}"
        out[f"{tag}.qweight"] = qw
        out[f"{tag}.qzeros"] = qz
        out[f"{tag}.qscales"] = s.numpy()
        out[f"{tag}.x"] = x.numpy()
        out[f"{tag}.dequant"] = W.numpy()
        out[f"{tag}.gemm"] = y.numpy()
    np.savez_compressed(os.path.join(HERE, "kernel_vectors.npz"), **out)
    print("kernel_vectors.npz", len(out), "arrays")


if __name__ == "__main__":
    torch.manual_seed(0)
    pack_cases()
    from_linear_cases()
    kernel_cases()
