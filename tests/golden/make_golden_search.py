"""Golden vectors of the AWQ calibration searches, from the reference itself.

Run once in a container that has the reference checked out:
    python tests/golden/make_golden_search.py /path/to/reference
It calls ``AWQQuantizer._compute_best_clip`` and ``AWQQuantizer._find_best_scales``
(nanoquantization/awq/quantizer.py:217-280, 370-429) on seeded fp32 tensors on CPU and writes
``awq_search_vectors.npz`` next to this file.  Nothing at test time needs the reference.
"""
import os
import sys

ref_path = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NANOQ_REFERENCE")
if not ref_path:
    raise SystemExit("give the path of the reference checkout")
sys.path.insert(0, ref_path)

import numpy as np  # noqa: E402
import torch  # noqa: E402
from nanoquantization.awq.quantizer import AWQQuantizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def quantizer(group_size, w_bits=4, zero_point=True):
    q = object.__new__(AWQQuantizer)   # the searches only read these three attributes
    q.group_size, q.w_bits, q.zero_point = group_size, w_bits, zero_point
    return q


def gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


out = {}
for i, (n_out, n_in, tokens, gs) in enumerate([(24, 256, 96, 128), (16, 128, 700, 64), (40, 384, 64, 128)]):
    w = torch.randn(n_out, n_in, generator=gen(10 + i)) * 0.05
    w[::5, ::17] *= 8.0                                   # outliers make clipping worthwhile
    x = torch.randn(2, tokens // 2, n_in, generator=gen(20 + i))
    clip = quantizer(gs)._compute_best_clip(w.clone(), x.clone())
    out[f"clip{i}.w"], out[f"clip{i}.x"], out[f"clip{i}.gs"], out[f"clip{i}.best"] = w.numpy(), x.numpy(), np.int64(gs), clip.numpy()


class Block(torch.nn.Module):
    def __init__(self, n_in, n_out):
        super().__init__()
        self.prev = torch.nn.Linear(n_in, n_in, bias=False)
        self.fc = torch.nn.Linear(n_in, n_out, bias=False)


for i, (n_out, n_in, tokens, gs) in enumerate([(48, 256, 64, 128), (32, 128, 40, 64)]):
    blk = Block(n_in, n_out)
    blk.fc.weight.data = torch.randn(n_out, n_in, generator=gen(30 + i)) * 0.05
    x = torch.randn(tokens, n_in, generator=gen(40 + i)) * (1.0 + 4.0 * torch.rand(n_in, generator=gen(50 + i)))
    w0 = blk.fc.weight.data.clone()
    res = quantizer(gs)._find_best_scales(blk, blk.prev, [blk.fc], x.clone())
    assert torch.equal(blk.fc.weight.data, w0)            # the reference restores the weights
    out[f"scale{i}.w"], out[f"scale{i}.x"], out[f"scale{i}.gs"] = w0.numpy(), x.numpy(), np.int64(gs)
    out[f"scale{i}.scales"] = res["weight_scales"].numpy()

np.savez_compressed(os.path.join(HERE, "awq_search_vectors.npz"), **out)
print("wrote", len(out), "arrays")
