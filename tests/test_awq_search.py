"""The batched AWQ calibration searches against vectors produced by the reference's
AWQQuantizer (tests/golden/make_golden_search.py), on CPU."""
import os

import numpy as np
import pytest
import torch

from nanoquantization_b200.awq import best_clip, best_scales, pseudo_quantize

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "awq_search_vectors.npz"))


def _clip_error(w, x, clip, gs):
    """Output error per (row, group) of clipping at `clip`, the quantity the search minimises."""
    n_out, n_in = w.shape
    xs = x.reshape(-1, n_in)
    xs = xs[::max(1, xs.shape[0] // 512)].reshape(-1, n_in // gs, gs)
    wg = w.reshape(n_out, n_in // gs, gs)
    q = pseudo_quantize(torch.clamp(wg, min=-clip, max=clip), gs)[0].reshape(wg.shape)
    return (torch.einsum("tgk,ogk->otg", xs, wg) - torch.einsum("tgk,ogk->otg", xs, q)).pow(2).mean(1)


@pytest.mark.parametrize("i", [0, 1, 2])
def test_best_clip_matches_the_reference(i):
    w, x = torch.from_numpy(GOLD[f"clip{i}.w"]), torch.from_numpy(GOLD[f"clip{i}.x"])
    gs, want = int(GOLD[f"clip{i}.gs"]), torch.from_numpy(GOLD[f"clip{i}.best"])
    got = best_clip(w, x, group_size=gs, rows_per_chunk=7)   # ragged chunks on purpose
    assert got.shape == want.shape
    same = got == want
    # the two sum in different orders, so grid points with (nearly) equal error may swap: then the errors agree
    assert same.float().mean() >= 0.97
    e_got, e_want = _clip_error(w, x, got, gs), _clip_error(w, x, want, gs)
    assert torch.allclose(e_got, e_want, rtol=1e-3, atol=1e-9)
    assert (got < w.reshape(w.shape[0], -1, gs).abs().amax(-1, keepdim=True)).any()   # something was clipped


@pytest.mark.parametrize("i", [0, 1])
def test_best_scales_matches_the_reference(i):
    w, x = torch.from_numpy(GOLD[f"scale{i}.w"]), torch.from_numpy(GOLD[f"scale{i}.x"])
    gs, want = int(GOLD[f"scale{i}.gs"]), torch.from_numpy(GOLD[f"scale{i}.scales"])
    w0 = w.clone()
    scales, ratio, history = best_scales(x, [w], group_size=gs)
    assert torch.equal(w, w0) and len(history) == 20 and 0.0 <= ratio < 1.0
    assert torch.allclose(scales, want, rtol=1e-5, atol=1e-7)
    # a custom forward (two linears sharing the input) goes through the same search
    both, _, _ = best_scales(x, [w, w * 0.5], group_size=gs, forward=lambda ws: torch.cat([x @ ws[0].t(), x @ ws[1].t()], -1))
    assert both.shape == scales.shape and torch.isfinite(both).all()


def test_pseudo_quantize_matches_the_oracle():
    import oracle.awq_oracle as O
    w = torch.randn(32, 256, generator=torch.Generator().manual_seed(1))
    a, sa, za = pseudo_quantize(w, 128)
    b, sb, zb = O.pseudo_quantize(w, 128, 4)
    assert torch.equal(a, b) and torch.equal(sa, sb) and torch.equal(za, zb)
    sym = pseudo_quantize(w, 64, 4, zero_point=False)
    assert sym[2] is None and sym[0].shape == w.shape


@pytest.mark.gpu
def test_searches_on_the_gpu_agree_with_the_cpu():
    w, x = torch.from_numpy(GOLD["clip0.w"]), torch.from_numpy(GOLD["clip0.x"])
    gs = int(GOLD["clip0.gs"])
    cpu = best_clip(w, x, group_size=gs)
    gpu = best_clip(w.cuda(), x.cuda(), group_size=gs).cpu()
    # different summation orders may swap grid points of nearly equal error: compare what they achieve
    assert (cpu == gpu).float().mean() >= 0.85
    e_gpu, e_cpu = _clip_error(w, x, gpu, gs), _clip_error(w, x, cpu, gs)
    assert float(e_gpu.sum()) <= 1.02 * float(e_cpu.sum()) and torch.allclose(e_gpu, e_cpu, rtol=0.3, atol=1e-9)
    ws, xs = torch.from_numpy(GOLD["scale0.w"]), torch.from_numpy(GOLD["scale0.x"])
    s_cpu = best_scales(xs, [ws], group_size=int(GOLD["scale0.gs"]))[0]
    s_gpu = best_scales(xs.cuda(), [ws.cuda()], group_size=int(GOLD["scale0.gs"]))[0].cpu()
    assert torch.allclose(s_cpu, s_gpu, rtol=1e-4, atol=1e-6)
