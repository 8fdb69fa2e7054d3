"""The two grid searches of AWQ calibration, batched so that they run as a few large tensor
operations on whatever device the tensors are on (the GPU in practice).

They follow the reference's ``AWQQuantizer`` (``nanoquantization/awq/quantizer.py``):

* ``best_clip``   — ``_compute_best_clip`` (:217-280): per output row and quantisation group, the
  clipping value (a fraction 1 - i/n_grid of the group's max |w|) whose clipped and fake-quantised
  weights reproduce the group's contribution to the output best.  The reference forms the
  ``[rows, tokens, groups, group_size]`` product of weights and inputs elementwise; here the
  per-group dot products are one batched matrix product per grid point, in chunks of rows.
* ``best_scales`` — ``_find_best_scales`` (:370-429): the exponent ``ratio`` in
  ``scales = mean|x| ** ratio`` (normalised) whose scaled, fake-quantised, unscaled weights change
  the inspected module's output least.
* ``pseudo_quantize`` — ``nanoquantization/utils/quantization.py:5-58``, the fake quantisation both
  use (the packing kernel ``nqb200_quantize_pack`` computes the same integers).

Offline code: none of it is on the inference path.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch


def pseudo_quantize(x: torch.Tensor, group_size: int, w_bits: int = 4, zero_point: bool = True):
    """Quantise and dequantise ``x`` in groups of ``group_size`` along its last dimension.
    Returns ``(x_dq, scales, zeros)`` as the reference does (``zeros`` is None for the symmetric form)."""
    orig_shape = x.shape
    if group_size > 0:
        assert x.shape[-1] % group_size == 0, "x.shape[-1] must be divisible by group_size"
        x = x.reshape(-1, group_size)
    assert not torch.isnan(x).any(), "weight should not contain nan"
    if zero_point:
        max_val, min_val = x.amax(dim=-1, keepdim=True), x.amin(dim=-1, keepdim=True)
        qmax = 2 ** w_bits - 1
        scales = (max_val - min_val).clamp(min=1e-5) / qmax
        zeros = (-torch.round(min_val / scales)).clamp(min=0, max=qmax)
        x = ((torch.round(x / scales) + zeros).clamp(min=0, max=qmax) - zeros) * scales
        zeros = zeros.view(orig_shape[0], -1)
    else:
        qmax, qmin = 2 ** (w_bits - 1) - 1, -(2 ** (w_bits - 1))
        scales = x.abs().amax(dim=-1, keepdim=True) / qmax
        x = torch.round(x / scales).clamp(min=qmin, max=qmax) * scales
        zeros = None
    return x.reshape(orig_shape), scales.view(orig_shape[0], -1), zeros


@torch.no_grad()
def best_clip(w: torch.Tensor, inp: torch.Tensor, group_size: int = 128, w_bits: int = 4, zero_point: bool = True,
              n_grid: int = 20, max_shrink: float = 0.5, n_sample_tokens: int = 512, rows_per_chunk: int = 1024) -> torch.Tensor:
    """``w [n_output, n_input]``, ``inp [..., n_input]`` -> the best clipping value ``[n_output, n_groups, 1]``."""
    assert w.ndim == 2, "weight should be 2D"
    gs = group_size if group_size > 0 else w.shape[-1]
    assert w.shape[-1] % gs == 0, "w.shape[-1] must be divisible by group_size"
    n_out, n_groups = w.shape[0], w.shape[-1] // gs
    x = inp.reshape(-1, inp.shape[-1])
    x = x[::max(1, x.shape[0] // n_sample_tokens)]                       # downsample the tokens as the reference does
    xg = x.reshape(x.shape[0], n_groups, gs).permute(1, 2, 0).contiguous()  # [groups, group_size, tokens]
    out = torch.empty(n_out, n_groups, 1, dtype=w.dtype, device=w.device)
    for r0 in range(0, n_out, rows_per_chunk):
        wc = w[r0:r0 + rows_per_chunk].reshape(-1, n_groups, gs)             # [rows, groups, group_size]
        rows = wc.shape[0]
        orig_max = wc.abs().amax(dim=-1, keepdim=True)                       # [rows, groups, 1]
        orig_out = torch.bmm(wc.transpose(0, 1), xg)                         # [groups, rows, tokens]
        min_err = torch.full((rows, n_groups, 1), float("inf"), dtype=w.dtype, device=w.device)
        best = orig_max.clone()
        for i in range(int(n_grid * max_shrink)):
            cur_max = orig_max * (1 - i / n_grid)
            q = pseudo_quantize(torch.clamp(wc, min=-cur_max, max=cur_max), gs, w_bits, zero_point)[0]
            cur_out = torch.bmm(q.reshape(rows, n_groups, gs).transpose(0, 1), xg)
            err = (orig_out - cur_out).pow(2).mean(dim=-1).transpose(0, 1).unsqueeze(-1)  # [rows, groups, 1]
            better = err < min_err
            min_err = torch.where(better, err, min_err)
            best = torch.where(better, cur_max, best)
        out[r0:r0 + rows] = best
    return out


@torch.no_grad()
def best_scales(inp: torch.Tensor, weights: Sequence[torch.Tensor], group_size: int = 128, w_bits: int = 4,
                zero_point: bool = True, n_grid: int = 20,
                forward: Optional[Callable[[Sequence[torch.Tensor]], torch.Tensor]] = None):
    """The per-input-channel scales that the reference's search picks for linears that share the input ``inp``.

    ``weights``: their ``[n_output, n_input]`` matrices.  ``forward(list_of_weights)`` returns the output of the
    inspected module for those weights; by default the inspected module is the single linear itself
    (``inp @ w.T``), the reference's case for ``o_proj`` and ``down_proj``.  Returns
    ``(scales [n_input], best_ratio, loss_history)``; nothing is modified."""
    if forward is None:
        assert len(weights) == 1, "a forward function is required for several layers"
        forward = lambda ws: inp @ ws[0].t()  # noqa: E731
    act = inp.reshape(-1, inp.shape[-1]).abs().mean(dim=0)
    orig = forward(list(weights))
    best_loss, best, best_ratio, history = float("inf"), None, -1, []
    for i in range(n_grid):
        ratio = i / n_grid
        s = act.pow(ratio).clamp(min=1e-4).view(-1)
        s = s / (s.max() * s.min()).sqrt()
        trial = [pseudo_quantize(w * s.view(1, -1), group_size, w_bits, zero_point)[0] / s.view(1, -1) for w in weights]
        loss = (orig - forward(trial)).float().pow(2).mean().item()
        history.append(loss)
        if loss < best_loss:
            best_loss, best, best_ratio = loss, s, ratio
    if best_ratio == -1:
        raise ValueError(f"Failed to find the best scales; loss history {history}")
    assert not torch.isnan(best).any()
    return best, best_ratio, history
