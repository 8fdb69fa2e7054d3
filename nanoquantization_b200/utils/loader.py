"""Checkpoint reader and writer for the quantised Qwen3 models.

On-disk format: the reference's (``nanoquantization/utils/loader.py:20-48`` reads
it, ``scripts/qwen3_0pt6_billion.py:179-235`` writes it): ``*.safetensors``
files holding one tensor per ``state_dict`` key
(``model.layers.{i}.self_attn.q_proj.qweight`` ...), copied by name into a
parameter or, failing that, a buffer, and a ``config.json`` whose
``quantization_config`` carries ``w_bits`` and ``group_size``.

``load_model(model, path)`` is the reference's call.  For a model built with
``tp_size > 1`` every rank reads only its own slice of each tensor from the file
(``safe_open(...).get_slice``): a column shard of q/k/v/gate/up (whole packed
words of ``qweight`` / ``qzeros``, the matching columns of ``qscales``), a row
shard of o/down on quantisation-group boundaries, a vocabulary shard of
``lm_head``.  No rank materialises a full tensor, and nothing is unpacked or
repacked.
"""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Optional

import torch
from torch import nn

_PACK = 8
_COLUMN = re.compile(r"\.(q_proj|k_proj|v_proj|gate_proj|up_proj)\.(qweight|qscales|qzeros|bias)$")
_ROW = re.compile(r"\.(o_proj|down_proj)\.(qweight|qscales|qzeros|bias)$")
_VOCAB = re.compile(r"^lm_head\.(weight|bias)$")


def _bounds(total: int, tp_size: int, tp_rank: int, unit: int, what: str) -> tuple[int, int]:
    if total % tp_size != 0 or (total // tp_size) % unit != 0:
        raise ValueError(f"{what}: {total} cannot be split into {tp_size} shards that are multiples of {unit}")
    per = total // tp_size
    return tp_rank * per, (tp_rank + 1) * per


def shard_slices(name: str, shape: tuple[int, ...], tp_size: int, tp_rank: int, group_size: int) -> tuple[slice, ...]:
    """The part of checkpoint tensor ``name`` (full shape ``shape``) that rank ``tp_rank`` of ``tp_size`` owns."""
    full = tuple(slice(0, s) for s in shape)
    if tp_size == 1:
        return full
    m = _COLUMN.search(name)
    if m:
        kind = m.group(2)
        if kind == "bias":
            return (slice(*_bounds(shape[0], tp_size, tp_rank, _PACK, name)),)
        # qweight / qzeros hold 8 output columns per word, qscales one per element: shard whole words
        unit = 1 if kind in ("qweight", "qzeros") else _PACK
        return (full[0], slice(*_bounds(shape[1], tp_size, tp_rank, unit, name)))
    m = _ROW.search(name)
    if m:
        kind = m.group(2)
        if kind == "bias":  # added once, after the all-reduce: every rank holds it whole
            return full
        # qweight has one row per input feature, qscales / qzeros one per quantisation group
        unit = group_size if kind == "qweight" else 1
        return (slice(*_bounds(shape[0], tp_size, tp_rank, unit, name)), full[1])
    if _VOCAB.search(name):
        return (slice(*_bounds(shape[0], tp_size, tp_rank, 1, name)),) + full[1:]
    return full  # embeddings and norms are replicated


def _destination(model: nn.Module, weight_name: str) -> torch.Tensor:
    # a parameter first, then a buffer (qweight, qscales, qzeros are buffers): loader.py:38-47
    try:
        return model.get_parameter(weight_name)
    except AttributeError:
        try:
            return model.get_buffer(weight_name)
        except AttributeError:
            raise AttributeError(f"`{weight_name}` is neither a parameter nor a buffer in the model")


def load_model(model: nn.Module, path: str, *, tp_size: Optional[int] = None, tp_rank: Optional[int] = None,
               group_size: Optional[int] = None) -> None:
    """Load every tensor of the checkpoint directory ``path`` into ``model`` by name.

    ``tp_size`` / ``tp_rank`` default to the model's own (``model.tp_size``, ``model.tp_rank``; 1 and 0 if
    it has none), ``group_size`` to the checkpoint's ``config.json`` or 128.  Call it before
    ``fuse_projections()``: the file's keys are the unfused q/k/v and gate/up projections.
    """
    from safetensors import safe_open

    tp_size = int(getattr(model, "tp_size", 1) if tp_size is None else tp_size)
    tp_rank = int(getattr(model, "tp_rank", 0) if tp_rank is None else tp_rank)
    if not 0 <= tp_rank < tp_size:
        raise ValueError(f"tp_rank={tp_rank} outside tp_size={tp_size}")
    if group_size is None:
        group_size = 128
        cfg_file = os.path.join(path, "config.json")
        if os.path.exists(cfg_file):
            with open(cfg_file) as fh:
                group_size = int(json.load(fh).get("quantization_config", {}).get("group_size", 128))
    tensor_files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not tensor_files:
        raise FileNotFoundError(f"no *.safetensors under {path}")
    for tensor_file in tensor_files:
        with safe_open(tensor_file, framework="pt", device="cpu") as f:
            for weight_name in f.keys():
                dst = _destination(model, weight_name)
                src = f.get_slice(weight_name)
                part = src[shard_slices(weight_name, tuple(src.get_shape()), tp_size, tp_rank, group_size)]
                if tuple(part.shape) != tuple(dst.shape):
                    raise ValueError(f"`{weight_name}`: this rank's slice has shape {tuple(part.shape)}, the model expects {tuple(dst.shape)}")
                dst.data.copy_(part)


def save_model(model: nn.Module, path: str, *, config: Optional[dict] = None, w_bits: int = 4, group_size: int = 128,
               zero_point: bool = True, calibration: Optional[dict] = None) -> None:
    """Write an unsharded (``tp_size == 1``), unfused model in the reference's layout
    (``scripts/qwen3_0pt6_billion.py:188-235``): ``model.safetensors`` with the ``state_dict`` keys,
    ``model.safetensors.index.json`` mapping every key to that file (:202-207) and, if ``config`` (the Hugging
    Face config as a dict) is given, ``config.json`` with the ``quantization_config`` block (:215-228).
    ``calibration`` is that block's ``calibration`` entry (``dataset``, ``dataset_subset``, ``n_samples``,
    ``max_seq_len``, ``apply_clip``); it is written when given."""
    from safetensors.torch import save_file

    if int(getattr(model, "tp_size", 1)) != 1:
        raise ValueError("save_model writes full tensors: build the model with tp_size=1")
    os.makedirs(path, exist_ok=True)
    # tied tensors are written under both names, as the reference's writer does
    tensors = {k: v.detach().to("cpu").contiguous().clone() for k, v in model.state_dict().items()}
    save_file(tensors, os.path.join(path, "model.safetensors"))
    index = {"metadata": {"format": "pt"}, "weight_map": {k: "model.safetensors" for k in tensors}}
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as fh:
        json.dump(index, fh, indent=2)
    if config is not None:
        cfg = dict(config)
        quant = {"quant_method": "awq", "w_bits": w_bits, "group_size": group_size, "zero_point": zero_point,
                 "version": "gemm", "modules_to_not_convert": []}
        if calibration is not None:
            quant["calibration"] = dict(calibration)
        cfg["quantization_config"] = quant
        with open(os.path.join(path, "config.json"), "w") as fh:
            json.dump(cfg, fh, indent=2)
