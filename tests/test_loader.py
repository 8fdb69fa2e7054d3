"""Checkpoint round trip and per-rank sliced reads (CPU): the reference's reader is
nanoquantization/utils/loader.py:20-48; the shards must equal slices of the full tensors."""
import json
import os

import pytest
import torch

from nanoquantization_b200.layers.parallel import shard_columns, shard_rows
from nanoquantization_b200.models.qwen3_quantized import Qwen3QuantizedForCausalLM
from nanoquantization_b200.utils import load_model, save_model, shard_slices

ARCH = dict(num_hidden_layers=2, vocab_size=512, hidden_size=256, total_num_heads=4, total_num_kv_heads=2,
            max_position_embeddings=64, intermediate_size=512, w_bits=4, group_size=128, head_dim=64)


def _randomise(model, seed):
    g = torch.Generator().manual_seed(seed)
    for name, t in list(model.named_buffers()) + list(model.named_parameters()):
        if t.dtype == torch.int32:
            t.data.copy_(torch.randint(-2**31, 2**31 - 1, t.shape, generator=g, dtype=torch.int64).to(torch.int32))
        else:
            t.data.copy_(torch.randn(t.shape, generator=g).to(t.dtype))


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("ckpt"))
    full = Qwen3QuantizedForCausalLM(**ARCH, device="cpu", dtype=torch.float16)
    _randomise(full, 5)
    save_model(full, path, config={"model_type": "qwen3"}, w_bits=4, group_size=128,
               calibration={"dataset": "wikitext", "dataset_subset": "wikitext-2-raw-v1", "n_samples": 128,
                            "max_seq_len": 512, "apply_clip": True})
    return path, full


def test_writer_layout_matches_the_reference_writer(checkpoint):
    # scripts/qwen3_0pt6_billion.py:188-235: model.safetensors, an index that maps every key to it, and a
    # quantization_config block with the calibration record
    path, full = checkpoint
    index = json.load(open(os.path.join(path, "model.safetensors.index.json")))
    assert index["metadata"] == {"format": "pt"}
    assert index["weight_map"] == {k: "model.safetensors" for k in full.state_dict()}
    quant = json.load(open(os.path.join(path, "config.json")))["quantization_config"]
    assert list(quant) == ["quant_method", "w_bits", "group_size", "zero_point", "version", "modules_to_not_convert",
                           "calibration"]
    assert quant["quant_method"] == "awq" and quant["version"] == "gemm" and quant["modules_to_not_convert"] == []
    assert list(quant["calibration"]) == ["dataset", "dataset_subset", "n_samples", "max_seq_len", "apply_clip"]


def test_round_trip_unsharded(checkpoint):
    path, full = checkpoint
    assert json.load(open(os.path.join(path, "config.json")))["quantization_config"]["group_size"] == 128
    again = Qwen3QuantizedForCausalLM(**ARCH, device="cpu", dtype=torch.float16)
    load_model(again, path)
    want = full.state_dict()
    got = again.state_dict()
    assert set(got) == set(want)
    for k in want:
        assert torch.equal(got[k], want[k]), k


@pytest.mark.parametrize("tp_size", [2])
def test_sharded_read_equals_slices_of_the_full_tensors(checkpoint, tp_size):
    path, full = checkpoint
    sd = full.state_dict()
    for rank in range(tp_size):
        m = Qwen3QuantizedForCausalLM(**ARCH, tp_size=tp_size, tp_rank=rank, device="cpu", dtype=torch.float16)
        load_model(m, path)
        got = m.state_dict()
        for i in range(ARCH["num_hidden_layers"]):
            for proj in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "mlp.gate_proj", "mlp.up_proj"):
                p = f"model.layers.{i}.{proj}."
                qw, qs, qz = shard_columns(sd[p + "qweight"], sd[p + "qscales"], sd[p + "qzeros"], tp_size, rank)
                assert torch.equal(got[p + "qweight"], qw) and torch.equal(got[p + "qscales"], qs) and torch.equal(got[p + "qzeros"], qz)
            for proj in ("self_attn.o_proj", "mlp.down_proj"):
                p = f"model.layers.{i}.{proj}."
                qw, qs, qz = shard_rows(sd[p + "qweight"], sd[p + "qscales"], sd[p + "qzeros"], 128, tp_size, rank)
                assert torch.equal(got[p + "qweight"], qw) and torch.equal(got[p + "qscales"], qs) and torch.equal(got[p + "qzeros"], qz)
            assert torch.equal(got[f"model.layers.{i}.input_layernorm.weight"], sd[f"model.layers.{i}.input_layernorm.weight"])
        v = ARCH["vocab_size"] // tp_size
        assert torch.equal(got["lm_head.weight"], sd["lm_head.weight"][rank * v:(rank + 1) * v])
        assert torch.equal(got["lm_head.bias"], sd["lm_head.bias"][rank * v:(rank + 1) * v])
        assert torch.equal(got["model.embed_tokens.weight"], sd["model.embed_tokens.weight"])


def test_slices_and_errors():
    # packed tensors shard by whole words, scales by 8 columns, row shards on group boundaries
    assert shard_slices("model.layers.0.mlp.up_proj.qweight", (256, 64), 2, 1, 128) == (slice(0, 256), slice(32, 64))
    assert shard_slices("model.layers.0.mlp.up_proj.qscales", (2, 512), 2, 1, 128) == (slice(0, 2), slice(256, 512))
    assert shard_slices("model.layers.0.mlp.down_proj.qweight", (512, 32), 2, 1, 128) == (slice(256, 512), slice(0, 32))
    assert shard_slices("model.layers.0.mlp.down_proj.qzeros", (4, 32), 2, 0, 128) == (slice(0, 2), slice(0, 32))
    assert shard_slices("model.norm.weight", (256,), 2, 1, 128) == (slice(0, 256),)
    with pytest.raises(ValueError):
        shard_slices("model.layers.0.mlp.down_proj.qweight", (384, 32), 2, 0, 128)  # 192 rows: not whole groups
    with pytest.raises(ValueError):
        shard_slices("model.layers.0.mlp.up_proj.qscales", (2, 24), 2, 0, 128)       # 12 columns: not whole words


def test_unknown_key_raises_like_the_reference(tmp_path):
    from safetensors.torch import save_file
    save_file({"model.layers.0.nothing.weight": torch.zeros(2)}, str(tmp_path / "x.safetensors"))
    m = Qwen3QuantizedForCausalLM(**ARCH, device="cpu", dtype=torch.float16)
    with pytest.raises(AttributeError, match="neither a parameter nor a buffer"):
        load_model(m, str(tmp_path))
