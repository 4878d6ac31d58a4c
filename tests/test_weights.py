"""Weights: the safetensors reader and writer, the one-error check, random weights (no GPU)."""
import os
import struct

import pytest
import torch

from vllm_oxide_b200 import models  # noqa: F401
from vllm_oxide_b200.errors import WeightsError, WeightsFormatError
from vllm_oxide_b200.models import llama_manifest
from vllm_oxide_b200.weights import (SafetensorsFile, TensorSpec, load_safetensors_weights, random_tensors,
                                     weights_from_tensors, write_random_model, write_safetensors)
from tests.util import TINY_A, TINY_B


def test_roundtrip_and_bit_patterns(tmp_path):
    # bf16 bit patterns as the reference's reader test (crates/engine/src/weights.rs:343-348)
    bits = torch.tensor([0x3F80, 0xC000 - 0x10000, 0x0000, 0x3DCD], dtype=torch.int16)
    t = {"a": bits.view(torch.bfloat16).reshape(2, 2), "b": torch.arange(6, dtype=torch.float32).reshape(3, 2),
         "c": torch.tensor([1, 2, 3], dtype=torch.int64)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    f = SafetensorsFile(p)
    assert sorted(f.names()) == ["a", "b", "c"]
    assert f.tensor("a").dtype == torch.bfloat16 and f.tensor("a").float().flatten().tolist() == [1.0, -2.0, 0.0, 0.10009765625]
    assert torch.equal(f.tensor("b"), t["b"]) and torch.equal(f.tensor("c"), t["c"])
    from safetensors.torch import load_file          # the official reader agrees
    lf = load_file(p)
    assert all(torch.equal(lf[k], t[k]) for k in t)


def test_storage_dtypes_are_kept(tmp_path):
    man = {"w": TensorSpec((2, 2)), "n": TensorSpec((2,), init="ones"), "h": TensorSpec((2,)), "i": TensorSpec((3,), kind="int")}
    d = str(tmp_path)
    write_safetensors(os.path.join(d, "model.safetensors"), {
        "w": torch.ones(2, 2, dtype=torch.bfloat16), "n": torch.ones(2, dtype=torch.float32),
        "h": torch.ones(2, dtype=torch.float16), "i": torch.tensor([1, 2, 3], dtype=torch.int64)})
    w = load_safetensors_weights(d, man)
    assert w.take("w").dtype == torch.bfloat16      # bfloat16 stays bfloat16
    assert w.take("n").dtype == torch.float32       # a tensor stored in 32-bit stays so
    assert w.take("h").dtype == torch.float32       # float16 is widened (exact)
    assert w.take("i").dtype == torch.int32         # integer tables become int32
    w.finish()


def test_one_error_lists_everything(tmp_path):
    cfg = TINY_A
    man = llama_manifest(cfg)
    t = random_tensors(man, 1)
    del t["model.layers.0.self_attn.q_proj.weight"]
    del t["model.norm.weight"]
    t["lm_head.weight"] = torch.zeros(cfg.vocab_size, cfg.hidden_size, dtype=torch.bfloat16)      # tied config: unexpected
    t["extra.tensor"] = torch.zeros(1)
    t["model.layers.1.mlp.down_proj.weight"] = t["model.layers.1.mlp.down_proj.weight"].t().contiguous()   # transposed
    t["model.layers.1.input_layernorm.weight"] = t["model.layers.1.input_layernorm.weight"].to(torch.int32)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightsError) as ei:
        load_safetensors_weights(str(tmp_path), man)
    e = ei.value
    assert e.missing == ["model.layers.0.self_attn.q_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["extra.tensor", "lm_head.weight"]
    assert e.wrong_shape == [("model.layers.1.mlp.down_proj.weight", (64, 128), (128, 64))]
    assert e.wrong_dtype == [("model.layers.1.input_layernorm.weight", "I32")]
    msg = str(e)
    for needle in ("missing (2)", "unexpected (2)", "expected [64, 128], file has [128, 64]", "model.norm.weight", "I32"):
        assert needle in msg


def test_untied_needs_lm_head(tmp_path):
    man = llama_manifest(TINY_B)
    assert "lm_head.weight" in man and "lm_head.weight" not in llama_manifest(TINY_A)
    t = random_tensors(man, 2)
    del t["lm_head.weight"]
    with pytest.raises(WeightsError) as ei:
        weights_from_tensors(t, man)
    assert ei.value.missing == ["lm_head.weight"]


def test_garbage_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(WeightsFormatError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightsFormatError, match="header length"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 8) + b"not json")
    with pytest.raises(WeightsFormatError, match="not JSON"):
        SafetensorsFile(str(p))
    hdr = b'{"a":{"dtype":"F32","shape":[4],"data_offsets":[0,64]}}'
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(WeightsFormatError, match="outside the file"):
        SafetensorsFile(str(p))
    with pytest.raises(WeightsFormatError, match="cannot open"):
        SafetensorsFile(str(tmp_path / "nope.safetensors"))


def test_random_weights_are_seeded_and_order_free(tmp_path):
    man = llama_manifest(TINY_A)
    a, b = random_tensors(man, 7), random_tensors(dict(reversed(list(man.items()))), 7)
    assert all(torch.equal(a[k], b[k]) for k in man)
    c = random_tensors(man, 8)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert torch.all(a["model.norm.weight"] == 1)
    w = a["model.layers.0.mlp.up_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    d = str(tmp_path / "m")
    write_random_model(d, TINY_B, seed=3, std=0.05)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    loaded = load_safetensors_weights(d, llama_manifest(TINY_B))
    assert loaded.param_count() == TINY_B.param_count()      # crates/engine/src/weights.rs:225-227
    again = random_tensors(llama_manifest(TINY_B), 3, 0.05)
    assert torch.equal(loaded.take("lm_head.weight"), again["lm_head.weight"])


def test_take_and_finish():
    man = {"a": TensorSpec((1,)), "b": TensorSpec((1,))}
    w = weights_from_tensors({"a": torch.zeros(1), "b": torch.zeros(1)}, man)
    w.take("a")
    with pytest.raises(WeightsError, match="did not use: b"):
        w.finish()
    with pytest.raises(WeightsError):
        w.take("zzz")


def test_checkpoint_in_shards(tmp_path):
    """A folder without model.safetensors but with model.safetensors.index.json: the shards its
    weight_map names are read as one checkpoint, and one error still lists everything wrong."""
    import json
    from vllm_oxide_b200.weights import write_safetensors
    manifest = llama_manifest(TINY_A)
    tensors = random_tensors(manifest, seed=5, std=0.05)
    names = sorted(tensors)
    cut = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:cut], "model-00002-of-00002.safetensors": names[cut:]}
    d = tmp_path / "sharded"
    d.mkdir()
    for fn, ns in shards.items():
        write_safetensors(str(d / fn), {n: tensors[n] for n in ns})
    (d / "model.safetensors.index.json").write_text(json.dumps(
        {"metadata": {"total_size": 0}, "weight_map": {n: fn for fn, ns in shards.items() for n in ns}}))
    ws = load_safetensors_weights(str(d), manifest)
    for n in names:
        assert torch.equal(ws.take(n), tensors[n])
    ws.finish()
    # a tensor missing from its shard, one left over, and one stored twice
    gone, extra = shards["model-00002-of-00002.safetensors"][0], "model.layers.9.extra.weight"
    second = {n: tensors[n] for n in shards["model-00002-of-00002.safetensors"] if n != gone}
    second[extra] = torch.zeros(2, dtype=torch.bfloat16)
    write_safetensors(str(d / "model-00002-of-00002.safetensors"), second)
    with pytest.raises(WeightsError) as e:
        load_safetensors_weights(str(d), manifest)
    assert e.value.missing == [gone] and e.value.unexpected == [extra]
    second[names[0]] = tensors[names[0]]
    write_safetensors(str(d / "model-00002-of-00002.safetensors"), second)
    with pytest.raises(WeightsError, match="more than one shard"):
        load_safetensors_weights(str(d), manifest)
    (d / "model.safetensors.index.json").write_text("{}")
    with pytest.raises(WeightsFormatError, match="not a shard index"):
        load_safetensors_weights(str(d), manifest)
