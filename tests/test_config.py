"""Configuration and registry (no GPU)."""
import json
import os

import pytest

from vllm_oxide_b200 import models  # noqa: F401
from vllm_oxide_b200.config import (EngineConfig, LlamaConfig, RopeScaling, architecture_for, known_architectures,
                                    read_config_json, write_config_json)
from vllm_oxide_b200.errors import ConfigError
from tests.util import TINY_A, TINY_B, TINY_C

# The public config.json of Llama 3.2 1B, by the keys the reference checks
# (crates/engine/src/config.rs:36-54; crates/engine/tests/real_model.rs:27-58).
LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu", "attention_bias": False,
    "mlp_bias": False, "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256,
    "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192, "rope_type": "llama3"},
    "tie_word_embeddings": True, "bos_token_id": 128000, "eos_token_id": 128001, "torch_dtype": "bfloat16",
}


def test_llama_1b_derived_sizes():
    c = LlamaConfig.from_dict(LLAMA_1B)
    # the reference's compile-time facts (crates/engine/src/config.rs:105-115)
    assert c.head_dim == 64 and c.gqa_group == 4
    assert c.param_count() == 1_235_814_400
    assert c.kv_bytes_per_token(4) == 64 * 1024 and c.kv_bytes_per_token(2) == 32 * 1024
    assert c.eos_token_ids == (128001,) and c.bos_token_id == 128000
    assert c.rope_scaling == RopeScaling(32.0, 1.0, 4.0, 8192)


def test_roundtrip_through_config_json(tmp_path):
    for cfg in (TINY_A, TINY_B, TINY_C):
        d = str(tmp_path / f"m{cfg.hidden_size}")
        write_config_json(d, cfg.to_dict())
        assert LlamaConfig.from_dict(read_config_json(d)) == cfg


def test_defaults_and_derivations():
    d = {k: v for k, v in LLAMA_1B.items() if k not in ("head_dim", "num_key_value_heads", "rope_scaling",
                                                       "tie_word_embeddings", "eos_token_id", "bos_token_id")}
    c = LlamaConfig.from_dict(d)
    assert c.head_dim == 2048 // 32 and c.num_key_value_heads == 32
    assert c.rope_scaling is None and c.tie_word_embeddings is False and c.eos_token_ids == ()
    d["eos_token_id"] = [1, 2, 3]
    assert LlamaConfig.from_dict(d).eos_token_ids == (1, 2, 3)
    d["head_dim"] = 48          # head_dim from config.json wins over hidden / heads
    assert LlamaConfig.from_dict(d).q_dim == 32 * 48


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta"])
def test_missing_required_key(key):
    d = dict(LLAMA_1B)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(d)


@pytest.mark.parametrize("patch,match", [
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"), ({"model_type": "mistral"}, "model_type"),
    ({"num_key_value_heads": 5}, "multiple"), ({"head_dim": 63}, "even"),
    ({"hidden_size": "2048"}, "integer"), ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "llama3"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
    ({"sliding_window": 4096}, "sliding_window"), ({"tie_word_embeddings": "yes"}, "true or false"),
    ({"sliding_window": 1}, "sliding_window"), ({"attention_dropout": 1}, "attention_dropout"),
    ({"attention_dropout": 0.1}, "attention_dropout"), ({"pretraining_tp": 2}, "pretraining_tp"),
    ({"pretraining_tp": 0}, "pretraining_tp"), ({"sliding_window": True}, "sliding_window"),
    ({"eos_token_id": "x"}, "eos_token_id"), ({"architectures": []}, "architectures"),
])
def test_bad_values_are_refused(patch, match):
    d = dict(LLAMA_1B)
    d.update(patch)
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict(d)


@pytest.mark.parametrize("patch", [{"sliding_window": None}, {"sliding_window": 0}, {"attention_dropout": 0.0},
                                   {"attention_dropout": 0}, {"pretraining_tp": 1}, {"pretraining_tp": None}])
def test_off_values_of_unsupported_features_pass(patch):
    d = dict(LLAMA_1B)
    d.update(patch)
    LlamaConfig.from_dict(d)


def test_registry():
    assert "LlamaForCausalLM" in known_architectures()
    arch = architecture_for(LLAMA_1B)
    assert arch.config_cls is LlamaConfig
    assert len(arch.manifest(LlamaConfig.from_dict(LLAMA_1B))) == 146      # crates/engine/tests/real_model.rs:66
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):             # the error lists what is known
        architecture_for({"architectures": ["GPT2LMHeadModel"]})


def test_unreadable_config(tmp_path):
    with pytest.raises(ConfigError, match="cannot read"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))


def test_engine_config():
    e = EngineConfig()
    # the reference's defaults (crates/engine/src/model.rs:56-66)
    assert (e.max_batch_tokens, e.max_seqs, e.max_model_len, e.block_size, e.kv_pool_bytes) == (2048, 32, 8192, 16, 2 << 30)
    assert EngineConfig(dtype="float32").dtype.is_floating_point
    with pytest.raises(ConfigError):
        EngineConfig(dtype="float16")
    with pytest.raises(ConfigError):
        EngineConfig(block_size=12)
    with pytest.raises(ConfigError):
        EngineConfig(max_seqs=0)
