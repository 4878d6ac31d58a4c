"""Typed model configuration read from a model folder's config.json.

The reference keeps Llama 3.2 1B's hyperparameters as a compile-time constant
with config.json's own key names (crates/engine/src/config.rs:10-54) and checks
the keys it relies on against the downloaded file once
(crates/engine/tests/real_model.rs:27-58). Here the file is the only source of
sizes: nothing below holds a number of any particular checkpoint.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, asdict
from typing import Optional, Tuple

from ..errors import ConfigError


@dataclass(frozen=True)
class RopeScaling:
    """llama3 frequency scaling (crates/engine/src/config.rs:26-32)."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_json(self) -> dict:
        d = asdict(self)
        d["rope_type"] = "llama3"
        return d


def _need(d: dict, key: str, typ, where: str):
    if key not in d:
        raise ConfigError(f"{where}: required key '{key}' is missing")
    return _typed(d, key, typ, where)


def _typed(d: dict, key: str, typ, where: str):
    v = d[key]
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{where}: '{key}' must be a number, got {v!r}")
        return float(v)
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{where}: '{key}' must be an integer, got {v!r}")
        return v
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"{where}: '{key}' must be true or false, got {v!r}")
        return v
    raise AssertionError(typ)


@dataclass(frozen=True)
class LlamaConfig:
    """The Llama dense decoder's hyperparameters, by config.json's key names."""
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    tie_word_embeddings: bool
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "LlamaForCausalLM"

    # ---- derived sizes (crates/engine/src/config.rs:72-101) ----
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def gqa_group(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def param_count(self) -> int:
        """Total parameters, a tied embedding counted once
        (crates/engine/src/config.rs:85-95)."""
        h = self.hidden_size
        attn = h * self.q_dim + 2 * h * self.kv_dim + self.q_dim * h
        mlp = 3 * h * self.intermediate_size
        norms = 2 * h
        embed = self.vocab_size * h
        head = 0 if self.tie_word_embeddings else self.vocab_size * h
        return embed + head + self.num_hidden_layers * (attn + mlp + norms) + h

    def kv_bytes_per_token(self, bytes_per_elem: int) -> int:
        """K and V of one token over all layers (crates/engine/src/config.rs:99-101)."""
        return 2 * self.num_hidden_layers * self.kv_dim * bytes_per_elem

    # ---- validation ----
    def validate(self) -> None:
        pos = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
               "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings")
        for k in pos:
            if getattr(self, k) <= 0:
                raise ConfigError(f"config: '{k}' must be positive, got {getattr(self, k)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config: head_dim {self.head_dim} must be even for rotate-half RoPE")
        if not (self.rms_norm_eps > 0 and math.isfinite(self.rms_norm_eps)):
            raise ConfigError(f"config: rms_norm_eps must be a positive number, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0 and math.isfinite(self.rope_theta)):
            raise ConfigError(f"config: rope_theta must be a positive number, got {self.rope_theta}")
        rs = self.rope_scaling
        if rs is not None:
            if rs.factor <= 0 or rs.original_max_position_embeddings <= 0:
                raise ConfigError("config: rope_scaling.factor and original_max_position_embeddings "
                                  "must be positive")
            if rs.high_freq_factor == rs.low_freq_factor:
                raise ConfigError("config: rope_scaling.high_freq_factor must differ from low_freq_factor")

    # ---- config.json ----
    @classmethod
    def from_dict(cls, d: dict, where: str = "config.json") -> "LlamaConfig":
        archs = d.get("architectures")
        if not (isinstance(archs, list) and len(archs) >= 1 and isinstance(archs[0], str)):
            raise ConfigError(f"{where}: 'architectures' must be a list with the model class name")
        # Keys whose value would change the math if it differed: refuse rather than ignore
        # (the reference asserts them, crates/engine/tests/real_model.rs:41-45).
        fixed = {"hidden_act": "silu", "attention_bias": False, "mlp_bias": False, "model_type": "llama"}
        for k, want in fixed.items():
            if k in d and d[k] != want:
                raise ConfigError(f"{where}: '{k}' = {d[k]!r} is not supported (only {want!r})")
        # keys that switch on something this architecture does not compute: only their "off" values pass
        off_values = {"sliding_window": (None, 0), "attention_dropout": (None, 0, 0.0), "pretraining_tp": (None, 1)}
        for k, allowed in off_values.items():
            v = d.get(k)
            if isinstance(v, bool) or not any(v is a or (a is not None and v == a) for a in allowed):
                raise ConfigError(f"{where}: '{k}' = {v!r} is not supported by this architecture")
        hidden = _need(d, "hidden_size", int, where)
        heads = _need(d, "num_attention_heads", int, where)
        if heads <= 0:
            raise ConfigError(f"{where}: 'num_attention_heads' must be positive")
        kv_heads = _typed(d, "num_key_value_heads", int, where) if d.get("num_key_value_heads") is not None else heads
        if d.get("head_dim") is not None:
            head_dim = _typed(d, "head_dim", int, where)
        else:
            if hidden % heads != 0:
                raise ConfigError(f"{where}: hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads} and 'head_dim' is not given")
            head_dim = hidden // heads
        rs = d.get("rope_scaling")
        scaling = None
        if rs is not None:
            if not isinstance(rs, dict):
                raise ConfigError(f"{where}: 'rope_scaling' must be an object or null")
            kind = rs.get("rope_type", rs.get("type"))
            if kind != "llama3":
                raise ConfigError(f"{where}: rope_scaling.rope_type {kind!r} is not supported (only 'llama3')")
            w = where + ": rope_scaling"
            scaling = RopeScaling(
                factor=_need(rs, "factor", float, w),
                low_freq_factor=_need(rs, "low_freq_factor", float, w),
                high_freq_factor=_need(rs, "high_freq_factor", float, w),
                original_max_position_embeddings=_need(rs, "original_max_position_embeddings", int, w))
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"{where}: 'eos_token_id' must be an integer or a list of integers")
        cfg = cls(
            hidden_size=hidden,
            intermediate_size=_need(d, "intermediate_size", int, where),
            num_hidden_layers=_need(d, "num_hidden_layers", int, where),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=_need(d, "vocab_size", int, where),
            max_position_embeddings=_need(d, "max_position_embeddings", int, where),
            rms_norm_eps=_need(d, "rms_norm_eps", float, where),
            rope_theta=_typed(d, "rope_theta", float, where) if "rope_theta" in d else _missing_theta(where),
            rope_scaling=scaling,
            tie_word_embeddings=_typed(d, "tie_word_embeddings", bool, where) if "tie_word_embeddings" in d else False,
            bos_token_id=_typed(d, "bos_token_id", int, where) if d.get("bos_token_id") is not None else None,
            eos_token_ids=eos_ids,
            architecture=archs[0],
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_json() if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return d


def _missing_theta(where: str):
    raise ConfigError(f"{where}: required key 'rope_theta' is missing")


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except OSError as e:
        raise ConfigError(f"cannot read {path}: {e}") from e
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d


def write_config_json(model_dir: str, d: dict) -> None:
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=2)
        f.write("\n")
