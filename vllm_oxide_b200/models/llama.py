"""The Llama dense decoder as a list of parts: the one architecture this engine serves.

Tensor names are the checkpoint's own (crates/engine/src/weights.rs:167-183): nothing is
renamed; q/k/v and gate/up are concatenated row-wise when the parts are built, which leaves
every output element as it was. `lm_head.weight` exists exactly when the configuration does
not tie the embeddings (the reference, which serves a tied model only, rejects the tensor:
crates/engine/src/weights.rs:154-156).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from ..config.model_config import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..parts import (Attention, Block, Embedding, LayerCall, LMHead, ModelSpec, RMSNorm, Rotary, SwiGLU)
from ..parts.linear import to_compute
from ..weights.loader import TensorSpec, WeightSet


@dataclass
class BuildContext:
    dtype: torch.dtype
    device: str


def llama_manifest(cfg: LlamaConfig) -> Dict[str, TensorSpec]:
    h, q, kv, inter, v = cfg.hidden_size, cfg.q_dim, cfg.kv_dim, cfg.intermediate_size, cfg.vocab_size
    m = {"model.embed_tokens.weight": TensorSpec((v, h))}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        m[p + "input_layernorm.weight"] = TensorSpec((h,), init="ones")
        m[p + "self_attn.q_proj.weight"] = TensorSpec((q, h))
        m[p + "self_attn.k_proj.weight"] = TensorSpec((kv, h))
        m[p + "self_attn.v_proj.weight"] = TensorSpec((kv, h))
        m[p + "self_attn.o_proj.weight"] = TensorSpec((h, q))
        m[p + "post_attention_layernorm.weight"] = TensorSpec((h,), init="ones")
        m[p + "mlp.gate_proj.weight"] = TensorSpec((inter, h))
        m[p + "mlp.up_proj.weight"] = TensorSpec((inter, h))
        m[p + "mlp.down_proj.weight"] = TensorSpec((h, inter))
    m["model.norm.weight"] = TensorSpec((h,), init="ones")
    if not cfg.tie_word_embeddings:
        m["lm_head.weight"] = TensorSpec((v, h))
    return m


def build_llama(cfg: LlamaConfig, weights: WeightSet, ctx: BuildContext) -> ModelSpec:
    """Every layer: RMSNorm -> attention (GQA, rotary) -> RMSNorm -> SwiGLU, chosen here layer by
    layer; layers run once each, in order, each with a cache of its own."""
    dt, dev = ctx.dtype, ctx.device
    rotary = Rotary(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling, dev)
    embedding = Embedding(weights.take("model.embed_tokens.weight"), dt, dev)
    blocks, schedule = [], []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = Attention(weights.take(p + "self_attn.q_proj.weight"), weights.take(p + "self_attn.k_proj.weight"),
                          weights.take(p + "self_attn.v_proj.weight"), weights.take(p + "self_attn.o_proj.weight"),
                          cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, position=rotary,
                          dtype=dt, device=dev)
        ff = SwiGLU(weights.take(p + "mlp.gate_proj.weight"), weights.take(p + "mlp.up_proj.weight"),
                    weights.take(p + "mlp.down_proj.weight"), dt, dev)
        blocks.append(Block(RMSNorm(weights.take(p + "input_layernorm.weight"), cfg.rms_norm_eps, dev), mixer,
                            RMSNorm(weights.take(p + "post_attention_layernorm.weight"), cfg.rms_norm_eps, dev), ff))
        schedule.append(LayerCall(layer=i, cache=i, write=True))
    final_norm = RMSNorm(weights.take("model.norm.weight"), cfg.rms_norm_eps, dev)
    if cfg.tie_word_embeddings:
        head = LMHead(embedding.table)
    else:
        head = LMHead(to_compute(weights.take("lm_head.weight"), dt, dev))
    weights.finish()
    wbytes = sum(b.weight_bytes() for b in blocks) + final_norm.weight_bytes() + head.weight_bytes()
    return ModelSpec(embedding=embedding, blocks=blocks, schedule=schedule, final_norm=final_norm, lm_head=head,
                     hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
                     max_position=cfg.max_position_embeddings, eos_token_ids=cfg.eos_token_ids, weight_bytes=wbytes)


LLAMA = Architecture(name="LlamaForCausalLM", config_cls=LlamaConfig, manifest=llama_manifest, build=build_llama)
register_architecture(LLAMA, replace=True)
