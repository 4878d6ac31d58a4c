"""Shared helpers of the tests: the two tiny configurations, model folders, comparisons."""
from __future__ import annotations

import dataclasses
import os
import random

import torch

from vllm_oxide_b200.config import LlamaConfig, RopeScaling
from vllm_oxide_b200.weights import write_random_model
from vllm_oxide_b200 import models  # noqa: F401  (registers the architecture)

# Two tiny configurations of the architecture that differ in every size and option.
TINY_A = LlamaConfig(
    hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, vocab_size=256, max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0,
    rope_scaling=None, tie_word_embeddings=True, bos_token_id=1, eos_token_ids=(2,))
TINY_B = LlamaConfig(
    hidden_size=96, intermediate_size=224, num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1,
    head_dim=32, vocab_size=384, max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=500000.0,
    rope_scaling=RopeScaling(8.0, 1.0, 4.0, 64), tie_word_embeddings=False, bos_token_id=0, eos_token_ids=(5, 7))
# head_dim given by config.json and different from hidden/heads; odd head and group counts
TINY_C = LlamaConfig(
    hidden_size=80, intermediate_size=176, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=3,
    head_dim=48, vocab_size=301, max_position_embeddings=512, rms_norm_eps=3e-5, rope_theta=20000.0,
    rope_scaling=RopeScaling(4.0, 1.0, 2.0, 32), tie_word_embeddings=True)

# head_dim 64: the size the bfloat16 engine's tensor-core attention kernels take (Llama 3.2 1B's)
TINY_D = LlamaConfig(
    hidden_size=96, intermediate_size=160, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
    head_dim=64, vocab_size=200, max_position_embeddings=1024, rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=RopeScaling(32.0, 1.0, 4.0, 128), tie_word_embeddings=True)

# The layer sizes of Llama 3.2 1B (hidden 2048, 32/8 heads of 64, intermediate 8192, vocabulary
# 128256, llama3 scaling 32/1/4/8192, tied), two layers: the sizes the benchmark runs, small enough
# for the plain implementation. Weights as in a checkpoint (std 0.02): with this width larger ones
# would saturate every softmax.
LAYERS_1B = LlamaConfig(
    hidden_size=2048, intermediate_size=8192, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8,
    head_dim=64, vocab_size=128256, max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=RopeScaling(32.0, 1.0, 4.0, 8192), tie_word_embeddings=True)

# The same layers with a vocabulary of 2,048: steps of dozens of requests and of thousands of rows
# stay affordable for the plain implementation (the head is the largest product at full vocabulary)
LAYERS_1B_V2K = dataclasses.replace(LAYERS_1B, vocab_size=2048)

# TINY_D for contexts of thousands of keys (the decode kernels choose by context length)
TINY_D_LONG = dataclasses.replace(TINY_D, max_position_embeddings=16384)

# Two layers of a wider model with head size 128 and three heads per kv head (Llama 3.2 3B's
# attention sizes; vocabulary and feed-forward kept small for the plain implementation), untied head
LAYERS_HD128 = LlamaConfig(
    hidden_size=3072, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=24, num_key_value_heads=8,
    head_dim=128, vocab_size=1000, max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=RopeScaling(32.0, 1.0, 4.0, 8192), tie_word_embeddings=False)

TINY = {"HD128": (LAYERS_HD128, 0.02, 16), "A": (TINY_A, 0.02, 16), "B": (TINY_B, 0.05, 8), "C": (TINY_C, 0.04, 16), "D": (TINY_D, 0.05, 16),
        "DL": (TINY_D_LONG, 0.05, 16), "1B": (LAYERS_1B, 0.02, 16), "1Bv": (LAYERS_1B_V2K, 0.02, 16)}   # config, std, page size


def make_model_dir(tmp_path, name: str, seed: int = 1234, std=None) -> str:
    cfg, s, _ = TINY[name]
    d = os.path.join(str(tmp_path), f"tiny_{name}_{seed}")
    if not os.path.exists(os.path.join(d, "model.safetensors")):
        # larger weights than a checkpoint's so that attention is far from uniform and a wrong
        # key or a stale page changes the logits visibly; norm weights away from 1
        write_random_model(d, cfg, seed, std=(std if std is not None else (s if name in ("1B", "1Bv", "HD128") else max(s, 0.08))), norm_jitter=0.3)
    return d


def random_tokens(n: int, vocab: int, seed: int):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def max_rel_diff(a: torch.Tensor, b: torch.Tensor) -> float:
    """max|a-b| / max|b|, the reference's measure (crates/engine/src/testutil.rs:94-98)."""
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


# Tolerances, stated once. float32: the engine and the float64 oracle differ by float32 rounding
# accumulated over a few hundred operations per logit; the reference allows 1e-5 relative between
# two float32 paths (crates/engine/src/model.rs:492,536), twice that against float64 here.
# bfloat16: activations, cache and weights are rounded to 8 mantissa bits (relative 2^-9 per
# rounding); about ten roundings per layer, independent, over <= 3 layers, on top of products
# accumulated in float32: 2^-9 * sqrt(30) ~ 1.1e-2 of the largest logit; 2e-2 leaves room for the
# vocabulary-wide maximum of that error (the worst seen over all traces is 1.5e-2). One wrong page
# read by one layer shows as 6e-2 and more (test_a_wrong_page_in_one_layer_is_seen_in_bfloat16).
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}
