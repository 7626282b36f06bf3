"""Shared by the tests: the tiny configurations and small utilities.

The two configurations differ in every size and option: layers, width, head
counts and grouping (GQA 2:1 against MQA 8:1), head size (hidden / heads
against a decoupled one), intermediate size, vocabulary (neither a power of two
in B), rope base, eps, tied against untied head, position limit, and the seed.
"""

from __future__ import annotations

import json
import random
from pathlib import Path

import torch

TINY_CONFIGS = {
    "A": dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3",
        vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, head_dim=16,
        max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=10000.0,
        tie_word_embeddings=True,
    ),
    "B": dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3",
        vocab_size=384, hidden_size=96, intermediate_size=224, num_hidden_layers=3,
        num_attention_heads=8, num_key_value_heads=1, head_dim=32,
        max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=1000000.0,
        tie_word_embeddings=False,
    ),
    # sizes that are no power of two anywhere, head size 48, 3 kv heads
    "C": dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3",
        vocab_size=517, hidden_size=168, intermediate_size=328, num_hidden_layers=2,
        num_attention_heads=6, num_key_value_heads=3, head_dim=48,
        max_position_embeddings=320, rms_norm_eps=3e-6, rope_theta=50000.0,
        tie_word_embeddings=False,
    ),
    # head size 64: the size at which the bfloat16 path takes the tensor-core attention kernels
    "D": dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3",
        vocab_size=300, hidden_size=136, intermediate_size=200, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, head_dim=64,
        max_position_embeddings=384, rms_norm_eps=2e-6, rope_theta=100000.0,
        tie_word_embeddings=True,
    ),
    # the serving geometry: heads of 128 in groups of four, pages of 64, contexts beyond a thousand positions.
    # In bfloat16 this is the configuration that runs the kernels the large models run: the tcgen05 prefill
    # attention, the projection with the rotation in its epilogue (prompts of more than 256 tokens), the
    # decode attention that makes its own queries, decode graphs per bucket of 512 positions.
    "E": dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3",
        vocab_size=1000, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
        num_attention_heads=8, num_key_value_heads=2, head_dim=128,
        max_position_embeddings=1536, rms_norm_eps=1e-6, rope_theta=1000000.0,
        tie_word_embeddings=False,
    ),
}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4}
PAGE_SIZES = {"A": 16, "B": 8, "C": 32, "D": 16, "E": 64}

# Bounds on |engine logits - plain float32 logits|. float32: only the order of sums and the device's exp, sin
# and cos differ. bfloat16: activations are rounded to 8 bits of mantissa between kernels; the bound of a
# configuration is about three times the worst error the engine shows on it over all four ways of cutting
# (measured: see TOL_BF16_MEASURED), so a key that is wrong, missing or stale (which moves these logits by
# several times the bound, checked in test_gpu_replay.py) cannot pass.
TOL_F32 = 2e-5
TOL_BF16_MEASURED = {"A": 3.3e-3, "B": 4.8e-3, "C": 7.7e-3, "D": 6.9e-3, "E": 8.1e-3}
TOL_BF16 = {k: 3.0 * v for k, v in TOL_BF16_MEASURED.items()}
# The sharpened copies (q_norm gains tripled, test_gpu_replay.py) round worse, because their softmax turns a
# score's rounding error into a larger change of weight; measured the same way. Two pages of a request's block
# table swapped change these logits by 0.12 (A) to 2.0 (E), four to seventeen times the bound.
TOL_BF16_SHARP_MEASURED = {"A": 6.8e-3, "B": 2.7e-2, "C": 2.9e-2, "D": 2.3e-2, "E": 4.0e-2}
TOL_BF16_SHARP = {k: 3.0 * v for k, v in TOL_BF16_SHARP_MEASURED.items()}


def make_folder(path, name: str, dtype=torch.bfloat16) -> Path:
    from quantinfer_b200.config import config_from_dict
    from quantinfer_b200.weights import write_model_folder

    cfg = config_from_dict(TINY_CONFIGS[name])
    return write_model_folder(path, cfg, SEEDS[name], dtype)


def random_tokens(n: int, vocab: int, seed: int) -> list:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def vocab_of(folder) -> int:
    return json.loads((Path(folder) / "config.json").read_text())["vocab_size"]


def max_abs_diff(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double().cpu() - b.double().cpu()).abs().max())
