"""Configurations drawn at random (head counts and grouping, head sizes from 16 to 256 in steps of
16, widths and vocabularies that are no power of two, page sizes that are none either) and random
requests through the engine, whole and cut in every way, against the plain implementation. The
long cases reach the kernels that only prompts of more than 256 tokens take (the projection with
the fused rotation, the tensor-memory attention at head size 128)."""

import random
from pathlib import Path

import pytest
import torch

from helpers import TOL_F32, random_tokens
from trace_tools import (mixed_trace, plain_rows, portions_trace, round64, run_trace_engine, tail_trace, whole_trace,
                         worst_diff)

pytestmark = pytest.mark.gpu

# the bound of the fixed configurations, for logits of a few units (larger logits scale it, see below)
TOL_BF16_RANDOM = 3e-2


def _case(tmp_path, seed: int, long: bool):
    from quantinfer_b200.config import config_from_dict
    from quantinfer_b200.weights import write_model_folder

    rng = random.Random(seed)
    nkv = rng.choice([1, 1, 2, 3, 4, 5, 8])
    nq = nkv * rng.choice([1, 1, 2, 3, 4, 7, 8])
    d = rng.choice([128, 128, 64, 96]) if long else rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128, 144, 256])
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3",
               vocab_size=rng.choice([50, 97, 256, 300, 517, 1000, 1031]),
               hidden_size=rng.choice([40, 64, 72, 100, 136, 200, 264, 90, 154]),
               intermediate_size=rng.choice([24, 56, 100, 136, 328, 250, 77]),
               num_hidden_layers=rng.choice([1, 2, 3]), num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d,
               max_position_embeddings=1024, rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-6, 1e-4]),
               rope_theta=rng.choice([1e4, 5e4, 1e6, 7.5e5]), tie_word_embeddings=rng.choice([True, False]))
    page = rng.choice([4, 8, 16, 32, 64, 24, 128])
    folder = write_model_folder(Path(tmp_path) / "m", config_from_dict(cfg), seed, torch.bfloat16)
    lens = ([rng.randint(257, 900) for _ in range(rng.randint(1, 2))] if long
            else [rng.randint(2, 200) for _ in range(rng.randint(1, 5))])
    if long:
        lens += [rng.randint(2, 200) for _ in range(3)]      # so that the long ones share steps with others
    requests = {f"r{i}": random_tokens(n, cfg["vocab_size"], seed=seed * 10 + i) for i, n in enumerate(lens)}
    expect = plain_rows(folder, requests)
    # the tolerances of the fixed configurations hold for logits of a few units; larger logits scale them
    scale = max(1.0, max(float(abs(v).max()) for v in expect.values()) / 3.0)
    room = sum(round64(n) + page for n in lens) + 256
    sizes = (2, 3, 17, 64, 130, 300) if long else (2, 3, 5, 8, 13, 16, 17, 30)
    for dtype, tol in (("float32", TOL_F32), ("bfloat16", TOL_BF16_RANDOM)):
        mixed, peak = mixed_trace(requests, seed=seed, max_tokens=round64(max(lens)) + 256 if len(lens) > 2 else None, sizes=sizes)
        for kind, steps, max_tokens in (("whole", whole_trace(requests), room), ("tail", tail_trace(requests, 32), room),
                                        ("portions", portions_trace(requests, seed=seed), room),
                                        ("mixed", mixed, peak + 4 * page)):
            got = run_trace_engine(folder, dtype, steps, max_tokens, page)
            worst, where = worst_diff(got, expect)
            assert worst <= tol * scale, f"{dtype} {kind}: {worst:.3g} at {where}; config {cfg}, pages of {page}, lengths {lens}"


@pytest.mark.parametrize("seed", [0, 5, 11, 14, 20, 26])
def test_random_configuration(tmp_path, seed):
    _case(tmp_path, seed, long=False)


@pytest.mark.parametrize("seed", [101, 106, 118])
def test_random_configuration_with_long_prompts(tmp_path, seed):
    _case(tmp_path, seed, long=True)
