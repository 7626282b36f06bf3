"""The plain implementation itself (no GPU): the reference's two literal vectors, the
parts against direct formulas in float64, the sampler."""

import math

import torch

from helpers import make_folder, random_tokens
from plain.plain_qwen3 import (plain_apply_rope, plain_argmax, plain_forward, plain_generate,
                               plain_gqa_attention, plain_linear, plain_load, plain_philox4x32_10,
                               plain_rms_norm, plain_rope_tables, plain_sample, plain_silu_mul, plain_uniform)


def test_reference_rope_vector():
    # backends/cpu/src/tests.rs:136-143: [1,2,3,4] with cos [0,1], sin [1,0] -> [-3,2,1,4]
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])
    y = plain_apply_rope(x, torch.tensor([[0.0, 1.0]]), torch.tensor([[1.0, 0.0]]))
    assert y.flatten().tolist() == [-3.0, 2.0, 1.0, 4.0]


def test_reference_matmul_vector():
    # backends/cpu/src/tests.rs:9-15: [[1,2,3],[4,5,6]] . [[1,2],[3,4],[5,6]] = [22,28,49,64]
    x = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    w_in_out = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    assert plain_linear(x, w_in_out.t().contiguous()).flatten().tolist() == [22.0, 28.0, 49.0, 64.0]


def test_rms_norm_and_silu():
    x = torch.tensor([[3.0, 4.0]])
    y = plain_rms_norm(x, torch.tensor([2.0, 0.5]), 1e-6)
    r = 1.0 / math.sqrt(12.5 + 1e-6)
    assert torch.allclose(y, torch.tensor([[3 * r * 2, 4 * r * 0.5]]), atol=1e-6)
    assert torch.allclose(plain_silu_mul(torch.tensor([1.0, -2.0]), torch.tensor([3.0, 0.5])),
                          torch.tensor([3.0 / (1 + math.exp(-1.0)), -1.0 / (1 + math.exp(2.0))]), atol=1e-6)


def test_rope_table_angles():
    cos, sin = plain_rope_tables(10000.0, 8, [0, 3], dtype=torch.float64)
    assert torch.allclose(cos[0], torch.ones(4, dtype=torch.float64)) and torch.allclose(sin[0], torch.zeros(4, dtype=torch.float64))
    for p in range(4):
        assert abs(float(cos[1, p]) - math.cos(3 * 10000.0 ** (-2 * p / 8))) < 1e-12


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(5, 4, 8), torch.randn(5, 2, 8), torch.randn(5, 2, 8)
    out = plain_gqa_attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # heads 0,1 -> kv 0; 2,3 -> kv 1
    s = (k[:3, 1] @ q[2, 2]) / math.sqrt(8)
    assert torch.allclose(out[2, 2], (torch.softmax(s, 0)[:, None] * v[:3, 1]).sum(0), atol=1e-6)
    w = plain_gqa_attention(q, k, v, window=2)
    s = (k[3:5, 0] @ q[4, 1]) / math.sqrt(8)
    assert torch.allclose(w[4, 1], (torch.softmax(s, 0)[:, None] * v[3:5, 0]).sum(0), atol=1e-6)


def test_forward_float32_agrees_with_float64(tmp_path):
    folder = make_folder(tmp_path / "B", "B")
    ids = random_tokens(40, 384, 5)
    cfg, w32 = plain_load(folder)
    _, w64 = plain_load(folder, torch.float64)
    a, b = plain_forward(w32, cfg, ids), plain_forward(w64, cfg, ids)
    assert a.shape == (40, 384) and float((a.double() - b).abs().max()) < 2e-5


def test_philox_known_answer_and_uniform_range():
    assert plain_philox4x32_10((0, 0, 0, 0), (0, 0)) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    us = [plain_uniform(7, c) for c in range(200)]
    assert all(0.0 <= u < 1.0 for u in us) and 0.35 < sum(us) / len(us) < 0.65
    assert plain_uniform(7, 3) != plain_uniform(8, 3)


def test_sampler_rules():
    assert plain_argmax([1.0, 5.0, 5.0, 2.0]) == 1                   # first maximum
    logits = torch.tensor([0.0, 3.0, 1.0, 3.0, -2.0])
    assert plain_sample(logits, 0.0, top_k=2, top_p=0.5) == 1         # temperature 0 is greedy
    assert all(plain_sample(logits, 1.0, top_k=1, seed=s) == 1 for s in range(20))   # ties keep the lowest index
    assert {plain_sample(logits, 1.0, top_k=2, seed=s) for s in range(40)} == {1, 3}
    assert {plain_sample(logits, 1.0, top_p=0.3, seed=s) for s in range(20)} == {1}
    counts = [0] * 5
    for s in range(2000):
        counts[plain_sample(logits, 1.0, seed=s)] += 1
    p = torch.softmax(logits, 0)
    assert all(abs(counts[i] / 2000 - float(p[i])) < 0.04 for i in range(5))


def test_generate_stops_on_eos(tmp_path):
    folder = make_folder(tmp_path / "A", "A")
    cfg, w = plain_load(folder)
    out = plain_generate(w, cfg, [3, 4, 5], 5)
    assert len(out) == 5
    eos = out[-1]
    assert plain_generate(w, cfg, [3, 4, 5], 5, eos=eos) == out[:out.index(eos) + 1]
