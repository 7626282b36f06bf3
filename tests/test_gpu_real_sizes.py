"""One layer at the true Qwen3-8B layer sizes (hidden 4096, 32 heads of 128 with 8 kv heads,
intermediate 12288, vocabulary 151936, which is no power of two) against the plain
implementation, in float32 and in bfloat16: the sizes at which the tensor-core kernels
(tcgen05 GEMM tiles and split-K plans, TMA-fed attention) actually run in serving."""

import pytest
import torch

from helpers import random_tokens
from plain.plain_qwen3 import plain_forward, plain_load

pytestmark = pytest.mark.gpu

CONFIG_8B_ONE_LAYER = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
    intermediate_size=12288, num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
)


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    from quantinfer_b200.config import config_from_dict
    from quantinfer_b200.weights import write_model_folder

    return write_model_folder(tmp_path_factory.mktemp("qwen3_8b_1layer"), config_from_dict(CONFIG_8B_ONE_LAYER), seed=8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_layer_at_8b_sizes(folder, dtype):
    from quantinfer_b200.engine import Engine, StepEntry

    ids = random_tokens(150, 151936, seed=3)
    cfg, w = plain_load(folder)
    want = [0, 1, 63, 64, 127, 128, 140]
    expect = plain_forward(w, cfg, ids)[want + [141, 142, 143, 144, 145, 146, 147, 148, 149]]
    del w
    eng = Engine.from_folder(folder, dtype=dtype, page_size=64, max_tokens=512, max_requests=2, max_seq_len=4096)
    eng.open("r")
    rows = [eng.step([StepEntry("r", ids[:130], [0, 1, 63, 64, 127, 128])]).cpu(),
            eng.step([StepEntry("r", ids[130:141], [10])]).cpu()]
    for t in range(141, 150):                       # decode steps: split-K plans and the split-key attention
        rows.append(eng.step([StepEntry("r", [ids[t]], [0])]).cpu())
    got = torch.cat(rows)
    # logits are of order 1 here; the float32 bound is the reference's own gate against an independent
    # float32 implementation (crates/quantinfer-runtime/tests/qwen3_conformance.rs:64-66), tightened tenfold
    tol = 1e-4 if dtype == "float32" else 5e-2
    diff = (got - expect).abs().max(dim=1).values
    assert float(diff.max()) <= tol, (diff.tolist(), float(expect.abs().max()))
