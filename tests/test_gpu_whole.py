"""The engine against the plain implementation: each request alone and whole."""

import pytest

from helpers import PAGE_SIZES, TOL_BF16, TOL_F32, max_abs_diff, random_tokens, vocab_of
from plain.plain_qwen3 import plain_forward, plain_load

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("length", [1, 5, 33, 100])
def test_whole_prompt_matches_plain(tiny_folders, name, dtype, length):
    from quantinfer_b200.engine import Engine, StepEntry

    folder = tiny_folders[name]
    ids = random_tokens(length, vocab_of(folder), seed=length)
    cfg, w = plain_load(folder)
    expect = plain_forward(w, cfg, ids)
    eng = Engine.from_folder(folder, dtype=dtype, page_size=PAGE_SIZES[name], max_tokens=256, max_requests=4)
    eng.open("r")
    got = eng.step([StepEntry("r", ids, list(range(length)))])
    eng.close("r")
    eng.cache.check_invariants()
    assert got.shape == expect.shape
    tol = TOL_F32 if dtype == "float32" else TOL_BF16[name]
    assert max_abs_diff(got, expect) <= tol
