"""Trace replay: the same requests whole, with the last 32 tokens one by one, in
portions of changing size, and mixed with other requests on a pool so small that
pages are used again; in float32 and in bfloat16; against the plain implementation.
A difference that shows in one way of cutting only is a fault of the cache or of
the batch; the assertion names the first wrong (request, position)."""

import pytest

from helpers import PAGE_SIZES, random_tokens, vocab_of
from trace_tools import (mixed_trace, plain_rows, portions_trace, round64, run_trace_cli, run_trace_engine,
                         tail_trace, whole_trace, worst_diff)

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 3e-2}
LENGTHS = {"A": [70, 45, 100, 33, 128, 64, 17], "B": [71, 40, 9, 130, 200, 65, 2], "C": [150, 64, 33, 97, 255, 12],
           "D": [130, 64, 300, 33, 65, 191, 5]}

_plain_cache = {}


def _requests(folder, name):
    v = vocab_of(folder)
    return {f"{name}{i}": random_tokens(n, v, seed=100 * i + n) for i, n in enumerate(LENGTHS[name])}


def _expect(folder, name):
    if name not in _plain_cache:
        _plain_cache[name] = plain_rows(folder, _requests(folder, name))
    return _plain_cache[name]


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_replay_family(tiny_folders, name, dtype, family):
    folder = tiny_folders[name]
    reqs = _requests(folder, name)
    if family == "whole":
        steps, max_tokens = whole_trace(reqs), round64(max(LENGTHS[name]))
    elif family == "tail":
        steps, max_tokens = tail_trace(reqs, 32), round64(max(LENGTHS[name]))
    elif family == "portions":
        steps, max_tokens = portions_trace(reqs), round64(max(LENGTHS[name]))
    else:
        budget = round64(max(LENGTHS[name])) + 2 * 128
        steps, peak = mixed_trace(reqs, seed=7, max_live=4, max_tokens=budget)
        max_tokens = peak
        assert sum(round64(n) for n in LENGTHS[name]) > max_tokens  # pages must be used again
        assert max(len(s["entries"]) for s in steps) >= 3
    got = run_trace_engine(folder, dtype, steps, max_tokens, PAGE_SIZES[name])
    worst, where = worst_diff(got, _expect(folder, name))
    assert worst <= TOL[dtype], f"first/worst difference {worst} at (request, position) {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tiny_folders, dtype):
    """bin/trace_run as a child process, default page size, mixed trace with page reuse."""
    folder = tiny_folders["B"]
    reqs = _requests(folder, "B")
    steps, peak = mixed_trace(reqs, seed=3, max_live=4, max_tokens=round64(200) + 192)
    got = run_trace_cli(folder, dtype, steps, peak)
    worst, where = worst_diff(got, _expect(folder, "B"))
    assert worst <= TOL[dtype], f"worst difference {worst} at (request, position) {where}"


def _sharp_folder(tiny_folders, tmp_path_factory, name):
    """The same model with its q_norm gains tripled: attention scores spread over +-10 or more, the
    softmax of each query is dominated by a few keys, and one wrong, missing or stale key changes the
    logits far beyond rounding. Random N(0, 0.02) weights alone give nearly uniform attention, which
    would hide such a fault from the bfloat16 comparison."""
    import shutil

    from safetensors.torch import load_file, save_file

    dst = tmp_path_factory.mktemp("sharp") / name
    shutil.copytree(tiny_folders[name], dst)
    t = load_file(str(dst / "model.safetensors"))
    for k in t:
        if k.endswith("q_norm.weight"):
            t[k] = t[k] * 3.0
    save_file(t, str(dst / "model.safetensors"))
    return dst


@pytest.mark.parametrize("name", ["A", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_with_peaked_attention(tiny_folders, tmp_path_factory, name, dtype):
    folder = _sharp_folder(tiny_folders, tmp_path_factory, name)
    reqs = _requests(folder, name)
    expect = plain_rows(folder, reqs)
    budget = round64(max(LENGTHS[name])) + 2 * 128
    steps, peak = mixed_trace(reqs, seed=11, max_live=4, max_tokens=budget)
    got = run_trace_engine(folder, dtype, steps, peak, PAGE_SIZES[name])
    worst, where = worst_diff(got, expect)
    assert worst <= TOL[dtype], f"worst difference {worst} at (request, position) {where}"
    # the point of the sharper model: one wrong key must show. Changing a single early token changes
    # the last position's logits by far more than the bfloat16 tolerance.
    from plain.plain_qwen3 import plain_forward, plain_load

    cfg, w = plain_load(folder)
    rid = max(reqs, key=lambda r: len(reqs[r]))
    ids = list(reqs[rid])
    base = plain_forward(w, cfg, ids)[-1]
    sensitivity = 0.0
    for pos in (1, len(ids) // 4, len(ids) // 2, 3 * len(ids) // 4, len(ids) - 2):
        other = list(ids)
        other[pos] = (other[pos] + 1) % vocab_of(folder)
        sensitivity = max(sensitivity, float((base - plain_forward(w, cfg, other)[-1]).abs().max()))
    assert sensitivity > 3 * TOL["bfloat16"], sensitivity
