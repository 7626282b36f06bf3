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
