"""Trace replay: the same requests whole, with the last 32 tokens one by one, in
portions of changing size, and mixed with other requests on a pool so small that
pages are used again; in float32 and in bfloat16; against the plain implementation.
A difference that shows in one way of cutting only is a fault of the cache or of
the batch; the assertion names the first wrong (request, position).

Random N(0, 0.02) weights give nearly uniform attention, under which one wrong key
among hundreds moves the logits by less than bfloat16 rounding does. So every
family also runs on a sharpened copy of each model (q_norm gains tripled: scores
spread over +-10, a few keys dominate each query), and one test breaks a request's
block table on purpose, between two steps, with pages that the request itself
holds, and demands that the comparison then fails."""

import pytest

from helpers import PAGE_SIZES, TOL_BF16, TOL_BF16_SHARP, TOL_F32, random_tokens, vocab_of
from trace_tools import (mixed_trace, plain_rows, portions_trace, round64, run_trace_cli, run_trace_engine,
                         tail_trace, whole_trace, worst_diff)

pytestmark = pytest.mark.gpu

NAMES = ["A", "B", "C", "D", "E"]
LENGTHS = {"A": [70, 45, 100, 33, 128, 64, 17], "B": [71, 40, 9, 130, 200, 65, 2], "C": [150, 64, 33, 97, 255, 12],
           "D": [130, 64, 300, 33, 65, 191, 5], "E": [600, 130, 1100, 33, 520, 64, 5, 200]}
# portions of the mixed family: E also takes portions long enough for the kernels that only many tokens reach
MIXED_SIZES = {"E": (2, 3, 17, 64, 130, 300, 400)}

_plain_cache = {}
_sharp_folders = {}


def tol(name, dtype, sharp=False):
    if dtype == "float32":
        return TOL_F32
    return TOL_BF16_SHARP[name] if sharp else TOL_BF16[name]


def _requests(folder, name):
    v = vocab_of(folder)
    return {f"{name}{i}": random_tokens(n, v, seed=100 * i + n) for i, n in enumerate(LENGTHS[name])}


def _expect(folder, name, key=None):
    key = key or name
    if key not in _plain_cache:
        _plain_cache[key] = plain_rows(folder, _requests(folder, name))
    return _plain_cache[key]


def _family(name, reqs, family, seed=7):
    """(steps, max_tokens) of one way of cutting the requests."""
    longest = round64(max(LENGTHS[name]))
    if family == "whole":
        return whole_trace(reqs), longest
    if family == "tail":
        return tail_trace(reqs, 32), longest
    if family == "portions":
        return portions_trace(reqs), longest
    kw = {"sizes": MIXED_SIZES[name]} if name in MIXED_SIZES else {}
    steps, peak = mixed_trace(reqs, seed=seed, max_live=4, max_tokens=longest + 2 * 128, **kw)
    assert sum(round64(n) for n in LENGTHS[name]) > peak            # pages must be used again
    assert max(len(s["entries"]) for s in steps) >= 3
    return steps, peak


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_replay_family(tiny_folders, name, dtype, family):
    folder = tiny_folders[name]
    steps, max_tokens = _family(name, _requests(folder, name), family)
    got = run_trace_engine(folder, dtype, steps, max_tokens, PAGE_SIZES[name])
    worst, where = worst_diff(got, _expect(folder, name))
    assert worst <= tol(name, dtype), f"first/worst difference {worst} at (request, position) {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tiny_folders, dtype):
    """bin/trace_run as a child process, default page size, mixed trace with page reuse."""
    folder = tiny_folders["B"]
    reqs = _requests(folder, "B")
    steps, peak = mixed_trace(reqs, seed=3, max_live=4, max_tokens=round64(200) + 192)
    got = run_trace_cli(folder, dtype, steps, peak)
    worst, where = worst_diff(got, _expect(folder, "B"))
    assert worst <= tol("B", dtype), f"worst difference {worst} at (request, position) {where}"


def _sharp_folder(tiny_folders, tmp_path_factory, name):
    """The same model with its q_norm gains tripled: attention scores spread over +-10 or more, the
    softmax of each query is dominated by a few keys, and a wrong, missing or stale key changes the
    logits far beyond rounding."""
    import shutil

    from safetensors.torch import load_file, save_file

    if name not in _sharp_folders:
        dst = tmp_path_factory.mktemp("sharp") / name
        shutil.copytree(tiny_folders[name], dst)
        t = load_file(str(dst / "model.safetensors"))
        for k in t:
            if k.endswith("q_norm.weight"):
                t[k] = t[k] * 3.0
        save_file(t, str(dst / "model.safetensors"))
        _sharp_folders[name] = dst
    return _sharp_folders[name]


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_replay_with_peaked_attention(tiny_folders, tmp_path_factory, name, dtype, family):
    folder = _sharp_folder(tiny_folders, tmp_path_factory, name)
    steps, max_tokens = _family(name, _requests(folder, name), family, seed=11)
    got = run_trace_engine(folder, dtype, steps, max_tokens, PAGE_SIZES[name])
    worst, where = worst_diff(got, _expect(folder, name, key="sharp" + name))
    assert worst <= tol(name, dtype, sharp=True), f"worst difference {worst} at (request, position) {where}"


def _swap_two_pages(engine, state):
    """Once, between two steps: in the block table of a request that holds at least two pages, the last
    of them partly filled, the first and the last entry change places. Both pages are the request's own,
    so every access stays inside the pool and inside what the request holds; only the order is wrong: the
    keys of the first positions now stand at the end (where the causal bound hides all but a few of them,
    and where the request's next keys overwrite them), and the rows of the last page that were never
    written count as keys of the first positions."""
    if state.get("done"):
        return
    cache = engine.cache
    for rc in cache.requests.values():
        table = rc.tables[0]
        if len(table) >= 2 and rc.length % cache.page_size and rc.length > cache.page_size:
            table[0], table[-1] = table[-1], table[0]
            cache.host_tables[0][rc.slot, 0], cache.host_tables[0][rc.slot, len(table) - 1] = table[0], table[-1]
            state["done"] = rc.request_id
            return


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("family", ["tail", "portions", "mixed"])
def test_a_wrong_page_in_a_block_table_shows(tiny_folders, tmp_path_factory, name, family):
    """The comparison that the tests above make must fail when the cache is wrong in a way that faults
    nothing: bfloat16, every configuration, every family that has more than one step a request."""
    folder = _sharp_folder(tiny_folders, tmp_path_factory, name)
    steps, max_tokens = _family(name, _requests(folder, name), family, seed=11)
    state = {}
    got = run_trace_engine(folder, "bfloat16", steps, max_tokens, PAGE_SIZES[name],
                           after_step=lambda engine: _swap_two_pages(engine, state))
    assert state.get("done") is not None, "no request ever held two pages with the last partly filled"
    expect = _expect(folder, name, key="sharp" + name)
    worst, where = worst_diff(got, expect)
    assert worst > tol(name, "bfloat16", sharp=True), f"two swapped pages of request {state['done']} changed the logits by only {worst}"
    # and only that request is touched: the others still match
    others = {k: v for k, v in got.items() if k[0] != state["done"]}
    worst_others, where = worst_diff(others, {k: expect[k] for k in others})
    assert worst_others <= tol(name, "bfloat16", sharp=True), f"{worst_others} at {where}"


@pytest.mark.parametrize("name", ["B", "D", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_tokens_in_front_of_prompt_portions(tiny_folders, name, dtype):
    """The steps a scheduler makes while it takes new prompts in: single decode tokens of running requests
    first, then portions of prompts. In such a step the decode kernel serves the entries in front and the
    flash kernel the portions (two launches over one batch); every row against the plain whole sequence."""
    folder = tiny_folders[name]
    reqs = _requests(folder, name)
    long_enough = [r for r in reqs if len(reqs[r]) >= 30]
    decoders, feeders = long_enough[:3], long_enough[3:5]
    ids = decoders + feeders
    assert len(ids) == 5
    steps = []
    pos = {r: 0 for r in ids}

    def entry(r, n):
        e = {"id": r, "tokens": reqs[r][pos[r]:pos[r] + n], "want": list(range(min(n, len(reqs[r]) - pos[r])))}
        pos[r] += len(e["tokens"])
        return e

    def step(entries):
        end = [e["id"] for e in entries if pos[e["id"]] == len(reqs[e["id"]])]
        steps.append({"step": len(steps), "entries": entries, "end": end})

    for r in decoders:                                   # all but the last 12 tokens of the three that will decode
        step([entry(r, len(reqs[r]) - 12)])
    sizes = [17, 2, 300, 64, 5, 130, 3, 40, 9, 31, 2, 200]
    for i in range(12):
        entries = [entry(r, 1) for r in decoders]
        for f in feeders:
            if pos[f] < len(reqs[f]):
                entries.append(entry(f, sizes[(i + len(entries)) % len(sizes)]))
        step(entries)
    for f in feeders:                                    # what is left of the prompts
        while pos[f] < len(reqs[f]):
            step([entry(f, 50)])
    assert sum(1 for s in steps if len(s["entries"]) >= 4 and len(s["entries"][0]["tokens"]) == 1 and len(s["entries"][-1]["tokens"]) > 1) >= 3
    got = run_trace_engine(folder, dtype, steps, sum(round64(len(reqs[r])) for r in ids), PAGE_SIZES[name])
    expect = {k: v for k, v in _expect(folder, name).items() if k[0] in ids}
    worst, where = worst_diff(got, expect)
    assert worst <= tol(name, dtype), f"worst difference {worst} at (request, position) {where}"
