"""Builds traces (lists of steps in trace_run's JSON form) and replays them,
either through the engine in this process or through bin/trace_run."""

from __future__ import annotations

import json
import random
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


def round64(n: int) -> int:
    return (n + 63) // 64 * 64


def whole_trace(requests: dict) -> list:
    """Each request alone and whole, every place wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def tail_trace(requests: dict, tail: int = 32) -> list:
    """Most of each request in one step, the last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(len(toks) - tail, 1)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for p in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions_trace(requests: dict, seed: int = 0, sizes=(7, 2, 16, 3, 2, 31, 5, 2, 64, 9)) -> list:
    """Portions of changing size, down to two tokens."""
    steps = []
    for k, (rid, toks) in enumerate(requests.items()):
        a, i = 0, k
        while a < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - a)
            i += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[a:a + n], "want": list(range(n))}],
                          "end": [rid] if a + n == len(toks) else []})
            a += n
    return steps


def mixed_trace(requests: dict, seed: int = 0, max_live: int = 4, decode_tail: int = 6, max_tokens: int | None = None,
                sizes=(2, 3, 5, 8, 13, 16, 17, 30)):
    """Up to `max_live` requests at a time, portions of some beside single tokens
    of others; a request may sit a step out. New requests start as earlier ones
    end, so that their pages are used again. Returns (steps, peak rounded tokens)."""
    rng = random.Random(seed)
    order = list(requests)
    nxt, live, pos = 0, [], {}
    steps, peak = [], 0
    while nxt < len(order) or live:
        while nxt < len(order) and len(live) < max_live:
            cand = order[nxt]
            held = sum(round64(len(requests[r])) for r in live)
            if max_tokens is not None and held + round64(len(requests[cand])) > max_tokens:
                break
            live.append(cand)
            pos[cand] = 0
            nxt += 1
        entries, end = [], []
        for rid in list(live):
            toks = requests[rid]
            left = len(toks) - pos[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            if left <= decode_tail:
                n = 1
            else:
                n = min(rng.choice(list(sizes)), left - decode_tail)
            entries.append({"id": rid, "tokens": toks[pos[rid]:pos[rid] + n], "want": list(range(n))})
            pos[rid] += n
            if pos[rid] == len(toks):
                end.append(rid)
        if not entries:
            continue
        peak = max(peak, sum(round64(len(requests[r])) for r in live))
        steps.append({"step": len(steps), "entries": entries, "end": end})
        for rid in end:
            live.remove(rid)
    return steps, peak


def collect(steps: list, outputs: dict) -> dict:
    """{(request, position): logits row} from per-step arrays [wanted, vocab]."""
    pos, rows = {}, {}
    for st in steps:
        arr = outputs.get(st["step"])
        i = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                rows[(e["id"], base + w)] = arr[i]
                i += 1
            pos[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            pos.pop(rid, None)
    return rows


def run_trace_engine(folder, dtype: str, steps: list, max_tokens: int, page_size: int, after_step=None) -> dict:
    """Replays `steps` through an engine of this process. `after_step(engine)` runs between steps
    (a test uses it to break the cache on purpose)."""
    from quantinfer_b200.engine import Engine, StepEntry

    eng = Engine.from_folder(folder, dtype=dtype, page_size=page_size, max_tokens=max_tokens, max_requests=8, check_finite=True)
    live, outputs = set(), {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            if e["id"] not in live:
                eng.open(e["id"])
                live.add(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = eng.step(entries)
        if logits.shape[0]:
            outputs[st["step"]] = logits.cpu().numpy()
        for rid in st["end"]:
            eng.close(rid)
            live.discard(rid)
        eng.cache.check_invariants()
        if after_step is not None:
            after_step(eng)
    assert not eng.cache.requests
    return collect(steps, outputs)


def run_trace_cli(folder, dtype: str, steps: list, max_tokens: int, page_size=None, env=None) -> dict:
    """Through bin/trace_run as a child process, the way a user runs it."""
    vocab = json.loads((Path(folder) / "config.json").read_text())["vocab_size"]
    with tempfile.TemporaryDirectory() as out:
        cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
               "--out", out, "--max-tokens", str(max_tokens)]
        if page_size:
            cmd += ["--page-size", str(page_size)]
        text = "".join(json.dumps(s) + "\n" for s in steps)
        r = subprocess.run(cmd, input=text, capture_output=True, text=True, env=env, timeout=600)
        assert r.returncode == 0, r.stderr[-4000:]
        done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
        assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps]
        outputs = {}
        for s in steps:
            f = Path(out) / f"{s['step']}.f32"
            wanted = sum(len(e["want"]) for e in s["entries"])
            if wanted:
                outputs[s["step"]] = np.fromfile(f, dtype="<f4").reshape(wanted, vocab)
            else:
                assert not f.exists()
    return collect(steps, outputs)


def plain_rows(folder, requests: dict) -> dict:
    from plain.plain_qwen3 import plain_forward, plain_load

    cfg, w = plain_load(folder)
    rows = {}
    for rid, toks in requests.items():
        logits = plain_forward(w, cfg, toks).numpy()
        for p in range(len(toks)):
            rows[(rid, p)] = logits[p]
    return rows


def worst_diff(got: dict, expect: dict):
    """(max abs difference, where) over all (request, position) rows; both must have the same keys."""
    assert set(got) == set(expect), (sorted(set(expect) - set(got))[:5], sorted(set(got) - set(expect))[:5])
    worst, where = 0.0, None
    for key in sorted(expect, key=str):
        d = float(np.abs(got[key].astype(np.float64) - expect[key].astype(np.float64)).max())
        if d > worst or where is None:
            worst, where = max(worst, d), key if d >= worst else where
    return worst, where
