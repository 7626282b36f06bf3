"""Generation through the entry points: greedy and sampled tokens against the plain
implementation, the command line's output, long decoding, the first tokens of a
sequence, batches through the scheduler, and decoding that stays on the device."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from helpers import PAGE_SIZES, TOL_BF16, TOL_F32, random_tokens, vocab_of
from plain.plain_qwen3 import plain_forward, plain_generate, plain_load

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(tiny_folders, name, dtype):
    import quantinfer_b200

    folder = tiny_folders[name]
    cfg, w = plain_load(folder)
    with quantinfer_b200.Model(folder, dtype=dtype, page_size=PAGE_SIZES[name], cache_tokens=1024, max_requests=4) as m:
        for n in (5, 17, 33):
            prompt = random_tokens(n, vocab_of(folder), seed=n)
            expect = plain_generate(w, cfg, prompt, 8)
            got = m.generate_tokens(prompt, max_new_tokens=8, eos_token_id=None)
            if dtype == "float32":
                assert got == expect
            else:
                # bfloat16 may pick another token where two logits are nearly tied; up to
                # the first such place the tokens agree, and that place must be a tie within
                # the error that bfloat16 logits have on this configuration (each of the two may be off by it)
                i = next((j for j in range(8) if got[j] != expect[j]), 8)
                if i < 8:
                    logits = plain_forward(w, cfg, prompt + expect[:i])[-1]
                    assert abs(float(logits[got[i]] - logits[expect[i]])) < 2 * TOL_BF16[name]
    with pytest.raises(quantinfer_b200.QuantInferError, match="closed"):
        m.generate_tokens([1], max_new_tokens=1)


def test_sampled_generation_matches_plain_under_a_seed(tiny_folders):
    import quantinfer_b200

    folder = tiny_folders["A"]
    cfg, w = plain_load(folder)
    prompt = random_tokens(9, 256, seed=4)
    with quantinfer_b200.Model(folder, dtype="float32", page_size=16, cache_tokens=512, max_requests=4) as m:
        for kw in (dict(temperature=0.8, seed=11), dict(temperature=1.2, top_k=20, seed=5), dict(temperature=0.7, top_p=0.8, seed=2**40 + 3)):
            expect = plain_generate(w, cfg, prompt, 10, **kw)
            assert m.generate_tokens(prompt, max_new_tokens=10, eos_token_id=None, **kw) == expect
        # the same request inside a batch draws the same tokens: the stream belongs to the request
        alone = m.generate_tokens(prompt, max_new_tokens=10, eos_token_id=None, temperature=0.8, seed=11)
        batch = m.generate_batch([prompt, random_tokens(30, 256, 1), random_tokens(3, 256, 2)], max_new_tokens=10,
                                 eos_token_id=None, temperature=0.8, seed=11)
        assert batch[0] == alone and len(batch[1]) == 10
        # EOS: emitted, then the request stops
        eos = alone[3]
        out = m.generate_tokens(prompt, max_new_tokens=10, eos_token_id=eos, temperature=0.8, seed=11)
        assert out == alone[:alone.index(eos) + 1]
        with pytest.raises(ValueError):
            m.generate_tokens(prompt, max_new_tokens=0)
        with pytest.raises(ValueError):
            m.generate_tokens([256], max_new_tokens=1)
        with pytest.raises(ValueError):
            m.generate_tokens(prompt, max_new_tokens=200)          # exceeds max_position_embeddings
        with pytest.raises(quantinfer_b200.QuantInferError):
            m.tokenize("text")


def test_batch_through_the_scheduler_equals_each_alone(tiny_folders):
    """Config B's workload: four requests of 1/9/40/71 tokens, prompt portions of 16 beside decode tokens."""
    import quantinfer_b200

    folder = tiny_folders["B"]
    cfg, w = plain_load(folder)
    prompts = [random_tokens(n, 384, seed=n) for n in (1, 9, 40, 71)]
    with quantinfer_b200.Model(folder, dtype="float32", page_size=8, cache_tokens=512, max_requests=4,
                               max_batch_tokens=24, chunk_size=16) as m:
        got = m.generate_batch(prompts, max_new_tokens=12, eos_token_id=None)
    for p, g in zip(prompts, got):
        assert g == plain_generate(w, cfg, p, 12)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tiny_folders, dtype):
    """A 3-token prompt, then 250 tokens decoded one by one (pages fill and new ones are taken many
    times, graphs are replayed across context buckets); every position's logits against the plain
    whole sequence, the very first positions included."""
    from quantinfer_b200.engine import Engine, StepEntry

    folder = tiny_folders["D"]
    ids = random_tokens(253, 300, seed=9)
    cfg, w = plain_load(folder)
    expect = plain_forward(w, cfg, ids)
    eng = Engine.from_folder(folder, dtype=dtype, page_size=16, max_tokens=320, max_requests=2)
    eng.open("r")
    rows = [eng.step([StepEntry("r", ids[:1], [0])]).cpu(), eng.step([StepEntry("r", ids[1:3], [0, 1])]).cpu()]
    for t in range(3, len(ids)):
        rows.append(eng.step([StepEntry("r", [ids[t]], [0])]).cpu())
    got = torch.cat(rows)
    diff = (got - expect).abs().max(dim=1).values
    tol = TOL_F32 if dtype == "float32" else TOL_BF16["D"]
    assert float(diff.max()) <= tol, f"first position above the tolerance: {int((diff > tol).nonzero()[0])}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_across_context_buckets(tiny_folders, dtype):
    """Decode steps are replayed from one CUDA graph per batch size and per bucket of 512 positions of the
    longest context. On the serving geometry (heads of 128, pages of 64): one request decoded from
    position 500 to 530 and, after another prompt portion, from 1,020 to 1,030, so that its steps move
    from one bucket's graph to the next one's twice; then three requests whose contexts lie in three
    different buckets decoded together. Every step's logits against the plain whole sequence."""
    from quantinfer_b200.engine import Engine, StepEntry

    folder = tiny_folders["E"]
    cfg, w = plain_load(folder)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16["E"]
    eng = Engine.from_folder(folder, dtype=dtype, page_size=64, max_tokens=4096, max_requests=4)
    assert eng.use_graphs
    ids = random_tokens(1030, 1000, seed=21)
    expect = plain_forward(w, cfg, ids)
    eng.open("r")
    rows, where = [eng.step([StepEntry("r", ids[:500], [499])]).cpu()], [499]
    for t in range(500, 530):
        rows.append(eng.step([StepEntry("r", [ids[t]], [0])]).cpu())
        where.append(t)
    buckets = sorted(bound for (b, bound) in eng._graphs if b == 1)
    assert buckets == [512, 1024], buckets                      # positions 501..512 and 513..530
    rows.append(eng.step([StepEntry("r", ids[530:1020], [0, 489])]).cpu())
    where += [530, 1019]
    for t in range(1020, 1030):
        rows.append(eng.step([StepEntry("r", [ids[t]], [0])]).cpu())
        where.append(t)
    assert sorted(bound for (b, bound) in eng._graphs if b == 1) == [512, 1024, 1536]
    eng.close("r")
    diff = (torch.cat(rows) - expect[where]).abs().max(dim=1).values
    assert float(diff.max()) <= tol, f"first position above the tolerance: {where[int((diff > tol).nonzero()[0])]}"
    # three requests in three buckets, one batch
    lens = {"x": 100, "y": 600, "z": 1100}
    seqs = {k: random_tokens(n + 12, 1000, seed=n) for k, n in lens.items()}
    want = {k: plain_forward(w, cfg, v) for k, v in seqs.items()}
    for k, n in lens.items():
        eng.open(k)
        eng.step([StepEntry(k, seqs[k][:n], [])])
    for j in range(12):
        out = eng.step([StepEntry(k, [seqs[k][lens[k] + j]], [0]) for k in lens]).cpu()
        for i, k in enumerate(lens):
            d = float((out[i] - want[k][lens[k] + j]).abs().max())
            assert d <= tol, f"request {k} (context {lens[k] + j + 1}) in a batch of three: {d}"
    assert any(b == 3 for (b, _) in eng._graphs)
    for k in lens:
        eng.close(k)
    eng.cache.check_invariants()


@pytest.mark.parametrize("name, lengths", [("D", (20, 70, 5)), ("E", (500, 70, 600))])
def test_decode_on_device_equals_step_by_step(tiny_folders, name, lengths):
    """Decoding that stays on the device (sampling and feeding the token back there) against one step at
    a time from the host, token for token. Both ways replay the graph of the bucket that the longest
    context lies in (on the serving geometry 601 to 640 positions: the bucket up to 1,024), so the key
    ranges are cut alike and the logits are the same bits."""
    from quantinfer_b200.engine import Engine, StepEntry
    from quantinfer_b200.sampling import GenerationConfig, Sampler

    folder = tiny_folders[name]
    prompts = [random_tokens(n, vocab_of(folder), seed=n) for n in lengths]
    cfgs = [GenerationConfig(max_new_tokens=64, temperature=t, seed=s) for t, s in ((0.0, 0), (0.9, 5), (0.6, 9))]

    def run(on_device):
        eng = Engine.from_folder(folder, dtype="bfloat16", page_size=PAGE_SIZES[name], max_tokens=4096, max_requests=4)
        sampler = Sampler(eng.device, eng.runtime.status)
        first = []
        for i, p in enumerate(prompts):
            eng.open(i)
            logits = eng.step([StepEntry(i, p, [len(p) - 1])])
            first.append(sampler.sample(logits, [(cfgs[i], 0)])[0])
        rows = [(c, 1) for c in cfgs]
        if on_device:
            return first, eng.decode_on_device([0, 1, 2], first, 40, rows, sampler).cpu().tolist()
        hist, cur = [], first
        for n in range(40):
            logits = eng.step([StepEntry(i, [cur[i]], [0]) for i in range(3)])
            cur = sampler.sample(logits, [(c, 1 + n) for c in cfgs])
            hist.append(cur)
        return first, hist

    assert run(True) == run(False)


@pytest.mark.parametrize("name, dtype", [("D", "bfloat16"), ("B", "float32")])
def test_steps_that_run_ahead_give_the_same_tokens(tiny_folders, name, dtype):
    """Decode steps launched before the host has read the tokens of the step before: the same tokens
    as with the host in every step, greedy and sampled, with an EOS that ends one request early (the
    step that ran ahead with it is dropped) and with more prompts than sequence slots (requests are
    admitted while others decode)."""
    import quantinfer_b200

    folder = tiny_folders[name]
    v = vocab_of(folder)
    prompts = [random_tokens(n, v, seed=n) for n in (3, 33, 18, 50, 7, 21)]
    outs = {}
    for ahead in (False, True):
        with quantinfer_b200.Model(folder, dtype=dtype, page_size=16, cache_tokens=1024, max_requests=4,
                                   max_batch_tokens=64, run_ahead=ahead) as m:
            res = [m.generate_batch(prompts, max_new_tokens=60, eos_token_id=None)]
            ahead_steps = m.last_scheduler.steps_ahead
            res.append(m.generate_batch(prompts, max_new_tokens=60, eos_token_id=None, temperature=0.8, top_k=40, top_p=0.95, seed=11))
            eos = res[1][1][9]          # the tenth sampled token of the second prompt becomes the EOS
            res.append(m.generate_batch(prompts, max_new_tokens=60, eos_token_id=eos, temperature=0.8, top_k=40, top_p=0.95, seed=11))
            assert len(res[2][1]) <= 10 and res[2][1][-1] == eos
            assert (ahead_steps > 30) if ahead else (ahead_steps == 0)
            m.engine.cache.check_invariants()
            assert not m.engine.cache.requests
        outs[ahead] = res
    # with the EOS the two runs hold different requests in some steps (the one that ended stays for the
    # step that ran ahead), so in bfloat16 their logits may differ by rounding and a draw may fall
    # elsewhere; in 32-bit every row is computed alone and the tokens are the same
    same = 3 if dtype == "float32" else 2
    assert outs[True][:same] == outs[False][:same]
    for out in outs[True][2]:
        assert len(out) == 60 or out[-1] == eos
    cfg, w = plain_load(folder)
    if dtype == "float32":
        assert outs[True][0][2] == plain_generate(w, cfg, prompts[2], 60)


def test_command_line(tiny_folders, tmp_path):
    folder = tiny_folders["A"]
    cfg, w = plain_load(folder)
    prompt = [5, 17, 3, 200, 9]
    expect = plain_generate(w, cfg, prompt, 8)
    report = tmp_path / "report.json"
    cmd = [sys.executable, str(ROOT / "bin" / "quantinfer"), "generate", "--input", str(folder), "--tokens", "5, 17,3,200 ,9",
           "--max-new-tokens", "8", "--dtype", "float32", "--page-size", "16", "--profile", "--profile-report", str(report)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    lines = dict(l.split("=", 1) for l in r.stdout.strip().splitlines())
    assert lines["prompt_tokens"] == str(prompt) and lines["generated_tokens"] == str(expect)
    assert lines["decode_tokens"] == "8" and float(lines["prefill_ms"]) > 0 and float(lines["decode_tokens_per_sec"]) > 0
    for key in ("model_load_ms", "ttft_ms", "profile_decode_ms", "kv_cache_bytes", "kv_cache_capacity_bytes", "max_sequence_length", "peak_rss_kib"):
        assert key in lines
    # the cache holds prompt + generated - 1 positions: 2 layers x 12 positions x 2 kv heads x 16 x (k, v) x 4 bytes
    assert int(lines["kv_cache_bytes"]) == 2 * 12 * 2 * 16 * 2 * 4
    assert json.loads(report.read_text())["decode_tokens"] == 8
    r2 = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r2.returncode == 2 and "already exists" in r2.stderr
    for bad, msg in ((["--prompt", "hi"], "exactly one"), (["--bogus"], "unknown option"), (["--max-new-tokens", "200"], "exceed"),
                     (["--eos-token-id", "999"], "outside the model vocabulary")):
        args = [a for a in cmd[:-3]] + bad if bad[0] != "--max-new-tokens" else [a for a in cmd[:-3] if a not in ("--max-new-tokens", "8")] + bad
        r3 = subprocess.run(args, capture_output=True, text=True, timeout=300)
        assert r3.returncode == 2 and msg in r3.stderr, (bad, r3.stderr)


def _cli(*args):
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "quantinfer"), "generate", *map(str, args)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    pairs = [l.split("=", 1) for l in r.stdout.strip().splitlines()]
    return ([json.loads(v) for k, v in pairs if k == "prompt_tokens"],
            [json.loads(v) for k, v in pairs if k == "generated_tokens"], dict(pairs))


def test_command_line_runs_a_batch_through_the_scheduler(tiny_folders):
    """Three prompts in one call, prompt portions of 16 under a budget of 24 tokens a step: each request's
    tokens are the plain implementation's, and the Python entry point gives the command line's tokens,
    greedy and under a seed."""
    import quantinfer_b200

    folder = tiny_folders["B"]
    cfg, w = plain_load(folder)
    prompts = [random_tokens(n, 384, seed=n) for n in (9, 40, 71)]
    text = ";".join(",".join(map(str, p)) for p in prompts)
    common = ["--input", folder, "--tokens", text, "--max-new-tokens", 12, "--dtype", "float32", "--page-size", 8,
              "--chunk-size", 16, "--max-batch-tokens", 24, "--profile"]
    got_prompts, got, lines = _cli(*common)
    assert got_prompts == prompts
    assert got == [plain_generate(w, cfg, p, 12) for p in prompts]
    assert lines["decode_tokens"] == "36"
    # 71 prompt tokens cannot pass in fewer than five steps of at most 16; the decode steps come on top
    assert int(lines["scheduler_steps"]) >= 5 + 11
    # the cache held prompt + generated - 1 positions of every request: 3 layers x 1 kv head x 32 x (k, v) x 4 bytes
    assert int(lines["kv_cache_bytes"]) == sum(len(p) + 11 for p in prompts) * 3 * 1 * 32 * 2 * 4
    sampled = ["--temperature", 0.8, "--top-k", 50, "--seed", 21]
    _, got_sampled, _ = _cli(*common, *sampled)
    _, again, _ = _cli(*common, *sampled, "--no-run-ahead")
    assert got_sampled == again                       # two runs under one seed agree
    with quantinfer_b200.Model(folder, dtype="float32", page_size=8, cache_tokens=512, max_requests=4,
                               max_batch_tokens=24, chunk_size=16) as m:
        assert m.generate_batch(prompts, max_new_tokens=12, eos_token_id=None) == got
        assert m.generate_batch(prompts, max_new_tokens=12, eos_token_id=None, temperature=0.8, top_k=50, seed=21) == got_sampled
        assert m.generate_tokens(prompts[1], max_new_tokens=12, eos_token_id=None, temperature=0.8, top_k=50, seed=22) == got_sampled[1]
    assert got_sampled[1] == plain_generate(w, cfg, prompts[1], 12, temperature=0.8, top_k=50, seed=22)


def test_command_line_with_random_weights_and_a_page_pool_that_is_too_small(tmp_path):
    from helpers import TINY_CONFIGS

    (tmp_path / "config.json").write_text(json.dumps(TINY_CONFIGS["D"]))
    args = ["--input", tmp_path / "config.json", "--random-weights", "--weights-seed", 5, "--tokens", "1,2,3;9,8,7,6",
            "--max-new-tokens", 20, "--page-size", 16]
    _, a, _ = _cli(*args)
    _, b, _ = _cli(*args[:1], tmp_path, *args[2:], "--num-pages", 2)     # one request at a time fits
    assert a == b and [len(t) for t in a] == [20, 20]
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "quantinfer"), "generate", *map(str, args), "--num-pages", "1"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode != 0 and "never fit the page pool" in r.stderr


def test_random_weights_command_and_engine_errors(tmp_path):
    from quantinfer_b200.engine import Engine, StepEntry
    from quantinfer_b200.errors import OutOfPages, QuantInferError
    from helpers import TINY_CONFIGS

    (tmp_path / "cfg.json").write_text(json.dumps(TINY_CONFIGS["C"]))
    out = tmp_path / "model"
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "quantinfer"), "random-weights", "--config", str(tmp_path / "cfg.json"),
                        "--output", str(out), "--seed", "2"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and (out / "model.safetensors").is_file() and (out / "config.json").is_file()
    eng = Engine.from_folder(out, dtype="float32", page_size=32, max_tokens=128, max_requests=2)
    eng.open("a")
    with pytest.raises(QuantInferError, match="outside the vocabulary"):
        eng.step([StepEntry("a", [517], [0])])
    with pytest.raises(QuantInferError, match="at least one token"):
        eng.step([StepEntry("a", [], [])])
    with pytest.raises(QuantInferError, match="not open"):
        eng.step([StepEntry("zzz", [1], [0])])
    with pytest.raises(QuantInferError, match="wanted place"):
        eng.step([StepEntry("a", [1, 2], [2])])
    eng.step([StepEntry("a", list(range(100)), [])])
    eng.open("b")
    free = eng.cache.free_pages()
    with pytest.raises(OutOfPages):                      # 4 pages in all, 4 taken by a
        eng.step([StepEntry("a", [1], [0]), StepEntry("b", list(range(40)), [])])
    assert eng.cache.free_pages() == free and eng.length("a") == 100 and eng.length("b") == 0   # nothing advanced
    eng.cache.check_invariants()


@pytest.mark.parametrize("run_ahead", [False, True])
def test_pages_taken_by_someone_else_preempt_the_newest_request(tiny_folders, run_ahead):
    """The scheduler reserves a request's pages at admission, so it runs out only when someone outside it
    takes pages from the same pool. Here a callback does, in the middle of a run: the step finds no page,
    the newest request gives everything back and is taken up again later with what it had emitted, and
    every request's tokens are still those of the plain implementation, drawn tokens included (the
    request's draw counter is written into its slot's record again when it is admitted again)."""
    import quantinfer_b200
    from quantinfer_b200.engine import StepEntry
    from quantinfer_b200.engine.scheduler import TokenEvent

    folder = tiny_folders["B"]
    cfg, w = plain_load(folder)
    prompts = [random_tokens(n, 384, seed=n) for n in (30, 41, 22)]
    with quantinfer_b200.Model(folder, dtype="float32", page_size=8, num_pages=30, max_requests=4, max_batch_tokens=64,
                               run_ahead=run_ahead) as m:
        eng = m.engine
        seen = {"events": 0, "held": False}

        def meddle(ev):
            if not isinstance(ev, TokenEvent):
                return
            seen["events"] += 1
            if seen["events"] == 6 and not seen["held"]:
                # an outsider takes every page that is free now
                eng.open("outsider")
                free = eng.cache.free_pages()
                eng.step([StepEntry("outsider", [1] * (free * 8), [])])
                seen["held"] = True
            elif seen["events"] == 30 and seen["held"]:
                eng.close("outsider")
                seen["held"] = False

        for kw in (dict(), dict(temperature=0.9, top_k=30, seed=5)):
            seen.update(events=0, held=False)
            got = m.generate_batch(prompts, max_new_tokens=24, eos_token_id=None, on_event=meddle, **kw)
            assert m.last_scheduler.preemptions >= 1
            for i, (p, g) in enumerate(zip(prompts, got)):
                want = plain_generate(w, cfg, p, 24, **{**kw, "seed": kw.get("seed", 0) + i})
                assert g == want, (kw, i)
            if seen["held"]:
                eng.close("outsider")
            eng.cache.check_invariants()
            assert not eng.cache.requests
