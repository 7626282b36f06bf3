"""The command line, in the manner of the reference's `quantinfer` binary
(apps/quantinfer-cli/src/commands/mod.rs:17-72, generate.rs:17-338).

    quantinfer generate --input MODEL_DIR --tokens 1,2,3[;4,5;...] [--max-new-tokens N]
        [--temperature T] [--seed N] [--eos-token-id ID] [--max-sequence-length N]
        [--top-k K] [--top-p P] [--dtype bfloat16|float32] [--backend cuda]
        [--page-size N] [--num-pages N] [--max-batch-tokens N] [--chunk-size N]
        [--random-weights [--weights-seed N]] [--check-finite]
        [--profile] [--profile-report NEW_REPORT.json]
    quantinfer random-weights --config CONFIG.json --output MODEL_DIR [--seed N] [--dtype bfloat16|float32]

Options keep the reference's names and meanings where it has them
(generate.rs:18-39): defaults max_new_tokens 128, temperature 0, seed 0
(generate.rs:51-85); exactly one of --tokens and --prompt (generate.rs:48-50) -
and --prompt is refused here, since there is no tokenizer; ids are
comma-separated, spaces allowed (commands/common.rs:3-13). Unknown, duplicate
and valueless options are errors (common.rs:43-67). The printed lines are the
reference's: prompt_tokens, generated_tokens, prefill_ms, decode_ms,
decode_tokens, decode_tokens_per_sec, and with --profile model_load_ms, ttft_ms,
profile_decode_ms, profile_decode_tokens_per_sec, kv_cache_bytes,
kv_cache_capacity_bytes, max_sequence_length, peak_rss_kib (generate.rs:278-336).
--input takes a model folder (config.json + safetensors) directly; the
reference first converts such a folder (README.md:32-41).

What this command adds. `--tokens` takes several prompts separated by `;`: they
run as one batch, request i draws with seed + i, and a prompt_tokens /
generated_tokens pair is printed for each in order. Generation goes through the
scheduler (engine/generation.py), the same loop the Python entry point uses:
`--max-batch-tokens` is a step's token budget, `--chunk-size` the longest prompt
portion in a step, `--num-pages` the size of the page pool (by default enough
for every prompt with its new tokens). `--random-weights` makes the weights on
the device from `--weights-seed` instead of reading them: `--input` then names
a config.json, or a folder that holds one. Times are taken where tokens reach
the host: prefill_ms ends when every request has its first token, decode_ms
runs from there to the last token.
"""

from __future__ import annotations

import json
import os
import sys
import time

HELP = """quantinfer commands:
  generate --input MODEL_DIR --tokens 1,2,3[;4,5;...] [--max-new-tokens N] [--max-sequence-length N] [--temperature T] [--top-k K] [--top-p P] [--seed N] [--eos-token-id ID] [--dtype bfloat16|float32] [--backend cuda] [--page-size N] [--num-pages N] [--max-batch-tokens N] [--chunk-size N] [--random-weights [--weights-seed N]] [--check-finite] [--no-run-ahead] [--profile] [--profile-report NEW_REPORT.json]
  random-weights --config CONFIG.json --output MODEL_DIR [--seed N] [--dtype bfloat16|float32]

MODEL_DIR holds config.json and model.safetensors (or model.safetensors.index.json with its shards);
with --random-weights, --input names a config.json (or a folder with one) and the weights are drawn on the device.
Several prompts separated by ';' run as one batch through the scheduler; request i draws with seed + i.
--prompt TEXT is not available: this engine has no tokenizer and works on token ids."""


class UsageError(Exception):
    pass


def parse_options(arguments, accepted):
    """Strict parsing: every option must be known, come once, and bring its value."""
    accepted = dict(accepted)
    entries = {}
    it = iter(arguments)
    for flag in it:
        if flag not in accepted:
            raise UsageError(f"unknown option {flag}; use --help for usage")
        value = None
        if accepted[flag]:
            try:
                value = next(it)
            except StopIteration:
                raise UsageError(f"{flag} requires a value") from None
        if flag in entries:
            raise UsageError(f"duplicate option {flag}; specify it only once")
        entries[flag] = value
    return entries


def parse_token_ids(value: str):
    out = []
    for token in value.split(","):
        token = token.strip()
        try:
            n = int(token)
            if n < 0 or not token.isdigit():
                raise ValueError
        except ValueError:
            raise UsageError(f"invalid token id {token!r}: not an unsigned integer") from None
        out.append(n)
    return out


def _number(opts, flag, kind, default=None):
    if flag not in opts:
        return default
    try:
        v = kind(opts[flag])
        if kind is int and v < 0:
            raise ValueError("negative")
        return v
    except ValueError as exc:
        raise UsageError(f"invalid {flag}: {exc}") from None


def _peak_rss_kib():
    try:
        for line in open("/proc/self/status"):
            if line.startswith("VmHWM:"):
                return int(line.split()[1])
    except OSError:
        pass
    return None


def parse_prompts(value: str):
    """`1,2,3` or several prompts `1,2,3;4,5`; an empty prompt is an error."""
    prompts = [parse_token_ids(part) for part in value.split(";")]
    return prompts


def _load_engine(opts, dtype, max_sequence_length, page, pool_tokens, num_pages, n_requests, spec, config):
    from ..engine import Engine

    common = dict(dtype=dtype, device=opts.get("--device", "cuda:0"), page_size=page, max_tokens=pool_tokens,
                  num_pages=num_pages, max_requests=n_requests, max_seq_len=max_sequence_length)
    if "--random-weights" not in opts:
        return Engine.from_folder(opts["--input"], check_finite="--check-finite" in opts, **common)
    import torch

    from ..engine import tensor_needs_of_spec
    from ..weights import random_tensors

    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = random_tensors(tensor_needs_of_spec(spec), _number(opts, "--weights-seed", int, 0), stored,
                             device=opts.get("--device", "cuda:0"))
    return Engine(spec, tensors, config=config, **common)


def generate(arguments) -> int:
    opts = parse_options(arguments, [
        ("--backend", True), ("--input", True), ("--tokens", True), ("--prompt", True),
        ("--max-new-tokens", True), ("--temperature", True), ("--eos-token-id", True), ("--seed", True),
        ("--max-sequence-length", True), ("--profile", False), ("--profile-report", True),
        ("--top-k", True), ("--top-p", True), ("--dtype", True), ("--page-size", True), ("--num-pages", True),
        ("--max-batch-tokens", True), ("--chunk-size", True), ("--device", True),
        ("--random-weights", False), ("--weights-seed", True), ("--check-finite", False), ("--no-run-ahead", False),
    ])
    backend = opts.get("--backend", "cuda")
    if backend != "cuda":
        raise UsageError(f"unsupported backend {backend!r}: this engine runs on cuda only")
    if "--input" not in opts:
        raise UsageError("generate requires --input")
    if ("--tokens" in opts) == ("--prompt" in opts):
        raise UsageError("generate requires exactly one of --tokens or --prompt")
    if "--prompt" in opts:
        raise UsageError("--prompt needs a tokenizer, which this engine does not have; pass --tokens")
    if "--weights-seed" in opts and "--random-weights" not in opts:
        raise UsageError("--weights-seed goes with --random-weights")
    prompts = parse_prompts(opts["--tokens"])
    if not all(prompts):
        raise UsageError("--tokens must contain at least one token id")
    max_new = _number(opts, "--max-new-tokens", int, 128)
    temperature = _number(opts, "--temperature", float, 0.0)
    eos = _number(opts, "--eos-token-id", int)
    seed = _number(opts, "--seed", int, 0)
    max_seq = _number(opts, "--max-sequence-length", int)
    top_k = _number(opts, "--top-k", int)
    top_p = _number(opts, "--top-p", float)
    dtype = opts.get("--dtype", "bfloat16")
    if dtype not in ("bfloat16", "float32"):
        raise UsageError("--dtype must be bfloat16 or float32")
    report = opts.get("--profile-report")
    if report is not None and os.path.exists(report):
        raise UsageError("profile report already exists")
    profile = "--profile" in opts or report is not None

    from ..config import load_config
    from ..engine.engine import DEFAULT_PAGE_SIZE
    from ..engine.generation import run_requests
    from ..sampling import GenerationConfig, Sampler

    load_started = time.perf_counter()
    config = load_config(opts["--input"])
    spec = config.to_model_spec()
    if any(t >= spec.vocab_size for p in prompts for t in p):
        raise UsageError("prompt token id is outside the model vocabulary")
    if eos is not None and eos >= spec.vocab_size:
        raise UsageError("EOS token id is outside the model vocabulary")
    max_sequence_length = max_seq if max_seq is not None else spec.max_positions
    if max_sequence_length == 0 or max_sequence_length > spec.max_positions:
        raise UsageError(f"--max-sequence-length must be between 1 and {spec.max_positions}")
    longest = max(len(p) for p in prompts)
    if longest > max_sequence_length:
        raise UsageError("prompt exceeds --max-sequence-length")
    if longest + max_new > max_sequence_length:
        raise UsageError("prompt and max_new_tokens exceed --max-sequence-length")
    configs = []
    for i in range(len(prompts)):
        gen = GenerationConfig(max_new_tokens=max_new, temperature=temperature, top_k=top_k, top_p=top_p,
                               eos_token_id=eos, seed=(seed + i) % (1 << 64))
        try:
            gen.validate(spec.vocab_size)
        except ValueError as exc:
            raise UsageError(f"invalid generation config: {exc}") from None
        configs.append(gen)
    page = _number(opts, "--page-size", int, DEFAULT_PAGE_SIZE)
    num_pages = _number(opts, "--num-pages", int)
    if page == 0 or num_pages == 0:
        raise UsageError("--page-size and --num-pages must be positive")
    unit = max(64, page)
    pool_tokens = sum(-(-(len(p) + max_new) // unit) * unit for p in prompts)
    budget = _number(opts, "--max-batch-tokens", int, 8192)
    chunk = _number(opts, "--chunk-size", int)
    if budget == 0 or chunk == 0:
        raise UsageError("--max-batch-tokens and --chunk-size must be positive")
    engine = _load_engine(opts, dtype, max_sequence_length, page, pool_tokens, num_pages, len(prompts), spec, config)
    import torch

    torch.cuda.synchronize()
    model_load_ms = (time.perf_counter() - load_started) * 1000.0
    sampler = Sampler.for_engine(engine)
    # One forward per emitted token except the last: a request's cache ends at
    # prompt + generated - 1 positions (crates/quantinfer-runtime/src/session.rs:153-164).
    run = run_requests(engine, sampler, prompts, configs, max_batch_tokens=max(budget, len(prompts)), chunk_size=chunk,
                       run_ahead="--no-run-ahead" not in opts)
    first_all = run.all_first_tokens_at()
    last = max(r.last_token_at for r in run.results)
    prefill_ms = (first_all - run.started_at) * 1000.0
    decode_s = last - first_all
    total = sum(len(r.tokens) for r in run.results)

    for r in run.results:
        print(f"prompt_tokens={r.prompt}")
        print(f"generated_tokens={r.tokens}")
    print(f"prefill_ms={prefill_ms:.3f}")
    print(f"decode_ms={decode_s * 1000.0:.3f}")
    print(f"decode_tokens={total}")
    if decode_s > 0:
        print(f"decode_tokens_per_sec={total / decode_s:.3f}")
    if profile:
        first = min(r.first_token_at for r in run.results)
        decode = last - first
        ttft_ms = (first - run.started_at) * 1000.0
        rate = (total - len(prompts)) / decode if decode > 0 else None
        token_bytes = engine.cache.pool_bytes() // max(engine.cache.num_pages * engine.page_size, 1)
        kv_bytes = sum(len(r.prompt) + len(r.tokens) - 1 for r in run.results) * token_bytes
        kv_capacity = engine.cache.pool_bytes()
        rss = _peak_rss_kib()
        print(f"model_load_ms={model_load_ms:.3f}")
        print(f"ttft_ms={ttft_ms:.3f}")
        print(f"profile_decode_ms={decode * 1000.0:.3f}")
        if rate is not None:
            print(f"profile_decode_tokens_per_sec={rate:.3f}")
        print(f"kv_cache_bytes={kv_bytes}")
        print(f"kv_cache_capacity_bytes={kv_capacity}")
        print(f"max_sequence_length={max_sequence_length}")
        print(f"peak_rss_kib={rss if rss is not None else 'unmeasured'}")
        print(f"scheduler_steps={run.scheduler.steps}")
        if report is not None:
            body = {
                "model": os.path.abspath(opts["--input"]), "dtype": dtype, "requests": len(prompts),
                "model_load_ms": model_load_ms, "prefill_ms": prefill_ms, "ttft_ms": ttft_ms,
                "decode_tokens": total, "profile_decode_ms": decode * 1000.0,
                "profile_decode_tokens_per_sec": rate, "kv_cache_bytes": kv_bytes,
                "kv_cache_capacity_bytes": kv_capacity, "max_sequence_length": max_sequence_length,
                "peak_rss_kib": rss, "scheduler_steps": run.scheduler.steps,
            }
            tmp = report + f".tmp{os.getpid()}"
            with open(tmp, "x") as f:
                json.dump(body, f, indent=2)
                f.write("\n")
            os.link(tmp, report)  # fails if the report appeared meanwhile
            os.unlink(tmp)
    return 0


def random_weights(arguments) -> int:
    opts = parse_options(arguments, [("--config", True), ("--output", True), ("--seed", True), ("--dtype", True)])
    if "--config" not in opts or "--output" not in opts:
        raise UsageError("random-weights requires --config and --output")
    import torch

    from ..config import config_from_dict
    from ..weights import write_model_folder

    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}.get(opts.get("--dtype", "bfloat16"))
    if dtype is None:
        raise UsageError("--dtype must be bfloat16 or float32")
    with open(opts["--config"]) as f:
        cfg = config_from_dict(json.load(f))
    write_model_folder(opts["--output"], cfg, _number(opts, "--seed", int, 0), dtype)
    print(f"wrote {opts['--output']}")
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("--help", "-h", "help"):
        print(HELP)
        return 0
    commands = {"generate": generate, "random-weights": random_weights}
    if argv[0] not in commands:
        print(f"unknown command {argv[0]}; use --help for usage", file=sys.stderr)
        return 2
    try:
        return commands[argv[0]](argv[1:])
    except UsageError as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 2
    except Exception as exc:  # config, weight and runtime errors: one line, no traceback
        print(f"error: {exc}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
