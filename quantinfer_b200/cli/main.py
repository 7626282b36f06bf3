"""The command line, in the manner of the reference's `quantinfer` binary
(apps/quantinfer-cli/src/commands/mod.rs:17-72, generate.rs:17-338).

    quantinfer generate --input MODEL_DIR --tokens 1,2,3 [--max-new-tokens N]
        [--temperature T] [--seed N] [--eos-token-id ID] [--max-sequence-length N]
        [--top-k K] [--top-p P] [--dtype bfloat16|float32] [--backend cuda]
        [--page-size N] [--max-batch-tokens N] [--chunk-size N]
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
"""

from __future__ import annotations

import json
import os
import sys
import time

HELP = """quantinfer commands:
  generate --input MODEL_DIR --tokens 1,2,3 [--max-new-tokens N] [--max-sequence-length N] [--temperature T] [--top-k K] [--top-p P] [--seed N] [--eos-token-id ID] [--dtype bfloat16|float32] [--backend cuda] [--page-size N] [--max-batch-tokens N] [--chunk-size N] [--profile] [--profile-report NEW_REPORT.json]
  random-weights --config CONFIG.json --output MODEL_DIR [--seed N] [--dtype bfloat16|float32]

MODEL_DIR holds config.json and model.safetensors (or model.safetensors.index.json with its shards).
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


def generate(arguments) -> int:
    opts = parse_options(arguments, [
        ("--backend", True), ("--input", True), ("--tokens", True), ("--prompt", True),
        ("--max-new-tokens", True), ("--temperature", True), ("--eos-token-id", True), ("--seed", True),
        ("--max-sequence-length", True), ("--profile", False), ("--profile-report", True),
        ("--top-k", True), ("--top-p", True), ("--dtype", True), ("--page-size", True),
        ("--max-batch-tokens", True), ("--chunk-size", True), ("--device", True),
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
    prompt = parse_token_ids(opts["--tokens"])
    if not prompt:
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
    from ..engine import Engine, StepEntry
    from ..engine.engine import DEFAULT_PAGE_SIZE
    from ..sampling import GenerationConfig, Sampler

    load_started = time.perf_counter()
    config = load_config(opts["--input"])
    spec = config.to_model_spec()
    if any(t >= spec.vocab_size for t in prompt):
        raise UsageError("prompt token id is outside the model vocabulary")
    if eos is not None and eos >= spec.vocab_size:
        raise UsageError("EOS token id is outside the model vocabulary")
    max_sequence_length = max_seq if max_seq is not None else spec.max_positions
    if max_sequence_length == 0 or max_sequence_length > spec.max_positions:
        raise UsageError(f"--max-sequence-length must be between 1 and {spec.max_positions}")
    if len(prompt) > max_sequence_length:
        raise UsageError("prompt exceeds --max-sequence-length")
    if len(prompt) + max_new > max_sequence_length:
        raise UsageError("prompt and max_new_tokens exceed --max-sequence-length")
    gen = GenerationConfig(max_new_tokens=max_new, temperature=temperature, top_k=top_k, top_p=top_p,
                           eos_token_id=eos, seed=seed)
    try:
        gen.validate(spec.vocab_size)
    except ValueError as exc:
        raise UsageError(f"invalid generation config: {exc}") from None
    page = _number(opts, "--page-size", int, DEFAULT_PAGE_SIZE)
    engine = Engine.from_folder(opts["--input"], dtype=dtype, device=opts.get("--device", "cuda:0"),
                                page_size=page, max_tokens=len(prompt) + max_new, max_requests=1,
                                max_seq_len=max_sequence_length)
    import torch

    torch.cuda.synchronize()
    model_load_ms = (time.perf_counter() - load_started) * 1000.0
    sampler = Sampler(engine.device, engine.runtime.status)
    chunk = _number(opts, "--chunk-size", int) or _number(opts, "--max-batch-tokens", int, 8192)
    engine.open(0)

    generated = []
    first_token_at = last_token_at = None
    prefill_started = time.perf_counter()
    logits = None
    for a in range(0, len(prompt), chunk):
        part = prompt[a:a + chunk]
        last = a + chunk >= len(prompt)
        logits = engine.step([StepEntry(0, part, [len(part) - 1] if last else [])])
    torch.cuda.synchronize()
    prefill_ms = (time.perf_counter() - prefill_started) * 1000.0
    decode_started = time.perf_counter()
    # One forward per emitted token except the last: the request's cache ends at
    # prompt + generated - 1 (crates/quantinfer-runtime/src/session.rs:153-164).
    for n in range(max_new):
        token = sampler.sample(logits, [(gen, n)])[0]
        if profile:
            now = time.perf_counter()
            first_token_at = first_token_at or now
            last_token_at = now
        generated.append(token)
        if token == eos or n + 1 == max_new:
            break
        logits = engine.step([StepEntry(0, [token], [0])])
    decode_s = time.perf_counter() - decode_started

    print(f"prompt_tokens={prompt}")
    print(f"generated_tokens={generated}")
    print(f"prefill_ms={prefill_ms:.3f}")
    print(f"decode_ms={decode_s * 1000.0:.3f}")
    print(f"decode_tokens={len(generated)}")
    if decode_s > 0:
        print(f"decode_tokens_per_sec={len(generated) / decode_s:.3f}")
    if profile and first_token_at is not None:
        decode = last_token_at - first_token_at
        ttft_ms = (first_token_at - prefill_started) * 1000.0
        rate = (len(generated) - 1) / decode if decode > 0 else None
        token_bytes = engine.cache.pool_bytes() // max(engine.cache.num_pages * engine.page_size, 1)
        kv_bytes = engine.length(0) * token_bytes
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
        if report is not None:
            body = {
                "model": os.path.abspath(opts["--input"]), "dtype": dtype,
                "model_load_ms": model_load_ms, "prefill_ms": prefill_ms, "ttft_ms": ttft_ms,
                "decode_tokens": len(generated), "profile_decode_ms": decode * 1000.0,
                "profile_decode_tokens_per_sec": rate, "kv_cache_bytes": kv_bytes,
                "kv_cache_capacity_bytes": kv_capacity, "max_sequence_length": max_sequence_length,
                "peak_rss_kib": rss,
            }
            tmp = report + f".tmp{os.getpid()}"
            with open(tmp, "x") as f:
                json.dump(body, f, indent=2)
                f.write("\n")
            os.link(tmp, report)  # fails if the report appeared meanwhile
            os.unlink(tmp)
    engine.close(0)
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
