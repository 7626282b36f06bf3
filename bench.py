#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Qwen3-8B layer sizes, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]

Prints ONE JSON line. `value` is decoded tokens per second at the given batch
(default 8) with 2,048-token prompts in a 4,096-token context, timed on the
device with CUDA events around K decode steps that run without the host in the
loop (CUDA-graph replay, sampling and feeding the token back on the device).
`e2e` is the same rate through the Python entry point (`Model.generate_batch`,
host token lists in and out; every step copies its batch arrays from pinned
host memory and reads the sampled tokens back), counted over the steps in which
every request of the batch decodes: from the moment the last request has its
first token until the first request ends (the scheduler starts requests one
prompt after the other, so they also end one after the other). `prefill` is one 2,048-token
prompt in one step; `points` are decode rates at batch 1 and 64; `roofline`
relates the decode step to HBM bandwidth (weights once + the live cache).
Weights are random (seeded) and token ids synthetic: there is no checkpoint or
dataset here. Peaks come from MEASURED_PEAKS.json when the driver wrote it.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
    intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
    head_dim=128, max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0,
    tie_word_embeddings=False,
)
SEED = 8
PROMPT_LEN = 2048
CONTEXT = 4096


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, tf, src = FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"
    try:
        d = json.load(open(path))
        hbm = float(d.get("hbm_gbs", hbm))
        tf = float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", tf)))
        src = "measured"
    except Exception:
        pass
    return hbm, tf, src


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.path = tempfile.NamedTemporaryFile(prefix="clocks_", suffix=".csv", delete=False).name
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 7:
                    continue
                try:
                    sm.append(float(f[0]))
                    mx.append(float(f[1]))
                except ValueError:
                    continue
                for name, v in zip(names, f[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons)}
        return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has (named in `config`)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="measure only the headline batch")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one part only (for profiler captures of a small case)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference",
                          "unavailable": "aiqubits/quantinfer is a Rust workspace: pip finds no setup.py/pyproject.toml at its root and there is no cargo/rustc offline, so it cannot be installed or run here"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from quantinfer_b200 import Model, kernels
    from quantinfer_b200.config import config_from_dict
    from quantinfer_b200.engine import Engine, StepEntry, tensor_needs_of_spec
    from quantinfer_b200.sampling import GenerationConfig, Sampler
    from quantinfer_b200.weights import random_tensors

    hbm_peak, tf_peak, peak_src = peaks()
    cfg_d = dict(QWEN3_8B)
    full_layers = cfg_d["num_hidden_layers"]
    if args.layers:
        cfg_d["num_hidden_layers"] = args.layers
    config = config_from_dict(cfg_d)
    spec = config.to_model_spec()
    dev = "cuda:0"
    torch.cuda.set_device(0)
    t0 = time.time()
    tensors = random_tensors(tensor_needs_of_spec(spec), SEED, torch.bfloat16, device=dev)
    max_b = 64 if not args.skip_points else max(args.batch, 1)
    n_new = args.warmup + args.steps + 2
    per_req = -(-(PROMPT_LEN + 2 * n_new + 64) // 64) * 64
    engine = Engine(spec, tensors, dtype="bfloat16", device=dev, page_size=64,
                    max_tokens=per_req * max(max_b, args.batch) + 4096, max_requests=max(max_b, args.batch),
                    max_seq_len=CONTEXT, config=config)
    del tensors
    torch.cuda.synchronize()
    load_s = time.time() - t0
    sampler = Sampler(engine.device, engine.runtime.status)
    g = torch.Generator().manual_seed(1234)
    vocab = spec.vocab_size

    def prompt(n=PROMPT_LEN):
        return torch.randint(0, vocab, (n,), generator=g).tolist()

    # ---- model arithmetic -----------------------------------------------------
    L, H, I = spec.layers and len(spec.layers), spec.hidden_size, config.intermediate_size
    nq, nkv, d = config.num_attention_heads, config.num_key_value_heads, config.effective_head_dim
    layer_params = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I
    weight_bytes = 2 * (L * layer_params + vocab * H)          # every matrix once, bf16 (head; one embedding row is negligible)
    kv_bytes_per_token = 2 * L * nkv * d * 2

    def prefill_flops(T):
        return 2.0 * T * L * layer_params + 4.0 * nq * d * (T * (T + 1) / 2) * L + 2.0 * H * vocab

    if args.only:
        args.skip_points = True
    # ---- prefill: one 2,048-token prompt in one step ---------------------------
    times = []
    for i in range(0 if args.only == "decode" else 2 + 5):
        engine.open("p")
        toks = prompt()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        engine.step([StepEntry("p", toks, [PROMPT_LEN - 1])], check_status=False)
        b.record()
        torch.cuda.synchronize()
        engine.raise_on_status()
        engine.close("p")
        if i >= 2:
            times.append(a.elapsed_time(b))
    pre_ms = sorted(times)[len(times) // 2] if times else float("nan")
    prefill = {"value": PROMPT_LEN / pre_ms * 1e3, "tokens": PROMPT_LEN, "ms": pre_ms,
               "frac": prefill_flops(PROMPT_LEN) / (pre_ms * 1e-3) / (tf_peak * 1e12)}

    # ---- decode on the device ---------------------------------------------------
    def fill(batch):
        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:
            engine.open(rid)
            engine.step([StepEntry(rid, prompt(), [])], check_status=False)
        engine.raise_on_status()
        return ids

    def decode_rate(batch, steps, warmup, sample_clocks=False):
        ids = fill(batch)
        rows = [(GenerationConfig(max_new_tokens=4096), 0)] * batch
        first = [1 + i for i in range(batch)]
        hist = engine.decode_on_device(ids, first, warmup, rows, sampler)
        last = hist[-1].tolist()
        torch.cuda.synchronize()
        clocks = ClockSampler() if sample_clocks else None
        before = kernels.launches
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.decode_on_device(ids, last, steps, rows, sampler)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        launches = kernels.launches - before
        ck = clocks.stop() if clocks else None
        ctx = engine.length(ids[0])
        for rid in ids:
            engine.close(rid)
        return batch * steps / ms * 1e3, ms / steps, launches, ck, ctx

    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "prefill": prefill}))
        return 0
    value, ms_per_step, launches, clocks, ctx_end = decode_rate(args.batch, args.steps, args.warmup, True)
    ctx_mid = ctx_end - args.steps / 2.0
    step_bytes = weight_bytes + args.batch * ctx_mid * kv_bytes_per_token
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    points = {}
    if not args.skip_points:
        for bsz in (1, 64):
            r, _, _, _, _ = decode_rate(bsz, min(args.steps, 32), 3)
            points[f"decode_b{bsz}"] = r

    if args.only == "decode":
        print(json.dumps({"only": "decode", "value": value, "ms_per_step": ms_per_step, "gpu_launches": launches}))
        return 0
    # ---- end to end through the Python entry point -----------------------------------
    model = Model.from_engine(engine, max_batch_tokens=PROMPT_LEN)
    prompts = [prompt() for _ in range(args.batch)]
    # warm-up through the same entry point (W decode steps): graphs are captured, buffers pinned
    model.generate_batch(prompts, max_new_tokens=args.warmup + 1, eos_token_id=None)
    stamps = []
    engine.h2d_bytes_max = 0
    model.generate_batch(prompts, max_new_tokens=n_new, eos_token_id=None,
                         on_event=lambda ev: stamps.append((time.perf_counter(), ev.request_id, getattr(ev, "stop_reason", None))))
    # bytes a decode step of the full batch copies host -> device: its packed batch arrays (token ids,
    # positions, lengths, slots, block tables)
    h2d_max = max([g["meta"].numel() * 4 for (b, _), g in engine._graphs.items() if b == args.batch] or [engine.h2d_bytes_max])
    # the window in which the whole batch decodes: after the last request's first token, up to the
    # step in which the first request ends
    seen, t_all_first, t_end, after = set(), None, None, 0
    for t, rid, stop in stamps:
        if t_all_first is None:
            seen.add(rid)
            if len(seen) == args.batch:
                t_all_first = t
        elif t - t_all_first < 1e-4:                 # the events of one step arrive together:
            continue                                 # the rest of the step that gave the last first token
        elif t_end is None or t - t_end < 1e-4:
            after += 1
            if stop is not None and t_end is None:
                t_end = t
    ok = t_all_first is not None and t_end is not None and after >= args.batch
    e2e = {"value": after / (t_end - t_all_first) if ok else None, "unit": "tokens/s", "h2d_bytes_per_step": h2d_max,
           "d2h_bytes_per_step": 4 * args.batch + 4, "steps": after // max(args.batch, 1) if ok else 0,
           "ms_per_step": (t_end - t_all_first) * 1e3 / (after / args.batch) if ok else None}

    line = {
        "metric": "decode tokens/s (Qwen3-8B sizes, random bf16 weights, 1 B200)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, seeded random weights", "impl": "ours",
        "config": {
            "model": "Qwen3-8B sizes", "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
            "layers": L, "layers_of_config": full_layers, "hidden": H, "heads": nq, "kv_heads": nkv, "head_dim": d,
            "intermediate": I, "vocab": vocab, "page_size": engine.page_size, "parallelism": "1 GPU",
            "l2": "inputs larger than L2 (weights %.1f GB per step)" % (weight_bytes / 1e9),
            "peaks": peak_src, "load_s": round(load_s, 1),
        },
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak},
        "points": points,
        "e2e": e2e,
        "gpu_launches": launches,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
