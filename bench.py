#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3 layer sizes, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model 8b|14b|32b] [--batch B] [--layers L]
                    [--impl reference] [--skip-points] [--skip-classes] [--skip-mixed] [--only decode|prefill|mixed]
    python bench.py --timeline [--batch B] [--only prefill]     a decode step (or a prefill) kernel by kernel (markdown, not the JSON line)

Prints ONE JSON line. `value` is decoded tokens per second at the headline batch
of the chosen model (8b: 8 requests with 2,048-token prompts in a 4,096-token
context, the default; 14b: 32 requests; 32b: 16 requests with 8,192-token
prompts in a 16,384-token context), timed on the device with CUDA events around
K decode steps that run without the host in the loop (CUDA-graph replay,
sampling and feeding the token back on the device).

`e2e` is the same rate through the Python entry point (`Model.generate_batch`,
host token lists in and out; every step copies its batch arrays from pinned
host memory and reads the sampled tokens back), counted over the steps in which
every request of the batch decodes: from the moment the last request has its
first token until the first request ends. It is taken at the headline batch and
at the other batches of `points`.

`prefill` is one prompt in one step (`frac` against the sustained matrix peak,
`frac_burst` against the burst peak). `points` are decode rates at the other
batches. `roofline` relates the decode step to HBM bandwidth (every weight once
plus the live cache). `classes` splits the decode step and the prefill step by
kernel class, by leaving one class out at a time and timing the rest: GEMMs,
attention, and what remains; each with its share of the bytes (decode) or flops
(prefill) and the fraction of the peak that gives. `mixed` is the scheduler
workload of the 14B configuration (32 requests, prompt lengths uniform in
[128, 4096], 128 new tokens each, temperature 0.7, context 8,192) at the chosen
model's sizes through `Model.generate_batch`: all tokens per second of wall
clock and the time to the first token.

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
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0

_COMMON = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, head_dim=128,
               num_key_value_heads=8, max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0,
               tie_word_embeddings=False)
# layer sizes, the seed of the random weights, and the workload: (prompt length, context, headline batch, other batches)
MODELS = {
    "8b": dict(config=dict(_COMMON, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32),
               seed=8, prompt_len=2048, context=4096, batch=8, points=(1, 64), name="Qwen3-8B sizes"),
    "14b": dict(config=dict(_COMMON, hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40),
                seed=14, prompt_len=2048, context=8192, batch=32, points=(1,), name="Qwen3-14B sizes"),
    "32b": dict(config=dict(_COMMON, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64),
                seed=32, prompt_len=8192, context=16384, batch=16, points=(1,), name="Qwen3-32B sizes"),
}
MIXED = dict(requests=32, prompt_lo=128, prompt_hi=4096, new_tokens=128, temperature=0.7, context=8192)


def peaks():
    """(HBM GB/s, sustained bf16 TFLOP/s, burst bf16 TFLOP/s, where they come from)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, burst, src = FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"
    sustained = burst
    try:
        d = json.load(open(path))
        hbm = float(d.get("hbm_gbs", hbm))
        burst = float(d.get("bf16_tflops", burst))
        sustained = float(d.get("bf16_tflops_sustained", burst))
        src = "measured"
    except Exception:
        pass
    return hbm, sustained, burst, src


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


def model_arithmetic(config, spec):
    """Parameter counts, bytes and flops of the configuration (every matrix bf16)."""
    L, H, I, V = len(spec.layers), spec.hidden_size, config.intermediate_size, spec.vocab_size
    nq, nkv, d = config.num_attention_heads, config.num_key_value_heads, config.effective_head_dim
    layer_params = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I
    a = dict(L=L, H=H, I=I, V=V, nq=nq, nkv=nkv, d=d, layer_params=layer_params)
    a["weight_bytes"] = 2 * (L * layer_params + V * H)       # the head's matrix too; one embedding row is negligible
    a["kv_bytes_per_token"] = 2 * L * nkv * d * 2
    a["gemm_flops"] = lambda T, rows=1: 2.0 * T * L * layer_params + 2.0 * H * V * rows
    a["attn_flops"] = lambda T: 4.0 * nq * d * (T * (T + 1) / 2) * L
    return a


def build_engine(args, entry, context, max_requests, pool_tokens):
    import torch

    from quantinfer_b200.config import config_from_dict
    from quantinfer_b200.engine import Engine, tensor_needs_of_spec
    from quantinfer_b200.weights import random_tensors

    cfg_d = dict(entry["config"])
    if args.layers:
        cfg_d["num_hidden_layers"] = args.layers
    config = config_from_dict(cfg_d)
    spec = config.to_model_spec()
    t0 = time.time()
    tensors = random_tensors(tensor_needs_of_spec(spec), entry["seed"], torch.bfloat16, device="cuda:0")
    engine = Engine(spec, tensors, dtype="bfloat16", device="cuda:0", page_size=64, max_tokens=pool_tokens,
                    max_requests=max_requests, max_seq_len=context, config=config)
    del tensors
    torch.cuda.synchronize()
    return engine, config, spec, time.time() - t0


class Bench:
    def __init__(self, args, entry):
        import torch

        from quantinfer_b200.sampling import Sampler

        self.args, self.entry, self.torch = args, entry, torch
        self.prompt_len, self.context = entry["prompt_len"], entry["context"]
        self.batches = [args.batch] + ([] if args.skip_points else [b for b in entry["points"] if b != args.batch])
        self.n_new = args.warmup + args.steps + 2
        # End to end, the first W steps in which the whole batch decodes are warm-up, as they are on the device, and
        # the window after them is at least 128 steps long, however few steps the device-timed run takes: for some
        # 70 ms after the prompts the chip stays at the clock the prefill left it at under the power cap (at
        # Qwen3-8B sizes 7 steps of 4.1 ms, then 11 of 3.8, then 3.53), which the device-timed run does not see,
        # because the capture of its graph lies between its prompts and its steps
        self.n_e2e = max(self.n_new, 128) + args.warmup
        max_b = max(self.batches)
        # a request decodes warm-up + timed steps on the device, or (end to end) as many steps as it takes until
        # the last request of its batch has joined plus the timed ones: room for the longer of the two
        per_req = -(-(self.prompt_len + self.n_new + self.n_e2e + max_b + 64) // 64) * 64
        self.engine, self.config, self.spec, self.load_s = build_engine(
            args, entry, self.context, max_b, per_req * max_b + self.prompt_len + 2048)
        self.sampler = Sampler(self.engine.device, self.engine.runtime.status)
        self.gen = torch.Generator().manual_seed(1234)
        self.arith = model_arithmetic(self.config, self.spec)

    def prompt(self, n=None):
        return self.torch.randint(0, self.spec.vocab_size, (n or self.prompt_len,), generator=self.gen).tolist()

    # ---- prefill: one prompt in one step --------------------------------------------
    def prefill_ms(self, runs=5, warm=2):
        from quantinfer_b200.engine import StepEntry

        torch, engine, times = self.torch, self.engine, []
        for i in range(warm + runs):
            engine.open("p")
            toks = self.prompt()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            engine.step([StepEntry("p", toks, [self.prompt_len - 1])], check_status=False)
            b.record()
            torch.cuda.synchronize()
            engine.raise_on_status()
            engine.close("p")
            if i >= warm:
                times.append(a.elapsed_time(b))
        return sorted(times)[len(times) // 2]

    # ---- decode on the device -----------------------------------------------------------
    def fill(self, batch):
        from quantinfer_b200.engine import StepEntry

        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:
            self.engine.open(rid)
            self.engine.step([StepEntry(rid, self.prompt(), [])], check_status=False)
        return ids

    def decode_rate(self, batch, steps, warmup, sample_clocks=False):
        from quantinfer_b200 import kernels
        from quantinfer_b200.sampling import GenerationConfig

        torch, engine = self.torch, self.engine
        ids = self.fill(batch)
        rows = [(GenerationConfig(max_new_tokens=1 << 20), 0)] * batch
        first = [1 + i for i in range(batch)]
        hist = engine.decode_on_device(ids, first, warmup, rows, self.sampler)
        vocab = self.spec.vocab_size
        last = [t if 0 <= t < vocab else 1 for t in hist[-1].tolist()]      # (with kernels left out the tokens mean nothing)
        torch.cuda.synchronize()
        clocks = ClockSampler() if sample_clocks else None
        before = kernels.launches
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.decode_on_device(ids, last, steps, rows, self.sampler)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        launches = kernels.launches - before
        ck = clocks.stop() if clocks else None
        ctx = engine.length(ids[0])
        for rid in ids:
            engine.close(rid)
        return dict(rate=batch * steps / ms * 1e3, ms=ms / steps, launches=launches, clocks=ck, ctx_mid=ctx - steps / 2.0)

    # ---- end to end through the Python entry point ---------------------------------------
    def e2e(self, model, batch):
        """Rate over the steps in which the whole batch decodes, after W such steps of warm-up, by the times at
        which tokens reach the host."""
        # requests join one prompt after the other: each decodes `batch` steps more than the warm-up and the timed
        # ones, so that the window in which all of them decode is that long
        engine, n_new = self.engine, min(self.n_e2e + batch, self.context - self.prompt_len)
        prompts = [self.prompt() for _ in range(batch)]
        # warm-up through the same entry point (W decode steps): graphs are captured, buffers pinned
        model.generate_batch(prompts, max_new_tokens=self.args.warmup + 1, eos_token_id=None)
        stamps = []
        engine.h2d_bytes_max = 0
        model.generate_batch(prompts, max_new_tokens=n_new, eos_token_id=None,
                             on_event=lambda ev: stamps.append((time.perf_counter(), ev.request_id, getattr(ev, "stop_reason", None))))
        # bytes a decode step of the full batch copies host -> device: its packed batch arrays (token ids,
        # positions, lengths, slots, block tables)
        h2d = max([g["meta"].numel() * 4 for (b, _), g in engine._graphs.items() if b == batch] or [engine.h2d_bytes_max])
        # the events of one step arrive together: steps = [time, events, one of them a stop]
        steps = []
        for t, rid, stop in stamps:
            if not steps or t - steps[-1][0] > 1e-4:
                steps.append([t, 0, False, set()])
            steps[-1][1] += 1
            steps[-1][2] |= stop is not None
            steps[-1][3].add(rid)
        # the window in which the whole batch decodes: from the step that gave the last request's first token and
        # the W warm-up steps after it, up to the step in which the first request ends
        seen, first, last = set(), None, None
        for i, (_, _, stopped, rids) in enumerate(steps):
            if first is None:
                seen |= rids
                if len(seen) == batch:
                    first = i + self.args.warmup
            elif stopped and last is None:
                last = i
        ok = first is not None and last is not None and last - first >= 8
        tokens = sum(n for _, n, _, _ in steps[first + 1:last + 1]) if ok else 0
        span = steps[last][0] - steps[first][0] if ok else None
        return {"value": tokens / span if ok else None, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * batch + 4, "steps": last - first if ok else 0, "warmup": self.args.warmup,
                "ms_per_step": span * 1e3 / (last - first) if ok else None}

    # ---- the step by kernel class ---------------------------------------------------------------
    def classes(self, full_decode_ms, full_prefill_ms, ctx_mid, peaks_):
        """Two timings for each class of kernels. `alone`: the step with every other class left out, so
        that the class's kernels run back to back: the rate at which they stream their bytes (decode) or
        do their flops (prefill). `left_out`: the full step's time less the step's without the class:
        what the class costs where it stands, after what overlaps with its neighbours. The sum of the
        `alone` times falls short of the step by what the hand-over from kernel to kernel costs."""
        from quantinfer_b200 import kernels

        hbm, sustained, burst, _ = peaks_
        a, batch, T = self.arith, self.args.batch, self.prompt_len
        steps = max(8, min(self.args.steps, 16))
        every = ("gemm", "attention", "norm", "rope", "other")
        work = {
            "gemm": (a["weight_bytes"], a["gemm_flops"](T)),
            "attention": (batch * ctx_mid * a["kv_bytes_per_token"], a["attn_flops"](T)),
        }

        def timed(knocked):
            kernels.knock_out = frozenset(knocked)
            self.engine._graphs.clear()
            try:
                return self.decode_rate(batch, steps, 3)["ms"], self.prefill_ms(runs=3, warm=1)
            finally:
                kernels.knock_out = frozenset()
                self.engine._graphs.clear()

        out = {"note": "alone: only this class runs; left_out: full step less the step without it. decode fractions "
                       "from alone (graph replays, no host in it), prefill fractions from left_out (a class alone is "
                       "too short a step for its host)"}
        rest = [full_decode_ms, full_prefill_ms]
        for cls in ("gemm", "attention", "norm"):
            d_alone, p_alone = timed([c for c in every if c != cls])
            d_without, p_without = timed([cls])
            p_cost = full_prefill_ms - p_without
            row = {"decode_alone_ms": round(d_alone, 4), "decode_left_out_ms": round(full_decode_ms - d_without, 4),
                   "prefill_alone_ms": round(p_alone, 4), "prefill_left_out_ms": round(p_cost, 4)}
            rest[0] -= d_alone
            rest[1] -= p_cost
            if cls in work and d_alone > 0 and p_cost > 0:
                gbs, tf = work[cls][0] / (d_alone * 1e-3) / 1e9, work[cls][1] / (p_cost * 1e-3) / 1e12
                row.update({"decode_gbs": round(gbs, 1), "decode_frac_hbm": round(gbs / hbm, 3), "prefill_tflops": round(tf, 1),
                            "prefill_frac_burst": round(tf / burst, 3), "prefill_frac_sustained": round(tf / sustained, 3)})
            out[cls] = row
        out["rest"] = {"decode_ms": round(rest[0], 4), "prefill_ms": round(rest[1], 4)}
        kernel = self.prefill_attention_kernel(burst)
        if kernel:      # the attention's prefill rate from its kernel alone, not from a difference of two capped steps
            out["attention"].update(kernel)
            out["attention"].update({"prefill_tflops": kernel["prefill_kernel_tflops"], "prefill_frac_burst": kernel["prefill_kernel_frac_burst"],
                                     "prefill_frac_sustained": round(kernel["prefill_kernel_tflops"] / sustained, 3)})
        return out

    def prefill_attention_kernel(self, burst):
        """The prefill attention kernel by itself, the prompt's shape, 20 launches back to back between two
        events (each takes longer than the host needs to issue it): in the step's `left_out` figure the clock
        under the power cap moves with what the neighbours multiply, here it does not."""
        from quantinfer_b200 import kernels

        torch, spec, T = self.torch, self.spec, self.prompt_len
        att = spec.layers[0].mixer
        nq, nkv, d, ps = att.num_heads, att.num_kv_heads, att.head_dim, 64
        if not kernels.attention_prefill_tcgen05_supported(nq, nkv, d, ps, T // ps + 2):
            return None
        dev = "cuda:0"
        as_int = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        n_pages = T // ps + 2
        kp = torch.randn(n_pages, nkv, ps, d, device=dev).to(torch.bfloat16)
        vp = torch.randn_like(kp)
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
        q = torch.randn(T, nq * d, device=dev).to(torch.bfloat16)
        o = torch.zeros_like(q)
        tiles = [(0, t0) for t0 in range(0, T, kernels.QUERY_TILE)][::-1]
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        args = (q, o, kp, vp, table, as_int([0, T]), as_int([0]), as_int([t[0] for t in tiles]), as_int([t[1] for t in tiles]),
                nq, nkv, d, d ** -0.5, 0, status)
        call = lambda: kernels.attention_prefill(*args, impl="tcgen05", max_kv_len=T, key_ranges=1)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = 20
        a.record()
        for _ in range(n):
            call()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) / n * 1e3
        tf = 4.0 * nq * d * T * (T + 1) / 2 / us / 1e6
        return {"prefill_kernel_us": round(us, 1), "prefill_kernel_tflops": round(tf, 1), "prefill_kernel_frac_burst": round(tf / burst, 3)}


def mixed_workload(args, entry):
    """The scheduler workload: 32 requests with prompts of 128 to 4,096 tokens (seeded), 128 new tokens each at
    temperature 0.7 in a context of 8,192, all submitted at once through Model.generate_batch. The first pass
    captures the decode graphs; the second is timed by the wall clock, host in the loop."""
    import torch

    from quantinfer_b200 import Model

    w = MIXED
    g = torch.Generator().manual_seed(4321)
    lens = torch.randint(w["prompt_lo"], w["prompt_hi"] + 1, (w["requests"],), generator=g).tolist()
    pool = sum(-(-(n + w["new_tokens"]) // 64) * 64 for n in lens) + 4096
    engine, config, spec, _ = build_engine(args, entry, w["context"], w["requests"], pool)
    prompts = [torch.randint(0, spec.vocab_size, (n,), generator=g).tolist() for n in lens]
    model = Model.from_engine(engine, max_batch_tokens=args.mixed_budget, chunk_size=args.mixed_chunk)
    out = {}
    for timed in (False, True):
        clocks = ClockSampler() if timed else None
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = model.generate_batch(prompts, max_new_tokens=w["new_tokens"], eos_token_id=None, temperature=w["temperature"], seed=7)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        if timed:
            run = model.last_run
            ttft = sorted((r.first_token_at - run.started_at) * 1e3 for r in run.results)
            generated = sum(len(t) for t in res)
            out = {"requests": w["requests"], "prompt_tokens": sum(lens), "generated_tokens": generated, "wall_s": round(wall, 4),
                   "tokens_per_s": round((sum(lens) + generated) / wall, 1), "generated_per_s": round(generated / wall, 1),
                   "ttft_ms_p50": round(ttft[len(ttft) // 2], 2), "ttft_ms_p90": round(ttft[int(len(ttft) * 0.9)], 2),
                   "ttft_ms_max": round(ttft[-1], 2), "steps": run.scheduler.steps, "steps_ahead": run.scheduler.steps_ahead,
                   "token_budget": args.mixed_budget, "chunk": args.mixed_chunk or args.mixed_budget,
                   "context": w["context"], "temperature": w["temperature"], "clocks": clocks.stop()}
    del model, engine
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    return out


TIMELINE_KINDS = {10: "add + norm", 11: "add + norm (clusters)", 20: "product", 21: "product + SiLU", 25: "product on CTA pairs",
                  26: "product on CTA pairs + SiLU", 27: "product on CTA pairs + q/k norm, RoPE, cache write", 30: "decode attention",
                  31: "range merge", 32: "prefill attention"}


def timeline_stamps(lib):
    """The records the instrumented kernels left since the last call (csrc/common.cuh, QI_TIMELINE)."""
    import ctypes as C

    class Stamp(C.Structure):
        _fields_ = [("t0", C.c_ulonglong), ("tw", C.c_ulonglong), ("td", C.c_ulonglong), ("t1", C.c_ulonglong),
                    ("kind", C.c_int), ("grid", C.c_int), ("cta", C.c_int), ("sm", C.c_int)]

    cap, out = 1 << 19, []
    for name in ("qi_timeline_norm", "qi_timeline_gemm", "qi_timeline_attention", "qi_timeline_prefill_attention"):
        n, buf = C.c_uint(0), (Stamp * cap)()
        getattr(lib, name)(buf, C.byref(n), 1)
        out += [(s.t0, s.tw, s.td, s.t1, s.kind, s.grid) for s in buf[:min(n.value, cap)]]
    return out


def timeline_launches(stamps):
    """Sorts CTA records into launches: records of one kind and grid size, in the order of their starts, as
    many as the grid has CTAs. Per launch: first start, first wake (the wait for the kernel before it ended),
    first data, first and last end."""
    launches, open_ = [], {}
    for s in sorted(stamps):
        key = (s[4], s[5])
        cur = open_.get(key)
        if cur is None or len(cur) >= s[5]:
            cur = open_[key] = []
            launches.append((key, cur))
        cur.append(s)
    rows = []
    for (kind, grid), recs in launches:
        if len(recs) != grid:
            continue
        wakes, datas = [r[1] for r in recs if r[1]], [r[2] for r in recs if r[2]]
        rows.append(dict(kind=kind, grid=grid, start=min(r[0] for r in recs), wake=min(wakes) if wakes else min(r[0] for r in recs),
                         data=min(datas) if datas else 0, first_end=min(r[3] for r in recs), end=max(r[3] for r in recs)))
    return sorted(rows, key=lambda r: r["wake"])


def timeline_report(bench, batch, prefill=False):
    """Markdown: the kernels of one layer of a decode step (or, `prefill`, of the prefill of one prompt) as they
    ran in their place (microseconds from the first listed kernel's wake), and the means over two steps by kind
    and grid. Needs the kernels built with their time stamps (QUANTINFER_B200_TIMELINE=1, which `--timeline`
    sets before the library is loaded)."""
    import collections

    from quantinfer_b200 import kernels
    from quantinfer_b200.sampling import GenerationConfig

    torch, engine, lib = bench.torch, bench.engine, kernels.library()
    ids = []
    if prefill:
        bench.prefill_ms(runs=1, warm=2)
        timeline_stamps(lib)                               # forget the warm-up
        ms = bench.prefill_ms(runs=1, warm=1)
        what = f"Two prefills of one prompt of {bench.prompt_len} tokens: {ms:.3f} ms each with the stamps in"
    else:
        ids = bench.fill(batch)
        rows = [(GenerationConfig(max_new_tokens=1 << 20), 0)] * batch
        hist = engine.decode_on_device(ids, [1 + i for i in range(batch)], 12, rows, bench.sampler)
        torch.cuda.synchronize()
        timeline_stamps(lib)                               # forget the warm-up
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.decode_on_device(ids, hist[-1].tolist(), 2, rows, bench.sampler)
        b.record()
        torch.cuda.synchronize()
        what = f"Two decode steps, batch {batch}: {a.elapsed_time(b) / 2:.3f} ms a step with the stamps in"
    launches = timeline_launches(timeline_stamps(lib))
    name = lambda r: f"{TIMELINE_KINDS.get(r['kind'], r['kind'])}, {r['grid']} CTAs"
    out = [f"{what}; {len(launches)} launches sorted.", "",
           "One layer from the middle of the second step (us from the first row's wake):", "",
           "| kernel | first CTA starts | wake | first data | first CTA ends | last CTA ends | wake after the kernel before ended | wake to end |",
           "|---|---|---|---|---|---|---|---|"]
    mid = len(launches) // 2 + len(launches) // 8
    first = next((i for i in range(mid, len(launches)) if launches[i]["kind"] in (10, 11)), mid)
    t00, prev_end = launches[first]["wake"], launches[first - 1]["end"] if first else None
    rel = lambda t: f"{(t - t00) / 1e3:.2f}" if t else "-"
    for r in launches[first:first + 9]:
        gap = f"{(r['wake'] - prev_end) / 1e3:.2f}" if prev_end else "-"
        out.append(f"| {name(r)} | {rel(r['start'])} | {rel(r['wake'])} | {rel(r['data'])} | {rel(r['first_end'])} | {rel(r['end'])} | {gap} | {(r['end'] - r['wake']) / 1e3:.2f} |")
        prev_end = r["end"]
    agg, prev_end = collections.OrderedDict(), None
    for r in launches:
        if prev_end is not None:
            g = agg.setdefault(name(r), [0, 0.0, 0.0, 0.0, 0.0])
            g[0] += 1
            g[1] += (r["wake"] - prev_end) / 1e3
            g[2] += (r["end"] - r["wake"]) / 1e3
            g[3] += (r["data"] - r["wake"]) / 1e3 if r["data"] else 0.0
            g[4] += (r["end"] - r["first_end"]) / 1e3
        prev_end = r["end"]
    out += ["", "Means over both steps (us):", "", "| kernel | launches | wake after the kernel before ended | wake to last end | wake to first data | first end to last end |",
            "|---|---|---|---|---|---|"]
    for k, g in agg.items():
        out.append(f"| {k} | {g[0]} | {g[1] / g[0]:.2f} | {g[2] / g[0]:.2f} | {g[3] / g[0]:.2f} | {g[4] / g[0]:.2f} |")
    for rid in ids:
        engine.close(rid)
    return "\n".join(out)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--model", default="8b", choices=sorted(MODELS))
    ap.add_argument("--batch", type=int, default=None, help="headline batch (default: the model's)")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has (named in `config`)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="measure only the headline batch")
    ap.add_argument("--skip-classes", action="store_true", help="no split of the steps by kernel class")
    ap.add_argument("--skip-mixed", action="store_true", help="no scheduler workload")
    ap.add_argument("--mixed-budget", type=int, default=2048, help="token budget of a step of the scheduler workload")
    ap.add_argument("--mixed-chunk", type=int, default=None, help="longest prompt portion of the scheduler workload")
    ap.add_argument("--only", choices=["decode", "prefill", "mixed"], default=None,
                    help="run one part only (for profiler captures of a small case)")
    ap.add_argument("--timeline", action="store_true",
                    help="build the kernels with their time stamps and print where a decode step's time goes, kernel by kernel")
    args = ap.parse_args()
    if args.timeline:
        os.environ["QUANTINFER_B200_TIMELINE"] = "1"      # before the library is built and loaded
        args.only = args.only if args.only == "prefill" else "decode"

    if args.impl == "reference":
        print(json.dumps({"impl": "reference",
                          "unavailable": "aiqubits/quantinfer is a Rust workspace: pip finds no setup.py/pyproject.toml at its root and there is no cargo/rustc offline, so it cannot be installed or run here"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    args.warmup = max(args.warmup, 3)
    entry = MODELS[args.model]
    args.batch = args.batch or entry["batch"]
    if args.only:
        args.skip_points = args.skip_classes = True

    import torch

    from quantinfer_b200 import Model

    torch.cuda.set_device(0)
    if args.only == "mixed":
        print(json.dumps({"only": "mixed", "mixed": mixed_workload(args, entry)}))
        return 0
    peaks_ = hbm_peak, tf_sustained, tf_burst, peak_src = peaks()
    bench = Bench(args, entry)
    a, T = bench.arith, bench.prompt_len
    flops = a["gemm_flops"](T) + a["attn_flops"](T)

    if args.timeline:
        print(timeline_report(bench, args.batch, prefill=args.only == "prefill"))
        return 0
    # the headline first: the K timed decode steps, before anything else has heated the device
    if args.only != "prefill":
        head = bench.decode_rate(args.batch, args.steps, args.warmup, sample_clocks=True)
        step_bytes = a["weight_bytes"] + args.batch * head["ctx_mid"] * a["kv_bytes_per_token"]
        achieved = step_bytes / (head["ms"] * 1e-3) / 1e9
    if args.only == "decode":
        print(json.dumps({"only": "decode", "value": head["rate"], "ms_per_step": head["ms"], "gpu_launches": head["launches"]}))
        return 0
    pre_ms = bench.prefill_ms()
    prefill = {"value": T / pre_ms * 1e3, "tokens": T, "ms": pre_ms, "frac": flops / (pre_ms * 1e-3) / (tf_sustained * 1e12),
               "frac_burst": flops / (pre_ms * 1e-3) / (tf_burst * 1e12), "tflops": flops / (pre_ms * 1e-3) / 1e12}
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "prefill": prefill}))
        return 0
    points = {}
    for bsz in bench.batches[1:]:
        r = bench.decode_rate(bsz, 64, 8)      # their own length: the first steps after the prompts run at the clock the prefill left
        points[f"decode_b{bsz}"] = r["rate"]
        points[f"decode_b{bsz}_frac_hbm"] = round((a["weight_bytes"] + bsz * r["ctx_mid"] * a["kv_bytes_per_token"]) / (r["ms"] * 1e-3) / 1e9 / hbm_peak, 3)

    model = Model.from_engine(bench.engine, max_batch_tokens=T)
    e2e = bench.e2e(model, args.batch)
    for bsz in bench.batches[1:]:
        points[f"e2e_b{bsz}"] = bench.e2e(model, bsz)["value"]
    del model
    classes = None if args.skip_classes else bench.classes(head["ms"], pre_ms, head["ctx_mid"], peaks_)
    engine = bench.engine
    config = {
        "model": entry["name"], "global_batch": args.batch, "seq_len": bench.context, "prompt_len": T,
        "layers": a["L"], "layers_of_config": entry["config"]["num_hidden_layers"], "hidden": a["H"], "heads": a["nq"],
        "kv_heads": a["nkv"], "head_dim": a["d"], "intermediate": a["I"], "vocab": a["V"], "page_size": engine.page_size,
        "parallelism": "1 GPU", "l2": "inputs larger than L2 (weights %.1f GB per step)" % (a["weight_bytes"] / 1e9),
        "peaks": peak_src, "load_s": round(bench.load_s, 1),
    }
    del bench, engine
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    mixed = None if args.skip_mixed else mixed_workload(args, entry)

    line = {
        "metric": "decode tokens/s (%s, random bf16 weights, 1 B200)" % entry["name"],
        "value": head["rate"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, seeded random weights", "impl": "ours",
        "config": config,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak},
        "points": points,
        "e2e": e2e,
        "classes": classes,
        "mixed": mixed,
        "gpu_launches": head["launches"],
        "clocks": head["clocks"],
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
