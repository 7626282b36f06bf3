"""Implementation of `bin/trace_run` (see its header for the protocol)."""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token traces through the engine and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=None, help="positions per cache page (default: the engine's)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from quantinfer_b200.engine import Engine, StepEntry
    from quantinfer_b200.engine.engine import DEFAULT_PAGE_SIZE

    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    engine = Engine.from_folder(args.model, dtype=args.dtype, device=args.device,
                                page_size=args.page_size or DEFAULT_PAGE_SIZE,
                                max_tokens=args.max_tokens, max_requests=8)
    live = set()
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = []
        for e in step.get("entries", []):
            rid = e["id"]
            if rid not in live:
                engine.open(rid)
                live.add(rid)
            entries.append(StepEntry(rid, list(e["tokens"]), list(e.get("want", []))))
        logits = engine.step(entries)
        if logits.shape[0] > 0:
            arr = logits.detach().cpu().numpy().astype("<f4", copy=False)
            arr.tofile(out / f"{step['step']}.f32")
        for rid in step.get("end", []):
            if rid in live:
                engine.close(rid)
                live.discard(rid)
        print(f"done {step['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
