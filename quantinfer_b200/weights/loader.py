"""Weights by tensor name.

A model states what it needs as `{name: TensorNeed}` (every part contributes
its own names); the loader opens the folder, compares names, shapes and element
classes, and reports everything that does not fit in one error. Tensors are
returned in their stored element type: bfloat16 stays bfloat16, 32-bit stays
32-bit, integer tables become int32. The model moves them to the device and
converts what its compute type needs.

Tensors that the model does not ask for (a buffer some exporter left in the
file; `lm_head.weight` beside a tied configuration, whose head is the embedding
table) do not stop a load: they are skipped and named once on stderr, as the
reference's converter passes unknown names through
(tools/quantinfer-convert/src/convert/gguf.rs:380-381) and builds a tied head
from the table (crates/quantinfer-runtime/src/qwen3/loader.rs:59). They are
still named in the error when something else is wrong, and `strict=True` makes
them an error of their own. `check_finite=True` reads every needed tensor once
more and refuses NaN and infinities by name, which the reference does at decode
time for every element (crates/quantinfer-format/src/safetensors/decode.rs:8-53);
it is off by default because it doubles the load time of a large checkpoint.

The names are those of the checkpoint (`model.layers.N.self_attn.q_proj.weight`
and so on), the same list the reference maps from
(crates/quantinfer-format/src/dense.rs:9-46) and requires
(tools/quantinfer-convert/src/model.rs:245-284); its messages for a missing
tensor and a wrong shape are crates/quantinfer-runtime/src/qwen3/mod.rs:79-84.
The projections keep the checkpoint's [out, in] layout (the reference
transposes them to [in, out] at conversion, dense.rs:80-106; here both GEMM
operands are read along K, so no transpose is needed).
"""

from __future__ import annotations

import sys
from dataclasses import dataclass

import torch

from ..errors import WeightError
from .safetensors_io import SafeTensorsFolder


@dataclass(frozen=True)
class TensorNeed:
    shape: tuple
    kind: str = "matrix"     # "matrix" | "table" (embedding) | "gain" | "int"
    init: str = "normal"     # how random weights fill it: "normal" | "gain" | "zeros"


def check_and_load(source, needs: dict, *, strict: bool = False, check_finite: bool = False, warn=None) -> dict:
    """Returns {name: CPU tensor} for every needed name, or raises one WeightError
    listing missing tensors, unexpected tensors, wrong shapes and wrong element classes.
    Unexpected tensors alone are skipped with one line through `warn` (stderr by default)
    unless `strict`."""
    have = set(source.names())
    want = set(needs)
    missing = sorted(want - have)
    unexpected = sorted(have - want)
    wrong_shape, wrong_type = [], []
    for name in sorted(want & have):
        need = needs[name]
        shape = tuple(source.shape(name))
        if shape != tuple(need.shape):
            wrong_shape.append(f"{name}: has {list(shape)}, expected {list(need.shape)}")
        dt = source.dtype(name)
        is_float = dt in (torch.float32, torch.float16, torch.bfloat16)
        if (need.kind == "int") == is_float:
            wrong_type.append(f"{name}: stored as {dt}, expected {'an integer' if need.kind == 'int' else 'a floating-point'} type")
    if missing or wrong_shape or wrong_type or (strict and unexpected):
        lines = ["the weight files do not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        if wrong_type:
            lines.append(f"  wrong element types ({len(wrong_type)}): " + "; ".join(wrong_type))
        raise WeightError("\n".join(lines))
    if unexpected:
        shown = ", ".join(unexpected[:8]) + (f", ... ({len(unexpected) - 8} more)" if len(unexpected) > 8 else "")
        note = ("the table serves as the head of this tied model; " if "lm_head.weight" in unexpected else "")
        (warn or _warn)(f"warning: {note}{len(unexpected)} tensors that the model does not use were skipped: {shown}")
    out = {}
    non_finite = []
    for name in needs:
        t = source.tensor(name)
        if check_finite and t.is_floating_point() and not bool(torch.isfinite(t).all()):
            bad = int((~torch.isfinite(t)).sum())
            non_finite.append(f"{name} ({bad} of {t.numel()} values)")
        if needs[name].kind == "int":
            if t.dtype != torch.int32:
                t = t.to(torch.int64).to(torch.int32)
        elif t.dtype == torch.float16:
            t = t.to(torch.float32)  # half is not a compute type here; widen exactly
        out[name] = t
    if non_finite:
        raise WeightError("the weight files hold values that are not finite: " + "; ".join(non_finite))
    return out


def _warn(line: str) -> None:
    print(line, file=sys.stderr, flush=True)


def load_folder(folder, needs: dict, *, strict: bool = False, check_finite: bool = False, warn=None) -> dict:
    return check_and_load(SafeTensorsFolder(folder), needs, strict=strict, check_finite=check_finite, warn=warn)
