"""Weights by tensor name.

A model states what it needs as `{name: TensorNeed}` (every part contributes
its own names); the loader opens the folder, compares names, shapes and element
classes, and reports everything that does not fit in one error. Tensors are
returned in their stored element type: bfloat16 stays bfloat16, 32-bit stays
32-bit, integer tables become int32. The model moves them to the device and
converts what its compute type needs.

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

from dataclasses import dataclass

import torch

from ..errors import WeightError
from .safetensors_io import SafeTensorsFolder


@dataclass(frozen=True)
class TensorNeed:
    shape: tuple
    kind: str = "matrix"     # "matrix" | "table" (embedding) | "gain" | "int"
    init: str = "normal"     # how random weights fill it: "normal" | "gain" | "zeros"


def check_and_load(source, needs: dict) -> dict:
    """Returns {name: CPU tensor} for every needed name, or raises one WeightError
    listing missing tensors, unexpected tensors, wrong shapes and wrong element classes."""
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
    if missing or unexpected or wrong_shape or wrong_type:
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
    out = {}
    for name in needs:
        t = source.tensor(name)
        if needs[name].kind == "int":
            if t.dtype != torch.int32:
                t = t.to(torch.int64).to(torch.int32)
        elif t.dtype == torch.float16:
            t = t.to(torch.float32)  # half is not a compute type here; widen exactly
        out[name] = t
    return out


def load_folder(folder, needs: dict) -> dict:
    return check_and_load(SafeTensorsFolder(folder), needs)
