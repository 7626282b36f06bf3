"""Random weights from a configuration and a seed.

`write_model_folder` writes `config.json` and `model.safetensors` so that the
result loads like any checkpoint. The reference has no random-weight mode for
models (only constant and arithmetic fixtures,
crates/quantinfer-test-support/src/lib.rs:29-41); the distributions are this
engine's: matrices and the embedding table N(0, 0.02), norm gains
1 + U(-0.1, 0.1). Tensor i (in the order the model lists its needs) is drawn
from a generator seeded with seed * 1000003 + i, so a tensor's values do not
depend on the others.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from .loader import TensorNeed
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
GAIN_SPREAD = 0.1


def random_tensor(need: TensorNeed, seed: int, index: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1000003 + index) % (1 << 63))
    if need.kind == "int":
        return torch.zeros(need.shape, dtype=torch.int32, device=device)
    if need.init == "gain":
        u = torch.rand(need.shape, generator=g, dtype=torch.float32, device=device)
        return 1.0 + (u * 2.0 - 1.0) * GAIN_SPREAD  # gains stay 32-bit
    if need.init == "zeros":
        return torch.zeros(need.shape, dtype=dtype, device=device)
    t = torch.randn(need.shape, generator=g, dtype=torch.float32, device=device) * MATRIX_STD
    return t.to(dtype)


def random_tensors(needs: dict, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu") -> dict:
    return {name: random_tensor(need, seed, i, dtype, device) for i, (name, need) in enumerate(needs.items())}


def write_model_folder(folder, config, seed: int, dtype: torch.dtype = torch.bfloat16) -> Path:
    """Writes config.json and model.safetensors for `config` (a typed config of a
    registered architecture). Matrices are stored in `dtype`, gains in float32."""
    from ..engine.model import tensor_needs_of_spec

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    needs = tensor_needs_of_spec(config.to_model_spec())
    d = config.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[dtype]
    (folder / "config.json").write_text(json.dumps(d, indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", random_tensors(needs, seed, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
