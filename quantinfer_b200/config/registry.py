"""One registry from an architecture's name to its config class.

A model folder's config.json names its class under `architectures`; that name
selects the config class here, and the config class turns the file into a
:class:`ModelSpec` from which the generic model is built. The reference picks
its model by a string match on the architecture name and fails with
"unsupported ... architecture" otherwise (crates/quantinfer/src/cpu/model.rs:74-90;
tools/quantinfer-convert/src/model.rs:24-52).

A config class needs: `from_dict(dict)`, `to_model_spec() -> ModelSpec`, and
`to_dict()` (used when a random-weights folder is written).
"""

from __future__ import annotations

import json
from pathlib import Path

from ..errors import ConfigError

_ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str, config_class: type) -> None:
    _ARCHITECTURES[name] = config_class


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unsupported architecture {name!r}; this engine knows {architectures()}") from None


def load_config(folder):
    """Reads `folder/config.json` (or `folder` itself, if it is a file) and returns the typed
    config its architecture names."""
    path = Path(folder)
    if not path.is_file():
        path = path / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from exc
    return config_from_dict(d)


def config_from_dict(d: dict):
    if not isinstance(d, dict):
        raise ConfigError("config.json must hold a JSON object")
    arch = d.get("architectures")
    if not isinstance(arch, list) or not arch or not isinstance(arch[0], str):
        raise ConfigError("config.json must name the model class under `architectures`")
    for name in arch:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name].from_dict(d)
    return config_class_for(arch[0]).from_dict(d)  # raises with the list of known names


def _register_builtin() -> None:
    from .qwen3 import ARCHITECTURE, Qwen3Config

    register_architecture(ARCHITECTURE, Qwen3Config)


_register_builtin()
