"""What every architecture's configuration offers, and the registry from a name to a model.

A configuration class reads its own `config.json` keys (`from_hf_dict`) and writes them back
(`to_hf_dict`). The registry maps the name found in `config.json` (`architectures[0]`, else
`model_type`) to an `Architecture`: the configuration class and a function that turns a
configuration into a `ModelSpec` (the list of layers, their parts and the order they run in).
The reference has one hard-wired `model_type` check (layover/config.py:36-37); here a new
architecture is one `register_architecture` call.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

DTYPE_BYTES = {"bf16": 2, "bfloat16": 2, "fp32": 4, "float32": 4}


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: str
    config_class: type
    build_spec: Callable[[Any], Any]


_BY_NAME: dict[str, Architecture] = {}
_BY_MODEL_TYPE: dict[str, Architecture] = {}


def register_architecture(name: str, model_type: str, config_class: type, build_spec: Callable) -> Architecture:
    """Make `name` (as in config.json's `architectures`) and `model_type` resolve to this model."""
    arch = Architecture(name, model_type, config_class, build_spec)
    _BY_NAME[name] = arch
    _BY_MODEL_TYPE[model_type] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _BY_NAME.pop(name, None)
    if arch is not None and _BY_MODEL_TYPE.get(arch.model_type) is arch:
        del _BY_MODEL_TYPE[arch.model_type]


def supported_architectures() -> list[str]:
    return sorted(_BY_NAME)


def resolve_architecture(raw: dict) -> Architecture:
    """The architecture that a config.json names, or a ValueError listing what is supported."""
    names = raw.get("architectures") or []
    for name in names:
        if name in _BY_NAME:
            return _BY_NAME[name]
    model_type = raw.get("model_type")
    if not names and model_type in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[model_type]
    if not names and model_type is None and len(_BY_NAME) == 1:
        # the reference assumes its one architecture when model_type is absent (layover/config.py:36)
        return next(iter(_BY_NAME.values()))
    raise ValueError(
        f"unsupported architecture {names or model_type!r}; supported: {supported_architectures()}"
    )


def read_config_json(folder: str | Path) -> dict:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {Path(folder)}")
    return json.loads(path.read_text())


def load_config(folder: str | Path):
    """(architecture, typed configuration) of a model folder."""
    raw = read_config_json(folder)
    arch = resolve_architecture(raw)
    return arch, arch.config_class.from_hf_dict(raw)
