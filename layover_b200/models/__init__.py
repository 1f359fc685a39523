"""Building a model from a folder, or from a configuration and a seed."""

from __future__ import annotations

from pathlib import Path

import torch

from ..config.base import load_config, resolve_architecture
from ..csrc import build as _build
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensors
from . import qwen3  # noqa: F401  (registers the architecture)
from .model import Model, assemble
from .runtime import make_runtime
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, ScheduleEntry

DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32}


def as_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    try:
        return DTYPES[dtype]
    except KeyError:
        raise ValueError(f"unknown dtype {dtype!r}; choose from {sorted(DTYPES)}") from None


def spec_for_config(config) -> ModelSpec:
    """The model spec of a typed configuration, through the registry."""
    arch = resolve_architecture({"architectures": [config.architecture], "model_type": config.model_type})
    return arch.build_spec(config)


def _head_sizes(value) -> set[int]:
    """Every `head_dim` found in a tree of part specifications."""
    found: set[int] = set()
    if isinstance(value, PartSpec):
        found |= _head_sizes(value.params)
    elif isinstance(value, dict):
        for key, item in value.items():
            if key == "head_dim" and isinstance(item, int):
                found.add(item)
            else:
                found |= _head_sizes(item)
    elif isinstance(value, (list, tuple)):
        for item in value:
            found |= _head_sizes(item)
    return found


def _build_for(spec: ModelSpec, runtime) -> None:
    """Compile what this model needs before its first step: the run's kernel libraries, without the
    tensor-core attention when no layer has the head size it takes (it would still be compiled at
    first use)."""
    names = list(runtime.kernel_libraries)
    if "attention_tcgen05" in names and 128 not in _head_sizes([layer.block for layer in spec.layers]):
        names.remove("attention_tcgen05")
    _build.ensure_built(names)


def _finish(spec: ModelSpec, config, tensors, dtype, device) -> Model:
    runtime = make_runtime(dtype, device)
    _build_for(spec, runtime)
    return assemble(spec, config).bind(tensors, runtime)


def load_model(name_or_path: str | Path, device: torch.device | str = "cuda", dtype=torch.bfloat16) -> Model:
    """The model of a folder with config.json and *.safetensors (layover/weights.py:23-50); the
    model class is the one config.json names."""
    dtype, device = as_dtype(dtype), torch.device(device)
    arch, config = load_config(name_or_path)
    spec = arch.build_spec(config)
    runtime = make_runtime(dtype, device)       # refuses a CPU before anything is read
    _build_for(spec, runtime)
    model = assemble(spec, config)
    tensors = load_tensors(name_or_path, model.tensor_specs(), dtype, device, set(spec.ignorable_tensors))
    return model.bind(tensors, runtime)


def random_model(config, seed: int = 0, device: torch.device | str = "cuda", dtype=torch.bfloat16,
                 std: float = 0.02, norm_std: float = 0.0) -> Model:
    """A model with seeded random weights made on the device, without touching the disk."""
    dtype, device = as_dtype(dtype), torch.device(device)
    spec = spec_for_config(config)
    runtime = make_runtime(dtype, device)
    _build_for(spec, runtime)
    model = assemble(spec, config)
    tensors = random_tensors(model.tensor_specs(), seed, dtype, device, std, norm_std)
    return model.bind(tensors, runtime)


__all__ = ["Model", "ModelSpec", "LayerSpec", "ScheduleEntry", "assemble", "load_model", "random_model",
           "spec_for_config", "make_runtime", "as_dtype"]
