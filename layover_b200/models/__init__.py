"""Building a model from a folder, or from a configuration and a seed."""

from __future__ import annotations

from pathlib import Path

import torch

from ..config.base import load_config, resolve_architecture
from ..csrc import build as _kernels
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensors
from . import qwen3  # noqa: F401  (registers the architecture)
from .model import Model, assemble
from .runtime import make_runtime
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


def _build(model: Model, dtype: torch.dtype, runtime) -> None:
    """Compile what this model needs before its first step: what its parts and the run's matrix
    product name, and nothing else (a model without the head size the tcgen05 attention takes does
    not wait for that library)."""
    _kernels.ensure_built(model.kernel_libraries(dtype, runtime))


def load_model(name_or_path: str | Path, device: torch.device | str = "cuda", dtype=torch.bfloat16) -> Model:
    """The model of a folder with config.json and *.safetensors (layover/weights.py:23-50); the
    model class is the one config.json names."""
    dtype, device = as_dtype(dtype), torch.device(device)
    arch, config = load_config(name_or_path)
    spec = arch.build_spec(config)
    runtime = make_runtime(dtype, device)       # refuses a CPU before anything is read
    model = assemble(spec, config)
    _build(model, dtype, runtime)
    tensors = load_tensors(name_or_path, model.tensor_specs(), dtype, device, set(spec.ignorable_tensors))
    return model.bind(tensors, runtime)


def random_model(config, seed: int = 0, device: torch.device | str = "cuda", dtype=torch.bfloat16,
                 std: float = 0.02, norm_std: float = 0.0) -> Model:
    """A model with seeded random weights made on the device, without touching the disk."""
    dtype, device = as_dtype(dtype), torch.device(device)
    spec = spec_for_config(config)
    runtime = make_runtime(dtype, device)
    model = assemble(spec, config)
    _build(model, dtype, runtime)
    tensors = random_tensors(model.tensor_specs(), seed, dtype, device, std, norm_std)
    return model.bind(tensors, runtime)


__all__ = ["Model", "ModelSpec", "LayerSpec", "ScheduleEntry", "assemble", "load_model", "random_model",
           "spec_for_config", "make_runtime", "as_dtype"]
