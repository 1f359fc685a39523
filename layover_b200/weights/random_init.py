"""Seeded random weights: in memory for a run, or written as a model folder.

The reference has no such mode; its tests seed torch and take the layers' default
initialisation (tests/test_hot_path.py:23-26). Here every tensor is drawn from its own
generator, seeded by the run's seed and the tensor's name, so a tensor's values do not depend
on which other tensors exist or in which order they are made: matrices ~ N(0, std), norm
weights 1 + N(0, norm_std).
"""

from __future__ import annotations

import json
import zlib
from pathlib import Path

import torch

from .loader import TensorSpec, target_dtype
from .safetensors_io import save_safetensors


def _generator(seed: int, name: str, device) -> torch.Generator:
    gen = torch.Generator(device=device)
    gen.manual_seed((int(seed) * 0x9E3779B1 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
    return gen


def random_tensor(spec: TensorSpec, seed: int, std: float, norm_std: float, device="cpu") -> torch.Tensor:
    """One tensor in 32-bit floats (int32 for integer tables)."""
    gen = _generator(seed, spec.name, device)
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=torch.float32, device=device)
    noise = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
    if spec.init == "ones":
        return 1.0 + norm_std * noise
    return std * noise


def random_tensors(specs: list[TensorSpec], seed: int, run_dtype: torch.dtype, device, std: float = 0.02,
                   norm_std: float = 0.0) -> dict[str, torch.Tensor]:
    """All wanted tensors made on `device`, converted as a loaded checkpoint would be."""
    out = {}
    for spec in specs:
        t = random_tensor(spec, seed, std, norm_std, device)
        if spec.kind == "vector":
            t = t.to(run_dtype)             # rounded as a loaded checkpoint's would be
        out[spec.name] = t.to(target_dtype(spec, t.dtype, run_dtype)).contiguous()
    return out


def write_model_folder(config, folder: str | Path, seed: int = 0, std: float = 0.02, norm_std: float = 0.0,
                       store_dtype: torch.dtype = torch.bfloat16, specs: list[TensorSpec] | None = None) -> Path:
    """Write config.json and model.safetensors for a configuration and a seed.

    Floating tensors are stored in `store_dtype` (bfloat16 by default, which a float32 run reads
    exactly); integer tables as int32; "keep32" tensors as float32."""
    from ..models import spec_for_config

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    if specs is None:
        specs = spec_for_config(config).tensor_specs()
    tensors = {}
    for spec in specs:
        t = random_tensor(spec, seed, std, norm_std, "cpu")
        if spec.kind == "matrix" or spec.kind == "vector":
            t = t.to(store_dtype)
        tensors[spec.name] = t
    save_safetensors(tensors, folder / "model.safetensors", {"format": "pt", "seed": seed})
    (folder / "config.json").write_text(json.dumps(config.to_hf_dict(), indent=1))
    return folder
