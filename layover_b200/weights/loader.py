"""Load a model folder's tensors by name into the tensors that the model's parts ask for.

Every part lists the tensors it wants as `TensorSpec`s (name, shape, how it is kept). The
loader reads all `*.safetensors` files of the folder in name order (layover/weights.py:27-35),
compares names and shapes with that list and raises ONE error that names every missing
tensor, every unexpected tensor and every wrong shape (the reference stops at the names,
layover/weights.py:38-41). How a tensor is kept:

  "matrix"  an operand of a matrix product: the run's dtype (bfloat16 for serving, float32 for
            the true 32-bit path); floating tensors are cast once at load (layover/weights.py:35)
  "vector"  a small per-channel parameter (norm weights): rounded to the run's dtype like every
            floating tensor (layover/weights.py:35 casts them all), then kept as float32 on the
            device, which holds any bfloat16 value exactly and is what the kernels read
  "keep32"  a tensor that must stay in 32-bit whatever the run's dtype is
  "int"     an integer table: int32
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import torch

from .safetensors_io import SafetensorsFile

KINDS = ("matrix", "vector", "keep32", "int")


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"          # "normal": N(0, std); "ones": 1 + N(0, norm_std); "zeros"
    optional_alias: str | None = None  # stored name that may stand in (a tied head reads the embedding)

    def __post_init__(self):
        if self.kind not in KINDS:
            raise ValueError(f"tensor {self.name!r}: unknown kind {self.kind!r}")


class CheckpointMismatch(ValueError):
    """The folder's tensors are not the ones the model needs."""


def resolve_checkpoint(name_or_path: str | Path) -> Path:
    """The model folder. Only local folders: there is no download path (layover/weights.py:14-20)."""
    path = Path(name_or_path)
    if not path.is_dir():
        raise FileNotFoundError(f"model folder {path} does not exist (only local folders are loaded)")
    return path


def open_checkpoint(folder: Path) -> dict[str, tuple[SafetensorsFile, str]]:
    files = sorted(folder.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files in {folder}")
    found: dict[str, tuple[SafetensorsFile, str]] = {}
    for path in files:
        handle = SafetensorsFile(path)
        for name in handle.names():
            found[name] = (handle, name)
    return found


def target_dtype(spec: TensorSpec, stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if spec.kind == "int":
        return torch.int32
    if spec.kind in ("vector", "keep32"):
        return torch.float32
    return run_dtype


def check_tensors(specs: list[TensorSpec], stored_shapes: dict[str, tuple[int, ...]],
                  ignorable: set[str] = frozenset()) -> None:
    """Raise one CheckpointMismatch listing missing, unexpected and misshapen tensors."""
    wanted = {s.name: s for s in specs}
    missing = sorted(n for n in wanted if n not in stored_shapes)
    unexpected = sorted(n for n in stored_shapes if n not in wanted and n not in ignorable)
    wrong = sorted(
        (n, tuple(wanted[n].shape), tuple(stored_shapes[n]))
        for n in wanted if n in stored_shapes and tuple(stored_shapes[n]) != tuple(wanted[n].shape)
    )
    if not (missing or unexpected or wrong):
        return
    lines = ["checkpoint mismatch:"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): "
                     + ", ".join(f"{n} expected {list(e)} got {list(g)}" for n, e, g in wrong))
    error = CheckpointMismatch("\n".join(lines))
    error.missing, error.unexpected, error.wrong_shape = missing, unexpected, wrong
    raise error


def load_tensors(folder: str | Path, specs: list[TensorSpec], run_dtype: torch.dtype, device: torch.device | str,
                 ignorable: set[str] = frozenset()) -> dict[str, torch.Tensor]:
    """The wanted tensors by name, on `device`, converted as their kind says."""
    root = resolve_checkpoint(folder)
    found = open_checkpoint(root)
    check_tensors(specs, {name: handle.shape(stored) for name, (handle, stored) in found.items()}, ignorable)
    out: dict[str, torch.Tensor] = {}
    for spec in specs:
        handle, stored = found[spec.name]
        host = handle.tensor(stored)
        if spec.kind == "int" and host.is_floating_point():
            raise CheckpointMismatch(f"checkpoint mismatch: {spec.name} must be an integer table, is {host.dtype}")
        if spec.kind != "int" and not host.is_floating_point():
            raise CheckpointMismatch(f"checkpoint mismatch: {spec.name} must be floating point, is {host.dtype}")
        if spec.kind == "vector":
            host = host.to(run_dtype)       # the value the reference's cast leaves, whatever the file stores
        out[spec.name] = host.to(device=device, dtype=target_dtype(spec, host.dtype, run_dtype)).contiguous()
    return out
