"""A model as data: its layers, the parts of each, and the order in which the layers run.

`ModelSpec` is what an architecture's `build_spec(config)` returns. Nothing in it is specific
to one architecture: layers may differ from one another (each names its own block and parts),
and `schedule` is a list that may run a layer twice or let an entry attend over the pages that
an earlier entry wrote.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..parts.base import PartSpec
from ..weights.loader import TensorSpec


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec          # the arrangement; its params hold the PartSpecs of norms, mixer, feed-forward
    prefix: str              # tensor-name prefix of the layer, e.g. "model.layers.3."


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                       # index into ModelSpec.layers
    reads_cache_of: int | None = None  # index of an earlier schedule entry whose pages this one reads


@dataclass
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position: int
    embedding: str                   # tensor name of the token table [vocab, hidden]
    final_norm: PartSpec
    head: str | None                 # tensor name of the output matrix; None: tied to the embedding
    layers: list[LayerSpec]
    schedule: list[ScheduleEntry] = field(default_factory=list)
    norm_prefix: str = ""
    init_std: float = 0.02
    init_norm_std: float = 0.0
    ignorable_tensors: frozenset = frozenset()

    def __post_init__(self):
        if not self.schedule:
            self.schedule = [ScheduleEntry(i) for i in range(len(self.layers))]
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {index} names layer {entry.layer} of {len(self.layers)}")
            if entry.reads_cache_of is not None and not 0 <= entry.reads_cache_of < index:
                raise ValueError(f"schedule entry {index} must read the cache of an earlier entry")

    def tensor_specs(self) -> list[TensorSpec]:
        """Every checkpoint tensor of the model (built without touching a device)."""
        from .model import assemble

        return assemble(self).tensor_specs()
