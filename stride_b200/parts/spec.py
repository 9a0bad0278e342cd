"""Data that describes a model: which parts each layer has, with what sizes, and
the order in which layers run. A specification holds no tensors and no code; the
architecture registry makes one from a config.json, and `parts.model.build_model`
turns it into parts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: `kind` names its class in the part registry, `params` holds its sizes
    and constants, `tensors` maps the part's own role names to checkpoint tensor names."""
    kind: str
    params: dict = field(default_factory=dict)
    tensors: dict = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer, a feed-forward and their norms."""
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    block: str = "prenorm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One call of a layer. `cache_of` is the index of an earlier schedule entry whose
    cache this call reads instead of writing one of its own."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    eos_token_ids: tuple = ()


@dataclass(frozen=True)
class TensorPlan:
    """What a part expects of one checkpoint tensor."""
    shape: tuple
    optional: bool = False
    integer: bool = False
