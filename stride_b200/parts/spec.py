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


class LayerSpec:
    """One layer: a block kind (the arrangement, a class registered under the category "block") and the parts it
    arranges, by role name. Which roles there are, and of which category each is, is the block class's own business
    (`Block.ROLES`): the pre-norm block has `mixer_norm`, `mixer`, `feed_forward_norm` and `feed_forward`; a block
    with other norms, one norm for two branches, or no feed-forward is another `Block` class with other roles.

        LayerSpec("prenorm", mixer=PartSpec(...), feed_forward=PartSpec(...), mixer_norm=..., feed_forward_norm=...)
        LayerSpec("my_block", {"attn": PartSpec(...), "norm": PartSpec(...)})

    The four roles of the pre-norm block may also be given in that order (mixer, feed_forward, mixer_norm,
    feed_forward_norm) with the block kind last, which is how this class was first written."""

    _ORDER = ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm")

    def __init__(self, *args, block: str = None, parts: dict = None, **named):
        args = list(args)
        kind = block
        if args and isinstance(args[0], str):
            kind = args.pop(0)
        if args and isinstance(args[0], dict):
            parts = dict(args.pop(0), **(parts or {}))
        roles = dict(parts or {})
        if len(args) > len(self._ORDER) + 1:
            raise TypeError("LayerSpec takes a block kind, a dict of parts, or the four parts of a pre-norm block")
        for name, value in zip(self._ORDER, args):
            roles[name] = value
        if len(args) == len(self._ORDER) + 1:
            kind = args[-1]
        roles.update(named)
        for name, value in roles.items():
            if not isinstance(value, PartSpec):
                raise TypeError(f"LayerSpec: role '{name}' is not a PartSpec")
        object.__setattr__(self, "block", kind or "prenorm")
        object.__setattr__(self, "parts", roles)

    def __getattr__(self, name):
        try:
            return self.__dict__["parts"][name]
        except KeyError:
            raise AttributeError(f"this layer has no part in the role '{name}' (roles: {', '.join(self.__dict__.get('parts', {}))})") from None

    def __setattr__(self, name, value):
        raise AttributeError("a LayerSpec is not changed after it is made")

    def __eq__(self, other):
        return isinstance(other, LayerSpec) and self.block == other.block and self.parts == other.parts

    def __hash__(self):
        return hash((self.block, tuple(sorted(self.parts))))

    def __repr__(self):
        return f"LayerSpec({self.block!r}, {self.parts!r})"


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
