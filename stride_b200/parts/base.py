"""Interfaces of the parts a model is put together from, and the part registry.

A part knows its own sizes and constants (from its `PartSpec`) and nothing about
the model it sits in. Five categories exist: "norm", "position", "mixer",
"feed_forward" and "block" (plus "embedding" and "head" at the ends of the model).
A new kind is one class registered under a category:

    @register_part("mixer", "my_kind")
    class MyMixer(Mixer): ...

Life of a part: `__init__(spec, env)`; `tensor_plan()` tells the loader which
checkpoint tensors it needs; `bind(tensors)` receives them (already on the
device); then `forward(...)` is called once per step and schedule entry.

A part may also describe its share of a step once, as operations of the native step
program (`emit(program, ...)`, the counterpart of `forward` over the full-size buffers;
see `kernels/native.py`): when every part of a model does, a step is one native call.
A part without `emit` makes the engine drive the model through `forward`, part by part.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..kernels.native import NotNative
from .spec import PartSpec, TensorPlan

_REGISTRY: dict = {}

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")


def register_part(category: str, kind: str):
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category '{category}' (known: {', '.join(CATEGORIES)})")

    def deco(cls):
        _REGISTRY[(category, kind)] = cls
        return cls
    return deco


def part_class(category: str, kind: str):
    try:
        return _REGISTRY[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise KeyError(f"no {category} part of kind '{kind}' is registered (registered: {', '.join(known)})") from None


@dataclass
class BuildEnv:
    """What a part may need to know of the engine it is built for."""
    device: torch.device
    compute_dtype: torch.dtype      # float32: everything 32-bit; bfloat16: the serving precision
    max_tokens: int                 # most tokens one step brings
    max_positions: int              # longest sequence
    max_logit_rows: int = 0         # most places of one step whose logits are wanted (0: max_tokens)
    max_requests: int = 0           # most requests alive at once (0: unknown)
    decode_chain: bool = False      # steps of decoded tokens only run their layers as one persistent kernel

    def __post_init__(self):
        if self.max_logit_rows <= 0:
            self.max_logit_rows = self.max_tokens

    @property
    def act_dtype(self) -> torch.dtype:
        """dtype of normed activations, queries, attention output, cached keys and values."""
        return self.compute_dtype


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer asks of the cache manager for one schedule entry.

    kind "pages": keys and values per token, `[2, kv_heads, page_size, head_dim]` per page
    and layer; `window` > 0 means only the last `window` tokens are ever read, so older
    pages may be given back. kind "state": `state_shape` elements of `state_dtype` per
    request, zeroed when a request takes its slot.
    """
    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    dtype: torch.dtype = torch.float32
    state_shape: tuple = ()
    state_dtype: torch.dtype = torch.float32


class Part:
    # True if `forward` launches the same kernels with the same arguments for every decode-only step of a
    # given batch size (no host-side branching on positions, no host-to-device copies), so that the step can be
    # recorded once as a CUDA graph and replayed. Parts written with host logic leave it False, and the
    # engine then runs every step directly.
    graph_safe = False

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.spec = spec
        self.env = env

    def tensor_plan(self) -> dict:
        """checkpoint tensor name -> TensorPlan."""
        return {}

    def bind(self, tensors: dict) -> None:
        """Receive the tensors named by `tensor_plan()` (absent optional ones are missing from the dict)."""

    def weight_bytes(self) -> int:
        """Bytes of weights one decode step has to read from this part."""
        return 0

    def kernel_libraries(self) -> set:
        """Names (keys of `kernels.build.SOURCES`) of the kernel libraries this part will most likely call, so that
        the engine can compile them side by side before the first step. A hint only: a library that is not
        listed is compiled when it is first called."""
        return set()

    def emit(self, program, *args) -> None:
        """The part's `forward` as operations appended to the native step program; the arguments are those of
        `forward` without the step's context, tensors being the full-size buffers. Optional."""
        raise NotNative(f"{type(self).__name__} has no native form")


class Norm(Part):
    def forward(self, ctx, stream, out: torch.Tensor) -> None:
        """out = norm(stream), where `stream` is the ResidualStream (pending partial sums are folded in)."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Holds whatever table its mixer's kernels read; built once for `env.max_positions`.

    The attention mixer of this package rotates queries and keys in pairs (d, d + rotary_dim / 2) of a head (the
    "rotate-half" pairing) and reads two attributes of its position part after `bind`:
        cos_sin     float32 [positions, rotary_dim / 2, 2] on the device: cos and sin of every position and pair
        rotary_dim  how many leading elements of a head are rotated (even, <= head_dim; 0: none)
    A position part that offers these (whatever its angles are: another base, another scaling, learned) works with it
    unchanged. An encoding of another nature (a bias on the scores, interleaved pairs, a norm of q and k) needs a mixer of
    its own; the attention mixer refuses a position part without the two attributes with a message that says so."""
    cos_sin = None
    rotary_dim = None


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, ctx, x: torch.Tensor, stream, cache) -> None:
        """Mix tokens: read the normed activations `x` [n, hidden], add the result to `stream`."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x: torch.Tensor, stream) -> None:
        """Per-token transform: read `x` [n, hidden], add the result to `stream`."""
        raise NotImplementedError


class Block(Part):
    """An arrangement of parts around the residual stream. `ROLES` names the parts a block of this kind is made of
    and the registry category of each; the model builds them from the layer's `LayerSpec.parts` and hands them over
    as `self.parts[role]` (also reachable as attributes: `self.mixer`). A new arrangement (other norms, one norm for two
    branches, no feed-forward) is a subclass with its own ROLES, `forward` and, if it has one, `emit`."""

    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, spec, env, parts: dict):
        super().__init__(spec, env)
        missing = [r for r in self.ROLES if r not in parts]
        if missing:
            raise ValueError(f"a '{getattr(spec, 'block', type(self).__name__)}' block needs the parts {', '.join(self.ROLES)}; missing: {', '.join(missing)}")
        self.parts = dict(parts)

    def __getattr__(self, name):
        parts = self.__dict__.get("parts")
        if parts is not None and name in parts:
            return parts[name]
        raise AttributeError(name)

    def all_parts(self):
        return tuple(self.parts[r] for r in self.ROLES)

    def cache_need(self):
        """What this block's layer asks of the cache manager: by default what its part in the role "mixer" asks."""
        mixer = self.parts.get("mixer")
        return mixer.cache_need() if mixer is not None else None

    def tensor_plan(self) -> dict:
        plan = {}
        for p in self.all_parts():
            plan.update(p.tensor_plan())
        return plan

    def bind(self, tensors: dict) -> None:
        for p in self.all_parts():
            p.bind(tensors)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.all_parts())

    def kernel_libraries(self) -> set:
        return set().union(*(p.kernel_libraries() for p in self.all_parts()))

    @property
    def all_graph_safe(self) -> bool:
        return self.graph_safe and all(p.graph_safe for p in self.all_parts())

    def forward(self, ctx, stream, cache) -> None:
        raise NotImplementedError

    def emit(self, program, cache) -> None:
        raise NotNative(f"{type(self).__name__} has no native form")
