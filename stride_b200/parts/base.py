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
    """Holds whatever table its mixer's kernels read; built once for `env.max_positions`."""


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
    """An arrangement of a mixer, a feed-forward and their norms around the residual stream."""

    def __init__(self, spec, env, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm):
        super().__init__(spec, env)
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def tensor_plan(self) -> dict:
        plan = {}
        for p in self.parts():
            plan.update(p.tensor_plan())
        return plan

    def bind(self, tensors: dict) -> None:
        for p in self.parts():
            p.bind(tensors)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts())

    def kernel_libraries(self) -> set:
        return set().union(*(p.kernel_libraries() for p in self.parts()))

    @property
    def all_graph_safe(self) -> bool:
        return self.graph_safe and all(p.graph_safe for p in self.parts())

    def forward(self, ctx, stream, cache) -> None:
        raise NotImplementedError

    def emit(self, program, cache) -> None:
        raise NotNative(f"{type(self).__name__} has no native form")
