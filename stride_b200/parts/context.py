"""What one step hands to the parts: the batch on the device, the residual stream,
and buffers that live as long as the engine."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


class Workspace:
    """Named device buffers, allocated once for the largest step and reused by every
    step, so that a step allocates nothing and buffer addresses stay fixed."""

    def __init__(self, device, max_tokens: int):
        self.device = torch.device(device)
        self.max_tokens = max_tokens
        self._buffers: dict = {}
        self.generation = 0          # bumped whenever a buffer that `grow` handed out moves
        self._iota = None

    def get(self, name: str, rows: int, tail: tuple, dtype: torch.dtype) -> torch.Tensor:
        """A `[rows, *tail]` view of the buffer `name` (rows <= max_tokens)."""
        if rows > self.max_tokens:
            raise ValueError(f"a step of {rows} tokens exceeds the engine's max_tokens {self.max_tokens}")
        key = (name, tuple(tail), dtype)
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.zeros((self.max_tokens, *tail), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:rows]

    def raw(self, name: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.zeros(tuple(shape), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf

    def grow(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A flat buffer of at least `numel` elements; reallocated (with headroom) when too small.
        Its address may change when it grows, so size it before a CUDA graph is captured."""
        key = (name, "grow", dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < numel:
            if buf is not None:
                self.generation += 1
            buf = torch.zeros(max(numel, 1) * 3 // 2 + 16, dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf

    def iota(self, n: int) -> torch.Tensor:
        """[0, 1, ..., n-1] int32 on the device (a view of one cached tensor)."""
        if self._iota is None or self._iota.numel() < n:
            self._iota = torch.arange(max(n, self.max_tokens), dtype=torch.int32, device=self.device)
        return self._iota[:n]

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


class ResidualStream:
    """The float32 residual `h` [n, hidden] plus, possibly, partial sums [S, n, hidden] that a
    split-K contraction left behind. The next reader (a norm, or the row gather before the
    head) adds them to `h` in ascending order of S, so the order of the sum is fixed."""

    def __init__(self, h: torch.Tensor):
        self.h = h
        self.pending: Optional[torch.Tensor] = None

    def take_pending(self) -> Optional[torch.Tensor]:
        p, self.pending = self.pending, None
        return p

    def set_pending(self, partials: torch.Tensor) -> None:
        if self.pending is not None:
            self.fold()
        self.pending = partials

    def fold(self) -> None:
        """Add pending partial sums now (used by parts that want `h` itself)."""
        p = self.take_pending()
        if p is not None:      # h + (p0 + p1 + ...), the order of the kernels that fold partials themselves
            total = p[0]
            for s in range(1, p.shape[0]):
                total = total + p[s]
            self.h.add_(total)

    def add_(self, update: torch.Tensor) -> None:
        """h += update, for parts that compute their output as a separate tensor."""
        self.fold()
        self.h.add_(update.to(self.h.dtype))


@dataclass
class StepContext:
    n: int                                   # tokens in this step
    token_ids: torch.Tensor                  # [n] int32, device
    positions: torch.Tensor                  # [n] int32
    slots: torch.Tensor                      # [n] int32: the request slot of every token
    workspace: Workspace
    compute_dtype: torch.dtype
    # One record per request of the step, rows of a request being contiguous and ascending:
    entry_slots: list = field(default_factory=list)       # host ints
    entry_first_row: list = field(default_factory=list)
    entry_length: list = field(default_factory=list)
    entry_first_pos: list = field(default_factory=list)
    entry_meta: Optional[torch.Tensor] = None              # [4, E] int32 on the device: slot, first row, length, first position
    upload_ints: Optional[object] = None                   # callable(np.ndarray int32) -> device tensor, valid for this step
    sampled: Optional[torch.Tensor] = None                 # [slots] int32: each request's last sampled token (a token id of -1 reads it)
    shared: dict = field(default_factory=dict)             # what parts compute once per step and share between layers
    # Set for a step that is recorded into a CUDA graph: every entry is one decoded token, the batch is
    # padded to a fixed size, and no key lies at or beyond `static_keys`. Parts must then launch the same
    # kernels with the same arguments whatever the positions are, and must not copy from the host.
    static_keys: int = 0

    @property
    def act_dtype(self) -> torch.dtype:
        return self.compute_dtype

    @property
    def decode_only(self) -> bool:
        return all(l == 1 for l in self.entry_length)
