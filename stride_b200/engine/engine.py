"""The engine: a model on one GPU, its cache, and ONE step function.

`Engine.step(entries)` takes a batch of (request slot, its next tokens, the places
among them whose logits are wanted): portions of prompts beside single decoded
tokens, cut anywhere. It runs exactly those tokens, as one batch, against the cache
that earlier steps left, appends their keys and values, and returns the logits at
the wanted places. Who decides what goes into a step (the scheduler, the replay
tool) also asks the cache manager for pages (`engine.cache.ensure`) beforehand.

Counterpart in arhaamatiq/stride: Engine::step over StepRow{slot,pos,token,mode}
(src/engine.h:17-54, src/engine.cpp:105-142). Rows of one request are contiguous and
ascending here, which is what the scheduler there produces too.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..config import resolve_architecture
from ..kernels.build import build_all
from ..parts import BuildEnv, DecoderModel, StepContext, Workspace
from ..weights.loader import check_plan, load_weights


class EngineError(RuntimeError):
    pass


@dataclass
class EngineOptions:
    """Names follow arhaamatiq/stride's EngineOptions (src/engine.h:24-38) where it has them."""
    dtype: str = "bfloat16"            # "bfloat16": serving precision; "float32": everything in true 32-bit
    max_rows: int = 256                # most tokens one step brings (the scheduler's token budget)
    max_full_rows: int = 32            # most places of one step whose logits are returned
    max_slots: int = 256               # most requests alive at once
    kv_bytes: int = 1 << 30            # size of the cache pool in bytes ...
    kv_pages: int = 0                  # ... or in pages per group (overrides kv_bytes)
    page_size: int = 64                # tokens per page
    max_context: int = 0               # longest sequence (0: config.json's max_position_embeddings)
    kv_shuffle_seed: int = 0           # tests: hand out pages in random order
    cuda_graphs: bool = True           # replay decode-only steps from CUDA graphs (one per batch and context bucket)
    device: str = "cuda:0"


@dataclass
class StepEntry:
    slot: int
    first_pos: int                     # position of tokens[0] in its sequence
    tokens: list
    want: list = field(default_factory=list)   # indices into `tokens` whose logits are wanted


_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


class Engine:
    def __init__(self, model_dir=None, options: Optional[EngineOptions] = None, *, config: Optional[dict] = None,
                 tensors: Optional[dict] = None):
        """Load `model_dir` (config.json + model.safetensors), or take `config` and `tensors` directly."""
        self.options = o = options or EngineOptions()
        if o.dtype not in _DTYPES:
            raise EngineError(f"dtype '{o.dtype}' is not supported (float32 or bfloat16)")
        self.device = torch.device(o.device)
        if self.device.type != "cuda":
            raise EngineError("stride_b200 runs on a CUDA device only; there is no CPU path")
        if not torch.cuda.is_available():
            raise EngineError("no CUDA device is available; stride_b200 has no CPU path")
        torch.cuda.set_device(self.device)
        if config is None:
            if model_dir is None:
                raise EngineError("give a model folder or a config")
            cfg_path = Path(model_dir) / "config.json"
            if not cfg_path.exists():
                raise EngineError(f"cannot open config.json in {model_dir}")
            config = json.loads(cfg_path.read_text())
        self.config_dict = config
        self.architecture = resolve_architecture(config)
        self.config = self.architecture.parse_config(config)
        self.spec = self.architecture.model_spec(self.config)
        self.max_context = o.max_context or self.spec.max_positions
        self.compute_dtype = _DTYPES[o.dtype]
        env = BuildEnv(device=self.device, compute_dtype=self.compute_dtype, max_tokens=o.max_rows,
                       max_positions=self.max_context, max_logit_rows=min(o.max_full_rows, o.max_rows),
                       max_requests=o.max_slots)
        self.env = env
        self.model = DecoderModel(self.spec, env)
        libraries = self.model.kernel_libraries()
        build_all(sorted(libraries))      # what this model needs, compiled side by side if missing
        # the word into which the tensor-core kernels' bounded waits report; the sampling kernels pass it on to the host
        self._status_device = None
        if self.device.type == "cuda" and libraries & {"gemm_tc", "attention_tc5"}:
            from ..kernels import ops
            self._status_device = ops.shared_status_word(libraries | {"sampling"})
        plan = self.model.tensor_plan()
        if tensors is None:
            tensors = load_weights(model_dir, plan, self.device)
        else:
            check_plan(plan, {n: tuple(t.shape) for n, t in tensors.items()}, "the given tensors")
            tensors = {n: t.to(self.device) for n, t in tensors.items()}
        self.model.bind(tensors)
        self.cache = CacheManager(self.model.cache_needs(), device=self.device, max_slots=o.max_slots,
                                  max_context=self.max_context, page_size=o.page_size,
                                  num_pages=o.kv_pages or None, cache_bytes=o.kv_bytes,
                                  shuffle_seed=o.kv_shuffle_seed)
        self.caches = [self.cache.layer_cache(i) for i in range(len(self.spec.schedule))]
        self.workspace = Workspace(self.device, o.max_rows)
        # One pinned staging buffer and one device buffer for all integer inputs of a step:
        # tokens, positions, slots, logit rows (max_rows each), entry records (4 x max_rows), and the slot of every logit row.
        self._ints = 9 * o.max_rows
        self._staging = torch.empty(self._ints, dtype=torch.int32, pin_memory=True)
        self._staging_np = self._staging.numpy()
        self._device_ints = torch.zeros(self._ints, dtype=torch.int32, device=self.device)
        self._copied = torch.cuda.Event()
        self._copy_pending = False
        # A second staging area for small integer tables that parts make during a step (work lists).
        self._aux_ints = 4 * o.max_rows + 64
        self._aux_staging = torch.empty(self._aux_ints, dtype=torch.int32, pin_memory=True)
        self._aux_np = self._aux_staging.numpy()
        self._aux_device = torch.zeros(self._aux_ints, dtype=torch.int32, device=self.device)
        self._aux_used = 0
        self._aux_copied = torch.cuda.Event()
        self._aux_pending = False
        # Each request's last sampled token, written by the sampling kernels: a step may name a token as -1 and the
        # embedding then reads it from here, so the step can be queued before the host has seen the token.
        self.sampled = torch.zeros(o.max_slots + 1, dtype=torch.int32, device=self.device)
        self.logit_slots = None        # device view: the slot of every logit row of the last step
        self.steps = 0
        self.graph_replays = 0
        self._graphs: dict = {}
        self._graph_generation = 0
        # Padding rows of a graph step write their key and value to the cache manager's spare slot.
        self._pad_slot = self.cache.pad_slot if (o.cuda_graphs and self.model.graph_safe) else -1

    @classmethod
    def from_random(cls, config: dict, seed: int, options: Optional[EngineOptions] = None) -> "Engine":
        """A model with random weights made directly on the device (no file)."""
        from ..weights.random_init import random_tensors
        o = options or EngineOptions()
        return cls(None, o, config=config, tensors=random_tensors(config, seed, o.device))

    def _upload_ints(self, values) -> torch.Tensor:
        """Copy a small int32 array to the device for the current step; returns the device view."""
        values = np.ascontiguousarray(values, dtype=np.int32).reshape(-1)
        k, at = values.shape[0], self._aux_used
        if at + k > self._aux_ints:
            raise EngineError("the step's integer tables exceed the staging area")
        self._aux_np[at:at + k] = values
        self._aux_device[at:at + k].copy_(self._aux_staging[at:at + k], non_blocking=True)
        self._aux_copied.record()
        self._aux_pending = True
        self._aux_used = at + ((k + 3) & ~3)
        return self._aux_device[at:at + k]

    # ------------------------------------------------------------------ the step
    def step(self, entries: list) -> Optional[torch.Tensor]:
        """Run one batch. Returns the logits [wanted, vocab] float32 on the device, in the order of
        the entries and of their `want` lists, or None if nothing is wanted. The tensor is a view of
        an engine buffer: it is overwritten by the next step."""
        o = self.options
        n = sum(len(e.tokens) for e in entries)
        if n == 0:
            return None
        if self._pad_slot >= 0 and n == len(entries):
            logits = self._graph_step(entries)
            if logits is not None:
                return logits
        if n > o.max_rows:
            raise EngineError(f"step of {n} tokens exceeds max_rows {o.max_rows}")
        count = sum(len(e.want) for e in entries)
        if count > self.env.max_logit_rows:
            raise EngineError(f"logits wanted at {count} places exceed max_full_rows {self.env.max_logit_rows}")
        R = o.max_rows
        if self._copy_pending:
            self._copied.synchronize()
        if self._aux_pending:
            self._aux_copied.synchronize()
            self._aux_pending = False
        self._aux_used = 0
        buf = self._staging_np
        tok, pos, slt, rows = buf[0:n], buf[R:R + n], buf[2 * R:2 * R + n], buf[3 * R:3 * R + count]
        meta = buf[4 * R:8 * R].reshape(4, R)
        at = w = 0
        seen = set()
        vocab = self.spec.vocab_size
        for i, e in enumerate(entries):
            L = len(e.tokens)
            if L == 0:
                raise EngineError("a step entry without tokens")
            if e.slot in seen:
                raise EngineError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.is_live(e.slot):
                raise EngineError(f"slot {e.slot} is not held by a request")
            if e.first_pos < 0 or e.first_pos + L > self.cache.length[e.slot]:
                raise EngineError(f"slot {e.slot}: tokens {e.first_pos}..{e.first_pos + L - 1} have no pages "
                                  f"(ensured up to {self.cache.length[e.slot]})")
            t = np.asarray(e.tokens, dtype=np.int64)
            if (t.min() < 0 and not (L == 1 and t[0] == -1)) or t.max() >= vocab:
                raise EngineError(f"token id out of range 0..{vocab - 1} in the entry of slot {e.slot}")
            tok[at:at + L] = t
            pos[at:at + L] = np.arange(e.first_pos, e.first_pos + L)
            slt[at:at + L] = e.slot
            for j in e.want:
                if not 0 <= j < L:
                    raise EngineError(f"wanted place {j} is outside the entry's {L} tokens")
                rows[w] = at + j
                buf[8 * R + w] = e.slot
                w += 1
            meta[0, i], meta[1, i], meta[2, i], meta[3, i] = e.slot, at, L, e.first_pos
            at += L
        self._device_ints.copy_(self._staging, non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        self.cache.sync()
        d = self._device_ints
        E = len(entries)
        ctx = StepContext(
            n=n, token_ids=d[0:n], positions=d[R:R + n], slots=d[2 * R:2 * R + n], workspace=self.workspace,
            compute_dtype=self.compute_dtype,
            entry_slots=[e.slot for e in entries], entry_first_row=[int(x) for x in meta[1, :E]],
            entry_length=[len(e.tokens) for e in entries], entry_first_pos=[e.first_pos for e in entries],
            entry_meta=d[4 * R:8 * R].view(4, R)[:, :E], upload_ints=self._upload_ints, sampled=self.sampled)
        logits = self.model.forward(ctx, self.caches, d[3 * R:3 * R + count], count)
        self.logit_slots = d[8 * R:8 * R + count]
        self.steps += 1
        return logits

    def check_kernels(self, code: int = 0) -> None:
        """Raises if a bounded wait inside a tensor-core kernel gave up, in which case the steps since are not valid:
        `code` is what the sampling kernels reported instead of a token, or 0 to read the status word now (which
        waits for the device)."""
        if self._status_device is None:
            return
        if code == 0:
            code = int(self._status_device.item())
        if code != 0:
            self._status_device.zero_()
            raise EngineError(f"a wait inside a tensor-core kernel gave up (code {code}): a signal was lost and the "
                              f"results of the step are not valid")

    # ------------------------------------------------------------------ decode steps as CUDA graphs
    def _graph_step(self, entries: list) -> Optional[torch.Tensor]:
        """A step in which every entry is one decoded token whose logits are wanted: padded to a batch
        bucket, run from a CUDA graph recorded for (batch bucket, context bucket). Returns None if the step
        does not qualify."""
        o = self.options
        E = len(entries)
        if self._pad_slot < 0 or E == 0 or E > self.env.max_logit_rows:
            return None
        for e in entries:
            if len(e.tokens) != 1 or e.want != [0]:
                return None
        B = 1
        while B < E:
            B *= 2
        if B > min(o.max_rows, self.env.max_logit_rows):
            B = E
        last = max(e.first_pos for e in entries)
        keys = 256
        while keys <= last:
            keys *= 2
        R, vocab = o.max_rows, self.spec.vocab_size
        if self._copy_pending:
            self._copied.synchronize()
        buf = self._staging_np
        meta = buf[4 * R:8 * R].reshape(4, R)
        seen = set()
        for i, e in enumerate(entries):
            if e.slot in seen or not self.cache.is_live(e.slot) or e.slot == self._pad_slot:
                raise EngineError(f"slot {e.slot} appears twice in one step or is not held by a request")
            seen.add(e.slot)
            if e.first_pos < 0 or e.first_pos + 1 > self.cache.length[e.slot]:
                raise EngineError(f"slot {e.slot}: token {e.first_pos} has no page (ensured up to {self.cache.length[e.slot]})")
            t = int(e.tokens[0])
            if not -1 <= t < vocab:
                raise EngineError(f"token id {t} out of range 0..{vocab - 1}")
            buf[i], buf[R + i], buf[2 * R + i], buf[8 * R + i] = t, e.first_pos, e.slot, e.slot
            meta[0, i], meta[1, i], meta[2, i], meta[3, i] = e.slot, i, 1, e.first_pos
        for i in range(E, B):
            buf[i], buf[R + i], buf[2 * R + i], buf[8 * R + i] = 0, 0, self._pad_slot, self._pad_slot
            meta[0, i], meta[1, i], meta[2, i], meta[3, i] = self._pad_slot, i, 1, 0
        buf[3 * R:3 * R + B] = np.arange(B)
        self._device_ints.copy_(self._staging, non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        self.cache.sync()
        if self._graph_generation != self.workspace.generation:
            self._graphs.clear()
            self._graph_generation = self.workspace.generation
        key = (B, keys)
        graph = self._graphs.get(key)
        d = self._device_ints

        def run():
            ctx = StepContext(
                n=B, token_ids=d[0:B], positions=d[R:R + B], slots=d[2 * R:2 * R + B], workspace=self.workspace,
                compute_dtype=self.compute_dtype, entry_slots=[0] * B, entry_first_row=list(range(B)),
                entry_length=[1] * B, entry_first_pos=[0] * B, entry_meta=d[4 * R:8 * R].view(4, R)[:, :B],
                upload_ints=None, static_keys=keys, sampled=self.sampled)
            return self.model.forward(ctx, self.caches, d[3 * R:3 * R + B], B)

        if graph is None:
            logits = run()                      # allocates what the step needs and gives this step's result
            if self._graph_generation != self.workspace.generation:
                self._graphs.clear()
                self._graph_generation = self.workspace.generation
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            from ..kernels import ops
            before = ops.launches
            with torch.cuda.graph(g):
                static_logits = run()
            self._graphs[key] = (g, static_logits, ops.launches - before)
            logits = static_logits              # recorded, not run: the eager run above left the same buffer filled
        else:
            graph[0].replay()
            logits = graph[1]
            self.graph_replays += 1
            from ..kernels import ops
            ops.launches += graph[2]
        self.logit_slots = d[8 * R:8 * R + E]
        self.steps += 1
        return logits[:E]

    def weight_bytes_per_step(self) -> int:
        return self.model.weight_bytes()
