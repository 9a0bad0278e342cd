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

import ctypes

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..config import resolve_architecture
from ..kernels.build import build_all
from ..kernels.native import NotNative, StepProgram
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
    native_step: bool = True           # launch a step's kernels from the native step program (else part by part from Python)
    decode_chain: bool = False         # native steps of decoded tokens only: all layers as one persistent kernel (the same bits; measured slower)
    device: str = "cuda:0"


@dataclass
class StepEntry:
    slot: int
    first_pos: int                     # position of tokens[0] in its sequence
    tokens: list
    want: list = field(default_factory=list)   # indices into `tokens` whose logits are wanted


_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}
_I32P = ctypes.POINTER(ctypes.c_int32)


def _i32(array: np.ndarray):
    if array.dtype != np.int32 or not array.flags["C_CONTIGUOUS"]:
        raise EngineError("a step's arrays must be contiguous int32")
    return array.ctypes.data_as(_I32P)


def _native_stager(lib):
    """The runtime library with the functions that check a step and fill its staging area typed."""
    if not getattr(lib, "_sb_stage_typed", False):
        vp, ci = ctypes.c_void_p, ctypes.c_int
        lib.sb_stage_step.restype, lib.sb_stage_step.argtypes = ci, [vp, ci, _I32P, _I32P, _I32P, _I32P, _I32P, _I32P, ci, ci, ci, _I32P, _I32P]
        lib.sb_stage_decode.restype, lib.sb_stage_decode.argtypes = ci, [vp, ci, ci, ci, _I32P, _I32P, _I32P, ci, ci, _I32P]
        lib._sb_stage_typed = True
    return lib


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
                       max_requests=o.max_slots, decode_chain=o.decode_chain and o.native_step)
        self.env = env
        self.model = DecoderModel(self.spec, env)
        libraries = self.model.kernel_libraries()
        build_all(sorted(libraries))      # what this model needs, compiled side by side if missing
        # the word into which the tensor-core kernels' bounded waits report; the sampling kernels pass it on to the host
        self._status_device = None
        if self.device.type == "cuda" and libraries & {"gemm_tc", "attention_tc5", "decode_chain"}:
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
        # tokens, positions, slots, logit rows (max_rows each), entry records (4 x max_rows), the slot of every logit row,
        # and the work lists of the attention kernels that the native step program plans.
        self._work_ints = 4 * o.max_rows + 64
        self._ints = 9 * o.max_rows + self._work_ints
        self._staging = torch.empty(self._ints, dtype=torch.int32, pin_memory=True)
        self._staging_np = self._staging.numpy()
        self._device_ints = torch.zeros(self._ints, dtype=torch.int32, device=self.device)
        self._staging_p = self._staging_np.ctypes.data_as(_I32P)
        self._staged = np.zeros(2, dtype=np.int32)          # rows and wanted rows of the step just staged
        self._staged_p = self._staged.ctypes.data_as(_I32P)
        self._stager = _native_stager(self.cache._lib)
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
        # The step as a native program: every part describes its operations once; a part that cannot leaves the
        # model to the Python driver (`DecoderModel.forward`), which launches the same kernels part by part.
        self._program, self._program_logits = None, None
        if o.native_step:
            from ..kernels import ops
            program = StepProgram(self.workspace, o.max_rows, self._work_ints, ops.gemm_tc_partial_tokens() if self.compute_dtype == torch.bfloat16 else 0)
            try:
                self._program_logits = self.model.emit(program, self.caches, self.sampled)
                self._program = program
            except NotNative:
                self._program = None
        self.h2d_bytes_per_step = self._ints * 4

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
        E = len(entries)
        if sum(len(e.tokens) for e in entries) == 0:
            return None
        for e in entries:
            if len(e.tokens) == 0:
                raise EngineError("a step entry without tokens")
        tokens = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64)
        if tokens.min() < -1 or tokens.max() >= self.spec.vocab_size:
            raise EngineError(f"token id out of range 0..{self.spec.vocab_size - 1}")
        want = np.fromiter((j for e in entries for j in e.want), dtype=np.int64)
        if want.size and (want.min() < 0 or want.max() >= (1 << 31)):
            raise EngineError("a wanted place is outside its entry's tokens")
        return self.step_arrays(E, np.fromiter((e.slot for e in entries), dtype=np.int32, count=E),
                                np.fromiter((e.first_pos for e in entries), dtype=np.int32, count=E),
                                np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=E), tokens.astype(np.int32),
                                np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=E), want.astype(np.int32))

    def step_arrays(self, E: int, slot, first, count, tokens, n_want, want) -> Optional[torch.Tensor]:
        """`step` for a batch given as int32 arrays (contiguous, at least as long as used): entry i < E is
        slot[i], first[i], its count[i] tokens taken one after another from `tokens`, and n_want[i] wanted places
        taken one after another from `want`. The native stager checks the batch against the cache's books and fills
        the staging area; the scheduler hands its plan over in this form."""
        o, R, lib = self.options, self.options.max_rows, self._stager
        n = int(count[:E].sum()) if E else 0
        if n == 0:
            return None
        if self._pad_slot >= 0 and n == E and E <= self.env.max_logit_rows and bool((n_want[:E] == 1).all()) and not want[:E].any():
            return self._graph_step(E, slot, first, tokens)
        if self._copy_pending:
            self._copied.synchronize()
        if self._aux_pending:
            self._aux_copied.synchronize()
            self._aux_pending = False
        self._aux_used = 0
        if lib.sb_stage_step(self.cache._pool, E, _i32(slot), _i32(first), _i32(count), _i32(tokens), _i32(n_want), _i32(want),
                             self.spec.vocab_size, R, self.env.max_logit_rows, self._staging_p, self._staged_p) < 0:
            raise EngineError(lib.sb_last_error().decode())
        wanted = int(self._staged[1])
        if self._program is not None:
            self._program.prepare(E, _i32(count), _i32(first), n, wanted, 0, self._staging_p, self._device_ints)
            self._device_ints.copy_(self._staging, non_blocking=True)
            self._copied.record()
            self._copy_pending = True
            self.cache.sync()
            self._program.run()
            self.logit_slots = self._device_ints[8 * R:8 * R + wanted]
            self.steps += 1
            return self._program_logits[:wanted] if wanted else None
        meta = self._staging_np[4 * R:8 * R].reshape(4, R)
        self._device_ints.copy_(self._staging, non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        self.cache.sync()
        d = self._device_ints
        ctx = StepContext(
            n=n, token_ids=d[0:n], positions=d[R:R + n], slots=d[2 * R:2 * R + n], workspace=self.workspace,
            compute_dtype=self.compute_dtype,
            entry_slots=slot[:E].tolist(), entry_first_row=meta[1, :E].tolist(),
            entry_length=count[:E].tolist(), entry_first_pos=first[:E].tolist(),
            entry_meta=d[4 * R:8 * R].view(4, R)[:, :E], upload_ints=self._upload_ints, sampled=self.sampled)
        logits = self.model.forward(ctx, self.caches, d[3 * R:3 * R + wanted], wanted)
        self.logit_slots = d[8 * R:8 * R + wanted]
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
            for chain in (self._program.chains if self._program is not None else ()):
                chain.reset()          # (a chain that gave up leaves its phase counter where it was)
            raise EngineError(f"a wait inside a tensor-core kernel gave up (code {code}): a signal was lost and the "
                              f"results of the step are not valid")

    # ------------------------------------------------------------------ decode steps as CUDA graphs
    def _graph_step(self, E: int, slot, first, tokens) -> torch.Tensor:
        """A step in which every entry is one decoded token whose logits are wanted: padded to a batch
        bucket, run from a CUDA graph recorded for (batch bucket, context bucket)."""
        o, lib = self.options, self._stager
        B = 1
        while B < E:
            B *= 2
        if B > min(o.max_rows, self.env.max_logit_rows):
            B = E
        last = int(first[:E].max())
        keys = 256
        while keys <= last:
            keys *= 2
        R = o.max_rows
        if self._copy_pending:
            self._copied.synchronize()
        if lib.sb_stage_decode(self.cache._pool, E, B, self._pad_slot, _i32(slot), _i32(first), _i32(tokens), self.spec.vocab_size, R,
                               self._staging_p) < 0:
            raise EngineError(lib.sb_last_error().decode())
        if self._program is not None:
            self._program.prepare(B, None, None, B, B, keys, self._staging_p, self._device_ints)
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
            if self._program is not None:
                self._program.run()
                return self._program_logits[:B]
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
