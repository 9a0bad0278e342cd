"""The native step program seen from Python: parts describe their share of a step once, as operations of
the kernel libraries (`csrc/step_ops.h`); every step is then one call into the runner of `csrc/runtime.cpp`,
which launches them in order with no interpreter in between.

A part takes part by implementing `emit(...)` (see `parts/base.py`): it asks the `StepProgram` for the
buffers it needs at their full size and appends operations with `program.add(library, function, ints, floats)`.
A part without `emit` raises `NotNative`, and the engine then drives the whole model from Python, part by part
(`DecoderModel.forward`): both ways launch the same kernels with the same arguments.

Counterpart in arhaamatiq/stride: Engine::step_exact / step_tensor_core (src/engine.cpp:144-462).
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_int, c_int32, c_int64, c_void_p

import torch

from . import ops
from .build import library

MAX_PLANS, OP_INTS, OP_FLOATS = 4, 28, 4


class NotNative(Exception):
    """A part (or a combination of parts) has no native form; the engine falls back to the Python driver."""


class SbTilePlan(ctypes.Structure):
    _fields_ = [("group", c_int32), ("tile_rows", c_int32), ("kv_heads", c_int32), ("fused_limit", c_int32),
                ("work_offset", c_int32), ("tiles", c_int32), ("items", c_int32), ("chunks", c_int32),
                ("fused", c_int32), ("reserved", c_int32 * 3)]


class SbStep(ctypes.Structure):
    _fields_ = [("n", c_int32), ("entries", c_int32), ("wanted", c_int32), ("static_keys", c_int32), ("max_rows", c_int32),
                ("n_plans", c_int32), ("ints", c_void_p), ("plan", SbTilePlan * MAX_PLANS)]


class SbOp(ctypes.Structure):
    _fields_ = [("fn", c_void_p), ("i", c_int64 * OP_INTS), ("f", c_double * OP_FLOATS), ("covers", c_int64)]


_I32P = ctypes.POINTER(c_int32)


def _runtime():
    lib = library("runtime")
    if not getattr(lib, "_sb_program_typed", False):
        lib.sb_program_create.restype, lib.sb_program_create.argtypes = c_void_p, [c_int, c_int]
        lib.sb_program_destroy.restype, lib.sb_program_destroy.argtypes = None, [c_void_p]
        lib.sb_program_plan.restype, lib.sb_program_plan.argtypes = c_int, [c_void_p, c_int, c_int, c_int, c_int]
        lib.sb_program_add.restype, lib.sb_program_add.argtypes = c_int, [c_void_p, ctypes.POINTER(SbOp)]
        lib.sb_program_size.restype, lib.sb_program_size.argtypes = c_int, [c_void_p]
        lib.sb_program_set_covers.restype, lib.sb_program_set_covers.argtypes = c_int, [c_void_p, c_int, c_int]
        lib.sb_program_prepare.restype = c_int
        lib.sb_program_prepare.argtypes = [c_void_p, c_int, _I32P, _I32P, c_int, c_int, c_int, _I32P, c_void_p, ctypes.POINTER(SbStep)]
        lib.sb_program_run.restype = c_int
        lib.sb_program_run.argtypes = [c_void_p, ctypes.POINTER(SbStep), c_void_p, _I32P, _I32P]
        lib._sb_program_typed = True
    return lib


def _value(v) -> int:
    """An operation's integer argument: a tensor stands for its address, None for 0."""
    if v is None:
        return 0
    if isinstance(v, torch.Tensor):
        return v.data_ptr()
    if isinstance(v, torch.dtype):
        return ops.dtype_code(v)
    return int(v)


NO_PHASE = "no phase"     # `chain=` of an operation that has nothing to do in a step of decoded tokens only


class DecodeChain:
    """The layers of a step of decoded tokens as phases of one persistent kernel (`csrc/decode_chain.cu`): the same
    arithmetic as the layers' separate operations, which it stands for in such steps. Parts add their phase beside
    their operation (`StepProgram.add(..., chain=...)`); the methods mirror the operations they stand for."""

    def __init__(self, max_rows: int):
        from ctypes import c_float
        self._lib = lib = library("decode_chain")
        if not getattr(lib, "_sb_chain_typed", False):
            lib.sb_chain_create.restype, lib.sb_chain_create.argtypes = c_void_p, [c_int]
            lib.sb_chain_destroy.restype, lib.sb_chain_destroy.argtypes = None, [c_void_p]
            lib.sb_chain_size.restype, lib.sb_chain_size.argtypes = c_int, [c_void_p]
            lib.sb_chain_finish.restype, lib.sb_chain_finish.argtypes = c_int, [c_void_p]
            lib.sb_chain_reset.restype, lib.sb_chain_reset.argtypes = c_int, [c_void_p]
            lib.sb_chain_max_tokens.restype, lib.sb_chain_max_tokens.argtypes = c_int, []
            lib.sb_chain_norm.restype = c_int
            lib.sb_chain_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float]
            lib.sb_chain_linear.restype = c_int
            lib.sb_chain_linear.argtypes = [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int]
            lib.sb_chain_attention.restype = c_int
            lib.sb_chain_attention.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64,
                                               c_int64, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int]
            lib._sb_chain_typed = True
        self.handle = lib.sb_chain_create(max_rows)
        self.keep: list = []

    def __del__(self):
        handle, self.handle = getattr(self, "handle", None), None
        if handle:
            self._lib.sb_chain_destroy(handle)

    def __len__(self):
        return self._lib.sb_chain_size(self.handle)

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise NotNative(self._lib.sb_last_error().decode())

    def norm(self, h, pending, gain, x, size: int, eps: float) -> None:
        flat, S, _ = pending if pending is not None else (None, 1, 0)
        self.keep += [h, flat, gain, x]
        self._check(self._lib.sb_chain_norm(self.handle, _value(h), _value(flat), S, _value(gain), _value(gain.dtype), _value(x), _value(x.dtype), size, eps))

    def linear(self, x, weight, out, swiglu: bool, splits: int) -> None:
        self.keep += [x, weight, out]
        M, K = weight.shape
        self._check(self._lib.sb_chain_linear(self.handle, _value(x), x.stride(0), _value(weight), weight.stride(0), _value(out), M, K, int(swiglu), splits))

    def attention(self, qkv, S: int, cos_sin, out, pages, table, scratch_note: int, counters, num_heads: int, num_kv_heads: int, head_dim: int,
                  window: int, scale: float, plan: int) -> None:
        self.keep += [qkv, cos_sin, out, pages, table, counters]
        self._check(self._lib.sb_chain_attention(self.handle, _value(qkv), S, _value(cos_sin), _value(out), _value(pages), _value(table), table.shape[1],
                                                 pages.shape[3], pages.stride(0), pages.stride(1), pages.stride(2), scratch_note, _value(counters),
                                                 num_heads, num_kv_heads, head_dim, window, scale, plan))

    def finish(self) -> None:
        self._check(self._lib.sb_chain_finish(self.handle))

    def reset(self) -> None:
        self._lib.sb_chain_reset(self.handle)


class StepProgram:
    """The operations of one engine's step, the tile plans its mixers asked for, and what the build of the
    operations shares: the workspace, and which partial sums are pending on the residual stream."""

    def __init__(self, workspace, max_rows: int, work_ints: int, few_tokens: int):
        self._lib = _runtime()
        self._handle = self._lib.sb_program_create(max_rows, work_ints)
        self.workspace = workspace
        self.max_rows = max_rows
        self.few_tokens = few_tokens          # up to this many tokens a projection leaves one buffer per K range
        self.h = None                         # the residual stream [max_rows, hidden] float32
        self.pending = None                   # (flat buffer, K ranges, width) left by the last projection, or None
        self._libraries: list = []            # per operation: the library its function lives in (for its error text)
        self._keep: list = []                 # tensors the operations point into
        self.step = SbStep()
        self._failed, self._launched = c_int32(0), c_int32(0)
        self._growing: dict = {}              # name -> [note (address, elements), dtype, {key: need(step) -> elements}]
        self.chain = None                     # the DecodeChain being built between begin_chain() and end_chain(), if still whole
        self._chain_at = -1                   # the index of the chain's operation
        self.chains: list = []                # finished chains (kept alive; reset after a failed launch)

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.sb_program_destroy(handle)

    def __len__(self):
        return self._lib.sb_program_size(self._handle)

    def plan(self, group: int, tile_rows: int, kv_heads: int, fused_limit: int) -> int:
        k = self._lib.sb_program_plan(self._handle, group, tile_rows, kv_heads, fused_limit)
        if k < 0:
            raise NotNative(self._lib.sb_last_error().decode())
        return k

    def begin_chain(self) -> None:
        """From here to `end_chain()` every operation is asked for its phase of the decode chain; if all of them
        have one, one operation in front of them stands for them all in steps of decoded tokens only."""
        chain = DecodeChain(self.max_rows)
        self._chain_at = len(self)
        self.add("decode_chain", "sb_op_decode_chain", [chain.handle])
        self.chain = chain

    def end_chain(self) -> bool:
        chain, self.chain = self.chain, None
        if chain is None or len(chain) == 0:
            return False
        chain.finish()
        if self._lib.sb_program_set_covers(self._handle, self._chain_at, len(self) - self._chain_at - 1) < 0:
            raise RuntimeError(self._lib.sb_last_error().decode())
        self.chains.append(chain)
        return True

    def add(self, library_name: str, function: str, ints, floats=(), chain=None) -> None:
        """Append the operation `function` of kernel library `library_name` with its fixed arguments. `chain`: while a
        decode chain is being built, a function that adds the operation's phase to it (called with the chain; it may
        raise `NotNative`), or NO_PHASE; an operation without one ends the building of the chain."""
        if len(ints) > OP_INTS or len(floats) > OP_FLOATS:
            raise ValueError(f"{function}: too many arguments for one operation")
        if self.chain is not None:
            building, self.chain = self.chain, None
            if chain is NO_PHASE:
                self.chain = building
            elif chain is not None:
                try:
                    chain(building)
                    self.chain = building
                except NotNative:
                    pass
        lib = library(library_name)
        op = SbOp()
        op.fn = ctypes.cast(getattr(lib, function), c_void_p).value
        for k, v in enumerate(ints):
            op.i[k] = _value(v)
            if isinstance(v, torch.Tensor):
                self._keep.append(v)
        for k, v in enumerate(floats):
            op.f[k] = float(v)
        if self._lib.sb_program_add(self._handle, ctypes.byref(op)) < 0:
            raise RuntimeError(self._lib.sb_last_error().decode())
        self._libraries.append(library_name)

    def growing_buffer(self, name: str, dtype: torch.dtype, key, need) -> int:
        """A flat buffer of the workspace whose size depends on the step (`Workspace.grow`): `need(step) -> elements` is
        asked before every step and the buffer enlarged when it is too small. Returns the host address of its note, two
        int64 (the buffer's device address, its size in elements), which an operation reads when it runs; operations
        that ask under one `name` share one buffer. `key` tells equal askers apart from different ones."""
        entry = self._growing.setdefault(name, [(c_int64 * 2)(0, 0), dtype, {}])
        entry[2].setdefault(key, need)
        return ctypes.addressof(entry[0])

    def _grow(self) -> None:
        for name, (note, dtype, askers) in self._growing.items():
            need = max(fn(self.step) for fn in askers.values())
            if need > note[1]:
                buf = self.workspace.grow(name, need, dtype)       # (moves the buffer: recorded graphs are dropped by the engine)
                note[0], note[1] = buf.data_ptr(), buf.numel()

    def take_pending(self):
        p, self.pending = self.pending, None
        return p

    def need_folded(self, who: str) -> None:
        """For operations that add to the residual stream itself: partial sums may not be pending then."""
        if self.pending is not None:
            raise NotNative(f"{who} adds to the residual stream while partial sums are pending on it")

    def prepare(self, E: int, count, first, n: int, wanted: int, static_keys: int, staging_p, device_ints: torch.Tensor) -> None:
        if self._lib.sb_program_prepare(self._handle, E, count, first, n, wanted, static_keys, staging_p, device_ints.data_ptr(),
                                        ctypes.byref(self.step)) < 0:
            raise RuntimeError(self._lib.sb_last_error().decode())
        if self._growing:
            self._grow()

    def run(self) -> None:
        """Launch the step that `prepare` described on the current torch stream."""
        rc = self._lib.sb_program_run(self._handle, ctypes.byref(self.step), ops._stream(), ctypes.byref(self._failed),
                                      ctypes.byref(self._launched))
        ops.launches += self._launched.value
        if rc != 0:
            k = self._failed.value
            raise RuntimeError(f"operation {k} of the step failed: " + library(self._libraries[k]).sb_last_error().decode(errors="replace"))
