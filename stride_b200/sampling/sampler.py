"""Choosing the next token from logits.

`SamplingParams` and the rule are arhaamatiq/stride's (src/scheduler.h:20-25,
src/scheduler.cpp:193-243): temperature <= 0 takes the largest logit (the smallest index
among equals); otherwise tokens are ranked by (logit descending, index ascending), cut to
top_k if > 0, weighted by exp((l - l_max) / T) in 64-bit, cut to the shortest prefix whose
normalised cumulative weight reaches top_p if < 1, and the token is the first whose
cumulative weight exceeds u = uniform * total. The uniform is keyed on (seed, number of
tokens the sequence has) only, never on a stream, so a request's draws do not depend
on what else was scheduled with it.

Greedy rows and plain temperature rows are chosen by CUDA kernels (`csrc/sampling.cu`);
rows with top_k or top_p are chosen on the host from the downloaded logits, as the
reference does for all rows.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from ..kernels import ops

_MASK = (1 << 64) - 1


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int = 0


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def keyed_uniform(seed: int, length: int) -> float:
    """In [0, 1): depends on the request's seed and its sequence length only."""
    r = splitmix64((seed & _MASK) ^ ((length * 0x9E3779B97F4A7C15) & _MASK))
    return float(r >> 11) * (1.0 / 9007199254740992.0)


def choose_token_host(logits: np.ndarray, params: SamplingParams, length: int):
    """The full rule on the host, in 64-bit. Returns (token, its logit)."""
    l = np.asarray(logits, dtype=np.float32)
    valid = ~np.isnan(l)
    best = int(np.argmax(np.where(valid, l, -np.inf)))
    if params.temperature <= 0.0:
        return best, float(l[best])
    order = np.lexsort((np.arange(l.shape[0]), -l.astype(np.float64)))
    count = l.shape[0]
    if params.top_k > 0:
        count = min(count, params.top_k)
    t = float(np.float32(params.temperature))
    ranked = l[order[:count]].astype(np.float64)
    probs = np.exp((ranked - ranked[0]) / t)
    total = math.fsum([]) if count == 0 else float(np.cumsum(probs)[-1])
    if params.top_p < 1.0:
        cum = np.cumsum(probs / total)
        kept = int(np.searchsorted(cum, float(np.float32(params.top_p)), side="left")) + 1
        count = min(kept, count)
        probs = probs[:count]
        total = float(np.cumsum(probs)[-1])
    u = keyed_uniform(params.seed, length) * total
    cum = np.cumsum(probs)
    i = int(np.searchsorted(cum, u, side="right"))
    i = min(i, count - 1)
    tok = int(order[i])
    return tok, float(l[tok])


class Sampler:
    """Chooses tokens for the rows of one step's logits.

    `choose` is the whole thing at once. `launch` + `collect` split it, so that a caller can queue the next
    step on the GPU before reading this step's tokens: `launch` enqueues the kernels and the copies of their
    results into pinned host memory (two sets of buffers, used alternately) and returns a ticket; `collect`
    waits for that ticket's copies. Rows with top_k or top_p need their logits on the host, so a launch that
    has such rows synchronises by itself. With `scatter`, the device kernels also leave every row's token at
    scatter[scatter_index[row]] (the engine's per-request table that the next step's embedding reads).
    """

    pipelined = True     # `launch` leaves tokens where the next step finds them: the scheduler may run a step ahead

    def __init__(self, device, max_rows: int):
        self.device = torch.device(device)
        self.max_rows = R = max_rows + (max_rows & 1)          # even, so that the 64-bit seeds stay 8-byte aligned
        # One device buffer and one copy each way per step: what the kernels read (temperatures, seeds, lengths: 4 R
        # 32-bit words) and what they write (greedy tokens and values, sampled tokens and values: 4 x rows words).
        self._inputs = torch.zeros(4 * R, dtype=torch.int32, device=self.device)
        self._outputs = torch.zeros(4 * R, dtype=torch.int32, device=self.device)
        self._temps = self._inputs[0:R].view(torch.float32)
        self._seeds = self._inputs[R:3 * R].view(torch.int64)
        self._lengths = self._inputs[3 * R:4 * R]
        self._host_inputs = [torch.zeros(4 * R, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._host_outputs = [torch.zeros(4 * R, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events = [torch.cuda.Event(), torch.cuda.Event()]
        self._turn = 0

    @staticmethod
    def on_device(p: SamplingParams) -> bool:
        """True if the row's token is chosen by a CUDA kernel (greedy, or temperature without top_k / top_p)."""
        return p.temperature <= 0.0 or (p.top_k <= 0 and p.top_p >= 1.0)

    def launch(self, logits: torch.Tensor, params: list, lengths: list, scatter_index=None, scatter=None):
        rows, R = logits.shape[0], self.max_rows
        if rows > R:
            raise ValueError(f"{rows} rows exceed the sampler's {R}")
        out = self._outputs
        tokens = [out[k * rows:(k + 1) * rows] for k in (0, 2)]
        values = [out[k * rows:(k + 1) * rows].view(torch.float32) for k in (1, 3)]
        ops.argmax(logits, tokens[0], values[0], scatter_index, scatter)
        device_rows = [i for i, p in enumerate(params) if p.temperature > 0.0 and p.top_k <= 0 and p.top_p >= 1.0]
        host_rows = [i for i, p in enumerate(params) if p.temperature > 0.0 and not (p.top_k <= 0 and p.top_p >= 1.0)]
        turn = self._turn
        self._turn ^= 1
        self._events[turn].synchronize()       # the launch that used this set of host buffers two turns ago is done
        if device_rows:
            host = self._host_inputs[turn].numpy()
            on = set(device_rows)
            # (rows not sampled on the device get temperature 0 and are skipped by the kernel)
            host[0:rows].view(np.float32)[:] = [p.temperature if i in on else 0.0 for i, p in enumerate(params)]
            host[R:R + 2 * rows].view(np.uint64)[:] = [p.seed & _MASK for p in params]
            host[3 * R:3 * R + rows] = lengths
            self._inputs.copy_(self._host_inputs[turn], non_blocking=True)
            ops.sample_temperature(logits, self._temps[:rows], self._seeds[:rows], self._lengths[:rows], tokens[1], values[1],
                                   scatter_index, scatter)
        words = (4 if device_rows else 2) * rows
        self._host_outputs[turn][:words].copy_(out[:words], non_blocking=True)
        host_logits = logits[host_rows].to("cpu") if host_rows else None      # synchronises
        self._events[turn].record()
        return (turn, rows, device_rows, host_rows, host_logits, params, lengths)

    def collect(self, ticket):
        """(tokens list, values list) of a launch."""
        turn, rows, device_rows, host_rows, host_logits, params, lengths = ticket
        self._events[turn].synchronize()
        host = self._host_outputs[turn]
        tokens = host[0:rows].tolist()
        values = host[rows:2 * rows].view(torch.float32).tolist()
        if rows and min(tokens) < 0:
            # the kernels report -1 - code instead of tokens: a wait inside a kernel that made these logits gave up
            return [min(tokens)] * rows, values
        if device_rows:
            sampled_tokens = host[2 * rows:3 * rows].tolist()
            sampled_values = host[3 * rows:4 * rows].view(torch.float32).tolist()
            for i in device_rows:
                tokens[i], values[i] = sampled_tokens[i], sampled_values[i]
        for k, i in enumerate(host_rows):
            tokens[i], values[i] = choose_token_host(host_logits[k].numpy(), params[i], lengths[i])
        return tokens, values

    def choose(self, logits: torch.Tensor, params: list, lengths: list):
        """logits [rows, vocab] on the device; params[i], lengths[i] belong to row i (length = tokens the
        sequence has before the new one). Returns (tokens list, values list)."""
        return self.collect(self.launch(logits, params, lengths))
