"""Python faces of the CUDA kernels: torch tensors in, raw pointers down.

Every function here launches hand-written CUDA from `stride_b200/csrc` on the
current torch stream. There is no torch or CPU implementation behind them: a
tensor that is not on a CUDA device, or a library that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from .build import library

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

_configured: set = set()


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"stride_b200 kernels take float32 or bfloat16 tensors, not {dtype}") from None


def _fn(lib_name: str, fn_name: str, argtypes):
    lib = library(lib_name)
    fn = getattr(lib, fn_name)
    if (lib_name, fn_name) not in _configured:
        fn.argtypes = argtypes
        fn.restype = c_int
        _configured.add((lib_name, fn_name))
    return lib, fn


launches = 0    # kernels launched through this module since import (bench.py reports the difference)


def _check(lib, rc: int) -> None:
    global launches
    launches += 1
    if rc != 0:
        raise RuntimeError(lib.sb_last_error().decode(errors="replace"))


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("stride_b200 kernels run on CUDA tensors only; got a tensor on " + str(t.device))


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current torch stream's handle (kernels are launched on it, so they order with torch's own work)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, slots=None, sampled=None) -> None:
    """out[i, :] = float32(table[tokens[i], :]); a token of -1 means sampled[slots[i]] (the request's last sampled token)."""
    _cuda(tokens, table, out, slots, sampled)
    lib, fn = _fn("elementwise", "sb_embed", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    n, H = out.shape
    _check(lib, fn(_ptr(tokens), _ptr(table), dtype_code(table.dtype), _ptr(out), n, H, table.shape[0], _ptr(slots),
                   _ptr(sampled) if slots is not None else 0, _stream()))


def rmsnorm(h: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, partials=None) -> None:
    """out = weight * (x / sqrt(mean(x^2) + eps)) with x = h (+ partials[0] + partials[1] ...).

    `partials` [S, n, H] float32 are summed into h left to right and h is updated in place.
    """
    _cuda(h, weight, out, partials)
    lib, fn = _fn("norm", "sb_rmsnorm", [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_int, c_void_p, c_int,
                                               c_int, c_int, c_float, c_void_p])
    n, H = h.shape
    S = 0 if partials is None else partials.shape[0]
    stride = 0 if partials is None else partials.stride(0)
    _check(lib, fn(_ptr(h), _ptr(partials), S, stride, _ptr(weight), dtype_code(weight.dtype), _ptr(out),
                   dtype_code(out.dtype), n, H, eps, _stream()))


def rope_append(qkv: torch.Tensor, positions, slots, cos_sin, rotary_dim: int, q_out, cache_layer, block_table,
                num_heads: int, num_kv_heads: int, head_dim: int, write_kv: bool = True) -> None:
    """Rotate q and k of `qkv` [S, n, (Hq + 2 Hkv) D] (partials summed), store q, append k and v to the pages.

    `cache_layer` is this layer's view [pages, 2, Hkv, page_size, D] of the arena.
    """
    _cuda(qkv, positions, slots, cos_sin, q_out, cache_layer, block_table)
    lib, fn = _fn("elementwise", "sb_rope_append",
                  [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                   c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p])
    if qkv.dim() == 2:
        qkv = qkv.unsqueeze(0)
    S, n, _ = qkv.shape
    _check(lib, fn(_ptr(qkv), S, qkv.stride(0), _ptr(positions), _ptr(slots), _ptr(cos_sin), rotary_dim, _ptr(q_out),
                   dtype_code(q_out.dtype), _ptr(cache_layer), dtype_code(cache_layer.dtype), _ptr(block_table),
                   block_table.shape[1], cache_layer.shape[3], cache_layer.stride(0), cache_layer.stride(1),
                   cache_layer.stride(2), n, num_heads, num_kv_heads, head_dim, int(write_kv), _stream()))


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[n, I] = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _cuda(gate_up, out)
    lib, fn = _fn("elementwise", "sb_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    n, I = out.shape
    _check(lib, fn(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), n, I, _stream()))


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor, partials=None) -> None:
    """out[i, :] = src[rows[i], :] (+ partials[s, rows[i], :] for every s)."""
    _cuda(src, rows, out, partials)
    lib, fn = _fn("elementwise", "sb_gather_rows", [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p])
    S = 0 if partials is None else partials.shape[0]
    stride = 0 if partials is None else partials.stride(0)
    _check(lib, fn(_ptr(src), _ptr(partials), S, stride, _ptr(rows), _ptr(out), out.shape[0], out.shape[1], _stream()))


def gemm_f32(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out[n, M] (+)= x[n, K] . weight[M, K]^T in true 32-bit FMA; x and weight float32 or bfloat16."""
    _cuda(x, weight, out)
    if out.dtype != torch.float32:
        raise TypeError("gemm_f32 writes float32")
    lib, fn = _fn("gemm_f32", "sb_gemm_f32", [c_void_p, c_int, c_int64, c_void_p, c_int, c_int64, c_void_p, c_int64, c_int,
                                              c_int, c_int, c_int, c_void_p])
    n, K = x.shape
    M = weight.shape[0]
    if weight.shape[1] != K or out.shape[0] != n or out.shape[1] != M:
        raise ValueError(f"gemm_f32 shapes: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    _check(lib, fn(_ptr(x), dtype_code(x.dtype), x.stride(0), _ptr(weight), dtype_code(weight.dtype), weight.stride(0), _ptr(out),
                   out.stride(0), n, M, K, int(accumulate), _stream()))


def attention_generic(q, out, cache_layer, block_table, positions, slots, num_heads: int, num_kv_heads: int,
                      head_dim: int, window: int, scale: float) -> None:
    """Causal paged attention of every token of the step over its request's cache (any head size)."""
    _cuda(q, out, cache_layer, block_table, positions, slots)
    if not (q.dtype == out.dtype == cache_layer.dtype):
        raise TypeError("attention_generic takes q, out and cache of one dtype")
    lib, fn = _fn("attention_generic", "sb_attention_generic",
                  [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p,
                   c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(lib, fn(_ptr(q), _ptr(out), dtype_code(q.dtype), _ptr(cache_layer), _ptr(block_table), block_table.shape[1],
                   cache_layer.shape[3], cache_layer.stride(0), cache_layer.stride(1), cache_layer.stride(2),
                   _ptr(positions), _ptr(slots), q.shape[0], num_heads, num_kv_heads, head_dim, window, scale, _stream()))


def argmax(logits: torch.Tensor, tokens: torch.Tensor, values: torch.Tensor, scatter_index=None, scatter=None) -> None:
    """tokens[i] = index of the largest logit of row i (smallest index among equals); values[i] = that logit.
    With `scatter`, also scatter[scatter_index[i]] = tokens[i]."""
    _cuda(logits, tokens, values, scatter_index, scatter)
    lib, fn = _fn("sampling", "sb_argmax", [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(lib, fn(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(tokens), _ptr(values),
                   _ptr(scatter_index), _ptr(scatter) if scatter_index is not None else 0, _stream()))


def sample_temperature(logits, temperatures, seeds, lengths, tokens, values, scatter_index=None, scatter=None) -> None:
    """Temperature sampling keyed on (seed, sequence length) for every row with temperature > 0 (other rows are left
    alone); see csrc/sampling.cu. With `scatter`, also scatter[scatter_index[i]] = tokens[i]."""
    _cuda(logits, temperatures, seeds, lengths, tokens, values, scatter_index, scatter)
    lib, fn = _fn("sampling", "sb_sample_temperature", [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(lib, fn(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(temperatures), _ptr(seeds),
                   _ptr(lengths), _ptr(tokens), _ptr(values), _ptr(scatter_index),
                   _ptr(scatter) if scatter_index is not None else 0, _stream()))


STORE, ADD, SWIGLU = 0, 1, 2


def gemm_tc_splits(M: int, K: int) -> int:
    """How many K ranges `gemm_tc` cuts a [M, K] weight into: a function of the weight's shape alone."""
    lib = library("gemm_tc")
    lib.sb_gemm_tc_splits.argtypes = [c_int, c_int]
    lib.sb_gemm_tc_splits.restype = c_int
    return lib.sb_gemm_tc_splits(M, K)


def gemm_tc_partial_tokens() -> int:
    """Up to this many tokens `gemm_tc` leaves one partial buffer per K range; with more it adds the ranges itself."""
    lib = library("gemm_tc")
    lib.sb_gemm_tc_partial_tokens.restype = c_int
    return lib.sb_gemm_tc_partial_tokens()


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int = STORE, splits: int = 1,
            half_rows: int = 0) -> None:
    """out = x . weight^T on the tcgen05 tensor cores; x [n, K] and weight [M, K] bfloat16.

    STORE: out float32 [n, M]. With splits > 1 (= gemm_tc_splits) and at most gemm_tc_partial_tokens() tokens, out is
    [splits, n, M]: one partial sum per K range, to be added in ascending order; with more tokens the kernel adds the
    ranges itself, in the same order, and out is [n, M].
    ADD: out float32 [n, M] += result (one range only).
    SWIGLU: weight is [2 I, K] (gate rows, then up rows) and out bfloat16 [n, I] = silu(x . gate^T) * (x . up^T).
    """
    _cuda(x, weight, out)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("gemm_tc takes bfloat16 operands")
    want = torch.bfloat16 if epilogue == SWIGLU else torch.float32
    if out.dtype != want:
        raise TypeError(f"gemm_tc epilogue {epilogue} writes {want}")
    lib, fn = _fn("gemm_tc", "sb_gemm_tc", [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int,
                                            c_int, c_int, c_int64, c_int, c_void_p])
    n, K = x.shape
    M = weight.shape[0]
    if weight.shape[1] != K:
        raise ValueError(f"gemm_tc shapes: x {tuple(x.shape)}, weight {tuple(weight.shape)}")
    if splits > 1 and n <= gemm_tc_partial_tokens():
        if out.dim() != 3 or out.shape[0] != splits:
            raise ValueError("gemm_tc with K ranges and few tokens writes [splits, n, M]")
        ldo, split_stride = out.stride(1), out.stride(0)
    else:
        o2 = out[0] if out.dim() == 3 else out
        ldo, split_stride = o2.stride(0), 0
    _check(lib, fn(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), ldo, n, M, K, epilogue, splits,
                   split_stride, half_rows, _stream()))


def gemm_tc_status() -> int:
    """0 if every wait inside the tensor-core kernels completed since the last call; synchronises."""
    lib = library("gemm_tc")
    lib.sb_gemm_tc_status.restype = c_int
    return lib.sb_gemm_tc_status()


_status_word = None
_status_users = {"gemm_tc": "sb_gemm_tc_use_status_word", "attention_tc5": "sb_attention_tc5_use_status_word",
                 "decode_chain": "sb_decode_chain_use_status_word",
                 "sampling": "sb_sampling_use_status_word"}   # the sampling kernels only read it
_status_registered: set = set()


def shared_status_word(libraries=("gemm_tc",)) -> torch.Tensor:
    """One int32 on the device into which the bounded waits of the tensor-core kernels report when they give up:
    0 = every wait completed. Made at the first call; those of `libraries` that have such waits (gemm_tc,
    attention_tc5) use it from then on, and the sampling kernels report -1 - its value instead of a token while it is
    not 0, so that a lost signal is an error and not a wrong token."""
    global _status_word
    if _status_word is None:
        _status_word = torch.zeros(1, dtype=torch.int32, device="cuda")
    for lib_name in sorted(set(libraries) & set(_status_users) - _status_registered):
        fn = getattr(library(lib_name), _status_users[lib_name])
        fn.argtypes, fn.restype = [c_void_p], None
        fn(_status_word.data_ptr())
        _status_registered.add(lib_name)
    return _status_word


def lost_signal_selftest(code: int = 9) -> None:
    """Launches a kernel whose only wait is never answered: after about a second it gives up and the status word
    reads `code`. Exercises the path by which a lost signal inside a tensor-core kernel becomes an error."""
    lib, fn = _fn("gemm_tc", "sb_gemm_tc_lost_signal_selftest", [c_int, c_void_p])
    _check(lib, fn(code, _stream()))


def attention_tc_scratch(items: int, num_kv_heads: int, chunks: int, head_dim: int) -> int:
    """Floats of scratch `attention_tc` needs."""
    return items * num_kv_heads * chunks * 16 * (head_dim + 2)


_decode_rope_limit = None


def attention_decode_rope_limit() -> int:
    """Up to this many CTAs (entries x key/value heads x chunks) `attention_decode_rope` runs all at once on this
    device and is the faster choice; asked of the library once."""
    global _decode_rope_limit
    if _decode_rope_limit is None:
        lib = library("attention_tc")
        lib.sb_attention_decode_rope_resident_ctas.restype = c_int
        _decode_rope_limit = int(lib.sb_attention_decode_rope_resident_ctas())
    return _decode_rope_limit


def attention_tc(q, out, cache_layer, block_table, entry_meta, work, n_tiles: int, n_items: int, chunks: int,
                 scratch, num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                 counters=None) -> None:
    """Tensor-core paged attention (bfloat16, head_dim 64 or 128); see csrc/attention_tc.cu for `work`.
    `counters`: int32 zeros, one per (decode entry, kv head); with them the decode kernel folds its own chunks."""
    _cuda(q, out, cache_layer, block_table, entry_meta, work, scratch, counters)
    if not (q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16):
        raise TypeError("attention_tc takes bfloat16 q, out and cache")
    lib, fn = _fn("attention_tc", "sb_attention_tc",
                  [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_int,
                   c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(lib, fn(_ptr(q), _ptr(out), _ptr(cache_layer), _ptr(block_table), block_table.shape[1], cache_layer.shape[3],
                   cache_layer.stride(0), cache_layer.stride(1), cache_layer.stride(2), _ptr(entry_meta),
                   entry_meta.stride(0), _ptr(work), n_tiles, n_items, chunks, _ptr(scratch), _ptr(counters), num_heads, num_kv_heads,
                   head_dim, window, scale, _stream()))


def attention_decode_rope(qkv, cos_sin, out, cache_layer, block_table, entry_meta, items, n_items: int, chunks: int, scratch,
                          counters, num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float) -> None:
    """The decode kernel of `attention_tc` with `rope_append` fused in, for steps whose entries all fit it: qkv
    [S, n, (Hq + 2 Hkv) D] float32 partial sums of the projection, cos_sin the table of a fully rotated head. Rotates
    q in shared memory, appends the step's rotated k and its v to the pages, attends. Same bits as the two kernels."""
    _cuda(qkv, cos_sin, out, cache_layer, block_table, entry_meta, items, scratch, counters)
    if not (out.dtype == cache_layer.dtype == torch.bfloat16) or qkv.dtype != torch.float32:
        raise TypeError("attention_decode_rope takes float32 qkv and bfloat16 out and cache")
    lib, fn = _fn("attention_tc", "sb_attention_decode_rope",
                  [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64,
                   c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    if qkv.dim() == 2:
        qkv = qkv.unsqueeze(0)
    _check(lib, fn(_ptr(qkv), qkv.shape[0], qkv.stride(0), _ptr(cos_sin), _ptr(out), _ptr(cache_layer), _ptr(block_table),
                   block_table.shape[1], cache_layer.shape[3], cache_layer.stride(0), cache_layer.stride(1),
                   cache_layer.stride(2), _ptr(entry_meta), entry_meta.stride(0), _ptr(items), n_items, chunks, _ptr(scratch),
                   _ptr(counters), num_heads, num_kv_heads, head_dim, window, scale, _stream()))


def attention_tc5_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """True if the tcgen05 prompt-attention kernel takes this shape (head size 64 or 128, pages of a power of two >= 8)."""
    if head_dim not in (64, 128) or num_kv_heads <= 0 or num_heads % num_kv_heads or num_heads // num_kv_heads > 128:
        return False
    return page_size >= 8 and page_size & (page_size - 1) == 0


def attention_tc5(q, out, cache_layer, block_table, entry_meta, work, n_tiles: int, num_heads: int, num_kv_heads: int,
                  head_dim: int, window: int, scale: float) -> None:
    """Prompt-portion attention on the tcgen05 tensor cores; `work` is [n_tiles, 2] = (entry, tile of 128 // G positions)."""
    _cuda(q, out, cache_layer, block_table, entry_meta, work)
    if not (q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16):
        raise TypeError("attention_tc5 takes bfloat16 q, out and cache")
    lib, fn = _fn("attention_tc5", "sb_attention_tc5",
                  [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_int,
                   c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(lib, fn(_ptr(q), _ptr(out), _ptr(cache_layer), cache_layer.shape[0], _ptr(block_table), block_table.shape[1],
                   cache_layer.shape[3], cache_layer.stride(0), cache_layer.stride(1), cache_layer.stride(2), _ptr(entry_meta),
                   entry_meta.stride(0), _ptr(work), n_tiles, q.shape[0], num_heads, num_kv_heads, head_dim, window, scale,
                   _stream()))


def attention_tc5_status() -> int:
    """0 if every wait inside the tcgen05 attention kernel completed since the last call; synchronises."""
    lib = library("attention_tc5")
    lib.sb_attention_tc5_status.restype = c_int
    return lib.sb_attention_tc5_status()
