"""The native step program on the CPU: how a step's entries are cut into attention tiles and decode items (against
the rule restated here), that operations run in order and may skip or fail, that a block's roles are checked, and that a
kernel library from outside the package is compiled like the package's own."""
from __future__ import annotations

import ctypes
import random

import numpy as np
import pytest

from stride_b200.kernels.build import BuildError, library, register_kernel_library
from stride_b200.kernels.native import SbOp, SbStep, _runtime

_I32P = ctypes.POINTER(ctypes.c_int32)
R, WORK = 64, 4 * 64 + 64


def _plain_plan(counts, firsts, group, tile_rows):
    """The rule: entries of at most 16 // group tokens are decode items; longer ones are cut into tiles of tile_rows //
    group positions, the tiles that see the most keys first (ties in the order of the entries); chunks of 256 keys."""
    ppt, few = tile_rows // group, 16 // group
    tiles, items, last = [], [], 0
    for e, (L, p0) in enumerate(zip(counts, firsts)):
        if L <= few:
            items.append(e)
            last = max(last, p0 + L - 1)
        else:
            tiles += [(p0 + min(L, (t + 1) * ppt), e, t) for t in range(-(-L // ppt))]
    tiles.sort(key=lambda k: -k[0])
    return [x for _, e, t in tiles for x in (e, t)] + items, len(tiles), len(items), (last // 256 + 1 if items else 0)


@pytest.mark.parametrize("seed", range(6))
def test_tile_plans_match_their_restatement(seed):
    lib = _runtime()
    rng = random.Random(seed)
    program = lib.sb_program_create(R, WORK)
    keys = [(4, 128, 8, 296), (1, 64, 3, -1), (16, 64, 2, 10)]
    plans = [lib.sb_program_plan(program, *k) for k in keys]
    assert plans == [0, 1, 2] and lib.sb_program_plan(program, *keys[1]) == 1       # equal requests share a plan
    E = rng.randint(1, 9)
    counts = [rng.choice([1, 1, 2, 3, 5, 17, 40]) for _ in range(E)]
    while sum(counts) > R:
        counts[counts.index(max(counts))] = 1
    firsts = [rng.randint(0, 700) for _ in range(E)]
    count, first = np.asarray(counts, dtype=np.int32), np.asarray(firsts, dtype=np.int32)
    staging = np.full(9 * R + WORK, -7, dtype=np.int32)
    step = SbStep()
    rc = lib.sb_program_prepare(program, E, count.ctypes.data_as(_I32P), first.ctypes.data_as(_I32P), int(count.sum()), 3, 0,
                                staging.ctypes.data_as(_I32P), 4096, ctypes.byref(step))
    assert rc == 0, lib.sb_last_error().decode()
    assert (step.n, step.entries, step.wanted, step.max_rows, step.n_plans, step.ints) == (int(count.sum()), E, 3, R, 3, 4096)
    assert (staging[:9 * R] == -7).all()                                           # only the work lists are written
    for k, (group, tile_rows, kv_heads, limit) in enumerate(keys):
        work, tiles, items, chunks = _plain_plan(counts, firsts, group, tile_rows)
        p = step.plan[k]
        assert (p.tiles, p.items, p.chunks) == (tiles, items, chunks)
        got = staging[9 * R + p.work_offset:9 * R + p.work_offset + len(work)].tolist()
        assert got == work
        assert bool(p.fused) == (tiles == 0 and items > 0 and limit >= 0 and items * kv_heads * chunks <= limit)
    # a recorded decode step: every entry one item, chunks from the key range it was recorded for
    rc = lib.sb_program_prepare(program, 5, None, None, 5, 5, 1024, staging.ctypes.data_as(_I32P), 4096, ctypes.byref(step))
    assert rc == 0
    p = step.plan[0]
    assert (p.tiles, p.items, p.chunks, step.static_keys) == (0, 5, 4, 1024)
    assert staging[9 * R + p.work_offset:9 * R + p.work_offset + 5].tolist() == [0, 1, 2, 3, 4]
    lib.sb_program_destroy(program)


def test_work_lists_that_do_not_fit_and_too_many_plans_are_refused():
    lib = _runtime()
    program = lib.sb_program_create(R, 8)
    assert lib.sb_program_plan(program, 1, 64, 1, -1) == 0
    count, first = np.asarray([1] * 20, dtype=np.int32), np.zeros(20, dtype=np.int32)
    staging = np.zeros(9 * R + 8, dtype=np.int32)
    step = SbStep()
    rc = lib.sb_program_prepare(program, 20, count.ctypes.data_as(_I32P), first.ctypes.data_as(_I32P), 20, 0, 0,
                                staging.ctypes.data_as(_I32P), 0, ctypes.byref(step))
    assert rc < 0 and "work lists" in lib.sb_last_error().decode()
    for k in range(1, 4):
        assert lib.sb_program_plan(program, 1, 64, 1 + k, -1) == k
    assert lib.sb_program_plan(program, 2, 64, 1, -1) < 0 and "at most" in lib.sb_last_error().decode()
    assert lib.sb_program_plan(program, 32, 64, 1, -1) < 0
    lib.sb_program_destroy(program)


_CALLS = []
_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(SbOp), ctypes.POINTER(SbStep), ctypes.c_void_p)


@_FN
def _record(op, step, stream):
    _CALLS.append((op.contents.i[0], step.contents.n, op.contents.f[0]))
    return int(op.contents.i[1])


def test_operations_run_in_order_and_may_skip_or_fail():
    lib = _runtime()
    program = lib.sb_program_create(R, WORK)
    for tag, rc in ((10, 0), (11, 2), (12, 0), (13, 1), (14, 0)):      # launched, skipped, launched, failed, never reached
        op = SbOp()
        op.fn = ctypes.cast(_record, ctypes.c_void_p).value
        op.i[0], op.i[1], op.f[0] = tag, rc, tag / 2
        assert lib.sb_program_add(program, ctypes.byref(op)) == tag - 10
    assert lib.sb_program_size(program) == 5
    step = SbStep()
    step.n = 7
    failed, launched = ctypes.c_int32(-1), ctypes.c_int32(-1)
    del _CALLS[:]
    rc = lib.sb_program_run(program, ctypes.byref(step), None, ctypes.byref(failed), ctypes.byref(launched))
    assert rc == -1 and failed.value == 3 and launched.value == 2
    assert _CALLS == [(10, 7, 5.0), (11, 7, 5.5), (12, 7, 6.0), (13, 7, 6.5)]
    empty = SbOp()
    assert lib.sb_program_add(program, ctypes.byref(empty)) < 0
    lib.sb_program_destroy(program)


def test_an_operation_may_stand_for_those_behind_it():
    """`covers`: when the operation launches, the runner passes over the covered ones; when it skips, they run."""
    lib = _runtime()
    for first_rc, expect in ((0, [20, 23]), (2, [20, 21, 22, 23])):
        program = lib.sb_program_create(R, WORK)
        for tag, rc in ((20, first_rc), (21, 0), (22, 0), (23, 0)):
            op = SbOp()
            op.fn = ctypes.cast(_record, ctypes.c_void_p).value
            op.i[0], op.i[1] = tag, rc
            lib.sb_program_add(program, ctypes.byref(op))
        assert lib.sb_program_set_covers(program, 0, 2) == 0
        assert lib.sb_program_set_covers(program, 2, 2) < 0 and "follow" in lib.sb_last_error().decode()     # beyond the end
        step = SbStep()
        failed, launched = ctypes.c_int32(-1), ctypes.c_int32(-1)
        del _CALLS[:]
        assert lib.sb_program_run(program, ctypes.byref(step), None, ctypes.byref(failed), ctypes.byref(launched)) == 0
        assert [c[0] for c in _CALLS] == expect
        assert launched.value == (2 if first_rc == 0 else 3)
        lib.sb_program_destroy(program)


def test_an_operation_without_a_phase_ends_the_building_of_the_chain(tmp_path):
    """Parts name their phase of the decode chain beside their operation; one operation that names none (a part from
    outside the package) and the layers have no chain: the placeholder operation stays and always skips."""
    from stride_b200.kernels.native import NO_PHASE, NotNative, StepProgram
    src = tmp_path / "phase_less.cu"
    src.write_text('#include "common.cuh"\n#include "step_ops.h"\nSB_DEFINE_LAST_ERROR()\n'
                   'SB_EXPORT int phase_less_op(const SbOp*, const SbStep*, void*) { return SB_OP_SKIPPED; }\n')
    register_kernel_library("phase_less_library", src)
    program = StepProgram(None, 64, 64, 512)
    program.begin_chain()
    assert program.chain is not None and len(program) == 1
    program.add("phase_less_library", "phase_less_op", [1], chain=NO_PHASE)
    assert program.chain is not None
    seen = []
    program.add("phase_less_library", "phase_less_op", [2], chain=lambda chain: seen.append(chain))
    assert program.chain is not None and seen == [program.chain]

    def refuses(chain):
        raise NotNative("this shape has no phase")
    program.add("phase_less_library", "phase_less_op", [3], chain=refuses)
    assert program.chain is None
    program.begin_chain()
    program.add("phase_less_library", "phase_less_op", [4])          # no phase named at all
    assert program.chain is None
    assert program.end_chain() is False and program.chains == []


def test_a_blocks_roles_are_checked():
    import torch

    from stride_b200.parts import BuildEnv, DecoderModel, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    norm = PartSpec("rmsnorm", {"size": 8, "eps": 1e-5}, {"weight": "n"})
    ff = PartSpec("swiglu", {"hidden_size": 8, "intermediate_size": 16}, {"gate": "g", "up": "u", "down": "d"})
    mixer = PartSpec("attention", {"hidden_size": 8, "num_heads": 2, "num_kv_heads": 1, "head_dim": 4, "position": None},
                     {"q": "q", "k": "k", "v": "v", "o": "o"})

    def model(layer):
        spec = ModelSpec(vocab_size=16, hidden_size=8, embedding=PartSpec("lookup", {"vocab_size": 16, "hidden_size": 8}, {"weight": "e"}),
                         layers=(layer,), schedule=(ScheduleEntry(0),), final_norm=norm,
                         head=PartSpec("linear", {"vocab_size": 16, "hidden_size": 8, "tied": True}, {"weight": "h", "tied_to": "e"}), max_positions=32)
        return DecoderModel(spec, BuildEnv(device=torch.device("cpu"), compute_dtype=torch.float32, max_tokens=4, max_positions=32))

    whole = LayerSpec("prenorm", mixer=mixer, feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm)
    assert whole == LayerSpec(mixer, ff, norm, norm) and whole.mixer is mixer and whole.block == "prenorm"
    assert set(model(whole).blocks[0].parts) == {"mixer", "feed_forward", "mixer_norm", "feed_forward_norm"}
    with pytest.raises(ValueError, match="missing: feed_forward_norm"):
        model(LayerSpec("prenorm", mixer=mixer, feed_forward=ff, mixer_norm=norm))
    with pytest.raises(ValueError, match="has no role extra_norm"):
        model(LayerSpec("prenorm", mixer=mixer, feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm, extra_norm=norm))
    with pytest.raises(KeyError, match="no block part of kind 'sandwich'"):
        model(LayerSpec("sandwich", mixer=mixer))
    with pytest.raises(AttributeError, match="no part in the role"):
        whole.router
    with pytest.raises(TypeError):
        LayerSpec("prenorm", mixer="attention")


def test_a_kernel_library_from_outside_the_package(tmp_path):
    src = tmp_path / "outside.cu"
    src.write_text('#include "common.cuh"\n#include "step_ops.h"\nSB_DEFINE_LAST_ERROR()\n'
                   'SB_EXPORT int outside_answer(const SbOp* op, const SbStep* s, void*) { return op->i[0] == 42 && s->n == 1 ? SB_OP_SKIPPED : sb::fail("no"); }\n')
    register_kernel_library("outside_test_library", src)
    register_kernel_library("outside_test_library", src)                     # again with the same source: fine
    with pytest.raises(BuildError, match="another source"):
        register_kernel_library("outside_test_library", __file__)
    with pytest.raises(BuildError, match="no source file"):
        register_kernel_library("nowhere", tmp_path / "missing.cu")
    with pytest.raises(BuildError, match="no kernel library named"):
        library("never_registered")
    lib = library("outside_test_library")                                    # compiled by nvcc for sm_100a, no GPU needed
    op, step = SbOp(), SbStep()
    op.i[0], step.n = 42, 1
    lib.outside_answer.argtypes = [ctypes.POINTER(SbOp), ctypes.POINTER(SbStep), ctypes.c_void_p]
    assert lib.outside_answer(ctypes.byref(op), ctypes.byref(step), None) == 2
    op.i[0] = 41
    assert lib.outside_answer(ctypes.byref(op), ctypes.byref(step), None) == 1 and lib.sb_last_error() == b"no"
