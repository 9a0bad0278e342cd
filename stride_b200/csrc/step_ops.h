// The native step program: what a step of the engine is once Python is out of the way.
//
// A model's parts describe their share of a step ONCE, when the engine is built, as a list of operations
// (`SbOp`): a function of the kernel library that launches it, and the operation's fixed arguments (buffer
// addresses, sizes, constants). Every step then fills one `SbStep` (how many tokens, entries and wanted rows it
// has, where its integer inputs lie on the device, how its entries are cut into attention tiles) and the runner
// (`sb_program_run` in runtime.cpp) calls the operations one after another on the stream, with no interpreter
// between two launches. Counterpart in arhaamatiq/stride: Engine::step_tensor_core / step_exact, which launch the
// layer sequence from C++ (src/engine.cpp:144-462).
//
// An operation function has the signature `int fn(const SbOp*, const SbStep*, void* stream)` and returns
// SB_OP_LAUNCHED, SB_OP_FAILED (the reason is in its library's sb_last_error()) or SB_OP_SKIPPED (this step needs
// nothing of it). Any library may provide operations; the runner knows none of them by name.
//
// An operation may stand for the `covers` operations that follow it (one kernel that does the work of many, for the
// steps it is made for): when it launches, the runner passes over those; when it skips, they run as usual.
#pragma once

#include <stdint.h>

#define SB_OP_LAUNCHED 0
#define SB_OP_FAILED 1
#define SB_OP_SKIPPED 2

#define SB_MAX_PLANS 4
#define SB_OP_INTS 28
#define SB_OP_FLOATS 4

// How the entries of a step are cut for the tensor-core attention kernels of one head ratio: entries of at most
// 16 / group tokens are "items" of the split-key decode kernel, longer ones are cut into tiles of tile_rows / group
// positions. `work` (on the device, at ints + 9 * max_rows + work_offset) holds (entry, tile) pairs, the tiles that
// see the most keys first, then the items' entries. chunks: 256-key chunks the longest item spans.
typedef struct SbTilePlan {
  int32_t group, tile_rows, kv_heads, fused_limit;   // the key: what a mixer asked for
  int32_t work_offset, tiles, items, chunks;
  int32_t fused;        // the step has items only and few enough CTAs: rotation and append run inside the decode kernel
  int32_t reserved[3];
} SbTilePlan;

typedef struct SbStep {
  int32_t n;             // tokens of the step (a recorded decode step: its padded batch)
  int32_t entries;       // requests of the step
  int32_t wanted;        // rows whose logits are wanted
  int32_t static_keys;   // > 0: a decode step recorded into a CUDA graph; no key lies at or beyond this position
  int32_t max_rows;      // R: the regions of `ints` are R apart
  int32_t n_plans;
  // The step's integer inputs on the device: tokens [0, R), positions [R, 2R), slots [2R, 3R), wanted rows [3R, 4R),
  // entry records [4R, 8R) (slot, first row, length, first position: four rows of R), the slot of every wanted
  // row [8R, 9R), work lists from 9R on.
  const int32_t* ints;
  SbTilePlan plan[SB_MAX_PLANS];
} SbStep;

typedef struct SbOp {
  void* fn;                    // SbOpFn
  int64_t i[SB_OP_INTS];       // the operation's own integer and pointer arguments (see each sb_op_* function)
  double f[SB_OP_FLOATS];
  int64_t covers;              // > 0: when this operation launches, the next `covers` operations do not run
} SbOp;

typedef int (*SbOpFn)(const SbOp*, const SbStep*, void*);

#ifdef __cplusplus
namespace sbstep {
inline const int32_t* tokens(const SbStep* s) { return s->ints; }
inline const int32_t* positions(const SbStep* s) { return s->ints + s->max_rows; }
inline const int32_t* slots(const SbStep* s) { return s->ints + 2 * static_cast<int64_t>(s->max_rows); }
inline const int32_t* wanted_rows(const SbStep* s) { return s->ints + 3 * static_cast<int64_t>(s->max_rows); }
inline const int32_t* entry_meta(const SbStep* s) { return s->ints + 4 * static_cast<int64_t>(s->max_rows); }
inline const int32_t* work(const SbStep* s, const SbTilePlan& p) { return s->ints + 9 * static_cast<int64_t>(s->max_rows) + p.work_offset; }
// Partial sums that a projection with K ranges left: [P, n, M] with P = S up to `few` tokens, else 1.
inline int partial_count(int64_t S, int64_t few, int n) { return (S > 1 && n <= few) ? static_cast<int>(S) : 1; }
template <class T>
inline T* ptr(int64_t v) { return reinterpret_cast<T*>(static_cast<intptr_t>(v)); }
}  // namespace sbstep
#endif
