// The host side of the cache manager and of the scheduler's decisions, in C++ behind a plain C interface.
//
// Pool: the books of the paged cache. Pages of every group (layers with the same kind of cache), a last-in-first-out
// free list per group, a slot per request, and the block tables, which are rows of memory that the caller owns
// (pinned host memory that is uploaded row by row): the pool writes page ids straight into them. A page is free or
// held by exactly one live slot. Counterpart in arhaamatiq/stride: KvCache (src/kv_cache.cpp:10-92), which has one
// group, no windows and the same last-in-first-out order.
//
// Planner and Sched: which tokens the next step runs. Requests with exactly one unprocessed token first (one row each), then
// portions of prompts in running order, under the token budget; then the page arithmetic of that plan, and what to
// do when pages run short (wait for steps in flight, preempt the youngest, or fail when one request alone does not
// fit). Counterpart: Scheduler::Admit / BuildBatch (src/scheduler.cpp:72-304).
//
// Nothing here touches a GPU; it is compiled by the host compiler alone.
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#define SB_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int32_t kNoPage = -1;
thread_local std::string g_error;

uint64_t splitmix64(uint64_t& s) {
  uint64_t z = (s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

struct Group {
  int window = 0;
  int num_pages = 0;
  int32_t* table = nullptr;            // [max_slots + 1, max_pages_per_seq], kNoPage where nothing is held
  std::vector<int32_t> free;           // back = next page handed out
  std::vector<int32_t> first, last;    // per slot: the indices [first, last) are the only ones that can hold a page
  std::vector<int32_t> count;          // per slot: pages held
};

struct Pool {
  int page_size = 0, max_slots = 0, max_pages = 0, max_context = 0;
  std::vector<Group> groups;
  std::vector<int32_t> free_slots;     // back = next slot handed out
  int32_t* length = nullptr;           // [max_slots], caller's memory: tokens the slot's pages have been ensured for
  uint8_t* live = nullptr;             // [max_slots], caller's memory
  std::vector<uint8_t> dirty_mark;     // [groups * (max_slots + 1)]
  std::vector<int32_t> dirty;          // group * (max_slots + 1) + slot of rows that changed
  bool shuffle = false;
  uint64_t rng = 0;

  int32_t* row(Group& g, int slot) { return g.table + (size_t)slot * max_pages; }
  void touch(int gi, int slot) {
    const int key = gi * (max_slots + 1) + slot;
    if (!dirty_mark[key]) {
      dirty_mark[key] = 1;
      dirty.push_back(key);
    }
  }
  void reshuffle(Group& g) {
    for (size_t i = g.free.size(); i > 1; --i) std::swap(g.free[i - 1], g.free[splitmix64(rng) % i]);
  }
  bool slot_ok(int slot) const { return slot >= 0 && slot < max_slots && live[slot]; }

  // Pages the slot lacks for tokens [start, end): indices are appended to `out` if it is given.
  int wanted(Group& g, int slot, int start, int end, std::vector<int32_t>* out) {
    if (end <= start) return 0;
    const int32_t* r = row(g, slot);
    int n = 0;
    for (int i = start / page_size, e = (end - 1) / page_size; i <= e; ++i)
      if (r[i] == kNoPage) {
        ++n;
        if (out) out->push_back(i);
      }
    return n;
  }
};

enum PlanResult { kPlanRun = 0, kPlanNothing = 1, kPlanDrain = 2, kPlanTooSmall = 3, kPlanPreempt = 4 };

}  // namespace

SB_API const char* sb_last_error() { return g_error.c_str(); }

// `tables[g]` points at group g's block table [max_slots + 1, max_pages_per_seq] (already filled with -1), `length`
// and `live` at arrays of max_slots entries (zeroed). A shuffle_seed other than 0 permutes the free lists at the
// start and after every page given back, so that tests see pages in every order.
SB_API void* sb_pool_create(int n_groups, const int32_t* windows, int32_t* const* tables, int page_size, int num_pages,
                            int max_slots, int max_pages_per_seq, int max_context, int32_t* length, uint8_t* live,
                            uint64_t shuffle_seed) {
  if (page_size <= 0 || max_slots <= 0 || max_pages_per_seq <= 0 || n_groups < 0 || (n_groups && num_pages <= 0)) {
    g_error = "sb_pool_create: sizes must be positive";
    return nullptr;
  }
  Pool* p = new Pool;
  p->page_size = page_size;
  p->max_slots = max_slots;
  p->max_pages = max_pages_per_seq;
  p->max_context = max_context;
  p->length = length;
  p->live = live;
  p->shuffle = shuffle_seed != 0;
  p->rng = shuffle_seed;
  p->groups.resize(n_groups);
  p->dirty_mark.assign((size_t)n_groups * (max_slots + 1), 0);
  for (int s = max_slots - 1; s >= 0; --s) p->free_slots.push_back(s);
  for (int gi = 0; gi < n_groups; ++gi) {
    Group& g = p->groups[gi];
    g.window = windows[gi];
    g.num_pages = num_pages;
    g.table = tables[gi];
    for (int pg = num_pages - 1; pg >= 0; --pg) g.free.push_back(pg);   // page 0 is handed out first
    if (p->shuffle) p->reshuffle(g);
    g.first.assign(max_slots, 0);
    g.last.assign(max_slots, 0);
    g.count.assign(max_slots, 0);
  }
  return p;
}

SB_API void sb_pool_destroy(void* pool) { delete static_cast<Pool*>(pool); }

// A free slot id, or -1 when every slot is taken.
SB_API int sb_pool_acquire_slot(void* pool) {
  Pool* p = static_cast<Pool*>(pool);
  if (p->free_slots.empty()) return -1;
  const int slot = p->free_slots.back();
  p->free_slots.pop_back();
  p->live[slot] = 1;
  p->length[slot] = 0;
  return slot;
}

// Gives back the slot and every page it holds. 0, or -1 if the slot is not held.
SB_API int sb_pool_release_slot(void* pool, int slot) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p->slot_ok(slot)) return -1;
  for (size_t gi = 0; gi < p->groups.size(); ++gi) {
    Group& g = p->groups[gi];
    if (!g.count[slot]) continue;
    int32_t* r = p->row(g, slot);
    for (int i = g.first[slot]; i < g.last[slot]; ++i)
      if (r[i] != kNoPage) {
        g.free.push_back(r[i]);
        r[i] = kNoPage;
      }
    g.count[slot] = g.first[slot] = g.last[slot] = 0;
    p->touch((int)gi, slot);
    if (p->shuffle) p->reshuffle(g);
  }
  p->live[slot] = 0;
  p->length[slot] = 0;
  p->free_slots.push_back(slot);
  return 0;
}

// Per group, how many new pages the slot needs to hold tokens up to position end - 1.
SB_API int sb_pool_pages_needed(void* pool, int slot, int end, int32_t* out) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p->slot_ok(slot)) return -1;
  end = std::min(end, p->max_pages * p->page_size);
  for (size_t gi = 0; gi < p->groups.size(); ++gi) out[gi] = p->wanted(p->groups[gi], slot, p->length[slot], end, nullptr);
  return 0;
}

SB_API void sb_pool_free_pages(void* pool, int32_t* out) {
  Pool* p = static_cast<Pool*>(pool);
  for (size_t gi = 0; gi < p->groups.size(); ++gi) out[gi] = (int32_t)p->groups[gi].free.size();
}

SB_API int sb_pool_free_slots(void* pool, int32_t* out, int capacity) {
  Pool* p = static_cast<Pool*>(pool);
  const int n = (int)p->free_slots.size();
  for (int i = 0; i < n && i < capacity; ++i) out[i] = p->free_slots[i];
  return n;
}

// The free list of a group, the next page to be handed out last.
SB_API int sb_pool_free_list(void* pool, int group, int32_t* out, int capacity) {
  Pool* p = static_cast<Pool*>(pool);
  const Group& g = p->groups[group];
  const int n = (int)g.free.size();
  for (int i = 0; i < n && i < capacity; ++i) out[i] = g.free[i];
  return n;
}

// Allocates pages so that the slot can hold tokens up to position end - 1. 1 = done, 0 = a group has too few free
// pages (nothing changed), -1 = the slot is not held, -2 = beyond the context capacity.
SB_API int sb_pool_ensure(void* pool, int slot, int end) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p->slot_ok(slot)) return -1;
  if (end > p->max_context) return -2;
  const int start = p->length[slot];
  for (Group& g : p->groups)
    if (p->wanted(g, slot, start, end, nullptr) > (int)g.free.size()) return 0;
  std::vector<int32_t> idx;
  for (size_t gi = 0; gi < p->groups.size(); ++gi) {
    Group& g = p->groups[gi];
    idx.clear();
    p->wanted(g, slot, start, end, &idx);
    if (idx.empty()) continue;
    int32_t* r = p->row(g, slot);
    for (int i : idx) {
      r[i] = g.free.back();
      g.free.pop_back();
    }
    if (!g.count[slot]) {
      g.first[slot] = idx.front();
      g.last[slot] = idx.back() + 1;
    } else {
      g.first[slot] = std::min(g.first[slot], idx.front());
      g.last[slot] = std::max(g.last[slot], idx.back() + 1);
    }
    g.count[slot] += (int)idx.size();
    p->touch((int)gi, slot);
  }
  p->length[slot] = std::max(p->length[slot], end);
  return 1;
}

// Gives back the pages of windowed groups that no token of the slot at position `length` or later can see
// (length < 0: all tokens the slot has pages for). Returns pages freed, -1 if the slot is not held.
SB_API int sb_pool_trim(void* pool, int slot, int length) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p->slot_ok(slot)) return -1;
  const int n = length < 0 ? p->length[slot] : std::min(length, p->length[slot]);
  int freed = 0;
  for (size_t gi = 0; gi < p->groups.size(); ++gi) {
    Group& g = p->groups[gi];
    if (g.window <= 0 || !g.count[slot]) continue;
    const int first_needed = n - g.window + 1;      // the oldest key the next token (position n) reads
    if (first_needed < p->page_size) continue;
    const int keep_from = first_needed / p->page_size;    // index i goes when (i + 1) * page_size <= first_needed
    int32_t* r = p->row(g, slot);
    int here = 0;
    for (int i = g.first[slot], e = std::min(keep_from, g.last[slot]); i < e; ++i)
      if (r[i] != kNoPage) {
        g.free.push_back(r[i]);
        r[i] = kNoPage;
        ++here;
      }
    if (here) {
      g.count[slot] -= here;
      g.first[slot] = std::max(g.first[slot], std::min(keep_from, g.last[slot]));
      p->touch((int)gi, slot);
      freed += here;
    }
    if (freed && p->shuffle) p->reshuffle(g);
  }
  return freed;
}

// The (group, slot) rows that changed since the last call, sorted, as pairs in `out`; the marks are cleared.
SB_API int sb_pool_take_dirty(void* pool, int32_t* out, int capacity_pairs) {
  Pool* p = static_cast<Pool*>(pool);
  std::sort(p->dirty.begin(), p->dirty.end());
  const int n = (int)p->dirty.size();
  if (n > capacity_pairs) return -n;
  for (int i = 0; i < n; ++i) {
    out[2 * i] = p->dirty[i] / (p->max_slots + 1);
    out[2 * i + 1] = p->dirty[i] % (p->max_slots + 1);
    p->dirty_mark[p->dirty[i]] = 0;
  }
  p->dirty.clear();
  return n;
}

SB_API int sb_pool_held_count(void* pool, int group, int slot) {
  Pool* p = static_cast<Pool*>(pool);
  return p->groups[group].count[slot];
}

// Invariants: every page is free or held by exactly one live slot, never both or twice; no slot is lost.
// 0, or -1 with the finding in sb_last_error().
SB_API int sb_pool_check(void* pool) {
  Pool* p = static_cast<Pool*>(pool);
  char msg[160];
  for (size_t gi = 0; gi < p->groups.size(); ++gi) {
    Group& g = p->groups[gi];
    std::vector<int32_t> owner(g.num_pages, -2);      // -2 unseen, -1 free, else the slot
    size_t seen = 0;
    for (int32_t pg : g.free) {
      if (pg < 0 || pg >= g.num_pages) {
        snprintf(msg, sizeof msg, "page id %d on the free list is out of range", pg);
        g_error = msg;
        return -1;
      }
      if (owner[pg] != -2) {
        snprintf(msg, sizeof msg, "page %d is on the free list twice", pg);
        g_error = msg;
        return -1;
      }
      owner[pg] = -1;
      ++seen;
    }
    for (int slot = 0; slot < p->max_slots; ++slot) {
      const int32_t* r = p->row(g, slot);
      int count = 0;
      for (int i = 0; i < p->max_pages; ++i) {
        const int32_t pg = r[i];
        if (pg == kNoPage) continue;
        ++count;
        if (!p->live[slot]) {
          snprintf(msg, sizeof msg, "slot %d holds pages but is not live", slot);
          g_error = msg;
          return -1;
        }
        if (pg < 0 || pg >= g.num_pages || i < g.first[slot] || i >= g.last[slot]) {
          snprintf(msg, sizeof msg, "block table of slot %d disagrees at index %d", slot, i);
          g_error = msg;
          return -1;
        }
        if (owner[pg] != -2) {
          if (owner[pg] == -1) snprintf(msg, sizeof msg, "page %d is held by slot %d and is also free", pg, slot);
          else snprintf(msg, sizeof msg, "page %d is held by slot %d and is also held by slot %d", pg, slot, owner[pg]);
          g_error = msg;
          return -1;
        }
        owner[pg] = slot;
        ++seen;
      }
      if (count != g.count[slot]) {
        snprintf(msg, sizeof msg, "slot %d holds %d pages but %d are counted", slot, count, g.count[slot]);
        g_error = msg;
        return -1;
      }
    }
    if (seen != (size_t)g.num_pages) {
      snprintf(msg, sizeof msg, "%d pages are lost", (int)(g.num_pages - seen));
      g_error = msg;
      return -1;
    }
    if (p->row(g, p->max_slots)[0] != g.num_pages) {
      g_error = "the padding slot lost its page";
      return -1;
    }
  }
  std::vector<uint8_t> is_free(p->max_slots, 0);
  int live = 0;
  for (int32_t s : p->free_slots) {
    if (s < 0 || s >= p->max_slots || is_free[s] || p->live[s]) {
      g_error = "slot bookkeeping is inconsistent";
      return -1;
    }
    is_free[s] = 1;
  }
  for (int s = 0; s < p->max_slots; ++s) live += p->live[s] != 0;
  if ((int)p->free_slots.size() + live != p->max_slots) {
    g_error = "a slot is lost";
    return -1;
  }
  return 0;
}

// Whether a waiting request of `tokens` tokens may start beside n_running others: free pages of every group must
// cover its tokens plus one page of growth per running request plus one, unless nothing is running.
SB_API int sb_sched_may_admit(void* pool, int n_running, int tokens) {
  Pool* p = static_cast<Pool*>(pool);
  if (p->free_slots.empty()) return 0;
  if (n_running == 0) return 1;
  const int need = (tokens + p->page_size - 1) / p->page_size + n_running + 1;
  for (const Group& g : p->groups)
    if ((int)g.free.size() < need) return 0;
  return 1;
}

// Plans the next step over the running requests (arrays in running order: slot, next unprocessed position, tokens
// known, closing = no further step is to be launched, inflight = steps launched whose tokens the host has not read,
// arrival number). Result kPlanRun: `out_index[i]`, `out_count[i]` for i < *out_n are the requests and how many of
// their tokens run, pages ensured. kPlanNothing: no request has a token to run. kPlanDrain: pages are short while
// steps are in flight. kPlanTooSmall: pages are short for a single request. kPlanPreempt: pages are short;
// out_index[0] is the youngest request, which the caller takes out before it plans again. -1: accounting failed.
SB_API int sb_sched_plan(void* pool, int n, const int32_t* slot, const int32_t* next_pos, const int32_t* total,
                         const uint8_t* closing, const uint8_t* inflight, const int64_t* arrival, int max_rows,
                         int prefill_chunk, int32_t* out_index, int32_t* out_count, int32_t* out_n) {
  Pool* p = static_cast<Pool*>(pool);
  int budget = max_rows, m = 0;
  for (int i = 0; i < n && budget > 0; ++i)
    if (total[i] - next_pos[i] == 1 && !closing[i]) {
      out_index[m] = i;
      out_count[m++] = 1;
      --budget;
    }
  for (int i = 0; i < n && budget > 0; ++i) {
    const int remaining = total[i] - next_pos[i];
    if (remaining > 1 && !closing[i]) {
      const int chunk = std::min(remaining, std::min(prefill_chunk, budget));
      out_index[m] = i;
      out_count[m++] = chunk;
      budget -= chunk;
    }
  }
  *out_n = m;
  if (m == 0) return kPlanNothing;
  for (int j = 0; j < m; ++j)
    if (!p->slot_ok(slot[out_index[j]])) {
      g_error = "sb_sched_plan: a running request has no slot";
      return -1;
    }
  bool is_short = false;
  for (Group& g : p->groups) {
    long need = 0;
    for (int j = 0; j < m; ++j) {
      const int i = out_index[j], s = slot[i];
      need += p->wanted(g, s, p->length[s], std::min(next_pos[i] + out_count[j], p->max_pages * p->page_size), nullptr);
    }
    if (need > (long)g.free.size()) is_short = true;
  }
  if (is_short) {
    for (int i = 0; i < n; ++i)
      if (inflight[i]) return kPlanDrain;     // pages of a request with a step in flight cannot be taken away yet
    if (n <= 1) return kPlanTooSmall;
    int victim = 0;
    for (int i = 1; i < n; ++i)
      if (arrival[i] > arrival[victim]) victim = i;
    out_index[0] = victim;
    return kPlanPreempt;
  }
  for (int j = 0; j < m; ++j) {
    const int i = out_index[j];
    const int r = sb_pool_ensure(pool, slot[i], next_pos[i] + out_count[j]);
    if (r == -2) {
      g_error = "sb_sched_plan: a request grows beyond the context capacity";
      return -1;
    }
    if (r != 1) {
      g_error = "page accounting failed: ensure() refused a planned allocation";
      return -1;
    }
  }
  return kPlanRun;
}

// ------------------------------------------------------------------ Sched: the requests and their tokens
//
// The scheduler's state and rules: every request's tokens, how far they have been run, what has been generated, which
// requests wait and which run, admission, the plan of a step (with preemption of the youngest when pages are short),
// and what a chosen token means for its request (stop token, length, fingerprint). The caller drives the engine and
// the sampler and keeps what cannot live here (callbacks, sampling parameters). Counterpart in arhaamatiq/stride:
// Scheduler (src/scheduler.cpp:72-304), whose policy this is; running one step ahead is this engine's own.
namespace {

constexpr uint64_t kFnvOffset = 14695981039346656037ull, kFnvPrime = 1099511628211ull;

uint64_t fnv_mix(uint64_t h, uint32_t v) {
  for (int i = 0; i < 4; ++i) {
    h ^= (v >> (i * 8)) & 0xFFu;
    h *= kFnvPrime;
  }
  return h;
}

// One turn of the batch-order shuffle's generator: the state becomes the mixed value.
uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

struct Seq {
  std::vector<int32_t> tokens;     // prompt, then generated tokens; -1 stands for a token that is being chosen
  std::vector<int32_t> stops;
  int prompt_len = 0, next_pos = 0, generated = 0, launched = 0, inflight = 0, slot = -1, max_new = 0;
  int64_t arrival = 0;
  uint64_t fingerprint = kFnvOffset;
  bool closing = false, done = false, cancelled = false, live = false;
};

struct SchedStats {
  int64_t steps = 0, rows = 0, generated = 0, preemptions = 0, replayed_rows = 0, peak_seqs = 0, peak_blocks = 0;
};

struct Sched {
  Pool* pool = nullptr;
  int max_seqs = 0, max_rows = 0, prefill_chunk = 0, max_context = 0;
  uint64_t shuffle_state = 0;
  bool shuffle = false;
  std::vector<Seq> seqs;             // by id; ids of finished requests are used again
  std::vector<int32_t> free_ids;
  std::vector<int32_t> waiting;      // front = next to be admitted
  std::vector<int32_t> running;      // in the order of admission
  int64_t next_arrival = 0;
  SchedStats stats;
  // scratch of the planner
  std::vector<int32_t> a_slot, a_next, a_total, o_index, o_count;
  std::vector<uint8_t> a_closing, a_inflight;
  std::vector<int64_t> a_arrival;

  void release(Seq& s) {
    if (s.slot >= 0) {
      sb_pool_release_slot(pool, s.slot);
      s.slot = -1;
    }
  }
  void retire(int id) {       // the request is over and holds nothing: its id may be used again
    Seq& s = seqs[id];
    s.live = false;
    s.tokens.clear();
    s.tokens.shrink_to_fit();
    free_ids.push_back(id);
  }
  void drop_finished() {
    size_t k = 0;
    for (int id : running) {
      Seq& s = seqs[id];
      if ((s.done && s.slot < 0) || !s.live) {
        if (s.live) retire(id);
      } else {
        running[k++] = id;
      }
    }
    running.resize(k);
  }
};

}  // namespace

SB_API void* sb_sched_create(void* pool, int max_seqs, int max_rows, int prefill_chunk, int max_context, uint64_t row_shuffle_seed) {
  if (!pool || max_seqs <= 0 || max_rows <= 0 || prefill_chunk <= 0) {
    g_error = "sb_sched_create: sizes must be positive";
    return nullptr;
  }
  Sched* s = new Sched;
  s->pool = static_cast<Pool*>(pool);
  s->max_seqs = max_seqs;
  s->max_rows = max_rows;
  s->prefill_chunk = prefill_chunk;
  s->max_context = max_context;
  s->shuffle = row_shuffle_seed != 0;
  s->shuffle_state = row_shuffle_seed;
  return s;
}

SB_API void sb_sched_destroy(void* sched) { delete static_cast<Sched*>(sched); }

// Takes a request in. Returns its id (>= 0), -1 for an empty prompt, -2 for a prompt that leaves no room in the
// context; both refusals use up an arrival number, as an accepted request does.
SB_API int sb_sched_add(void* sched, const int32_t* prompt, int n, int max_new, const int32_t* stops, int n_stops) {
  Sched* sc = static_cast<Sched*>(sched);
  const int64_t arrival = sc->next_arrival++;
  if (n <= 0) return -1;
  const int room = sc->max_context - n;
  if (room <= 0) return -2;
  int id;
  if (!sc->free_ids.empty()) {
    id = sc->free_ids.back();
    sc->free_ids.pop_back();
  } else {
    id = (int)sc->seqs.size();
    sc->seqs.emplace_back();
  }
  Seq& s = sc->seqs[id];
  s = Seq();
  s.tokens.assign(prompt, prompt + n);
  s.stops.assign(stops, stops + n_stops);
  s.prompt_len = n;
  s.max_new = std::min(max_new, room);
  s.arrival = arrival;
  s.live = true;
  sc->waiting.push_back(id);
  return id;
}

// The request is dropped at the next step (or, while one of its steps is in flight, once that has been read back).
SB_API void sb_sched_cancel(void* sched, int id) {
  Sched* sc = static_cast<Sched*>(sched);
  if (id >= 0 && id < (int)sc->seqs.size() && sc->seqs[id].live) sc->seqs[id].cancelled = true;
}

// counts[0] = requests waiting, counts[1] = requests running.
SB_API void sb_sched_counts(void* sched, int32_t* counts) {
  Sched* sc = static_cast<Sched*>(sched);
  counts[0] = (int32_t)sc->waiting.size();
  counts[1] = (int32_t)sc->running.size();
}

SB_API int sb_sched_queue(void* sched, int which, int32_t* out, int capacity) {
  Sched* sc = static_cast<Sched*>(sched);
  const std::vector<int32_t>& q = which == 0 ? sc->waiting : sc->running;
  for (int i = 0; i < (int)q.size() && i < capacity; ++i) out[i] = q[i];
  return (int)q.size();
}

// steps, rows, generated, preemptions, replayed_rows, peak_seqs, peak_blocks
SB_API void sb_sched_stats(void* sched, int64_t* out) {
  const SchedStats& t = static_cast<Sched*>(sched)->stats;
  const int64_t v[7] = {t.steps, t.rows, t.generated, t.preemptions, t.replayed_rows, t.peak_seqs, t.peak_blocks};
  std::memcpy(out, v, sizeof v);
}

// Begins a step: drops cancelled requests, admits waiting ones while slots and pages allow, plans the batch under the
// token budget (preempting the youngest running request while pages are short) and ensures its pages. On kPlanRun the
// entries are ent_id / ent_slot / ent_first / ent_count / ent_last (last: the entry reaches the request's last known
// token, so a token is to be chosen for it), their tokens one after another in `tokens` (-1: a token still being
// chosen), *out_n entries; every request's position has been moved on. Other results leave nothing to run:
// kPlanNothing, kPlanDrain (the steps in flight have to be read back before a decision can be taken), kPlanTooSmall.
SB_API int sb_sched_begin_step(void* sched, int32_t* ent_id, int32_t* ent_slot, int32_t* ent_first, int32_t* ent_count,
                               uint8_t* ent_last, int32_t* tokens, int32_t* out_n) {
  Sched* sc = static_cast<Sched*>(sched);
  Pool* pool = sc->pool;
  *out_n = 0;
  // cancelled requests: while a step of one is in flight nothing can be given back yet
  for (int id : sc->running)
    if (sc->seqs[id].cancelled && sc->seqs[id].inflight > 0) return kPlanDrain;
  {
    size_t k = 0;
    for (int id : sc->running) {
      Seq& s = sc->seqs[id];
      if (s.cancelled) {
        sc->release(s);
        sc->retire(id);
      } else {
        sc->running[k++] = id;
      }
    }
    sc->running.resize(k);
  }
  // admission: room for the request's tokens and one page of growth per running request, and a free slot
  while (!sc->waiting.empty() && (int)sc->running.size() < sc->max_seqs) {
    const int id = sc->waiting.front();
    Seq& s = sc->seqs[id];
    if (s.cancelled) {
      sc->waiting.erase(sc->waiting.begin());
      sc->retire(id);
      continue;
    }
    if (!sb_sched_may_admit(pool, (int)sc->running.size(), (int)s.tokens.size())) break;
    const int slot = sb_pool_acquire_slot(pool);
    if (slot < 0) break;
    s.slot = slot;
    s.next_pos = 0;        // (re)computed from the first token: its pages were given back on preemption
    sc->waiting.erase(sc->waiting.begin());
    sc->running.push_back(id);
  }
  sc->stats.peak_seqs = std::max<int64_t>(sc->stats.peak_seqs, (int64_t)sc->running.size());

  int m = 0;
  while (true) {
    const int n = (int)sc->running.size();
    if (n == 0) return kPlanNothing;
    sc->a_slot.resize(n), sc->a_next.resize(n), sc->a_total.resize(n), sc->a_closing.resize(n), sc->a_inflight.resize(n);
    sc->a_arrival.resize(n), sc->o_index.resize(std::max(n, 1)), sc->o_count.resize(std::max(n, 1));
    for (int i = 0; i < n; ++i) {
      const Seq& s = sc->seqs[sc->running[i]];
      sc->a_slot[i] = s.slot, sc->a_next[i] = s.next_pos, sc->a_total[i] = (int)s.tokens.size();
      sc->a_closing[i] = s.closing, sc->a_inflight[i] = s.inflight > 0, sc->a_arrival[i] = s.arrival;
    }
    int32_t planned = 0;
    const int r = sb_sched_plan(pool, n, sc->a_slot.data(), sc->a_next.data(), sc->a_total.data(), sc->a_closing.data(),
                                sc->a_inflight.data(), sc->a_arrival.data(), sc->max_rows, sc->prefill_chunk, sc->o_index.data(),
                                sc->o_count.data(), &planned);
    if (r == kPlanPreempt) {
      // the youngest goes back to the front of the queue and is later recomputed from its first token
      const int at = sc->o_index[0], id = sc->running[at];
      Seq& victim = sc->seqs[id];
      sc->release(victim);
      sc->stats.preemptions += 1;
      sc->stats.replayed_rows += victim.next_pos;
      sc->running.erase(sc->running.begin() + at);
      sc->waiting.insert(sc->waiting.begin(), id);
      continue;
    }
    if (r != kPlanRun) return r;
    m = planned;
    break;
  }
  if (sc->shuffle)
    for (int i = m - 1; i > 0; --i) {
      sc->shuffle_state = mix64(sc->shuffle_state);
      const int j = (int)(sc->shuffle_state % (uint64_t)(i + 1));
      std::swap(sc->o_index[i], sc->o_index[j]);
      std::swap(sc->o_count[i], sc->o_count[j]);
    }
  int at = 0;
  for (int j = 0; j < m; ++j) {
    const int id = sc->running[sc->o_index[j]], count = sc->o_count[j];
    Seq& s = sc->seqs[id];
    ent_id[j] = id, ent_slot[j] = s.slot, ent_first[j] = s.next_pos, ent_count[j] = count;
    ent_last[j] = s.next_pos + count == (int)s.tokens.size();
    std::memcpy(tokens + at, s.tokens.data() + s.next_pos, sizeof(int32_t) * count);
    at += count;
    s.next_pos += count;
  }
  *out_n = m;
  sc->stats.steps += 1;
  sc->stats.rows += at;
  int64_t used = 0;
  for (const Group& g : pool->groups) used = std::max<int64_t>(used, (int64_t)g.num_pages - (int64_t)g.free.size());
  sc->stats.peak_blocks = std::max(sc->stats.peak_blocks, used);
  return kPlanRun;
}

// The tokens of these requests are being chosen by a step that was queued without waiting for them: each gets a
// placeholder; a request whose last token (by its limit) this is takes part in no further step.
SB_API void sb_sched_launched(void* sched, const int32_t* ids, int n) {
  Sched* sc = static_cast<Sched*>(sched);
  for (int i = 0; i < n; ++i) {
    Seq& s = sc->seqs[ids[i]];
    s.tokens.push_back(-1);
    s.inflight += 1;
    s.launched += 1;
    if (s.launched >= s.max_new) s.closing = true;
  }
}

// The chosen tokens (and their logits) of requests ids[0..n): ahead = 0, the step was waited for: the token is
// appended; ahead = 1, the step had been queued ahead (sb_sched_launched): the token takes the place of the
// request's oldest placeholder, and a request that a stop token finished a step ago ignores its surplus row.
// Per row: kind 0 = ignored, 1 = a token, 2 = a token that stops the request, 3 = a token that reaches its limit;
// the token's index among the generated ones and the fingerprint (FNV-1a over token and logit bits) so far.
// A finished request gives its slot and pages back as soon as none of its steps is in flight.
SB_API void sb_sched_commit(void* sched, int ahead, const int32_t* ids, const int32_t* tokens, const float* values, int n,
                            uint8_t* kind, int32_t* index, uint64_t* fingerprint) {
  Sched* sc = static_cast<Sched*>(sched);
  for (int i = 0; i < n; ++i) {
    Seq& s = sc->seqs[ids[i]];
    kind[i] = 0, index[i] = 0, fingerprint[i] = s.fingerprint;
    if (ahead) {
      s.inflight -= 1;
      if (s.done) {                                   // finished by a stop token a step ago: this row was surplus
        if (s.inflight == 0) sc->release(s);
        continue;
      }
    }
    const int32_t tok = tokens[i];
    uint32_t bits;
    std::memcpy(&bits, &values[i], sizeof bits);
    s.fingerprint = fnv_mix(fnv_mix(s.fingerprint, (uint32_t)tok), bits);
    if (ahead) s.tokens[s.prompt_len + s.generated] = tok;   // the oldest placeholder
    else s.tokens.push_back(tok);
    s.generated += 1;
    sc->stats.generated += 1;
    index[i] = s.generated - 1;
    fingerprint[i] = s.fingerprint;
    kind[i] = 1;
    if (std::find(s.stops.begin(), s.stops.end(), tok) != s.stops.end()) kind[i] = 2;
    else if (s.generated >= s.max_new) kind[i] = 3;
    if (kind[i] >= 2) {
      s.done = s.closing = true;
      if (!ahead || s.inflight == 0) sc->release(s);   // else its slot goes back when the surplus step is read
    }
  }
}

// Ends a step that has finished on the GPU: windowed groups give back the pages behind the window of the requests
// that ran (ids with the position each had reached, or end < 0 for all its tokens), finished requests leave.
SB_API void sb_sched_end_step(void* sched, const int32_t* ids, const int32_t* ends, int n) {
  Sched* sc = static_cast<Sched*>(sched);
  bool windowed = false;
  for (const Group& g : sc->pool->groups) windowed |= g.window > 0;
  if (windowed)
    for (int i = 0; i < n; ++i) {
      const Seq& s = sc->seqs[ids[i]];
      if (s.live && s.slot >= 0 && !s.done) sb_pool_trim(sc->pool, s.slot, ends[i]);
    }
  sc->drop_finished();
}

// ------------------------------------------------------------------ staging a step's integer inputs
//
// One array of 9 R int32 (R = the most rows of a step) carries every integer input of a step to the device in one
// copy: tokens [0, R), positions [R, 2R), slots [2R, 3R), rows whose logits are wanted [3R, 4R), the entries'
// records [4R, 8R) as four rows of R (slot, first row, length, first position), and the slot of every wanted row
// [8R, 9R). These functions check a step against the pool's books and fill that array.
namespace {

int stage_fail(const char* fmt, long a = 0, long b = 0, long c = 0) {
  char msg[200];
  snprintf(msg, sizeof msg, fmt, a, b, c);
  g_error = msg;
  return -1;
}

}  // namespace

// Entries i < E: slot[i], first[i] (position of its first token), count[i] tokens taken one after another from
// `tokens`, n_want[i] places (indices into the entry's tokens) taken one after another from `want`. A token id is
// 0 .. vocab - 1, or -1 for the single token of an entry of one (the token is still being chosen and is read on the
// device). out[0] = rows, out[1] = wanted rows. 0, or -1 with the reason in sb_last_error(); nothing but `staging`
// is written.
SB_API int sb_stage_step(void* pool, int E, const int32_t* slot, const int32_t* first, const int32_t* count, const int32_t* tokens,
                         const int32_t* n_want, const int32_t* want, int vocab, int R, int max_logit_rows, int32_t* staging,
                         int32_t* out) {
  Pool* p = static_cast<Pool*>(pool);
  long n = 0, w_total = 0;
  for (int i = 0; i < E; ++i) {
    if (count[i] <= 0) return stage_fail("a step entry without tokens");
    n += count[i];
    w_total += n_want[i];
  }
  if (n > R) return stage_fail("step of %ld tokens exceeds max_rows %ld", n, R);
  if (w_total > max_logit_rows) return stage_fail("logits wanted at %ld places exceed max_full_rows %ld", w_total, max_logit_rows);
  std::vector<uint8_t> seen(p->max_slots, 0);
  int32_t *tok = staging, *pos = staging + R, *slt = staging + 2 * R, *rows = staging + 3 * R, *meta = staging + 4 * R,
          *row_slot = staging + 8 * R;
  int at = 0, w = 0, wi = 0;
  for (int i = 0; i < E; ++i) {
    const int s = slot[i], L = count[i];
    if (!p->slot_ok(s)) return stage_fail("slot %ld is not held by a request", s);
    if (seen[s]) return stage_fail("slot %ld appears twice in one step", s);
    seen[s] = 1;
    if (first[i] < 0 || first[i] + L > p->length[s])
      return stage_fail("slot %ld: tokens up to position %ld have no pages (ensured up to %ld)", s, (long)first[i] + L - 1, p->length[s]);
    for (int j = 0; j < L; ++j) {
      const int32_t t = tokens[at + j];
      if (!((t >= 0 && t < vocab) || (t == -1 && L == 1)))
        return stage_fail("token id %ld out of range 0..%ld in the entry of slot %ld", t, (long)vocab - 1, s);
      tok[at + j] = t;
      pos[at + j] = first[i] + j;
      slt[at + j] = s;
    }
    for (int k = 0; k < n_want[i]; ++k, ++wi) {
      const int j = want[wi];
      if (j < 0 || j >= L) return stage_fail("wanted place %ld is outside the entry's %ld tokens", j, L);
      rows[w] = at + j;
      row_slot[w] = s;
      ++w;
    }
    meta[i] = s, meta[R + i] = at, meta[2 * R + i] = L, meta[3 * R + i] = first[i];
    at += L;
  }
  out[0] = at;
  out[1] = w;
  return 0;
}

// A step of E decoded tokens, each wanted, padded to B rows for a recorded graph: the padding rows belong to
// `pad_slot` at position 0 with token 0. token[i] may be -1 (still being chosen).
SB_API int sb_stage_decode(void* pool, int E, int B, int pad_slot, const int32_t* slot, const int32_t* first, const int32_t* token,
                           int vocab, int R, int32_t* staging) {
  Pool* p = static_cast<Pool*>(pool);
  if (E <= 0 || B < E || B > R) return stage_fail("a decode step of %ld rows padded to %ld does not fit max_rows %ld", E, B, R);
  std::vector<uint8_t> seen(p->max_slots, 0);
  int32_t *tok = staging, *pos = staging + R, *slt = staging + 2 * R, *rows = staging + 3 * R, *meta = staging + 4 * R,
          *row_slot = staging + 8 * R;
  for (int i = 0; i < E; ++i) {
    const int s = slot[i];
    if (!p->slot_ok(s) || s == pad_slot || seen[s]) return stage_fail("slot %ld appears twice in one step or is not held by a request", s);
    seen[s] = 1;
    if (first[i] < 0 || first[i] + 1 > p->length[s])
      return stage_fail("slot %ld: token %ld has no page (ensured up to %ld)", s, first[i], p->length[s]);
    if (token[i] < -1 || token[i] >= vocab) return stage_fail("token id %ld out of range 0..%ld", token[i], (long)vocab - 1);
    tok[i] = token[i], pos[i] = first[i], slt[i] = s, row_slot[i] = s;
    meta[i] = s, meta[R + i] = i, meta[2 * R + i] = 1, meta[3 * R + i] = first[i];
  }
  for (int i = E; i < B; ++i) {
    tok[i] = 0, pos[i] = 0, slt[i] = pad_slot, row_slot[i] = pad_slot;
    meta[i] = pad_slot, meta[R + i] = i, meta[2 * R + i] = 1, meta[3 * R + i] = 0;
  }
  for (int i = 0; i < B; ++i) rows[i] = i;
  return 0;
}

// Gives up every request: slots and pages go back, the queues are empty. For a caller that met an error in the middle
// of a run and wants the pool as it found it (it has made sure that no step is still running on the GPU).
SB_API void sb_sched_abort(void* sched) {
  Sched* sc = static_cast<Sched*>(sched);
  for (int id : sc->running) sc->release(sc->seqs[id]);
  for (size_t id = 0; id < sc->seqs.size(); ++id)
    if (sc->seqs[id].live) sc->retire((int)id);
  sc->running.clear();
  sc->waiting.clear();
}

// ------------------------------------------------------------------ the step program
//
// The operations of a step, recorded once when the engine is built (see step_ops.h), and the runner that calls them
// in order for every step. `sb_program_prepare` fills the step's record: its sizes, and for every tile plan that a
// mixer asked for the cut of the step's entries into attention tiles and decode items, written behind the step's
// other integer inputs in the staging area so that everything travels in one copy. Counterpart in arhaamatiq/stride:
// the launch sequences of Engine::step_exact / step_tensor_core and the attention items built on the host
// (src/engine.cpp:93-103, 144-462).
#include "step_ops.h"

namespace {

struct Program {
  std::vector<SbOp> ops;
  std::vector<SbTilePlan> plans;     // keys only
  int R = 0;
  int work_ints = 0;                  // room for work lists behind the 9 R fixed regions
  int launched = 0;                   // operations that launched something in the last run
};

}  // namespace

// R: the most rows of a step; work_ints: int32 of room for the plans' work lists behind the staging area's 9 R.
SB_API void* sb_program_create(int R, int work_ints) {
  Program* p = new Program();
  p->R = R;
  p->work_ints = work_ints;
  return p;
}

SB_API void sb_program_destroy(void* program) { delete static_cast<Program*>(program); }

// A tile plan for mixers of head ratio `group` whose prompt kernel takes tiles of `tile_rows` rows, with `kv_heads`
// key/value heads; fused_limit >= 0: steps of items only run rotation and append inside the decode kernel while
// items x kv_heads x chunks stays within it. Returns the plan's index in SbStep::plan (equal requests share one), or -1.
SB_API int sb_program_plan(void* program, int group, int tile_rows, int kv_heads, int fused_limit) {
  Program* p = static_cast<Program*>(program);
  if (group <= 0 || group > 16 || tile_rows < group) {
    g_error = "a tile plan needs a head ratio of 1..16 and tiles of at least one position";
    return -1;
  }
  for (size_t k = 0; k < p->plans.size(); ++k) {
    const SbTilePlan& q = p->plans[k];
    if (q.group == group && q.tile_rows == tile_rows && q.kv_heads == kv_heads && q.fused_limit == fused_limit) return (int)k;
  }
  if (p->plans.size() >= SB_MAX_PLANS) {
    g_error = "a model may ask for at most " + std::to_string(SB_MAX_PLANS) + " different tile plans";
    return -1;
  }
  SbTilePlan q{};
  q.group = group, q.tile_rows = tile_rows, q.kv_heads = kv_heads, q.fused_limit = fused_limit;
  p->plans.push_back(q);
  return (int)p->plans.size() - 1;
}

SB_API int sb_program_add(void* program, const SbOp* op) {
  Program* p = static_cast<Program*>(program);
  if (op == nullptr || op->fn == nullptr) {
    g_error = "an operation without a function";
    return -1;
  }
  p->ops.push_back(*op);
  return (int)p->ops.size() - 1;
}

SB_API int sb_program_size(void* program) { return (int)static_cast<Program*>(program)->ops.size(); }

// Operation `index` stands for the `count` operations behind it whenever it launches (SbOp::covers).
SB_API int sb_program_set_covers(void* program, int index, int count) {
  Program* p = static_cast<Program*>(program);
  if (index < 0 || count < 0 || (size_t)index + (size_t)count >= p->ops.size()) {
    g_error = "an operation can only stand for operations that follow it";
    return -1;
  }
  p->ops[index].covers = count;
  return 0;
}

// Fills `step` for a batch whose integer inputs were staged at `staging` (sb_stage_step or sb_stage_decode: E entries
// of count[i] tokens from position first[i]; n rows, `wanted` of them wanted) and will lie at `device_ints` once
// copied. static_keys > 0: a recorded decode step of E single-token entries (the padding included), planned for keys
// below static_keys whatever the positions are. 0, or -1 when the work lists do not fit.
SB_API int sb_program_prepare(void* program, int E, const int32_t* count, const int32_t* first, int n, int wanted, int static_keys,
                              int32_t* staging, const int32_t* device_ints, SbStep* step) {
  Program* p = static_cast<Program*>(program);
  memset(step, 0, sizeof(SbStep));
  step->n = n, step->entries = E, step->wanted = wanted, step->static_keys = static_keys, step->max_rows = p->R;
  step->n_plans = (int)p->plans.size();
  step->ints = device_ints;
  int32_t* work = staging + 9 * (int64_t)p->R;
  int at = 0;
  for (size_t k = 0; k < p->plans.size(); ++k) {
    SbTilePlan q = p->plans[k];
    q.work_offset = at;
    if (static_keys > 0) {
      if (at + E > p->work_ints) return stage_fail("the step's work lists exceed the staging area");
      for (int e = 0; e < E; ++e) work[at + e] = e;
      q.tiles = 0, q.items = E, q.chunks = (static_keys + 255) / 256;
      at += E;
    } else {
      const int ppt = q.tile_rows / q.group, few = 16 / q.group;
      struct Tile { int key, entry, tile; };
      std::vector<Tile> tiles;
      std::vector<int> items;
      int last = 0;
      for (int e = 0; e < E; ++e) {
        const int L = count[e], p0 = first[e];
        if (L <= few) {
          items.push_back(e);
          last = std::max(last, p0 + L - 1);
        } else {
          for (int t = 0; t < (L + ppt - 1) / ppt; ++t) tiles.push_back({p0 + std::min(L, (t + 1) * ppt), e, t});
        }
      }
      // the tiles that see the most keys first: CTAs start in this order, and the short ones fill the end
      std::stable_sort(tiles.begin(), tiles.end(), [](const Tile& a, const Tile& b) { return a.key > b.key; });
      const int need = 2 * (int)tiles.size() + (int)items.size();
      if (at + need > p->work_ints) return stage_fail("the step's work lists exceed the staging area");
      for (const Tile& t : tiles) work[at++] = t.entry, work[at++] = t.tile;
      for (int e : items) work[at++] = e;
      q.tiles = (int)tiles.size(), q.items = (int)items.size(), q.chunks = items.empty() ? 0 : last / 256 + 1;
    }
    q.fused = q.tiles == 0 && q.items > 0 && q.fused_limit >= 0 && (int64_t)q.items * q.kv_heads * q.chunks <= q.fused_limit;
    at = (at + 3) & ~3;
    step->plan[k] = q;
  }
  return 0;
}

// Runs the program's operations in order on `stream`. 0, or -1 with *failed = the index of the operation that failed
// (its library's sb_last_error() has the reason). *launched = operations that launched something.
SB_API int sb_program_run(void* program, const SbStep* step, void* stream, int32_t* failed, int32_t* launched) {
  Program* p = static_cast<Program*>(program);
  int count = 0;
  for (size_t k = 0; k < p->ops.size(); ++k) {
    const SbOp& op = p->ops[k];
    const int rc = reinterpret_cast<SbOpFn>(op.fn)(&op, step, stream);
    if (rc == SB_OP_LAUNCHED) {
      ++count;
      k += (size_t)op.covers;
    } else if (rc != SB_OP_SKIPPED) {
      if (failed) *failed = (int32_t)k;
      if (launched) *launched = count;
      return -1;
    }
  }
  if (launched) *launched = count;
  return 0;
}

// The same run with the host's time for every operation (microseconds into per_op_us[sb_program_size()]): what the
// launches themselves cost the CPU, for finding an operation whose set-up is slow. Returns like sb_program_run.
SB_API int sb_program_run_timed(void* program, const SbStep* step, void* stream, double* per_op_us) {
  Program* p = static_cast<Program*>(program);
  for (size_t k = 0; k < p->ops.size(); ++k) {
    const SbOp& op = p->ops[k];
    const auto t0 = std::chrono::steady_clock::now();
    const int rc = reinterpret_cast<SbOpFn>(op.fn)(&op, step, stream);
    per_op_us[k] = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
    if (rc != SB_OP_LAUNCHED && rc != SB_OP_SKIPPED) return -1;
    if (rc == SB_OP_LAUNCHED)
      for (int64_t c = 0; c < op.covers && k + 1 < p->ops.size(); ++c) per_op_us[++k] = 0.0;
  }
  return 0;
}
