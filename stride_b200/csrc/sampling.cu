// Token choice on the device: argmax (greedy) and temperature sampling.
//
// Greedy keeps the largest logit and, among equal logits, the smallest index,
// whatever the order in which threads meet them.
//
// Temperature sampling restates arhaamatiq/stride's host sampler
// (src/scheduler.cpp:193-243) without sorting: tokens are ranked by (logit
// descending, index ascending), weight_i = exp((l_i - l_max) / T) in 64-bit (kept
// as an integer multiple of 2^-40, so that sums do not depend on their order),
// u = uniform * sum of weights, and the token is the first in rank order whose
// cumulative weight exceeds u. The rank order is walked by weighted histograms:
// 256 bins of the distance from the largest logit, then a radix search over the
// logit's bit pattern inside the chosen bin (four passes of eight bits).
// The uniform is keyed on (seed, length of the sequence) alone:
// r = splitmix64(seed ^ (length * 0x9E3779B97F4A7C15)), uniform = (r >> 11) * 2^-53,
// so a draw does not depend on the batch or the schedule.
#include "common.cuh"

SB_DEFINE_LAST_ERROR()

namespace {

constexpr int kThreads = 1024;
constexpr int kSampleThreads = 512;   // threads of a CTA of the temperature sampler

__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ULL;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
  return x ^ (x >> 31);
}

// (value, index) -> one 64-bit word whose unsigned order is value ascending, then index descending.
__device__ __forceinline__ unsigned long long pack_best(float v, int idx) {
  return (static_cast<unsigned long long>(order_key(v)) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(idx));
}

// `watch` (optional): the status word of the kernels that made the logits. If a wait inside one of them gave up
// (the word is not 0), the token reported to the host is -1 - code instead of a token id, so that the failure
// travels with the step's result and costs no copy of its own; what is scattered for the next step stays a token id.
__device__ __forceinline__ int poisoned(int token, const int* watch) {
  if (watch == nullptr) return token;
  const int code = *reinterpret_cast<const volatile int*>(watch);
  return code != 0 ? -1 - code : token;
}

// `scatter` (optional): the chosen token is also stored at scatter[scatter_index[row]] (the request's slot), where
// the next step's embedding looks for it.
__global__ void __launch_bounds__(kThreads) argmax_kernel(const float* __restrict__ logits, int64_t ld, int vocab,
                                                           int32_t* __restrict__ tokens, float* __restrict__ values,
                                                           const int32_t* __restrict__ scatter_index,
                                                           int32_t* __restrict__ scatter, const int* __restrict__ watch) {
  __shared__ unsigned long long best_s[32];
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const float* l = logits + static_cast<int64_t>(blockIdx.x) * ld;
  unsigned long long best = 0;
  for (int i = threadIdx.x; i < vocab; i += kThreads) {
    const float v = l[i];
    if (v == v) {
      const unsigned long long c = pack_best(v, i);
      best = c > best ? c : best;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) best_s[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kThreads / 32; ++i) best = best_s[i] > best ? best_s[i] : best;
    const int idx = best == 0 ? 0 : static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(best & 0xFFFFFFFFu));
    tokens[blockIdx.x] = poisoned(idx, watch);
    values[blockIdx.x] = l[idx];
    if (scatter != nullptr) scatter[scatter_index[blockIdx.x]] = idx;
  }
}

// Weights are kept as integers, w_i = floor(exp((l_i - l_max) / T) * 2^40) with the exponential in 64-bit floating
// point: integer sums do not depend on the order in which threads add, so the histograms below, and with them the
// token, are the same in every run and every batch. (The largest logit has weight 2^40 exactly; a token whose weight
// is below 2^-40 of it is never drawn; a vocabulary of four million tokens still sums below 2^63.)
__device__ __forceinline__ unsigned long long fixed_weight(float v, double top, double T) {
  return __double2ull_rd(exp((static_cast<double>(v) - top) / T) * 1099511627776.0);
}

// The same choice with a row's vocabulary cut into `splits` slices, one CTA each, so that a few rows still occupy the GPU
// (one CTA reads a row of 128,256 logits in 17 us, thirty-one read it in 3): every CTA offers its slice's best (value,
// index) word to the row's word with an atomic maximum, which no order of arrival changes, and the CTA that arrives last
// publishes the row's token and clears the row's word and ticket for the next call. The words live in this library
// (zero when it is loaded), so calls that overlap on different streams would disturb one another; the engine has one stream.
constexpr int kSplitRows = 16384;
constexpr int kSplitThreads = 256;
__device__ unsigned long long g_row_best[kSplitRows];
__device__ unsigned int g_row_done[kSplitRows];

__global__ void __launch_bounds__(kSplitThreads) argmax_split_kernel(const float* __restrict__ logits, int64_t ld, int vocab, int slice,
                                                                     int32_t* __restrict__ tokens, float* __restrict__ values,
                                                                     const int32_t* __restrict__ scatter_index,
                                                                     int32_t* __restrict__ scatter, const int* __restrict__ watch) {
  __shared__ unsigned long long best_s[kSplitThreads / 32];
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int row = blockIdx.y;
  const float* l = logits + static_cast<int64_t>(row) * ld;
  const int begin = blockIdx.x * slice, end = min(vocab, begin + slice);
  unsigned long long best = 0;
  for (int i = begin + threadIdx.x; i < end; i += kSplitThreads) {
    const float v = l[i];
    if (v == v) {
      const unsigned long long c = pack_best(v, i);
      best = c > best ? c : best;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) best_s[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kSplitThreads / 32; ++i) best = best_s[i] > best ? best_s[i] : best;
    if (best != 0) atomicMax(&g_row_best[row], best);
    __threadfence();
    if (atomicAdd(&g_row_done[row], 1u) == gridDim.x - 1) {      // every slice of the row has made its offer
      __threadfence();
      best = atomicExch(&g_row_best[row], 0ull);
      g_row_done[row] = 0;
      const int idx = best == 0 ? 0 : static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(best & 0xFFFFFFFFu));
      tokens[row] = poisoned(idx, watch);
      values[row] = l[idx];
      if (scatter != nullptr) scatter[scatter_index[row]] = idx;
    }
  }
}

// f(logit, index) for the logits [begin, end) of a row, in no particular order (what the callers add up does not depend
// on it). With `vec` (the row starts 16-byte aligned and `begin` is a multiple of four) a thread has four 16-byte loads in
// flight at a time: with one, a walk over a row took as long as its trips to memory one after another.
template <class F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ l, int begin, int end, bool vec, F f) {
  const int t = threadIdx.x;
  int done = begin;
  if (vec) {
    const float4* l4 = reinterpret_cast<const float4*>(l);
    const int b4 = begin / 4, e4 = end / 4;
    for (int i0 = b4 + t; i0 < e4; i0 += 4 * kSampleThreads) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * kSampleThreads < e4) v[u] = l4[i0 + u * kSampleThreads];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kSampleThreads;
        if (i < e4) {
          f(v[u].x, 4 * i);
          f(v[u].y, 4 * i + 1);
          f(v[u].z, 4 * i + 2);
          f(v[u].w, 4 * i + 3);
        }
      }
    }
    done = max(begin, e4 * 4);
  }
  for (int i = done + t; i < end; i += kSampleThreads) f(l[i], i);
}

// Shared memory of another CTA of the cluster: the address of `p` (a shared-memory address of this CTA) in CTA `rank`.
__device__ __forceinline__ uint32_t peer_shared(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))), "r"(rank));
  return out;
}
__device__ __forceinline__ unsigned long long peer_load_u64(uint32_t addr) {
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t peer_load_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t n;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
  return n;
}

// The rank order (logit descending, index ascending) is walked in two levels. First 256 bins of the distance from the
// largest logit, d = max - l, linear over [0, min(max - min, 30 T)]: a monotone function of the logit, so the bins follow
// the rank order, and one that spreads a vocabulary's bulk over many bins whatever the temperature is (the leading byte of
// the logit's bit pattern would put it into a handful, and a hundred thousand additions to a handful of shared-memory
// words take a millisecond). A token further than 30 T from the top has weight floor(e^-30 * 2^40) = 0 and is passed
// over. Then, inside the chosen bin, the radix search over the logit's bit pattern, eight bits a pass.
//
// A row belongs to a cluster of CTAs (blockIdx.x = the CTA's rank, blockIdx.y = the row): each takes a slice of the
// vocabulary and keeps histograms of its own, since the 64-bit exponentials of a large vocabulary are more than one
// SM's few 64-bit units do in a decode step's time; after every walk the first CTA adds the cluster's histograms up
// through distributed shared memory (integers: no order to keep), decides, and the others read its decision.
constexpr int kMaxMatches = 512;    // equal logits of one slice that are listed; more are walked one by one
constexpr int kCandidates = 512;    // logits of the chosen bin that a CTA lists from its slice
constexpr int kAllCandidates = 8 * kCandidates;   // .. and that the first CTA gathers from the whole cluster

// The logit whose order_key is `key`.
__device__ __forceinline__ float key_value(uint32_t key) { return __uint_as_float((key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key); }

// The bin in which a draw falls, found by one warp instead of one thread: position p of the rank order is bin p
// (ascending) or 255 - p (descending); lane L takes positions 8 L .. 8 L + 7, the lanes' sums are scanned with
// shuffles, the lane whose range holds the draw walks its eight bins. Returns the bin (-1: the draw lies beyond every
// bin) and leaves the weight in front of it in `before`; `total` is the sum of all bins. All 32 lanes call it.
__device__ __forceinline__ unsigned long long bins_total(const unsigned long long* hist, bool descending, unsigned long long& mine,
                                                         unsigned long long& inclusive) {
  const int lane = threadIdx.x & 31;
  mine = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int p = 8 * lane + k;
    mine += hist[descending ? 255 - p : p];
  }
  inclusive = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long up = __shfl_up_sync(0xffffffffu, inclusive, o);
    if (lane >= o) inclusive += up;
  }
  return __shfl_sync(0xffffffffu, inclusive, 31);
}
__device__ __forceinline__ int pick_bin(const unsigned long long* hist, bool descending, unsigned long long u, unsigned long long mine,
                                        unsigned long long inclusive, unsigned long long& before) {
  const int lane = threadIdx.x & 31;
  const unsigned holds = __ballot_sync(0xffffffffu, u < inclusive);
  if (holds == 0) {
    before = 0;
    return -1;
  }
  const int owner = __ffs(holds) - 1;
  int chosen = -1;
  unsigned long long cum = inclusive - mine;
  if (lane == owner) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int p = 8 * lane + k, b = descending ? 255 - p : p;
      if (chosen < 0) {
        if (u < cum + hist[b]) chosen = b;
        else cum += hist[b];
      }
    }
  }
  before = __shfl_sync(0xffffffffu, cum, owner);
  return __shfl_sync(0xffffffffu, chosen, owner);
}

struct Decision {
  unsigned long long u;      // what is left of the draw inside the chosen part
  uint32_t prefix;           // the logit's bits chosen so far
  int bin, found;
};

__global__ void __launch_bounds__(kSampleThreads) sample_temperature_kernel(
    const float* __restrict__ logits, int64_t ld, int vocab, const float* __restrict__ temperatures,
    const unsigned long long* __restrict__ seeds, const int32_t* __restrict__ lengths, int32_t* __restrict__ tokens,
    float* __restrict__ values, const int32_t* __restrict__ scatter_index, int32_t* __restrict__ scatter,
    const int* __restrict__ watch) {
  __shared__ unsigned long long hist[256];
  __shared__ unsigned int count[256];
  __shared__ float red[32];
  __shared__ float extremes[2];
  __shared__ Decision decision;
  __shared__ int match_n, cand_n;
  __shared__ int match_idx[kMaxMatches];
  __shared__ uint32_t cand_key[kCandidates];
  __shared__ int cand_idx[kCandidates];
  __shared__ uint32_t all_key[kAllCandidates];     // (used by the cluster's first CTA)
  __shared__ int all_idx[kAllCandidates];
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int row = blockIdx.y, t = threadIdx.x;
  const uint32_t rank = sb::cluster_rank(), ranks = cluster_size();
  const float* l = logits + static_cast<int64_t>(row) * ld;
  const bool sampled = temperatures[row] > 0.0f;     // (a greedy row: the argmax kernel has chosen its token; the cluster
  const double T = static_cast<double>(temperatures[row]);   // still walks through its barriers together)
  // this CTA's slice, a multiple of four logits so that every slice starts 16-byte aligned within an aligned row
  const int slice = ((vocab + static_cast<int>(ranks) - 1) / static_cast<int>(ranks) + 3) & ~3;
  const int begin = sampled ? min(vocab, static_cast<int>(rank) * slice) : 0, end = sampled ? min(vocab, begin + slice) : 0;
  const bool vec = (reinterpret_cast<uintptr_t>(l) & 15) == 0;

  float mx = -INFINITY, mn = INFINITY;
  for_each_logit(l, begin, end, vec, [&](float v, int) {
    if (v == v) {
      mx = fmaxf(mx, v);
      mn = fminf(mn, v);
    }
  });
  mx = sb::block_max(mx, red);
  mn = -sb::block_max(-mn, red);
  if (t == 0) extremes[0] = mx, extremes[1] = mn;
  sb::cluster_sync();
  for (uint32_t r = 0; r < ranks; ++r) {
    mx = fmaxf(mx, __uint_as_float(peer_load_u32(peer_shared(&extremes[0], r))));
    mn = fminf(mn, __uint_as_float(peer_load_u32(peer_shared(&extremes[1], r))));
  }
  const double top = static_cast<double>(mx);
  const float cut = 30.0f * temperatures[row];
  float range = fminf(mx - mn, cut);
  if (!(range > 0.0f)) range = 1.0f;             // one distinct logit (or none): everything lands in bin 0
  const float per_bin = 255.0f / range;
  // the bin of a logit: 0 for the largest, ascending with the distance from it; -1: weight 0, never drawn
  auto bin_of = [&](float v) {
    const float d = mx - v;
    if (!(d <= cut)) return -1;
    const float b = d * per_bin;
    return b >= 255.0f ? 255 : static_cast<int>(b);
  };
  // the cluster's histograms added up by its first CTA (thread b takes bin b)
  auto cluster_sum = [&](int b, unsigned long long& weight, unsigned int& number) {
    weight = 0, number = 0;
    for (uint32_t r = 0; r < ranks; ++r) {
      weight += peer_load_u64(peer_shared(&hist[b], r));
      number += peer_load_u32(peer_shared(&count[b], r));
    }
  };

  for (int b = t; b < 256; b += kSampleThreads) hist[b] = 0, count[b] = 0;
  __syncthreads();
  for_each_logit(l, begin, end, vec, [&](float v, int) {
    if (v != v) return;
    const int b = bin_of(v);
    if (b < 0) return;
    const unsigned long long w = fixed_weight(v, top, T);
    if (w != 0) atomicAdd(&hist[b], w);
  });
  sb::cluster_sync();
  if (rank == 0) {
    unsigned long long w = 0;
    unsigned int c = 0;
    if (t < 256) cluster_sum(t, w, c);
    __syncthreads();         // (this CTA's own histogram has been read: it is overwritten with the sums)
    if (t < 256) hist[t] = w;
    __syncthreads();
    if (t < 32) {
      unsigned long long mine, inclusive, before;
      const unsigned long long total = bins_total(hist, false, mine, inclusive);
      // u = floor(uniform * total), uniform = (r >> 11) * 2^-53: a 53 x 62 bit product, shifted down by 53; u < total
      const unsigned long long r =
          splitmix64(seeds[row] ^ (static_cast<unsigned long long>(static_cast<uint32_t>(lengths[row])) * 0x9E3779B97F4A7C15ULL));
      const unsigned long long m = r >> 11;
      const unsigned long long u = (__umul64hi(m, total) << 11) | ((m * total) >> 53);
      const int chosen = pick_bin(hist, false, u, mine, inclusive, before);
      if (t == 0) {
        decision.bin = chosen < 0 ? 0 : chosen;     // (no number in the row: nothing will be found in bin 0 either)
        decision.u = u - before;
        decision.prefix = 0;
        decision.found = 0;
      }
    }
  }
  sb::cluster_sync();
  const int bin = static_cast<int>(peer_load_u32(peer_shared(&decision.bin, 0)));

  // The chosen bin usually holds a few hundred logits. Every CTA lists those of its slice (bits and index); if all lists
  // fit, the first CTA finishes alone, reading the others' lists through distributed shared memory: no further walk over
  // the row and no further barrier but the last. Otherwise (a vocabulary of nearly equal logits) the walks below go on.
  if (t == 0) cand_n = 0;
  __syncthreads();
  for_each_logit(l, begin, end, vec, [&](float v, int i) {
    if (v != v || bin_of(v) != bin) return;
    const int k = atomicAdd(&cand_n, 1);
    if (k < kCandidates) cand_key[k] = order_key(v), cand_idx[k] = i;
  });
  sb::cluster_sync();
  bool listed = true;
  for (uint32_t r = 0; r < ranks; ++r) listed = listed && peer_load_u32(peer_shared(&cand_n, r)) <= static_cast<uint32_t>(kCandidates);
  if (listed) {
    if (rank == 0 && sampled) {
      // candidate c of the cluster: entry c - first[r] of CTA r's list
      __shared__ int first_of[9];
      if (t == 0) {
        first_of[0] = 0;
        for (uint32_t r = 0; r < ranks; ++r) first_of[r + 1] = first_of[r] + static_cast<int>(peer_load_u32(peer_shared(&cand_n, r)));
      }
      __syncthreads();
      const int total = first_of[ranks];
      // fetched once through distributed shared memory, then worked on here
      for (uint32_t r = 0; r < ranks; ++r)
        for (int c = first_of[r] + t; c < first_of[r + 1]; c += kSampleThreads) {
          all_key[c] = peer_load_u32(peer_shared(&cand_key[c - first_of[r]], r));
          all_idx[c] = static_cast<int>(peer_load_u32(peer_shared(&cand_idx[c - first_of[r]], r)));
        }
      __syncthreads();
      auto candidate = [&](int c, uint32_t& ckey, int& cidx) { ckey = all_key[c], cidx = all_idx[c]; };
      uint32_t prefix = 0;
      for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = t; b < 256; b += kSampleThreads) hist[b] = 0, count[b] = 0;
        __syncthreads();
        const uint32_t mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
        for (int c = t; c < total; c += kSampleThreads) {
          uint32_t ckey;
          int cidx;
          candidate(c, ckey, cidx);
          if ((ckey & mask) != prefix) continue;
          const int b = (ckey >> shift) & 0xFF;
          atomicAdd(&hist[b], fixed_weight(key_value(ckey), top, T));
          atomicAdd(&count[b], 1u);
        }
        __syncthreads();
        if (t < 32) {
          unsigned long long mine, inclusive, before;
          bins_total(hist, true, mine, inclusive);
          const unsigned long long u = decision.u;
          const int chosen = pick_bin(hist, true, u, mine, inclusive, before);
          __syncwarp();
          if (t == 0) {      // (nothing chosen: a row without a single number; the token is then 0)
            decision.u = chosen < 0 ? 0 : u - before;
            decision.prefix = prefix | (static_cast<uint32_t>(chosen < 0 ? 0 : chosen) << shift);
            decision.found = chosen < 0 ? 0 : static_cast<int>(count[chosen]);
          }
        }
        __syncthreads();
        prefix = decision.prefix;
      }
      // the tokens with the chosen bits rank by index: the one that has as many smaller indices as the draw passes over
      const int found = decision.found;
      if (found == 0) {
        if (t == 0) {
          tokens[row] = poisoned(0, watch);
          values[row] = l[0];
          if (scatter != nullptr) scatter[scatter_index[row]] = 0;
        }
      } else {
        const float v_key = key_value(prefix);
        const unsigned long long w = fixed_weight(v_key, top, T);
        unsigned long long skip = w > 0 ? decision.u / w : static_cast<unsigned long long>(found - 1);
        if (skip > static_cast<unsigned long long>(found - 1)) skip = found - 1;
        auto publish = [&](int i) {
          tokens[row] = poisoned(i, watch);
          values[row] = v_key;
          if (scatter != nullptr) scatter[scatter_index[row]] = i;
        };
        if (t == 0) match_n = 0;
        __syncthreads();
        if (found <= kMaxMatches) {
          // list the tokens with the chosen bits; the wanted one has exactly `skip` smaller indices among them
          for (int c = t; c < total; c += kSampleThreads) {
            uint32_t ckey;
            int cidx;
            candidate(c, ckey, cidx);
            if (ckey == prefix) match_idx[atomicAdd(&match_n, 1)] = cidx;
          }
          __syncthreads();
          for (int a = t; a < found; a += kSampleThreads) {
            unsigned long long smaller = 0;
            for (int b = 0; b < found; ++b) smaller += match_idx[b] < match_idx[a];
            if (smaller == skip) publish(match_idx[a]);
          }
        } else {
          for (int c = t; c < total; c += kSampleThreads) {
            uint32_t ckey;
            int cidx;
            candidate(c, ckey, cidx);
            if (ckey != prefix) continue;
            unsigned long long smaller = 0;
            for (int o = 0; o < total; ++o) {
              uint32_t okey;
              int oidx;
              candidate(o, okey, oidx);
              smaller += okey == prefix && oidx < cidx;
            }
            if (smaller == skip) publish(cidx);
          }
        }
      }
    }
    sb::cluster_sync();      // the other CTAs' lists stay until the first CTA is done with them
    return;
  }

  for (int shift = 24; shift >= 0; shift -= 8) {
    // (the first CTA has read every histogram of the walk before, and does not touch its decision again before the
    // barrier after this walk: no barrier is needed here)
    const uint32_t prefix = peer_load_u32(peer_shared(&decision.prefix, 0));
    for (int b = t; b < 256; b += kSampleThreads) hist[b] = 0, count[b] = 0;
    __syncthreads();
    const uint32_t mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for_each_logit(l, begin, end, vec, [&](float v, int) {
      if (v != v || bin_of(v) != bin) return;
      const uint32_t key = order_key(v);
      if ((key & mask) != prefix) return;
      const int b = (key >> shift) & 0xFF;
      atomicAdd(&hist[b], fixed_weight(v, top, T));
      atomicAdd(&count[b], 1u);
    });
    sb::cluster_sync();
    if (rank == 0) {
      unsigned long long w = 0;
      unsigned int c = 0;
      if (t < 256) cluster_sum(t, w, c);
      __syncthreads();
      if (t < 256) hist[t] = w, count[t] = c;
      __syncthreads();
      if (t < 32) {
        unsigned long long mine, inclusive, before;
        bins_total(hist, true, mine, inclusive);
        const unsigned long long u = decision.u;
        const int chosen = pick_bin(hist, true, u, mine, inclusive, before);
        __syncwarp();
        if (t == 0) {      // (nothing chosen: a row without a single number; the token is then 0)
          decision.u = chosen < 0 ? 0 : u - before;
          decision.prefix = prefix | (static_cast<uint32_t>(chosen < 0 ? 0 : chosen) << shift);
          decision.found = chosen < 0 ? 0 : static_cast<int>(count[chosen]);
        }
      }
    }
    sb::cluster_sync();
  }

  // Every token whose key is the chosen one has the same logit and weight; they rank by index, and the draw's remainder
  // says how many of them to pass over. (Equal logits are no rarity: a vocabulary of 128 k has hundreds of pairs.) Each
  // CTA lists the matches of its slice; the slices lie in index order, so the counts of the CTAs in front tell a CTA
  // whether the wanted match is one of its own, and which.
  const uint32_t key = peer_load_u32(peer_shared(&decision.prefix, 0));
  const unsigned long long u_left = peer_load_u64(peer_shared(&decision.u, 0));
  if (t == 0) match_n = 0;
  __syncthreads();
  for_each_logit(l, begin, end, vec, [&](float v, int i) {
    if (v == v && order_key(v) == key) {
      const int k = atomicAdd(&match_n, 1);
      if (k < kMaxMatches) match_idx[k] = i;
    }
  });
  sb::cluster_sync();
  int before = 0, found = 0;
  for (uint32_t r = 0; r < ranks; ++r) {
    const int c = static_cast<int>(peer_load_u32(peer_shared(&match_n, r)));
    if (r < rank) before += c;
    found += c;
  }
  sb::cluster_sync();        // nobody leaves while another CTA may still read its shared memory
  if (!sampled) return;
  if (found == 0) {          // a row without a single number: token 0
    if (rank == 0 && t == 0) {
      tokens[row] = poisoned(0, watch);
      values[row] = l[0];
      if (scatter != nullptr) scatter[scatter_index[row]] = 0;
    }
    return;
  }
  const float v_key = key_value(key);
  const unsigned long long w = fixed_weight(v_key, top, T);
  unsigned long long skip = w > 0 ? u_left / w : static_cast<unsigned long long>(found - 1);
  if (skip > static_cast<unsigned long long>(found - 1)) skip = found - 1;
  const int local = static_cast<int>(skip) - before, mine = match_n;
  if (local < 0 || local >= mine) return;
  auto publish = [&](int i) {
    tokens[row] = poisoned(i, watch);
    values[row] = v_key;
    if (scatter != nullptr) scatter[scatter_index[row]] = i;
  };
  if (mine <= kMaxMatches) {
    // the match with exactly `local` smaller indices among this CTA's matches
    for (int a = t; a < mine; a += kSampleThreads) {
      int smaller = 0;
      for (int b = 0; b < mine; ++b) smaller += match_idx[b] < match_idx[a];
      if (smaller == local) publish(match_idx[a]);
    }
  } else if (t == 0) {       // more equal logits in one slice than the list holds: walk the slice in index order
    int seen = 0;
    for (int i = begin; i < end; ++i) {
      if (l[i] == l[i] && order_key(l[i]) == key && seen++ == local) {
        publish(i);
        break;
      }
    }
  }
}

}  // namespace

namespace {
const int* g_watch = nullptr;
}
// From now on the kernels of this library look at `device_word` (the status word of the kernels that make the
// logits; null: at nothing) and report -1 - its value instead of a token while it is not 0.
SB_EXPORT void sb_sampling_use_status_word(const int* device_word) { g_watch = device_word; }

SB_EXPORT int sb_argmax(const float* logits, int64_t ld, int rows, int vocab, int32_t* tokens, float* values,
                        const int32_t* scatter_index, int32_t* scatter, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return sb::fail("sb_argmax: empty vocabulary");
  // slices of at least 4,096 logits, about two CTAs an SM
  const int splits = min((2 * sb::sm_count() + rows - 1) / rows, vocab / 4096);
  if (splits > 1 && rows <= kSplitRows && rows <= 65535) {
    const int slice = (vocab + splits - 1) / splits;
    sb::launch_pdl(argmax_split_kernel, dim3((vocab + slice - 1) / slice, rows), dim3(kSplitThreads), 0, stream, logits, ld, vocab, slice, tokens,
                   values, scatter_index, scatter, g_watch);
    return sb::check_launch("sb_argmax");
  }
  sb::launch_pdl(argmax_kernel, dim3(rows), dim3(kThreads), 0, stream, logits, ld, vocab, tokens, values, scatter_index, scatter, g_watch);
  return sb::check_launch("sb_argmax");
}

SB_EXPORT int sb_sample_temperature(const float* logits, int64_t ld, int rows, int vocab, const float* temperatures,
                                    const unsigned long long* seeds, const int32_t* lengths, int32_t* tokens,
                                    float* values, const int32_t* scatter_index, int32_t* scatter, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return sb::fail("sb_sample_temperature: empty vocabulary");
  if (rows > 65535) return sb::fail("sb_sample_temperature: %d rows exceed the grid", rows);
  // a cluster of up to eight CTAs a row: slices of at least 4,096 logits
  unsigned ranks = 1;
  while (ranks < 8 && vocab / static_cast<int>(2 * ranks) >= 4096) ranks *= 2;
  sb::launch_pdl_cluster(sample_temperature_kernel, dim3(ranks, rows), dim3(kSampleThreads), 0, stream, dim3(ranks, 1, 1), logits, ld, vocab, temperatures,
                         seeds, lengths, tokens, values, scatter_index, scatter, g_watch);
  return sb::check_launch("sb_sample_temperature");
}
