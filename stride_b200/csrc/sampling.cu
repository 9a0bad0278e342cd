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
// cumulative weight exceeds u. The rank order is walked by a radix search over
// the logit's bit pattern (four passes of eight bits, weighted histograms).
// The uniform is keyed on (seed, length of the sequence) alone:
// r = splitmix64(seed ^ (length * 0x9E3779B97F4A7C15)), uniform = (r >> 11) * 2^-53,
// so a draw does not depend on the batch or the schedule.
#include "common.cuh"

SB_DEFINE_LAST_ERROR()

namespace {

constexpr int kThreads = 1024;

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

__global__ void __launch_bounds__(kThreads) sample_temperature_kernel(
    const float* __restrict__ logits, int64_t ld, int vocab, const float* __restrict__ temperatures,
    const unsigned long long* __restrict__ seeds, const int32_t* __restrict__ lengths, int32_t* __restrict__ tokens,
    float* __restrict__ values, const int32_t* __restrict__ scatter_index, int32_t* __restrict__ scatter,
    const int* __restrict__ watch) {
  __shared__ unsigned long long hist[256];
  __shared__ int count[256];
  __shared__ float red[32];
  __shared__ unsigned long long total_s;
  __shared__ uint32_t prefix_s;
  __shared__ unsigned long long u_s;
  __shared__ int found_s;
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int row = blockIdx.x, t = threadIdx.x;
  const float* l = logits + static_cast<int64_t>(row) * ld;
  if (!(temperatures[row] > 0.0f)) return;     // a greedy row: the argmax kernel has chosen its token
  const double T = static_cast<double>(temperatures[row]);

  float mx = -INFINITY;
  for (int i = t; i < vocab; i += kThreads) {
    const float v = l[i];
    if (v == v) mx = fmaxf(mx, v);
  }
  mx = sb::block_max(mx, red);
  const double top = static_cast<double>(mx);

  if (t == 0) total_s = 0;
  __syncthreads();
  unsigned long long sum = 0;
  for (int i = t; i < vocab; i += kThreads) {
    const float v = l[i];
    if (v == v) sum += fixed_weight(v, top, T);
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((t & 31) == 0) atomicAdd(&total_s, sum);
  __syncthreads();
  if (t == 0) {
    // u = floor(uniform * total), uniform = (r >> 11) * 2^-53: a 53 x 62 bit product, shifted down by 53
    const unsigned long long r =
        splitmix64(seeds[row] ^ (static_cast<unsigned long long>(static_cast<uint32_t>(lengths[row])) * 0x9E3779B97F4A7C15ULL));
    const unsigned long long m = r >> 11, total = total_s;
    u_s = (__umul64hi(m, total) << 11) | ((m * total) >> 53);
    prefix_s = 0;
  }
  __syncthreads();

  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = t; b < 256; b += kThreads) {
      hist[b] = 0;
      count[b] = 0;
    }
    __syncthreads();
    const uint32_t prefix = prefix_s;
    const uint32_t mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = t; i < vocab; i += kThreads) {
      const float v = l[i];
      if (v != v) continue;
      const uint32_t key = order_key(v);
      if ((key & mask) != prefix) continue;
      const int b = (key >> shift) & 0xFF;
      atomicAdd(&hist[b], fixed_weight(v, top, T));
      atomicAdd(&count[b], 1);
    }
    __syncthreads();
    if (t == 0) {
      unsigned long long u = u_s, cum = 0;
      int chosen = -1, lowest = 0;
      for (int b = 255; b >= 0; --b) {
        if (count[b] == 0) continue;
        lowest = b;
        if (u < cum + hist[b]) {
          chosen = b;
          break;
        }
        cum += hist[b];
      }
      if (chosen < 0) {  // only tokens of weight 0 are left: the last token in rank order
        chosen = lowest;
        cum = 0;
        u = hist[lowest];
      }
      u_s = u - cum;
      prefix_s = prefix | (static_cast<uint32_t>(chosen) << shift);
      found_s = count[chosen];
    }
    __syncthreads();
  }

  // Every token whose key is prefix_s has the same logit and weight; they rank by index.
  const uint32_t key = prefix_s;
  if (found_s == 1) {
    for (int i = t; i < vocab; i += kThreads) {
      const float v = l[i];
      if (v == v && order_key(v) == key) {
        tokens[row] = poisoned(i, watch);
        values[row] = v;
        if (scatter != nullptr) scatter[scatter_index[row]] = i;
      }
    }
  } else if (t == 0) {
    int first = -1;
    for (int i = 0; i < vocab && first < 0; ++i)
      if (l[i] == l[i] && order_key(l[i]) == key) first = i;
    int pick = 0;
    if (first >= 0) {     // (a row without a single number has no such token: token 0 then)
      const unsigned long long w = fixed_weight(l[first], top, T);
      unsigned long long skip = w > 0 ? u_s / w : static_cast<unsigned long long>(found_s - 1);
      if (skip > static_cast<unsigned long long>(found_s - 1)) skip = found_s - 1;
      pick = first;
      for (int i = first; i < vocab; ++i) {
        if (l[i] == l[i] && order_key(l[i]) == key) {
          pick = i;
          if (skip-- == 0) break;
        }
      }
    }
    tokens[row] = poisoned(pick, watch);
    values[row] = l[pick];
    if (scatter != nullptr) scatter[scatter_index[row]] = pick;
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
  sb::launch_pdl(sample_temperature_kernel, dim3(rows), dim3(kThreads), 0, stream, logits, ld, vocab, temperatures, seeds, lengths, tokens, values, scatter_index,
                 scatter, g_watch);
  return sb::check_launch("sb_sample_temperature");
}
