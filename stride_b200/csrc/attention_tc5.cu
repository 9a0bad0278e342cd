// Paged causal attention for prompt portions on Blackwell's tcgen05 tensor cores (head size 64, bfloat16).
//
// One CTA per (tile of 128 query rows of an entry, key/value head). The query heads that share the key/value
// head are stacked as rows: row r is (position r / G, head r % G), G = Hq / Hkv, so a tile covers 128 / G
// positions. The CTA walks the spans of 128 keys [128 t, 128 t + 128) its rows can see:
//
//   control warp (one thread): TMA loads of the query tile (a 3-D box over [token][head][64]) and of the key
//     and value spans, page by page through the block table, into 128-byte-swizzled shared memory (three
//     buffers); S = Q K^T by tcgen05.mma (M 128, N 128, K 64) into one of two TMEM accumulators, issued one
//     span ahead so that it runs under the softmax of the span before; O_0 = P_0 V_0 and O_1 = P_1 V_1 for the
//     span's two tiles of 64 keys by tcgen05.mma (M 128, N 64, K 64, V as an MN-major operand straight from
//     its [key][64] page layout), each into an accumulator of its own, from zero.
//   eight softmax warps (two threads per row, TMEM lane = row; thread `half` owns the span's tile `half` and
//     the output elements [32 half, 32 half + 32)): read S with tcgen05.ld (once a span, kept in registers), take
//     the tile's maximum, write the weights to tensor memory with tcgen05.st as two bfloat16 parts (p = hi + lo, so
//     the value product sees nearly 32-bit weights, as the reference's 32-bit softmax does; the value product takes
//     them from there as its A operand), then fold O_0 and O_1 into the row's chunk state (registers) and, every
//     256 keys, the chunk into the row's state (shared memory), all in float32.
//
// The arithmetic is that of attention_math.cuh, shared with the mma.sync kernels of attention_tc.cu: a row has
// the same bits from either. Every mbarrier wait is bounded and reports through a status word. Key spans past
// a request's last page are read from its last page instead (finite data, masked by position), so no
// unallocated page is touched.
// Counterpart in arhaamatiq/stride: AttentionPage / AttentionCombine (src/kernel_common.h:90-309), scalar.
#include "attention_math.cuh"
#include "tc5.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using namespace sb::tc5;
using bf16 = __nv_bfloat16;

constexpr int kRows = 128;
constexpr int kKeys = 128;
constexpr int kSubTileBytes = 128 * 128;   // 128 rows of 64 bfloat16: one 128-byte-swizzled piece of a tile
constexpr int kSoftmaxThreads = 256;    // two threads per row: each takes 64 of the span's 128 keys and half of the outputs
constexpr int kThreads = kSoftmaxThreads + 32;
constexpr int kMaxRing = 6;
constexpr int kPagesCached = 512;       // block-table entries of the request kept in shared memory
constexpr uint32_t kTmemCols = 512, kTmemO = 128;

// What depends on the head size D (64 or 128). A tile of 128 rows (queries, keys or values) is D / 64 pieces of 128 x 64
// elements, each in the 128-byte swizzle. Keys and values of the spans travel through one ring of tile buffers, the keys of
// span i as load 2 i, its values as load 2 i + 1: six buffers at head size 64 (three spans in flight), three at 128, where a
// buffer is free again as soon as its keys have been multiplied (early) or its values have (a span later).
// Tensor memory (512 columns): S [0, 128); the value products of the span's two tiles, D columns each, from 128 on; then
// the weights, 128 columns a span (P hi 64, P lo 64; tile t in columns 32 t ..): two buffers by span parity at head size
// 64, one at 128, where the weights of span i + 1 wait for the value product of span i.
template <int D>
struct Shape {
  static constexpr int kSub = D / 64;
  static constexpr int kTileBytes = kSub * kSubTileBytes;
  static constexpr int kRing = D == 64 ? 6 : 3;
  static constexpr int kRowStateBytes = kRows * D * 4;     // the rows' weighted values over the finished chunks, [output][row] float32
  static constexpr int kSmemBytes = (1 + kRing) * kTileBytes + kRowStateBytes;   // Q | ring | row state
  static constexpr uint32_t kTmemP = kTmemO + 2 * D;
  static constexpr int kPBuffers = (kTmemCols - kTmemP) / 128;
  static_assert(kPBuffers >= 1 && kRing <= kMaxRing, "tensor memory or the ring is over budget");
};
using namespace sb::attn;
static_assert(kKeys == 2 * kTileKeys && kChunkKeys == 2 * kKeys, "a span is two tiles, a chunk two spans");

__device__ __forceinline__ void softmax_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

struct Fa5Params {
  bf16* out;
  const int32_t* block_table;
  int max_pages, page_size, page_shift;
  int rows_per_page, rows_v, rows_head;   // distances in rows of D elements inside the key/value map
  int box_rows;                            // rows one TMA box brings: min(page_size, 128)
  const int32_t* meta;
  int meta_stride;
  const int32_t* work;                     // [tiles][2] = (entry, tile in entry)
  int Hq, Hkv, window;
  float scale_log2;
  int* status;
};

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const Fa5Params p) {
  using SH = Shape<D>;
  constexpr int kSub = SH::kSub, kTileBytes = SH::kTileBytes, kRing = SH::kRing, kPB = SH::kPBuffers, kHalfD = D / 2;
  constexpr uint32_t kTmemP = SH::kTmemP;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full, kv_full[kMaxRing], s_full, s_free, p_full[2], o_full, o_free;
  __shared__ uint32_t tmem_base_s;
  __shared__ int32_t pages_s[kPagesCached];
  __shared__ float2 xch[3][2][kRows];      // [span % 3][tile][row]: the tile's maximum and sum, for the row's other thread

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem0 - smem_u32(smem_raw));
  const uint32_t sQ = smem0, sRing = smem0 + kTileBytes;

  const int g = blockIdx.y;
  const int G = p.Hq / p.Hkv, ppt = kRows / G;
  const int e = p.work[2 * blockIdx.x], tile = p.work[2 * blockIdx.x + 1];
  const int slot = p.meta[e], first_row = p.meta[p.meta_stride + e], L = p.meta[2 * p.meta_stride + e],
            first_pos = p.meta[3 * p.meta_stride + e];
  const int p_lo = tile * ppt;
  const int npos = min(ppt, L - p_lo);
  const int row0 = first_row + p_lo, pos0 = first_pos + p_lo, pos_hi = pos0 + npos - 1;
  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int kt0 = key_lo / kKeys, T = pos_hi / kKeys - kt0 + 1;

  if (tid == 0) {
    mbar_init(smem_u32(&q_full), 1);
    for (int i = 0; i < kRing; ++i) mbar_init(smem_u32(&kv_full[i]), 1);
    mbar_init(smem_u32(&s_full), 1);
    mbar_init(smem_u32(&s_free), kSoftmaxThreads);
    for (int i = 0; i < 2; ++i) mbar_init(smem_u32(&p_full[i]), kSoftmaxThreads);   // one per buffer of weights
    mbar_init(smem_u32(&o_full), 1);
    mbar_init(smem_u32(&o_free), kSoftmaxThreads);
    mbar_init_fence();
  }
  if (warp == 8) tmem_alloc(smem_u32(&tmem_base_s), kTmemCols);
  // rows of the query tile that no (position, head) pair fills (G does not divide 128) must still be finite
  for (int i = tid; i < kSub * (kRows - ppt * G) * 8; i += kThreads) {
    const int h = i / ((kRows - ppt * G) * 8), rest = i % ((kRows - ppt * G) * 8);
    *reinterpret_cast<uint4*>(smem + h * kSubTileBytes + (ppt * G * 8 + rest) * 16) = make_uint4(0, 0, 0, 0);
  }
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  sb::grid_launch_dependents();
  sb::grid_dependency_wait();

  if (warp == 8) {
    // the request's block-table entries for the keys this CTA reads, fetched by the whole warp at once
    const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;
    const int page_first = (kt0 * kKeys) >> p.page_shift, page_last = pos_hi >> p.page_shift;
    const bool cached = page_last - page_first < kPagesCached;
    if (cached)
      for (int i = page_first + lane; i <= page_last; i += 32) pages_s[i - page_first] = table[i];
    __syncwarp();
    if (lane == 0) {
      // ------------------------------------------------ control: TMA and MMA issue
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_kv);
      if constexpr (kRing == 6) {
        // Head size 64: three spans in flight, the keys and values of a span under one barrier, the next span's loads
        // issued when the value product of the span before has freed its buffers. (The general ring below, which loads keys
        // and values apart and keys as early as their buffer allows, ran this head size at 100 us instead of 84 for a
        // prompt of 2,048 tokens.)
        constexpr int kStages = 3;
        const uint32_t sK = sRing, sV = sRing + kStages * kTileBytes;
        auto load_kv = [&](int i) {
          const int buf = i % kStages;
          const uint32_t bar = smem_u32(&kv_full[buf]);
          mbar_expect_tx(bar, 2 * kTileBytes);
          for (int sub = 0; sub < kKeys / p.box_rows; ++sub) {
            const int key = (kt0 + i) * kKeys + sub * p.box_rows;
            const int pidx = min(key, pos_hi) >> p.page_shift;
            const int page = cached ? pages_s[pidx - page_first] : table[pidx];
            const int in_page = p.page_size > p.box_rows ? (key & (p.page_size - 1)) : 0;
            const int row = page * p.rows_per_page + g * p.rows_head + in_page;
            tma_load_2d(sK + buf * kTileBytes + sub * p.box_rows * 128, &map_kv, bar, 0, row);
            tma_load_2d(sV + buf * kTileBytes + sub * p.box_rows * 128, &map_kv, bar, 0, row + p.rows_v);
          }
        };
        const uint32_t idesc_qk = instr_desc(kRows, kKeys, false), idesc_pv = instr_desc(kRows, 64, true);
        const uint64_t dQ = smem_desc_sw128(sQ), dK = smem_desc_sw128(sK), dV = smem_desc_sw128(sV);
        constexpr uint64_t kTileStep = kTileBytes >> 4, kVStep = 2048 >> 4;
        auto issue_qk = [&](int i) {
          const uint64_t db = dK + (i % kStages) * kTileStep;
  #pragma unroll
          for (int k = 0; k < 64 / 16; ++k) umma_bf16(tmem_base, dQ + 2 * k, db + 2 * k, idesc_qk, k > 0 ? 1u : 0u);
          umma_commit(smem_u32(&s_full));
        };
        mbar_expect_tx(smem_u32(&q_full), ppt * G * 128);
        tma_load_3d(sQ, &map_q, smem_u32(&q_full), 0, g * G, row0);
        for (int i = 0; i < kStages && i < T; ++i) load_kv(i);
        mbar_wait(smem_u32(&q_full), 0, p.status, 1);
        mbar_wait(smem_u32(&kv_full[0]), 0, p.status, 2);
        fence_after_sync();
        issue_qk(0);
        for (int i = 0; i < T; ++i) {
          mbar_wait(smem_u32(&s_free), i & 1, p.status, 7);
          if (i + 1 < T) {
            mbar_wait(smem_u32(&kv_full[(i + 1) % kStages]), ((i + 1) / kStages) & 1, p.status, 2);
            fence_after_sync();
            issue_qk(i + 1);
          }
          if (i >= 1) {
            mbar_wait(smem_u32(&o_full), (i - 1) & 1, p.status, 4);
            if (i - 1 + kStages < T) load_kv(i - 1 + kStages);
          }
          mbar_wait(smem_u32(&p_full[i & 1]), (i >> 1) & 1, p.status, 3);
          if (i >= 1) mbar_wait(smem_u32(&o_free), (i - 1) & 1, p.status, 8);
          fence_after_sync();
          const uint64_t dv = dV + (i % kStages) * kTileStep;
          const uint32_t tp = tmem_base + kTmemP + (i & 1) * 128;
  #pragma unroll
          for (int ks = 0; ks < kKeys / 16; ++ks) {
            const uint32_t pa = ks * 8;
            const uint32_t d = tmem_base + kTmemO + (ks >> 2) * 64;
            umma_ts_bf16(d, tp + pa, dv + ks * kVStep, idesc_pv, (ks & 3) > 0 ? 1u : 0u);
            umma_ts_bf16(d, tp + 64 + pa, dv + ks * kVStep, idesc_pv, 1u);
          }
          umma_commit(smem_u32(&o_full));
        }
      } else {
        // load j: the keys (j even) or values (j odd) of span j / 2, into buffer j % kRing
        auto load = [&](int j) {
          const int buf = j % kRing, i = j >> 1;
          const uint32_t bar = smem_u32(&kv_full[buf]);
          mbar_expect_tx(bar, kTileBytes);
          for (int sub = 0; sub < kKeys / p.box_rows; ++sub) {
            const int key = (kt0 + i) * kKeys + sub * p.box_rows;
            const int pidx = min(key, pos_hi) >> p.page_shift;       // past the end: the request's last page again
            const int page = cached ? pages_s[pidx - page_first] : table[pidx];
            const int in_page = p.page_size > p.box_rows ? (key & (p.page_size - 1)) : 0;
            const int row = page * p.rows_per_page + g * p.rows_head + in_page + ((j & 1) ? p.rows_v : 0);
  #pragma unroll
            for (int h = 0; h < kSub; ++h)
              tma_load_2d(sRing + buf * kTileBytes + h * kSubTileBytes + sub * p.box_rows * 128, &map_kv, bar, 64 * h, row);
          }
        };
        auto wait_load = [&](int j) { mbar_wait(smem_u32(&kv_full[j % kRing]), (j / kRing) & 1, p.status, 2); };
        // A buffer is free for load j once load j - kRing has been used up: keys by the score product of their span
        // (known when the softmax threads have read the scores), values by the value product of theirs.
        int next = 0, qk_seen = -1, pv_seen = -1;
        auto try_loads = [&]() {
          while (next < 2 * T) {
            const int prev = next - kRing;
            if (prev >= 0 && (prev >> 1) > ((prev & 1) ? pv_seen : qk_seen)) break;
            load(next++);
          }
        };
        // descriptors are built once; a tile, a piece of it, a 64-key half or a K step only adds to the start-address field
        const uint32_t idesc_qk = instr_desc(kRows, kKeys, false), idesc_pv = instr_desc(kRows, 64, true);
        const uint64_t dQ = smem_desc_sw128(sQ), dRing = smem_desc_sw128(sRing);
        constexpr uint64_t kTileStep = kTileBytes >> 4, kSubStep = kSubTileBytes >> 4, kVStep = 2048 >> 4;
        auto issue_qk = [&](int i) {
          const uint64_t db = dRing + ((2 * i) % kRing) * kTileStep;
  #pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_bf16(tmem_base, dQ + (k >> 2) * kSubStep + 2 * (k & 3), db + (k >> 2) * kSubStep + 2 * (k & 3), idesc_qk, k > 0 ? 1u : 0u);
          umma_commit(smem_u32(&s_full));
        };
        mbar_expect_tx(smem_u32(&q_full), kSub * ppt * G * 128);
  #pragma unroll
        for (int h = 0; h < kSub; ++h) tma_load_3d(sQ + h * kSubTileBytes, &map_q, smem_u32(&q_full), 64 * h, g * G, row0);
        try_loads();
        mbar_wait(smem_u32(&q_full), 0, p.status, 1);
        wait_load(0);
        fence_after_sync();
        issue_qk(0);
        // The softmax threads keep a span's scores in registers, so the one S accumulator is free for span i + 1 as soon
        // as all of them have read span i; the value product of span i runs while they compute the weights of span i + 1
        // (with one buffer of weights: while they compute them, before they store them).
        for (int i = 0; i < T; ++i) {
          mbar_wait(smem_u32(&s_free), i & 1, p.status, 7);
          qk_seen = i;
          try_loads();
          bool o_waited = i == 0;
          if (i + 1 < T) {
            if (next <= 2 * (i + 1)) {       // (the short ring only) the next span's keys wait for the buffer of span i - 1's values
              if (!o_waited) {
                mbar_wait(smem_u32(&o_full), (i - 1) & 1, p.status, 4);
                pv_seen = i - 1;
                o_waited = true;
              }
              try_loads();
            }
            wait_load(2 * (i + 1));
            fence_after_sync();
            issue_qk(i + 1);
          }
          if (!o_waited) {
            mbar_wait(smem_u32(&o_full), (i - 1) & 1, p.status, 4);     // then span i - 1's values' buffer is free
            pv_seen = i - 1;
          }
          try_loads();
          // (the softmax threads may be a span ahead: they fill the other buffer of weights while this one is waited for,
          // hence a barrier per buffer)
          mbar_wait(smem_u32(&p_full[i % kPB]), (i / kPB) & 1, p.status, 3);
          if (i >= 1) mbar_wait(smem_u32(&o_free), (i - 1) & 1, p.status, 8);   // the O accumulators have been folded
          wait_load(2 * i + 1);
          fence_after_sync();
          const uint64_t dv = dRing + ((2 * i + 1) % kRing) * kTileStep;
          const uint32_t tp = tmem_base + kTmemP + (i % kPB) * 128;
  #pragma unroll
          for (int ks = 0; ks < kKeys / 16; ++ks) {
            const uint32_t pa = ks * 8;                                    // sixteen keys are eight columns of P
            const uint32_t d = tmem_base + kTmemO + (ks >> 2) * D;         // the tile's accumulator
  #pragma unroll
            for (int h = 0; h < kSub; ++h) {                               // the outputs, 64 at a time
              umma_ts_bf16(d + 64 * h, tp + pa, dv + h * kSubStep + ks * kVStep, idesc_pv, (ks & 3) > 0 ? 1u : 0u);
              umma_ts_bf16(d + 64 * h, tp + 64 + pa, dv + h * kSubStep + ks * kVStep, idesc_pv, 1u);
            }
          }
          umma_commit(smem_u32(&o_full));
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------ softmax: two threads per row of the tile (= TMEM lane);
    // thread `half` takes keys [64 half, 64 half + 64) of every span (one tile) and outputs [D/2 half, D/2 half + D/2)
    const int r = tid & (kRows - 1), half = tid >> 7;
    const int pi = r / G, hh = r % G;
    const bool valid = pi < npos;
    const int row_pos = valid ? pos0 + pi : -1;
    const int row_lo = p.window > 0 ? row_pos - p.window + 1 : 0;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // the chunk in progress and the chunks before it; both threads of a row keep the same maxima and sums
    float m_c = -INFINITY, l_c = 0.0f, m_r = -INFINITY, l_r = 0.0f;
    // (the finished chunks' values live in shared memory, element [output][row], touched once a chunk: registers are
    // needed for the scores of the span in flight)
    float o_c[kHalfD];
    float* o_r = reinterpret_cast<float*>(smem + (1 + kRing) * kTileBytes) + half * kHalfD * kRows + r;
#pragma unroll
    for (int d = 0; d < kHalfD; ++d) {
      o_c[d] = 0.0f;
      o_r[d * kRows] = 0.0f;
    }

    // The scores of span i for this thread's tile: read from tensor memory once (both halves in flight together),
    // the keys the row does not see set to -inf (their weight then comes out as ex2(-inf) = 0), and their maximum.
    auto span_masked = [&](int i) {
      return (kt0 + i) * kKeys + kKeys - 1 > pos0 || (p.window > 0 && (kt0 + i) * kKeys < pos_hi - p.window + 1) || npos * G < kRows;
    };
    uint32_t sv[64];
    auto read_scores = [&](int i) {
      mbar_wait(smem_u32(&s_full), i & 1, p.status, 5);
      fence_after_sync();
      const uint32_t s_addr = tmem_base + lane_addr + half * 64;
      tmem_load32_nowait(s_addr, sv);
      tmem_load32_nowait(s_addr + 32, sv + 32);
      tmem_load_wait();
      fence_before_sync();
      mbar_arrive(smem_u32(&s_free));      // this thread has its scores: the accumulator may be overwritten
      if (span_masked(i)) {
        const int key0 = (kt0 + i) * kKeys + half * 64;
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (!(key0 + j <= row_pos && key0 + j >= row_lo)) sv[j] = 0xff800000u;   // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int j = 0; j < 64; j += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(sv[j]));
        mx1 = fmaxf(mx1, __uint_as_float(sv[j + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(sv[j + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(sv[j + 3]));
      }
      return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
    };

    // Folds the two tiles of span j (their value products are complete) into the chunk, and the chunk into the row.
    auto fold_span = [&](int j) {
      mbar_wait(smem_u32(&o_full), j & 1, p.status, 6);
      fence_after_sync();
      softmax_barrier();    // both threads of every row have written xch[j % 3]; it is rewritten three spans later
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const float2 ml = xch[j % 3][t][r];
        FoldFactors f = fold_factors(m_c, ml.x == -INFINITY ? m_c : ml.x);
#pragma unroll
        for (int q = 0; q < kHalfD / 32; ++q) {
          float v[32];
          tmem_load32(tmem_base + kTmemO + t * D + lane_addr + half * kHalfD + 32 * q, v);
          if (ml.x != -INFINITY) {
#pragma unroll
            for (int k = 0; k < 32; ++k) o_c[32 * q + k] = fold_value(o_c[32 * q + k], v[k], f);
          }
        }
        if (ml.x != -INFINITY) {
          l_c = fold_value(l_c, ml.y, f);
          m_c = f.m;
        }
      }
      fence_before_sync();
      mbar_arrive(smem_u32(&o_free));       // the accumulators may take the next span's products
      if (((kt0 + j) & 1) || j == T - 1) {      // the chunk of 256 keys is complete
        if (m_c != -INFINITY) {
          const FoldFactors f = fold_factors(m_r, m_c);
          l_r = fold_value(l_r, l_c, f);
#pragma unroll
          for (int k = 0; k < kHalfD; ++k) o_r[k * kRows] = fold_value(o_r[k * kRows], o_c[k], f);
          m_r = f.m;
        }
        m_c = -INFINITY;
        l_c = 0.0f;
#pragma unroll
        for (int k = 0; k < kHalfD; ++k) o_c[k] = 0.0f;
      }
    };

    float raw_max = read_scores(0);
    for (int i = 0; i < T; ++i) {
      // weights of span i from the scores in registers, into the weight buffer of its parity
      const float m_t = tile_max(raw_max, p.scale_log2);
      const float ref = tile_ref(m_t);
      const uint32_t tp = tmem_base + kTmemP + (i % kPB) * 128 + lane_addr + half * 32;
      float u0 = 0.0f, u1 = 0.0f, u2 = 0.0f, u3 = 0.0f;     // key j of the tile belongs to class (j % 8) / 2
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float p0 = weight(__uint_as_float(sv[c * 32 + j]), p.scale_log2, ref);
          const float p1 = weight(__uint_as_float(sv[c * 32 + j + 1]), p.scale_log2, ref);
          if ((j & 6) == 0) u0 = __fadd_rn(__fadd_rn(u0, p0), p1);
          else if ((j & 6) == 2) u1 = __fadd_rn(__fadd_rn(u1, p0), p1);
          else if ((j & 6) == 4) u2 = __fadd_rn(__fadd_rn(u2, p0), p1);
          else u3 = __fadd_rn(__fadd_rn(u3, p0), p1);
          split_hi_lo(p0, p1, hi[j >> 1], lo[j >> 1]);
        }
        if (kPB == 1 && c == 0 && i >= 1) {
          // one buffer of weights: the value product of the span before still reads it until its accumulators are full
          mbar_wait(smem_u32(&o_full), (i - 1) & 1, p.status, 9);
          fence_after_sync();
        }
        // 32 keys = sixteen columns of this row (lane), the tile's columns 32 half .. 32 half + 31 of P hi and of P lo
        tmem_store16(tp + c * 16, hi);
        tmem_store16(tp + 64 + c * 16, lo);
      }
      tmem_store_wait();
      xch[i % 3][half][r] = make_float2(m_t, class_sum(u0, u1, u2, u3));
      fence_before_sync();
      mbar_arrive(smem_u32(&p_full[i % kPB]));
      if (i + 1 < T) raw_max = read_scores(i + 1);     // the scores of the next span, computed during the weights of this one
      if (i >= 1) fold_span(i - 1);                    // its value product ran during the weights of span i
    }
    fold_span(T - 1);
    if (valid) {
      bf16* dst = p.out + (static_cast<int64_t>(row0 + pi) * p.Hq + g * G + hh) * D + half * kHalfD;
#pragma unroll
      for (int c = 0; c < kHalfD / 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(finish(o_r[(c * 8 + 2 * j) * kRows], l_r), finish(o_r[(c * 8 + 2 * j + 1) * kRows], l_r));
          w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

// 1 if sb_attention_tc5 takes this shape (head size 64 or 128, at most 128 query heads per key/value head, pages of a
// power of two of at least 8 tokens), else 0.
SB_EXPORT int sb_attention_tc5_supported(int Hq, int Hkv, int D, int page_size) {
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > kRows) return 0;
  if (page_size < 8 || (page_size & (page_size - 1)) != 0) return 0;
  return 1;
}

// Attention of prompt portions. q, out: [n_tokens][Hq * D] bfloat16. k_base: this layer's keys of page 0 inside an
// arena of `pages` pages; strides in elements. work: [n_tiles][2] = (entry, tile), a tile being 128 / (Hq / Hkv)
// consecutive positions of the entry. meta as for sb_attention_tc.
SB_EXPORT int sb_attention_tc5(const void* q, void* out, const void* k_base, int pages, const int32_t* block_table,
                               int max_pages, int page_size, int64_t page_stride, int64_t v_offset, int64_t head_stride,
                               const int32_t* meta, int meta_stride, const int32_t* work, int n_tiles, int n_tokens, int Hq,
                               int Hkv, int D, int window, float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!sb_attention_tc5_supported(Hq, Hkv, D, page_size)) return sb::fail("sb_attention_tc5: shape not supported (Hq %d Hkv %d D %d page %d)", Hq, Hkv, D, page_size);
  if ((page_stride | v_offset | head_stride) % D != 0 || ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_base) | reinterpret_cast<uintptr_t>(out)) & 15))
    return sb::fail("sb_attention_tc5: the cache strides must be multiples of the head size and the pointers 16-byte aligned");
  if (Hkv > 65535) return sb::fail("sb_attention_tc5: too many key/value heads");
  int* status = status_word();
  if (!status) return sb::fail("sb_attention_tc5: cannot allocate the status word");
  const int G = Hq / Hkv, ppt = kRows / G;
  Fa5Params p{};
  p.out = static_cast<bf16*>(out);
  p.block_table = block_table;
  p.max_pages = max_pages;
  p.page_size = page_size;
  p.page_shift = 0;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  p.rows_per_page = static_cast<int>(page_stride / D);
  p.rows_v = static_cast<int>(v_offset / D);
  p.rows_head = static_cast<int>(head_stride / D);
  p.box_rows = page_size < kKeys ? page_size : kKeys;
  p.meta = meta;
  p.meta_stride = meta_stride;
  p.work = work;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.window = window;
  p.scale_log2 = scale * kLog2e;
  p.status = status;

  CUtensorMap map_q, map_kv;
  // (a box is 64 elements wide, one row of the 128-byte swizzle: a head of 128 is fetched as two pieces)
  const int64_t qdims[3] = {D, Hq, n_tokens}, qstrides[3] = {1, D, static_cast<int64_t>(Hq) * D};
  const int qbox[3] = {64, G, ppt};
  const int64_t kv_rows = static_cast<int64_t>(pages - 1) * p.rows_per_page + p.rows_v + static_cast<int64_t>(Hkv) * p.rows_head;
  const int64_t kdims[2] = {D, kv_rows}, kstrides[2] = {1, D};
  const int kbox[2] = {64, p.box_rows};
  if (!tensor_map_bf16(q, 3, qdims, qstrides, qbox, &map_q) || !tensor_map_bf16(k_base, 2, kdims, kstrides, kbox, &map_kv))
    return sb::fail("sb_attention_tc5: cuTensorMapEncodeTiled failed");
  static sb::DeviceOnce once;
  if (once.needed()) {
    if (cudaFuncSetAttribute(attn_prefill_tc5_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<64>::kSmemBytes + 1024) != cudaSuccess ||
        cudaFuncSetAttribute(attn_prefill_tc5_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<128>::kSmemBytes + 1024) != cudaSuccess)
      return sb::fail("sb_attention_tc5: cannot raise the shared memory limit");
    once.done();
  }
  if (D == 64)
    sb::launch_pdl(attn_prefill_tc5_kernel<64>, dim3(n_tiles, Hkv), dim3(kThreads), static_cast<size_t>(Shape<64>::kSmemBytes + 1024), stream, map_q, map_kv, p);
  else
    sb::launch_pdl(attn_prefill_tc5_kernel<128>, dim3(n_tiles, Hkv), dim3(kThreads), static_cast<size_t>(Shape<128>::kSmemBytes + 1024), stream, map_q, map_kv, p);
  return sb::check_launch("sb_attention_tc5");
}

// From now on the kernel reports into `device_word` (see sb_gemm_tc_use_status_word); null: into its own again.
SB_EXPORT void sb_attention_tc5_use_status_word(int* device_word) { status_word_given() = device_word; }

// Reads and clears the status word: 0 = every wait completed. Synchronises the device.
SB_EXPORT int sb_attention_tc5_status() {
  int* status = status_word();
  if (!status) return -1;
  int host = 0;
  if (cudaMemcpy(&host, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (host != 0) cudaMemset(status, 0, sizeof(int));
  return host;
}

// ------------------------------------------------------------------ operation of the native step program (step_ops.h)
// The tiles of the step's tile plan (prompt portions) on the tcgen05 kernel.
// i: 0 q, 1 out, 2 cache layer, 3 pages of the arena, 4 block table, 5 pages per sequence, 6 page size, 7 page stride,
//    8 v offset, 9 head stride, 10 Hq, 11 Hkv, 12 D, 13 window, 14 tile plan; f: 0 scale
SB_EXPORT int sb_op_attention_tc5(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  const SbTilePlan& plan = s->plan[op->i[14]];
  if (plan.fused || plan.tiles <= 0) return SB_OP_SKIPPED;
  return sb_attention_tc5(ptr<const void>(op->i[0]), ptr<void>(op->i[1]), ptr<const void>(op->i[2]), (int)op->i[3],
                          ptr<const int32_t>(op->i[4]), (int)op->i[5], (int)op->i[6], op->i[7], op->i[8], op->i[9], entry_meta(s),
                          s->max_rows, work(s, plan), plan.tiles, s->n, (int)op->i[10], (int)op->i[11], (int)op->i[12], (int)op->i[13],
                          static_cast<float>(op->f[0]), static_cast<cudaStream_t>(stream));
}
