// Paged causal attention of the bfloat16 path on tensor cores (mma.sync m16n8k16, float32
// accumulation, float32 softmax whose weights enter the value product as two bfloat16 parts), for
// head sizes 64 and 128 and any group ratio up to 16.
//
// The query heads that share a key/value head are stacked as rows of one tile: row r of a
// tile is (position r / G, head r % G), G = Hq / Hkv, so a key/value tile read once serves
// all of them. Two kernels cover a step:
//
// * attn_chunk_kernel: prompt portions. One CTA (4 warps, 16 rows each) per (64-row tile
//   of an entry, key/value head); it walks the key tiles [64 t, 64 t + 64) that any of its
//   rows can see and writes the finished rows.
// * attn_decode_kernel: entries whose rows fit one 16-row tile (a decoded token, or a very
//   short portion). One CTA per (entry, key/value head, chunk of 256 absolute key
//   positions); each of its 4 warps takes one 64-key tile, the four results are folded in
//   key order, and the chunk's (max, sum, weighted values) go to scratch memory. The CTA
//   that finishes an entry's last chunk (or attn_combine_kernel) folds the chunks in
//   ascending order and writes bfloat16.
//
// Both follow the arithmetic of attention_math.cuh (tiles of 64 keys, chunks of 256, cut by
// absolute position, each folded from an empty state), as does the tcgen05 kernel of
// attention_tc5.cu: a row's result has the same bits whichever kernel computes it, whatever
// else the step holds and however the request was cut into steps.
//
// Keys and values come from the paged cache through the request's block table
// ([pages][2][Hkv][page_size][D] per layer); a key tile may span several pages.
// Counterparts in arhaamatiq/stride: AttentionPage / AttentionCombine with KvT = bfloat16
// (src/kernel_common.h:90-309), which are scalar.
#include <algorithm>

#include "attention_tc.cuh"
#include "step_ops.h"
#include "noalloc.h"


SB_DEFINE_LAST_ERROR()

namespace {

using namespace sb::attn_tc;
#ifndef SB_DECODE_CTAS64
#define SB_DECODE_CTAS64 6
#endif
constexpr int kDecodeCtas64 = SB_DECODE_CTAS64;   // CTAs of the decode kernel per SM at head size 64 (bounds its registers)


// ------------------------------------------------------------------ prompt portions
template <int D>
__global__ void __launch_bounds__(128) attn_chunk_kernel(const AttnTcParams p) {
  constexpr int LD = D + 8, CH = D / 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);  // [64][LD]
  bf16* sK = sQ + 64 * LD;                       // [2][64][LD]
  bf16* sV = sK + 2 * 64 * LD;                   // [2][64][LD]
  float* sT = reinterpret_cast<float*>(sV + 2 * 64 * LD);   // [64][D]: the rows' weighted values over the finished chunks

  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tq = lane & 3;
  const int g = blockIdx.y;
  const int G = p.Hq / p.Hkv, ppt = 64 / G;
  const int e = p.work[2 * blockIdx.x], t = p.work[2 * blockIdx.x + 1];
  const int slot = p.meta[e], first_row = p.meta[p.meta_stride + e], L = p.meta[2 * p.meta_stride + e],
            first_pos = p.meta[3 * p.meta_stride + e];
  const int p_lo = t * ppt;
  const int npos = min(ppt, L - p_lo);
  const int row0 = first_row + p_lo, pos0 = first_pos + p_lo, pos_hi = pos0 + npos - 1;
  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;
  const bf16* kplane = p.k_base + static_cast<int64_t>(g) * p.head_stride;

  // Q tile: row r = (position r / G, head g * G + r % G)
  for (int idx = tid; idx < 64 * CH; idx += 128) {
    const int r = idx / CH, c = idx % CH;
    const int pi = div_g(p, r), hh = r - pi * G;
    bf16* d = sQ + r * LD + c * 8;
    if (pi < npos)
      cp_async16(smem_u32(d), p.q + (static_cast<int64_t>(row0 + pi) * p.Hq + g * G + hh) * D + c * 8);
    else
      *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
  }
  const int kt0 = key_lo / kKeys, kt1 = pos_hi / kKeys;
  load_kv_tiles<D>(sK, sV, kplane, p.v_offset, table, p.page_size, p.page_shift, p.page_stride, kt0 * kKeys, key_lo, pos_hi, tid, 128);
  cp_commit();

  // rows of this thread: warp * 16 + gid and + 8
  int row_pos[2], row_lo[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + gid + 8 * h;
    const int pi = div_g(p, r);
    row_pos[h] = pi < npos ? pos0 + pi : -1;
    row_lo[h] = p.window > 0 ? row_pos[h] - p.window + 1 : 0;
  }
  // the positions of this warp's rows that are in use (none: -1)
  const int warp_pi = warp * 16 / G;
  const int warp_pos_lo = warp_pi < npos ? pos0 + warp_pi : -1;
  const int warp_pos_hi = pos0 + min(npos - 1, (warp * 16 + 15) / G);
  // the chunk in progress (registers) and the chunks before it (maximum and sum in registers, values in sT,
  // every element of which belongs to one thread)
  float m_c[2] = {-INFINITY, -INFINITY}, l_c[2] = {0.0f, 0.0f}, m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};
  float o_c[D / 8][4];
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      o_c[dt][x] = 0.0f;
      sT[(warp * 16 + gid + 8 * (x >> 1)) * D + dt * 8 + tq * 2 + (x & 1)] = 0.0f;
    }

  for (int kt = kt0; kt <= kt1; ++kt) {
    const int buf = (kt - kt0) & 1;
    cp_wait<0>();
    __syncthreads();
    if (kt < kt1) {
      load_kv_tiles<D>(sK + (buf ^ 1) * 64 * LD, sV + (buf ^ 1) * 64 * LD, kplane, p.v_offset, table, p.page_size, p.page_shift,
                       p.page_stride, (kt + 1) * kKeys, key_lo, pos_hi, tid, 128);
      cp_commit();
    }
    {
      float s[8][4], o_t[D / 8][4], m_t[2], l_t[2];
      qk_tile<D>(s, sQ + warp * 16 * LD, sK + buf * 64 * LD, lane);
      // every row of this warp that is in use sees every key of the tile: nothing to mask
      const bool full = warp_pos_lo >= 0 && kt * kKeys + kKeys - 1 <= warp_pos_lo &&
                        kt * kKeys >= (p.window > 0 ? warp_pos_hi - p.window + 1 : 0);
      tile_partial<D>(s, o_t, m_t, l_t, kt * kKeys, row_pos, row_lo, p.scale_log2, sV + buf * 64 * LD, lane, full);
      fold_rows<D>(m_c, l_c, o_c, m_t, l_t, o_t);
    }
    if ((kt + 1) % (kChunk / kKeys) == 0 || kt == kt1) {
      // the chunk is complete: fold it into the row's state and start an empty one
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (m_c[h] != -INFINITY) {
          const FoldFactors f = fold_factors(m_r[h], m_c[h]);
          l_r[h] = fold_value(l_r[h], l_c[h], f);
          float* row = sT + (warp * 16 + gid + 8 * h) * D + tq * 2;
#pragma unroll
          for (int dt = 0; dt < D / 8; ++dt) {
            row[dt * 8] = fold_value(row[dt * 8], o_c[dt][2 * h], f);
            row[dt * 8 + 1] = fold_value(row[dt * 8 + 1], o_c[dt][2 * h + 1], f);
          }
          m_r[h] = f.m;
        }
        m_c[h] = -INFINITY;
        l_c[h] = 0.0f;
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) o_c[dt][2 * h] = o_c[dt][2 * h + 1] = 0.0f;
      }
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + gid + 8 * h;
    const int pi = div_g(p, r), hh = r - pi * G;
    if (pi < npos) {
      const float* row = sT + r * D + tq * 2;
      bf16* dst = p.out + (static_cast<int64_t>(row0 + pi) * p.Hq + g * G + hh) * D;
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt)
        *reinterpret_cast<uint32_t*>(dst + dt * 8 + tq * 2) = pack_bf16(finish(row[dt * 8], l_r[h]), finish(row[dt * 8 + 1], l_r[h]));
    }
  }
}

// ------------------------------------------------------------------ decoded tokens
// One CTA per unit of attention_tc.cuh's decode_unit. FUSED: the step's queries, keys and values are taken from the
// projection's partial sums, rotated there, and the keys and values are appended to the cache by the CTA whose chunk
// holds their position (no rotation kernel runs).
struct BlockEnv {
  static constexpr bool kFoldAhead = true;    // the next group of chunk records is requested while one is folded
  __device__ __forceinline__ void sync() { __syncthreads(); }
  __device__ __forceinline__ void wait_inputs() { sb::grid_dependency_wait(); }
};
template <int D, bool FUSED, bool CLUSTER>
__global__ void __launch_bounds__(128, FUSED ? 3 : (D == 64 ? kDecodeCtas64 : 3)) attn_decode_kernel(const AttnTcParams p) {
  extern __shared__ __align__(128) uint8_t smem_tiles[];
  __shared__ int is_last_s;
  sb::grid_launch_dependents();
  BlockEnv env;
  // (CLUSTER: the chunk's record lies over the used-up key/value tiles, behind the warps' results [4][16][D + 2]; the
  // cluster is the grid's z extent, so the rank is the chunk)
  static_assert((4 * 16 * (D + 2) + decode_record_floats<D>()) * sizeof(float) <= 4 * 64 * D * sizeof(bf16), "the record must fit over the tiles");
  float* record = CLUSTER ? reinterpret_cast<float*>(smem_tiles) + 4 * 16 * (D + 2) : nullptr;
  decode_unit<D, FUSED, CLUSTER>(p, blockIdx.x, blockIdx.y, blockIdx.z, smem_tiles, &is_last_s, threadIdx.x, env, record);
}

template <int D>
__global__ void __launch_bounds__(D) attn_combine_kernel(const AttnTcParams p) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int item = blockIdx.x, g = blockIdx.y, d = threadIdx.x;
  const int G = p.Hq / p.Hkv;
  const int e = p.work[item];
  const int first_row = p.meta[p.meta_stride + e], L = p.meta[2 * p.meta_stride + e], first_pos = p.meta[3 * p.meta_stride + e];
  const int pos_hi = first_pos + L - 1;
  const int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int c0 = key_lo / kChunk, c1 = pos_hi / kChunk;
  const int64_t rec0 = (static_cast<int64_t>(item) * p.Hkv + g) * p.chunks;
  for (int r = 0; r < L * G; ++r)
    p.out[(static_cast<int64_t>(first_row + r / G) * p.Hq + g * G + r % G) * D + d] =
        __float2bfloat16_rn(fold_chunks<D>(p.part_o, p.part_ml, rec0, c0, c1, r, d));
}

// The same fold for long contexts (tens to hundreds of chunks an entry), where the requests for the records and the
// latency of a chunk's own operations, not their number, set the time. The records of as many chunks as a stage of
// shared memory holds are brought in with asynchronous copies, all in flight at once, while the stage before them is
// folded; and the fold of a stage is taken apart by what hangs on what: (A) a row's running maximum before every chunk,
// a warp's scan (a maximum is exact in any order); (B) the chunks' factors a = ex2(m - m'), b = ex2(m_t - m'), which hang
// on those maxima alone, and the products v_t * b, all threads at once; (C) the sums l and o, one fused multiply-add a
// chunk and element, which is all that has to wait for the chunk before. The operations and their operands are those
// of fold_records. One request of 131,072 cached tokens (512 chunks): the keys and values themselves take 43 us a
// layer; the fold by the CTA that finishes last another 63, this kernel 29.
// A CTA takes kStreamSlice of a head's D outputs: the maxima and factors are computed by every slice's CTA anew, the
// values are shared out.
constexpr int kStreamThreads = 256, kStreamChunks = 128, kStreamSlice = 16;   // threads; most chunks a stage; outputs a CTA
template <int D>
__global__ void __launch_bounds__(kStreamThreads) attn_combine_stream_kernel(const AttnTcParams p, int stage_floats) {
  extern __shared__ __align__(16) float stages[];   // [2][stage_floats]
  __shared__ float before[kStreamChunks][16];        // [chunk of the stage][row]: the row's maximum before the chunk
  __shared__ float factor_a[kStreamChunks][16];      // a of (chunk, row); 1 where the row sees no key of the chunk
  __shared__ float l_rows[16];
  sb::grid_launch_dependents();
  const int item = blockIdx.x, g = blockIdx.y, d0 = blockIdx.z * kStreamSlice;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.Hq / p.Hkv;
  // (the step's work list and entries were copied in before its first kernel: read before waiting for the records)
  const int e = p.work[item];
  const int first_row = p.meta[p.meta_stride + e], L = p.meta[2 * p.meta_stride + e], first_pos = p.meta[3 * p.meta_stride + e];
  sb::grid_dependency_wait();
  const int pos_hi = first_pos + L - 1;
  const int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int c0 = key_lo / kChunk, c1 = pos_hi / kChunk;
  const int64_t rec0 = (static_cast<int64_t>(item) * p.Hkv + g) * p.chunks;
  const int rows = L * G;                                       // at most 16
  // a chunk in a stage: its rows' values of this slice [rows][kStreamSlice], then the rows' (maximum, sum) pairs, padded to 16 bytes
  const int o_floats = rows * kStreamSlice, chunk_floats = o_floats + (rows * 2 + 3) / 4 * 4;
  const int S = max(8, min(kStreamChunks, stage_floats / chunk_floats) & ~7);   // chunks a stage, a multiple of 8 (the host sizes a stage for at least 32 chunks of 16 rows)
  auto request = [&](int first, int buf) {     // a warp brings whole chunks, 16 bytes a lane and copy
    const int n = min(S, c1 - first + 1);
    const uint32_t dst = smem_u32(stages + buf * stage_floats);
    for (int c = warp; c < n; c += kStreamThreads / 32) {
      const float* src_o = p.part_o + (rec0 + first + c) * 16 * D + d0;
      const float* src_ml = p.part_ml + (rec0 + first + c) * 32;
      for (int q = 4 * lane; q < chunk_floats; q += 128)
        cp_async16(dst + (c * chunk_floats + q) * 4,
                   q < o_floats ? src_o + (q / kStreamSlice) * D + q % kStreamSlice : src_ml + (q - o_floats));
    }
    cp_commit();
  };
  float m_row = -INFINITY;                       // (A) the running maximum of row `warp`, in every lane of warps < rows
  // (C) thread (row r_c, j_c): j_c < kStreamSlice / 2: the outputs d0 + 2 j_c and the next; j_c == kStreamSlice / 2: the sum l (in o0)
  constexpr int kCols = kStreamSlice / 2 + 1;
  float o0 = 0.0f, o1 = 0.0f;
  const int r_c = tid / kCols, j_c = tid % kCols;
  request(c0, 0);
  int buf = 0;
  for (int first = c0; first <= c1; first += S, buf ^= 1) {
    const bool more = first + S <= c1;
    if (more) request(first + S, buf ^ 1);
    if (more) cp_wait<1>();
    else cp_wait<0>();
    __syncthreads();
    float* src = stages + buf * stage_floats;
    const int n = min(S, c1 - first + 1);
    // (A) warp r scans row r's maxima, 32 chunks at a time (a maximum is exact in any order)
    for (int r = warp; r < rows; r += kStreamThreads / 32) {
      float m_run = __shfl_sync(0xffffffffu, m_row, r / (kStreamThreads / 32));   // lane j keeps the warp's j-th row
      for (int cb = 0; cb < n; cb += 32) {
        const int c = cb + lane;
        // (a chunk without a key for the row has -inf, which leaves a maximum as it is)
        float incl = c < n ? src[c * chunk_floats + o_floats + r * 2] : -INFINITY;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float y = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl = fmaxf(incl, y);
        }
        float excl = __shfl_up_sync(0xffffffffu, incl, 1);
        excl = lane == 0 ? m_run : fmaxf(m_run, excl);
        if (c < n) before[c][r] = excl;
        m_run = fmaxf(m_run, __shfl_sync(0xffffffffu, incl, 31));
      }
      if (lane == r / (kStreamThreads / 32)) m_row = m_run;
    }
    __syncthreads();
    // (B) the factors of every (chunk, row), and the chunk's values and sum times b, in place. A chunk in which the row
    // sees no key, and the places that fill the stage's last group of eight, get a = 1 and values -0: (C) then leaves
    // the sums as they are, bit for bit (x * 1 + -0 = x for every x, either zero included), without asking.
    for (int i = tid; i < ((n + 7) & ~7) * rows; i += kStreamThreads) {
      const int c = i / rows, r = i - c * rows;
      float* rec = src + c * chunk_floats;
      const float m_t = c < n ? rec[o_floats + r * 2] : -INFINITY;
      float a = 1.0f, b = 0.0f;
      if (m_t != -INFINITY) {
        const FoldFactors f = fold_factors(before[c][r], m_t);
        a = f.a, b = f.b;
      }
      const bool use = m_t != -INFINITY;
      rec[o_floats + r * 2 + 1] = use ? __fmul_rn(rec[o_floats + r * 2 + 1], b) : -0.0f;
#pragma unroll
      for (int q = 0; q < kStreamSlice / 4; ++q) {
        float4 v = *reinterpret_cast<float4*>(rec + r * kStreamSlice + 4 * q);
        v.x = use ? __fmul_rn(v.x, b) : -0.0f, v.y = use ? __fmul_rn(v.y, b) : -0.0f;
        v.z = use ? __fmul_rn(v.z, b) : -0.0f, v.w = use ? __fmul_rn(v.w, b) : -0.0f;
        *reinterpret_cast<float4*>(rec + r * kStreamSlice + 4 * q) = v;
      }
      factor_a[c][r] = a;
    }
    __syncthreads();
    // (C) the sums; eight chunks' operands are read before they are chained
    if (r_c < rows) {
      const float* wp = j_c < kStreamSlice / 2 ? src + r_c * kStreamSlice + 2 * j_c : src + o_floats + r_c * 2;   // (the sum: the pair (m_t, l_t b))
      const float* ap = &factor_a[0][r_c];
      int off[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) off[u] = u * chunk_floats;
      for (int c = 0; c < n; c += 8, wp += 8 * chunk_floats, ap += 8 * 16) {
        float a[8];
        float2 w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          a[u] = ap[u * 16];
          w[u] = *reinterpret_cast<const float2*>(wp + off[u]);
        }
        if (j_c < kStreamSlice / 2) {
#pragma unroll
          for (int u = 0; u < 8; ++u) o0 = __fmaf_rn(o0, a[u], w[u].x), o1 = __fmaf_rn(o1, a[u], w[u].y);
        } else {
#pragma unroll
          for (int u = 0; u < 8; ++u) o0 = __fmaf_rn(o0, a[u], w[u].y);
        }
      }
    }
    __syncthreads();   // this stage is requested again in the next round; `before` and `factor_a` are rewritten
  }
  if (r_c < rows && j_c == kStreamSlice / 2) l_rows[r_c] = o0;
  __syncthreads();
  if (r_c < rows && j_c < kStreamSlice / 2) {
    const int pi = div_g(p, r_c);
    const float l = l_rows[r_c];
    *reinterpret_cast<uint32_t*>(p.out + (static_cast<int64_t>(first_row + pi) * p.Hq + g * G + r_c - pi * G) * D + d0 + 2 * j_c) =
        pack_bf16(finish(o0, l), finish(o1, l));
  }
}

// From this many chunks on the records are folded by attn_combine_stream_kernel, while the entries are few (with many,
// the fold by each entry's last CTA hides under the other entries' CTAs).
constexpr int kStreamFoldChunks = 32;
constexpr size_t kStreamStageBytes = 40 * 1024;

template <int D>
int launch(const AttnTcParams& p, int n_tiles, int n_items, cudaStream_t stream) {
  constexpr int LD = D + 8;
  if (n_tiles > 0) {
    const size_t smem = static_cast<size_t>(5) * 64 * LD * sizeof(bf16) + static_cast<size_t>(64) * D * sizeof(float);
    static sb::DeviceOnce once;
    if (once.needed()) {
      if (cudaFuncSetAttribute(attn_chunk_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return sb::fail("sb_attention_tc: cannot raise the shared memory limit");
      once.done();
    }
    sb::launch_pdl(attn_chunk_kernel<D>, dim3(n_tiles, p.Hkv), dim3(128), smem, stream, p);
  }
  if (n_items > 0) {
    // queries and the warps' tiles (keys and values, or one for both in turn); the results (4 x 16 x (D + 2) floats) reuse the tiles
    const size_t smem_fused = static_cast<size_t>(16 * LD + 8 * 64 * LD) * sizeof(bf16);
    const size_t smem = static_cast<size_t>(16 * LD + 4 * 64 * D) * sizeof(bf16);
    static_assert(4 * 64 * D * sizeof(bf16) >= 4 * 16 * (D + 2) * sizeof(float), "the results must fit over the tiles");
    static sb::DeviceOnce once;
    if (once.needed()) {
      if (cudaFuncSetAttribute(attn_decode_kernel<D, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
          cudaFuncSetAttribute(attn_decode_kernel<D, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_fused) != cudaSuccess ||
          cudaFuncSetAttribute(attn_decode_kernel<D, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
          cudaFuncSetAttribute(attn_decode_kernel<D, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_fused) != cudaSuccess)
        return sb::fail("sb_attention_tc: cannot raise the shared memory limit");
      once.done();
    }
    AttnTcParams pd = p;
    pd.work = p.work + 2 * n_tiles;
    const bool stream_fold = p.chunks >= kStreamFoldChunks && static_cast<long long>(n_items) * p.Hkv * (D / kStreamSlice) <= 2ll * sb::sm_count();
    if (stream_fold) pd.counters = nullptr;    // every chunk leaves its record; no CTA folds
    const dim3 grid(n_items, p.Hkv, p.chunks);
    // 2 to 8 chunks whose records the kernel folds itself: the chunks of an entry as one cluster (records through
    // distributed shared memory); one chunk needs no fold, more than 8 go through records in global memory and a ticket
    // (measured: a cluster of two is the faster way at every batch size; larger clusters only while all CTAs of the
    // launch run at once: 128 entries x 8 heads x 3 chunks 83 us with records in global memory, 91 us in clusters)
    const bool cluster = pd.counters != nullptr && p.chunks >= 2 && p.chunks <= 8 &&
                         (p.chunks == 2 || static_cast<long long>(n_items) * p.Hkv * p.chunks <= 2ll * sb::sm_count());
    if (cluster) {
      const dim3 shape(1, 1, p.chunks);
      if (p.qkv != nullptr) sb::launch_pdl_cluster(attn_decode_kernel<D, true, true>, grid, dim3(128), smem_fused, stream, shape, pd);
      else sb::launch_pdl_cluster(attn_decode_kernel<D, false, true>, grid, dim3(128), smem, stream, shape, pd);
    } else if (p.qkv != nullptr) {
      sb::launch_pdl(attn_decode_kernel<D, true, false>, grid, dim3(128), smem_fused, stream, pd);
    } else {
      sb::launch_pdl(attn_decode_kernel<D, false, false>, grid, dim3(128), smem, stream, pd);
    }
    if (stream_fold) {
      // two stages, each with room for all chunks (of 16 rows, in whole groups of eight) if that fits
      const size_t chunk_bytes = static_cast<size_t>(16 * kStreamSlice + 32) * sizeof(float);
      const size_t stage = std::min(kStreamStageBytes, static_cast<size_t>((p.chunks + 7) / 8 * 8) * chunk_bytes);
      static sb::DeviceOnce once_stream;
      if (once_stream.needed()) {
        if (cudaFuncSetAttribute(attn_combine_stream_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * kStreamStageBytes)) != cudaSuccess)
          return sb::fail("sb_attention_tc: cannot raise the shared memory limit");
        once_stream.done();
      }
      sb::launch_pdl(attn_combine_stream_kernel<D>, dim3(n_items, p.Hkv, D / kStreamSlice), dim3(kStreamThreads), 2 * stage, stream, pd,
                     static_cast<int>(stage / sizeof(float)));
    } else if (pd.counters == nullptr) {
      sb::launch_pdl(attn_combine_kernel<D>, dim3(n_items, p.Hkv), dim3(D), 0, stream, pd);
    }
  }
  return sb::check_launch("sb_attention_tc");
}

}  // namespace

// Floats of scratch that `sb_attention_tc` needs for `items` short entries and `chunks` key chunks.
// How many CTAs of the fused rotate + append + attend decode kernel run at once on the current device: up to this many
// (entries x key/value heads x chunks) the fused kernel is the faster choice, beyond it the separate rotation kernel is
// (both give the same bits). Two CTAs of its shared-memory size fit an SM.
SB_EXPORT int sb_attention_decode_rope_resident_ctas() { return 2 * sb::sm_count(); }

SB_EXPORT int64_t sb_attention_tc_scratch(int items, int Hkv, int chunks, int D) {
  return static_cast<int64_t>(items) * Hkv * chunks * 16 * (D + 2);
}

// work: [n_tiles][2] (entry, tile) for the portion kernel, followed by [n_items] entries for the decode
// kernel. An entry belongs to the decode kernel iff length * (Hq / Hkv) <= 16. chunks = greatest
// (last position of a decode entry) / 256 + 1. scratch: sb_attention_tc_scratch(...) floats.
namespace {
int attention_tc_impl(const void* q, void* out, const void* k_base, const int32_t* block_table, int max_pages,
                      int page_size, int64_t page_stride, int64_t v_offset, int64_t head_stride,
                      const int32_t* meta, int meta_stride, const int32_t* work, int n_tiles, int n_items,
                      int chunks, float* scratch, int* counters, int Hq, int Hkv, int D, int window, float scale,
                      const float* qkv, int n_partials, int64_t partial_stride, const float* cos_sin, cudaStream_t stream) {
  if (n_tiles <= 0 && n_items <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > 16)
    return sb::fail("sb_attention_tc: group ratio %d/%d is not supported (1..16)", Hq, Hkv);
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_base)) & 15 || (page_stride | v_offset | head_stride) % 8)
    return sb::fail("sb_attention_tc: q and the cache must be 16-byte aligned");
  if (Hkv > 65535 || chunks > 65535) return sb::fail("sb_attention_tc: grid too large");
  AttnTcParams p{};
  p.q = static_cast<const bf16*>(q);
  p.out = static_cast<bf16*>(out);
  p.k_base = static_cast<const bf16*>(k_base);
  p.block_table = block_table;
  p.max_pages = max_pages;
  p.page_size = page_size;
  p.page_shift = -1;
  for (int b = 0; b < 31; ++b)
    if ((1 << b) == page_size) p.page_shift = b;
  p.page_stride = page_stride;
  p.v_offset = v_offset;
  p.head_stride = head_stride;
  p.meta = meta;
  p.meta_stride = meta_stride;
  p.work = work;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.g_mul = (65536 + Hq / Hkv - 1) / (Hq / Hkv);
  for (int r = 0; r < 64; ++r)
    if (((r * p.g_mul) >> 16) != r / (Hq / Hkv)) return sb::fail("sb_attention_tc: the row arithmetic does not hold for %d/%d heads", Hq, Hkv);
  p.window = window;
  p.scale_log2 = scale * kLog2e;
  p.chunks = chunks;
  p.part_o = scratch;
  p.part_ml = scratch + static_cast<int64_t>(n_items) * Hkv * chunks * 16 * D;
  p.counters = counters;
  p.qkv = qkv;
  p.n_partials = n_partials;
  p.partial_stride = partial_stride;
  p.cos_sin = cos_sin;
  if (D == 64) return launch<64>(p, n_tiles, n_items, stream);
  if (D == 128) return launch<128>(p, n_tiles, n_items, stream);
  return sb::fail("sb_attention_tc: head_dim %d has no tensor-core kernel (64 or 128)", D);
}
}  // namespace

SB_EXPORT int sb_attention_tc(const void* q, void* out, const void* k_base, const int32_t* block_table, int max_pages,
                              int page_size, int64_t page_stride, int64_t v_offset, int64_t head_stride,
                              const int32_t* meta, int meta_stride, const int32_t* work, int n_tiles, int n_items,
                              int chunks, float* scratch, int* counters, int Hq, int Hkv, int D, int window, float scale,
                              cudaStream_t stream) {
  return attention_tc_impl(q, out, k_base, block_table, max_pages, page_size, page_stride, v_offset, head_stride, meta, meta_stride,
                           work, n_tiles, n_items, chunks, scratch, counters, Hq, Hkv, D, window, scale, nullptr, 0, 0, nullptr, stream);
}

// The decode kernel with the rotation and the append fused in, for a step whose entries all fit it (length * (Hq / Hkv)
// <= 16 each): qkv [n_partials][n][(Hq + 2 Hkv) D] float32 are the projection's partial sums (added in ascending
// order), cos_sin [positions][D / 2][2] the rotation table of a fully rotated head. Queries are rotated in shared
// memory; the step's keys and values are rotated, rounded and written to the cache (k_base is written) by the CTA
// whose chunk holds their position. Same bits as sb_rope_append followed by sb_attention_tc.
SB_EXPORT int sb_attention_decode_rope(const float* qkv, int n_partials, int64_t partial_stride, const float* cos_sin, void* out,
                                       void* k_base, const int32_t* block_table, int max_pages, int page_size, int64_t page_stride,
                                       int64_t v_offset, int64_t head_stride, const int32_t* meta, int meta_stride,
                                       const int32_t* items, int n_items, int chunks, float* scratch, int* counters, int Hq, int Hkv,
                                       int D, int window, float scale, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (qkv == nullptr || cos_sin == nullptr || n_partials < 1) return sb::fail("sb_attention_decode_rope: qkv and cos_sin are required");
  if ((reinterpret_cast<uintptr_t>(cos_sin) & 7) != 0) return sb::fail("sb_attention_decode_rope: cos_sin must be 8-byte aligned");
  return attention_tc_impl(out, out, k_base, block_table, max_pages, page_size, page_stride, v_offset, head_stride, meta, meta_stride,
                           items, 0, n_items, chunks, scratch, counters, Hq, Hkv, D, window, scale, qkv, n_partials, partial_stride,
                           cos_sin, stream);
}


// ------------------------------------------------------------------ the entry point that allocates nothing
namespace {

// Scratch of sb_attention_decode_noalloc: the chunk records of the decode kernel. Every GPU that loads
// this library holds these 16 MiB from load to exit, whether the entry point is used or not.
static __device__ __align__(256) float g_noalloc_scratch[SB_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_noalloc_scratch_ptr[kMaxDevices] = {nullptr};

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a kernel can use; the
// device address has to be asked for, once per device, with that device current.
int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return sb::fail("sb_attention_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return sb::fail("sb_attention_decode_noalloc: device %d is beyond the %d this library tracks", dev, kMaxDevices);
  if (g_noalloc_scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return sb::fail("sb_attention_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_noalloc_scratch_ptr[dev] = ptr;
  }
  *out = g_noalloc_scratch_ptr[dev];
  return 0;
}

}  // namespace

SB_EXPORT int sb_attention_decode_noalloc(const void* q, void* out, const void* k_base, const int32_t* block_table,
                                          int max_pages, int page_size, int64_t page_stride, int64_t v_offset,
                                          int64_t head_stride, const int32_t* meta, int meta_stride, const int32_t* items,
                                          int n_items, int chunks, int Hq, int Hkv, int D, int window, float scale,
                                          cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (chunks <= 0 || Hkv <= 0) return sb::fail("sb_attention_decode_noalloc: chunks and Hkv must be positive");
  const int64_t need = sb_attention_tc_scratch(n_items, Hkv, chunks, D);
  if (need > SB_NOALLOC_SCRATCH_FLOATS)
    return sb::fail("sb_attention_decode_noalloc: %d entries x %d kv heads x %d chunks x head_dim %d need %lld floats of scratch; "
                    "the built-in array holds %lld (use sb_attention_tc with your own scratch for larger steps)",
                    n_items, Hkv, chunks, D, (long long)need, (long long)SB_NOALLOC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  if (int rc = noalloc_scratch(&scratch)) return rc;
  return sb_attention_tc(q, out, k_base, block_table, max_pages, page_size, page_stride, v_offset, head_stride, meta,
                         meta_stride, items, 0, n_items, chunks, scratch, nullptr, Hq, Hkv, D, window, scale, stream);
}

// ------------------------------------------------------------------ operation of the native step program (step_ops.h)
// The decode items of the step's tile plan (and its tiles, unless the tcgen05 kernel took them) on the mma.sync
// kernels; with a fused plan, rotation and append run inside the decode kernel, from the projection's partial sums.
// i: 0 q, 1 out, 2 cache layer, 3 block table, 4 pages per sequence, 5 page size, 6 page stride, 7 v offset, 8 head stride,
//    9 where the scratch buffer is noted (two int64 on the host: its device address and its size in floats; the engine
//    enlarges the buffer before a step that needs more), 10 unused, 11 counters, 12 Hq, 13 Hkv, 14 D, 15 window, 16 tile plan,
//    17 the tiles went to the tcgen05 kernel, 18 qkv partial sums (flat), 19 their width, 20 K ranges S,
//    21 most tokens with a buffer per range, 22 cos_sin; f: 0 scale
SB_EXPORT int sb_op_attention_tc(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  const SbTilePlan& plan = s->plan[op->i[16]];
  const int Hq = (int)op->i[12], Hkv = (int)op->i[13], D = (int)op->i[14];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t* noted = ptr<const int64_t>(op->i[9]);
  float* scratch = ptr<float>(noted[0]);
  if (plan.items > 0 && sb_attention_tc_scratch(plan.items, Hkv, plan.chunks, D) > noted[1])
    return sb::fail("sb_op_attention_tc: %d decode entries over %d chunks need more scratch than the engine set aside (%lld floats)",
                    plan.items, plan.chunks, (long long)noted[1]);
  if (plan.fused) {
    const int P = partial_count(op->i[20], op->i[21], s->n);
    return sb_attention_decode_rope(ptr<const float>(op->i[18]), P, static_cast<int64_t>(s->n) * op->i[19], ptr<const float>(op->i[22]),
                                    ptr<void>(op->i[1]), ptr<void>(op->i[2]), ptr<const int32_t>(op->i[3]), (int)op->i[4], (int)op->i[5],
                                    op->i[6], op->i[7], op->i[8], entry_meta(s), s->max_rows, work(s, plan), plan.items, plan.chunks,
                                    scratch, ptr<int>(op->i[11]), Hq, Hkv, D, (int)op->i[15], static_cast<float>(op->f[0]), st);
  }
  const int tiles = op->i[17] ? 0 : plan.tiles;
  if (tiles <= 0 && plan.items <= 0) return SB_OP_SKIPPED;
  const int32_t* list = work(s, plan) + (op->i[17] ? 2 * plan.tiles : 0);
  return sb_attention_tc(ptr<const void>(op->i[0]), ptr<void>(op->i[1]), ptr<const void>(op->i[2]), ptr<const int32_t>(op->i[3]),
                         (int)op->i[4], (int)op->i[5], op->i[6], op->i[7], op->i[8], entry_meta(s), s->max_rows, list, tiles, plan.items,
                         plan.chunks, scratch, ptr<int>(op->i[11]), Hq, Hkv, D, (int)op->i[15], static_cast<float>(op->f[0]), st);
}
