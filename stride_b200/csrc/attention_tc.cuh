// Device code of the mma.sync attention kernels (attention_tc.cu), shared with the fused decode chain (decode_chain.cu):
// the parameters, the tile loads, the score / weight / value products of one 64-key tile for one warp, and the work of
// one (entry, key/value head, 256-key chunk) unit of the decode kernel. All arithmetic follows attention_math.cuh.
#pragma once

#include "attention_math.cuh"
#include "common.cuh"

namespace sb {
namespace attn_tc {

using bf16 = __nv_bfloat16;
using namespace sb::attn;
constexpr int kKeys = kTileKeys;    // keys per tile
constexpr int kChunk = kChunkKeys;  // keys per chunk (4 tiles; the decode kernel gives each warp one)

struct AttnTcParams {
  const bf16* q;     // [n][Hq * D]
  bf16* out;         // [n][Hq * D]
  const bf16* k_base;
  const int32_t* block_table;
  int max_pages, page_size, page_shift;   // page_shift: log2(page_size), or -1 if it is no power of two
  int64_t page_stride, v_offset, head_stride;
  const int32_t* meta;   // [4][meta_stride]: slot, first row, length, first position of every entry
  int meta_stride;
  const int32_t* work;   // chunk kernel: [tiles][2] = (entry, tile in entry); decode kernel: [items] = entry
  int Hq, Hkv;
  int g_mul;             // ceil(65536 / (Hq / Hkv)): r / G = (r * g_mul) >> 16 for the row numbers that occur (checked on the host)
  int window;
  float scale_log2;      // softmax scale * log2(e)
  // decode only
  float* part_o;         // [items][Hkv][chunks][16][D]
  float* part_ml;        // [items][Hkv][chunks][16][2]
  int chunks;
  int* counters;         // [items][Hkv], zero between launches; null: the chunks are folded by attn_combine_kernel
  // decode with the rotation fused in (qkv != null): q, k, v come from the projection's partial sums
  const float* qkv;      // [n_partials][n][(Hq + 2 Hkv) D], summed in ascending order
  int n_partials;
  int64_t partial_stride;
  const float* cos_sin;  // [positions][D / 2][2]
};

// Row r of a tile is (position r / G, head r % G); G is not known at compile time, so the division is a multiplication.
__device__ __forceinline__ int div_g(const AttnTcParams& p, int r) { return (r * p.g_mul) >> 16; }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copies keys and values [key0, key0 + 64) of one kv head into dstK and dstV ([64][D + 8] each); keys outside
// [key_lo, key_hi] are zero-filled. `threads` threads of the caller take part (tid in 0..threads-1): D / 8
// threads share a key (one 16-byte piece each), so the page is looked up once for a key's key and value rows.
// Element offset of the 16-byte piece `piece` of row `row` of a [64][D] tile. SW = false: rows of D + 8 elements
// (the padding keeps ldmatrix off bank conflicts). SW = true: rows of D elements, the piece's low three bits XORed
// with the row's, which does the same without the padding.
template <int D, bool SW>
__device__ __forceinline__ int tile_offset(int row, int piece) {
  return SW ? row * D + ((piece ^ (row & 7)) << 3) : row * (D + 8) + (piece << 3);
}

// WHICH: 1 = keys only, 2 = values only, 3 = both.
template <int D, int WHICH = 3, bool SW = false>
__device__ __forceinline__ void load_kv_tiles(bf16* dstK, bf16* dstV, const bf16* kplane, int64_t v_offset,
                                              const int32_t* table, int page_size, int page_shift, int64_t page_stride,
                                              int key0, int key_lo, int key_hi, int tid, int threads,
                                              int zero_lo = 0, int zero_hi = -1) {
  // keys in [key_lo, key_hi] are copied; keys outside [zero_lo, zero_hi] (by default: outside the copied range) are
  // zero-filled; keys in between are left for a later call
  if (zero_hi < zero_lo) {
    zero_lo = key_lo;
    zero_hi = key_hi;
  }
  constexpr int LD = D + 8, CH = D / 8;
  const int c = tid % CH;
  // A tile starts at a multiple of 64 keys, so with pages of 64, 128, ... keys it lies in one page, which is looked
  // up once (the copies then do not wait for a table entry each). The entry is only used for keys that are copied.
  const bool one_page = page_shift >= 6;
  const bf16* page0 = one_page && key_lo <= key_hi ? kplane + static_cast<int64_t>(table[key0 >> page_shift]) * page_stride : kplane;
  if (one_page && key0 >= key_lo && key0 + kKeys - 1 <= key_hi) {
    // the whole tile is wanted and lies in one page: 64 rows of D elements in a row, copied without a test per key
    // (one address of each kind is computed; the copies differ by constants)
    const int i0 = tid / CH;
    const bf16* srck = page0 + ((key0 & (page_size - 1)) + i0) * D + c * 8;
    const bf16* srcv = srck + v_offset;
    constexpr int RS = SW ? D : LD;       // elements per row of the tile
    if (threads == 32) {
      // rows i0 + ph * S + 8 j: those of one ph share the row's low three bits, hence the swizzled piece
      constexpr int S = 32 / CH, P = 8 / S;
#pragma unroll
      for (int ph = 0; ph < P; ++ph) {
        const int off = tile_offset<D, SW>(i0 + ph * S, c);
        const uint32_t dk = smem_u32(dstK + off), dv = smem_u32(dstV + off);
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) {
          if (WHICH & 1) cp_async16(dk + j * 8 * RS * 2, srck + (ph * S + 8 * j) * D);
          if (WHICH & 2) cp_async16(dv + j * 8 * RS * 2, srcv + (ph * S + 8 * j) * D);
        }
      }
    } else {
      // 128 threads: a thread's rows are 8 or 16 apart
      const int off = tile_offset<D, SW>(i0, c);
      const uint32_t dk = smem_u32(dstK + off), dv = smem_u32(dstV + off);
#pragma unroll
      for (int it = 0; it < kKeys / (128 / CH); ++it) {
        if (WHICH & 1) cp_async16(dk + it * (128 / CH) * RS * 2, srck + it * (128 / CH) * D);
        if (WHICH & 2) cp_async16(dv + it * (128 / CH) * RS * 2, srcv + it * (128 / CH) * D);
      }
    }
    return;
  }
  for (int i = tid / CH; i < kKeys; i += threads / CH) {
    const int key = key0 + i;
    bf16* dk = dstK + tile_offset<D, SW>(i, c);
    bf16* dv = dstV + tile_offset<D, SW>(i, c);
    if (key >= key_lo && key <= key_hi) {
      const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
      const int in_page = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
      const bf16* src = (one_page ? page0 : kplane + static_cast<int64_t>(table[pi]) * page_stride) + in_page * D + c * 8;
      if (WHICH & 1) cp_async16(smem_u32(dk), src);
      if (WHICH & 2) cp_async16(smem_u32(dv), src + v_offset);
    } else if (key < zero_lo || key > zero_hi) {
      if (WHICH & 1) *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
      if (WHICH & 2) *reinterpret_cast<uint4*>(dv) = make_uint4(0, 0, 0, 0);
    }
  }
}

// S[16 x 64] = Q[16 x D] K^T for one warp; Q rows at sQ (16 rows of this warp) and the K tile in shared memory.
template <int D, bool SW = false>
__device__ __forceinline__ void qk_tile(float (*s)[4], const bf16* sQ, const bf16* sK, int lane) {
  constexpr int LD = D + 8;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
  const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t qf[4];
    ldsm_x4(qf, smem_u32(sQ + (lane & 15) * LD + ks * 16 + (lane >> 4) * 8));
#pragma unroll
    for (int nt = 0; nt < 8; nt += 2) {
      uint32_t b[4];
      ldsm_x4(b, smem_u32(sK + tile_offset<D, SW>(nt * 8 + (mi >> 1) * 8 + rr, ks * 2 + (mi & 1))));
      mma_16816(s[nt], qf, b[0], b[1]);
      mma_16816(s[nt + 1], qf, b[2], b[3]);
    }
  }
}

// O[16 x D] = P[16 x 64] V[64 x D] from zero; P given as float weights in the layout of qk_tile's accumulators.
// Each weight enters as two bfloat16 parts (split_hi_lo), hi . V then lo . V for every step of 16 keys.
// kUpper = false: rows 8..15 of the tile are not in use; their weights are taken as zero without being looked at.
template <int D, bool kUpper = true, bool SW = false>
__device__ __forceinline__ void pv_tile(float (*o)[4], const float (*s)[4], const bf16* sV, int lane) {
  const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
    for (int x = 0; x < 4; ++x) o[dt][x] = 0.0f;
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      if (!kUpper && (x & 1)) hi[x] = lo[x] = 0u;
      else split_hi_lo(s[2 * kk + (x >> 1)][(x & 1) * 2], s[2 * kk + (x >> 1)][(x & 1) * 2 + 1], hi[x], lo[x]);
    }
#pragma unroll
    for (int dt = 0; dt < D / 8; dt += 2) {
      uint32_t b[4];
      ldsm_x4_trans(b, smem_u32(sV + tile_offset<D, SW>(kk * 16 + (mi & 1) * 8 + rr, dt + (mi >> 1))));
      mma_16816(o[dt], hi, b[0], b[1]);
      mma_16816(o[dt + 1], hi, b[2], b[3]);
      mma_16816(o[dt], lo, b[0], b[1]);
      mma_16816(o[dt + 1], lo, b[2], b[3]);
    }
  }
}

// The weights of one tile for one warp: s holds the raw scores of keys key0 .. key0 + 63 for the thread's two rows
// (gid, gid + 8) and leaves their weights; m_t, l_t are the tile's maximum and sum per row. `full` (the same for the
// whole warp): every row in use sees every key of the tile, so nothing is masked. kUpper = false: rows 8..15 are not
// in use and are left out (maximum -inf, sum 0; their entries of s are not touched).
template <bool kUpper>
__device__ __forceinline__ void tile_weights(float (*s)[4], float* m_t, float* l_t, int key0, const int* row_pos, const int* row_lo,
                                             float c, int lane, bool full) {
  constexpr int X = kUpper ? 4 : 2, H = kUpper ? 2 : 1;
  const int tq = lane & 3;
  if (!full) {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int x = 0; x < X; ++x) {
        const int h = x >> 1;
        const int key = key0 + nt * 8 + tq * 2 + (x & 1);
        if (!(key <= row_pos[h] && key >= row_lo[h])) s[nt][x] = -INFINITY;
      }
  }
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int x = 0; x < X; ++x) mx[x >> 1] = fmaxf(mx[x >> 1], s[nt][x]);
  float ref[2], u[2] = {0.0f, 0.0f};
  m_t[1] = -INFINITY;
  l_t[1] = 0.0f;
#pragma unroll
  for (int h = 0; h < H; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    m_t[h] = tile_max(mx[h], c);
    ref[h] = tile_ref(m_t[h]);
  }
  // this thread holds class tq of its rows' keys, in ascending order; a score of -inf (a masked key) weighs 0, which
  // is also what ex2 makes of it
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int x = 0; x < X; ++x) {
      const int h = x >> 1;
      const float p = weight(s[nt][x], c, ref[h]);
      s[nt][x] = p;
      u[h] = __fadd_rn(u[h], p);
    }
#pragma unroll
  for (int h = 0; h < H; ++h) {
    u[h] = __fadd_rn(u[h], __shfl_xor_sync(0xffffffffu, u[h], 1));
    l_t[h] = __fadd_rn(u[h], __shfl_xor_sync(0xffffffffu, u[h], 2));
  }
}

// One tile for one warp: weights from the raw scores in s, then o_t = the tile's weighted values per row.
template <int D, bool kUpper = true>
__device__ __forceinline__ void tile_partial(float (*s)[4], float (*o_t)[4], float* m_t, float* l_t, int key0, const int* row_pos,
                                             const int* row_lo, float c, const bf16* sV, int lane, bool full = false) {
  tile_weights<kUpper>(s, m_t, l_t, key0, row_pos, row_lo, c, lane, full);
  pv_tile<D, kUpper>(o_t, s, sV, lane);
}

// Folds a part into a state, row by row of the thread's two rows; rows whose part is empty are left alone.
template <int D>
__device__ __forceinline__ void fold_rows(float* m, float* l, float (*o)[4], const float* m_t, const float* l_t, const float (*o_t)[4]) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (m_t[h] == -INFINITY) continue;
    const FoldFactors f = fold_factors(m[h], m_t[h]);
    l[h] = fold_value(l[h], l_t[h], f);
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      o[dt][2 * h] = fold_value(o[dt][2 * h], o_t[dt][2 * h], f);
      o[dt][2 * h + 1] = fold_value(o[dt][2 * h + 1], o_t[dt][2 * h + 1], f);
    }
    m[h] = f.m;
  }
}

// ------------------------------------------------------------------ decoded tokens
// Folds the records of chunks c0..c1 of one (entry, key/value head) for element (r, d) and returns the finished value.
// Folds the records of chunks c0..c1, in ascending order, into the state (m, l, o0, o1) of two elements of a row.
// load(c, ml, v) fetches chunk c's (maximum, sum) and its two values. The records of kFoldAhead chunks are requested
// while the kFoldAhead before them are folded, and a group's factors (which hang on the chain of maxima alone) are all
// computed before its sums: the operations and their order are those of one chunk after the other, but a long context
// no longer pays a round trip to L2 per chunk (131,072 keys, one request: the fold of 512 chunks by the entry's last
// CTA took 120 us with one record requested at a time, 63 with eight).
constexpr int kFoldAhead = 8;
// AHEAD false: a group is requested when the group before it has been folded (fewer registers: for kernels whose
// contexts are short or that have none to spare).
template <bool AHEAD = true, class Load>
__device__ __forceinline__ void fold_records(int c0, int c1, Load load, float& m, float& l, float& o0, float& o1) {
  float2 ml[kFoldAhead], v[kFoldAhead];
#pragma unroll
  for (int u = 0; u < kFoldAhead; ++u)
    if (c0 + u <= c1) load(c0 + u, ml[u], v[u]);
  for (int c = c0; c <= c1; c += kFoldAhead) {
    float2 ml_next[kFoldAhead], v_next[kFoldAhead];
    if (AHEAD) {
#pragma unroll
      for (int u = 0; u < kFoldAhead; ++u)
        if (c + kFoldAhead + u <= c1) load(c + kFoldAhead + u, ml_next[u], v_next[u]);
    }
    FoldFactors f[kFoldAhead];
    bool use[kFoldAhead];
#pragma unroll
    for (int u = 0; u < kFoldAhead; ++u) {
      use[u] = c + u <= c1 && ml[u].x != -INFINITY;     // a chunk in which the row sees no key leaves the state as it is
      f[u] = fold_factors(m, use[u] ? ml[u].x : 0.0f);
      if (use[u]) m = f[u].m;
    }
#pragma unroll
    for (int u = 0; u < kFoldAhead; ++u)
      if (use[u]) {
        l = fold_value(l, ml[u].y, f[u]);
        o0 = fold_value(o0, v[u].x, f[u]);
        o1 = fold_value(o1, v[u].y, f[u]);
      }
    if (AHEAD) {
#pragma unroll
      for (int u = 0; u < kFoldAhead; ++u) ml[u] = ml_next[u], v[u] = v_next[u];
    } else {
#pragma unroll
      for (int u = 0; u < kFoldAhead; ++u)
        if (c + kFoldAhead + u <= c1) load(c + kFoldAhead + u, ml[u], v[u]);
    }
  }
}

// The finished value of element (r, d) of one (entry, key/value head) from the records of its chunks c0..c1.
template <int D>
__device__ __forceinline__ float fold_chunks(const float* part_o, const float* part_ml, int64_t rec0, int c0, int c1, int r, int d) {
  float m = -INFINITY, l = 0.0f, o = 0.0f, unused = 0.0f;
  fold_records(c0, c1, [&](int c, float2& ml, float2& v) {
    ml = __ldcg(reinterpret_cast<const float2*>(&part_ml[((rec0 + c) * 16 + r) * 2]));
    v = make_float2(__ldcg(&part_o[(rec0 + c) * 16 * D + r * D + d]), 0.0f);
  }, m, l, o, unused);
  return finish(o, l);
}

// The same for elements (r, d) and (r, d + 1), d even: the row's factors are computed once.
template <int D, bool AHEAD = true>
__device__ __forceinline__ void fold_chunks2(const float* part_o, const float* part_ml, int64_t rec0, int c0, int c1, int r, int d,
                                             float& a, float& b) {
  float m = -INFINITY, l = 0.0f, o0 = 0.0f, o1 = 0.0f;
  fold_records<AHEAD>(c0, c1, [&](int c, float2& ml, float2& v) {
    ml = __ldcg(reinterpret_cast<const float2*>(&part_ml[((rec0 + c) * 16 + r) * 2]));
    v = __ldcg(reinterpret_cast<const float2*>(&part_o[(rec0 + c) * 16 * D + r * D + d]));
  }, m, l, o0, o1);
  a = finish(o0, l);
  b = finish(o1, l);
}

// Element j and j + D / 2 of one head of one token from the projection's partial sums, rotated by the position's
// angle j unless it is a value: the arithmetic of rope_append_kernel (elementwise.cu), operation by operation.
template <int D>
__device__ __forceinline__ void projected_pair(const AttnTcParams& p, int row, int head, int pos, int j, bool rotate, float& a, float& b) {
  const float* src = p.qkv + static_cast<int64_t>(row) * (p.Hq + 2 * p.Hkv) * D + static_cast<int64_t>(head) * D;
  // (read from L2: inside the decode chain the partial sums were written by other SMs during the same kernel; up to
  // kInFlight partial sums are requested at once, each being a round trip to L2, then added in ascending order)
  constexpr int kInFlight = 8;
  float pa[kInFlight], pb[kInFlight];
#pragma unroll
  for (int s = 0; s < kInFlight; ++s) {
    if (s < p.n_partials) {
      pa[s] = __ldcg(src + s * p.partial_stride + j);
      pb[s] = __ldcg(src + s * p.partial_stride + j + D / 2);
    }
  }
  a = pa[0];
  b = pb[0];
#pragma unroll
  for (int s = 1; s < kInFlight; ++s) {
    if (s < p.n_partials) {
      a += pa[s];
      b += pb[s];
    }
  }
  for (int s = kInFlight; s < p.n_partials; ++s) {
    a += __ldcg(src + s * p.partial_stride + j);
    b += __ldcg(src + s * p.partial_stride + j + D / 2);
  }
  if (rotate) {
    const float2 cs = *reinterpret_cast<const float2*>(p.cos_sin + (static_cast<int64_t>(pos) * (D / 2) + j) * 2);
    const float ra = __fsub_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y));
    const float rb = __fadd_rn(__fmul_rn(b, cs.x), __fmul_rn(a, cs.y));
    a = ra;
    b = rb;
  }
}

// FUSED: the step's queries, keys and values are taken from the projection's partial sums, rotated here, and the
// keys and values are appended to the cache by the CTA whose chunk holds their position (no rotation kernel runs).
// One unit of the decode kernel: (item, key/value head g, chunk), run by 128 threads (tid 0..127, four whole warps) that
// synchronise through env.sync(); Env::wait_inputs() returns once the step's own inputs (queries, or the projection's
// partial sums) may be read. smem_tiles: decode_unit_smem<D, FUSED>() bytes, 128-byte aligned; is_last_s: one int of
// shared memory. A caller that runs several units in a row synchronises between them.
template <int D, bool FUSED>
__host__ __device__ constexpr size_t decode_unit_smem() {
  return FUSED ? static_cast<size_t>(16 * (D + 8) + 8 * 64 * (D + 8)) * sizeof(bf16) : static_cast<size_t>(16 * (D + 8) + 4 * 64 * D) * sizeof(bf16);
}
// CLUSTER: the CTAs of an entry's chunks are one thread-block cluster (rank = chunk, at most 8): every CTA leaves its
// chunk's record in its own shared memory (cluster_record: decode_record_floats<D>() floats that nothing else uses), and
// the CTA of rank 0 folds them in ascending order through distributed shared memory: two cluster barriers instead of a
// record in global memory, a ticket and a second look at memory (3.2 us a layer for a decode step at the 1B sizes).
template <int D>
__host__ __device__ constexpr int decode_record_floats() { return 16 * (D + 2); }
template <int D, bool FUSED, bool CLUSTER, class Env>
__device__ __forceinline__ void decode_unit(const AttnTcParams& p, int item, int g, int chunk, uint8_t* smem_tiles, int* is_last_p, int tid, Env& env,
                                            float* cluster_record = nullptr) {
  constexpr int LD = D + 8, CH = D / 8;
  // FUSED: tiles [4 warps][K, V][64][D + 8]. Otherwise [4 warps][64][D], swizzled: a warp's values take the place of
  // its keys once the scores are out, which lets twice as many warps live on an SM; the values travel while the
  // weights are computed.
  constexpr bool SW = !FUSED;
  constexpr int kBufs = FUSED ? 2 : 1, kTile = SW ? 64 * D : 64 * LD;
  bf16* sKV = reinterpret_cast<bf16*>(smem_tiles);
  bf16* sQ = sKV + 4 * kBufs * kTile;                      // [16][LD]
  float* sO = reinterpret_cast<float*>(sKV);               // [4][16][D], over the key/value tiles once they are used up
  float* sML = sO + 4 * 16 * D;                           // [4][16][2]
  int& is_last_s = *is_last_p;
  const int warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tq = lane & 3;
  const int G = p.Hq / p.Hkv;
  const int e = p.work[item];
  const int slot = p.meta[e], first_row = p.meta[p.meta_stride + e], L = p.meta[2 * p.meta_stride + e],
            first_pos = p.meta[3 * p.meta_stride + e];
  const int pos_hi = first_pos + L - 1;
  const int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int rows = L * G;
  constexpr int PR = D / 2;
  const int d = (tid % PR) * 2;
  const int c0 = key_lo / kChunk, c1 = pos_hi / kChunk;
  // CLUSTER: once every CTA's record is in its shared memory, rank 0 folds the entry's chunks in ascending order (the
  // arithmetic of fold_chunks2) and writes the rows; the others stay until it has read them.
  auto cluster_fold = [&]() {
    sb::cluster_sync();
    if (chunk == 0) {
      for (int r = tid / PR; r < rows; r += 128 / PR) {
        float m = -INFINITY, l = 0.0f, o0 = 0.0f, o1 = 0.0f;
        fold_records<false>(c0, c1, [&](int c, float2& ml, float2& v) {
          ml = sb::cluster_load_float2(sb::cluster_peer_address(cluster_record + 16 * D + r * 2, c));
          v = sb::cluster_load_float2(sb::cluster_peer_address(cluster_record + r * D + d, c));
        }, m, l, o0, o1);
        const int pi = div_g(p, r);
        *reinterpret_cast<uint32_t*>(p.out + (static_cast<int64_t>(first_row + pi) * p.Hq + g * G + r - pi * G) * D + d) =
            pack_bf16(finish(o0, l), finish(o1, l));
      }
    }
    sb::cluster_sync();
  };
  if (chunk * kChunk > pos_hi || chunk * kChunk + kChunk - 1 < key_lo) {   // no key of this chunk is visible
    env.wait_inputs();
    if (CLUSTER) cluster_fold();
    return;
  }
  const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;
  const bf16* kplane = p.k_base + static_cast<int64_t>(g) * p.head_stride;

  bf16* sK = sKV + warp * kBufs * kTile;
  bf16* sV = sK + (kBufs - 1) * kTile;
  const int key0 = chunk * kChunk + warp * kKeys;
  const bool any = key0 <= pos_hi && key0 + kKeys - 1 >= key_lo;
  // Keys before this step's first position were written by earlier steps: their tiles are requested before
  // waiting for the kernels in front (which write this step's keys and the queries).
  if (any) load_kv_tiles<D, FUSED ? 3 : 1, SW>(sK, sV, kplane, p.v_offset, table, p.page_size, p.page_shift, p.page_stride, key0, key_lo,
                                           first_pos - 1, lane, 32, key_lo, pos_hi);
  env.wait_inputs();
  if (FUSED) {
    constexpr int half = D / 2;
    for (int idx = tid; idx < 16 * half; idx += 128) {
      const int r = idx / half, j = idx % half;
      float a = 0.0f, b = 0.0f;
      if (r < rows) projected_pair<D>(p, first_row + r / G, g * G + r % G, first_pos + r / G, j, true, a, b);
      sQ[r * LD + j] = __float2bfloat16_rn(a);
      sQ[r * LD + j + half] = __float2bfloat16_rn(b);
    }
    // the step's own keys and values that lie in this chunk: into the warps' tiles and into the cache
    const int lo = max(first_pos, chunk * kChunk), hi = min(pos_hi, chunk * kChunk + kChunk - 1);
    for (int idx = tid; idx < (hi - lo + 1) * D; idx += 128) {
      const int pos = lo + idx / D, jj = idx % D;
      const bool is_v = jj >= half;
      const int j = jj % half;
      float a, b;
      projected_pair<D>(p, first_row + pos - first_pos, p.Hq + (is_v ? p.Hkv : 0) + g, pos, j, !is_v, a, b);
      const bf16 ha = __float2bfloat16_rn(a), hb = __float2bfloat16_rn(b);
      bf16* tile = sKV + ((pos - chunk * kChunk) / kKeys) * 2 * 64 * LD + (is_v ? 64 * LD : 0) + (pos % kKeys) * LD;
      tile[j] = ha;
      tile[j + half] = hb;
      const int pi = p.page_shift >= 0 ? pos >> p.page_shift : pos / p.page_size;
      const int in_page = p.page_shift >= 0 ? pos & (p.page_size - 1) : pos % p.page_size;
      bf16* dst = const_cast<bf16*>(kplane) + static_cast<int64_t>(table[pi]) * p.page_stride + in_page * D + (is_v ? p.v_offset : 0);
      dst[j] = ha;
      dst[j + half] = hb;
    }
  } else {
    for (int idx = tid; idx < 16 * CH; idx += 128) {
      const int r = idx / CH, c = idx % CH;
      bf16* d = sQ + r * LD + c * 8;
      if (r < rows)
        cp_async16(smem_u32(d), p.q + (static_cast<int64_t>(first_row + div_g(p, r)) * p.Hq + g * G + r - div_g(p, r) * G) * D + c * 8);
      else
        *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
    if (any && key0 + kKeys - 1 >= first_pos)
      load_kv_tiles<D, 1, SW>(sK, sV, kplane, p.v_offset, table, p.page_size, p.page_shift, p.page_stride, key0, max(first_pos, key_lo),
                              pos_hi, lane, 32, key_lo, pos_hi);
  }
  cp_commit();
  cp_wait<0>();
  env.sync();

  // every warp computes the tile of its 64 keys
  float m_t[2] = {-INFINITY, -INFINITY}, l_t[2] = {0.0f, 0.0f};
  float o_t[D / 8][4];
  if (any) {
    int row_pos[2], row_lo[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = gid + 8 * h;
      row_pos[h] = r < rows ? first_pos + div_g(p, r) : -1;
      row_lo[h] = p.window > 0 ? row_pos[h] - p.window + 1 : 0;
    }
    float s[8][4];
    qk_tile<D, SW>(s, sQ, sK, lane);
    if (!FUSED) {
      __syncwarp();     // every lane has read the keys; the values take their place
      load_kv_tiles<D, 2, SW>(sK, sV, kplane, p.v_offset, table, p.page_size, p.page_shift, p.page_stride, key0, key_lo, pos_hi, lane, 32);
      cp_commit();
    }
    const bool full = key0 + kKeys - 1 <= first_pos && key0 >= (p.window > 0 ? pos_hi - p.window + 1 : 0);
    if (rows > 8) tile_weights<true>(s, m_t, l_t, key0, row_pos, row_lo, p.scale_log2, lane, full);
    else tile_weights<false>(s, m_t, l_t, key0, row_pos, row_lo, p.scale_log2, lane, full);
    if (!FUSED) {
      cp_wait<0>();
      __syncwarp();
    }
    if (rows > 8) pv_tile<D, true, SW>(o_t, s, sV, lane);
    else pv_tile<D, false, SW>(o_t, s, sV, lane);
  } else {
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
      for (int x = 0; x < 4; ++x) o_t[dt][x] = 0.0f;
  }
  env.sync();   // all warps are done with their key/value tiles, whose space the results take
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = gid + 8 * h;
    if (r >= rows) continue;     // only rows in use are folded below
    if (tq == 0) {
      sML[(warp * 16 + r) * 2] = m_t[h];
      sML[(warp * 16 + r) * 2 + 1] = l_t[h];
    }
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
      *reinterpret_cast<float2*>(&sO[(warp * 16 + r) * D + dt * 8 + tq * 2]) = make_float2(o_t[dt][2 * h], o_t[dt][2 * h + 1]);
  }
  env.sync();
  // the chunk's record: its tiles folded in key order into an empty state; a thread takes two neighbouring
  // elements of a row, which share the row's factors
  const int64_t rec = (static_cast<int64_t>(item) * p.Hkv + g) * p.chunks + chunk;
  // The entry's only chunk (at most 256 keys in view): its record is the row, so it is folded into the empty row state here,
  // with the operations the last CTA of several would use, and written; no record, no ticket, no second look at memory.
  const bool alone = !CLUSTER && p.counters != nullptr && c0 == c1;
  for (int r = tid / PR; r < rows; r += 128 / PR) {
    float m = -INFINITY, l = 0.0f, o0 = 0.0f, o1 = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float2 ml = *reinterpret_cast<const float2*>(&sML[(w * 16 + r) * 2]);
      if (ml.x == -INFINITY) continue;
      const FoldFactors f = fold_factors(m, ml.x);
      const float2 v = *reinterpret_cast<const float2*>(&sO[(w * 16 + r) * D + d]);
      l = fold_value(l, ml.y, f);
      o0 = fold_value(o0, v.x, f);
      o1 = fold_value(o1, v.y, f);
      m = f.m;
    }
    if (alone) {
      float lr = 0.0f, a = 0.0f, b = 0.0f;
      if (m != -INFINITY) {
        const FoldFactors f = fold_factors(-INFINITY, m);
        lr = fold_value(lr, l, f);
        a = fold_value(a, o0, f);
        b = fold_value(b, o1, f);
      }
      const int pi = div_g(p, r);
      *reinterpret_cast<uint32_t*>(p.out + (static_cast<int64_t>(first_row + pi) * p.Hq + g * G + r - pi * G) * D + d) =
          pack_bf16(finish(a, lr), finish(b, lr));
      continue;
    }
    if (CLUSTER) {
      *reinterpret_cast<float2*>(cluster_record + r * D + d) = make_float2(o0, o1);
      if (d == 0) *reinterpret_cast<float2*>(cluster_record + 16 * D + r * 2) = make_float2(m, l);
      continue;
    }
    *reinterpret_cast<float2*>(&p.part_o[rec * 16 * D + r * D + d]) = make_float2(o0, o1);
    if (d == 0) *reinterpret_cast<float2*>(&p.part_ml[(rec * 16 + r) * 2]) = make_float2(m, l);
  }
  if (CLUSTER) {
    cluster_fold();      // (also when this chunk is the entry's only one: the other CTAs of the cluster wait at its barriers)
    return;
  }
  if (p.counters == nullptr || alone) return;
  // The CTA that finishes an entry's last chunk folds all of them, in ascending order, and writes the rows.
  env.sync();
  if (tid == 0) {
    __threadfence();   // the CTA's records (made visible to this thread by the barrier) before the ticket
    int* counter = p.counters + item * p.Hkv + g;
    const int ticket = atomicAdd(counter, 1);
    is_last_s = ticket == c1 - c0;
    if (is_last_s) *counter = 0;
  }
  env.sync();
  if (!is_last_s) return;
  __threadfence();
  const int64_t rec0 = (static_cast<int64_t>(item) * p.Hkv + g) * p.chunks;
  for (int r = tid / PR; r < rows; r += 128 / PR) {
    float a, b;
    fold_chunks2<D, Env::kFoldAhead>(p.part_o, p.part_ml, rec0, c0, c1, r, d, a, b);
    const int pi = div_g(p, r);
    *reinterpret_cast<uint32_t*>(p.out + (static_cast<int64_t>(first_row + pi) * p.Hq + g * G + r - pi * G) * D + d) = pack_bf16(a, b);
  }
}

}  // namespace attn_tc
}  // namespace sb
