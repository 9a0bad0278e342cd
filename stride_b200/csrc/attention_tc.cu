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
#include "attention_math.cuh"
#include "common.cuh"
#include "step_ops.h"
#include "noalloc.h"


SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;

using namespace sb::attn;
constexpr int kKeys = kTileKeys;    // keys per tile
constexpr int kChunk = kChunkKeys;  // keys per chunk (4 tiles; the decode kernel gives each warp one)
#ifndef SB_DECODE_CTAS64
#define SB_DECODE_CTAS64 6
#endif
constexpr int kDecodeCtas64 = SB_DECODE_CTAS64;   // CTAs of the decode kernel per SM at head size 64 (bounds its registers)

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
// Folds the records of chunks c0..c1 of one (entry, key/value head) for element (r, d) and returns the finished value.
template <int D>
__device__ __forceinline__ float fold_chunks(const float* part_o, const float* part_ml, int64_t rec0, int c0, int c1, int r, int d) {
  float m = -INFINITY, l = 0.0f, o = 0.0f;
  for (int c = c0; c <= c1; ++c) {
    const float m_c = __ldcg(&part_ml[((rec0 + c) * 16 + r) * 2]);
    if (m_c == -INFINITY) continue;
    const FoldFactors f = fold_factors(m, m_c);
    l = fold_value(l, __ldcg(&part_ml[((rec0 + c) * 16 + r) * 2 + 1]), f);
    o = fold_value(o, __ldcg(&part_o[(rec0 + c) * 16 * D + r * D + d]), f);
    m = f.m;
  }
  return finish(o, l);
}

// The same for elements (r, d) and (r, d + 1), d even: the row's factors are computed once.
template <int D>
__device__ __forceinline__ void fold_chunks2(const float* part_o, const float* part_ml, int64_t rec0, int c0, int c1, int r, int d,
                                             float& a, float& b) {
  float m = -INFINITY, l = 0.0f, o0 = 0.0f, o1 = 0.0f;
  for (int c = c0; c <= c1; ++c) {
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(&part_ml[((rec0 + c) * 16 + r) * 2]));
    if (ml.x == -INFINITY) continue;
    const FoldFactors f = fold_factors(m, ml.x);
    const float2 v = __ldcg(reinterpret_cast<const float2*>(&part_o[(rec0 + c) * 16 * D + r * D + d]));
    l = fold_value(l, ml.y, f);
    o0 = fold_value(o0, v.x, f);
    o1 = fold_value(o1, v.y, f);
    m = f.m;
  }
  a = finish(o0, l);
  b = finish(o1, l);
}

// Element j and j + D / 2 of one head of one token from the projection's partial sums, rotated by the position's
// angle j unless it is a value: the arithmetic of rope_append_kernel (elementwise.cu), operation by operation.
template <int D>
__device__ __forceinline__ void projected_pair(const AttnTcParams& p, int row, int head, int pos, int j, bool rotate, float& a, float& b) {
  const float* src = p.qkv + static_cast<int64_t>(row) * (p.Hq + 2 * p.Hkv) * D + static_cast<int64_t>(head) * D;
  a = src[j];
  b = src[j + D / 2];
  for (int s = 1; s < p.n_partials; ++s) {
    a += src[s * p.partial_stride + j];
    b += src[s * p.partial_stride + j + D / 2];
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
template <int D, bool FUSED>
__global__ void __launch_bounds__(128, FUSED ? 3 : (D == 64 ? kDecodeCtas64 : 3)) attn_decode_kernel(const AttnTcParams p) {
  constexpr int LD = D + 8, CH = D / 8;
  // FUSED: tiles [4 warps][K, V][64][D + 8]. Otherwise [4 warps][64][D], swizzled: a warp's values take the place of
  // its keys once the scores are out, which lets twice as many warps live on an SM; the values travel while the
  // weights are computed.
  constexpr bool SW = !FUSED;
  constexpr int kBufs = FUSED ? 2 : 1, kTile = SW ? 64 * D : 64 * LD;
  extern __shared__ __align__(128) uint8_t smem_tiles[];
  bf16* sKV = reinterpret_cast<bf16*>(smem_tiles);
  bf16* sQ = sKV + 4 * kBufs * kTile;                      // [16][LD]
  float* sO = reinterpret_cast<float*>(sKV);               // [4][16][D], over the key/value tiles once they are used up
  float* sML = sO + 4 * 16 * D;                           // [4][16][2]
  __shared__ int is_last_s;

  sb::grid_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tq = lane & 3;
  const int item = blockIdx.x, g = blockIdx.y, chunk = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int e = p.work[item];
  const int slot = p.meta[e], first_row = p.meta[p.meta_stride + e], L = p.meta[2 * p.meta_stride + e],
            first_pos = p.meta[3 * p.meta_stride + e];
  const int pos_hi = first_pos + L - 1;
  const int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  if (chunk * kChunk > pos_hi || chunk * kChunk + kChunk - 1 < key_lo) {   // no key of this chunk is visible
    sb::grid_dependency_wait();
    return;
  }
  const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;
  const bf16* kplane = p.k_base + static_cast<int64_t>(g) * p.head_stride;
  const int rows = L * G;

  bf16* sK = sKV + warp * kBufs * kTile;
  bf16* sV = sK + (kBufs - 1) * kTile;
  const int key0 = chunk * kChunk + warp * kKeys;
  const bool any = key0 <= pos_hi && key0 + kKeys - 1 >= key_lo;
  // Keys before this step's first position were written by earlier steps: their tiles are requested before
  // waiting for the kernels in front (which write this step's keys and the queries).
  if (any) load_kv_tiles<D, FUSED ? 3 : 1, SW>(sK, sV, kplane, p.v_offset, table, p.page_size, p.page_shift, p.page_stride, key0, key_lo,
                                           first_pos - 1, lane, 32, key_lo, pos_hi);
  sb::grid_dependency_wait();
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
  __syncthreads();

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
  __syncthreads();   // all warps are done with their key/value tiles, whose space the results take
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
  __syncthreads();
  // the chunk's record: its tiles folded in key order into an empty state; a thread takes two neighbouring
  // elements of a row, which share the row's factors
  const int64_t rec = (static_cast<int64_t>(item) * p.Hkv + g) * p.chunks + chunk;
  constexpr int PR = D / 2;
  const int d = (tid % PR) * 2;
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
    *reinterpret_cast<float2*>(&p.part_o[rec * 16 * D + r * D + d]) = make_float2(o0, o1);
    if (d == 0) *reinterpret_cast<float2*>(&p.part_ml[(rec * 16 + r) * 2]) = make_float2(m, l);
  }
  if (p.counters == nullptr) return;
  // The CTA that finishes an entry's last chunk folds all of them, in ascending order, and writes the rows.
  const int c0 = key_lo / kChunk, c1 = pos_hi / kChunk;
  __syncthreads();
  if (tid == 0) {
    __threadfence();   // the CTA's records (made visible to this thread by the barrier) before the ticket
    int* counter = p.counters + item * p.Hkv + g;
    const int ticket = atomicAdd(counter, 1);
    is_last_s = ticket == c1 - c0;
    if (is_last_s) *counter = 0;
  }
  __syncthreads();
  if (!is_last_s) return;
  __threadfence();
  const int64_t rec0 = (static_cast<int64_t>(item) * p.Hkv + g) * p.chunks;
  for (int r = tid / PR; r < rows; r += 128 / PR) {
    float a, b;
    fold_chunks2<D>(p.part_o, p.part_ml, rec0, c0, c1, r, d, a, b);
    const int pi = div_g(p, r);
    *reinterpret_cast<uint32_t*>(p.out + (static_cast<int64_t>(first_row + pi) * p.Hq + g * G + r - pi * G) * D + d) = pack_bf16(a, b);
  }
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
      if (cudaFuncSetAttribute(attn_decode_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
          cudaFuncSetAttribute(attn_decode_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_fused) != cudaSuccess)
        return sb::fail("sb_attention_tc: cannot raise the shared memory limit");
      once.done();
    }
    AttnTcParams pd = p;
    pd.work = p.work + 2 * n_tiles;
    if (p.qkv != nullptr) sb::launch_pdl(attn_decode_kernel<D, true>, dim3(n_items, p.Hkv, p.chunks), dim3(128), smem_fused, stream, pd);
    else sb::launch_pdl(attn_decode_kernel<D, false>, dim3(n_items, p.Hkv, p.chunks), dim3(128), smem, stream, pd);
    if (pd.counters == nullptr) sb::launch_pdl(attn_combine_kernel<D>, dim3(n_items, p.Hkv), dim3(D), 0, stream, pd);
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
