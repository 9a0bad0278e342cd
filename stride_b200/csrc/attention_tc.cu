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
//   rows can see, with the usual running maximum and sum, and writes the finished rows.
// * attn_decode_kernel: entries whose rows fit one 16-row tile (a decoded token, or a very
//   short portion). One CTA per (entry, key/value head, chunk of 256 absolute key
//   positions); each of its 4 warps takes 64 of the keys, the four results are merged in
//   warp order, and the chunk's (max, sum, weighted values) go to scratch memory.
//   attn_combine_kernel then folds an entry's chunks in ascending order and writes bfloat16.
//   Chunks are cut by absolute position, never by page or by batch, so a token's arithmetic
//   is the same whatever else the step holds.
//
// Keys and values come from the paged cache through the request's block table
// ([pages][2][Hkv][page_size][D] per layer); a key tile may span several pages.
// Counterparts in arhaamatiq/stride: AttentionPage / AttentionCombine with KvT = bfloat16
// (src/kernel_common.h:90-309), which are scalar.
#include "common.cuh"
#include "noalloc.h"

SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;

constexpr int kKeys = 64;        // keys per tile
constexpr int kChunk = 256;      // keys per decode chunk (4 warps x 64)
constexpr float kLog2e = 1.4426950408889634f;

// 2^x by the hardware's approximation (two units in the last place); exp2f adds a slow path for subnormals.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

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
  int window;
  float scale_log2;      // softmax scale * log2(e)
  // decode only
  float* part_o;         // [items][Hkv][chunks][16][D]
  float* part_ml;        // [items][Hkv][chunks][16][2]
  int chunks;
  int* counters;         // [items][Hkv], zero between launches; null: the chunks are folded by attn_combine_kernel
};

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
template <int D>
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
  for (int i = tid / CH; i < kKeys; i += threads / CH) {
    const int key = key0 + i;
    bf16* dk = dstK + i * LD + c * 8;
    bf16* dv = dstV + i * LD + c * 8;
    if (key >= key_lo && key <= key_hi) {
      const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
      const int in_page = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
      const bf16* src = kplane + static_cast<int64_t>(table[pi]) * page_stride + in_page * D + c * 8;
      cp_async16(smem_u32(dk), src);
      cp_async16(smem_u32(dv), src + v_offset);
    } else if (key < zero_lo || key > zero_hi) {
      *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(dv) = make_uint4(0, 0, 0, 0);
    }
  }
}

// S[16 x 64] = Q[16 x D] K^T for one warp; q fragments in registers, K tile in shared memory.
template <int D>
__device__ __forceinline__ void qk_tile(float (*s)[4], const uint32_t (*qf)[4], const bf16* sK, int lane) {
  constexpr int LD = D + 8;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
  const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int nt = 0; nt < 8; nt += 2) {
      uint32_t b[4];
      ldsm_x4(b, smem_u32(sK + (nt * 8 + (mi >> 1) * 8 + rr) * LD + ks * 16 + (mi & 1) * 8));
      mma_16816(s[nt], qf[ks], b[0], b[1]);
      mma_16816(s[nt + 1], qf[ks], b[2], b[3]);
    }
  }
}

// O[16 x D] += P[16 x 64] V[64 x D]; P given as the float accumulators of qk_tile after exponentiation.
// The softmax weights stay (nearly) 32-bit: each is split into a bfloat16 head and a bfloat16 remainder,
// p = hi + lo with |p - hi - lo| <= 2^-17 p, and both parts are multiplied with V. With the head alone the
// weights would carry a rounding of 2^-9 that the 32-bit softmax of the reference does not have.
template <int D>
__device__ __forceinline__ void pv_tile(float (*o)[4], const float (*s)[4], const bf16* sV, int lane) {
  constexpr int LD = D + 8;
  const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const float p0 = s[2 * kk + (x >> 1)][(x & 1) * 2], p1 = s[2 * kk + (x >> 1)][(x & 1) * 2 + 1];
      const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
      hi[x] = *reinterpret_cast<const uint32_t*>(&h);
      lo[x] = pack_bf16(p0 - __low2float(h), p1 - __high2float(h));
    }
#pragma unroll
    for (int dt = 0; dt < D / 8; dt += 2) {
      uint32_t b[4];
      ldsm_x4_trans(b, smem_u32(sV + (kk * 16 + (mi & 1) * 8 + rr) * LD + (dt + (mi >> 1)) * 8));
      mma_16816(o[dt], hi, b[0], b[1]);
      mma_16816(o[dt], lo, b[0], b[1]);
      mma_16816(o[dt + 1], hi, b[2], b[3]);
      mma_16816(o[dt + 1], lo, b[2], b[3]);
    }
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
    const int pi = r / G, hh = r % G;
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
    const int pi = r / G;
    row_pos[h] = pi < npos ? pos0 + pi : -1;
    row_lo[h] = p.window > 0 ? row_pos[h] - p.window + 1 : 0;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float o[D / 8][4];
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
    for (int x = 0; x < 4; ++x) o[dt][x] = 0.0f;
  uint32_t qf[D / 16][4];

  for (int kt = kt0; kt <= kt1; ++kt) {
    const int buf = (kt - kt0) & 1;
    cp_wait<0>();
    __syncthreads();
    if (kt == kt0) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        ldsm_x4(qf[ks], smem_u32(sQ + (warp * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8));
    }
    if (kt < kt1) {
      load_kv_tiles<D>(sK + (buf ^ 1) * 64 * LD, sV + (buf ^ 1) * 64 * LD, kplane, p.v_offset, table, p.page_size, p.page_shift,
                       p.page_stride, (kt + 1) * kKeys, key_lo, pos_hi, tid, 128);
      cp_commit();
    }
    float s[8][4];
    qk_tile<D>(s, qf, sK + buf * 64 * LD, lane);
    // scale, mask, running softmax (base 2)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int h = x >> 1;
        const int key = kt * kKeys + nt * 8 + tq * 2 + (x & 1);
        const bool ok = key <= row_pos[h] && key >= row_lo[h];
        s[nt][x] = ok ? s[nt][x] * p.scale_log2 : -INFINITY;
        mx[h] = fmaxf(mx[h], s[nt][x]);
      }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.0f : m_new;
      alpha[h] = fast_exp2(m[h] - m_use[h]);
      m[h] = m_new;
      l[h] *= alpha[h];
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float e2 = fast_exp2(s[nt][x] - m_use[x >> 1]);
        s[nt][x] = e2;
        l[x >> 1] += e2;
      }
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      o[dt][0] *= alpha[0];
      o[dt][1] *= alpha[0];
      o[dt][2] *= alpha[1];
      o[dt][3] *= alpha[1];
    }
    pv_tile<D>(o, s, sV + buf * 64 * LD, lane);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    const int r = warp * 16 + gid + 8 * h;
    const int pi = r / G, hh = r % G;
    if (pi < npos) {
      const float inv = 1.0f / l[h];
      bf16* dst = p.out + (static_cast<int64_t>(row0 + pi) * p.Hq + g * G + hh) * D;
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt)
        *reinterpret_cast<uint32_t*>(dst + dt * 8 + tq * 2) = pack_bf16(o[dt][2 * h] * inv, o[dt][2 * h + 1] * inv);
    }
  }
}

// ------------------------------------------------------------------ decoded tokens
template <int D>
__global__ void __launch_bounds__(128) attn_decode_kernel(const AttnTcParams p) {
  constexpr int LD = D + 8, CH = D / 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);           // [16][LD]
  bf16* sKV = sQ + 16 * LD;                               // [4 warps][K, V][64][LD]
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

  bf16* sK = sKV + warp * 2 * 64 * LD;
  bf16* sV = sK + 64 * LD;
  const int key0 = chunk * kChunk + warp * kKeys;
  const bool any = key0 <= pos_hi && key0 + kKeys - 1 >= key_lo;
  // Keys before this step's first position were written by earlier steps: their tiles are requested before
  // waiting for the kernels in front (which write this step's keys and the queries).
  if (any) load_kv_tiles<D>(sK, sV, kplane, p.v_offset, table, p.page_size, p.page_shift, p.page_stride, key0, key_lo, first_pos - 1,
                            lane, 32, key_lo, pos_hi);
  sb::grid_dependency_wait();
  for (int idx = tid; idx < 16 * CH; idx += 128) {
    const int r = idx / CH, c = idx % CH;
    bf16* d = sQ + r * LD + c * 8;
    if (r < rows)
      cp_async16(smem_u32(d), p.q + (static_cast<int64_t>(first_row + r / G) * p.Hq + g * G + r % G) * D + c * 8);
    else
      *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
  }
  if (any && key0 + kKeys - 1 >= first_pos)
    load_kv_tiles<D>(sK, sV, kplane, p.v_offset, table, p.page_size, p.page_shift, p.page_stride, key0, max(first_pos, key_lo), pos_hi,
                     lane, 32, key_lo, pos_hi);
  cp_commit();
  cp_wait<0>();
  __syncthreads();

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float o[D / 8][4];
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
    for (int x = 0; x < 4; ++x) o[dt][x] = 0.0f;
  if (any) {
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldsm_x4(qf[ks], smem_u32(sQ + (lane & 15) * LD + ks * 16 + (lane >> 4) * 8));
    int row_pos[2], row_lo[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = gid + 8 * h;
      row_pos[h] = r < rows ? first_pos + r / G : -1;
      row_lo[h] = p.window > 0 ? row_pos[h] - p.window + 1 : 0;
    }
    float s[8][4];
    qk_tile<D>(s, qf, sK, lane);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int h = x >> 1;
        const int key = key0 + nt * 8 + tq * 2 + (x & 1);
        const bool ok = key <= row_pos[h] && key >= row_lo[h];
        s[nt][x] = ok ? s[nt][x] * p.scale_log2 : -INFINITY;
        m[h] = fmaxf(m[h], s[nt][x]);
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m[h] = fmaxf(m[h], __shfl_xor_sync(0xffffffffu, m[h], 1));
      m[h] = fmaxf(m[h], __shfl_xor_sync(0xffffffffu, m[h], 2));
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float mu = m[x >> 1] == -INFINITY ? 0.0f : m[x >> 1];
        const float e2 = fast_exp2(s[nt][x] - mu);
        s[nt][x] = e2;
        l[x >> 1] += e2;
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    pv_tile<D>(o, s, sV, lane);
  }
  // every warp leaves (m, l, O) of its 64 keys; they are merged in warp order
  __syncthreads();   // all warps are done with their key/value tiles, whose space the results take
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = gid + 8 * h;
    if (tq == 0) {
      sML[(warp * 16 + r) * 2] = m[h];
      sML[(warp * 16 + r) * 2 + 1] = l[h];
    }
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      sO[(warp * 16 + r) * D + dt * 8 + tq * 2] = o[dt][2 * h];
      sO[(warp * 16 + r) * D + dt * 8 + tq * 2 + 1] = o[dt][2 * h + 1];
    }
  }
  __syncthreads();
  const int64_t rec = (static_cast<int64_t>(item) * p.Hkv + g) * p.chunks + chunk;
  for (int idx = tid; idx < rows * D; idx += 128) {
    const int r = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sML[(w * 16 + r) * 2]);
    const float mu = mm == -INFINITY ? 0.0f : mm;
    float acc = 0.0f, ll = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = fast_exp2(sML[(w * 16 + r) * 2] - mu);
      acc += sO[(w * 16 + r) * D + d] * f;
      ll += sML[(w * 16 + r) * 2 + 1] * f;
    }
    p.part_o[rec * 16 * D + idx] = acc;
    if (d == 0) {
      p.part_ml[(rec * 16 + r) * 2] = mm;
      p.part_ml[(rec * 16 + r) * 2 + 1] = ll;
    }
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
  for (int idx = tid; idx < rows * D; idx += 128) {
    const int r = idx / D, d = idx % D;
    float mm = -INFINITY;
    for (int c = c0; c <= c1; ++c) mm = fmaxf(mm, __ldcg(&p.part_ml[((rec0 + c) * 16 + r) * 2]));
    float acc = 0.0f, ll = 0.0f;
    for (int c = c0; c <= c1; ++c) {
      const float f = fast_exp2(__ldcg(&p.part_ml[((rec0 + c) * 16 + r) * 2]) - mm);
      acc += __ldcg(&p.part_o[(rec0 + c) * 16 * D + r * D + d]) * f;
      ll += __ldcg(&p.part_ml[((rec0 + c) * 16 + r) * 2 + 1]) * f;
    }
    p.out[(static_cast<int64_t>(first_row + r / G) * p.Hq + g * G + r % G) * D + d] = __float2bfloat16_rn(acc / ll);
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
  for (int r = 0; r < L * G; ++r) {
    float mm = -INFINITY;
    for (int c = c0; c <= c1; ++c) mm = fmaxf(mm, p.part_ml[((rec0 + c) * 16 + r) * 2]);
    float acc = 0.0f, ll = 0.0f;
    for (int c = c0; c <= c1; ++c) {
      const float f = fast_exp2(p.part_ml[((rec0 + c) * 16 + r) * 2] - mm);
      acc += p.part_o[(rec0 + c) * 16 * D + r * D + d] * f;
      ll += p.part_ml[((rec0 + c) * 16 + r) * 2 + 1] * f;
    }
    p.out[(static_cast<int64_t>(first_row + r / G) * p.Hq + g * G + r % G) * D + d] = __float2bfloat16_rn(acc / ll);
  }
}

template <int D>
int launch(const AttnTcParams& p, int n_tiles, int n_items, cudaStream_t stream) {
  constexpr int LD = D + 8;
  if (n_tiles > 0) {
    const size_t smem = static_cast<size_t>(5) * 64 * LD * sizeof(bf16);
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(attn_chunk_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return sb::fail("sb_attention_tc: cannot raise the shared memory limit");
      set = true;
    }
    sb::launch_pdl(attn_chunk_kernel<D>, dim3(n_tiles, p.Hkv), dim3(128), smem, stream, p);
  }
  if (n_items > 0) {
    const size_t smem = static_cast<size_t>(16 * LD + 8 * 64 * LD) * sizeof(bf16);   // results (4 x 16 x (D + 2) floats) reuse the tiles
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(attn_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return sb::fail("sb_attention_tc: cannot raise the shared memory limit");
      set = true;
    }
    AttnTcParams pd = p;
    pd.work = p.work + 2 * n_tiles;
    sb::launch_pdl(attn_decode_kernel<D>, dim3(n_items, p.Hkv, p.chunks), dim3(128), smem, stream, pd);
    if (pd.counters == nullptr) sb::launch_pdl(attn_combine_kernel<D>, dim3(n_items, p.Hkv), dim3(D), 0, stream, pd);
  }
  return sb::check_launch("sb_attention_tc");
}

}  // namespace

// Floats of scratch that `sb_attention_tc` needs for `items` short entries and `chunks` key chunks.
SB_EXPORT int64_t sb_attention_tc_scratch(int items, int Hkv, int chunks, int D) {
  return static_cast<int64_t>(items) * Hkv * chunks * 16 * (D + 2);
}

// work: [n_tiles][2] (entry, tile) for the portion kernel, followed by [n_items] entries for the decode
// kernel. An entry belongs to the decode kernel iff length * (Hq / Hkv) <= 16. chunks = greatest
// (last position of a decode entry) / 256 + 1. scratch: sb_attention_tc_scratch(...) floats.
SB_EXPORT int sb_attention_tc(const void* q, void* out, const void* k_base, const int32_t* block_table, int max_pages,
                              int page_size, int64_t page_stride, int64_t v_offset, int64_t head_stride,
                              const int32_t* meta, int meta_stride, const int32_t* work, int n_tiles, int n_items,
                              int chunks, float* scratch, int* counters, int Hq, int Hkv, int D, int window, float scale,
                              cudaStream_t stream) {
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
  p.window = window;
  p.scale_log2 = scale * kLog2e;
  p.chunks = chunks;
  p.part_o = scratch;
  p.part_ml = scratch + static_cast<int64_t>(n_items) * Hkv * chunks * 16 * D;
  p.counters = counters;
  if (D == 64) return launch<64>(p, n_tiles, n_items, stream);
  if (D == 128) return launch<128>(p, n_tiles, n_items, stream);
  return sb::fail("sb_attention_tc: head_dim %d has no tensor-core kernel (64 or 128)", D);
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
