// Paged causal attention for any head size, head count and group ratio, in 32-bit
// arithmetic: the attention of the float32 path, and the fall-back of the bfloat16
// path for head sizes without a tensor-core kernel.
//
// One block per (token of the step, query head). The token's own key and value
// are already in the cache; it sees the keys first..pos, first = 0 or
// pos - window + 1. Keys are taken in tiles of 128 absolute positions
// [128c, 128c+128): each tile gives a partial (max, sum, weighted values) that is
// folded into the running result left to right. The tiles are cut by position,
// not by page, so the arithmetic of a query does not depend on the page size, on
// where its pages lie, or on what else is in the batch.
//
// Counterparts in arhaamatiq/stride: AttentionPage and AttentionCombine
// (src/kernel_common.h:90-253, 256-309), which cut by 64-token page.
#include <algorithm>

#include "common.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;
constexpr int kTile = 128;
constexpr int kMaxDimsPerThread = 4;  // head_dim <= 512

struct AttnParams {
  const void* q;
  void* out;
  const void* k_base;
  const int32_t* block_table;
  int max_pages;
  int page_size;
  int64_t page_stride, v_offset, head_stride;
  const int32_t* positions;
  const int32_t* slots;
  int Hq, Hkv, D;
  int window;
  float scale;
};

template <class TQ, class TKV, class TO>
__global__ void __launch_bounds__(kTile) attention_generic_kernel(AttnParams p) {
  extern __shared__ __align__(16) float smem[];
  float* qs = smem;                // [D]
  float* ps = qs + p.D;            // [kTile]
  __shared__ int64_t koff[kTile];  // element offset of each key row of the tile
  __shared__ float red[32];

  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int row = blockIdx.x, head = blockIdx.y, t = threadIdx.x;
  const int D = p.D;
  const int kvh = head / (p.Hq / p.Hkv);
  const int pos = p.positions[row];
  const int slot = p.slots[row];
  const int first = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const TQ* q = static_cast<const TQ*>(p.q) + static_cast<int64_t>(row) * p.Hq * D + static_cast<int64_t>(head) * D;
  for (int d = t; d < D; d += kTile) qs[d] = sb::widen(q[d]);
  __syncthreads();

  const TKV* kbase = static_cast<const TKV*>(p.k_base) + static_cast<int64_t>(kvh) * p.head_stride;
  const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;

  float m_run = -INFINITY, l_run = 0.0f;
  float acc_run[kMaxDimsPerThread];
#pragma unroll
  for (int i = 0; i < kMaxDimsPerThread; ++i) acc_run[i] = 0.0f;

  for (int c = first / kTile; c <= pos / kTile; ++c) {
    const int key = c * kTile + t;
    const bool valid = key >= first && key <= pos;
    float s = -INFINITY;
    if (valid) {
      const int page = table[key / p.page_size];
      const int64_t off = static_cast<int64_t>(page) * p.page_stride + static_cast<int64_t>(key % p.page_size) * D;
      koff[t] = off;
      const TKV* kr = kbase + off;
      float dot = 0.0f;
      for (int d = 0; d < D; ++d) dot = fmaf(qs[d], sb::widen(kr[d]), dot);
      s = dot * p.scale;
    }
    const float m_c = sb::block_max(s, red);
    const float e = valid ? expf(s - m_c) : 0.0f;
    ps[t] = e;
    const float l_c = sb::block_sum(e, red);  // includes the barriers that publish ps and koff
    const int lo = max(first, c * kTile) - c * kTile;
    const int hi = min(pos, c * kTile + kTile - 1) - c * kTile;
    const float m_new = fmaxf(m_run, m_c);
    const float fa = expf(m_run - m_new), fb = expf(m_c - m_new);
#pragma unroll
    for (int u = 0; u < kMaxDimsPerThread; ++u) {
      const int d = t + u * kTile;
      if (d < D) {
        float acc = 0.0f;
        for (int i = lo; i <= hi; ++i) acc = fmaf(ps[i], sb::widen(kbase[koff[i] + p.v_offset + d]), acc);
        acc_run[u] = acc_run[u] * fa + acc * fb;
      }
    }
    l_run = l_run * fa + l_c * fb;
    m_run = m_new;
    __syncthreads();  // ps and koff are rewritten by the next tile
  }
  TO* o = static_cast<TO*>(p.out) + static_cast<int64_t>(row) * p.Hq * D + static_cast<int64_t>(head) * D;
#pragma unroll
  for (int u = 0; u < kMaxDimsPerThread; ++u) {
    const int d = t + u * kTile;
    if (d < D) o[d] = sb::narrow<TO>(acc_run[u] / l_run);
  }
}

// Four consecutive values, widened; p is aligned to four elements.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u), __uint_as_float(raw.y << 16),
                     __uint_as_float(raw.y & 0xFFFF0000u));
}

__device__ __forceinline__ float cluster_load_float(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// One tile's partial folded into the running result; written once so that every kernel rounds it the same way.
__device__ __forceinline__ void fold_tile(float m_c, float l_c, const float (&acc_c)[kMaxDimsPerThread], float& m_run, float& l_run,
                                          float (&acc_run)[kMaxDimsPerThread]) {
  const float m_new = fmaxf(m_run, m_c);
  const float fa = expf(m_run - m_new), fb = expf(m_c - m_new);
#pragma unroll
  for (int u = 0; u < kMaxDimsPerThread; ++u) acc_run[u] = __fmaf_rn(acc_run[u], fa, __fmul_rn(acc_c[u], fb));
  l_run = __fmaf_rn(l_run, fa, __fmul_rn(l_c, fb));
  m_run = m_new;
}

constexpr int kEarlyValues = 16;  // value rows of a thread's key class that are requested together with the key

// The partial (max, sum, weighted values) of tile c for head sizes that are a multiple of four with rows aligned to
// four elements. The memory requests of a tile are issued many at a time instead of one after the other. A score is
// the same chain over the head's dimensions as in the kernel above, its key row read four values a request, eight
// requests in flight. The weighted values are summed by key class: with C = D / 4 column groups and G = 128 / C
// classes, thread (g, c) adds the keys g, g + G, g + 2G, ... of the tile in ascending order for its four columns, and
// the G classes are then added in ascending order. The classes are counted from the tile's start, an absolute
// position, so the order is a function of the query's position and the window alone. EARLY: the first value rows of
// the class are requested before the scores are computed (a block that is alone with its keys waits for every request
// it makes); the additions are the same. Thread t leaves with the sums of the dimensions t, t + 128, ...; the caller
// puts a barrier before the next tile.
template <class TKV, bool EARLY>
__device__ __forceinline__ void tile_partial(const AttnParams& p, const TKV* kbase, const int32_t* table, int c, int first, int pos, int t,
                                             const float* qs, float* ps, float* part, int64_t* koff, float* red, float& m_c, float& l_c,
                                             float (&acc_c)[kMaxDimsPerThread]) {
  const int D = p.D, C = D / 4, G = kTile / C;
  const int col = (t % C) * 4, cls = t / C;  // cls >= G: no part in the weighted values
  const int key = c * kTile + t;
  const bool valid = key >= first && key <= pos;
  const int lo = max(first, c * kTile) - c * kTile;
  const int hi = min(pos, c * kTile + kTile - 1) - c * kTile;
  const TKV* kr = kbase;
  if (valid) {
    const int page = table[key / p.page_size];
    const int64_t off = static_cast<int64_t>(page) * p.page_stride + static_cast<int64_t>(key % p.page_size) * D;
    koff[t] = off;
    kr = kbase + off;
  }
  const TKV* vbase = kbase + p.v_offset + col;
  float4 k0[8], early[EARLY ? kEarlyValues : 1];
  if (valid) {
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (4 * u < D) k0[u] = load4(kr + 4 * u);
  }
  if (EARLY) {
    __syncthreads();  // koff of the whole tile
    if (cls < G) {
#pragma unroll
      for (int u = 0; u < kEarlyValues; ++u) {
        const int i = cls + u * G;
        if (i >= lo && i <= hi) early[u] = load4(vbase + koff[i]);
      }
    }
  }
  float s = -INFINITY;
  if (valid) {
    float dot = 0.0f;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (4 * u < D) {
        const float4 qv = *reinterpret_cast<const float4*>(qs + 4 * u);
        dot = fmaf(qv.x, k0[u].x, dot), dot = fmaf(qv.y, k0[u].y, dot);
        dot = fmaf(qv.z, k0[u].z, dot), dot = fmaf(qv.w, k0[u].w, dot);
      }
    for (int d0 = 32; d0 < D; d0 += 32) {
      float4 kv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (d0 + 4 * u < D) kv[u] = load4(kr + d0 + 4 * u);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (d0 + 4 * u < D) {
          const float4 qv = *reinterpret_cast<const float4*>(qs + d0 + 4 * u);
          dot = fmaf(qv.x, kv[u].x, dot), dot = fmaf(qv.y, kv[u].y, dot);
          dot = fmaf(qv.z, kv[u].z, dot), dot = fmaf(qv.w, kv[u].w, dot);
        }
    }
    s = dot * p.scale;
  }
  m_c = sb::block_max(s, red);
  const float e = valid ? expf(s - m_c) : 0.0f;
  ps[t] = e;
  l_c = sb::block_sum(e, red);  // includes the barriers that publish ps and koff
  if (cls < G) {
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    int i0 = cls;
    if (EARLY) {
#pragma unroll
      for (int u = 0; u < kEarlyValues; ++u) {
        const int i = cls + u * G;
        if (i >= lo && i <= hi) {
          const float pr = ps[i];
          acc.x = fmaf(pr, early[u].x, acc.x), acc.y = fmaf(pr, early[u].y, acc.y);
          acc.z = fmaf(pr, early[u].z, acc.z), acc.w = fmaf(pr, early[u].w, acc.w);
        }
      }
      i0 += kEarlyValues * G;
    }
    for (; i0 < kTile; i0 += 8 * G) {
      float4 vv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * G;
        if (i >= lo && i <= hi) vv[u] = load4(vbase + koff[i]);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * G;
        if (i >= lo && i <= hi) {
          const float pr = ps[i];
          acc.x = fmaf(pr, vv[u].x, acc.x), acc.y = fmaf(pr, vv[u].y, acc.y);
          acc.z = fmaf(pr, vv[u].z, acc.z), acc.w = fmaf(pr, vv[u].w, acc.w);
        }
      }
    }
    *reinterpret_cast<float4*>(part + cls * D + col) = acc;
  }
  __syncthreads();
#pragma unroll
  for (int u = 0; u < kMaxDimsPerThread; ++u) {
    const int d = t + u * kTile;
    float acc = 0.0f;
    if (d < D) {
      acc = part[d];
      for (int g = 1; g < G; ++g) acc += part[g * D + d];
    }
    acc_c[u] = acc;
  }
}

// Shared memory of the kernel below, in floats: the query, a tile's weights, the classes' sums, and with a cluster
// the partials (D values, max, sum) of `slots` tiles.
__host__ __device__ constexpr int vec_smem_floats(int D, int slots) { return D + kTile + 4 * kTile + slots * (D + 2); }

// One block per (token of the step, query head), tiles left to right; or, CLUSTER, a cluster of gridDim.z blocks per
// (token, head): block r of it takes the tiles first, first + z, ... counted from r, keeps their partials in its shared
// memory, and block 0 folds all of them left to right out of the others' shared memory. The fold sees the same
// partials in the same order either way, so both give the same bits; the cluster shortens the path of a decoded token,
// whose tiles otherwise wait for one another.
template <class TQ, class TKV, class TO, bool CLUSTER>
__global__ void __launch_bounds__(kTile, CLUSTER ? 1 : 3) attention_generic_vec_kernel(AttnParams p, int slots) {
  extern __shared__ __align__(16) float smem[];
  float* qs = smem;                // [D]
  float* ps = qs + p.D;            // [kTile]
  float* part = ps + kTile;        // [G][D], G * D <= 4 * kTile
  float* rec = part + 4 * kTile;   // [slots][D + 2]
  __shared__ int64_t koff[kTile];  // element offset of each key row of the tile
  __shared__ float red[32];

  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int row = blockIdx.x, head = blockIdx.y, t = threadIdx.x;
  const int D = p.D;
  const int kvh = head / (p.Hq / p.Hkv);
  const int pos = p.positions[row];
  const int slot = p.slots[row];
  const int first = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const TQ* q = static_cast<const TQ*>(p.q) + static_cast<int64_t>(row) * p.Hq * D + static_cast<int64_t>(head) * D;
  for (int d = t; d < D; d += kTile) qs[d] = sb::widen(q[d]);
  __syncthreads();

  const TKV* kbase = static_cast<const TKV*>(p.k_base) + static_cast<int64_t>(kvh) * p.head_stride;
  const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;
  const int c_first = first / kTile, c_last = pos / kTile;

  float m_run = -INFINITY, l_run = 0.0f;
  float acc_run[kMaxDimsPerThread];
#pragma unroll
  for (int i = 0; i < kMaxDimsPerThread; ++i) acc_run[i] = 0.0f;

  if (!CLUSTER) {
    for (int c = c_first; c <= c_last; ++c) {
      float m_c, l_c, acc_c[kMaxDimsPerThread];
      tile_partial<TKV, false>(p, kbase, table, c, first, pos, t, qs, ps, part, koff, red, m_c, l_c, acc_c);
      fold_tile(m_c, l_c, acc_c, m_run, l_run, acc_run);
      __syncthreads();  // ps, koff and part are rewritten by the next tile
    }
  } else {
    const int rank = static_cast<int>(sb::cluster_rank()), size = static_cast<int>(gridDim.z);
    // more tiles than the cluster holds (the host sizes `slots` for the longest sequence; kept as a guard): block 0
    // computes those itself after the others', in order
    const int held = min(c_last - c_first + 1, slots * size);
    for (int j = rank; j < held; j += size) {
      float m_c, l_c, acc_c[kMaxDimsPerThread];
      tile_partial<TKV, true>(p, kbase, table, c_first + j, first, pos, t, qs, ps, part, koff, red, m_c, l_c, acc_c);
      float* r = rec + (j / size) * (D + 2);
#pragma unroll
      for (int u = 0; u < kMaxDimsPerThread; ++u)
        if (t + u * kTile < D) r[t + u * kTile] = acc_c[u];
      if (t == 0) r[D] = m_c, r[D + 1] = l_c;
      __syncthreads();
    }
    sb::cluster_sync();
    if (rank == 0) {
      for (int j0 = 0; j0 < held; j0 += 4) {
        float2 ml[4];
        float acc_c[4][kMaxDimsPerThread];
#pragma unroll
        for (int v = 0; v < 4; ++v)
          if (j0 + v < held) {
            const uint32_t r = sb::cluster_peer_address(rec + ((j0 + v) / size) * (D + 2), (j0 + v) % size);
            ml[v] = sb::cluster_load_float2(r + 4 * D);
#pragma unroll
            for (int u = 0; u < kMaxDimsPerThread; ++u) acc_c[v][u] = t + u * kTile < D ? cluster_load_float(r + 4 * (t + u * kTile)) : 0.0f;
          }
#pragma unroll
        for (int v = 0; v < 4; ++v)
          if (j0 + v < held) fold_tile(ml[v].x, ml[v].y, acc_c[v], m_run, l_run, acc_run);
      }
    }
    sb::cluster_sync();  // the others' shared memory has been read
    if (rank != 0) return;
    for (int c = c_first + held; c <= c_last; ++c) {
      float m_c, l_c, acc_c[kMaxDimsPerThread];
      tile_partial<TKV, false>(p, kbase, table, c, first, pos, t, qs, ps, part, koff, red, m_c, l_c, acc_c);
      fold_tile(m_c, l_c, acc_c, m_run, l_run, acc_run);
      __syncthreads();
    }
  }
  TO* o = static_cast<TO*>(p.out) + static_cast<int64_t>(row) * p.Hq * D + static_cast<int64_t>(head) * D;
#pragma unroll
  for (int u = 0; u < kMaxDimsPerThread; ++u) {
    const int d = t + u * kTile;
    if (d < D) o[d] = sb::narrow<TO>(acc_run[u] / l_run);
  }
}

}  // namespace

// dtype: 0 = float32 (q, cache and out), 1 = bfloat16 (q, cache and out).
SB_EXPORT int sb_attention_generic(const void* q, void* out, int dtype, const void* k_base,
                                   const int32_t* block_table, int max_pages, int page_size, int64_t page_stride,
                                   int64_t v_offset, int64_t head_stride, const int32_t* positions,
                                   const int32_t* slots, int n, int Hq, int Hkv, int D, int window, float scale,
                                   cudaStream_t stream) {
  if (n <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0) return sb::fail("sb_attention_generic: %d query heads do not divide into %d groups", Hq, Hkv);
  if (D <= 0 || D > kTile * kMaxDimsPerThread) return sb::fail("sb_attention_generic: head_dim %d not in 1..%d", D, kTile * kMaxDimsPerThread);
  if (Hq > 65535) return sb::fail("sb_attention_generic: too many heads");
  AttnParams p{q, out, k_base, block_table, max_pages, page_size, page_stride, v_offset, head_stride,
               positions, slots, Hq, Hkv, D, window, scale};
  dim3 grid(n, Hq);
  // rows of four aligned elements: requests of four values, many in flight (a function of the sizes and of where the
  // buffers lie, never of the batch)
  const int esz = dtype == 0 ? 4 : 2;
  const bool vec = D % 4 == 0 && page_stride % 4 == 0 && v_offset % 4 == 0 && head_stride % 4 == 0 &&
                   reinterpret_cast<uintptr_t>(k_base) % (4 * esz) == 0;
  if (vec) {
    // The tiles of the longest sequence (of the window, if there is one). Few blocks (decoded tokens): a cluster per
    // (token, head) takes its tiles side by side. Both kernels give the same bits, so the choice may depend on the batch.
    int64_t tiles = (static_cast<int64_t>(max_pages) * page_size + kTile - 1) / kTile;
    if (window > 0) tiles = std::min<int64_t>(tiles, (window - 1) / kTile + 2);
    const int size = static_cast<int>(std::min<int64_t>(8, tiles));
    const int slots = static_cast<int>((tiles + size - 1) / std::max(size, 1));
    const size_t smem_cluster = static_cast<size_t>(vec_smem_floats(D, slots)) * sizeof(float);
    const bool cluster = size >= 2 && static_cast<int64_t>(n) * Hq * size <= 4 * sb::sm_count() && smem_cluster <= 48 * 1024;
    if (cluster) {
      const dim3 cgrid(n, Hq, size), cdim(1, 1, size);
      if (dtype == 0) sb::launch_pdl_cluster(attention_generic_vec_kernel<float, float, float, true>, cgrid, dim3(kTile), smem_cluster, stream, cdim, p, slots);
      else if (dtype == 1) sb::launch_pdl_cluster(attention_generic_vec_kernel<bf16, bf16, bf16, true>, cgrid, dim3(kTile), smem_cluster, stream, cdim, p, slots);
      else return sb::fail("sb_attention_generic: unsupported dtype %d", dtype);
    } else {
      const size_t smem = static_cast<size_t>(vec_smem_floats(D, 0)) * sizeof(float);
      if (dtype == 0) sb::launch_pdl(attention_generic_vec_kernel<float, float, float, false>, grid, dim3(kTile), smem, stream, p, 0);
      else if (dtype == 1) sb::launch_pdl(attention_generic_vec_kernel<bf16, bf16, bf16, false>, grid, dim3(kTile), smem, stream, p, 0);
      else return sb::fail("sb_attention_generic: unsupported dtype %d", dtype);
    }
    return sb::check_launch("sb_attention_generic");
  }
  const size_t smem = static_cast<size_t>(D + kTile) * sizeof(float);
  if (dtype == 0) sb::launch_pdl(attention_generic_kernel<float, float, float>, grid, dim3(kTile), smem, stream, p);
  else if (dtype == 1) sb::launch_pdl(attention_generic_kernel<bf16, bf16, bf16>, grid, dim3(kTile), smem, stream, p);
  else return sb::fail("sb_attention_generic: unsupported dtype %d", dtype);
  return sb::check_launch("sb_attention_generic");
}

// ------------------------------------------------------------------ operation of the native step program (step_ops.h)
// i: 0 q, 1 out, 2 dtype, 3 cache layer, 4 block table, 5 pages per sequence, 6 page size, 7 page stride, 8 v offset,
//    9 head stride, 10 Hq, 11 Hkv, 12 D, 13 window; f: 0 scale
SB_EXPORT int sb_op_attention_generic(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  return sb_attention_generic(ptr<const void>(op->i[0]), ptr<void>(op->i[1]), (int)op->i[2], ptr<const void>(op->i[3]),
                              ptr<const int32_t>(op->i[4]), (int)op->i[5], (int)op->i[6], op->i[7], op->i[8], op->i[9], positions(s),
                              slots(s), s->n, (int)op->i[10], (int)op->i[11], (int)op->i[12], (int)op->i[13], static_cast<float>(op->f[0]),
                              static_cast<cudaStream_t>(stream));
}
