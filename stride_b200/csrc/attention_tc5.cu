// Paged causal attention for prompt portions on Blackwell's tcgen05 tensor cores (head size 64, bfloat16).
//
// One CTA per (tile of 128 query rows of an entry, key/value head). The query heads that share the key/value
// head are stacked as rows: row r is (position r / G, head r % G), G = Hq / Hkv, so a tile covers 128 / G
// positions. The CTA walks the key tiles [128 t, 128 t + 128) its rows can see:
//
//   control warp (one thread): TMA loads of the query tile (a 3-D box over [token][head][64]) and of the key
//     and value tiles, page by page through the block table, into 128-byte-swizzled shared memory (two
//     buffers); S = Q K^T by tcgen05.mma (M 128, N 128, K 64) into one of two TMEM accumulators, issued one
//     tile ahead so that it runs under the softmax of the tile before; O_t = P V by tcgen05.mma (M 128, N 64,
//     K 128, V as an MN-major operand straight from its [key][64] page layout).
//   four softmax warps (thread = row, TMEM lane = row): read S with tcgen05.ld, scale, mask by position, keep
//     the running maximum and sum in float32, write the weights to shared memory as two bfloat16 parts
//     (p = hi + lo, so the value product sees nearly 32-bit weights, as the reference's 32-bit softmax does),
//     then fold O_t into the row's float32 output registers: o = o * 2^(m_old - m_new) + O_t.
//
// Every mbarrier wait is bounded and reports through a status word. Key tiles past a request's last page are
// read from its last page instead (finite data, masked by position), so no unallocated page is touched.
// Counterpart in arhaamatiq/stride: AttentionPage / AttentionCombine (src/kernel_common.h:90-309), scalar.
#include "tc5.cuh"

SB_DEFINE_LAST_ERROR()

namespace {

using namespace sb::tc5;
using bf16 = __nv_bfloat16;

constexpr int kD = 64;
constexpr int kRows = 128;
constexpr int kKeys = 128;
constexpr int kTileBytes = 128 * 128;   // 128 rows of 64 bfloat16
constexpr int kThreads = 160;
constexpr float kLog2e = 1.4426950408889634f;
// shared memory: Q | K0 K1 | V0 V1 | P hi (two 64-key halves) | P lo
constexpr int kSmemBytes = 9 * kTileBytes;
constexpr uint32_t kTmemCols = 512;     // S0 [0,128) S1 [128,256) O_t [256,320)

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Fa5Params {
  bf16* out;
  const int32_t* block_table;
  int max_pages, page_size, page_shift;
  int rows_per_page, rows_v, rows_head;   // distances in rows of 64 elements inside the key/value map
  int box_rows;                            // rows one TMA box brings: min(page_size, 128)
  const int32_t* meta;
  int meta_stride;
  const int32_t* work;                     // [tiles][2] = (entry, tile in entry)
  int Hq, Hkv, window;
  float scale_log2;
  int* status;
};

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const Fa5Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full, kv_full[2], s_full[2], p_full, o_full;
  __shared__ uint32_t tmem_base_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem0 - smem_u32(smem_raw));
  const uint32_t sQ = smem0, sK = smem0 + kTileBytes, sV = smem0 + 3 * kTileBytes, sPhi = smem0 + 5 * kTileBytes,
                 sPlo = smem0 + 7 * kTileBytes;

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
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&kv_full[i]), 1);
      mbar_init(smem_u32(&s_full[i]), 1);
    }
    mbar_init(smem_u32(&p_full), 128);
    mbar_init(smem_u32(&o_full), 1);
    mbar_init_fence();
  }
  if (warp == 4) tmem_alloc(smem_u32(&tmem_base_s), kTmemCols);
  // rows of the query tile that no (position, head) pair fills (G does not divide 128) must still be finite
  for (int i = ppt * G * 8 + tid; i < kRows * 8; i += kThreads) *reinterpret_cast<uint4*>(smem + i * 16) = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  sb::grid_launch_dependents();
  sb::grid_dependency_wait();

  if (warp == 4) {
    if (lane == 0) {
      // ------------------------------------------------ control: TMA and MMA issue
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_kv);
      const int32_t* table = p.block_table + static_cast<int64_t>(slot) * p.max_pages;
      auto load_kv = [&](int i) {
        const int buf = i & 1;
        const uint32_t bar = smem_u32(&kv_full[buf]);
        mbar_expect_tx(bar, 2 * kTileBytes);
        for (int sub = 0; sub < kKeys / p.box_rows; ++sub) {
          const int key = (kt0 + i) * kKeys + sub * p.box_rows;
          const int key_c = min(key, pos_hi);                 // past the end: the request's last page again
          const int page = table[key_c >> p.page_shift];
          const int in_page = p.page_size > p.box_rows ? (key & (p.page_size - 1)) : 0;
          const int row = page * p.rows_per_page + g * p.rows_head + in_page;
          tma_load_2d(sK + buf * kTileBytes + sub * p.box_rows * 128, &map_kv, bar, 0, row);
          tma_load_2d(sV + buf * kTileBytes + sub * p.box_rows * 128, &map_kv, bar, 0, row + p.rows_v);
        }
      };
      auto issue_qk = [&](int i) {
        const uint32_t idesc = instr_desc(kRows, kKeys, false);
        const uint64_t da = smem_desc_sw128(sQ), db = smem_desc_sw128(sK + (i & 1) * kTileBytes);
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) umma_bf16(tmem_base + (i & 1) * kKeys, da + 2 * k, db + 2 * k, idesc, k > 0 ? 1u : 0u);
        umma_commit(smem_u32(&s_full[i & 1]));
      };
      mbar_expect_tx(smem_u32(&q_full), ppt * G * 128);
      tma_load_3d(sQ, &map_q, smem_u32(&q_full), 0, g * G, row0);
      load_kv(0);
      if (T > 1) load_kv(1);
      mbar_wait(smem_u32(&q_full), 0, p.status, 1);
      mbar_wait(smem_u32(&kv_full[0]), 0, p.status, 2);
      fence_after_sync();
      issue_qk(0);
      const uint32_t idesc_pv = instr_desc(kRows, kD, true);
      for (int i = 0; i < T; ++i) {
        if (i + 1 < T) {
          mbar_wait(smem_u32(&kv_full[(i + 1) & 1]), ((i + 1) >> 1) & 1, p.status, 2);
          fence_after_sync();
          issue_qk(i + 1);
        }
        mbar_wait(smem_u32(&p_full), i & 1, p.status, 3);
        fence_after_sync();
        const uint32_t v = sV + (i & 1) * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < kKeys / 16; ++ks) {
          const uint32_t off = (ks >> 2) * kTileBytes;     // which 64-key half of P
          const uint64_t db = smem_desc_sw128(v + ks * 2048);
          umma_bf16(tmem_base + 2 * kKeys, smem_desc_sw128(sPhi + off) + 2 * (ks & 3), db, idesc_pv, ks > 0 ? 1u : 0u);
          umma_bf16(tmem_base + 2 * kKeys, smem_desc_sw128(sPlo + off) + 2 * (ks & 3), db, idesc_pv, 1u);
        }
        umma_commit(smem_u32(&o_full));
        mbar_wait(smem_u32(&o_full), i & 1, p.status, 4);     // then this tile's key/value buffers are free
        if (i + 2 < T) load_kv(i + 2);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------ softmax: thread = row of the tile = TMEM lane
    const int r = tid;
    const int pi = r / G, hh = r % G;
    const bool valid = pi < npos;
    const int row_pos = valid ? pos0 + pi : -1;
    const int row_lo = p.window > 0 ? row_pos - p.window + 1 : 0;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float m = -INFINITY, l = 0.0f;
    float o[kD];
#pragma unroll
    for (int d = 0; d < kD; ++d) o[d] = 0.0f;
    for (int i = 0; i < T; ++i) {
      mbar_wait(smem_u32(&s_full[i & 1]), (i >> 1) & 1, p.status, 5);
      fence_after_sync();
      const uint32_t s_addr = tmem_base + (i & 1) * kKeys + lane_addr;
      const int key0 = (kt0 + i) * kKeys;
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        float v[32];
        tmem_load32(s_addr + c * 32, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int key = key0 + c * 32 + j;
          if (key <= row_pos && key >= row_lo) mx = fmaxf(mx, v[j] * p.scale_log2);
        }
      }
      const float m_new = fmaxf(m, mx);
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;
      const float alpha = fast_exp2(m - m_use);
      l *= alpha;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        float v[32];
        tmem_load32(s_addr + c * 32, v);
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float pj[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int key = key0 + c * 32 + j + u;
            pj[u] = (key <= row_pos && key >= row_lo) ? fast_exp2(v[j + u] * p.scale_log2 - m_use) : 0.0f;
            l += pj[u];
          }
          const __nv_bfloat162 h = __floats2bfloat162_rn(pj[0], pj[1]);
          const __nv_bfloat162 w = __floats2bfloat162_rn(pj[0] - __low2float(h), pj[1] - __high2float(h));
          hi[j >> 1] = *reinterpret_cast<const uint32_t*>(&h);
          lo[j >> 1] = *reinterpret_cast<const uint32_t*>(&w);
        }
        // 32 keys = four 16-byte pieces of this row in the 64-key half c / 2, at pieces (c % 2) * 4 .. + 3
        const uint32_t row_off = (c >> 1) * kTileBytes + r * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t piece = (((c & 1) * 4 + q) ^ (r & 7)) * 16;
          *reinterpret_cast<uint4*>(smem + 5 * kTileBytes + row_off + piece) = make_uint4(hi[4 * q], hi[4 * q + 1], hi[4 * q + 2], hi[4 * q + 3]);
          *reinterpret_cast<uint4*>(smem + 7 * kTileBytes + row_off + piece) = make_uint4(lo[4 * q], lo[4 * q + 1], lo[4 * q + 2], lo[4 * q + 3]);
        }
      }
      fence_before_sync();
      fence_async_smem();
      mbar_arrive(smem_u32(&p_full));
      mbar_wait(smem_u32(&o_full), i & 1, p.status, 6);
      fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float v[32];
        tmem_load32(tmem_base + 2 * kKeys + lane_addr + c * 32, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) o[c * 32 + j] = o[c * 32 + j] * alpha + v[j];
      }
      m = m_new;
      fence_before_sync();
    }
    if (valid) {
      const float inv = 1.0f / l;
      bf16* dst = p.out + (static_cast<int64_t>(row0 + pi) * p.Hq + g * G + hh) * kD;
#pragma unroll
      for (int c = 0; c < kD / 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(o[c * 8 + 2 * j] * inv, o[c * 8 + 2 * j + 1] * inv);
          w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

// 1 if sb_attention_tc5 takes this shape (head size 64, at most 128 query heads per key/value head, pages of a
// power of two of at least 8 tokens), else 0.
SB_EXPORT int sb_attention_tc5_supported(int Hq, int Hkv, int D, int page_size) {
  if (D != kD || Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > kRows) return 0;
  if (page_size < 8 || (page_size & (page_size - 1)) != 0) return 0;
  return 1;
}

// Attention of prompt portions. q, out: [n_tokens][Hq * 64] bfloat16. k_base: this layer's keys of page 0 inside an
// arena of `pages` pages; strides in elements. work: [n_tiles][2] = (entry, tile), a tile being 128 / (Hq / Hkv)
// consecutive positions of the entry. meta as for sb_attention_tc.
SB_EXPORT int sb_attention_tc5(const void* q, void* out, const void* k_base, int pages, const int32_t* block_table,
                               int max_pages, int page_size, int64_t page_stride, int64_t v_offset, int64_t head_stride,
                               const int32_t* meta, int meta_stride, const int32_t* work, int n_tiles, int n_tokens, int Hq,
                               int Hkv, int D, int window, float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!sb_attention_tc5_supported(Hq, Hkv, D, page_size)) return sb::fail("sb_attention_tc5: shape not supported (Hq %d Hkv %d D %d page %d)", Hq, Hkv, D, page_size);
  if ((page_stride | v_offset | head_stride) % kD != 0 || ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_base) | reinterpret_cast<uintptr_t>(out)) & 15))
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
  p.rows_per_page = static_cast<int>(page_stride / kD);
  p.rows_v = static_cast<int>(v_offset / kD);
  p.rows_head = static_cast<int>(head_stride / kD);
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
  const int64_t qdims[3] = {kD, Hq, n_tokens}, qstrides[3] = {1, kD, static_cast<int64_t>(Hq) * kD};
  const int qbox[3] = {kD, G, ppt};
  const int64_t kv_rows = static_cast<int64_t>(pages - 1) * p.rows_per_page + p.rows_v + static_cast<int64_t>(Hkv) * p.rows_head;
  const int64_t kdims[2] = {kD, kv_rows}, kstrides[2] = {1, kD};
  const int kbox[2] = {kD, p.box_rows};
  if (!tensor_map_bf16(q, 3, qdims, qstrides, qbox, &map_q) || !tensor_map_bf16(k_base, 2, kdims, kstrides, kbox, &map_kv))
    return sb::fail("sb_attention_tc5: cuTensorMapEncodeTiled failed");
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes + 1024) != cudaSuccess)
      return sb::fail("sb_attention_tc5: cannot raise the shared memory limit");
    attr_set = true;
  }
  sb::launch_pdl(attn_prefill_tc5_kernel, dim3(n_tiles, Hkv), dim3(kThreads), static_cast<size_t>(kSmemBytes + 1024), stream, map_q, map_kv, p);
  return sb::check_launch("sb_attention_tc5");
}

// Reads and clears the status word: 0 = every wait completed. Synchronises the device.
SB_EXPORT int sb_attention_tc5_status() {
  int* status = status_word();
  if (!status) return -1;
  int host = 0;
  if (cudaMemcpy(&host, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (host != 0) cudaMemset(status, 0, sizeof(int));
  return host;
}
