// Linear layers of the bfloat16 path on the 5th-generation tensor cores (sm_100a):
// D[m, n] = sum_k W[m, k] * X[n, k], W [M, K] and X [N, K] bfloat16 with K contiguous,
// float32 accumulation in tensor memory.
//
// One CTA computes a tile of 128 weight rows (the M operand of tcgen05.mma, one TMEM
// lane per row) by BN tokens (the N operand, one TMEM column per token), BN in
// {16, 32, 64, 128, 256}, over a range of K. Warp 0 streams 128 x 64 and BN x 64 element
// tiles into 128-byte-swizzled shared memory with TMA (cp.async.bulk.tensor, no
// multicast) through a ring of stages guarded by mbarriers; one thread of warp 1 issues
// tcgen05.mma (four K = 16 steps per stage) and tcgen05.commit; warps 2-5 read the
// accumulator with tcgen05.ld and apply the epilogue:
//   kStore   out[n, m]  = d            (with split-K: one partial buffer per K range)
//   kAdd     out[n, m] += d            (the residual add)
//   kSwiglu  out[n, j]  = silu(g) * u  (bfloat16; the tile holds 64 gate rows and their
//                                      64 up rows, exchanged through shared memory)
// The K ranges of a weight depend on its shape alone (sb_gemm_tc_splits), never on the number of
// tokens: every range is accumulated from zero in tensor memory and the ranges' sums are added in
// float32 in ascending order, by the consumer of the partial buffers (up to 128 tokens: one CTA per
// range, so that a few tokens still occupy the GPU) or inside gemm_tc_fold_kernel (more tokens: a
// CTA walks a tile's ranges through two accumulators while eight epilogue warps add them up in
// registers). A token's result therefore has the same bits whatever the size of its batch.
// Rows or columns of a tile that lie outside the
// matrix are zero-filled by TMA and masked in the epilogue, so M, N and K need not be
// multiples of the tile (K must be a multiple of 8: TMA strides are multiples of 16 bytes).
//
// Every wait on an mbarrier is bounded: after about a second it records an error code in
// `status` (device memory owned by this library) and goes on, so the kernel always ends
// and frees its tensor memory; the host reads the status after the launch it cares about.
//
// Counterparts in arhaamatiq/stride: TcQkv, TcGemmResidual, TcMlp13, TcLmFull on wmma
// (src/kernels_tc.cu:347-655).
#include "gemm_tc_tile.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using namespace sb::tc5;
using namespace sb::gemm_tile;

constexpr int kMaxStages = 8;
constexpr int kThreads = 192;
constexpr int kSmemBudget = 200 * 1024;

// Where a thread stands in the ring of stages: the stage and the parity of its current use, kept by counting (a
// division per K step costs the issuing thread more than the products it issues). A producer starts with parity 1: a
// wait on that parity of a barrier nobody has arrived on yet returns at once, so its first round through the ring is free.
struct RingPos {
  uint32_t slot, par;
  const uint32_t stages;
  __device__ __forceinline__ RingPos(int stages_, uint32_t par0) : slot(0), par(par0), stages(static_cast<uint32_t>(stages_)) {}
  __device__ __forceinline__ void advance() {
    if (++slot == stages) slot = 0, par ^= 1;
  }
};
// The shared-memory descriptor of a tile `offset` bytes (a multiple of 16) into the stage at `slot`.
__device__ __forceinline__ uint64_t stage_desc(uint64_t desc_fixed, uint32_t smem0, uint32_t slot, uint32_t stage_bytes, uint32_t offset) {
  return desc_fixed | (((smem0 + offset) & 0x3FFFF) >> 4) + slot * (stage_bytes >> 4);
}

struct GemmParams {
  float* out;           // kStore / kAdd: float32 [N, ldo]; kSwiglu: bfloat16 [N, ldo]
  int64_t ldo;
  int64_t split_stride;  // elements between split-K partial buffers
  int M, N, K;
  int block_n;           // BN
  int stages;
  int kblocks_per_split;
  int tiles_m, tiles_n, splits;
  int half_rows;         // kSwiglu: rows of the gate half (intermediate size); W is [2 * half_rows, K]
  int* status;
};

// One tile per CTA: the lean form used when every tile has a CTA of its own (every decode-sized launch).
// blockIdx = (weight tile, token tile, K range).
template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_single_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BN = p.block_n;
  const int stage_b = BN * 128;
  const int stage_bytes = kStageA + stage_b;
  // Dynamic shared memory is only guaranteed 16-byte alignment: round up to the swizzle's 1024.
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int tile_m = blockIdx.x, tile_n = blockIdx.y, split = blockIdx.z;
  const int kblocks = (p.K + kTileK - 1) / kTileK;
  const int kb0 = split * p.kblocks_per_split;
  const int kb1 = min(kblocks, kb0 + p.kblocks_per_split);
  const int iters = kb1 - kb0;
  const uint32_t tmem_cols = tmem_alloc_cols(BN);

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&accum_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_s), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  sb::grid_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer: TMA loads. The weights do not depend on the kernels before this one,
      // so the first ring of weight tiles is requested before waiting for them to finish; the tokens'
      // tiles follow once their producer is done.
      const int row_w = EPI == kSwiglu ? tile_m * 64 : tile_m * kTileM;
      auto load_w = [&](int i) {
        const int s = i % p.stages;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t a = smem0 + s * stage_bytes;
        mbar_expect_tx(bar, stage_bytes);
        const int k = (kb0 + i) * kTileK;
        if (EPI == kSwiglu) {
          tma_load_2d(a, &map_w, bar, k, row_w);
          tma_load_2d(a + kStageA / 2, &map_w, bar, k, p.half_rows + row_w);
        } else {
          tma_load_2d(a, &map_w, bar, k, row_w);
        }
      };
      auto load_x = [&](int i) {
        const int s = i % p.stages;
        tma_load_2d(smem0 + s * stage_bytes + kStageA, &map_x, smem_u32(&full_bar[s]), (kb0 + i) * kTileK, tile_n * BN);
      };
      const int ahead = min(iters, p.stages);
      for (int i = 0; i < ahead; ++i) load_w(i);
      sb::grid_dependency_wait();
      for (int i = 0; i < ahead; ++i) load_x(i);
      // (the stage and its parity are counted, not divided out: with so few tokens a K step is bounded by the
      // instructions of the threads that issue it)
      int st = ahead == p.stages ? 0 : ahead;
      uint32_t par = 0;
      for (int i = ahead; i < iters; ++i) {
        mbar_wait(smem_u32(&empty_bar[st]), par, p.status, 1);
        const uint32_t bar = smem_u32(&full_bar[st]);
        const uint32_t a = smem0 + st * stage_bytes;
        const int k = (kb0 + i) * kTileK;
        mbar_expect_tx(bar, stage_bytes);
        tma_load_2d(a, &map_w, bar, k, row_w);
        if (EPI == kSwiglu) tma_load_2d(a + kStageA / 2, &map_w, bar, k, p.half_rows + row_w);
        tma_load_2d(a + kStageA, &map_x, bar, k, tile_n * BN);
        if (++st == p.stages) st = 0, par ^= 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer
      const uint32_t idesc = instr_desc(BN);
      const uint64_t desc_fixed = smem_desc_sw128(0);
      const uint32_t a_lo = (smem0 & 0x3FFFF) >> 4, stage_lo = static_cast<uint32_t>(stage_bytes) >> 4;
      const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
      uint32_t st = 0, par = 0, accumulate = 0;
      for (int i = 0; i < iters; ++i) {
        mbar_wait(full0 + 8 * st, par, p.status, 2);
        tc_fence_after();
        const uint64_t da = desc_fixed | (a_lo + st * stage_lo), db = da + (kStageA >> 4);
        // 16 elements = 32 bytes along K: +2 in the descriptor's 16-byte address units
        umma_bf16(tmem_base, da, db, idesc, accumulate);
        umma_bf16(tmem_base, da + 2, db + 2, idesc, 1u);
        umma_bf16(tmem_base, da + 4, db + 4, idesc, 1u);
        umma_bf16(tmem_base, da + 6, db + 6, idesc, 1u);
        accumulate = 1u;
        umma_commit(empty0 + 8 * st);
        if (++st == static_cast<uint32_t>(p.stages)) st = 0, par ^= 1;
      }
      umma_commit(smem_u32(&accum_bar));
    }
    __syncwarp();
  } else {
    // ---------------- epilogue: warps 2..5 own TMEM lanes 32 * (warp % 4) ..
    const int quarter = warp & 3;
    sb::grid_dependency_wait();
    const bool ok = iters > 0 && mbar_wait(smem_u32(&accum_bar), 0, p.status, 3);
    tc_fence_after();
    const int n0 = tile_n * BN;
    if (EPI == kSwiglu) {
      float* xch = reinterpret_cast<float*>(smem_raw + ((smem0 - smem_u32(smem_raw))));  // stage 0 is free by now
      swiglu_tile(tmem_base, xch, reinterpret_cast<bf16*>(p.out), p.ldo, tile_m, p.half_rows, n0, p.N, BN, quarter, lane, ok);
    } else {
      store_tile<EPI>(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16), p.out + static_cast<int64_t>(split) * p.split_stride,
                      tile_m * kTileM + quarter * 32 + lane, p.M, n0, p.N, p.ldo, BN, ok);
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

template <int EPI, bool MULTI>   // MULTI: a CTA may walk several tiles (two accumulators); else exactly one
__global__ void __launch_bounds__(kThreads)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t accum_full[2];
  __shared__ __align__(8) uint64_t accum_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ float xch[EPI == kSwiglu ? 16 * 64 : 1];   // gate/up exchange of the SwiGLU epilogue

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BN = p.block_n;
  const int stage_bytes = kStageA + BN * 128;
  // Dynamic shared memory is only guaranteed 16-byte alignment: round up to the swizzle's 1024.
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int kblocks = (p.K + kTileK - 1) / kTileK;
  // Tiles are numbered with the weight tile fastest, so CTAs that run together share token tiles in L2.
  const int total_tiles = p.tiles_m * p.tiles_n * p.splits;
  const uint32_t tmem_cols = tmem_alloc_cols((MULTI ? 2 : 1) * BN);   // MULTI: one accumulator fills while the other drains

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&accum_full[a]), 1);
      mbar_init(smem_u32(&accum_empty[a]), 4);   // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_s), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  sb::grid_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer: TMA loads. The weights do not depend on the kernels before this one,
      // so the first ring of weight tiles is requested before waiting for them to finish; the tokens'
      // tiles follow once their producer is done.
      RingPos pos(p.stages, 1);     // over the K blocks of all tiles of this CTA
      bool waited = false;
      for (int tile = blockIdx.x; tile < total_tiles; tile += MULTI ? gridDim.x : total_tiles) {
        const int tile_m = tile % p.tiles_m, rest = tile / p.tiles_m;
        const int tile_n = rest % p.tiles_n, split = rest / p.tiles_n;
        const int kb0 = split * p.kblocks_per_split;
        const int iters = min(kblocks, kb0 + p.kblocks_per_split) - kb0;
        const int row_w = EPI == kSwiglu ? tile_m * 64 : tile_m * kTileM;
        auto load_w = [&](int i, int slot) {
          const uint32_t bar = smem_u32(&full_bar[slot]);
          const uint32_t a = smem0 + slot * stage_bytes;
          mbar_expect_tx(bar, stage_bytes);
          const int k = (kb0 + i) * kTileK;
          if (EPI == kSwiglu) {
            tma_load_2d(a, &map_w, bar, k, row_w);
            tma_load_2d(a + kStageA / 2, &map_w, bar, k, p.half_rows + row_w);
          } else {
            tma_load_2d(a, &map_w, bar, k, row_w);
          }
        };
        auto load_x = [&](int i, int slot) {
          tma_load_2d(smem0 + slot * stage_bytes + kStageA, &map_x, smem_u32(&full_bar[slot]), (kb0 + i) * kTileK, tile_n * BN);
        };
        int i = 0;
        if (!waited) {
          const int ahead = min(iters, p.stages);
          for (int j = 0; j < ahead; ++j) load_w(j, j);
          sb::grid_dependency_wait();
          waited = true;
          for (int j = 0; j < ahead; ++j) load_x(j, j), pos.advance();
          i = ahead;
        }
        for (; i < iters; ++i) {
          mbar_wait(smem_u32(&empty_bar[pos.slot]), pos.par, p.status, 1);
          load_w(i, pos.slot);
          load_x(i, pos.slot);
          pos.advance();
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer
      const uint32_t idesc = instr_desc(BN);
      const uint64_t desc_fixed = smem_desc_sw128(0);
      RingPos pos(p.stages, 0);
      int ti = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += MULTI ? gridDim.x : total_tiles, ++ti) {
        const int split = tile / (p.tiles_m * p.tiles_n);
        const int kb0 = split * p.kblocks_per_split;
        const int iters = min(kblocks, kb0 + p.kblocks_per_split) - kb0;
        const int acc = ti & 1;
        // the epilogue must have drained this accumulator (tile ti - 2) before it is overwritten
        if (MULTI && ti >= 2) mbar_wait(smem_u32(&accum_empty[acc]), ((ti >> 1) - 1) & 1, p.status, 4);
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int i = 0; i < iters; ++i) {
          mbar_wait(smem_u32(&full_bar[pos.slot]), pos.par, p.status, 2);
          tc_fence_after();
          const uint64_t da = stage_desc(desc_fixed, smem0, pos.slot, stage_bytes, 0), db = stage_desc(desc_fixed, smem0, pos.slot, stage_bytes, kStageA);
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k) {
            // 16 elements = 32 bytes along K: +2 in the descriptor's 16-byte address units
            umma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[pos.slot]));
          pos.advance();
        }
        umma_commit(smem_u32(&accum_full[acc]));
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue: warps 2..5 own TMEM lanes 32 * (warp % 4) ..
    const int quarter = warp & 3;
    sb::grid_dependency_wait();
    int ti = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += MULTI ? gridDim.x : total_tiles, ++ti) {
      const int tile_m = tile % p.tiles_m, rest = tile / p.tiles_m;
      const int tile_n = rest % p.tiles_n, split = rest / p.tiles_n;
      const int acc = ti & 1;
      const bool ok = mbar_wait(smem_u32(&accum_full[acc]), (ti >> 1) & 1, p.status, 3);
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const int n0 = tile_n * BN;
      if (EPI == kSwiglu) {
        // lanes 0..63 hold gate rows, lanes 64..127 the matching up rows
        const int j = tile_m * 64 + (quarter & 1) * 32 + lane;  // output feature
        bf16* out = reinterpret_cast<bf16*>(p.out);
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float v[16];
          tmem_load16(tmem_d + c0, v);
          // gate warps hand over columns 8..15, up warps columns 0..7: every warp then finishes eight columns
          if (quarter >= 2) {
  #pragma unroll
            for (int c = 0; c < 8; ++c) xch[c * 64 + (quarter - 2) * 32 + lane] = v[c];
          } else {
  #pragma unroll
            for (int c = 0; c < 8; ++c) xch[(8 + c) * 64 + quarter * 32 + lane] = v[8 + c];
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (ok && j < p.half_rows) {
            const int cb = quarter >= 2 ? 8 : 0;
  #pragma unroll
            for (int c = 0; c < 8; ++c) {
              const int n = n0 + c0 + cb + c;
              if (n < p.N) {
                const float other = xch[(cb + c) * 64 + (quarter & 1) * 32 + lane];
                const float g = quarter >= 2 ? other : v[c], u = quarter >= 2 ? v[8 + c] : other;
                out[static_cast<int64_t>(n) * p.ldo + j] = __float2bfloat16_rn(silu_fast(g) * u);
              }
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      } else {
        store_tile<EPI>(tmem_d, p.out + static_cast<int64_t>(split) * p.split_stride, tile_m * kTileM + quarter * 32 + lane,
                        p.M, n0, p.N, p.ldo, BN, ok);
      }
      // this warp has read its part of the accumulator: let the MMA issuer reuse it
      if (MULTI) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&accum_empty[acc])) : "memory");
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// Many tokens and a weight that is cut into K ranges: persistent CTAs, each walking tiles of 128 weight rows by
// BN tokens; a tile's ranges go through the two accumulators in turn (each range accumulated from zero, as a CTA of
// the single-tile kernel does it), and eight epilogue warps (a lane quarter and a half of the columns each) add the
// ranges in ascending order in registers and store the sum (a residual add is left to the consumer, as with few
// tokens: reading the old values here would stall the epilogue on their latency).
constexpr int kFoldThreads = 64 + 256;
constexpr int kFoldCols = 128;            // columns per epilogue thread: BN / 2 <= 128

__global__ void __launch_bounds__(kFoldThreads, 1)
gemm_tc_fold_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t accum_full[2];
  __shared__ __align__(8) uint64_t accum_empty[2];
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BN = p.block_n;
  const int stage_bytes = kStageA + BN * 128;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int kblocks = (p.K + kTileK - 1) / kTileK;
  const int total_tiles = p.tiles_m * p.tiles_n;
  const uint32_t tmem_cols = tmem_alloc_cols(2 * BN);

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&accum_full[a]), 1);
      mbar_init(smem_u32(&accum_empty[a]), 8);   // one arrival per epilogue warp
    }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_s), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  sb::grid_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer: the K blocks of a tile in ascending order (its ranges are consecutive)
      sb::grid_dependency_wait();
      RingPos pos(p.stages, 1);
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const int tile_m = tile % p.tiles_m, tile_n = tile / p.tiles_m;
        for (int i = 0; i < kblocks; ++i) {
          mbar_wait(smem_u32(&empty_bar[pos.slot]), pos.par, p.status, 1);
          const uint32_t bar = smem_u32(&full_bar[pos.slot]);
          const uint32_t a = smem0 + pos.slot * stage_bytes;
          mbar_expect_tx(bar, stage_bytes);
          tma_load_2d(a, &map_w, bar, i * kTileK, tile_m * kTileM);
          tma_load_2d(a + kStageA, &map_x, bar, i * kTileK, tile_n * BN);
          pos.advance();
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer: range q of this CTA (counted over all its tiles) fills accumulator q & 1
      const uint32_t idesc = instr_desc(BN);
      const uint64_t desc_fixed = smem_desc_sw128(0);
      RingPos pos(p.stages, 0);
      int q = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        for (int r = 0; r < p.splits; ++r, ++q) {
          const int kb0 = r * p.kblocks_per_split;
          const int iters = min(kblocks, kb0 + p.kblocks_per_split) - kb0;
          const int acc = q & 1;
          if (q >= 2) mbar_wait(smem_u32(&accum_empty[acc]), ((q >> 1) - 1) & 1, p.status, 4);
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + acc * BN;
          for (int i = 0; i < iters; ++i) {
            mbar_wait(smem_u32(&full_bar[pos.slot]), pos.par, p.status, 2);
            tc_fence_after();
            const uint64_t da = stage_desc(desc_fixed, smem0, pos.slot, stage_bytes, 0), db = stage_desc(desc_fixed, smem0, pos.slot, stage_bytes, kStageA);
#pragma unroll
            for (int k = 0; k < kTileK / 16; ++k) umma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
            umma_commit(smem_u32(&empty_bar[pos.slot]));
            pos.advance();
          }
          umma_commit(smem_u32(&accum_full[acc]));
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue: warps 2..9; warp w reads TMEM lanes 32 * (w % 4) .. and columns [half * BN / 2, ..)
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int cols = BN / 2;
    sb::grid_dependency_wait();
    int q = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int tile_m = tile % p.tiles_m, tile_n = tile / p.tiles_m;
      const int m = tile_m * kTileM + quarter * 32 + lane;
      const int n0 = tile_n * BN + half * cols;
      const bool live = m < p.M;
      float* o = p.out + static_cast<int64_t>(n0) * p.ldo + m;
      float run[kFoldCols];
#pragma unroll 1
      for (int r = 0; r < p.splits; ++r, ++q) {
        const int acc = q & 1;
        mbar_wait(smem_u32(&accum_full[acc]), (q >> 1) & 1, p.status, 3);
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN + half * cols + (static_cast<uint32_t>(quarter * 32) << 16);
        if (r == 0) {
#pragma unroll
          for (int c0 = 0; c0 < kFoldCols; c0 += 16)
            if (c0 < cols) tmem_load16(tmem_d + c0, run + c0);
        } else {
#pragma unroll
          for (int c0 = 0; c0 < kFoldCols; c0 += 16) {
            if (c0 < cols) {
              float v[16];
              tmem_load16(tmem_d + c0, v);
#pragma unroll
              for (int c = 0; c < 16; ++c) run[c0 + c] += v[c];
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&accum_empty[acc]));
      }
      if (live) {
#pragma unroll
        for (int c = 0; c < kFoldCols; ++c)
          if (c < cols && n0 + c < p.N) o[static_cast<int64_t>(c) * p.ldo] = run[c];
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// Many tokens on a pair of CTAs (cta_group::2): a tile of 256 weight rows (kStore) or of 128 gate and 128 up rows
// (kSwiglu) by BN tokens. Each CTA of the pair loads its half of the weight rows and its half of the tokens, so
// that a K step of 64 brings 16 KB + BN * 64 bytes a CTA instead of 16 KB + BN * 128: it is the traffic from L2
// to the SMs that bounds these products. The leader issues the MMAs for both; each CTA's tensor memory holds its
// 128 rows of the tile and each CTA runs the epilogue for them: the K ranges added in ascending order in registers
// (kStore, eight epilogue warps as in gemm_tc_fold_kernel) or the SwiGLU product (four warps). A token's result has
// the bits of the single-CTA kernels: the same accumulation chain per element and the same order of the ranges.
template <int EPI>
__global__ void __launch_bounds__(kFoldThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
  constexpr int kEpiWarps = 8;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];    // used in the leader: both CTAs' tiles have landed
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];   // in each CTA: the MMAs that read its stage are done
  __shared__ __align__(8) uint64_t accum_full[2];           // in each CTA: an accumulator is complete
  __shared__ __align__(8) uint64_t accum_empty[2];          // used in the leader: both CTAs have drained an accumulator
  __shared__ uint32_t tmem_base_s;
  __shared__ float xch2[EPI == kSwiglu ? 2 : 1][EPI == kSwiglu ? 16 * 64 : 1];   // gate/up exchange of the SwiGLU epilogue, per warp set

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(sb::cluster_rank());
  const int BN = p.block_n, half_n = BN / 2;
  const int stage_bytes = kStageA + half_n * 128;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int kblocks = (p.K + kTileK - 1) / kTileK;
  const int total_tiles = p.tiles_m * p.tiles_n;            // tiles of the pair
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&accum_full[a]), 1);
      mbar_init(smem_u32(&accum_empty[a]), 2 * kEpiWarps);   // one arrival per epilogue warp of either CTA
    }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(&tmem_base_s), 512);
  tc_fence_before();
  __syncthreads();
  sb::cluster_sync();      // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  sb::grid_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer of this CTA: its half of the weight rows and of the tokens, counted on the leader's barrier
      sb::grid_dependency_wait();
      RingPos pos(p.stages, 1);
      for (int tile = pair; tile < total_tiles; tile += pairs) {
        const int tile_m = tile % p.tiles_m, tile_n = tile / p.tiles_m;
        for (int i = 0; i < kblocks; ++i, pos.advance()) {
          const uint32_t slot = pos.slot;
          mbar_wait(smem_u32(&empty_bar[slot]), pos.par, p.status, 1);
          const uint32_t bar = smem_u32(&full_bar[slot]);
          const uint32_t a = smem0 + slot * stage_bytes;
          if (rank == 0) mbar_expect_tx(bar, 2 * stage_bytes);
          const int k = i * kTileK;
          if (EPI == kSwiglu) {
            const int row_w = tile_m * 128 + rank * 64;        // 64 gate rows and their 64 up rows
            tma_load_2d_pair(a, &map_w, bar, k, row_w);
            tma_load_2d_pair(a + kStageA / 2, &map_w, bar, k, p.half_rows + row_w);
          } else {
            tma_load_2d_pair(a, &map_w, bar, k, tile_m * 256 + rank * kTileM);
          }
          tma_load_2d_pair(a + kStageA, &map_x, bar, k, tile_n * BN + rank * half_n);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---------------- MMA issuer of the pair
      const uint32_t idesc = sb::tc5::instr_desc(256, BN, false);
      const uint64_t desc_fixed = smem_desc_sw128(0);
      RingPos pos(p.stages, 0);
      int q = 0;
      for (int tile = pair; tile < total_tiles; tile += pairs) {
        for (int r = 0; r < p.splits; ++r, ++q) {
          const int kb0 = r * p.kblocks_per_split;
          const int iters = min(kblocks, kb0 + p.kblocks_per_split) - kb0;
          const int acc = q & 1;
          if (q >= 2) mbar_wait(smem_u32(&accum_empty[acc]), ((q >> 1) - 1) & 1, p.status, 4);
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + acc * BN;
          for (int i = 0; i < iters; ++i) {
            mbar_wait(smem_u32(&full_bar[pos.slot]), pos.par, p.status, 2);
            tc_fence_after();
            const uint64_t da = stage_desc(desc_fixed, smem0, pos.slot, stage_bytes, 0), db = stage_desc(desc_fixed, smem0, pos.slot, stage_bytes, kStageA);
#pragma unroll
            for (int k = 0; k < kTileK / 16; ++k) umma_pair_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
            umma_pair_commit(smem_u32(&empty_bar[pos.slot]));
            pos.advance();
          }
          umma_pair_commit(smem_u32(&accum_full[acc]));
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue of this CTA's 128 rows
    const int quarter = warp & 3;
    sb::grid_dependency_wait();
    int q = 0;
    for (int tile = pair; tile < total_tiles; tile += pairs) {
      const int tile_m = tile % p.tiles_m, tile_n = tile / p.tiles_m;
      if (EPI == kSwiglu) {
        const int acc = q & 1;
        const bool ok = mbar_wait(smem_u32(&accum_full[acc]), (q >> 1) & 1, p.status, 3);
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
        const int n0 = tile_n * BN;
        // lanes 0..63 hold gate rows, lanes 64..127 the matching up rows; the two sets of four warps take
        // alternate groups of sixteen tokens, each set with its own exchange buffer and barrier
        const int j = tile_m * 128 + rank * 64 + (quarter & 1) * 32 + lane;  // output feature
        const int set = (warp - 2) >> 2;
        float* xch = xch2[set];
        bf16* out = reinterpret_cast<bf16*>(p.out);
        for (int c0 = 16 * set; c0 < BN; c0 += 32) {
          float v[16];
          tmem_load16(tmem_d + c0, v);
          // gate warps hand over columns 8..15, up warps columns 0..7: every warp then finishes eight columns
          if (quarter >= 2) {
#pragma unroll
            for (int c = 0; c < 8; ++c) xch[c * 64 + (quarter - 2) * 32 + lane] = v[c];
          } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) xch[(8 + c) * 64 + quarter * 32 + lane] = v[8 + c];
          }
          if (set == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
          else asm volatile("bar.sync 2, 128;" ::: "memory");
          if (ok && j < p.half_rows) {
            const int cb = quarter >= 2 ? 8 : 0;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const int n = n0 + c0 + cb + c;
              if (n < p.N) {
                const float other = xch[(cb + c) * 64 + (quarter & 1) * 32 + lane];
                const float g = quarter >= 2 ? other : v[c], u = quarter >= 2 ? v[8 + c] : other;
                out[static_cast<int64_t>(n) * p.ldo + j] = __float2bfloat16_rn(silu_fast(g) * u);
              }
            }
          }
          if (set == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
          else asm volatile("bar.sync 2, 128;" ::: "memory");
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_leader(smem_u32(&accum_empty[acc]));
        ++q;
      } else {
        const int half = (warp - 2) >> 2, cols = BN / 2;
        const int m = tile_m * 256 + rank * kTileM + quarter * 32 + lane;
        const int n0 = tile_n * BN + half * cols;
        const bool live = m < p.M;
        float* o = p.out + static_cast<int64_t>(n0) * p.ldo + m;
        float run[kFoldCols];
#pragma unroll 1
        for (int r = 0; r < p.splits; ++r, ++q) {
          const int acc = q & 1;
          mbar_wait(smem_u32(&accum_full[acc]), (q >> 1) & 1, p.status, 3);
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + acc * BN + half * cols + (static_cast<uint32_t>(quarter * 32) << 16);
          if (r == 0) {
#pragma unroll
            for (int c0 = 0; c0 < kFoldCols; c0 += 16)
              if (c0 < cols) tmem_load16(tmem_d + c0, run + c0);
          } else {
#pragma unroll
            for (int c0 = 0; c0 < kFoldCols; c0 += 16) {
              if (c0 < cols) {
                float v[16];
                tmem_load16(tmem_d + c0, v);
#pragma unroll
                for (int c = 0; c < 16; ++c) run[c0 + c] += v[c];
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_leader(smem_u32(&accum_empty[acc]));
        }
        if (live) {
#pragma unroll
          for (int c = 0; c < kFoldCols; ++c)
            if (c < cols && n0 + c < p.N) o[static_cast<int64_t>(c) * p.ldo] = run[c];
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  sb::cluster_sync();      // neither CTA frees the pair's tensor memory, or leaves, while the other still works
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// The gate|up projection of many tokens with two weight tiles against one token tile: 128 gate rows and their 128 up
// rows accumulate side by side (two accumulators of BN columns, all of tensor memory), so that a K step of 64 brings
// 32 KB + BN * 128 bytes for twice the products of a single tile: what bounds these products is the ~26 KB per 512
// cycles that one SM takes in by TMA. A thread of the epilogue finds a feature's gate and up value in the same lane
// of the two accumulators: no exchange through shared memory. The accumulators are not double-buffered; the
// epilogue (eight warps) is short beside the main loop. Same bits as the other SwiGLU epilogues of this file.
__global__ void __launch_bounds__(kFoldThreads, 1)
gemm_tc_wide_swiglu_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t accum_full, accum_empty;
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BN = p.block_n;
  const int stage_bytes = 2 * kStageA + BN * 128;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int kblocks = (p.K + kTileK - 1) / kTileK;
  const int total_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&accum_full), 1);
    mbar_init(smem_u32(&accum_empty), 8);   // one arrival per epilogue warp
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_s), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  sb::grid_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer
      sb::grid_dependency_wait();
      RingPos pos(p.stages, 1);
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const int tile_m = tile % p.tiles_m, tile_n = tile / p.tiles_m;
        for (int i = 0; i < kblocks; ++i) {
          mbar_wait(smem_u32(&empty_bar[pos.slot]), pos.par, p.status, 1);
          const uint32_t bar = smem_u32(&full_bar[pos.slot]);
          const uint32_t a = smem0 + pos.slot * stage_bytes;
          mbar_expect_tx(bar, stage_bytes);
          tma_load_2d(a, &map_w, bar, i * kTileK, tile_m * kTileM);
          tma_load_2d(a + kStageA, &map_w, bar, i * kTileK, p.half_rows + tile_m * kTileM);
          tma_load_2d(a + 2 * kStageA, &map_x, bar, i * kTileK, tile_n * BN);
          pos.advance();
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer: gate rows into columns [0, BN), up rows into [256, 256 + BN)
      const uint32_t idesc = instr_desc(BN);
      const uint64_t desc_fixed = smem_desc_sw128(0);
      RingPos pos(p.stages, 0);
      int ti = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++ti) {
        if (ti >= 1) mbar_wait(smem_u32(&accum_empty), (ti - 1) & 1, p.status, 4);
        tc_fence_after();
        for (int i = 0; i < kblocks; ++i, pos.advance()) {
          const uint32_t slot = pos.slot;
          mbar_wait(smem_u32(&full_bar[slot]), pos.par, p.status, 2);
          tc_fence_after();
          const uint64_t dg = stage_desc(desc_fixed, smem0, slot, stage_bytes, 0), du = stage_desc(desc_fixed, smem0, slot, stage_bytes, kStageA),
                         db = stage_desc(desc_fixed, smem0, slot, stage_bytes, 2 * kStageA);
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k) {
            umma_bf16(tmem_base, dg + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
            umma_bf16(tmem_base + 256, du + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[slot]));
        }
        umma_commit(smem_u32(&accum_full));
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue: warp w reads TMEM lanes 32 * (w % 4) .. and the tile's columns [half * BN / 2, ..)
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    sb::grid_dependency_wait();
    bf16* out = reinterpret_cast<bf16*>(p.out);
    int ti = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++ti) {
      const int tile_m = tile % p.tiles_m, tile_n = tile / p.tiles_m;
      const bool ok = mbar_wait(smem_u32(&accum_full), ti & 1, p.status, 3);
      tc_fence_after();
      const int j = tile_m * kTileM + quarter * 32 + lane;     // output feature
      const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
      for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 16) {
        float g[16], u[16];
        tmem_load16(tmem_base + lane_addr + c0, g);
        tmem_load16(tmem_base + 256 + lane_addr + c0, u);
        if (ok && j < p.half_rows) {
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const int n = tile_n * BN + c0 + c;
            if (n < p.N) out[static_cast<int64_t>(n) * p.ldo + j] = __float2bfloat16_rn(silu_fast(g[c]) * u[c]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&accum_empty));
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------ host side
// Tensor map of a row-major bfloat16 matrix [rows, cols] with leading dimension ld (elements) and a box of
// box_rows x 64 elements in the 128-byte swizzle.
bool tensor_map(const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, CUtensorMap* out) {
  const int64_t dims[2] = {cols, rows}, strides[2] = {1, ld};
  const int box[2] = {kTileK, box_rows};
  return tensor_map_bf16(base, 2, dims, strides, box, out);
}

}  // namespace

// The number of K ranges of a [M, K] weight: enough CTAs to occupy the GPU with a few tokens when the weight
// alone gives too few tiles, limited so that the partial sums stay small beside the weight. It depends on the
// weight's shape alone, so that a token's sums have the same order in every batch.
SB_EXPORT int sb_gemm_tc_splits(int M, int K) {
  const int tiles_m = (M + kTileM - 1) / kTileM;
  const int kblocks = (K + kTileK - 1) / kTileK;
  // (the literal is the SM count of the GPU this engine is written for: the ranges must follow from the weight's shape
  // alone, never from the device that happens to run it, or two devices would add a token's sums in different orders)
  int splits = 148 / tiles_m;   // at most one wave of CTAs
  splits = min(splits, kblocks / 2);
  splits = max(splits, 1);
  const int per = (kblocks + splits - 1) / splits;
  return (kblocks + per - 1) / per;
}

// The most tokens for which sb_gemm_tc leaves one partial buffer per K range; with more it adds the ranges itself.
// (Measured at the 1B layer sizes: up to 512 tokens a CTA per K range and the consumer's additions beat one CTA that
// walks all ranges of its tile, since the tiles of so few tokens leave most SMs idle: a step of 256 tokens 2.28 ms
// against 3.0 ms, of 512 tokens 2.94 against 3.15; at 1,024 tokens the partial sums' traffic costs more than it saves.)
SB_EXPORT int sb_gemm_tc_partial_tokens() { return 512; }

// out = x . W^T on the tensor cores.
//   epilogue 0: out float32 [n, ldo]; `splits` K ranges (sb_gemm_tc_splits, or 1). Up to sb_gemm_tc_partial_tokens()
//               tokens, range s is stored at out + s * split_stride and the caller adds the ranges in ascending
//               order; with more tokens the kernel adds them itself and stores the sum at out.
//   epilogue 1: out float32 [n, ldo] += result (one range)
//   epilogue 2: W is [2 * half_rows, K] (gate rows then up rows); out bfloat16 [n, ldo] = silu(gate) * up
SB_EXPORT int sb_gemm_tc(const void* x, int64_t ldx, const void* w, int64_t ldw, void* out, int64_t ldo, int n, int M, int K,
                         int epilogue, int splits, int64_t split_stride, int half_rows, cudaStream_t stream) {
  if (n <= 0 || M <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0)
    return sb::fail("sb_gemm_tc: K %d and the leading dimensions (%lld, %lld) must be multiples of 8", K, (long long)ldx, (long long)ldw);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15)
    return sb::fail("sb_gemm_tc: operands must be 16-byte aligned");
  if (epilogue < 0 || epilogue > 2) return sb::fail("sb_gemm_tc: unknown epilogue %d", epilogue);
  const bool fold = splits > 1 && n > sb_gemm_tc_partial_tokens();   // the kernel adds the ranges
  if (epilogue == kSwiglu && splits != 1) return sb::fail("sb_gemm_tc: the SwiGLU epilogue takes no K ranges");
  if (epilogue == kAdd && splits != 1) return sb::fail("sb_gemm_tc: the sum of K ranges is added to the residual by its consumer (plain store)");
  if (epilogue == kSwiglu && (half_rows <= 0 || M != 2 * half_rows)) return sb::fail("sb_gemm_tc: swiglu needs M = 2 * half_rows");
  const int kblocks = (K + kTileK - 1) / kTileK;
  if (splits < 1 || splits > kblocks) return sb::fail("sb_gemm_tc: %d splits for %d blocks of K", splits, kblocks);
  int* status = status_word();
  if (!status) return sb::fail("sb_gemm_tc: cannot allocate the status word");

  const long long sms = sb::sm_count(), pairs = sms / 2;
  GemmParams p{};
  p.out = static_cast<float*>(out);
  p.ldo = ldo;
  p.split_stride = split_stride;
  p.M = M;
  p.N = n;
  p.K = K;
  if (n <= 128) {
    p.block_n = n <= 16 ? 16 : n <= 32 ? 32 : n <= 64 ? 64 : 128;
  } else {
    // Token tiles of 32..256: the width that needs the fewest cycles, counting whole waves of 148 CTAs. A K step of
    // 64 costs about max(2 BN, 128 + BN) cycles: the tensor cores or, for narrow tiles, the operands' shared-memory reads.
    // (A token's result does not depend on the width: every element is its own chain over K.)
    const long long tm = epilogue == kSwiglu ? (half_rows + 63) / 64 : (M + kTileM - 1) / kTileM;
    long long best = -1;
    for (int bn = 256; bn >= 32; bn -= 32) {
      const long long tiles = tm * ((n + bn - 1) / bn) * (fold ? 1 : splits);
      const long long cost = ((tiles + sms - 1) / sms) * (2 * bn > 128 + bn ? 2 * bn : 128 + bn);
      if (best < 0 || cost < best) {
        best = cost;
        p.block_n = bn;
      }
    }
  }
  // K ranges on CTAs of their own and more than 256 tokens: each tile's K loop is short (4 to 15 steps at the 1B
  // sizes), so a tile is mostly pipeline fill and epilogue; tiles of 64 tokens run three CTAs an SM, which hides that
  // (measured, 384 tokens: [2048, 2048] 12.2 us against 21.5, [3072, 2048] 13.7 against 22.9, [2048, 8192] 22.2 against 27.9).
  if (!fold && splits > 1 && n > 256) p.block_n = 64;
  const int stage_bytes = kStageA + p.block_n * 128;
  p.stages = min(kMaxStages, kSmemBudget / stage_bytes);
  {
    // Many tiles and few tokens (a bandwidth-bound stream such as the head): three CTAs an SM with shorter
    // rings, so that one's prologue and epilogue overlap with the others' streaming. Many tiles and many
    // tokens: one CTA an SM with the deepest ring; its two accumulators overlap epilogue and main loop.
    const long long tiles = static_cast<long long>(epilogue == kSwiglu ? (half_rows + 63) / 64 : (M + kTileM - 1) / kTileM) *
                            ((n + p.block_n - 1) / p.block_n) * splits;
    if (tiles > 2 * sms && p.block_n <= 64) p.stages = max(2, min(p.stages, (kSmemBudget + 16 * 1024) / 3 / stage_bytes));
    // Between one and two tiles an SM with at most 128 tokens (gate|up of the 8B shape: 224 tiles): two CTAs an SM with
    // half the ring each, all tiles resident at once. With one CTA an SM the second round keeps half the SMs busy, each
    // with one ring's worth of bytes in flight, which is half of what HBM needs (8B gate|up at 128 tokens: 57 -> 50 us).
    else if (tiles > sms && tiles <= 2 * sms && n <= 128) p.stages = max(2, min(p.stages, (111 * 1024) / stage_bytes));
  }
  p.kblocks_per_split = (kblocks + splits - 1) / splits;
  if ((kblocks + p.kblocks_per_split - 1) / p.kblocks_per_split != splits)
    return sb::fail("sb_gemm_tc: %d splits leave an empty K range (use sb_gemm_tc_splits)", splits);
  // Few tokens: a ring of at most six stages, and no longer than the CTA's K range. Six stages of 16 KB a CTA keep
  // HBM busy (more changed nothing), and a CTA of at most ~110 KB leaves room on its SM for the CTAs of the next
  // projection of the step, which then become resident early and have their first weight tiles under way while this
  // kernel still runs (a decode step of batch 8 at the 1B sizes: 0.891 ms with eight stages, 0.865 with six, 0.883 with
  // four, 0.940 with three).
  if (n <= 128) p.stages = max(2, min(p.stages, min(6, p.kblocks_per_split)));
  p.half_rows = half_rows;
  p.status = status;

  // The SwiGLU product of many tokens runs on pairs of CTAs or with two weight tiles a CTA; both bring the same bytes
  // from L2 (what bounds these products), the pairs in units half as large. Whichever needs fewer rounds of units of
  // 128 features x 256 tokens a CTA takes it (two weight tiles on a tie: no traffic between the SMs of a pair).
  bool wide = false;
  if (n > 256 && epilogue == kSwiglu) {
    const long long tn = (n + 255) / 256;
    const long long pair_rounds = (((half_rows + 127) / 128) * tn + pairs - 1) / pairs;
    const long long wide_rounds = 2 * ((((half_rows + kTileM - 1) / kTileM) * tn + sms - 1) / sms);
    wide = wide_rounds <= pair_rounds;
  }
  if (wide) {
    const long long tm = (half_rows + kTileM - 1) / kTileM;
    p.block_n = 256;
    const int wide_stage = 2 * kStageA + p.block_n * 128;
    p.stages = min(kMaxStages, kSmemBudget / wide_stage);
    p.kblocks_per_split = kblocks;
    p.half_rows = half_rows;
    p.status = status;
    p.tiles_m = static_cast<int>(tm);
    p.tiles_n = (n + p.block_n - 1) / p.block_n;
    p.splits = 1;
    CUtensorMap ww, wx;
    if (!tensor_map(w, M, K, ldw, kTileM, &ww) || !tensor_map(x, n, K, ldx, p.block_n, &wx))
      return sb::fail("sb_gemm_tc: cuTensorMapEncodeTiled failed (M %d N %d K %d)", M, n, K);
    const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
    if (tiles > (1ll << 30)) return sb::fail("sb_gemm_tc: too many tiles");
    static sb::DeviceOnce once;
    if (once.needed()) {
      if (cudaFuncSetAttribute(gemm_tc_wide_swiglu_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 2048) != cudaSuccess)
        return sb::fail("sb_gemm_tc: cannot raise the shared memory limit");
      once.done();
    }
    sb::launch_pdl(gemm_tc_wide_swiglu_kernel, dim3(static_cast<unsigned>(min(tiles, sms))), dim3(kFoldThreads),
                   static_cast<size_t>(p.stages) * wide_stage + 1024, stream, ww, wx, p);
    return sb::check_launch("sb_gemm_tc");
  }
  // (pairs from 129 tokens on when K is one range: a CTA of a pair takes in half of the token tile, and with more than
  // 128 tokens a single CTA's intake of both operands, not HBM, bounds a K step: a step of 256 tokens 1.52 -> 1.44 ms)
  if (n > 128 && epilogue != kAdd && (splits == 1 || fold)) {
    // Pairs of CTAs: tiles of 256 weight rows (or 128 gate + 128 up rows) by BN tokens, BN chosen by whole waves of 74 pairs.
    const long long tm = epilogue == kSwiglu ? (half_rows + 127) / 128 : (M + 255) / 256;
    long long best = -1;
    int bn_best = 256;
    // (narrower tiles bring more bytes from L2 for the same products, which is what bounds a large product: only a
    // step of fewer than 1,024 tokens is cut into narrower tiles to fill its rounds)
    for (int bn = 256; bn >= 128; bn -= 32) {
      // cycles of a K step of 64: the tensor cores (2 BN), or the bytes a CTA takes in (16 KB of weights and its half
      // of the token tile) at about 51 bytes a cycle; times whole rounds of 74 pairs
      const long long step = max(2ll * bn, (16384ll + 64 * bn) / 51);
      const long long cost = ((tm * ((n + bn - 1) / bn) + pairs - 1) / pairs) * step;
      if (best < 0 || cost < best) {
        best = cost;
        bn_best = bn;
      }
    }
    p.block_n = bn_best;
    const int pair_stage = kStageA + (p.block_n / 2) * 128;
    p.stages = min(kMaxStages, kSmemBudget / pair_stage);
    p.kblocks_per_split = (kblocks + splits - 1) / splits;
    if ((kblocks + p.kblocks_per_split - 1) / p.kblocks_per_split != splits)
      return sb::fail("sb_gemm_tc: %d splits leave an empty K range (use sb_gemm_tc_splits)", splits);
    p.half_rows = half_rows;
    p.status = status;
    p.tiles_m = static_cast<int>(tm);
    p.tiles_n = (n + p.block_n - 1) / p.block_n;
    p.splits = splits;
    CUtensorMap pw, px;
    if (!tensor_map(w, M, K, ldw, epilogue == kSwiglu ? 64 : kTileM, &pw) || !tensor_map(x, n, K, ldx, p.block_n / 2, &px))
      return sb::fail("sb_gemm_tc: cuTensorMapEncodeTiled failed (M %d N %d K %d)", M, n, K);
    const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
    if (tiles > (1ll << 30)) return sb::fail("sb_gemm_tc: too many tiles");
    const dim3 grid(static_cast<unsigned>(2 * min(tiles, pairs)));
    const size_t psmem = static_cast<size_t>(p.stages) * pair_stage + 1024;
    static sb::DeviceOnce once;
    if (once.needed()) {
      if (cudaFuncSetAttribute(gemm_tc_pair_kernel<kStore>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 2048) != cudaSuccess ||
          cudaFuncSetAttribute(gemm_tc_pair_kernel<kSwiglu>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 2048) != cudaSuccess)
        return sb::fail("sb_gemm_tc: cannot raise the shared memory limit");
      once.done();
    }
    if (epilogue == kStore)
      sb::launch_pdl_cluster(gemm_tc_pair_kernel<kStore>, grid, dim3(kFoldThreads), psmem, stream, dim3(2, 1, 1), pw, px, p);
    else
      sb::launch_pdl_cluster(gemm_tc_pair_kernel<kSwiglu>, grid, dim3(kFoldThreads), psmem, stream, dim3(2, 1, 1), pw, px, p);
    return sb::check_launch("sb_gemm_tc");
  }

  CUtensorMap map_w, map_x;
  const int box_w = epilogue == kSwiglu ? 64 : kTileM;
  if (!tensor_map(w, M, K, ldw, box_w, &map_w) || !tensor_map(x, n, K, ldx, p.block_n, &map_x))
    return sb::fail("sb_gemm_tc: cuTensorMapEncodeTiled failed (M %d N %d K %d)", M, n, K);

  p.tiles_m = epilogue == kSwiglu ? (half_rows + 63) / 64 : (M + kTileM - 1) / kTileM;
  p.tiles_n = (n + p.block_n - 1) / p.block_n;
  p.splits = splits;
  const long long total_tiles = static_cast<long long>(p.tiles_m) * p.tiles_n * (fold ? 1 : splits);
  if (total_tiles > (1ll << 30)) return sb::fail("sb_gemm_tc: too many tiles");
  const size_t smem = static_cast<size_t>(p.stages) * stage_bytes + 1024;
  if (fold) {
    const dim3 grid(static_cast<unsigned>(min(total_tiles, sms)));
    static sb::DeviceOnce once;
    if (once.needed()) {
      if (cudaFuncSetAttribute(gemm_tc_fold_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 2048) != cudaSuccess)
        return sb::fail("sb_gemm_tc: cannot raise the shared memory limit");
      once.done();
    }
    sb::launch_pdl(gemm_tc_fold_kernel, grid, dim3(kFoldThreads), smem, stream, map_w, map_x, p);
    return sb::check_launch("sb_gemm_tc");
  }
  // Persistent CTAs: as many as fit the GPU at once (by shared and tensor memory), each walking tiles.
  int per_sm = static_cast<int>((227 * 1024) / (smem + 2048));
  per_sm = max(1, min(per_sm, 512 / static_cast<int>(tmem_alloc_cols(2 * p.block_n))));
  const long long resident = sms * per_sm;
  const bool multi = total_tiles > resident;
  if (!multi && (p.tiles_n > 65535 || splits > 65535)) return sb::fail("sb_gemm_tc: grid too large");
  const dim3 grid(static_cast<unsigned>(multi ? resident : total_tiles));
#define SB_LAUNCH_M(EPI, MULTI)                                                                         \
  do {                                                                                                  \
    static sb::DeviceOnce once;                                                                       \
    if (once.needed()) {                                                                                    \
      if (cudaFuncSetAttribute(gemm_tc_kernel<EPI, MULTI>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                               kSmemBudget + 2048) != cudaSuccess)                                      \
        return sb::fail("sb_gemm_tc: cannot raise the shared memory limit");                            \
      once.done();                                                                                  \
    }                                                                                                   \
    sb::launch_pdl(gemm_tc_kernel<EPI, MULTI>, grid, dim3(kThreads), smem, stream, map_w, map_x, p);    \
  } while (0)
#define SB_LAUNCH_S(EPI)                                                                                \
  do {                                                                                                  \
    static sb::DeviceOnce once;                                                                       \
    if (once.needed()) {                                                                                    \
      if (cudaFuncSetAttribute(gemm_tc_single_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                               kSmemBudget + 2048) != cudaSuccess)                                      \
        return sb::fail("sb_gemm_tc: cannot raise the shared memory limit");                            \
      once.done();                                                                                  \
    }                                                                                                   \
    sb::launch_pdl(gemm_tc_single_kernel<EPI>, dim3(p.tiles_m, p.tiles_n, splits), dim3(kThreads), smem, stream, map_w, map_x, p); \
  } while (0)
#define SB_LAUNCH(EPI)                  \
  do {                                  \
    if (multi) SB_LAUNCH_M(EPI, true);  \
    else SB_LAUNCH_S(EPI);              \
  } while (0)
  if (epilogue == kStore) SB_LAUNCH(kStore);
  else if (epilogue == kAdd) SB_LAUNCH(kAdd);
  else SB_LAUNCH(kSwiglu);
#undef SB_LAUNCH
#undef SB_LAUNCH_S
#undef SB_LAUNCH_M
  return sb::check_launch("sb_gemm_tc");
}

// From now on the kernels of this library report into `device_word` (an int of device memory that the caller
// keeps alive and has zeroed); null: into the library's own word again. Kernels already recorded in a CUDA graph keep
// the word they were recorded with.
SB_EXPORT void sb_gemm_tc_use_status_word(int* device_word) { status_word_given() = device_word; }

namespace {
// A wait that nothing ends: one thread waits on a barrier on which nobody arrives, gives up after the usual limit
// and reports `code`.
__global__ void lost_signal_kernel(int* status, int code) {
  __shared__ __align__(8) uint64_t bar;
  mbar_init(smem_u32(&bar), 1);
  mbar_init_fence();
  mbar_wait(smem_u32(&bar), 0, status, code);
}
}  // namespace

// Self-test of the reporting path: launches the kernel above (about a second) and returns; the status word then
// reads `code` until somebody clears it.
SB_EXPORT int sb_gemm_tc_lost_signal_selftest(int code, cudaStream_t stream) {
  int* status = status_word();
  if (!status) return sb::fail("sb_gemm_tc: cannot allocate the status word");
  lost_signal_kernel<<<1, 1, 0, stream>>>(status, code);
  return sb::check_launch("sb_gemm_tc_lost_signal_selftest");
}

// Reads and clears the status word: 0 = every wait completed; 1, 2, 3 = the producer, the MMA issuer or
// the epilogue gave up waiting. Synchronises the device.
SB_EXPORT int sb_gemm_tc_status() {
  int* status = status_word();
  if (!status) return -1;
  int host = 0;
  if (cudaMemcpy(&host, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (host != 0) cudaMemset(status, 0, sizeof(int));
  return host;
}

// ------------------------------------------------------------------ operation of the native step program (step_ops.h)
// i: 0 x (bfloat16 [n, ldx]), 1 ldx, 2 weight, 3 ldw, 4 out, 5 M, 6 K,
//    7 mode: 0 = out float32 [n, M], K in one range; 1 = partial sums [P, n, M] of the weight's K ranges (P = S up to
//            sb_gemm_tc_partial_tokens() tokens, else 1: the kernel adds the ranges); 2 = out float32 [n, M] += result;
//            3 = SwiGLU, out bfloat16 [n, M / 2]
//    8 K ranges S (mode 1), 9 rows: 0 = the step's tokens, 1 = the rows whose logits are wanted
SB_EXPORT int sb_op_linear_tc(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  const int n = op->i[9] ? s->wanted : s->n;
  if (n <= 0) return SB_OP_SKIPPED;
  const int M = (int)op->i[5], K = (int)op->i[6], mode = (int)op->i[7], S = (int)op->i[8];
  const void* x = ptr<const void>(op->i[0]);
  const void* w = ptr<const void>(op->i[2]);
  void* out = ptr<void>(op->i[4]);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (mode) {
    case 0: return sb_gemm_tc(x, op->i[1], w, op->i[3], out, M, n, M, K, kStore, 1, 0, 0, st);
    case 1: {
      const bool buffers = S > 1 && n <= sb_gemm_tc_partial_tokens();
      return sb_gemm_tc(x, op->i[1], w, op->i[3], out, M, n, M, K, kStore, S, buffers ? static_cast<int64_t>(n) * M : 0, 0, st);
    }
    case 2: return sb_gemm_tc(x, op->i[1], w, op->i[3], out, M, n, M, K, kAdd, 1, 0, 0, st);
    case 3: return sb_gemm_tc(x, op->i[1], w, op->i[3], out, M / 2, n, M, K, kSwiglu, 1, 0, M / 2, st);
    default: return sb::fail("sb_op_linear_tc: unknown mode %d", mode);
  }
}
