// What the tcgen05 linear kernels share (gemm_tc.cu and the fused decode chain, decode_chain.cu): the tile sizes, the
// accumulator loads, and the epilogues of one accumulator tile of 128 weight rows by BN tokens, so that a token's
// product has the same bits whichever kernel computed it.
#pragma once

#include "tc5.cuh"

namespace sb {
namespace gemm_tile {

using namespace sb::tc5;
using bf16 = __nv_bfloat16;

constexpr int kTileM = 128;
constexpr int kTileK = 64;            // elements: 128 bytes of bfloat16, one swizzle row
constexpr int kStageA = kTileM * 128;  // bytes

enum Epilogue { kStore = 0, kAdd = 1, kSwiglu = 2 };

// ------------------------------------------------------------------ helpers on top of tc5.cuh
__device__ __forceinline__ void tmem_load16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  tmem_load_wait();
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_fence_before() { fence_before_sync(); }
__device__ __forceinline__ void tc_fence_after() { fence_after_sync(); }
// Tensor memory is allocated in powers of two of at least 32 columns.
__host__ __device__ __forceinline__ uint32_t tmem_alloc_cols(int cols) {
  uint32_t c = 32;
  while (c < static_cast<uint32_t>(cols)) c <<= 1;
  return c;
}
// Instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t instr_desc(int n) { return sb::tc5::instr_desc(kTileM, n, false); }

// silu(g) = g / (1 + e^-g) with the hardware's approximations of e^x and of the division (two units in the last
// place each, far below the bfloat16 rounding that follows): the same instruction sequence in every kernel of this
// file, so that a token's product has the same bits from each.
__device__ __forceinline__ float silu_fast(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// Rows of one accumulator tile to global memory: out[n, m] = d (kStore) or out[n, m] += d (kAdd). Each thread
// owns output feature m and walks the tile's tokens sixteen at a time; for kAdd the residual values of the
// next sixteen are requested before the current sixteen are summed and stored.
template <int EPI>
__device__ __forceinline__ void store_tile(uint32_t tmem_row, float* out, int m, int M, int n0, int N, int64_t ldo, int BN, bool ok) {
  const bool live = m < M && ok;
  float nxt[16];
  if (EPI == kAdd && live) {
#pragma unroll
    for (int c = 0; c < 16; ++c) nxt[c] = (n0 + c < N) ? out[static_cast<int64_t>(n0 + c) * ldo + m] : 0.0f;
  }
  for (int c0 = 0; c0 < BN; c0 += 16) {
    float v[16], old[16];
    float* o = out + static_cast<int64_t>(n0 + c0) * ldo + m;
    if (EPI == kAdd && live) {
#pragma unroll
      for (int c = 0; c < 16; ++c) old[c] = nxt[c];
      if (c0 + 16 < BN) {
#pragma unroll
        for (int c = 0; c < 16; ++c) nxt[c] = (n0 + c0 + 16 + c < N) ? o[static_cast<int64_t>(16 + c) * ldo] : 0.0f;
      }
    }
    tmem_load16(tmem_row + c0, v);
    if (live) {
#pragma unroll
      for (int c = 0; c < 16; ++c)
        if (n0 + c0 + c < N) o[static_cast<int64_t>(c) * ldo] = EPI == kAdd ? old[c] + v[c] : v[c];
    }
  }
}

// The SwiGLU epilogue of one accumulator tile by the four epilogue warps (128 threads that meet on named barrier 1):
// lanes 0..63 of the tile hold 64 gate rows, lanes 64..127 the matching up rows; out[n, j] = silu(gate) * up as
// bfloat16, j = tile_m * 64 + row. `quarter` = warp % 4 (the TMEM lanes this warp may read), xch: 16 x 64 floats of
// shared memory that nothing else uses meanwhile.
__device__ __forceinline__ void swiglu_tile(uint32_t tmem_base, float* xch, bf16* out, int64_t ldo, int tile_m, int half_rows, int n0,
                                            int N, int BN, int quarter, int lane, bool ok) {
  const int j = tile_m * 64 + (quarter & 1) * 32 + lane;  // output feature
  for (int c0 = 0; c0 < BN; c0 += 16) {
    float v[16];
    tmem_load16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c0, v);
    // gate warps hand over columns 8..15, up warps columns 0..7: every warp then finishes eight columns
    if (quarter >= 2) {
#pragma unroll
      for (int c = 0; c < 8; ++c) xch[c * 64 + (quarter - 2) * 32 + lane] = v[c];
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) xch[(8 + c) * 64 + quarter * 32 + lane] = v[8 + c];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (ok && j < half_rows) {
      const int cb = quarter >= 2 ? 8 : 0;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int n = n0 + c0 + cb + c;
        if (n < N) {
          const float other = xch[(cb + c) * 64 + (quarter & 1) * 32 + lane];
          const float g = quarter >= 2 ? other : v[c], u = quarter >= 2 ? v[8 + c] : other;
          out[static_cast<int64_t>(n) * ldo + j] = __float2bfloat16_rn(silu_fast(g) * u);
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
  }
}

}  // namespace gemm_tile
}  // namespace sb
