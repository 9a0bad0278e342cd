// The one arithmetic of the bfloat16 attention kernels, so that a query row gets the same bits from each of
// them (tcgen05 or mma.sync, a prompt portion or a decoded token, alone or in a batch):
//
//   tile   64 keys by absolute position [64 t, 64 t + 64). s_j = q . k_j on the tensor cores (float32 accumulation
//          over K steps of 16 in ascending order), m = (max s_j) * c with c = scale * log2(e),
//          p_j = ex2(fma(s_j, c, -m)), 0 for a key the row does not see. l = sum of p_j: key j belongs to class
//          (j % 8) / 2, each class is added in ascending order of j, then l = (u0 + u1) + (u2 + u3).
//          p = hi + lo, two bfloat16 parts (p rounded, then the remainder rounded); o = sum over steps of 16 keys,
//          ascending, of hi . V then lo . V, accumulated on the tensor cores from zero.
//   chunk  256 keys [256 c, 256 c + 256): the tiles a row sees are folded left to right into an empty state.
//   row    the chunks a row sees are folded left to right into an empty state; out = o * (1 / l).
//   fold   (m, l, o) <- (m_t, l_t, o_t): m' = max(m, m_t), a = ex2(m - m'), b = ex2(m_t - m'),
//          l = fma(l, a, l_t * b), o = fma(o, a, o_t * b). The empty state is (-inf, 0, 0).
//
// tcgen05.mma (kind::f16) and mma.sync m16n8k16 give the same bits for the same products in the same order of
// K steps on this hardware (checked by the tests), which is what lets kernels built on either share this.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace sb {
namespace attn {

constexpr int kTileKeys = 64;
constexpr int kChunkKeys = 256;
constexpr float kLog2e = 1.4426950408889634f;

// 2^x by the hardware's approximation: a pure function of x, the same in every kernel.
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The tile's maximum in the exponent's units, from the maximum of the raw scores (c > 0).
__device__ __forceinline__ float tile_max(float raw_max, float c) { return __fmul_rn(raw_max, c); }
// The subtrahend of the exponent: the maximum, or 0 for a tile without a visible key.
__device__ __forceinline__ float tile_ref(float m) { return m == -INFINITY ? 0.0f : m; }
__device__ __forceinline__ float weight(float s, float c, float ref) { return ex2(__fmaf_rn(s, c, -ref)); }
__device__ __forceinline__ float class_sum(float u0, float u1, float u2, float u3) {
  return __fadd_rn(__fadd_rn(u0, u1), __fadd_rn(u2, u3));
}

// p0, p1 -> packed bfloat16 pairs (p0 in the low half): hi = p rounded to bfloat16, lo = the remainder p - hi (exact in
// float32) rounded to bfloat16: |p - hi - lo| <= 2^-18 p, without bias.
__device__ __forceinline__ void split_hi_lo(float p0, float p1, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  const float r0 = __fsub_rn(p0, __uint_as_float(hi << 16)), r1 = __fsub_rn(p1, __uint_as_float(hi & 0xFFFF0000u));
  const __nv_bfloat162 l = __floats2bfloat162_rn(r0, r1);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

struct FoldFactors {
  float m, a, b;
};
// Factors of folding a part with maximum m_t (finite) into a state with maximum m (finite or -inf).
__device__ __forceinline__ FoldFactors fold_factors(float m, float m_t) {
  FoldFactors f;
  f.m = fmaxf(m, m_t);
  f.a = ex2(__fsub_rn(m, f.m));
  f.b = ex2(__fsub_rn(m_t, f.m));
  return f;
}
__device__ __forceinline__ float fold_value(float v, float v_t, const FoldFactors& f) {
  return __fmaf_rn(v, f.a, __fmul_rn(v_t, f.b));
}
__device__ __forceinline__ float finish(float o, float l) { return __fmul_rn(o, __frcp_rn(l)); }

}  // namespace attn
}  // namespace sb
