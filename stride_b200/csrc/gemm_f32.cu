// True 32-bit linear layer: out[n, M] (+)= x[n, K] . W[M, K]^T with FMA on the
// CUDA cores, no tensor cores and no reduced-precision matrix mode. Weights may be
// stored in bfloat16 (widened exactly) or in float32.
//
// The order of a dot product's additions is fixed, whatever the number of rows n and however the kernel is tiled, so a
// token's result does not depend on its batch: k is cut into pieces of eight, piece j belongs to class j % 32, every
// class is one chain of fused multiply-adds over its elements in ascending k (from zero), and the 32 classes are added
// by the butterfly of a warp (xor 16, 8, 4, 2, 1). A warp computes TM features by TN tokens; lane c is class c: it reads
// its pieces of the weight rows (16 bytes of bfloat16 at once, the 32 lanes 512 consecutive bytes) and of the tokens.
// One token is then a stream over the weights (gemv_f32_kernel below). With one dependent chain per output, the order
// before this one, the latency of K fused multiply-adds bounded it: 5 ms a decoded token at the sizes of Llama 3.2 1B,
// 1.07 ms now.
//
// Counterparts in arhaamatiq/stride: gemm_partial and its users GemmResidual,
// Mlp13, LmFull of the exact path (src/kernels.cu:63-94, 294-325, 329-363, 427-452), which add 32 interleaved
// partial sums likewise.
#include <algorithm>

#include "common.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;

// Eight consecutive values, widened. VEC: they start 16-byte aligned and all exist (one or two 16-byte loads);
// else element by element, those at or beyond `left` read as zero (a product with zero leaves a chain as it is).
template <bool VEC>
__device__ __forceinline__ void load8(const bf16* p, int left, float* v) {
  if (VEC) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = e < left ? __bfloat162float(p[e]) : 0.0f;
  }
}
template <bool VEC>
__device__ __forceinline__ void load8(const float* p, int left, float* v) {
  if (VEC) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = e < left ? p[e] : 0.0f;
  }
}

constexpr int kWarps = 4;      // warps of a block, each with features of its own

// blockIdx.x: kWarps * TM features, blockIdx.y: TN tokens. VEC: K is a multiple of 8 and every row of x and w starts
// 16-byte aligned. P: the pieces of every weight row that a lane requests at once, as a group; it changes what is in
// flight (P to 2P pieces a row), not the order of the additions.
template <class TX, class TW, bool VEC, int TM, int TN, int P>
__global__ void __launch_bounds__(kWarps * 32) gemm_f32_kernel(const TX* __restrict__ x, int64_t ldx, const TW* __restrict__ w,
                                                                int64_t ldw, float* __restrict__ out, int64_t ldo, int n, int M, int K,
                                                                int accumulate) {
  sb::grid_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = (blockIdx.x * kWarps + warp) * TM, n0 = blockIdx.y * TN;
  if (m0 >= M) return;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
  // rows beyond the matrix are read as the last one (their results are not stored)
  const TW* wrow[TM];
#pragma unroll
  for (int i = 0; i < TM; ++i) wrow[i] = w + static_cast<int64_t>(min(m0 + i, M - 1)) * ldw;
  const TX* xrow[TN];
#pragma unroll
  for (int j = 0; j < TN; ++j) xrow[j] = x + static_cast<int64_t>(min(n0 + j, n - 1)) * ldx;

  // Two groups of P pieces of every row are kept requested: when a group has been multiplied, the group two places on is
  // requested into its registers (a group's requests finish together, which is how the hardware counts them). The
  // weights do not depend on the kernels before this one: the first groups are requested before waiting for those.
  float wv[2][P][TM][8];
  const int k0 = lane * 8;
  auto request = [&](int h, int k) {
#pragma unroll
    for (int s = 0; s < P; ++s)
      if (k + 256 * s < K) {
#pragma unroll
        for (int i = 0; i < TM; ++i) load8<VEC>(wrow[i] + k + 256 * s, K - k - 256 * s, wv[h][s][i]);
      }
  };
  request(0, k0);
  request(1, k0 + 256 * P);
  sb::grid_dependency_wait();
  for (int k = k0; k < K; k += 512 * P) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int s = 0; s < P; ++s) {
        const int kk = k + 256 * (h * P + s);
        if (kk < K) {
#pragma unroll
          for (int j = 0; j < TN; ++j) {
            float xv[8];
            load8<VEC>(xrow[j] + kk, K - kk, xv);
#pragma unroll
            for (int e = 0; e < 8; ++e)
#pragma unroll
              for (int i = 0; i < TM; ++i) acc[i][j] = fmaf(xv[e], wv[h][s][i][e], acc[i][j]);
          }
        }
      }
      request(h, k + 256 * (h * P + 2 * P));
    }
  }
  // the 32 classes of every output, added by the butterfly; lane (i * TN + j) % 32 stores output (i, j)
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      float v = acc[i][j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == ((i * TN + j) & 31) && m0 + i < M && n0 + j < n) {
        float* dst = out + static_cast<int64_t>(n0 + j) * ldo + m0 + i;
        *dst = accumulate ? (*dst + v) : v;
      }
    }
}

template <class TX, class TW, bool VEC, int TM, int TN, int P>
void launch(const void* x, int64_t ldx, const void* w, int64_t ldw, float* out, int64_t ldo, int n, int M, int K, int accumulate,
            cudaStream_t stream) {
  const dim3 grid((M + kWarps * TM - 1) / (kWarps * TM), (n + TN - 1) / TN);
  sb::launch_pdl(gemm_f32_kernel<TX, TW, VEC, TM, TN, P>, grid, dim3(kWarps * 32), 0, stream, static_cast<const TX*>(x), ldx,
                 static_cast<const TW*>(w), ldw, out, ldo, n, M, K, accumulate);
}

// Eight consecutive values as they lie in memory (16 bytes of bfloat16, 32 of float32), widened when they are used:
// what a lane keeps in flight of a weight row costs half the registers for bfloat16.
template <class T>
struct Raw8;
template <>
struct Raw8<bf16> {
  uint4 v;
  __device__ __forceinline__ void load(const bf16* p) { v = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void widen(float* f) const {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) f[2 * i] = __uint_as_float(w[i] << 16), f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
};
template <>
struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) { a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4); }
  __device__ __forceinline__ void widen(float* f) const {
    f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
  }
};

// One token (a decoded token's linear layers): the token lies in shared memory and the weights are one stream. As many
// blocks as the GPU holds at once; warp g of all G takes the features g, g + G, g + 2G, ... and keeps NG groups of
// P pieces of their rows requested (a group is requested again as soon as it has been multiplied), across the end of
// a row into the next one, so that the requests in flight do not drain at every feature. The additions of a feature are those of the kernel above. K is a multiple of 8, rows 16-byte aligned.
template <class TX, class TW, int TM, int NG, int P>
__global__ void __launch_bounds__(kWarps * 32) gemv_f32_kernel(const TX* __restrict__ x, const TW* __restrict__ w, int64_t ldw,
                                                                float* __restrict__ out, int M, int K, int accumulate) {
  // The token, piece by piece: a piece's first four values of all 32 lanes, then its last four (a lane reads its
  // eight with two requests of 16 bytes, each of them consecutive over the lanes). Padded to whole pieces of 256.
  extern __shared__ __align__(16) float xs[];
  sb::grid_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.x * kWarps + warp, G = gridDim.x * kWarps;
  const int pieces = (K + 255) >> 8;  // of a row, for a lane (the last may lie beyond K for the upper lanes)
  const int groups = (M + TM - 1) / TM;  // of TM features; warp g takes the groups g, g + G, ...
  const int mine = g < groups ? (groups - g + G - 1) / G : 0;
  const int total = mine * pieces;
  const int kl = lane * 8;

  Raw8<TW> ring[NG][P][TM];
  int next_group = 0, next_piece = 0;  // the piece that is requested next
  auto request = [&](int h) {
#pragma unroll
    for (int s = 0; s < P; ++s)
      if (next_group < mine) {
        const int k = kl + 256 * next_piece;
        if (k < K) {
          const int m = (g + next_group * G) * TM;
#pragma unroll
          for (int i = 0; i < TM; ++i) ring[h][s][i].load(w + static_cast<int64_t>(min(m + i, M - 1)) * ldw + k);  // beyond M: read, not stored
        }
        if (++next_piece == pieces) next_piece = 0, ++next_group;
      }
  };
  // the weights do not depend on the kernels before this one
#pragma unroll
  for (int h = 0; h < NG; ++h) request(h);
  sb::grid_dependency_wait();
#pragma unroll 4
  for (int k = threadIdx.x * 8; k < K; k += kWarps * 32 * 8) {
    float v[8];
    load8<true>(x + k, 8, v);
    float* at = xs + (k & ~255) + ((k >> 3) & 31) * 4;
    *reinterpret_cast<float4*>(at) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(at + 128) = make_float4(v[4], v[5], v[6], v[7]);
  }
  __syncthreads();

  float acc[TM];
#pragma unroll
  for (int i = 0; i < TM; ++i) acc[i] = 0.0f;
  int group = 0, piece = 0;  // the piece that is multiplied next
  for (int q = 0; q < total; q += NG * P) {
#pragma unroll
    for (int h = 0; h < NG; ++h) {
#pragma unroll
      for (int s = 0; s < P; ++s) {
        if (q + h * P + s < total) {
          if (kl + 256 * piece < K) {
            const float4 xa = *reinterpret_cast<const float4*>(xs + 256 * piece + lane * 4);
            const float4 xb = *reinterpret_cast<const float4*>(xs + 256 * piece + 128 + lane * 4);
            const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
            float wv[TM][8];
#pragma unroll
            for (int i = 0; i < TM; ++i) ring[h][s][i].widen(wv[i]);
#pragma unroll
            for (int e = 0; e < 8; ++e)
#pragma unroll
              for (int i = 0; i < TM; ++i) acc[i] = fmaf(xv[e], wv[i][e], acc[i]);
          }
          if (++piece == pieces) {
            const int m = (g + group * G) * TM;
#pragma unroll
            for (int i = 0; i < TM; ++i) {
              float v = acc[i];
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
              if (lane == i && m + i < M) out[m + i] = accumulate ? (out[m + i] + v) : v;
              acc[i] = 0.0f;
            }
            piece = 0, ++group;
          }
        }
      }
      request(h);
    }
  }
}

constexpr int kGemvFeatures = 1, kGemvPieces = 4;
constexpr size_t kGemvMaxShared = 200 * 1024;
inline size_t gemv_shared(int K) { return static_cast<size_t>((K + 255) / 256) * 256 * sizeof(float); }

template <class TX, class TW, int NG>
void launch_gemv_groups(const void* x, const void* w, int64_t ldw, float* out, int M, int K, int accumulate, cudaStream_t stream) {
  auto kernel = gemv_f32_kernel<TX, TW, kGemvFeatures, NG, kGemvPieces>;
  const size_t smem = gemv_shared(K);
  static sb::DeviceOnce once;
  if (once.needed()) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kGemvMaxShared));
    once.done();
  }
  int resident = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, kWarps * 32, smem) != cudaSuccess || resident < 1) resident = 1;
  const int per_block = kWarps * kGemvFeatures;
  const int blocks = std::min((M + per_block - 1) / per_block, resident * sb::sm_count());
  sb::launch_pdl(kernel, dim3(blocks), dim3(kWarps * 32), smem, stream, static_cast<const TX*>(x), static_cast<const TW*>(w), ldw, out, M, K,
                 accumulate);
}

// Measured on a B200 with bfloat16 weights, microseconds. A feature per warp and two groups: 16384 x 2048 17.8,
// 128256 x 2048 106, 2048 x 8192 16.5. Four groups: 20.6, 155, 13.9: with few features (fewer warps than the GPU holds)
// every warp has to keep more requested; with many, more warps do better than more requests a warp. Two features a
// warp (fewer instructions a byte, half the warps): 19.2, 137, 22.8.
template <class TX, class TW>
void launch_gemv(const void* x, const void* w, int64_t ldw, float* out, int M, int K, int accumulate, cudaStream_t stream) {
  if ((M + kWarps - 1) / kWarps < 4 * sb::sm_count()) launch_gemv_groups<TX, TW, 4>(x, w, ldw, out, M, K, accumulate, stream);
  else launch_gemv_groups<TX, TW, 2>(x, w, ldw, out, M, K, accumulate, stream);
}

// The warp's tile by the number of tokens: one token is a stream over the weights with a feature per warp (the most
// warps, the most bytes in flight); a few tokens share the weights a warp reads; many tokens also share the tokens' pieces
// among four features. Every shape adds in the same order.
template <class TX, class TW, bool VEC>
void dispatch(const void* x, int64_t ldx, const void* w, int64_t ldw, float* out, int64_t ldo, int n, int M, int K, int accumulate,
              cudaStream_t stream) {
  if (!VEC) return launch<TX, TW, false, 1, 4, 1>(x, ldx, w, ldw, out, ldo, n, M, K, accumulate, stream);
  if (n == 1 && gemv_shared(K) <= kGemvMaxShared) return launch_gemv<TX, TW>(x, w, ldw, out, M, K, accumulate, stream);
  if (n == 1) return launch<TX, TW, true, 1, 1, 4>(x, ldx, w, ldw, out, ldo, n, M, K, accumulate, stream);
  if (n <= 4) return launch<TX, TW, true, 1, 4, 2>(x, ldx, w, ldw, out, ldo, n, M, K, accumulate, stream);
  if (n <= 16) return launch<TX, TW, true, 2, 8, 1>(x, ldx, w, ldw, out, ldo, n, M, K, accumulate, stream);
  return launch<TX, TW, true, 4, 8, 1>(x, ldx, w, ldw, out, ldo, n, M, K, accumulate, stream);
}

}  // namespace

// out[n, M] = x . W^T, or out += x . W^T when `accumulate` is set (the residual add).
// x_dtype, weight_dtype: 0 = float32, 1 = bfloat16 (widened exactly; the products and
// sums are float32 either way). Leading dimensions in elements.
SB_EXPORT int sb_gemm_f32(const void* x, int x_dtype, int64_t ldx, const void* w, int weight_dtype, int64_t ldw, float* out,
                          int64_t ldo, int n, int M, int K, int accumulate, cudaStream_t stream) {
  if (n <= 0 || M <= 0) return 0;
  if (K <= 0) return sb::fail("sb_gemm_f32: K must be positive");
  if (weight_dtype != 0 && weight_dtype != 1) return sb::fail("sb_gemm_f32: unsupported weight dtype %d", weight_dtype);
  if (x_dtype != 0 && x_dtype != 1) return sb::fail("sb_gemm_f32: unsupported activation dtype %d", x_dtype);
  if ((n + 7) / 8 > 65535) return sb::fail("sb_gemm_f32: %d rows exceed the grid (max %d)", n, 65535 * 8);
  const int xb = x_dtype == 0 ? 4 : 2, wb = weight_dtype == 0 ? 4 : 2;
  const bool vec = K % 8 == 0 && (ldx * xb) % 16 == 0 && (ldw * wb) % 16 == 0 &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
#define SB_F32(TX, TW)                                                                          \
  do {                                                                                          \
    if (vec) dispatch<TX, TW, true>(x, ldx, w, ldw, out, ldo, n, M, K, accumulate, stream);     \
    else dispatch<TX, TW, false>(x, ldx, w, ldw, out, ldo, n, M, K, accumulate, stream);        \
  } while (0)
  if (x_dtype == 0 && weight_dtype == 0) SB_F32(float, float);
  else if (x_dtype == 0) SB_F32(float, bf16);
  else if (weight_dtype == 0) SB_F32(bf16, float);
  else SB_F32(bf16, bf16);
#undef SB_F32
  return sb::check_launch("sb_gemm_f32");
}

// ------------------------------------------------------------------ operation of the native step program (step_ops.h)
// i: 0 x, 1 x dtype, 2 ldx, 3 weight, 4 weight dtype, 5 ldw, 6 out, 7 ldo, 8 M, 9 K, 10 accumulate,
//    11 rows: 0 = the step's tokens, 1 = the rows whose logits are wanted
SB_EXPORT int sb_op_linear_f32(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  const int n = op->i[11] ? s->wanted : s->n;
  if (n <= 0) return SB_OP_SKIPPED;
  return sb_gemm_f32(ptr<const void>(op->i[0]), (int)op->i[1], op->i[2], ptr<const void>(op->i[3]), (int)op->i[4], op->i[5],
                     ptr<float>(op->i[6]), op->i[7], n, (int)op->i[8], (int)op->i[9], (int)op->i[10], static_cast<cudaStream_t>(stream));
}
