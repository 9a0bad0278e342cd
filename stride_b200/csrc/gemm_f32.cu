// True 32-bit linear layer: out[n, M] (+)= x[n, K] . W[M, K]^T with FMA on the
// CUDA cores, no tensor cores and no reduced-precision matrix mode. Weights may be
// stored in bfloat16 (widened exactly) or in float32. Every output element is one
// chain of fused multiply-adds over k = 0 .. K-1 in ascending order, whatever the
// number of rows n, so a token's result does not depend on its batch.
//
// Counterparts in arhaamatiq/stride: gemm_partial and its users GemmResidual,
// Mlp13, LmFull of the exact path (src/kernels.cu:63-94, 294-325, 329-363, 427-452).
#include "common.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;

constexpr int TM = 64;  // rows of x (tokens) per block
constexpr int TN = 64;  // rows of W (output features) per block
constexpr int TK = 16;

template <class TX, class TW, bool ACC>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const TX* __restrict__ x, int64_t ldx,
                                                        const TW* __restrict__ w, int64_t ldw,
                                                        float* __restrict__ out, int64_t ldo, int n, int M, int K) {
  __shared__ float xs[TK][TM + 4];
  __shared__ float ws[TK][TN + 4];
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int t = threadIdx.x;
  const int row0 = blockIdx.y * TM, col0 = blockIdx.x * TN;
  const int ty = t / 16, tx = t % 16;  // 16 x 16 threads, each 4 x 4 outputs
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  const int lr = t / 4;        // 0..63: tile row loaded by this thread
  const int lk = (t % 4) * 4;  // 0,4,8,12: first k of its four
  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int xr = row0 + lr, wr = col0 + lr;
      xs[lk + e][lr] = (xr < n && k < K) ? sb::widen(x[static_cast<int64_t>(xr) * ldx + k]) : 0.0f;
      ws[lk + e][lr] = (wr < M && k < K) ? sb::widen(w[static_cast<int64_t>(wr) * ldw + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= n) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c >= M) continue;
      float* o = out + static_cast<int64_t>(r) * ldo + c;
      *o = ACC ? (*o + acc[i][j]) : acc[i][j];
    }
  }
}

// ------------------------------------------------------------------ few tokens (decode steps)
// Up to 16 tokens: the product is a stream over the weights, and the tile kernel above would leave most of the GPU idle
// (its 64 x 64 tiles give a [2048, 2048] weight 32 blocks). Here a block of 128 threads takes 32 output features:
// thread (f, g) owns feature f and tokens 4 g .. 4 g + 3, one chain of fused multiply-adds each over k = 0 .. K - 1 in
// ascending order from zero, exactly the chain of the tile kernel, so a token has the same bits from either. The
// weights' and tokens' next 64 values of k travel into registers while the current 64 are multiplied from shared memory.
constexpr int SF = 32;   // features per block
constexpr int SK = 64;   // k per round
constexpr int ST = 16;   // most tokens

constexpr int SR = 4;    // rounds of loads in flight per thread

// Eight consecutive values as they are stored, fetched in one or two 16-byte loads and widened when they are used.
template <class T>
struct Raw8;
template <>
struct Raw8<bf16> {
  uint4 raw;
  __device__ __forceinline__ void load(const bf16* p, bool ok) {
    raw = make_uint4(0, 0, 0, 0);
    if (ok) raw = *reinterpret_cast<const uint4*>(p);
  }
  __device__ __forceinline__ void set(int e, float v) {
    uint32_t* w = &raw.x;
    const uint32_t bits = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));   // exact: v was widened from bfloat16
    w[e >> 1] = (e & 1) ? ((w[e >> 1] & 0x0000FFFFu) | (bits << 16)) : ((w[e >> 1] & 0xFFFF0000u) | bits);
  }
  __device__ __forceinline__ void widen(float* v) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
};
template <>
struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p, bool ok) {
    a = make_float4(0, 0, 0, 0), b = a;
    if (ok) {
      a = *reinterpret_cast<const float4*>(p);
      b = *reinterpret_cast<const float4*>(p + 4);
    }
  }
  __device__ __forceinline__ void set(int e, float v) { (&a.x)[e] = v; }     // a and b are adjacent: e = 0 .. 7
  __device__ __forceinline__ void widen(float* v) const {
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  }
};

// VEC: rows of x and w start 16-byte aligned and K is a multiple of 8, so that eight values load at once.
template <class TX, class TW, bool ACC, bool VEC>
__global__ void __launch_bounds__(128) gemm_f32_small_kernel(const TX* __restrict__ x, int64_t ldx, const TW* __restrict__ w,
                                                              int64_t ldw, float* __restrict__ out, int64_t ldo, int n, int M, int K) {
  __shared__ float ws[SK][SF + 1];
  __shared__ __align__(16) float xs[SK][ST];     // [k][token]: a thread's four tokens are one 16-byte read
  sb::grid_launch_dependents();
  const int t = threadIdx.x;
  const int f0 = blockIdx.x * SF;
  // what this thread fetches each round: eight consecutive k of weight rows t / 8 and t / 8 + 16 and of token t / 8.
  // SR rounds are in flight at a time: a stream over the weights needs that many bytes on their way to keep HBM busy.
  const int lk = (t % 8) * 8, lr = t / 8;
  Raw8<TW> wv[SR][2];
  Raw8<TX> xv[SR];
  auto fetch_w = [&](Raw8<TW>* dst, int k0) {
    const int k = k0 + lk;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int row = f0 + lr + 16 * j;
      if (VEC) {
        dst[j].load(w + static_cast<int64_t>(row) * ldw + k, row < M && k < K);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) dst[j].set(e, (row < M && k + e < K) ? sb::widen(w[static_cast<int64_t>(row) * ldw + k + e]) : 0.0f);
      }
    }
  };
  auto fetch_x = [&](Raw8<TX>& dst, int k0) {
    const int k = k0 + lk;
    if (VEC) {
      dst.load(x + static_cast<int64_t>(lr) * ldx + k, lr < n && k < K);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) dst.set(e, (lr < n && k + e < K) ? sb::widen(x[static_cast<int64_t>(lr) * ldx + k + e]) : 0.0f);
    }
  };
  // the weights do not depend on the kernels before this one: their first rounds are requested before waiting
#pragma unroll
  for (int r = 0; r < SR; ++r) fetch_w(wv[r], r * SK);
  sb::grid_dependency_wait();
#pragma unroll
  for (int r = 0; r < SR; ++r) fetch_x(xv[r], r * SK);
  const int f = t % SF, g = t / SF;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int k0 = 0; k0 < K; k0 += SR * SK) {
#pragma unroll
    for (int r = 0; r < SR; ++r) {
      const int kk = k0 + r * SK;
      if (kk >= K) break;
      float v[8];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        wv[r][j].widen(v);
#pragma unroll
        for (int e = 0; e < 8; ++e) ws[lk + e][lr + 16 * j] = v[e];
      }
      xv[r].widen(v);
#pragma unroll
      for (int e = 0; e < 8; ++e) xs[lk + e][lr] = v[e];
      __syncthreads();
      fetch_w(wv[r], kk + SR * SK);     // (past the end: nothing is read)
      fetch_x(xv[r], kk + SR * SK);
      if (4 * g < n) {      // (a warp has one g: warps whose tokens the step does not have only help with the loads)
#pragma unroll 16
        for (int k = 0; k < SK; ++k) {
          const float b = ws[k][f];
          const float4 a = *reinterpret_cast<const float4*>(&xs[k][4 * g]);
          acc[0] = fmaf(a.x, b, acc[0]);
          acc[1] = fmaf(a.y, b, acc[1]);
          acc[2] = fmaf(a.z, b, acc[2]);
          acc[3] = fmaf(a.w, b, acc[3]);
        }
      }
      __syncthreads();
    }
  }
  const int c = f0 + f;
  if (c < M) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 4 * g + i;
      if (r < n) {
        float* o = out + static_cast<int64_t>(r) * ldo + c;
        *o = ACC ? (*o + acc[i]) : acc[i];
      }
    }
  }
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
  if (n <= ST) {
    const int xb = x_dtype == 0 ? 4 : 2, wb = weight_dtype == 0 ? 4 : 2;
    const bool vec = K % 8 == 0 && (ldx * xb) % 16 == 0 && (ldw * wb) % 16 == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
    const dim3 sgrid((M + SF - 1) / SF);
#define SB_SMALL(TX, TW, ACC, VEC)                                                                                        \
  sb::launch_pdl(gemm_f32_small_kernel<TX, TW, ACC, VEC>, sgrid, dim3(128), 0, stream, static_cast<const TX*>(x), ldx, \
                 static_cast<const TW*>(w), ldw, out, ldo, n, M, K)
#define SB_SMALL_V(TX, TW, ACC) \
  do {                          \
    if (vec) SB_SMALL(TX, TW, ACC, true); \
    else SB_SMALL(TX, TW, ACC, false);    \
  } while (0)
#define SB_SMALL_A(TX, TW)                      \
  do {                                          \
    if (accumulate) SB_SMALL_V(TX, TW, true);   \
    else SB_SMALL_V(TX, TW, false);             \
  } while (0)
    if (x_dtype == 0 && weight_dtype == 0) SB_SMALL_A(float, float);
    else if (x_dtype == 0) SB_SMALL_A(float, bf16);
    else if (weight_dtype == 0) SB_SMALL_A(bf16, float);
    else SB_SMALL_A(bf16, bf16);
#undef SB_SMALL_A
#undef SB_SMALL_V
#undef SB_SMALL
    return sb::check_launch("sb_gemm_f32");
  }
  dim3 grid((M + TN - 1) / TN, (n + TM - 1) / TM);
  if (grid.y > 65535) return sb::fail("sb_gemm_f32: %d rows exceed the grid (max %d)", n, 65535 * TM);
#define SB_GEMM(TX, TW, ACC)                                                                          \
  sb::launch_pdl(gemm_f32_kernel<TX, TW, ACC>, grid, dim3(256), 0, stream, static_cast<const TX*>(x), ldx,         \
                 static_cast<const TW*>(w), ldw, out, ldo, n, M, K)
#define SB_GEMM_W(TX)                                                     \
  do {                                                                    \
    if (weight_dtype == 0 && accumulate) SB_GEMM(TX, float, true);        \
    else if (weight_dtype == 0) SB_GEMM(TX, float, false);                \
    else if (accumulate) SB_GEMM(TX, bf16, true);                         \
    else SB_GEMM(TX, bf16, false);                                        \
  } while (0)
  if (weight_dtype != 0 && weight_dtype != 1) return sb::fail("sb_gemm_f32: unsupported weight dtype %d", weight_dtype);
  if (x_dtype == 0) SB_GEMM_W(float);
  else if (x_dtype == 1) SB_GEMM_W(bf16);
  else return sb::fail("sb_gemm_f32: unsupported activation dtype %d", x_dtype);
#undef SB_GEMM_W
#undef SB_GEMM
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
