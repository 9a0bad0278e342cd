// RMSNorm, fused with the reduction of split-K partial sums into the residual. All arithmetic is
// 32-bit; only the gain and the normed values may be bfloat16.
//
// Counterpart in arhaamatiq/stride: RmsNorm (src/kernels.cu:119-200).
#include "common.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;
constexpr int kRowsKernelMin = 1536;   // more rows than this, and no partial sums: the warp-per-row kernel

// ------------------------------------------------------------------ rmsnorm
// One block per row. The row is h + (partial_0 + partial_1 + ...), the partials summed left to
// right first (as the tensor-core kernel adds its K ranges when it does so itself) and then added
// to h; when partials are given the sum is written back to h. Then
// r = 1/sqrt(sum(x^2)/H + eps) and out = w * (x * r). VEC = 4 reads float4 (H % 4 == 0);
// the partials are fetched four at a time so that their loads overlap.
template <int VEC>
struct VecF;
template <>
struct VecF<4> { using type = float4; };
template <>
struct VecF<1> { using type = float; };

__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float add4(float a, float b) { return a + b; }

template <class TW, class TO, int VEC, int MAXT>     // MAXT: the most threads of a block (1024, or 512 with more registers each)
__global__ void __launch_bounds__(MAXT) rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ partials, int n_partials,
                               int64_t partial_stride, const TW* __restrict__ weight, TO* __restrict__ out,
                               int H, float eps) {
  using V = typename VecF<VEC>::type;
  extern __shared__ __align__(16) float row[];
  __shared__ float red[32];
  sb::grid_launch_dependents();
  const int r = blockIdx.x;
  const int units = H / VEC;
  // The gain does not depend on the kernels before this one: fetch this thread's first piece of it before waiting.
  float w_first[VEC];
  if (threadIdx.x < units) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) w_first[e] = sb::widen(weight[threadIdx.x * VEC + e]);
  }
  sb::grid_dependency_wait();
  V* hr = reinterpret_cast<V*>(h + static_cast<int64_t>(r) * H);
  float ss = 0.0f;
  for (int i = threadIdx.x; i < units; i += blockDim.x) {
    V v = hr[i];
    if (n_partials > 0) {
      // up to kInFlight partial sums are requested at once (every load of a few tokens' row is a round trip to L2,
      // and they are what this kernel's time consists of), then added left to right
      constexpr int kInFlight = MAXT > 512 ? 8 : 12;
      const V* p = reinterpret_cast<const V*>(partials + static_cast<int64_t>(r) * H) + i;
      const int64_t ps = partial_stride / VEC;
      V part[kInFlight];
#pragma unroll
      for (int s = 0; s < kInFlight; ++s)
        if (s < n_partials) part[s] = p[s * ps];
      V sum = part[0];
#pragma unroll
      for (int s = 1; s < kInFlight; ++s)
        if (s < n_partials) sum = add4(sum, part[s]);
      for (int s = kInFlight; s < n_partials; ++s) sum = add4(sum, p[s * ps]);
      v = add4(v, sum);
      hr[i] = v;
    }
    reinterpret_cast<V*>(row)[i] = v;
    if constexpr (VEC == 4) {
      ss = fmaf(v.x, v.x, ss);
      ss = fmaf(v.y, v.y, ss);
      ss = fmaf(v.z, v.z, ss);
      ss = fmaf(v.w, v.w, ss);
    } else {
      ss = fmaf(v, v, ss);
    }
  }
  const float total = sb::block_sum(ss, red);
  const float scale = 1.0f / sqrtf(total / static_cast<float>(H) + eps);
  TO* o = out + static_cast<int64_t>(r) * H;
  for (int i = threadIdx.x; i < units; i += blockDim.x) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float w = i == static_cast<int>(threadIdx.x) ? w_first[e] : sb::widen(weight[i * VEC + e]);
      o[i * VEC + e] = sb::narrow<TO>(w * (row[i * VEC + e] * scale));
    }
  }
}

// Many rows (a prompt portion): one warp per row, two rows per block (small blocks spread evenly over the SMs), no shared memory and no block barrier.
// Pass 1 folds the partials (written back to h) and sums the squares; pass 2 re-reads the row (it is in L2) and
// writes the normed values. H % 4 == 0. The squares are added in the order of rmsnorm_kernel with 32 W threads, so
// that a row's result has the same bits whichever kernel the size of the step selects: lane l stands for that
// kernel's threads l, l + 32, .., one chain of fused multiply-adds each, the 32 chains of a warp are combined by
// xor shuffles and the W warps' sums are added in ascending order.
// JT > 0: the row has at most JT rounds of 32 W pieces and stays in registers between the passes; 0: any width,
// pass 2 re-reads it.
// Four gains from element i of a bfloat16 or float32 vector (the widening is exact).
__device__ __forceinline__ float4 load_gain4(const void* w, bool is_bf16, int i) {
  if (is_bf16) {
    const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const bf16*>(w) + i);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  return *reinterpret_cast<const float4*>(static_cast<const float*>(w) + i);
}
template <class TO>
__device__ __forceinline__ void store_normed4(TO* o, float4 v, float4 w, float scale) {
  if constexpr (sizeof(TO) == 2) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(w.x * (v.x * scale), w.y * (v.y * scale));
    __nv_bfloat162 hi = __floats2bfloat162_rn(w.z * (v.z * scale), w.w * (v.w * scale));
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(o) = packed;
  } else {
    *reinterpret_cast<float4*>(o) = make_float4(w.x * (v.x * scale), w.y * (v.y * scale), w.z * (v.z * scale), w.w * (v.w * scale));
  }
}

template <class TO, int W, int JT>
__global__ void __launch_bounds__(64) rmsnorm_rows_kernel(float* __restrict__ h, const float* __restrict__ partials,
                                                           int n_partials, int64_t partial_stride,
                                                           const void* __restrict__ weight, bool weight_bf16,
                                                           TO* __restrict__ out, int n, int H, float eps) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int r = blockIdx.x * 2 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n) return;
  float4* hr = reinterpret_cast<float4*>(h + static_cast<int64_t>(r) * H);
  const int units = H / 4;
  const int64_t ps = partial_stride / 4;
  float chain[W];
  float4 keep[JT > 0 ? JT * W : 1];
#pragma unroll
  for (int w = 0; w < W; ++w) chain[w] = 0.0f;
  auto round = [&](int i0, int jt) {
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const int i = i0 + 32 * w + lane;
      if (i < units) {
        float4 v = hr[i];
        if (n_partials > 0) {
          const float4* p = reinterpret_cast<const float4*>(partials + static_cast<int64_t>(r) * H) + i;
          float4 sum = p[0];
          for (int s = 1; s < n_partials; ++s) sum = add4(sum, p[s * ps]);
          v = add4(v, sum);
          hr[i] = v;
        }
        if (JT > 0) keep[jt * W + w] = v;
        chain[w] = fmaf(v.x, v.x, chain[w]);
        chain[w] = fmaf(v.y, v.y, chain[w]);
        chain[w] = fmaf(v.z, v.z, chain[w]);
        chain[w] = fmaf(v.w, v.w, chain[w]);
      }
    }
  };
  if constexpr (JT > 0) {
#pragma unroll
    for (int jt = 0; jt < JT; ++jt) round(jt * 32 * W, jt);
  } else {
    for (int i0 = 0; i0 < units; i0 += 32 * W) round(i0, 0);
  }
  float ss = 0.0f;
#pragma unroll
  for (int w = 0; w < W; ++w) {
    float c = chain[w];
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    ss = w == 0 ? c : ss + c;
  }
  const float scale = 1.0f / sqrtf(ss / static_cast<float>(H) + eps);
  TO* o = out + static_cast<int64_t>(r) * H;
  if constexpr (JT > 0) {
#pragma unroll
    for (int jt = 0; jt < JT; ++jt)
#pragma unroll
      for (int w = 0; w < W; ++w) {
        const int i = jt * 32 * W + 32 * w + lane;
        if (i < units) store_normed4<TO>(o + 4 * i, keep[jt * W + w], load_gain4(weight, weight_bf16, 4 * i), scale);
      }
  } else {
    for (int i = lane; i < units; i += 32) store_normed4<TO>(o + 4 * i, hr[i], load_gain4(weight, weight_bf16, 4 * i), scale);
  }
}

}  // namespace

// dtype codes shared with the Python side: 0 = float32, 1 = bfloat16.
SB_EXPORT int sb_rmsnorm(float* h, const float* partials, int n_partials, int64_t partial_stride, const void* weight,
                         int weight_dtype, void* out, int out_dtype, int n, int H, float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  const size_t smem = static_cast<size_t>(H) * sizeof(float);
  if (smem > 200 * 1024) return sb::fail("sb_rmsnorm: width %d does not fit the row buffer (max 51200)", H);
  const bool vec = H % 4 == 0 && partial_stride % 4 == 0 && ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(partials)) & 15) == 0;
  const int units = vec ? H / 4 : H;
  const int threads = units >= 1024 ? 1024 : units >= 512 ? 512 : units >= 256 ? 256 : 128;
  // (a block per row is the faster of the two up to about 1,500 rows, and whenever partial sums are to be added:
  // measured at H = 2048, 256 rows: 2.9 us against 9.7 us; 2,048 rows: 19.4 against 18.7)
  if (vec && n > kRowsKernelMin && n_partials <= 1 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(weight)) & 15) == 0) {
    // the warp-per-row kernel adds the squares in the order of the block-per-row kernel with `threads` threads
    const dim3 grid((n + 1) / 2);
#define SB_ROWS_J(TO, W, JT) \
  sb::launch_pdl(rmsnorm_rows_kernel<TO, W, JT>, grid, dim3(64), 0, stream, h, partials, n_partials, partial_stride, \
                 weight, weight_dtype == 1, static_cast<TO*>(out), n, H, eps)
  // the row stays in registers between the passes while it has at most 16 pieces a lane; wider rows are read again from
  // L2 in the second pass (measured: 32 pieces in registers leave too few warps an SM: width 4096 58 -> 38 us for 2,048
  // rows, width 3072 48 -> 30; at width 2048, 16 pieces, registers are the faster way, 17 us against 21)
#define SB_ROWS(TO)                                                      \
  do {                                                                   \
    if (threads == 1024) SB_ROWS_J(TO, 32, 0);                           \
    else if (threads == 512 && units <= 512) SB_ROWS_J(TO, 16, 1);   \
    else if (threads == 512) SB_ROWS_J(TO, 16, 0);                   \
    else if (threads == 256 && units <= 256) SB_ROWS_J(TO, 8, 1);    \
    else if (threads == 256) SB_ROWS_J(TO, 8, 2);                    \
    else if (units <= 128) SB_ROWS_J(TO, 4, 1);                      \
    else SB_ROWS_J(TO, 4, 2);                                        \
  } while (0)
    if ((weight_dtype != 0 && weight_dtype != 1) || (out_dtype != 0 && out_dtype != 1))
      return sb::fail("sb_rmsnorm: unsupported dtypes weight=%d out=%d", weight_dtype, out_dtype);
    if (out_dtype == 0) SB_ROWS(float);
    else SB_ROWS(bf16);
#undef SB_ROWS
#undef SB_ROWS_J
    return sb::check_launch("sb_rmsnorm");
  }
#define SB_NORM_V(TW, TO, VEC)                                                                                   \
  do {                                                                                                           \
    if (threads > 512) {                                                                                         \
      if (smem > 48 * 1024)                                                                                      \
        cudaFuncSetAttribute(rmsnorm_kernel<TW, TO, VEC, 1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      sb::launch_pdl(rmsnorm_kernel<TW, TO, VEC, 1024>, n, threads, smem, stream, h, partials, n_partials, partial_stride, \
                     static_cast<const TW*>(weight), static_cast<TO*>(out), H, eps);                            \
    } else {                                                                                                     \
      if (smem > 48 * 1024)                                                                                      \
        cudaFuncSetAttribute(rmsnorm_kernel<TW, TO, VEC, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      sb::launch_pdl(rmsnorm_kernel<TW, TO, VEC, 512>, n, threads, smem, stream, h, partials, n_partials, partial_stride, \
                     static_cast<const TW*>(weight), static_cast<TO*>(out), H, eps);                            \
    }                                                                                                            \
  } while (0)
#define SB_NORM(TW, TO)          \
  do {                           \
    if (vec) SB_NORM_V(TW, TO, 4); \
    else SB_NORM_V(TW, TO, 1);   \
  } while (0)
  if (weight_dtype == 0 && out_dtype == 0) SB_NORM(float, float);
  else if (weight_dtype == 0 && out_dtype == 1) SB_NORM(float, bf16);
  else if (weight_dtype == 1 && out_dtype == 0) SB_NORM(bf16, float);
  else if (weight_dtype == 1 && out_dtype == 1) SB_NORM(bf16, bf16);
  else return sb::fail("sb_rmsnorm: unsupported dtypes weight=%d out=%d", weight_dtype, out_dtype);
#undef SB_NORM
#undef SB_NORM_V
  return sb::check_launch("sb_rmsnorm");
}

// ------------------------------------------------------------------ operation of the native step program (step_ops.h)
// i: 0 h, 1 pending partial sums (flat; 0: none), 2 K ranges S, 3 most tokens with a buffer per range, 4 weight,
//    5 weight dtype, 6 out, 7 out dtype, 8 H, 9 rows: 0 = the step's tokens, 1 = the rows whose logits are wanted
// f: 0 eps
SB_EXPORT int sb_op_rmsnorm(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  const int n = op->i[9] ? s->wanted : s->n;
  if (n <= 0) return SB_OP_SKIPPED;
  const float* partials = ptr<const float>(op->i[1]);
  const int P = partials ? partial_count(op->i[2], op->i[3], n) : 0;
  return sb_rmsnorm(ptr<float>(op->i[0]), partials, P, static_cast<int64_t>(n) * op->i[8], ptr<const void>(op->i[4]), (int)op->i[5],
                    ptr<void>(op->i[6]), (int)op->i[7], n, (int)op->i[8], static_cast<float>(op->f[0]), static_cast<cudaStream_t>(stream));
}
