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
  extern __shared__ float smem[];
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
