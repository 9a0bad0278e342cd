// Memory-bound kernels of the decoder that are no contraction: embedding lookup,
// rotary position encoding fused with the append to the paged cache, the SwiGLU
// product, and the row gather before the head (RMSNorm is in norm.cu). All
// arithmetic is 32-bit; only loads and stores may be bfloat16.
//
// Counterparts in arhaamatiq/stride: Embed (src/kernels.cu:98-116), the rotation
// and append at the end of Qkv
// (src/kernels.cu:247-281), the activation of Mlp13 (src/kernels.cu:359-360),
// Compact (src/kernels.cu:365-380).
#include "common.cuh"
#include "step_ops.h"

SB_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;

// ------------------------------------------------------------------ embedding
// A token id of -1 stands for "the token last sampled for this row's request": it is read from
// sampled[slots[row]], which the sampling kernels of the step before wrote, so a decode step can be launched
// before the host has seen its input token.
template <class TW>
__global__ void embed_kernel(const int32_t* __restrict__ tokens, const TW* __restrict__ table,
                             float* __restrict__ out, int H, int vocab, const int32_t* __restrict__ slots,
                             const int32_t* __restrict__ sampled) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int row = blockIdx.x;
  int tok = tokens[row];
  if (tok == -1 && sampled != nullptr) tok = sampled[slots[row]];
  const bool ok = tok >= 0 && tok < vocab;
  const TW* src = table + static_cast<int64_t>(ok ? tok : 0) * H;
  float* dst = out + static_cast<int64_t>(row) * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ok ? sb::widen(src[i]) : 0.0f;
}

__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

// ------------------------------------------------------------------ rope + append
struct RopeAppendParams {
  const float* qkv;          // [n_partials][n][(Hq + 2 Hkv) D], partials summed left to right
  int n_partials;
  int64_t partial_stride;
  const int32_t* positions;  // [n]
  const int32_t* slots;      // [n]
  const float* cos_sin;      // [max_pos][rotary_dim / 2][2]
  int rotary_dim;
  void* q_out;               // [n][Hq D]
  void* k_base;              // this layer's key plane of page 0
  const int32_t* block_table;  // [slots][max_pages]
  int max_pages;
  int page_size;
  int64_t page_stride;  // elements between pages
  int64_t v_offset;     // elements from a page's keys to its values
  int64_t head_stride;  // elements between kv heads (= page_size * D)
  int Hq, Hkv, D;
  int write_kv;
};

// One thread per (head, rotation pair) of a token; blockIdx.y walks the token's pairs.
template <class TQ, class TKV>
__global__ void rope_append_kernel(RopeAppendParams p) {
  sb::grid_launch_dependents();
  const int row = blockIdx.x;
  const int D = p.D, half = D / 2, rh = p.rotary_dim / 2;
  const int heads = p.Hq + 2 * p.Hkv;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  if (item >= heads * half) return;
  const int pos = p.positions[row];
  const int slot = p.slots[row];
  const int width = heads * D;
  const int head = item / half, j = item % half;
  int d0, d1;
  if (j < rh) {
    d0 = j;
    d1 = j + rh;
  } else {
    d0 = p.rotary_dim + 2 * (j - rh);
    d1 = d0 + 1;
  }
  const bool is_v = head >= p.Hq + p.Hkv;
  const bool rotate = j < rh && !is_v;
  float c = 1.0f, sn = 0.0f;
  if (rotate) {
    const float2 cs = *reinterpret_cast<const float2*>(p.cos_sin + (static_cast<int64_t>(pos) * rh + j) * 2);
    c = cs.x;
    sn = cs.y;
  }
  int page = 0;
  if (p.write_kv && head >= p.Hq) page = p.block_table[static_cast<int64_t>(slot) * p.max_pages + pos / p.page_size];
  // positions, slots, the block table and the cos/sin table are inputs of the step; only qkv comes from the kernel before
  sb::grid_dependency_wait();
  const float* src = p.qkv + static_cast<int64_t>(row) * width + static_cast<int64_t>(head) * D;
  // the K ranges' sums are added in ascending order; up to kInFlight of them are requested at once (each is a round
  // trip to L2, and with few tokens those are what this kernel's time consists of)
  constexpr int kInFlight = 8;
  float pa[kInFlight], pb[kInFlight];
#pragma unroll
  for (int s = 0; s < kInFlight; ++s) {
    if (s < p.n_partials) {
      pa[s] = src[s * p.partial_stride + d0];
      pb[s] = src[s * p.partial_stride + d1];
    }
  }
  float a = pa[0], b = pb[0];
#pragma unroll
  for (int s = 1; s < kInFlight; ++s) {
    if (s < p.n_partials) {
      a += pa[s];
      b += pb[s];
    }
  }
  for (int s = kInFlight; s < p.n_partials; ++s) {
    a += src[s * p.partial_stride + d0];
    b += src[s * p.partial_stride + d1];
  }
  if (rotate) {
    const float ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn));
    const float rb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn));
    a = ra;
    b = rb;
  }
  if (head < p.Hq) {
    TQ* q = static_cast<TQ*>(p.q_out) + static_cast<int64_t>(row) * p.Hq * D + static_cast<int64_t>(head) * D;
    q[d0] = sb::narrow<TQ>(a);
    q[d1] = sb::narrow<TQ>(b);
  } else if (p.write_kv) {
    const int kvh = is_v ? head - p.Hq - p.Hkv : head - p.Hq;
    TKV* dst = static_cast<TKV*>(p.k_base) + static_cast<int64_t>(page) * p.page_stride +
               static_cast<int64_t>(pos % p.page_size) * D + static_cast<int64_t>(kvh) * p.head_stride + (is_v ? p.v_offset : 0);
    dst[d0] = sb::narrow<TKV>(a);
    dst[d1] = sb::narrow<TKV>(b);
  }
}

// The common case (the whole head is rotated, D % 8 == 0): one thread per (head, four adjacent rotation pairs),
// 16-byte loads of both halves and of cos/sin, 8- or 16-byte stores. Same arithmetic as rope_append_kernel.
template <class T>
__device__ __forceinline__ void store4(T* dst, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<bf16>(bf16* dst, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 packed;
  packed.x = *reinterpret_cast<uint32_t*>(&lo);
  packed.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = packed;
}

template <class TQ, class TKV>
__global__ void rope_append_vec_kernel(RopeAppendParams p) {
  sb::grid_launch_dependents();
  const int row = blockIdx.x;
  const int D = p.D, half = D / 2, quads = half / 4;
  const int heads = p.Hq + 2 * p.Hkv;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  if (item >= heads * quads) {
    sb::grid_dependency_wait();
    return;
  }
  const int pos = p.positions[row];
  const int slot = p.slots[row];
  const int head = item / quads, j = (item % quads) * 4;
  const bool is_v = head >= p.Hq + p.Hkv;
  int page = 0;
  if (p.write_kv && head >= p.Hq) page = p.block_table[static_cast<int64_t>(slot) * p.max_pages + pos / p.page_size];
  float4 c01 = make_float4(1.0f, 0.0f, 1.0f, 0.0f), c23 = c01;   // (cos, sin) of pairs j, j+1 and j+2, j+3
  if (!is_v) {
    const float4* cs = reinterpret_cast<const float4*>(p.cos_sin + (static_cast<int64_t>(pos) * half + j) * 2);
    c01 = cs[0];
    c23 = cs[1];
  }
  sb::grid_dependency_wait();   // everything above is an input of the step; qkv comes from the kernel before
  const float* src = p.qkv + static_cast<int64_t>(row) * heads * D + static_cast<int64_t>(head) * D;
  // the K ranges' sums are added in ascending order; up to kInFlight of them are requested at once
  constexpr int kInFlight = 8;
  float4 pa[kInFlight], pb[kInFlight];
#pragma unroll
  for (int s = 0; s < kInFlight; ++s) {
    if (s < p.n_partials) {
      pa[s] = *reinterpret_cast<const float4*>(src + s * p.partial_stride + j);
      pb[s] = *reinterpret_cast<const float4*>(src + s * p.partial_stride + half + j);
    }
  }
  float4 a = pa[0], b = pb[0];
#pragma unroll
  for (int s = 1; s < kInFlight; ++s) {
    if (s < p.n_partials) {
      a = add4(a, pa[s]);
      b = add4(b, pb[s]);
    }
  }
  for (int s = kInFlight; s < p.n_partials; ++s) {
    a = add4(a, *reinterpret_cast<const float4*>(src + s * p.partial_stride + j));
    b = add4(b, *reinterpret_cast<const float4*>(src + s * p.partial_stride + half + j));
  }
  if (!is_v) {
    const float ax = a.x, ay = a.y, az = a.z, aw = a.w;
    a.x = __fsub_rn(__fmul_rn(ax, c01.x), __fmul_rn(b.x, c01.y));
    b.x = __fadd_rn(__fmul_rn(b.x, c01.x), __fmul_rn(ax, c01.y));
    a.y = __fsub_rn(__fmul_rn(ay, c01.z), __fmul_rn(b.y, c01.w));
    b.y = __fadd_rn(__fmul_rn(b.y, c01.z), __fmul_rn(ay, c01.w));
    a.z = __fsub_rn(__fmul_rn(az, c23.x), __fmul_rn(b.z, c23.y));
    b.z = __fadd_rn(__fmul_rn(b.z, c23.x), __fmul_rn(az, c23.y));
    a.w = __fsub_rn(__fmul_rn(aw, c23.z), __fmul_rn(b.w, c23.w));
    b.w = __fadd_rn(__fmul_rn(b.w, c23.z), __fmul_rn(aw, c23.w));
  }
  if (head < p.Hq) {
    TQ* q = static_cast<TQ*>(p.q_out) + static_cast<int64_t>(row) * p.Hq * D + static_cast<int64_t>(head) * D;
    store4<TQ>(q + j, a.x, a.y, a.z, a.w);
    store4<TQ>(q + half + j, b.x, b.y, b.z, b.w);
  } else if (p.write_kv) {
    const int kvh = is_v ? head - p.Hq - p.Hkv : head - p.Hq;
    TKV* dst = static_cast<TKV*>(p.k_base) + static_cast<int64_t>(page) * p.page_stride +
               static_cast<int64_t>(pos % p.page_size) * D + static_cast<int64_t>(kvh) * p.head_stride + (is_v ? p.v_offset : 0);
    store4<TKV>(dst + j, a.x, a.y, a.z, a.w);
    store4<TKV>(dst + half + j, b.x, b.y, b.z, b.w);
  }
}

// ------------------------------------------------------------------ swiglu
template <class TO>
__global__ void swiglu_kernel(const float* __restrict__ gate_up, TO* __restrict__ out, int n, int I) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int64_t total = static_cast<int64_t>(n) * I;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / I, c = i % I;
    const float a = gate_up[r * 2 * I + c], b = gate_up[r * 2 * I + I + c];
    out[i] = sb::narrow<TO>((a / (1.0f + expf(-a))) * b);
  }
}

// ------------------------------------------------------------------ gather
__global__ void gather_rows_kernel(const float* __restrict__ in, const float* __restrict__ partials, int n_partials,
                                   int64_t partial_stride, const int32_t* __restrict__ rows,
                                   float* __restrict__ out, int H) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int src = rows[blockIdx.x];
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = in[static_cast<int64_t>(src) * H + i];
    if (n_partials > 0) {
      constexpr int kInFlight = 12;     // partial sums requested at once, then added in ascending order
      const float* p = partials + static_cast<int64_t>(src) * H + i;
      float part[kInFlight];
#pragma unroll
      for (int s = 0; s < kInFlight; ++s)
        if (s < n_partials) part[s] = p[s * partial_stride];
      float sum = part[0];
#pragma unroll
      for (int s = 1; s < kInFlight; ++s)
        if (s < n_partials) sum += part[s];
      for (int s = kInFlight; s < n_partials; ++s) sum += p[s * partial_stride];
      v += sum;
    }
    out[static_cast<int64_t>(blockIdx.x) * H + i] = v;
  }
}

}  // namespace

// dtype codes shared with the Python side: 0 = float32, 1 = bfloat16.

SB_EXPORT int sb_embed(const int32_t* tokens, const void* table, int table_dtype, float* out, int n, int H, int vocab,
                       const int32_t* slots, const int32_t* sampled, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (table_dtype == 0)
    sb::launch_pdl(embed_kernel<float>, n, 256, 0, stream, tokens, static_cast<const float*>(table), out, H, vocab, slots, sampled);
  else if (table_dtype == 1)
    sb::launch_pdl(embed_kernel<bf16>, n, 256, 0, stream, tokens, static_cast<const bf16*>(table), out, H, vocab, slots, sampled);
  else
    return sb::fail("sb_embed: unsupported table dtype %d", table_dtype);
  return sb::check_launch("sb_embed");
}

SB_EXPORT int sb_rope_append(const float* qkv, int n_partials, int64_t partial_stride, const int32_t* positions,
                             const int32_t* slots, const float* cos_sin, int rotary_dim, void* q_out, int q_dtype,
                             void* k_base, int kv_dtype, const int32_t* block_table, int max_pages, int page_size,
                             int64_t page_stride, int64_t v_offset, int64_t head_stride, int n, int Hq, int Hkv, int D,
                             int write_kv, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (D % 2 != 0 || rotary_dim % 2 != 0 || rotary_dim > D || rotary_dim < 0)
    return sb::fail("sb_rope_append: head_dim %d / rotary_dim %d must be even and rotary_dim <= head_dim", D, rotary_dim);
  if (n_partials < 1) return sb::fail("sb_rope_append: n_partials must be >= 1");
  RopeAppendParams p{qkv, n_partials, partial_stride, positions, slots, cos_sin, rotary_dim, q_out, k_base,
                     block_table, max_pages, page_size, page_stride, v_offset, head_stride, Hq, Hkv, D, write_kv};
  const int threads = 128;
  const bool aligned = ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_base) |
                         reinterpret_cast<uintptr_t>(cos_sin)) & 15) == 0;
  if (rotary_dim == D && D % 8 == 0 && aligned && partial_stride % 4 == 0 && page_stride % 8 == 0 && v_offset % 8 == 0 &&
      head_stride % 8 == 0) {
    const dim3 vgrid(n, ((Hq + 2 * Hkv) * (D / 8) + threads - 1) / threads);
    if (q_dtype == 0 && kv_dtype == 0) sb::launch_pdl(rope_append_vec_kernel<float, float>, vgrid, threads, 0, stream, p);
    else if (q_dtype == 1 && kv_dtype == 1) sb::launch_pdl(rope_append_vec_kernel<bf16, bf16>, vgrid, threads, 0, stream, p);
    else if (q_dtype == 0 && kv_dtype == 1) sb::launch_pdl(rope_append_vec_kernel<float, bf16>, vgrid, threads, 0, stream, p);
    else if (q_dtype == 1 && kv_dtype == 0) sb::launch_pdl(rope_append_vec_kernel<bf16, float>, vgrid, threads, 0, stream, p);
    else return sb::fail("sb_rope_append: unsupported dtypes q=%d kv=%d", q_dtype, kv_dtype);
    return sb::check_launch("sb_rope_append");
  }
  const dim3 grid(n, ((Hq + 2 * Hkv) * (D / 2) + threads - 1) / threads);
  if (q_dtype == 0 && kv_dtype == 0) sb::launch_pdl(rope_append_kernel<float, float>, grid, threads, 0, stream, p);
  else if (q_dtype == 1 && kv_dtype == 1) sb::launch_pdl(rope_append_kernel<bf16, bf16>, grid, threads, 0, stream, p);
  else if (q_dtype == 0 && kv_dtype == 1) sb::launch_pdl(rope_append_kernel<float, bf16>, grid, threads, 0, stream, p);
  else if (q_dtype == 1 && kv_dtype == 0) sb::launch_pdl(rope_append_kernel<bf16, float>, grid, threads, 0, stream, p);
  else return sb::fail("sb_rope_append: unsupported dtypes q=%d kv=%d", q_dtype, kv_dtype);
  return sb::check_launch("sb_rope_append");
}

SB_EXPORT int sb_swiglu(const float* gate_up, void* out, int out_dtype, int n, int I, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int64_t total = static_cast<int64_t>(n) * I;
  const int blocks = static_cast<int>((total + 255) / 256 < sb::sm_count() * 16 ? (total + 255) / 256 : sb::sm_count() * 16);
  if (out_dtype == 0) sb::launch_pdl(swiglu_kernel<float>, blocks, 256, 0, stream, gate_up, static_cast<float*>(out), n, I);
  else if (out_dtype == 1) sb::launch_pdl(swiglu_kernel<bf16>, blocks, 256, 0, stream, gate_up, static_cast<bf16*>(out), n, I);
  else return sb::fail("sb_swiglu: unsupported out dtype %d", out_dtype);
  return sb::check_launch("sb_swiglu");
}

SB_EXPORT int sb_gather_rows(const float* in, const float* partials, int n_partials, int64_t partial_stride,
                             const int32_t* rows, float* out, int count, int H, cudaStream_t stream) {
  if (count <= 0) return 0;
  sb::launch_pdl(gather_rows_kernel, count, 256, 0, stream, in, partials, n_partials, partial_stride, rows, out, H);
  return sb::check_launch("sb_gather_rows");
}

// ------------------------------------------------------------------ operations of the native step program (step_ops.h)
// i: 0 table, 1 table dtype, 2 out (float32 [n, H]), 3 H, 4 vocab, 5 the table of last sampled tokens (or 0)
SB_EXPORT int sb_op_embed(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  const int32_t* sampled = ptr<const int32_t>(op->i[5]);
  return sb_embed(tokens(s), ptr<const void>(op->i[0]), (int)op->i[1], ptr<float>(op->i[2]), s->n, (int)op->i[3], (int)op->i[4],
                  sampled ? slots(s) : nullptr, sampled, static_cast<cudaStream_t>(stream));
}

// i: 0 qkv partial sums (flat), 1 their width, 2 K ranges S, 3 most tokens with a buffer per range, 4 cos_sin, 5 rotary_dim,
//    6 q_out, 7 q dtype, 8 cache layer, 9 cache dtype, 10 block table, 11 pages per sequence, 12 page size,
//    13 page stride, 14 v offset, 15 head stride, 16 Hq, 17 Hkv, 18 D, 19 write_kv, 20 tile plan (-1: none)
SB_EXPORT int sb_op_rope_append(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (op->i[20] >= 0 && s->plan[op->i[20]].fused) return SB_OP_SKIPPED;     // the decode kernel rotates and appends itself
  const int P = partial_count(op->i[2], op->i[3], s->n);
  return sb_rope_append(ptr<const float>(op->i[0]), P, static_cast<int64_t>(s->n) * op->i[1], positions(s), slots(s),
                        ptr<const float>(op->i[4]), (int)op->i[5], ptr<void>(op->i[6]), (int)op->i[7], ptr<void>(op->i[8]), (int)op->i[9],
                        ptr<const int32_t>(op->i[10]), (int)op->i[11], (int)op->i[12], op->i[13], op->i[14], op->i[15], s->n,
                        (int)op->i[16], (int)op->i[17], (int)op->i[18], (int)op->i[19], static_cast<cudaStream_t>(stream));
}

// i: 0 gate_up (float32 [n, 2 I]), 1 out, 2 out dtype, 3 I
SB_EXPORT int sb_op_swiglu(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  return sb_swiglu(ptr<const float>(op->i[0]), ptr<void>(op->i[1]), (int)op->i[2], s->n, (int)op->i[3], static_cast<cudaStream_t>(stream));
}

// The rows whose logits are wanted, with the pending partial sums of the last projection added.
// i: 0 h, 1 pending partial sums (flat; 0: none), 2 K ranges S, 3 most tokens with a buffer per range, 4 out, 5 H
SB_EXPORT int sb_op_gather_rows(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  if (s->wanted <= 0) return SB_OP_SKIPPED;
  const float* partials = ptr<const float>(op->i[1]);
  const int P = partials ? partial_count(op->i[2], op->i[3], s->n) : 0;
  return sb_gather_rows(ptr<const float>(op->i[0]), partials, P, static_cast<int64_t>(s->n) * op->i[5], wanted_rows(s), ptr<float>(op->i[4]),
                        s->wanted, (int)op->i[5], static_cast<cudaStream_t>(stream));
}
