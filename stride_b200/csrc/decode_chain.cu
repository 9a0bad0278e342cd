// The layers of a decode step as ONE persistent kernel (bfloat16 path, sm_100a).
//
// A step of a few decoded tokens is a chain of short dependent kernels (seven a layer: norm, q|k|v, attention, output
// projection, norm, gate|up, down), each of which reads its weights only after the kernel in front of it has ended. Here
// one CTA per SM lives through all layers of the step and walks the same chain as a list of phases:
//
// * one thread streams this CTA's weight tiles of ALL phases, in the order of their use, through a ring of shared-memory
//   stages with TMA. Weights depend on nothing the step computes, so the stream runs ahead of the phases as far as the
//   ring reaches and HBM stays busy while the few microseconds of dependent work of a phase run;
// * one thread streams the token tiles of a phase (what the phase in front wrote) once that phase is complete;
// * one thread issues tcgen05.mma, accumulating in tensor memory; four warps are the phase's workers: the epilogue of a
//   linear layer, the rows of a norm, the (entry, key/value head, chunk) units of attention.
//
// Phases are ordered by one counter in global memory: every CTA adds one when its share of a phase is written, and a
// phase's readers wait until the counter shows that all CTAs have finished the phase in front. All waits are bounded
// (tc5.cuh): a lost signal ends the kernel within about a second with a code in the status word.
//
// Every phase does the arithmetic of the kernel it stands for, operation by operation: the K ranges of a weight
// (sb_gemm_tc_splits), tcgen05.mma with the same instruction shape and order over K, partial sums added in ascending
// order by their reader, the sum of squares of a norm in the order of rmsnorm_kernel, attention by attention_tc.cuh's
// decode_unit. A token's logits therefore have the same bits as from the separate kernels.
//
// Counterpart in arhaamatiq/stride: the launch sequence of Engine::step_tensor_core (src/engine.cpp:300-462).
#include "attention_tc.cuh"
#include "gemm_tc_tile.cuh"
#include "step_ops.h"

#include <cstring>
#include <string>

SB_DEFINE_LAST_ERROR()

namespace {

using namespace sb::gemm_tile;   // and sb::tc5
namespace at = sb::attn_tc;
using sb::tc5::smem_u32;

enum PhaseKind { kPhaseNorm = 0, kPhaseLinear = 1, kPhaseAttention = 2 };

constexpr int kChainThreads = 224;       // warp 0: weights, warp 1: MMA, warps 2-5: workers, warp 6: token tiles
constexpr int kWorkerBarrier = 1;        // named barrier of the 128 worker threads
constexpr int kMaxStages = 12;
constexpr int kMaxTokens = 64;           // a step of more tokens runs as separate kernels
constexpr int kSmemLimit = 227 * 1024;

struct Phase {
  int32_t kind;
  // linear layer: out = x . W^T in the weight's K ranges
  int32_t swiglu;            // 0: float32 partial sums [splits][n][M]; 1: bfloat16 silu(gate) * up [n][half_rows]
  int32_t M, K, kblocks_per_split, tiles_m, splits, half_rows;
  int32_t map_w;             // index of the weight's tensor map
  int32_t map_x;             // index of the first of the token operand's three maps (token tiles of 16, 32, 64 rows)
  // norm: h += sum of pending partial sums; x = gain * (h * r)
  int32_t H, n_partials, gain_bf16;
  float eps;
  // attention
  int32_t attention;         // index into the attention parameters
  int32_t reserved;
  int64_t out;               // linear: the output; norm: x (bfloat16 [n][H])
  int64_t h, partials, gain; // norm
};

struct ChainParams {
  const Phase* phases;
  int n_phases;
  const CUtensorMap* maps;
  const at::AttnTcParams* attention;   // per attention phase: what does not change from step to step
  int n;                   // tokens of the step
  int bn_log;              // token tile: 16 << bn_log
  int items, chunks;       // decode entries of the step and the 256-key chunks the longest spans
  const int32_t* meta;     // the step's entry records [4][meta_stride]
  int meta_stride;
  const int32_t* work;     // [items] entries
  float* scratch;          // the attention units' chunk records
  unsigned* sync;          // [0] arrivals of all phases so far, [1] CTAs that have left; both zero between launches
  int* status;
  int w_stages;            // stages of the ring (a weight tile and a token tile each)
  unsigned long long* trace;   // null, or [2][phases][CTAs][4] nanoseconds of every CTA's workers and MMA issuer (sb_chain_trace)
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// (release at GPU scope: what this CTA's workers wrote before their barrier is visible to whoever sees the count)
__device__ __forceinline__ void arrive_release(unsigned* p) {
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
// Bounded wait until *counter >= target (one thread). False after about a second, with `code` in the status word, or at
// once when another wait of the launch has given up.
__device__ __forceinline__ bool wait_count(const unsigned* counter, unsigned target, int* status, int code) {
  if (ld_acquire(counter) >= target) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (ld_acquire(counter) < target) {
    if ((++spins & 63) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (clock64() - t0 > kWaitCycles) {
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync %0, 128;" ::"n"(kWorkerBarrier) : "memory"); }
// What a phase's reader does between seeing the phase in front complete and reading its output with TMA: the writes
// were made with ordinary stores on other SMs.
__device__ __forceinline__ void fence_generic_to_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ Phase load_phase(const Phase* p) {
  Phase f;
  const int4* src = reinterpret_cast<const int4*>(p);
  int4* dst = reinterpret_cast<int4*>(&f);
  static_assert(sizeof(Phase) % 16 == 0, "phases are copied in 16-byte pieces");
#pragma unroll
  for (int i = 0; i < static_cast<int>(sizeof(Phase) / 16); ++i) dst[i] = __ldg(src + i);
  return f;
}

// The workers' view of the chain for attention_tc.cuh's decode_unit: the 128 workers meet on their named barrier, and
// the unit's inputs are there once the phase in front is complete.
struct ChainEnv {
  static constexpr bool kFoldAhead = false;
  const unsigned* counter;
  unsigned target;
  int* status;
  int wtid;
  bool waited;
  __device__ __forceinline__ void sync() { worker_sync(); }
  __device__ __forceinline__ void wait_inputs() {
    if (waited) return;
    if (wtid == 0) wait_count(counter, target, status, 24);
    worker_sync();
    waited = true;
  }
};

// One row of a norm by the 128 workers, with the arithmetic of rmsnorm_kernel (norm.cu): every element is
// h + (p0 + p1 + ...), the partial sums added left to right; the squares are added in the order of that kernel with T
// threads, T = 1024, 512, 256 or 128 by the row's width as there: worker u stands for its threads u, u + 128, ..: one
// chain of fused multiply-adds over pieces t, t + T, .. each; the chains of a warp of that kernel are added by xor
// shuffles, the warps' sums left to right. Which worker adds up which element does not matter to the bits, so the
// fold takes two pieces a round with all their loads in flight at once.
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ void norm_row(const Phase& f, int r, int n, float* row, float* red, int wtid) {
  constexpr int kInFlight = 9;
  const int units = f.H / 4;
  const int T = units >= 1024 ? 1024 : units >= 512 ? 512 : units >= 256 ? 256 : 128;
  float4* hr = reinterpret_cast<float4*>(reinterpret_cast<float*>(f.h) + static_cast<int64_t>(r) * f.H);
  const float4* part = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(f.partials) + static_cast<int64_t>(r) * f.H);
  const int64_t ps = static_cast<int64_t>(n) * f.H / 4;
  const int lane = wtid & 31, w4 = wtid >> 5;
  for (int i = wtid; i < units; i += 256) {
    const int i2 = i + 128;
    const bool two = i2 < units;
    float4 va = hr[i], vb = two ? hr[i2] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (f.n_partials > 0) {
      float4 pa[kInFlight], pb[kInFlight];
#pragma unroll
      for (int k = 0; k < kInFlight; ++k) {
        if (k < f.n_partials) {
          pa[k] = __ldcg(part + i + k * ps);
          if (two) pb[k] = __ldcg(part + i2 + k * ps);
        }
      }
      float4 sa = pa[0], sb = pb[0];
#pragma unroll
      for (int k = 1; k < kInFlight; ++k) {
        if (k < f.n_partials) {
          sa = add4(sa, pa[k]);
          if (two) sb = add4(sb, pb[k]);
        }
      }
      for (int k = kInFlight; k < f.n_partials; ++k) {
        sa = add4(sa, __ldcg(part + i + k * ps));
        if (two) sb = add4(sb, __ldcg(part + i2 + k * ps));
      }
      va = add4(va, sa);
      hr[i] = va;
      if (two) {
        vb = add4(vb, sb);
        hr[i2] = vb;
      }
    }
    reinterpret_cast<float4*>(row)[i] = va;
    if (two) reinterpret_cast<float4*>(row)[i2] = vb;
  }
  worker_sync();
  for (int j = 0; j < T / 128; ++j) {
    const int t = wtid + 128 * j;
    float ss = 0.0f;
    for (int i = t; i < units; i += T) {
      const float4 v = reinterpret_cast<const float4*>(row)[i];
      ss = fmaf(v.x, v.x, ss);
      ss = fmaf(v.y, v.y, ss);
      ss = fmaf(v.z, v.z, ss);
      ss = fmaf(v.w, v.w, ss);
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[w4 + 4 * j] = ss;      // that kernel's warp t / 32
  }
  worker_sync();
  float total = red[0];
  for (int i = 1; i < T / 32; ++i) total += red[i];
  const float scale = 1.0f / sqrtf(total / static_cast<float>(f.H) + f.eps);
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(f.out) + static_cast<int64_t>(r) * f.H;
  for (int i = wtid; i < units; i += 128) {
    const float4 v = reinterpret_cast<const float4*>(row)[i];
    float4 w;
    if (f.gain_bf16) {
      const uint2 raw = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(f.gain) + 4 * i));
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      w = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    } else {
      w = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(f.gain) + 4 * i));
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(w.x * (v.x * scale), w.y * (v.y * scale));
    __nv_bfloat162 hi = __floats2bfloat162_rn(w.z * (v.z * scale), w.w * (v.w * scale));
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(o + 4 * i) = packed;
  }
  worker_sync();     // row and red are free again
}

// Walks the weight tiles of one CTA in the order of their use: all linear phases, this CTA's tiles of each, their K steps.
struct WeightCursor {
  const ChainParams& p;
  const int cta, G;
  int ph, t, tiles, kb, kb1;
  int kblocks, per_split, tiles_m, half_rows;
  bool valid, swiglu;
  const CUtensorMap* map;
  int k, row_w, row_up;
  __device__ __forceinline__ WeightCursor(const ChainParams& p_, int cta_, int G_) : p(p_), cta(cta_), G(G_), ph(-1), t(0), tiles(0), kb(0), kb1(0), valid(true) {
    next();
  }
  __device__ __forceinline__ void set_tile() {
    const int tile_m = t % tiles_m, split = t / tiles_m;
    kb = split * per_split;
    kb1 = min(kblocks, kb + per_split);
    row_w = swiglu ? tile_m * 64 : tile_m * kTileM;
    row_up = half_rows + row_w;
  }
  __device__ __forceinline__ void next() {
    if (ph >= 0 && ++kb < kb1) {
      k = kb * kTileK;
      return;
    }
    if (ph >= 0 && (t += G) < tiles) {
      set_tile();
      k = kb * kTileK;
      return;
    }
    for (++ph; ph < p.n_phases; ++ph) {
      const Phase f = load_phase(p.phases + ph);
      if (f.kind != kPhaseLinear || cta >= f.tiles_m * f.splits) continue;
      tiles = f.tiles_m * f.splits;
      t = cta;
      swiglu = f.swiglu != 0;
      kblocks = (f.K + kTileK - 1) / kTileK;
      per_split = f.kblocks_per_split, tiles_m = f.tiles_m, half_rows = f.half_rows;
      map = p.maps + f.map_w;
      set_tile();
      k = kb * kTileK;
      return;
    }
    valid = false;
  }
};

// Shared memory: [weight ring][token ring][SwiGLU exchange 4 KB][attention tiles | a norm's row]
template <int D>
__global__ void __launch_bounds__(kChainThreads, 1) decode_chain_kernel(const ChainParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t ring_full[kMaxStages], ring_empty[kMaxStages];
  __shared__ __align__(8) uint64_t acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int is_last_s;
  __shared__ float red_s[32];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  const int BN = 16 << p.bn_log;
  const int x_stage = BN * 128;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base = smem_raw + (smem0 - smem_u32(smem_raw));
  const uint32_t w_ring = smem0, x_ring = smem0 + p.w_stages * kStageA;
  float* xch = reinterpret_cast<float*>(base + p.w_stages * (kStageA + x_stage));
  uint8_t* work_smem = reinterpret_cast<uint8_t*>(xch) + 4096;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.w_stages; ++s) {
      mbar_init(smem_u32(&ring_full[s]), 2);      // the weight tile's producer and the token tile's
      mbar_init(smem_u32(&ring_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&acc_full[b]), 1);
      mbar_init(smem_u32(&acc_empty[b]), 1);
    }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_s), 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  sb::grid_launch_dependents();

  // One ring of stages for both operands: stage s holds a weight tile (16 KB) and the token tile of the same K step;
  // full[s] completes when both have landed (two producers, one arrival each), empty[s] when the products that read
  // them are done. The three loops below walk the same K steps in the same order and keep the stage and its parity
  // by counting, so that an iteration is a few dozen instructions: the issuing thread's own instructions bound a K step
  // of so few tokens.
  const uint32_t full0 = smem_u32(&ring_full[0]), empty0 = smem_u32(&ring_empty[0]);
  const int S = p.w_stages;
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- the weight stream: every tile of every linear phase that this CTA computes, in order.
      // (Asking tiles into L2 ahead of the ring with cp.async.bulk.prefetch.tensor, so that HBM would stream on while
      // the ring is full, made the large products slower, not faster: 14.3 -> 17.7 us for gate|up at 24 K steps ahead.)
      uint32_t s = 0, par = 1;        // (a wait on parity 1 of a fresh barrier returns at once: the first round is free)
      for (WeightCursor load(p, cta, G); load.valid; load.next()) {
        mbar_wait(empty0 + 8 * s, par, p.status, 21);
        const uint32_t bar = full0 + 8 * s, a = w_ring + s * kStageA;
        mbar_expect_tx(bar, kStageA);
        tma_load_2d(a, load.map, bar, load.k, load.row_w);
        if (load.swiglu) tma_load_2d(a + kStageA / 2, load.map, bar, load.k, load.row_up);
        if (++s == S) s = 0, par ^= 1;
      }
    }
  } else if (warp == 6) {
    if (lane == 0) {
      // ---------------- the token tiles of a phase, once the phase in front is complete
      sb::grid_dependency_wait();
      uint32_t s = 0, par = 1;
      for (int ph = 0; ph < p.n_phases; ++ph) {
        const Phase f = load_phase(p.phases + ph);
        if (f.kind != kPhaseLinear || cta >= f.tiles_m * f.splits) continue;
        if (ph > 0) wait_count(p.sync, static_cast<unsigned>(ph) * G, p.status, 22);
        fence_generic_to_async();
        const CUtensorMap* map = p.maps + f.map_x + p.bn_log;
        const int kblocks = (f.K + kTileK - 1) / kTileK;
        for (int t = cta; t < f.tiles_m * f.splits; t += G) {
          const int split = t / f.tiles_m;
          const int kb0 = split * f.kblocks_per_split, kb1 = min(kblocks, kb0 + f.kblocks_per_split);
          for (int k = kb0 * kTileK; k < kb1 * kTileK; k += kTileK) {
            mbar_wait(empty0 + 8 * s, par, p.status, 23);
            const uint32_t bar = full0 + 8 * s;
            mbar_expect_tx(bar, x_stage);
            tma_load_2d(x_ring + s * x_stage, map, bar, k, 0);
            if (++s == S) s = 0, par ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer
      const uint32_t idesc = sb::tc5::instr_desc(kTileM, BN, false);
      const uint64_t desc_fixed = smem_desc_sw128(0);
      const uint32_t w_lo = (w_ring & 0x3FFFF) >> 4, x_lo = (x_ring & 0x3FFFF) >> 4, x_step = x_stage >> 4;
      uint32_t s = 0, par = 0;
      int tile = 0;
      for (int ph = 0; ph < p.n_phases; ++ph) {
        const Phase f = load_phase(p.phases + ph);
        if (f.kind != kPhaseLinear) continue;
        const int kblocks = (f.K + kTileK - 1) / kTileK;
        for (int t = cta; t < f.tiles_m * f.splits; t += G, ++tile) {
          const int split = t / f.tiles_m;
          const int kb0 = split * f.kblocks_per_split, kb1 = min(kblocks, kb0 + f.kblocks_per_split);
          const int b = tile & 1;
          mbar_wait(smem_u32(&acc_empty[b]), ((tile >> 1) & 1) ^ 1, p.status, 25);
          tc_fence_after();
          const uint32_t acc = tmem_base + b * 64;
          unsigned long long waited = 0, first = 0;
          uint32_t accumulate = 0;
          for (int kb = kb0; kb < kb1; ++kb) {
            if (p.trace == nullptr) {
              mbar_wait(full0 + 8 * s, par, p.status, 26);
            } else {
              const unsigned long long ta = global_ns();
              mbar_wait(full0 + 8 * s, par, p.status, 26);
              const unsigned long long tb = global_ns();
              waited += tb - ta;
              if (kb == kb0) first = tb;
            }
            tc_fence_after();
            const uint64_t da = desc_fixed | (w_lo + s * (kStageA >> 4)), db = desc_fixed | (x_lo + s * x_step);
            umma_bf16(acc, da, db, idesc, accumulate);
            umma_bf16(acc, da + 2, db + 2, idesc, 1u);      // 16 elements = 32 bytes along K: +2 in 16-byte units
            umma_bf16(acc, da + 4, db + 4, idesc, 1u);
            umma_bf16(acc, da + 6, db + 6, idesc, 1u);
            accumulate = 1u;
            umma_commit(empty0 + 8 * s);
            if (++s == S) s = 0, par ^= 1;
          }
          umma_commit(smem_u32(&acc_full[b]));
          if (p.trace && t == cta) {
            unsigned long long* m = p.trace + (static_cast<int64_t>(p.n_phases + ph) * G + cta) * 4;
            m[0] = first, m[1] = waited, m[2] = 0, m[3] = global_ns();
          }
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- workers: warps 2..5, TMEM lanes 32 * (warp % 4) ..
    const int wtid = threadIdx.x - 64, quarter = warp & 3;
    sb::grid_dependency_wait();
    int tile = 0;
    for (int ph = 0; ph < p.n_phases; ++ph) {
      const Phase f = load_phase(p.phases + ph);
      const unsigned before = static_cast<unsigned>(ph) * G;      // the counter once the phase in front is complete
      const bool stamp = p.trace != nullptr && wtid == 0;
      unsigned long long* stamps = p.trace + (static_cast<int64_t>(ph) * G + cta) * 4;
      if (stamp) stamps[0] = global_ns(), stamps[1] = 0;
      if (f.kind == kPhaseLinear) {
        const int tiles = f.tiles_m * f.splits;
        if (cta >= tiles) {
          if (wtid == 0 && ph > 0) wait_count(p.sync, before, p.status, 28);
        }
        for (int t = cta; t < tiles; t += G, ++tile) {
          const int tile_m = t % f.tiles_m, split = t / f.tiles_m;
          const int b = tile & 1;
          const bool ok = mbar_wait(smem_u32(&acc_full[b]), (tile >> 1) & 1, p.status, 29);
          tc_fence_after();
          if (stamp && t == cta) stamps[1] = global_ns();
          const uint32_t acc = tmem_base + b * 64;
          if (f.swiglu) {
            swiglu_tile(acc, xch, reinterpret_cast<bf16*>(f.out), f.half_rows, tile_m, f.half_rows, 0, p.n, BN, quarter, lane, ok);
          } else {
            store_tile<kStore>(acc + (static_cast<uint32_t>(quarter * 32) << 16),
                               reinterpret_cast<float*>(f.out) + static_cast<int64_t>(split) * p.n * f.M,
                               tile_m * kTileM + quarter * 32 + lane, f.M, 0, p.n, f.M, BN, ok);
          }
          tc_fence_before();
          worker_sync();
          if (wtid == 0) mbar_arrive(smem_u32(&acc_empty[b]));
        }
      } else if (f.kind == kPhaseNorm) {
        if (wtid == 0 && ph > 0) wait_count(p.sync, before, p.status, 30);
        if (stamp) stamps[1] = global_ns();
        worker_sync();
        for (int r = cta; r < p.n; r += G) norm_row(f, r, p.n, reinterpret_cast<float*>(work_smem), red_s, wtid);
      } else {
        at::AttnTcParams a = p.attention[f.attention];
        a.meta = p.meta;
        a.meta_stride = p.meta_stride;
        a.work = p.work;
        a.chunks = p.chunks;
        a.part_o = p.scratch;
        a.part_ml = p.scratch + static_cast<int64_t>(p.items) * a.Hkv * p.chunks * 16 * D;
        a.partial_stride = static_cast<int64_t>(p.n) * (a.Hq + 2 * a.Hkv) * D;
        ChainEnv env{p.sync, before, p.status, wtid, ph == 0};
        const int units = p.items * a.Hkv * p.chunks;
        for (int u = cta; u < units; u += G) {
          worker_sync();       // the unit in front is done with the tiles
          const int item = u % p.items, g = (u / p.items) % a.Hkv, chunk = u / (p.items * a.Hkv);
          at::decode_unit<D, true, false>(a, item, g, chunk, work_smem, &is_last_s, wtid, env);
        }
        env.wait_inputs();     // (a CTA without units still sees the phase in front complete before it arrives)
      }
      worker_sync();
      if (stamp) stamps[2] = global_ns();
      if (wtid == 0) arrive_release(p.sync);
      if (stamp) stamps[3] = global_ns();
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
  if (threadIdx.x == 0) {
    // the CTA that leaves last puts the counters back to zero for the next launch
    __threadfence();
    const unsigned ticket = atomicAdd(p.sync + 1, 1u);
    if (ticket == static_cast<unsigned>(G) - 1) {
      p.sync[0] = 0;
      p.sync[1] = 0;
    }
  }
}

// ------------------------------------------------------------------ host side
struct Chain {
  std::vector<Phase> phases;
  std::vector<CUtensorMap> maps;
  std::vector<at::AttnTcParams> attention;
  std::vector<int64_t> scratch_note;       // per attention phase: where the scratch buffer is noted
  int max_rows = 0, D = 0, plan = -1;
  // on the device, after sb_chain_finish
  Phase* d_phases = nullptr;
  CUtensorMap* d_maps = nullptr;
  at::AttnTcParams* d_attention = nullptr;
  unsigned* d_sync = nullptr;
  unsigned long long* trace = nullptr;
  bool finished = false;
};

bool tensor_map(const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, CUtensorMap* out) {
  const int64_t dims[2] = {cols, rows}, strides[2] = {1, ld};
  const int box[2] = {kTileK, box_rows};
  return tensor_map_bf16(base, 2, dims, strides, box, out);
}

template <int D>
size_t chain_smem(int stages, int BN, int max_H) {
  const size_t work = std::max(at::decode_unit_smem<D, true>(), static_cast<size_t>(max_H) * sizeof(float));
  return 1024 + static_cast<size_t>(stages) * (kStageA + BN * 128) + 4096 + work;
}

}  // namespace

// A chain for steps of up to max_rows tokens (the rows of the buffers its phases name).
SB_EXPORT void* sb_chain_create(int max_rows) {
  Chain* c = new Chain();
  c->max_rows = max_rows;
  return c;
}

SB_EXPORT void sb_chain_destroy(void* chain) {
  Chain* c = static_cast<Chain*>(chain);
  if (c == nullptr) return;
  cudaFree(c->d_phases);
  cudaFree(c->d_maps);
  cudaFree(c->d_attention);
  cudaFree(c->d_sync);
  delete c;
}

SB_EXPORT int sb_chain_size(void* chain) { return static_cast<int>(static_cast<Chain*>(chain)->phases.size()); }

// h [rows][H] float32 += the S pending partial sums [S][n][H] (partials null: none); x [rows][H] bfloat16 = gain * (h * r).
SB_EXPORT int sb_chain_norm(void* chain, void* h, const void* partials, int S, const void* gain, int gain_dtype, void* x, int x_dtype,
                            int H, float eps) {
  Chain* c = static_cast<Chain*>(chain);
  if (H % 4 != 0 || H > 16384) return sb::fail("sb_chain_norm: width %d (a multiple of 4 up to 16384)", H);
  if (x_dtype != 1 || (gain_dtype != 0 && gain_dtype != 1)) return sb::fail("sb_chain_norm: bfloat16 output and a float32 or bfloat16 gain");
  if ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(partials) | reinterpret_cast<uintptr_t>(gain) | reinterpret_cast<uintptr_t>(x)) & 15)
    return sb::fail("sb_chain_norm: buffers must be 16-byte aligned");
  Phase f{};
  f.kind = kPhaseNorm;
  f.H = H;
  f.n_partials = partials ? S : 0;
  f.gain_bf16 = gain_dtype == 1;
  f.eps = eps;
  f.h = reinterpret_cast<int64_t>(h);
  f.partials = reinterpret_cast<int64_t>(partials);
  f.gain = reinterpret_cast<int64_t>(gain);
  f.out = reinterpret_cast<int64_t>(x);
  c->phases.push_back(f);
  return 0;
}

// out = x . W^T, x bfloat16 [rows][ldx], W bfloat16 [M][ldw]. swiglu 0: the S = sb_gemm_tc_splits(M, K) partial sums, float32
// [S][n][M]; swiglu 1: W = [gate rows; up rows], out bfloat16 [n][M / 2] = silu(gate) * up, one K range.
SB_EXPORT int sb_chain_linear(void* chain, const void* x, int64_t ldx, const void* w, int64_t ldw, void* out, int M, int K, int swiglu, int S) {
  Chain* c = static_cast<Chain*>(chain);
  if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return sb::fail("sb_chain_linear: K %d and the leading dimensions must be multiples of 8", K);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15)
    return sb::fail("sb_chain_linear: operands must be 16-byte aligned");
  const int kblocks = (K + kTileK - 1) / kTileK;
  if (swiglu && (S != 1 || M % 2)) return sb::fail("sb_chain_linear: the SwiGLU epilogue takes one K range and an even M");
  if (S < 1 || S > kblocks) return sb::fail("sb_chain_linear: %d K ranges for %d blocks of K", S, kblocks);
  Phase f{};
  f.kind = kPhaseLinear;
  f.swiglu = swiglu;
  f.M = M;
  f.K = K;
  f.splits = S;
  f.kblocks_per_split = (kblocks + S - 1) / S;
  if (static_cast<int64_t>(S - 1) * f.kblocks_per_split >= kblocks) return sb::fail("sb_chain_linear: %d K ranges leave an empty range", S);
  f.half_rows = swiglu ? M / 2 : 0;
  f.tiles_m = swiglu ? (f.half_rows + 63) / 64 : (M + kTileM - 1) / kTileM;
  f.out = reinterpret_cast<int64_t>(out);
  CUtensorMap m;
  if (!tensor_map(w, M, K, ldw, swiglu ? 64 : kTileM, &m)) return sb::fail("sb_chain_linear: cuTensorMapEncodeTiled failed for the weight");
  f.map_w = static_cast<int>(c->maps.size());
  c->maps.push_back(m);
  f.map_x = static_cast<int>(c->maps.size());
  for (int bn = 16; bn <= kMaxTokens; bn *= 2) {
    if (!tensor_map(x, c->max_rows, K, ldx, bn, &m)) return sb::fail("sb_chain_linear: cuTensorMapEncodeTiled failed for the tokens");
    c->maps.push_back(m);
  }
  c->phases.push_back(f);
  return 0;
}

// Rotation, append and attention of the step's decode entries from the projection's partial sums qkv [S][n][(Hq + 2 Hkv) D]
// (sb_attention_decode_rope's arguments; the step's own come with every launch). scratch_note: where the engine notes
// the chunk records' buffer (two int64 on the host: device address, floats). plan: the step's tile plan of this head ratio.
SB_EXPORT int sb_chain_attention(void* chain, const void* qkv, int S, const void* cos_sin, void* out, void* k_base, const void* block_table,
                                 int max_pages, int page_size, int64_t page_stride, int64_t v_offset, int64_t head_stride,
                                 int64_t scratch_note, void* counters, int Hq, int Hkv, int D, int window, float scale, int plan) {
  Chain* c = static_cast<Chain*>(chain);
  if (D != 64 && D != 128) return sb::fail("sb_chain_attention: head_dim %d (64 or 128)", D);
  if (c->D != 0 && (c->D != D || c->plan != plan)) return sb::fail("sb_chain_attention: one head size and one tile plan per chain");
  if (Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > 16) return sb::fail("sb_chain_attention: group ratio %d/%d is not supported (1..16)", Hq, Hkv);
  if ((reinterpret_cast<uintptr_t>(k_base) & 15) || (page_stride | v_offset | head_stride) % 8 || (reinterpret_cast<uintptr_t>(cos_sin) & 7))
    return sb::fail("sb_chain_attention: the cache must be 16-byte aligned and cos_sin 8-byte aligned");
  c->D = D;
  c->plan = plan;
  at::AttnTcParams p{};
  p.q = static_cast<const at::bf16*>(out);
  p.out = static_cast<at::bf16*>(out);
  p.k_base = static_cast<const at::bf16*>(k_base);
  p.block_table = static_cast<const int32_t*>(block_table);
  p.max_pages = max_pages;
  p.page_size = page_size;
  p.page_shift = -1;
  for (int b = 0; b < 31; ++b)
    if ((1 << b) == page_size) p.page_shift = b;
  p.page_stride = page_stride;
  p.v_offset = v_offset;
  p.head_stride = head_stride;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.g_mul = (65536 + Hq / Hkv - 1) / (Hq / Hkv);
  for (int r = 0; r < 64; ++r)
    if (((r * p.g_mul) >> 16) != r / (Hq / Hkv)) return sb::fail("sb_chain_attention: the row arithmetic does not hold for %d/%d heads", Hq, Hkv);
  p.window = window;
  p.scale_log2 = scale * sb::attn::kLog2e;
  p.counters = static_cast<int*>(counters);
  p.qkv = static_cast<const float*>(qkv);
  p.n_partials = S;
  p.cos_sin = static_cast<const float*>(cos_sin);
  Phase f{};
  f.kind = kPhaseAttention;
  f.attention = static_cast<int>(c->attention.size());
  c->attention.push_back(p);
  c->scratch_note.push_back(scratch_note);
  c->phases.push_back(f);
  return 0;
}

// Copies the phases to the device; the chain can run from then on and takes no more phases.
SB_EXPORT int sb_chain_finish(void* chain) {
  Chain* c = static_cast<Chain*>(chain);
  if (c->finished) return sb::fail("sb_chain_finish: called twice");
  if (c->phases.empty()) return sb::fail("sb_chain_finish: a chain without phases");
  auto up = [](auto** dst, const auto& v) {
    const size_t bytes = v.size() * sizeof(v[0]);
    if (bytes == 0) return true;
    return cudaMalloc(reinterpret_cast<void**>(dst), bytes) == cudaSuccess && cudaMemcpy(*dst, v.data(), bytes, cudaMemcpyHostToDevice) == cudaSuccess;
  };
  if (!up(&c->d_phases, c->phases) || !up(&c->d_maps, c->maps) || !up(&c->d_attention, c->attention))
    return sb::fail("sb_chain_finish: cannot copy the chain to the device (%s)", cudaGetErrorString(cudaGetLastError()));
  if (cudaMalloc(reinterpret_cast<void**>(&c->d_sync), 2 * sizeof(unsigned)) != cudaSuccess ||
      cudaMemset(c->d_sync, 0, 2 * sizeof(unsigned)) != cudaSuccess)
    return sb::fail("sb_chain_finish: cannot allocate the phase counter");
  c->finished = true;
  return 0;
}

// After a launch whose waits gave up the counters are left as they were: zero them before the next launch.
SB_EXPORT int sb_chain_reset(void* chain) {
  Chain* c = static_cast<Chain*>(chain);
  if (c->d_sync && cudaMemset(c->d_sync, 0, 2 * sizeof(unsigned)) != cudaSuccess) return sb::fail("sb_chain_reset: cudaMemset failed");
  return 0;
}

// From now on every launch of the chain leaves nanosecond stamps (%globaltimer) per phase and CTA in `stamps`
// ([2][phases][SMs][4] uint64 on the device). [0]: when the CTA's workers reached the phase, when its input was there (0:
// the CTA had no share in the phase), when their share was written, when their arrival was counted. [1], linear phases:
// when the MMA issuer had its first operands, how long it waited for weight tiles and for token tiles in all, when
// it had issued the last product. Null: no stamps.
SB_EXPORT void sb_chain_trace(void* chain, unsigned long long* stamps) { static_cast<Chain*>(chain)->trace = stamps; }

SB_EXPORT void sb_decode_chain_use_status_word(int* device_word) { status_word_given() = device_word; }

// The most tokens of a step that the chain takes.
SB_EXPORT int sb_chain_max_tokens() { return kMaxTokens; }

// ------------------------------------------------------------------ operation of the native step program (step_ops.h)
// Stands for the operations of all layers when the step consists of decode entries only (no tile of a prompt portion in
// any plan) and has at most sb_chain_max_tokens() tokens; otherwise it skips and the layers' own operations run.
// i: 0 the chain
SB_EXPORT int sb_op_decode_chain(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  Chain* c = ptr<Chain>(op->i[0]);
  if (!c->finished || s->n <= 0 || s->n > kMaxTokens || s->n > c->max_rows) return SB_OP_SKIPPED;
  for (int k = 0; k < s->n_plans; ++k)
    if (s->plan[k].tiles > 0) return SB_OP_SKIPPED;
  ChainParams p{};
  p.phases = c->d_phases;
  p.n_phases = static_cast<int>(c->phases.size());
  p.maps = c->d_maps;
  p.attention = c->d_attention;
  p.n = s->n;
  p.bn_log = s->n <= 16 ? 0 : s->n <= 32 ? 1 : 2;
  int max_H = 0;
  for (const Phase& f : c->phases) max_H = std::max(max_H, f.H);
  if (!c->attention.empty()) {
    const SbTilePlan& plan = s->plan[c->plan];
    if (plan.items <= 0) return SB_OP_SKIPPED;
    p.items = plan.items;
    p.chunks = plan.chunks;
    p.work = work(s, plan);
    const int64_t need = static_cast<int64_t>(plan.items) * c->attention[0].Hkv * plan.chunks * 16 * (c->D + 2);
    float* scratch = nullptr;
    for (int64_t note : c->scratch_note) {
      const int64_t* noted = ptr<const int64_t>(note);
      if (need > noted[1])
        return sb::fail("sb_op_decode_chain: %d decode entries over %d chunks need more scratch than the engine set aside (%lld floats)",
                        plan.items, plan.chunks, (long long)noted[1]);
      if (scratch != nullptr && scratch != ptr<float>(noted[0])) return sb::fail("sb_op_decode_chain: the attention phases must share one scratch buffer");
      scratch = ptr<float>(noted[0]);
    }
    p.scratch = scratch;
  }
  p.meta = entry_meta(s);
  p.meta_stride = s->max_rows;
  p.sync = c->d_sync;
  p.trace = c->trace;
  p.status = status_word();
  if (!p.status) return sb::fail("sb_op_decode_chain: cannot allocate the status word");
  const int BN = 16 << p.bn_log;
  const int D = c->D ? c->D : 64;
  const size_t fixed = D == 128 ? chain_smem<128>(0, BN, max_H) : chain_smem<64>(0, BN, max_H);
  if (fixed + 2 * (kStageA + BN * 128) > kSmemLimit - 1024) return SB_OP_SKIPPED;      // (no room for a ring: the separate kernels run)
  p.w_stages = static_cast<int>(std::min<size_t>(kMaxStages, (kSmemLimit - 1024 - fixed) / (kStageA + BN * 128)));
  const size_t smem = fixed + static_cast<size_t>(p.w_stages) * (kStageA + BN * 128);
  const int grid = sb::sm_count();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  static sb::DeviceOnce once;
  if (once.needed()) {
    if (cudaFuncSetAttribute(decode_chain_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit - 1024) != cudaSuccess ||
        cudaFuncSetAttribute(decode_chain_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit - 1024) != cudaSuccess)
      return sb::fail("sb_op_decode_chain: cannot raise the shared memory limit");
    once.done();
  }
  if (D == 128) sb::launch_pdl(decode_chain_kernel<128>, dim3(grid), dim3(kChainThreads), smem, st, p);
  else sb::launch_pdl(decode_chain_kernel<64>, dim3(grid), dim3(kChainThreads), smem, st, p);
  return sb::check_launch("sb_op_decode_chain") ? SB_OP_FAILED : SB_OP_LAUNCHED;
}
