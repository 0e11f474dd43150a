// attn_fwd on tcgen05 / TMEM: FlashAttention-2 forward for 16-bit elements,
// head dimension 64 or 128, optional causal mask.
//
// Semantics: Sources/TritonMetalBench/AttentionKernel.swift:40-250 - per query
// block, walk the key blocks with an online softmax in base 2
// (qk_scale = sm_scale*log2 e), P rounded to the element type before P.V,
// O = acc / l, and the row statistic L = m + log2(l) in log2 units.
//
// Persistent: one CTA per SM walks its list of query blocks (256 rows of one (batch, head);
// the lists are balanced on the host, attn_schedule.h); the loads and the first score MMAs of
// the next block run under the output pass of the current one.
// A query block is two 128-row tiles that take turns on the tensor core, so the
// exponentials of one tile overlap the MMAs of the other:
//   warps 0-7   softmax: tile t = warp / 4.  A thread owns one query row (its TMEM lane):
//               it copies the row's 128 scores of a key block into registers once, takes
//               the maximum, then exp2 / row sum / round, and writes the 16-bit P back over
//               the scores.  Nothing is exchanged between threads.
//   warp 8      TMA: Q (both tiles) once per query block, then K and V blocks of 128
//               keys into 2-stage rings
//   warp 9      MMA issuer: S_t = Q_t K^T (128x128xD, operands in shared memory),
//               O_t += P_t V (128xDx128, P read from TMEM)
//   warps 10-11 idle: they complete the third warpgroup, which hands most of its registers to
//               the softmax warpgroups (setmaxnreg), so that a softmax thread can hold a whole
//               row of scores: with more warps (and the row split between two threads) every key block
// cost a second TMEM read of the scores and an exchange of half-row maxima through shared
// memory behind a named barrier, and the softmax of a tile - which sits on the critical path
// S -> P -> P.V -> next S - took about twice the 1024 cycles its exponentials need.
// The running max used for the exponentials only advances when it grew by more
// than 8 (log2 units): P stays <= 256 and most iterations skip the O rescale in
// TMEM; O/l at the end is exact either way.
//
// TMEM columns: S_0 | S_1 | O_0 | O_1.
// HBM layout: Q, K, V, O [BH, S, D] with D contiguous (stride_seq == D),
// L [BH, S] fp32.

#include "attn_schedule.h"
#include "sm100_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <type_traits>

namespace tmc {
namespace {

using namespace ptx;

constexpr int BLOCK_M = 128, BLOCK_N = 128;
constexpr int TILES = 2;                       // query tiles per CTA
constexpr int NUM_THREADS = 384;                // 8 softmax warps + a warpgroup holding the TMA and MMA warps
constexpr int LOAD_WARP = 8, MMA_WARP = 9;
// Registers per thread after the warpgroups have traded.  The CTA owns what it was launched
// with - LAUNCH_REGS per thread for three warpgroups - and setmaxnreg.inc WAITS, without any
// bound, until the registers it asks for are free in that pool: the two softmax warpgroups may
// only take what the third one gives up, or the kernel never starts.
constexpr int LAUNCH_REGS = 168;                // what ptxas allots at 384 threads per CTA
constexpr int SOFTMAX_REGS = 208, ISSUE_REGS = 88;
static_assert(2 * SOFTMAX_REGS + ISSUE_REGS <= 3 * LAUNCH_REGS, "setmaxnreg.inc would wait for ever");
static_assert(SOFTMAX_REGS % 8 == 0 && ISSUE_REGS % 8 == 0, "setmaxnreg takes multiples of 8");
constexpr int TMEM_COLS = 512;
constexpr float kLog2e = 1.44269504088896340736f;
constexpr float kRescaleThreshold = 8.0f;

enum Site : uint32_t {
  kLoadQEmpty = 10, kLoadKEmpty = 11, kLoadVEmpty = 12, kMmaQ = 13, kMmaK = 14, kMmaV = 15, kMmaP = 16,
  kSoftS = 17, kSoftFinal = 19, kDrainLoad = 20
};

struct Shared {
  alignas(8) uint64_t q_full, q_empty;
  alignas(8) uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  alignas(8) uint64_t s_full[TILES], p_full[TILES], pv_done[TILES];
  uint32_t tmem_base;
  int abort_flag;
};

struct Params {
  void* o;
  float* lse;
  float sm_scale;
  int64_t stride_head, stride_seq, stride_lse;
  int n_ctx, rows, causal;
};

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ---- softmax of one row of a 128-column score tile ---------------------------------
// The row sits in four register arrays of 32 scores (one tcgen05.ld each).
struct MaskInfo {
  int n0, q_row, n_ctx, causal;     // n0: key of column 0
  __device__ __forceinline__ bool masked(int col) const {
    const int key = n0 + col;
    return key >= n_ctx || (causal && key > q_row);
  }
};

template <bool MASKED>
__device__ __forceinline__ float max_chunk(const uint32_t (&r)[32], int col0, const MaskInfo& mi) {
  float m0 = -INFINITY, m1 = -INFINITY;
  if (!MASKED) {
    // four independent chains of three-input maxima (the four chunks of a row make sixteen)
    float m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      m0 = max3(m0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
      m1 = max3(m1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
      m2 = max3(m2, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
      m3 = max3(m3, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
    }
    return max3(m0, m1, fmaxf(m2, m3));
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      if (!mi.masked(col0 + i)) m0 = fmaxf(m0, __uint_as_float(r[i]));
      if (!mi.masked(col0 + i + 1)) m1 = fmaxf(m1, __uint_as_float(r[i + 1]));
    }
  }
  return fmaxf(m0, m1);
}

// P = exp2(s*qk_scale + neg_m) for 32 columns, rounded to T and written to `dst` (16 packed
// columns); returns the fp32 sum.  Off the mask boundary the scaling and the row sum run two
// wide (fma.f32x2 / add.f32x2): per element that leaves half an fma, the exponential, half an
// add and half a conversion.
template <typename T, bool MASKED>
__device__ __forceinline__ float exp_chunk(const uint32_t (&r)[32], uint32_t dst, float qk_scale,
                                           float neg_m, int col0, const MaskInfo& mi) {
  uint32_t packed[16];
  if (!MASKED) {
    const uint64_t scale2 = pack_f32x2(qk_scale, qk_scale), neg_m2 = pack_f32x2(neg_m, neg_m);
    uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      float x0, x1, x2, x3;
      unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), scale2, neg_m2), x0, x1);
      unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])), scale2, neg_m2), x2, x3);
      const float p0 = fast_exp2(x0), p1 = fast_exp2(x1), p2 = fast_exp2(x2), p3 = fast_exp2(x3);
      acc0 = add_f32x2(acc0, pack_f32x2(p0, p1));
      acc1 = add_f32x2(acc1, pack_f32x2(p2, p3));
      packed[i / 2] = pack2<T>(p0, p1);
      packed[i / 2 + 1] = pack2<T>(p2, p3);
    }
    tmem_st_32x16(dst, packed);
    float a, b;
    unpack_f32x2(add_f32x2(acc0, acc1), a, b);
    return a + b;
  }
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const float x0 = fmaf(__uint_as_float(r[i]), qk_scale, neg_m);
    const float x1 = fmaf(__uint_as_float(r[i + 1]), qk_scale, neg_m);
    float p0 = fast_exp2(x0);
    float p1 = fast_exp2(x1);
    if (mi.masked(col0 + i)) p0 = 0.f;
    if (mi.masked(col0 + i + 1)) p1 = 0.f;
    s0 += p0;
    s1 += p1;
    packed[i / 2] = pack2<T>(p0, p1);
  }
  tmem_st_32x16(dst, packed);
  return s0 + s1;
}

// ---- the plain score block, scheduled by hand -----------------------------------------
// A softmax warp is alone on its scheduler while it works (the other tile's warp waits for its
// scores), it issues in order, and every exponential costs the special-function unit 8 cycles:
// the exponentials of a row take 1024 cycles at best, and they only do if an ex2 is issued
// every 8 cycles with the scaling of later elements and the sum / rounding of earlier ones
// filling the slots in between.  Left to the compiler the pass took about 1800 cycles (the
// dependent instructions of one element end up back to back and wait for each other), so the
// order is fixed here: every statement is a volatile asm, which the compiler keeps in sequence.
// Values are transformed in place (score -> scaled score -> probability).
__device__ __forceinline__ void scale_pair(uint32_t& a, uint32_t& b, uint64_t scale2, uint64_t neg_m2) {
  asm volatile(
      "{\n.reg .b64 t;\nmov.b64 t, {%0, %1};\nfma.rn.f32x2 t, t, %2, %3;\nmov.b64 {%0, %1}, t;\n}"
      : "+r"(a), "+r"(b)
      : "l"(scale2), "l"(neg_m2));
}
__device__ __forceinline__ void exp2_inplace(uint32_t& a) {
  asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+r"(a));
}
__device__ __forceinline__ void sum_pair(uint64_t& acc, uint32_t a, uint32_t b) {
  asm volatile("{\n.reg .b64 t;\nmov.b64 t, {%1, %2};\nadd.rn.f32x2 %0, %0, t;\n}" : "+l"(acc) : "r"(a), "r"(b));
}
template <typename T> __device__ __forceinline__ uint32_t round_pair(uint32_t lo, uint32_t hi);
template <> __device__ __forceinline__ uint32_t round_pair<__nv_bfloat16>(uint32_t lo, uint32_t hi) {
  uint32_t d;
  asm volatile("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(d) : "r"(lo), "r"(hi));
  return d;
}
template <> __device__ __forceinline__ uint32_t round_pair<__half>(uint32_t lo, uint32_t hi) {
  uint32_t d;
  asm volatile("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(d) : "r"(lo), "r"(hi));
  return d;
}

// P = exp2(s * qk_scale + neg_m) over a whole row (four 32-column chunks), rounded and written
// to `dst` (64 packed columns); returns the fp32 row sum.  LAG pairs separate an ex2 from the
// instructions that consume its result.
template <typename T>
__device__ __forceinline__ float exp_row_plain(uint32_t (&s0)[32], uint32_t (&s1)[32], uint32_t (&s2)[32],
                                               uint32_t (&s3)[32], uint32_t dst, float qk_scale, float neg_m) {
  constexpr int LAG = 4;
  const uint64_t scale2 = pack_f32x2(qk_scale, qk_scale), neg_m2 = pack_f32x2(neg_m, neg_m);
  uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0;
  uint32_t packed[64];
  auto elem = [&](int i) -> uint32_t& {          // element i of the row, 0 ... 127
    return i < 32 ? s0[i] : (i < 64 ? s1[i - 32] : (i < 96 ? s2[i - 64] : s3[i - 96]));
  };
  // scale the first LAG + 2 pairs ahead of the exponentials
#pragma unroll
  for (int q = 0; q < LAG + 2; ++q) scale_pair(elem(2 * q), elem(2 * q + 1), scale2, neg_m2);
#pragma unroll
  for (int q = 0; q < 64 + LAG; ++q) {
    if (q < 64) {
      exp2_inplace(elem(2 * q));
      if (q + LAG + 2 < 64) scale_pair(elem(2 * (q + LAG + 2)), elem(2 * (q + LAG + 2) + 1), scale2, neg_m2);
      exp2_inplace(elem(2 * q + 1));
    }
    if (q >= LAG) {
      const int d = q - LAG;                       // the pair whose exponentials have had time to finish
      if (d & 1) sum_pair(acc1, elem(2 * d), elem(2 * d + 1));
      else sum_pair(acc0, elem(2 * d), elem(2 * d + 1));
      packed[d] = round_pair<T>(elem(2 * d), elem(2 * d + 1));
      if (d % 16 == 15) {                           // a chunk of P is complete: store it
        uint32_t out[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) out[k] = packed[d - 15 + k];
        tmem_st_32x16(dst + (d / 16) * 16, out);
      }
    }
  }
  float a, b;
  unpack_f32x2(add_f32x2(acc0, acc1), a, b);
  return a + b;
}

// The chunk of a diagonal block that the diagonal itself crosses: row `lane` of the warp keeps
// columns 0 ... lane of the chunk (key <= query), the others are masked.
__device__ __forceinline__ float max_chunk_diag(const uint32_t (&r)[32], int lane) {
  float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    if (i <= lane) m0 = fmaxf(m0, __uint_as_float(r[i]));
    if (i + 1 <= lane) m1 = fmaxf(m1, __uint_as_float(r[i + 1]));
  }
  return fmaxf(m0, m1);
}
template <typename T>
__device__ __forceinline__ float exp_chunk_diag(const uint32_t (&r)[32], uint32_t dst, float qk_scale, float neg_m,
                                                int lane) {
  uint32_t packed[16];
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float p0 = fast_exp2(fmaf(__uint_as_float(r[i]), qk_scale, neg_m));
    float p1 = fast_exp2(fmaf(__uint_as_float(r[i + 1]), qk_scale, neg_m));
    if (i > lane) p0 = 0.f;
    if (i + 1 > lane) p1 = 0.f;
    s0 += p0;
    s1 += p1;
    packed[i / 2] = pack2<T>(p0, p1);
  }
  tmem_st_32x16(dst, packed);
  return s0 + s1;
}
__device__ __forceinline__ void zero_chunk(uint32_t dst) {
  uint32_t packed[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) packed[i] = 0u;
  tmem_st_32x16(dst, packed);
}

// ---- persistent schedule -------------------------------------------------------------
// A CTA walks its own list of work items (attn_schedule.h): item = one (batch, head) and one
// 256-row query block.  All three roles read the same list.
template <typename T, int D, uint32_t FMT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, Params prm, DeviceWorkList work, DeviceStatus* status) {
  constexpr int HALVES = D / 64;                        // 64-column swizzle atoms per row
  constexpr int TILE_BYTES = BLOCK_M * D * 2;           // one 128-row tile of Q, K or V
  constexpr int HALF_BYTES = BLOCK_M * 128;             // one [128 x 64] swizzled box
  constexpr int S_COL = 0, O_COL = 256;                 // S_t at t*128, O_t at 256 + t*D
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // layout: Q0 Q1 | K0 K1 | V0 V1 | barriers
  const uint32_t q_addr = smem_u32(smem);
  const uint32_t k_addr = q_addr + TILES * TILE_BYTES;
  const uint32_t v_addr = k_addr + 2 * TILE_BYTES;
  Shared& ss = *reinterpret_cast<Shared*>(smem + (TILES + 4) * TILE_BYTES);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  WaitCtx wc{&ss.abort_flag, status};

  // key blocks tile t of the query block starting at row m0 walks: everything, or up to
  // its own diagonal
  auto key_blocks = [&](int m0, int t) {
    int key_end = prm.n_ctx;
    if (prm.causal) key_end = min(prm.n_ctx, m0 + (t + 1) * BLOCK_M);
    return (key_end + BLOCK_N - 1) / BLOCK_N;
  };

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ss.q_full), 1);
    mbar_init(smem_u32(&ss.q_empty), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&ss.k_full[s]), 1);
      mbar_init(smem_u32(&ss.k_empty[s]), 1);
      mbar_init(smem_u32(&ss.v_full[s]), 1);
      mbar_init(smem_u32(&ss.v_empty[s]), 1);
    }
    for (int t = 0; t < TILES; ++t) {
      mbar_init(smem_u32(&ss.s_full[t]), 1);
      mbar_init(smem_u32(&ss.p_full[t]), 4);
      mbar_init(smem_u32(&ss.pv_done[t]), 1);
    }
    ss.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(&ss.tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ss.tmem_base;

  // All three roles walk the same sequence of query blocks.  Barrier phases follow running
  // counters that never reset: `item` counts query blocks, `g` key blocks through the K/V
  // rings, `c` score blocks of one tile.
  if (warp >= LOAD_WARP) {
  warpgroup_reg_dec<ISSUE_REGS>();
  if (warp == LOAD_WARP) {
    // ---------------------------------------------------------------- loads
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      uint32_t item = 0, g = 0, q_loads = 0, k_loads = 0, v_loads = 0;
      bool ok = true;
      {
        for (WorkCursor w(work); w.valid() && ok; w.advance(), ++item) {
          const int bh = w.cur.x;
          const int m0 = w.cur.y * (TILES * BLOCK_M);
          const int nb_max = key_blocks(m0, TILES - 1);
          // Q is single-buffered: the previous block's last score MMA must have retired
          if (!mbar_wait(smem_u32(&ss.q_empty), (item & 1) ^ 1, wc, kLoadQEmpty)) { ok = false; break; }
          mbar_expect_tx(smem_u32(&ss.q_full), TILES * TILE_BYTES);
#pragma unroll
          for (int t = 0; t < TILES; ++t)
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
              tma_load_3d(q_addr + t * TILE_BYTES + h * HALF_BYTES, &map_q, smem_u32(&ss.q_full), h * 64,
                          m0 + t * BLOCK_M, bh);
          q_loads = item + 1;
          for (int j = 0; j < nb_max; ++j, ++g) {
            const int s = g & 1;
            const uint32_t ph = (g >> 1) & 1;
            if (!mbar_wait(smem_u32(&ss.k_empty[s]), ph ^ 1, wc, kLoadKEmpty)) { ok = false; break; }
            mbar_expect_tx(smem_u32(&ss.k_full[s]), TILE_BYTES);
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
              tma_load_3d(k_addr + s * TILE_BYTES + h * HALF_BYTES, &map_k, smem_u32(&ss.k_full[s]), h * 64,
                          j * BLOCK_N, bh);
            k_loads = g + 1;
            if (!mbar_wait(smem_u32(&ss.v_empty[s]), ph ^ 1, wc, kLoadVEmpty)) { ok = false; break; }
            mbar_expect_tx(smem_u32(&ss.v_full[s]), TILE_BYTES);
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
              tma_load_3d(v_addr + s * TILE_BYTES + h * HALF_BYTES, &map_v, smem_u32(&ss.v_full[s]), h * 64,
                          j * BLOCK_N, bh);
            v_loads = g + 1;
          }
        }
      }
      // every copy started here must have landed before the CTA exits
      auto drain = [&](uint64_t* bar, uint32_t parity, uint32_t info) {
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(bar), parity)) {
          if (clock64() - t0 > kWaitCycles) { report_timeout(wc, kDrainLoad, info); break; }
        }
      };
      if (q_loads) drain(&ss.q_full, (q_loads - 1) & 1, 0);
      for (uint32_t n = k_loads > 2 ? k_loads - 2 : 0; n < k_loads; ++n) drain(&ss.k_full[n & 1], (n >> 1) & 1, 1);
      for (uint32_t n = v_loads > 2 ? v_loads - 2 : 0; n < v_loads; ++n) drain(&ss.v_full[n & 1], (n >> 1) & 1, 2);
    }
  } else if (warp == MMA_WARP) {
    // ---------------------------------------------------------------- MMA issue
    // The whole warp runs this loop, converged; one elected lane issues (see mma_f16_ss_elect).
    {
      constexpr uint32_t idesc_qk = make_idesc(FMT, BLOCK_M, BLOCK_N, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(FMT, BLOCK_M, D, 0, 1);
      // S_t = Q_t K^T with K in ring stage `stage`.  The caller has made sure K has landed.
      // operand descriptors are built once; per instruction only the address field moves
      const SmemDesc q_desc = make_desc_sw128(q_addr, 0, 1024), k_desc = make_desc_sw128(k_addr, 0, 1024);
      const SmemDesc v_desc = make_desc_sw128(v_addr, HALF_BYTES, 1024);
      auto issue_qk = [&](int t, int stage) {
        const SmemDesc kb = k_desc.advanced(stage * TILE_BYTES);
        const SmemDesc qb = q_desc.advanced(t * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * HALF_BYTES + (kk % 4) * 32;
          mma_f16_ss_elect(tmem + S_COL + t * BLOCK_N, qb.at_here(off), kb.at_here(off), idesc_qk, kk != 0);
        }
        mma_commit_elect(smem_u32(&ss.s_full[t]));
      };
      uint32_t item = 0, g = 0, c[TILES] = {0, 0};
      bool ok = true;
      {
        for (WorkCursor w(work); w.valid() && ok; w.advance(), ++item) {
          const int m0 = w.cur.y * (TILES * BLOCK_M);
          int nb[TILES];
#pragma unroll
          for (int t = 0; t < TILES; ++t) nb[t] = key_blocks(m0, t);
          const int nb_max = nb[TILES - 1];               // later rows see at least as many keys
          if (!mbar_wait_warp(smem_u32(&ss.q_full), item & 1, wc, kMmaQ)) { ok = false; break; }
          if (!mbar_wait_warp(smem_u32(&ss.k_full[g & 1]), (g >> 1) & 1, wc, kMmaK)) { ok = false; break; }
          tc_fence_after();
          // The first scores of this query block go over the last P of the previous one, and
          // its first P.V starts a fresh O: MMAs run in issue order, and the softmax threads
          // hand over P(0) only after they have read the previous O out of TMEM.
#pragma unroll
          for (int t = 0; t < TILES; ++t) issue_qk(t, g & 1);
          mma_commit_elect(smem_u32(&ss.k_empty[g & 1]));      // K(0) is free once both S(0) retire
          if (nb_max == 1) mma_commit_elect(smem_u32(&ss.q_empty));
          // One key block.  `steady` (a compile-time constant at both call sites) marks blocks with
          // two more to come for both tiles: every condition below is then known, and the issuing
          // thread - alone in its warp, it pays tens of cycles for each compare-and-branch - keeps
          // only the barrier waits.
          auto key_block = [&](int j, auto steady_tag) {
            constexpr bool steady = decltype(steady_tag)::value;
            const int s = g & 1;
            if (!mbar_wait_warp(smem_u32(&ss.v_full[s]), (g >> 1) & 1, wc, kMmaV)) { ok = false; return; }
            if ((steady || j + 1 < nb_max) &&
                !mbar_wait_warp(smem_u32(&ss.k_full[s ^ 1]), ((g + 1) >> 1) & 1, wc, kMmaK)) {
              ok = false;
              return;
            }
#pragma unroll
            for (int t = 0; t < TILES; ++t) {
              if (steady || j < nb[t]) {
                if (!mbar_wait_warp(smem_u32(&ss.p_full[t]), c[t] & 1, wc, kMmaP)) { ok = false; return; }
                ++c[t];
                tc_fence_after();
                const SmemDesc vb = v_desc.advanced(s * TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
                  // P: TMEM operand, 16 keys = 8 packed 32-bit columns from the start of the score
                  // buffer.  V: MN-major, 16 keys = 2048 bytes further, 64-column halves
                  // HALF_BYTES apart.
                  mma_f16_ts_elect(tmem + O_COL + t * D, tmem + S_COL + t * BLOCK_N + kk * 8,
                             vb.at_here(kk * 2048), idesc_pv, (j | kk) != 0);
                }
                // O_t is only read after the last block; rescales in between are ordered by the
                // next s_full (a commit covers every MMA issued before it, P.V(j) included)
                if (!steady && j + 1 == nb[t]) mma_commit_elect(smem_u32(&ss.pv_done[t]));
              }
              // V(j) has been read by both tiles: release it as early as possible
              if (t == TILES - 1) mma_commit_elect(smem_u32(&ss.v_empty[s]));
              // the next scores of this tile overwrite its P: MMAs run in issue order
              if (steady || j + 1 < nb[t]) issue_qk(t, s ^ 1);
              if (t == TILES - 1 && (steady || j + 1 < nb_max)) {
                // the last tile always walks every block: K(j+1) is free once its S retires,
                // and after the last block's scores so is Q
                mma_commit_elect(smem_u32(&ss.k_empty[s ^ 1]));
                if (!steady && j + 2 == nb_max) mma_commit_elect(smem_u32(&ss.q_empty));
              }
            }
          };
          int j = 0;
          for (; j + 2 < nb[0] && ok; ++j, ++g) key_block(j, std::true_type{});
          for (; j < nb_max && ok; ++j, ++g) key_block(j, std::false_type{});
        }
      }
    }
  }
  } else {
    warpgroup_reg_inc<SOFTMAX_REGS>();
    // ---------------------------------------------------------------- softmax
    // Tile t = warp / 4; thread = query row = TMEM lane; the whole row of a score block lives
    // in this thread's registers between the max and the exponentials.
    const int t = warp / 4;
    const int row_in_tile = (warp % 4) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp % 4) * 32) << 16;
    const uint32_t s_tmem = tmem + lane_addr + S_COL + t * BLOCK_N;
    const uint32_t o_tmem = tmem + lane_addr + O_COL + t * D;
    const float qk_scale = prm.sm_scale * kLog2e;
    uint32_t c = 0;                               // score blocks this tile has consumed
    uint32_t item = 0;                            // query blocks done (phase of pv_done)
    bool ok = true;
    {
      for (WorkCursor w(work); w.valid() && ok; w.advance(), ++item) {
        const int bh = w.cur.x;
        const int m0 = w.cur.y * (TILES * BLOCK_M);
        const int q_row = m0 + t * BLOCK_M + row_in_tile;
        const int my_blocks = key_blocks(m0, t);
        float m_used = -INFINITY, l = 0.f;
        for (int j = 0; j < my_blocks; ++j, ++c) {
          if (!mbar_wait(smem_u32(&ss.s_full[t]), c & 1, wc, kSoftS)) { ok = false; break; }
          tc_fence_after();
          uint32_t s0[32], s1[32], s2[32], s3[32];
          tmem_ld_32x32(s_tmem, s0);
          tmem_ld_32x32(s_tmem + 32, s1);
          tmem_ld_32x32(s_tmem + 64, s2);
          tmem_ld_32x32(s_tmem + 96, s3);
          tmem_ld_wait();
          const int n0 = j * BLOCK_N;
          // Three kinds of block.  Plain: no key is masked.  Diagonal: the block on the causal
          // diagonal of this tile, all of it inside the sequence - for the rows of this warp the
          // 32-column chunks left of the diagonal are plain, the chunks right of it are masked as
          // a whole (P = 0, nothing is computed), and only the chunk the diagonal crosses needs a
          // test per element.  Ragged: a block that runs past the end of the sequence.
          const bool ragged = n0 + BLOCK_N > prm.n_ctx;
          const bool diagonal = !ragged && prm.causal && n0 == m0 + t * BLOCK_M;
          const int wchunk = warp % 4;                     // the chunk the diagonal crosses for this warp
          const MaskInfo mi{n0, q_row, prm.n_ctx, prm.causal};
          // row max of the raw scores (qk_scale > 0, so the scaled max is max * qk_scale)
          float mx;
          if (ragged) {
            mx = fmaxf(fmaxf(max_chunk<true>(s0, 0, mi), max_chunk<true>(s1, 32, mi)),
                       fmaxf(max_chunk<true>(s2, 64, mi), max_chunk<true>(s3, 96, mi)));
          } else if (diagonal) {
            mx = wchunk == 0 ? max_chunk_diag(s0, lane) : max_chunk<false>(s0, 0, mi);
            if (wchunk >= 1) mx = fmaxf(mx, wchunk == 1 ? max_chunk_diag(s1, lane) : max_chunk<false>(s1, 32, mi));
            if (wchunk >= 2) mx = fmaxf(mx, wchunk == 2 ? max_chunk_diag(s2, lane) : max_chunk<false>(s2, 64, mi));
            if (wchunk >= 3) mx = fmaxf(mx, max_chunk_diag(s3, lane));
          } else {
            mx = fmaxf(fmaxf(max_chunk<false>(s0, 0, mi), max_chunk<false>(s1, 32, mi)),
                       fmaxf(max_chunk<false>(s2, 64, mi), max_chunk<false>(s3, 96, mi)));
          }
          mx *= qk_scale;
          // advance the working max only when it moved far (or on the first block)
          float alpha = 1.f;
          bool rescale = false;
          if (mx > m_used + kRescaleThreshold) {
            alpha = fast_exp2(m_used - mx);      // 0 on the first block (m_used = -inf)
            m_used = mx;
            rescale = j > 0;
          }
          if (__any_sync(0xffffffffu, rescale)) {
            // O_t may only be touched once the P.V MMA of block j-1 has finished: it has, the
            // s_full this thread waited for above was committed after it.
#pragma unroll 1
            for (int cc = 0; cc < D / 32; ++cc) {
              uint32_t r[32];
              tmem_ld_32x32(o_tmem + cc * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32(o_tmem + cc * 32, r);
            }
          }
          // exponentials, row sum, 16-bit P over the first 64 columns of the scores
          float sum;
          const float neg_m = -m_used;
          if (ragged) {
            sum = exp_chunk<T, true>(s0, s_tmem, qk_scale, neg_m, 0, mi) +
                  exp_chunk<T, true>(s1, s_tmem + 16, qk_scale, neg_m, 32, mi);
            sum += exp_chunk<T, true>(s2, s_tmem + 32, qk_scale, neg_m, 64, mi) +
                   exp_chunk<T, true>(s3, s_tmem + 48, qk_scale, neg_m, 96, mi);
          } else if (diagonal) {
            sum = wchunk == 0 ? exp_chunk_diag<T>(s0, s_tmem, qk_scale, neg_m, lane)
                              : exp_chunk<T, false>(s0, s_tmem, qk_scale, neg_m, 0, mi);
            if (wchunk >= 1) {
              sum += wchunk == 1 ? exp_chunk_diag<T>(s1, s_tmem + 16, qk_scale, neg_m, lane)
                                 : exp_chunk<T, false>(s1, s_tmem + 16, qk_scale, neg_m, 32, mi);
            } else {
              zero_chunk(s_tmem + 16);
            }
            if (wchunk >= 2) {
              sum += wchunk == 2 ? exp_chunk_diag<T>(s2, s_tmem + 32, qk_scale, neg_m, lane)
                                 : exp_chunk<T, false>(s2, s_tmem + 32, qk_scale, neg_m, 64, mi);
            } else {
              zero_chunk(s_tmem + 32);
            }
            if (wchunk >= 3) sum += exp_chunk_diag<T>(s3, s_tmem + 48, qk_scale, neg_m, lane);
            else zero_chunk(s_tmem + 48);
          } else {
            sum = exp_row_plain<T>(s0, s1, s2, s3, s_tmem, qk_scale, neg_m);
          }
          l = l * alpha + sum;
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ss.p_full[t]));   // one arrival per warp
        }
        // ---- O / l and the row statistic of this query block
        if (ok && my_blocks > 0) ok = mbar_wait(smem_u32(&ss.pv_done[t]), item & 1, wc, kSoftFinal);
        tc_fence_after();
        if (ok && my_blocks > 0) {
          const float inv_l = 1.f / l;
          const bool live = q_row < prm.rows;
          T* orow = (T*)prm.o + (int64_t)bh * prm.stride_head + (int64_t)q_row * prm.stride_seq;
#pragma unroll 1
          for (int cc = 0; cc < D / 32; ++cc) {
            uint32_t r[32];
            tmem_ld_32x32(o_tmem + cc * 32, r);
            tmem_ld_wait();
            if (live) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 out;
                out.x = pack2<T>(__uint_as_float(r[v * 8 + 0]) * inv_l, __uint_as_float(r[v * 8 + 1]) * inv_l);
                out.y = pack2<T>(__uint_as_float(r[v * 8 + 2]) * inv_l, __uint_as_float(r[v * 8 + 3]) * inv_l);
                out.z = pack2<T>(__uint_as_float(r[v * 8 + 4]) * inv_l, __uint_as_float(r[v * 8 + 5]) * inv_l);
                out.w = pack2<T>(__uint_as_float(r[v * 8 + 6]) * inv_l, __uint_as_float(r[v * 8 + 7]) * inv_l);
                *reinterpret_cast<uint4*>(orow + cc * 32 + v * 8) = out;
              }
            }
          }
          if (live && prm.lse) prm.lse[(int64_t)bh * prm.stride_lse + q_row] = m_used + log2f(l);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

WorkListCache g_lists;     // work lists already in device memory, by problem shape

template <typename T, int D, uint32_t FMT>
std::string launch_typed(const AttnProblem& p, const LaunchCtx& ctx, CUtensorMapDataType type) {
  CUtensorMap maps[3];
  const void* bases[3] = {p.q, p.k, p.v};
  for (int i = 0; i < 3; ++i) {
    uint64_t dims[3] = {(uint64_t)D, (uint64_t)p.n_ctx, (uint64_t)p.bh};
    uint64_t strides[2] = {(uint64_t)p.stride_seq * 2, (uint64_t)p.stride_head * 2};
    uint32_t box[3] = {64u, (uint32_t)BLOCK_M, 1u};
    std::string e = make_tensor_map(&maps[i], type, 3, bases[i], dims, strides, box);
    if (!e.empty()) return e;
  }
  Params prm{};
  prm.o = p.out0;
  prm.lse = p.lse;
  prm.sm_scale = p.sm_scale;
  prm.stride_head = p.stride_head;
  prm.stride_seq = p.stride_seq;
  prm.stride_lse = p.stride_lse;
  prm.n_ctx = (int)p.n_ctx;
  prm.rows = (int)p.rows;
  prm.causal = p.causal;
  // at least 120 KiB so that two CTAs (each wanting all 512 TMEM columns) never share an SM
  size_t smem = (TILES + 4) * (BLOCK_M * D * 2) + sizeof(Shared) + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;
  auto kernel = attn_fwd_tc_kernel<T, D, FMT>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return std::string("attn_fwd: ") + cudaGetErrorString(e);
  std::string werr;
  const WorkListCache::Key key{0, (int)p.bh, (int)p.rows, (int)p.n_ctx, p.causal, ctx.sm_count};
  const DeviceWorkList work = g_lists.get(
      key, [&] { return schedule_attn_fwd((int)p.bh, (int)p.rows, (int)p.n_ctx, p.causal != 0, ctx.sm_count); },
      ctx.stream, werr);
  if (!werr.empty()) return werr;
  kernel<<<work.ctas, NUM_THREADS, smem, ctx.stream>>>(maps[0], maps[1], maps[2], prm, work, ctx.status);
  ++*ctx.launches;
  e = cudaGetLastError();
  if (e != cudaSuccess) return std::string("attn_fwd launch failed: ") + cudaGetErrorString(e);
  return std::string();
}

}  // namespace

bool attn_fwd_tc_eligible(const AttnProblem& p, std::string* why) {
  auto no = [&](const char* m) {
    if (why) *why = m;
    return false;
  };
  if (p.elt == Elt::F32) return no("fp32 attention takes the generic kernel");
  if (p.head_dim != 64 && p.head_dim != 128) return no("head dimension is not 64 or 128");
  if (p.stride_seq != p.head_dim) return no("rows are not contiguous (stride_seq != head_dim)");
  if (p.stride_head % 8) return no("stride_head is not a multiple of 16 bytes");
  if (p.stride_head < p.n_ctx * p.stride_seq) return no("heads overlap");
  if (((uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.out0) % 16)
    return no("base pointers are not 16-byte aligned");
  if (p.n_ctx < 128) return no("sequence shorter than one 128-row tile");
  if (p.n_ctx > 0x7fffffff / 256 || p.bh > 65535 || (p.rows / 256 + 1) * p.bh > 0x7fffffff)
    return no("extent out of range");
  if (!(p.sm_scale > 0.f)) return no("softmax scale is not positive");
  return true;
}

std::string launch_attn_fwd_tc(const AttnProblem& p, const LaunchCtx& ctx) {
  if (p.elt == Elt::BF16) {
    return p.head_dim == 64
               ? launch_typed<__nv_bfloat16, 64, 1>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16)
               : launch_typed<__nv_bfloat16, 128, 1>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  }
  return p.head_dim == 64 ? launch_typed<__half, 64, 0>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16)
                          : launch_typed<__half, 128, 0>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
}

}  // namespace tmc
