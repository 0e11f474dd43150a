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
//   warps 0-15  softmax: tile t = warp / 8; inside a tile warps 0-3 own columns 0-63
//               of every 128-column score block and warps 4-7 columns 64-127.  A thread
//               owns one query row (its TMEM lane) and 64 columns: max over them, one
//               exchange of the half-row maxima through shared memory, then exp2 /
//               partial sum / round, writing the 16-bit P back over the scores it read.
//   warp 16     TMA: Q (both tiles) once per query block, then K and V blocks of 128
//               keys into 2-stage rings
//   warp 17     MMA issuer: S_t = Q_t K^T (128x128xD, operands in shared memory),
//               O_t += P_t V (128xDx128, P read from TMEM)
// The running max used for the exponentials only advances when it grew by more
// than 8 (log2 units): P stays <= 256 and most iterations skip the O rescale in
// TMEM; O/l at the end is exact either way.  The element-wise code is kept short
// (64 columns per thread, no full unrolling over the row): straight-line code for a
// whole row does not stay resident in the instruction cache and ran 1.6x slower.
// Measured against this arrangement and slower on causal shapes (6 % at S4096, equal without a
// mask): eight softmax warps with one thread per row and the whole row in registers (registers
// traded between warpgroups, the exponential pass ordered by hand) - no exchange of maxima and
// one TMEM read per block, but one warp per scheduler instead of two wherever a tile works
// alone (the first and last blocks of every item, a quarter of a causal item), and four times
// the straight-line code.
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
constexpr int NUM_THREADS = 576;                // 16 softmax warps + TMA warp + MMA warp
constexpr int LOAD_WARP = 16, MMA_WARP = 17;
constexpr int HALF_N = BLOCK_N / 2;             // columns of a score tile owned by one softmax group
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
  float half_max[TILES][2][2][BLOCK_M];   // [tile][block parity][column half][row]
  float half_sum[TILES][2][BLOCK_M];      // [tile][column half][row]
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

// ---- softmax passes over one 128-column score tile in TMEM ------------------------
// Both passes are written as short loops (two 32-column chunks per trip, the next chunk's
// tcgen05.ld in flight while the current one is processed) rather than fully unrolled:
// the softmax warps execute this code once per key block, and straight-line code for 128
// columns does not stay resident in the instruction cache.
struct MaskInfo {
  int n0, q_row, n_ctx, causal;
  __device__ __forceinline__ bool masked(int col) const {
    const int key = n0 + col;
    return key >= n_ctx || (causal && key > q_row);
  }
  // Every column from `col` on is masked for all 32 rows of this warp (which start at a multiple
  // of 32): right of the causal diagonal, or past the end of the sequence.  Uniform over the warp.
  __device__ __forceinline__ bool all_masked_from(int col) const {
    const int key = n0 + col;
    return key >= n_ctx || (causal && key > (q_row | 31));
  }
};

// Row max of this thread's 64 columns (raw scores).
template <bool MASKED>
__device__ __forceinline__ float max_half(uint32_t s_tmem, const MaskInfo& mi) {
  uint32_t ra[32], rb[32];
  tmem_ld_32x32(s_tmem, ra);
  tmem_ld_32x32(s_tmem + 32, rb);
  tmem_ld_wait();
  float m0 = -INFINITY, m1 = -INFINITY;
  if (!MASKED) {
    float m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      // four chains of three-input maxima
      m0 = max3(m0, __uint_as_float(ra[i]), __uint_as_float(ra[i + 1]));
      m1 = max3(m1, __uint_as_float(ra[i + 2]), __uint_as_float(ra[i + 3]));
      m2 = max3(m2, __uint_as_float(rb[i]), __uint_as_float(rb[i + 1]));
      m3 = max3(m3, __uint_as_float(rb[i + 2]), __uint_as_float(rb[i + 3]));
    }
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    if (!mi.masked(i)) m0 = fmaxf(m0, __uint_as_float(ra[i]));
    if (!mi.masked(32 + i)) m1 = fmaxf(m1, __uint_as_float(rb[i]));
  }
  return fmaxf(m0, m1);
}

// P = exp2(s*qk_scale + neg_m) for 32 columns, rounded to T and written to `dst` (16 packed
// columns); returns the fp32 sum.  Off the mask boundary the scaling and the sum run two wide
// (fma.f32x2 / add.f32x2) and the row max uses three-input maxima: 1.2 % of the kernel, measured.  The special-function unit runs at about 80% of its rate
// over the whole kernel (16384 exponentials per score tile).  Moving one exponential in 2, 4
// or 8 to a cubic on the FMA pipe, and taking two at a time in the 16-bit type, were all
// measured equal or slower: the extra instructions cost as much issue time as they save.
template <typename T, bool MASKED>
__device__ __forceinline__ float exp_chunk(const uint32_t (&r)[32], uint32_t dst, float qk_scale,
                                           float neg_m, int col0, const MaskInfo& mi) {
  uint32_t packed[16];
  float s0 = 0.f, s1 = 0.f;
  if (MASKED && mi.all_masked_from(col0)) {
    // nothing of this chunk survives for any row of the warp: P = 0 without the exponentials
#pragma unroll
    for (int i = 0; i < 16; ++i) packed[i] = 0u;
    tmem_st_32x16(dst, packed);
    return 0.f;
  }
  if (!MASKED) {
    const uint64_t scale2 = pack_f32x2(qk_scale, qk_scale), neg_m2 = pack_f32x2(neg_m, neg_m);
    uint64_t acc = pack_f32x2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float x0, x1;
      unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), scale2, neg_m2), x0, x1);
      const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
      acc = add_f32x2(acc, pack_f32x2(p0, p1));
      packed[i / 2] = pack2<T>(p0, p1);
    }
    tmem_st_32x16(dst, packed);
    unpack_f32x2(acc, s0, s1);
    return s0 + s1;
  }
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

// Exponentials of this thread's 64 columns; P goes back over the first 32 of them.
template <typename T, bool MASKED>
__device__ __forceinline__ float exp_half(uint32_t s_tmem, float qk_scale, float neg_m, const MaskInfo& mi) {
  uint32_t ra[32], rb[32];
  tmem_ld_32x32(s_tmem, ra);
  tmem_ld_32x32(s_tmem + 32, rb);
  tmem_ld_wait();
  float sum = exp_chunk<T, MASKED>(ra, s_tmem, qk_scale, neg_m, 0, mi);
  sum += exp_chunk<T, MASKED>(rb, s_tmem + 16, qk_scale, neg_m, 32, mi);
  return sum;
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
      mbar_init(smem_u32(&ss.p_full[t]), 8);
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
          mma_f16_ss_elect(tmem + S_COL + t * BLOCK_N, qb.at(off), kb.at(off), idesc_qk, kk != 0);
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
                  // P: TMEM operand, 16 keys = 8 packed 32-bit columns; keys 0-63 sit at the start
                  // of the score buffer, keys 64-127 at its column 64 (one piece per softmax group).
                  // V: MN-major, 16 keys = 2048 bytes further, 64-column halves HALF_BYTES apart.
                  mma_f16_ts_elect(tmem + O_COL + t * D,
                             tmem + S_COL + t * BLOCK_N + (kk / 4) * HALF_N + (kk % 4) * 8,
                             vb.at(kk * 2048), idesc_pv, (j | kk) != 0);
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
  } else {
    // ---------------------------------------------------------------- softmax
    // Tile t = warp / 8; within a tile, warps 0-3 own columns 0-63 of every score block and
    // warps 4-7 columns 64-127.  The two threads that share a row exchange their half-row
    // maxima through shared memory once per block and otherwise work independently (each
    // keeps a partial row sum; the halves are added at the end).
    const int t = warp / 8;
    const int half = (warp / 4) & 1;
    const int row_in_tile = (warp % 4) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp % 4) * 32) << 16;
    const uint32_t s_tmem = tmem + lane_addr + S_COL + t * BLOCK_N + half * HALF_N;
    const uint32_t o_tmem = tmem + lane_addr + O_COL + t * D + half * (D / 2);
    const float qk_scale = prm.sm_scale * kLog2e;
    const int pair_barrier = 1 + t;               // named barrier of the tile's 256 threads
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
        for (int j = 0; j < my_blocks && ok; ++j, ++c) {
          // A wait that gave up is not acted on alone: the flag goes through the tile's named
          // barrier below, and all 256 threads leave in this same iteration.
          const bool got = mbar_wait(smem_u32(&ss.s_full[t]), c & 1, wc, kSoftS);
          tc_fence_after();
          const int n0 = j * BLOCK_N + half * HALF_N;
          const bool boundary = (n0 + HALF_N > prm.n_ctx) || (prm.causal && n0 + HALF_N > m0 + t * BLOCK_M);
          const MaskInfo mi{n0, q_row, prm.n_ctx, prm.causal};
          // pass 1: max of the raw scores over this half row, then over the whole row
          // (qk_scale > 0, so the scaled max is max * qk_scale)
          // (after a failed wait the scores read here are stale: harmless, the block is abandoned)
          float mx = boundary ? max_half<true>(s_tmem, mi) : max_half<false>(s_tmem, mi);
          ss.half_max[t][c & 1][half][row_in_tile] = mx;
          if (!bar_sync_and(pair_barrier, 256, got)) { ok = false; break; }
          mx = fmaxf(mx, ss.half_max[t][c & 1][half ^ 1][row_in_tile]) * qk_scale;
          // advance the working max only when it moved far (or on the first block); both
          // threads of a row see the same numbers and take the same decision
          float alpha = 1.f;
          bool rescale = false;
          if (mx > m_used + kRescaleThreshold) {
            alpha = fast_exp2(m_used - mx);      // 0 on the first block (m_used = -inf)
            m_used = mx;
            rescale = j > 0;
          }
          if (__any_sync(0xffffffffu, rescale)) {
            // O_t may only be touched once the P.V MMA of block j-1 has finished: it has, the
            // s_full this thread waited for above was committed after it.  Each half rescales
            // its own D/2 columns of the accumulator.
#pragma unroll 1
            for (int cc = 0; cc < D / 64; ++cc) {
              uint32_t r[32];
              tmem_ld_32x32(o_tmem + cc * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32(o_tmem + cc * 32, r);
            }
            tmem_st_wait();
          }
          // pass 2: exponentials, partial row sum, 16-bit P over the scores already read
          const float sum = boundary ? exp_half<T, true>(s_tmem, qk_scale, -m_used, mi)
                                     : exp_half<T, false>(s_tmem, qk_scale, -m_used, mi);
          l = l * alpha + sum;
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ss.p_full[t]));   // one arrival per warp
        }
        // ---- whole-row sum, O / l and the row statistic of this query block
        ss.half_sum[t][half][row_in_tile] = l;
        // the last P.V must have retired before O is read; the outcome of that wait, too, is
        // agreed on by the whole tile at the barrier that publishes the half-row sums
        if (ok && my_blocks > 0) ok = mbar_wait(smem_u32(&ss.pv_done[t]), item & 1, wc, kSoftFinal);
        ok = bar_sync_and(pair_barrier, 256, ok);
        l += ss.half_sum[t][half ^ 1][row_in_tile];
        tc_fence_after();
        if (ok && my_blocks > 0) {
          const float inv_l = 1.f / l;
          const bool live = q_row < prm.rows;
          T* orow = (T*)prm.o + (int64_t)bh * prm.stride_head + (int64_t)q_row * prm.stride_seq + half * (D / 2);
#pragma unroll 1
          for (int cc = 0; cc < D / 64; ++cc) {
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
          if (live && half == 0 && prm.lse) prm.lse[(int64_t)bh * prm.stride_lse + q_row] = m_used + log2f(l);
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
