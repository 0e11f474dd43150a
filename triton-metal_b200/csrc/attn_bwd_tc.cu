// attn_bwd_dq and attn_bwd_dkdv on tcgen05 / TMEM for 16-bit elements, head
// dimension 64 or 128, optional causal mask.
//
// Semantics: Sources/TritonMetalBench/AttentionBackwardKernel.swift:151-344 (dq)
// and :354-575 (dkdv).  P is rebuilt from the forward's row statistic L (log2
// units): P = exp2(qk_scale * QK^T - L);  dP = dO V^T;  dS = P (dP - Delta);
// dQ = sm_scale dS K;  dV = P^T dO;  dK = sm_scale dS^T Q.  dS and P are
// rounded to the element type before they enter a contraction.  The two
// directions stay separate kernels, as in the reference, so every gradient is
// deterministic (no atomics).
//
// Both kernels are persistent: one CTA per SM walks its list of work items - 128 resident rows
// of one (batch, head) (queries for dq, keys for dkdv); the other side streams through in
// blocks of 128 rows (MMAs with N = 128:
// narrower score tiles ran the tensor pipe at half rate, measured).
// Warp 16 issues TMA loads, warp 17 - converged, one lane elected per instruction - issues every
// tcgen05.mma, and four warpgroups (warps
// 0-15) do the exponentials and products: a thread owns one resident row (its TMEM lane)
// and one quarter of the 128 columns of a block, so the TMEM round trips of one group are
// covered by the arithmetic of the others.  The element-wise warps copy a fresh score (or
// dP) tile into registers and release its TMEM columns at once, so that the next MMA into
// those columns does not wait for the exponentials.  dS (and P in dq) go back into TMEM over
// the fp32 columns they were computed from and feed the next MMA as TMEM operands; P^T in
// dkdv goes through shared memory (see there).  Measured on a B200, per SM: a tcgen05.mma
// costs its issuer about 57 cycles from one lane of a diverged warp and 39 from a converged
// warp, whatever its size (a 128 x 128 x 16 one occupies the tensor pipe for 64, and N = 64
// runs at half rate), a tcgen05.commit or a completed barrier wait about 50, a branch of the
// lone issuing warp tens of cycles; two issuing warps interleave their MMAs and were slower;
// ex2.approx runs at 16 per cycle.
//
// TMEM columns (512):  dq:    S[2] (dS aliases) | dP | dQ
//                      dkdv:  S^T | dP^T (dS^T aliases) | dV | dK
//
// HBM layout: Q, K, V, dO, dQ, dK, dV [BH, S, D] with D contiguous; L, Delta
// [BH, S] fp32.

#include "attn_schedule.h"
#include "sm100_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tmc {
namespace {

using namespace ptx;

constexpr int BLK = 128;              // rows per tile on both sides
constexpr int GROUPS = 4;             // element-wise groups (four warps each)
constexpr int GCOLS = BLK / GROUPS;   // columns of a block owned by one group
constexpr int EW_THREADS = GROUPS * 128;
constexpr int LOAD_WARP = 16, MMA_WARP = 17;
constexpr int NUM_THREADS = 576;      // warps 0-15 element-wise, 16 TMA, 17 MMA
constexpr int TMEM_COLS = 512;
constexpr float kLog2e = 1.44269504088896340736f;

struct Params {
  void* out0;         // dQ | dK
  void* out1;         // dV
  const float* lse;
  const float* delta;
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
template <typename T> __device__ __forceinline__ void unpack2(uint32_t u, float& lo, float& hi);
template <> __device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t u, float& lo, float& hi) {
  lo = __uint_as_float(u << 16);
  hi = __uint_as_float(u & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack2<__half>(uint32_t u, float& lo, float& hi) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u));
  lo = f.x;
  hi = f.y;
}

template <int D>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar, int row0,
                                          int bh) {
#pragma unroll
  for (int h = 0; h < D / 64; ++h) tma_load_3d(dst + h * (BLK * 128), map, bar, h * 64, row0, bh);
}

// D_tmem[128 x 128] = A[128 x D] * B[128 x D]^T, both K-major tiles.
template <int D>
__device__ __forceinline__ void mma_nt(uint32_t d_tmem, SmemDesc a, SmemDesc b, uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const uint32_t off = (kk / 4) * (BLK * 128) + (kk % 4) * 32;
    mma_f16_ss_elect(d_tmem, a.at(off), b.at(off), idesc, kk != 0);
  }
}

// D_tmem[128 x D] (+)= A_tmem[128 x 128] * B[128 x D]; B a row-major (MN-major) tile of
// 128 rows.  The 16-bit A operand is stored by the element-wise groups in pieces: group g
// packs its 32 columns of the block into the 16 words at a_tmem + 32 g.
template <int D>
__device__ __forceinline__ void mma_tn(uint32_t d_tmem, uint32_t a_tmem, SmemDesc b, uint32_t idesc,
                                       bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < BLK / 16; ++kk)
    mma_f16_ts_elect(d_tmem, a_tmem + (kk / 2) * GCOLS + (kk % 2) * 8, b.at(kk * 2048), idesc, accumulate || kk != 0);
}

// D_tmem[128 x D] (+)= A[128 x 128] * B[128 x D]: A a K-major 128 x 128 tile in shared memory
// (two 64-column atoms), B a row-major (MN-major) tile of 128 rows.
template <int D>
__device__ __forceinline__ void mma_sn(uint32_t d_tmem, SmemDesc a, SmemDesc b, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < BLK / 16; ++kk)
    mma_f16_ss_elect(d_tmem, a.at((kk / 4) * (BLK * 128) + (kk % 4) * 32), b.at(kk * 2048), idesc, accumulate || kk != 0);
}

// Descriptors of a K-major tile (operand of mma_nt) and of a row-major tile used as the
// MN-major B operand of mma_tn, built once per kernel; `advanced` selects a ring stage.
__device__ __forceinline__ SmemDesc kmajor(uint32_t addr) { return make_desc_sw128(addr, 0, 1024); }
__device__ __forceinline__ SmemDesc mnmajor(uint32_t addr) { return make_desc_sw128(addr, BLK * 128, 1024); }

__device__ __forceinline__ void drain(uint32_t bar, uint32_t parity, const WaitCtx& wc, uint32_t site) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitCycles) { report_timeout(wc, site, parity); break; }
  }
}

// ---- element-wise passes over one group's 32 columns of a block --------------------
// Sixteen warps share the work so that four are resident on every scheduler: the passes are
// chains of TMEM round trips and special-function latency, and with two warps per scheduler
// (64 columns per thread) they, not the tensor pipe, set the time of an iteration.
struct KeyMask {
  int n0, q_row, n_ctx, causal;
  __device__ __forceinline__ bool masked(int col) const {
    const int key = n0 + col;
    return key >= n_ctx || (causal && key > q_row);
  }
};

// dq: dS = exp2(S*qk_scale - L) * (dP - Delta), rounded, written over S, from the register
// copies `s` and `d` of the group's 32 columns of S and dP; km.n0 is the first column's key.
template <typename T, bool MASKED>
__device__ __forceinline__ void ds_part(uint32_t s_tmem, const uint32_t (&s)[32], const uint32_t (&d)[32],
                                        float qk_scale, float neg_lse, float delta, const KeyMask& km) {
  uint32_t packed[16];
  if (!MASKED) {
    // two elements per instruction wherever the hardware has one (fma / add / mul on register
    // pairs): per element half an fma, the exponential, half an add, half a mul, half a conversion
    const uint64_t scale2 = pack_f32x2(qk_scale, qk_scale), neg_lse2 = pack_f32x2(neg_lse, neg_lse);
    const uint64_t neg_delta2 = pack_f32x2(-delta, -delta);
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float x0, x1, r0, r1;
      unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), scale2, neg_lse2), x0, x1);
      const uint64_t p2 = pack_f32x2(fast_exp2(x0), fast_exp2(x1));
      const uint64_t t2 = add_f32x2(pack_f32x2(__uint_as_float(d[i]), __uint_as_float(d[i + 1])), neg_delta2);
      unpack_f32x2(mul_f32x2(p2, t2), r0, r1);
      packed[i / 2] = pack2<T>(r0, r1);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float p0 = fast_exp2(fmaf(__uint_as_float(s[i]), qk_scale, neg_lse));
      float p1 = fast_exp2(fmaf(__uint_as_float(s[i + 1]), qk_scale, neg_lse));
      if (km.masked(i)) p0 = 0.f;
      if (km.masked(i + 1)) p1 = 0.f;
      packed[i / 2] = pack2<T>(p0 * (__uint_as_float(d[i]) - delta), p1 * (__uint_as_float(d[i + 1]) - delta));
    }
  }
  tmem_st_32x16(s_tmem, packed);
}

// 2^x for a pair of values on the fma pipe instead of the special-function unit: x is split into
// its nearest integer n and f = x - n in [-0.5, 0.5] by the add-a-big-constant trick, 2^f is a
// cubic (relative error 1e-4, an order below one bf16 / f16 rounding of the result), and n goes
// into the exponent field with an integer multiply-add.  x is clamped at -125 from below
// (everything smaller would be a denormal; the result there is < 2^-125).
__device__ __forceinline__ void exp2_cubic_x2(uint64_t x, float& r0, float& r1) {
  float x0, x1;
  unpack_f32x2(x, x0, x1);
  const uint64_t xc = pack_f32x2(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
  const uint64_t magic = pack_f32x2(12582912.f, 12582912.f);          // 1.5 * 2^23
  const uint64_t t = add_f32x2(xc, magic);                            // low mantissa bits = round(x)
  const uint64_t n = add_f32x2(t, pack_f32x2(-12582912.f, -12582912.f));
  const uint64_t f = fma_f32x2(n, pack_f32x2(-1.f, -1.f), xc);
  uint64_t p = fma_f32x2(f, pack_f32x2(0.05500893f, 0.05500893f), pack_f32x2(0.24221095f, 0.24221095f));
  p = fma_f32x2(p, f, pack_f32x2(0.6932829f, 0.6932829f));
  p = fma_f32x2(p, f, pack_f32x2(1.f, 1.f));
  float p0, p1, t0, t1;
  unpack_f32x2(p, p0, p1);
  unpack_f32x2(t, t0, t1);
  // bits(p) + (bits(t) << 23): the shift drops the constant's bits and leaves n in the exponent
  r0 = __uint_as_float(__float_as_uint(t0) * 0x800000u + __float_as_uint(p0));
  r1 = __uint_as_float(__float_as_uint(t1) * 0x800000u + __float_as_uint(p1));
}

// dkdv pass A: P^T = exp2(S^T*qk_scale - L[query]) from the register copy `s` of the group's
// 32 columns, rounded and packed (16 words).  `neg_lse_s` holds -L of the 32 queries (the sign is
// flipped once when the statistics are staged, so that the scaling is one two-wide fma per pair).
// `k_minus_q0` > column means key row > query: masked.
// `CUBIC` is a mask over every eight pairs of columns: the pairs whose bit is set take the cubic
// on the fma pipe instead of ex2.  At D = 64, where the exponentials and not the MMAs bound the
// kernel, a quarter of them there is worth 5 % of the kernel's time (measured); a half is a loss.
template <typename T, bool DIAG, uint32_t CUBIC>
__device__ __forceinline__ void pt_part(const uint32_t (&s)[32], float qk_scale, const float* neg_lse_s,
                                        int k_minus_q0, uint32_t (&keep)[16]) {
  const uint64_t scale2 = pack_f32x2(qk_scale, qk_scale);
  auto exp2_pair = [](uint64_t x, int pair, float& r0, float& r1) {
    if ((CUBIC >> (pair & 7)) & 1u) {
      exp2_cubic_x2(x, r0, r1);
    } else {
      float x0, x1;
      unpack_f32x2(x, x0, x1);
      r0 = fast_exp2(x0);
      r1 = fast_exp2(x1);
    }
  };
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float4 nl = *reinterpret_cast<const float4*>(neg_lse_s + i);
    float p0, p1, p2, p3;
    exp2_pair(fma_f32x2(pack_f32x2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), scale2, pack_f32x2(nl.x, nl.y)),
              i / 2, p0, p1);
    exp2_pair(fma_f32x2(pack_f32x2(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3])), scale2, pack_f32x2(nl.z, nl.w)),
              i / 2 + 1, p2, p3);
    if (DIAG) {
      if (k_minus_q0 > i) p0 = 0.f;
      if (k_minus_q0 > i + 1) p1 = 0.f;
      if (k_minus_q0 > i + 2) p2 = 0.f;
      if (k_minus_q0 > i + 3) p3 = 0.f;
    }
    keep[i / 2] = pack2<T>(p0, p1);
    keep[i / 2 + 1] = pack2<T>(p2, p3);
  }
}

// dkdv pass B: dS^T = P^T * (dP^T - Delta[query]) from the register copy of P^T; `neg_delta_s`
// holds -Delta of the 32 queries.
template <typename T>
__device__ __forceinline__ void dst_part(uint32_t dpt_tmem, const float* neg_delta_s, const uint32_t (&keep)[16]) {
  float4 nd[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) nd[i] = *reinterpret_cast<const float4*>(neg_delta_s + i * 4);
  uint32_t d[32];
  tmem_ld_32x32(dpt_tmem, d);
  tmem_ld_wait();
  uint32_t packed[16];
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float4 dl = nd[i / 4];
    float p0, p1, p2, p3, r0, r1, r2, r3;
    unpack2<T>(keep[i / 2], p0, p1);
    unpack2<T>(keep[i / 2 + 1], p2, p3);
    const uint64_t ta = add_f32x2(pack_f32x2(__uint_as_float(d[i]), __uint_as_float(d[i + 1])), pack_f32x2(dl.x, dl.y));
    const uint64_t tb = add_f32x2(pack_f32x2(__uint_as_float(d[i + 2]), __uint_as_float(d[i + 3])), pack_f32x2(dl.z, dl.w));
    unpack_f32x2(mul_f32x2(pack_f32x2(p0, p1), ta), r0, r1);
    unpack_f32x2(mul_f32x2(pack_f32x2(p2, p3), tb), r2, r3);
    packed[i / 2] = pack2<T>(r0, r1);
    packed[i / 2 + 1] = pack2<T>(r2, r3);
  }
  tmem_st_32x16(dpt_tmem, packed);
}

// Read-out of `COLS` columns of a fp32 accumulator row: scale, round, store.
template <typename T, int COLS>
__device__ __forceinline__ void store_rows(uint32_t acc_tmem, T* orow, float scale, bool live) {
#pragma unroll 1
  for (int c = 0; c < COLS / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(acc_tmem + c * 32, r);
    tmem_ld_wait();
    if (live) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        uint4 out;
        out.x = pack2<T>(__uint_as_float(r[v * 8 + 0]) * scale, __uint_as_float(r[v * 8 + 1]) * scale);
        out.y = pack2<T>(__uint_as_float(r[v * 8 + 2]) * scale, __uint_as_float(r[v * 8 + 3]) * scale);
        out.z = pack2<T>(__uint_as_float(r[v * 8 + 4]) * scale, __uint_as_float(r[v * 8 + 5]) * scale);
        out.w = pack2<T>(__uint_as_float(r[v * 8 + 6]) * scale, __uint_as_float(r[v * 8 + 7]) * scale);
        *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = out;
      }
    }
  }
}

// ===========================================================================
// dQ
// ===========================================================================
constexpr int K_STAGES = 3, V_STAGES = 2;

struct SharedDq {
  alignas(8) uint64_t qdo_full, qdo_empty;
  alignas(8) uint64_t k_full[K_STAGES], k_empty[K_STAGES], v_full[V_STAGES], v_empty[V_STAGES];
  alignas(8) uint64_t s_full[2];
  alignas(8) uint64_t dp_full, dp_read, ds_full, dq_done;
  uint32_t tmem_base;
  int abort_flag;
};

// Work of a persistent kernel: every CTA walks its own list of items (attn_schedule.h), an item
// being one (batch, head) and one 128-row tile of the resident side.  Under a causal mask the
// tiles differ in length - query tile i sees i + 1 key blocks, key tile i is seen by T - i query
// blocks - and the lists are balanced on the host.

// Pipeline of block j (keys j*128 ...):
//   MMA   S(j) = Q K(j)^T into S[j&1]            (issued two blocks ahead)
//   MMA   dP(j) = dO V(j)^T into the single dP buffer, as soon as the element-wise warps have
//         loaded dP(j-1) into registers (they signal that before they start computing)
//   elem  dS(j) written over S[j&1]
//   MMA   dQ += dS(j) K(j)
// so the chain from one block's element-wise pass to the next is one MMA (dP) long.
// Persistent: one CTA per SM walks its units; barrier phases follow running counters (`item`
// query tiles, `c` key blocks), the K and V rings run on across tiles, and the loads and first
// MMAs of the next tile go out while the element-wise warps still store the current dQ.
template <typename T, int D, uint32_t FMT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                      Params prm, DeviceWorkList work, DeviceStatus* status) {
  constexpr int TILE = BLK * D * 2;
  constexpr int S_COL = 0, DP_COL = 256, DQ_COL = 384;     // S[b] at b*128
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t q_addr = smem_u32(smem), do_addr = q_addr + TILE, k_addr = do_addr + TILE,
                 v_addr = k_addr + K_STAGES * TILE;
  SharedDq& ss = *reinterpret_cast<SharedDq*>(smem + (2 + K_STAGES + V_STAGES) * TILE);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  WaitCtx wc{&ss.abort_flag, status};
  // key blocks the query tile starting at row m0 walks
  auto key_blocks = [&](int m0) {
    int key_end = prm.n_ctx;
    if (prm.causal) key_end = min(prm.n_ctx, m0 + BLK);
    return (key_end + BLK - 1) / BLK;
  };

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ss.qdo_full), 1);
    mbar_init(smem_u32(&ss.qdo_empty), 1);
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(smem_u32(&ss.k_full[s]), 1);
      mbar_init(smem_u32(&ss.k_empty[s]), 1);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(smem_u32(&ss.v_full[s]), 1);
      mbar_init(smem_u32(&ss.v_empty[s]), 1);
    }
    mbar_init(smem_u32(&ss.s_full[0]), 1);
    mbar_init(smem_u32(&ss.s_full[1]), 1);
    mbar_init(smem_u32(&ss.dp_full), 1);
    mbar_init(smem_u32(&ss.dp_read), EW_THREADS / 32);
    mbar_init(smem_u32(&ss.ds_full), EW_THREADS / 32);
    mbar_init(smem_u32(&ss.dq_done), 1);
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

  if (warp == LOAD_WARP) {
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      tma_prefetch_desc(&map_do);
      // ring positions run on across tiles; K is two blocks ahead of V inside a tile
      uint32_t item = 0, k_issued = 0, v_issued = 0;
      bool ok = true;
      auto load_k = [&](int j, int bh) {
        const int s = k_issued % K_STAGES;
        if (!mbar_wait(smem_u32(&ss.k_empty[s]), ((k_issued / K_STAGES) & 1) ^ 1, wc, 31)) return false;
        mbar_expect_tx(smem_u32(&ss.k_full[s]), TILE);
        load_tile<D>(k_addr + s * TILE, &map_k, smem_u32(&ss.k_full[s]), j * BLK, bh);
        ++k_issued;
        return true;
      };
      auto load_v = [&](int j, int bh) {
        const int s = v_issued % V_STAGES;
        if (!mbar_wait(smem_u32(&ss.v_empty[s]), ((v_issued / V_STAGES) & 1) ^ 1, wc, 32)) return false;
        mbar_expect_tx(smem_u32(&ss.v_full[s]), TILE);
        load_tile<D>(v_addr + s * TILE, &map_v, smem_u32(&ss.v_full[s]), j * BLK, bh);
        ++v_issued;
        return true;
      };
      {
        for (WorkCursor w(work); w.valid() && ok; w.advance(), ++item) {
          const int bh = w.cur.x;
          const int m0 = w.cur.y * BLK;
          const int n_blocks = key_blocks(m0);
          // Q and dO are single-buffered: the previous tile's last S and dP must have retired
          if (!mbar_wait(smem_u32(&ss.qdo_empty), (item & 1) ^ 1, wc, 30)) { ok = false; break; }
          mbar_expect_tx(smem_u32(&ss.qdo_full), 2 * TILE);
          load_tile<D>(q_addr, &map_q, smem_u32(&ss.qdo_full), m0, bh);
          load_tile<D>(do_addr, &map_do, smem_u32(&ss.qdo_full), m0, bh);
          ok = load_k(0, bh) && load_v(0, bh);
          if (ok && n_blocks > 1) ok = load_k(1, bh);
          for (int j = 0; j < n_blocks && ok; ++j) {
            if (j + 1 < n_blocks && !load_v(j + 1, bh)) { ok = false; break; }
            if (j + 2 < n_blocks && !load_k(j + 2, bh)) { ok = false; break; }
          }
        }
      }
      // every copy started here must have landed before the CTA exits
      if (item) drain(smem_u32(&ss.qdo_full), (item - 1) & 1, wc, 39);
      for (uint32_t n = k_issued > K_STAGES ? k_issued - K_STAGES : 0; n < k_issued; ++n)
        drain(smem_u32(&ss.k_full[n % K_STAGES]), (n / K_STAGES) & 1, wc, 39);
      for (uint32_t n = v_issued > V_STAGES ? v_issued - V_STAGES : 0; n < v_issued; ++n)
        drain(smem_u32(&ss.v_full[n % V_STAGES]), (n / V_STAGES) & 1, wc, 39);
    }
  } else if (warp == MMA_WARP) {
    // One warp issues every MMA.  A tcgen05.mma costs its issuer about 39 cycles whatever its
    // size when the warp stays converged (57 from one diverged lane; a 128 x 128 x 16 one occupies
    // the pipe for 64), a commit or a barrier wait about 50 more, every branch tens of cycles.
    // the whole warp runs this loop, converged; one elected lane issues (see mma_f16_ss_elect)
    {
      constexpr uint32_t idesc_nt = make_idesc(FMT, BLK, BLK, 0, 0);
      constexpr uint32_t idesc_tn = make_idesc(FMT, BLK, D, 0, 1);
      const SmemDesc q_km = kmajor(q_addr), do_km = kmajor(do_addr), k_km = kmajor(k_addr), v_km = kmajor(v_addr);
      const SmemDesc k_mn = mnmajor(k_addr);
      auto wait = [&](uint64_t* bar, uint32_t parity, uint32_t site) {
        mbar_wait_warp(smem_u32(bar), parity, wc, site);
      };
      // running positions: c = key blocks done (S buffer c & 1, phases of dp/ds barriers),
      // K ring position of the block dQ uses next (ks, kp) and of the block S uses next
      // (ks2, kp2), V ring position (vs, vp)
      uint32_t item = 0, c = 0, c_qk = 0;
      int ks = 0, ks2 = 0, vs = 0;
      uint32_t kp2 = 0, vp = 0;
      auto issue_qk = [&]() {          // S of the next block not yet issued, into S[c_qk & 1]
        wait(&ss.k_full[ks2], kp2, 34);
        tc_fence_after();
        mma_nt<D>(tmem + S_COL + (c_qk & 1) * BLK, q_km, k_km.advanced(ks2 * TILE), idesc_nt);
        mma_commit_elect(smem_u32(&ss.s_full[c_qk & 1]));
        ++c_qk;
        if (++ks2 == K_STAGES) { ks2 = 0; kp2 ^= 1; }
      };
      auto issue_dp = [&]() {
        wait(&ss.v_full[vs], vp, 35);
        tc_fence_after();
        mma_nt<D>(tmem + DP_COL, do_km, v_km.advanced(vs * TILE), idesc_nt);
        mma_commit_elect(smem_u32(&ss.v_empty[vs]));
        mma_commit_elect(smem_u32(&ss.dp_full));
        if (++vs == V_STAGES) { vs = 0; vp ^= 1; }
      };
      // one key block: `next` = another block follows in this tile, `next2` = two do
      auto block = [&](bool first, bool next, bool next2) {
        if (next) {
          // the element-wise warps have dP(j) in registers: the next dP may overwrite it while
          // they are still working on block j
          wait(&ss.dp_read, c & 1, 41);
          issue_dp();
          // Q and dO are free once the tile's last S (issued a block earlier) and dP retire
          if (!next2) mma_commit_elect(smem_u32(&ss.qdo_empty));
        }
        wait(&ss.ds_full, c & 1, 36);
        tc_fence_after();
        mma_tn<D>(tmem + DQ_COL, tmem + S_COL + (c & 1) * BLK, k_mn.advanced(ks * TILE), idesc_tn, !first);
        mma_commit_elect(smem_u32(&ss.k_empty[ks]));
        if (!next) mma_commit_elect(smem_u32(&ss.dq_done));
        // S(j+2) reuses the buffer dS(j) sits in: MMAs run in issue order
        if (next2) issue_qk();
        ++c;
        if (++ks == K_STAGES) ks = 0;
      };
      {
        for (WorkCursor w(work); w.valid(); w.advance(), ++item) {
          const int n_blocks = key_blocks(w.cur.y * BLK);
          // The first S and dP of this tile go out while the element-wise warps may still be
          // storing the previous dQ: they use other TMEM columns, and the first dQ MMA waits
          // for ds_full, which those warps only signal after that store.
          wait(&ss.qdo_full, item & 1, 33);
          issue_qk();
          issue_dp();
          if (n_blocks > 1) issue_qk();
          else mma_commit_elect(smem_u32(&ss.qdo_empty));
          int j = 0;
          if (n_blocks > 2) {
            block(true, true, true);
            for (j = 1; j + 2 < n_blocks; ++j) block(false, true, true);
          }
          if (j + 1 < n_blocks) { block(j == 0, true, false); ++j; }
          block(j == 0, false, false);
        }
      }
    }
  } else if (warp < EW_THREADS / 32) {
    const int group = warp / 4;                   // owns columns group*32 ... of every block
    const int row_in_tile = (warp % 4) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp % 4) * 32) << 16;
    const float qk_scale = prm.sm_scale * kLog2e;
    uint32_t item = 0, c = 0;
    bool ok = true;
    {
      for (WorkCursor w(work); w.valid() && ok; w.advance(), ++item) {
        const int bh = w.cur.x;
        const int m0 = w.cur.y * BLK;
        const int n_blocks = key_blocks(m0);
        const int q_row = m0 + row_in_tile;
        float lse = 0.f, delta = 0.f;
        if (q_row < prm.n_ctx) {
          lse = prm.lse[(int64_t)bh * prm.stride_lse + q_row];
          delta = prm.delta[(int64_t)bh * prm.stride_lse + q_row];
        }
        for (int j = 0; j < n_blocks && ok; ++j, ++c) {
          if (!mbar_wait(smem_u32(&ss.s_full[c & 1]), (c >> 1) & 1, wc, 37)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&ss.dp_full), c & 1, wc, 38)) { ok = false; break; }
          tc_fence_after();
          const int n0 = j * BLK + group * GCOLS;
          const bool boundary = (n0 + GCOLS > prm.n_ctx) || (prm.causal && n0 + GCOLS > m0);
          const KeyMask km{n0, q_row, prm.n_ctx, prm.causal};
          const uint32_t s_tmem = tmem + lane_addr + S_COL + (c & 1) * BLK + group * GCOLS;
          const uint32_t dp_tmem = tmem + lane_addr + DP_COL + group * GCOLS;
          uint32_t sv[32], dv[32];
          tmem_ld_32x32(dp_tmem, dv);
          tmem_ld_32x32(s_tmem, sv);
          tmem_ld_wait();
          // dP(j) is in registers: let the next dP start
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ss.dp_read));
          if (boundary) ds_part<T, true>(s_tmem, sv, dv, qk_scale, -lse, delta, km);
          else ds_part<T, false>(s_tmem, sv, dv, qk_scale, -lse, delta, km);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ss.ds_full));   // one arrival per warp
        }
        if (ok) ok = mbar_wait(smem_u32(&ss.dq_done), item & 1, wc, 40);
        tc_fence_after();
        if (ok) {
          // the groups share the columns of dQ, 32 at a time
          constexpr int SC = 32;
          if (group * SC < D) {
            T* orow = (T*)prm.out0 + (int64_t)bh * prm.stride_head + (int64_t)q_row * prm.stride_seq + group * SC;
            store_rows<T, SC>(tmem + lane_addr + DQ_COL + group * SC, orow, prm.sm_scale, q_row < prm.rows);
          }
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

// ===========================================================================
// dK, dV
// ===========================================================================
constexpr int MAX_RING = 4;
// Stages of the Q and dO rings of dkdv.  At D = 128 shared memory is full (K, V, four streamed
// tiles and the P^T tile take 224 KiB): two stages each.  A Q tile is held from the scores of
// its block to the dK of that block, two blocks later, so the refill of the slot that dK(t-1)
// frees (about 1300 cycles for 32 KiB) sits in front of S^T(t+1) in every block - the issuing
// warp spends 1280 of a block's 3100 cycles waiting for it (timestamps taken inside the
// kernel).  Splitting the four tiles 3 + 1 moves the wait to dO (measured: 3400 cycles a
// block); a fifth tile does not fit.  At D = 64 there is room for four stages of each.
template <int D> __host__ __device__ constexpr int q_stages() { return D == 64 ? 4 : 2; }
template <int D> __host__ __device__ constexpr int do_stages() { return D == 64 ? 4 : 2; }

struct SharedDkdv {
  alignas(8) uint64_t kv_full, kv_empty;
  alignas(8) uint64_t q_full[MAX_RING][2], q_empty[MAX_RING], do_full[MAX_RING], do_empty[MAX_RING];   // q_full[stage][64-column half]
  alignas(8) uint64_t st_full, s_read, p_full, dpt_full, ds_full, done;
  alignas(16) float lse[2][BLK];
  alignas(16) float delta[2][BLK];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int P_TILE = BLK * BLK * 2;     // the 16-bit P^T tile in shared memory

// Pipeline of streamed query block t (S^T single-buffered in TMEM, all 512 columns taken):
//   MMA   S^T(t) = K Q(t)^T                     as soon as the element-wise warps hold S^T(t-1)
//                                               in registers (they signal that before computing)
//   elem  P^T(t) = exp2(...) -> shared memory   (K-major, 128-byte swizzle, like a loaded tile)
//   MMA   dV += P^T(t) dO(t)                    both operands from shared memory
//   MMA   dP^T(t) = V dO(t)^T                   issued one block ahead
//   elem  dS^T(t) = P^T (dP^T - Delta)          written over dP^T in TMEM
//   MMA   dK += dS^T(t) Q(t)                    A operand from TMEM
// P^T goes through shared memory because in TMEM it can only sit on top of S^T, and then
// S^T(t+1) has to wait for dV(t), which has to wait for the whole exponential pass: that chain
// (about 3500 cycles a block, measured) and not the 2048 cycles of tensor work set the pace.
// Persistent like dq: one CTA per SM walks its units; phases follow running counters (`item` key
// tiles, `c` query blocks), the Q and dO rings run on across tiles, and the next tile's K, V and
// first MMAs go out while the element-wise warps still store the current dK and dV.
template <typename T, int D, uint32_t FMT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_dkdv_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                        Params prm, DeviceWorkList work, DeviceStatus* status) {
  constexpr int TILE = BLK * D * 2;
  constexpr int NQ = q_stages<D>(), NDO = do_stages<D>();   // stages of the Q and dO rings
  constexpr int ST_COL = 0, DPT_COL = 128, DV_COL = 256, DK_COL = 256 + D;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  // layout: K | V | Q ring | dO ring | P^T | barriers and row statistics
  const uint32_t k_addr = smem_u32(smem), v_addr = k_addr + TILE, q_addr = v_addr + TILE,
                 do_addr = q_addr + NQ * TILE, p_addr = do_addr + NDO * TILE;
  SharedDkdv& ss = *reinterpret_cast<SharedDkdv*>(smem + (2 + NQ + NDO) * TILE + P_TILE);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  WaitCtx wc{&ss.abort_flag, status};
  const int total_q_blocks = (prm.n_ctx + BLK - 1) / BLK;
  // first query block that sees the key tile starting at row n0 (earlier queries never do)
  auto first_block = [&](int n0) { return prm.causal ? n0 / BLK : 0; };

  // the swizzled tiles need the 1024-byte alignment asked for above
  if (k_addr & 1023u) {
    if (threadIdx.x == 0) {
      ss.abort_flag = 0;
      report_timeout(wc, 62, k_addr);
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ss.kv_full), 1);
    mbar_init(smem_u32(&ss.kv_empty), 1);
    for (int s = 0; s < NQ; ++s) {
      mbar_init(smem_u32(&ss.q_full[s][0]), 1);
      mbar_init(smem_u32(&ss.q_full[s][1]), 1);
      mbar_init(smem_u32(&ss.q_empty[s]), 1);
    }
    for (int s = 0; s < NDO; ++s) {
      mbar_init(smem_u32(&ss.do_full[s]), 1);
      mbar_init(smem_u32(&ss.do_empty[s]), 1);
    }
    mbar_init(smem_u32(&ss.st_full), 1);
    mbar_init(smem_u32(&ss.s_read), EW_THREADS / 32);
    mbar_init(smem_u32(&ss.p_full), EW_THREADS / 32);
    mbar_init(smem_u32(&ss.dpt_full), 1);
    mbar_init(smem_u32(&ss.ds_full), EW_THREADS / 32);
    mbar_init(smem_u32(&ss.done), 1);
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

  if (warp == LOAD_WARP) {
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      tma_prefetch_desc(&map_do);
      uint32_t issued = 0, do_issued = 0;
      uint32_t item = 0, c = 0;          // key tiles and query blocks loaded so far
      bool ok = true;
      {
        for (WorkCursor w(work); w.valid() && ok; w.advance(), ++item) {
          const int bh = w.cur.x;
          const int n0 = w.cur.y * BLK;
          const int first = first_block(n0), n_iter = total_q_blocks - first;
          // K and V are single-buffered: the previous tile's last S^T and dP^T must have retired
          if (!mbar_wait(smem_u32(&ss.kv_empty), (item & 1) ^ 1, wc, 50)) { ok = false; break; }
          mbar_expect_tx(smem_u32(&ss.kv_full), 2 * TILE);
          load_tile<D>(k_addr, &map_k, smem_u32(&ss.kv_full), n0, bh);
          load_tile<D>(v_addr, &map_v, smem_u32(&ss.kv_full), n0, bh);
          for (int t = 0; t < n_iter; ++t, ++c) {
            const int sq = c % NQ, sd = c % NDO;
            const uint32_t phq = (c / NQ) & 1, phd = (c / NDO) & 1;
            const int row0 = (first + t) * BLK;
            // With two stages each (D = 128) dO(t)'s slot is freed by dV(t-2), half a block before
            // dK(t-2) frees Q(t)'s: dO goes first, so that the Q refill - 32 KiB, on the critical path
            // of S^T(t) - is not queued behind a wait for it (measured: 2 to 3 % of the kernel).  With
            // four stages both slots were freed long ago and Q, which S^T(t) waits for, goes first.
            constexpr bool DO_FIRST = NQ <= 2;
            auto load_do = [&]() -> bool {
              if (!mbar_wait(smem_u32(&ss.do_empty[sd]), phd ^ 1, wc, 52)) return false;
              mbar_expect_tx(smem_u32(&ss.do_full[sd]), TILE);
              load_tile<D>(do_addr + sd * TILE, &map_do, smem_u32(&ss.do_full[sd]), row0, bh);
              ++do_issued;
              return true;
            };
            if (DO_FIRST && !load_do()) { ok = false; break; }
            if (!mbar_wait(smem_u32(&ss.q_empty[sq]), phq ^ 1, wc, 51)) { ok = false; break; }
            // one barrier per 64-column half: the scores start on the first half while the second
            // is still in flight
#pragma unroll
            for (int h = 0; h < D / 64; ++h) {
              mbar_expect_tx(smem_u32(&ss.q_full[sq][h]), BLK * 128);
              tma_load_3d(q_addr + sq * TILE + h * (BLK * 128), &map_q, smem_u32(&ss.q_full[sq][h]), h * 64, row0, bh);
            }
            ++issued;
            if (!DO_FIRST && !load_do()) { ok = false; break; }
          }
        }
      }
      // every copy started here must have landed before the CTA exits
      if (item) drain(smem_u32(&ss.kv_full), (item - 1) & 1, wc, 59);
      for (uint32_t n = issued > NQ ? issued - NQ : 0; n < issued; ++n)
        for (int h = 0; h < D / 64; ++h) drain(smem_u32(&ss.q_full[n % NQ][h]), (n / NQ) & 1, wc, 59);
      for (uint32_t n = do_issued > NDO ? do_issued - NDO : 0; n < do_issued; ++n)
        drain(smem_u32(&ss.do_full[n % NDO]), (n / NDO) & 1, wc, 59);
    }
  } else if (warp == MMA_WARP) {
    // One warp issues every MMA (cost of issuing: see the head of this file): per block five
    // waits and five commits, no branch that does not depend on a barrier.
    // the whole warp runs this loop, converged; one elected lane issues (see mma_f16_ss_elect)
    {
      constexpr uint32_t idesc_nt = make_idesc(FMT, BLK, BLK, 0, 0);
      constexpr uint32_t idesc_tn = make_idesc(FMT, BLK, D, 0, 1);
      const SmemDesc k_km = kmajor(k_addr), v_km = kmajor(v_addr), q_km = kmajor(q_addr), do_km = kmajor(do_addr);
      const SmemDesc q_mn = mnmajor(q_addr), do_mn = mnmajor(do_addr), p_km = kmajor(p_addr);
      auto wait = [&](uint64_t* bar, uint32_t parity, uint32_t site) {
        mbar_wait_warp(smem_u32(bar), parity, wc, site);
      };
      // S^T = K Q(t)^T, one 64-column half of the head dimension at a time as Q's halves land
      auto issue_scores = [&](int stage, uint32_t parity) {
        const SmemDesc q = q_km.advanced(stage * TILE);
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          wait(&ss.q_full[stage][h], parity, 54);
          tc_fence_after();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const uint32_t off = h * (BLK * 128) + q4 * 32;
            mma_f16_ss_elect(tmem + ST_COL, k_km.at(off), q.at(off), idesc_nt, (h | q4) != 0);
          }
        }
        mma_commit_elect(smem_u32(&ss.st_full));
      };
      // One query block; c counts them across tiles (ring stages c mod NQ / NDO, phases from c).
      // `first` = first block of its key tile, `more` = another block of this tile follows;
      // every block but a tile's last also starts the next block's S^T and dP^T.
      uint32_t item = 0, c = 0;
      auto block = [&](bool first, bool more, bool release_kv) {
        const int sq = c % NQ, sd = c % NDO, sq_next = (c + 1) % NQ, sd_next = (c + 1) % NDO;
        const uint32_t phq_next = ((c + 1) / NQ) & 1, phd_next = ((c + 1) / NDO) & 1;
        if (more) {
          // S^T(t) is in registers and Q(t+1) has landed: the next scores can go
          wait(&ss.s_read, c & 1, 63);
          issue_scores(sq_next, phq_next);
        }
        wait(&ss.p_full, c & 1, 56);
        tc_fence_after();
        mma_sn<D>(tmem + DV_COL, p_km, do_mn.advanced(sd * TILE), idesc_tn, !first);
        mma_commit_elect(smem_u32(&ss.do_empty[sd]));         // last use of dO(t)
        wait(&ss.ds_full, c & 1, 57);
        tc_fence_after();
        mma_tn<D>(tmem + DK_COL, tmem + DPT_COL, q_mn.advanced(sq * TILE), idesc_tn, !first);
        mma_commit_elect(smem_u32(&ss.q_empty[sq]));          // last use of Q(t)
        if (more) {
          wait(&ss.do_full[sd_next], phd_next, 55);
          tc_fence_after();
          mma_nt<D>(tmem + DPT_COL, v_km, do_km.advanced(sd_next * TILE), idesc_nt);
          mma_commit_elect(smem_u32(&ss.dpt_full));
          // K and V are free once the tile's last S^T and dP^T (both just issued) retire
          if (release_kv) mma_commit_elect(smem_u32(&ss.kv_empty));
        } else {
          mma_commit_elect(smem_u32(&ss.done));
        }
        ++c;
      };
      {
        for (WorkCursor w(work); w.valid(); w.advance(), ++item) {
          const int n_iter = total_q_blocks - first_block(w.cur.y * BLK);
          // The first S^T and dP^T of this tile go out while the element-wise warps may still be
          // storing the previous dK and dV: they use other TMEM columns, and the first dV and dK
          // MMAs wait for p_full / ds_full, which those warps only signal after that store.
          wait(&ss.kv_full, item & 1, 53);
          issue_scores(c % NQ, (c / NQ) & 1);
          wait(&ss.do_full[c % NDO], (c / NDO) & 1, 55);
          tc_fence_after();
          mma_nt<D>(tmem + DPT_COL, v_km, do_km.advanced((c % NDO) * TILE), idesc_nt);
          mma_commit_elect(smem_u32(&ss.dpt_full));
          if (n_iter == 1) mma_commit_elect(smem_u32(&ss.kv_empty));
          int t = 0;
          if (n_iter > 2) {
            block(true, true, false);
            for (t = 1; t + 2 < n_iter; ++t) block(false, true, false);
          }
          if (t + 1 < n_iter) { block(t == 0, true, true); ++t; }
          block(t == 0, false, false);
        }
      }
    }
  } else if (warp < EW_THREADS / 32) {
    const int group = warp / 4;                   // owns query columns group*32 ... of every block
    const int row_in_tile = (warp % 4) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp % 4) * 32) << 16;
    const float qk_scale = prm.sm_scale * kLog2e;
    // This thread's 64 bytes of a P^T row in the K-major, 128-byte-swizzled tile: 64-query
    // atoms 16 KiB apart, rows of 128 bytes, 16-byte chunks XORed with the row (mod 8).
    const uint32_t p_row = p_addr + (group / 2) * (BLK * 128) + row_in_tile * 128;
    const uint32_t p_chunk0 = (group % 2) * 4, p_xor = row_in_tile & 7;
    uint32_t item = 0, c = 0;
    bool ok = true;
    {
      for (WorkCursor w(work); w.valid() && ok; w.advance(), ++item) {
        const int bh = w.cur.x;
        const float* lse_base = prm.lse + (int64_t)bh * prm.stride_lse;
        const float* delta_base = prm.delta + (int64_t)bh * prm.stride_lse;
        const int n0 = w.cur.y * BLK;
        const int first = first_block(n0), n_iter = total_q_blocks - first;
        const int k_row = n0 + row_in_tile;
        // Row statistics of the streamed query block go through shared memory (every thread
        // needs 32 of each): the threads of group 0 fetch the 128 values of L, those of group 1
        // the 128 values of Delta.  The global load for block t+1 is issued at the top of
        // iteration t into a register and stored to shared memory at its end, so its latency is
        // off the critical path.  Both are staged negated (the passes add them); -inf as -L makes
        // exp2(x - L) vanish for queries past the end.
        auto fetch_stat = [&](int t) -> float {
          const int q = (first + t) * BLK + row_in_tile;
          float v = group ? 0.f : INFINITY;
          if (group < 2 && q < prm.n_ctx) {
            const float* src = (group ? delta_base : lse_base) + q;
            asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(src));
          }
          return -v;           // the passes add: -L and -Delta are staged
        };
        auto put_stat = [&](uint32_t slot, float v) {
          if (group == 1) ss.delta[slot & 1][row_in_tile] = v;
          else if (group == 0) ss.lse[slot & 1][row_in_tile] = v;
        };
        // slot c & 1 was last read in block c - 2, two barriers ago
        put_stat(c, fetch_stat(0));
        for (int t = 0; t < n_iter; ++t, ++c) {
          // all element-wise threads: statistics of block t are visible, block t-1 is no longer read.
          // The barrier also carries every thread's "still fine" flag: a thread whose wait gave up
          // keeps walking (it skips the rest of its block) until this barrier, where all 512 leave
          // in the same iteration.
          if (!bar_sync_and(1, EW_THREADS, ok)) { ok = false; break; }
          float next_stat = 0.f;
          if (t + 1 < n_iter) next_stat = fetch_stat(t + 1);
          const float* lse_s = ss.lse[c & 1] + group * GCOLS;
          const float* delta_s = ss.delta[c & 1] + group * GCOLS;
          const int q0 = (first + t) * BLK + group * GCOLS;     // first query of this group's columns
          const bool diagonal = prm.causal && q0 < n0 + BLK;
          if (!mbar_wait(smem_u32(&ss.st_full), c & 1, wc, 58)) { ok = false; continue; }
          tc_fence_after();
          uint32_t sv[32];
          tmem_ld_32x32(tmem + lane_addr + ST_COL + group * GCOLS, sv);
          tmem_ld_wait();
          // S^T(t) is in registers: the next scores may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ss.s_read));
          uint32_t keep[16];
          constexpr uint32_t CUBIC = D == 64 ? 0x11u : 0u;     // pairs 0 and 4 of every eight
          if (diagonal) pt_part<T, true, CUBIC>(sv, qk_scale, lse_s, k_row - q0, keep);
          else pt_part<T, false, CUBIC>(sv, qk_scale, lse_s, 0, keep);
          // dV(t-1) must have read the previous P^T before it is replaced: dP^T(t) was issued after
          // it, so its commit covers it (and is waited for here instead of before the dS^T pass)
          if (!mbar_wait(smem_u32(&ss.dpt_full), c & 1, wc, 60)) { ok = false; continue; }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t dst = p_row + (((p_chunk0 + i) ^ p_xor) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(keep[4 * i]),
                         "r"(keep[4 * i + 1]), "r"(keep[4 * i + 2]), "r"(keep[4 * i + 3])
                         : "memory");
          }
          fence_proxy_async();          // the tensor core reads shared memory through the async proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ss.p_full));
          tc_fence_after();
          dst_part<T>(tmem + lane_addr + DPT_COL + group * GCOLS, delta_s, keep);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ss.ds_full));   // one arrival per warp
          if (t + 1 < n_iter) put_stat(c + 1, next_stat);
        }
        if (ok) ok = mbar_wait(smem_u32(&ss.done), item & 1, wc, 61);
        // agreed on by all 512 threads, so that they enter (or skip) the next key tile together
        ok = bar_sync_and(1, EW_THREADS, ok);
        tc_fence_after();
        if (ok) {
          // groups 0 and 1 store the halves of dV, groups 2 and 3 those of dK
          const bool live = k_row < prm.rows;
          const int c0 = (group & 1) * (D / 2);
          const int64_t row_off = (int64_t)bh * prm.stride_head + (int64_t)k_row * prm.stride_seq + c0;
          if (group < 2) store_rows<T, D / 2>(tmem + lane_addr + DV_COL + c0, (T*)prm.out1 + row_off, 1.f, live);
          else store_rows<T, D / 2>(tmem + lane_addr + DK_COL + c0, (T*)prm.out0 + row_off, prm.sm_scale, live);
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

template <typename T, int D>
std::string make_maps(const AttnProblem& p, CUtensorMapDataType type, CUtensorMap* maps) {
  const void* bases[4] = {p.q, p.k, p.v, p.d_o};
  for (int i = 0; i < 4; ++i) {
    uint64_t dims[3] = {(uint64_t)D, (uint64_t)p.n_ctx, (uint64_t)p.bh};
    uint64_t strides[2] = {(uint64_t)p.stride_seq * 2, (uint64_t)p.stride_head * 2};
    uint32_t box[3] = {64u, (uint32_t)BLK, 1u};
    std::string e = make_tensor_map(&maps[i], type, 3, bases[i], dims, strides, box);
    if (!e.empty()) return e;
  }
  return std::string();
}

Params make_params(const AttnProblem& p) {
  Params prm{};
  prm.out0 = p.out0;
  prm.out1 = p.out1;
  prm.lse = p.lse;
  prm.delta = p.delta;
  prm.sm_scale = p.sm_scale;
  prm.stride_head = p.stride_head;
  prm.stride_seq = p.stride_seq;
  prm.stride_lse = p.stride_lse;
  prm.n_ctx = (int)p.n_ctx;
  prm.rows = (int)p.rows;
  prm.causal = p.causal;
  return prm;
}

WorkListCache g_lists;     // work lists already in device memory, by problem shape

template <typename T, int D, uint32_t FMT>
std::string launch_typed(const AttnProblem& p, const LaunchCtx& ctx, CUtensorMapDataType type, bool dkdv) {
  CUtensorMap maps[4];
  std::string err = make_maps<T, D>(p, type, maps);
  if (!err.empty()) return err;
  Params prm = make_params(p);
  const char* what = dkdv ? "attn_bwd_dkdv" : "attn_bwd_dq";
  // never less than 120 KiB so two CTAs (each wanting all of TMEM) do not share an SM
  // dkdv: six operand tiles and the P^T tile, on a 1024-byte aligned base (no slack: 227 KiB
  // is the limit at D = 128); dq: its tiles plus slack for rounding the base up
  size_t smem = dkdv ? (2 + q_stages<D>() + do_stages<D>()) * (size_t)(BLK * D * 2) + P_TILE + sizeof(SharedDkdv)
                     : (2 + K_STAGES + V_STAGES) * (size_t)(BLK * D * 2) + sizeof(SharedDq) + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;
  cudaError_t e;
  std::string werr;
  const WorkListCache::Key key{dkdv ? 2 : 1, (int)p.bh, (int)p.rows, (int)p.n_ctx, p.causal, ctx.sm_count};
  const DeviceWorkList work = g_lists.get(
      key,
      [&] { return schedule_attn_bwd((int)p.bh, (int)p.rows, (int)p.n_ctx, p.causal != 0, !dkdv, ctx.sm_count); },
      ctx.stream, werr);
  if (!werr.empty()) return werr;
  if (dkdv) {
    auto kernel = attn_bwd_dkdv_tc_kernel<T, D, FMT>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return std::string(what) + ": " + cudaGetErrorString(e);
    kernel<<<work.ctas, NUM_THREADS, smem, ctx.stream>>>(maps[0], maps[1], maps[2], maps[3], prm, work, ctx.status);
  } else {
    auto kernel = attn_bwd_dq_tc_kernel<T, D, FMT>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return std::string(what) + ": " + cudaGetErrorString(e);
    kernel<<<work.ctas, NUM_THREADS, smem, ctx.stream>>>(maps[0], maps[1], maps[2], maps[3], prm, work, ctx.status);
  }
  ++*ctx.launches;
  e = cudaGetLastError();
  if (e != cudaSuccess) return std::string(what) + " launch failed: " + cudaGetErrorString(e);
  return std::string();
}

std::string dispatch(const AttnProblem& p, const LaunchCtx& ctx, bool dkdv) {
  if (p.elt == Elt::BF16) {
    return p.head_dim == 64
               ? launch_typed<__nv_bfloat16, 64, 1>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, dkdv)
               : launch_typed<__nv_bfloat16, 128, 1>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, dkdv);
  }
  return p.head_dim == 64 ? launch_typed<__half, 64, 0>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, dkdv)
                          : launch_typed<__half, 128, 0>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, dkdv);
}

}  // namespace

bool attn_bwd_tc_eligible(const AttnProblem& p, std::string* why) {
  auto no = [&](const char* m) {
    if (why) *why = m;
    return false;
  };
  if (p.elt == Elt::F32) return no("fp32 attention takes the generic kernel");
  if (p.head_dim != 64 && p.head_dim != 128) return no("head dimension is not 64 or 128");
  if (p.stride_seq != p.head_dim) return no("rows are not contiguous (stride_seq != head_dim)");
  if (p.stride_head % 8) return no("stride_head is not a multiple of 16 bytes");
  if (p.stride_head < p.n_ctx * p.stride_seq) return no("heads overlap");
  if (((uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.d_o | (uintptr_t)p.out0 |
       (uintptr_t)p.out1) % 16)
    return no("base pointers are not 16-byte aligned");
  if (p.n_ctx < 128) return no("sequence shorter than one 128-row tile");
  if (p.n_ctx > 0x7fffffff / 256 || p.bh > 65535 || (p.rows / 128 + 1) * p.bh > 0x7fffffff)
    return no("extent out of range");
  return true;
}

std::string launch_attn_bwd_dq_tc(const AttnProblem& p, const LaunchCtx& ctx) { return dispatch(p, ctx, false); }
std::string launch_attn_bwd_dkdv_tc(const AttnProblem& p, const LaunchCtx& ctx) { return dispatch(p, ctx, true); }

}  // namespace tmc
