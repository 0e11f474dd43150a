// attn_fwd on tcgen05 / TMEM: FlashAttention-2 forward for 16-bit elements,
// head dimension 64 or 128, optional causal mask.
//
// Semantics: Sources/TritonMetalBench/AttentionKernel.swift:40-250 - per query
// block, walk the key blocks with an online softmax in base 2
// (qk_scale = sm_scale*log2 e), P rounded to the element type before P.V,
// O = acc / l, and the row statistic L = m + log2(l) in log2 units.
//
// One CTA owns 128 query rows of one (batch, head):
//   warp 4    TMA: Q once, then K and V blocks of 128 keys into 2-stage rings
//   warp 5    MMA issuer: S = Q K^T (128x128xD) into one of two TMEM score
//             buffers, O += P V (128xDx128) into the TMEM output accumulator
//   warps 0-3 softmax, one thread per query row (the row lives in that thread's
//             TMEM lane, so row max / row sum need no cross-thread traffic):
//             tcgen05.ld S, mask, running max, exp2, round P into a swizzled
//             shared-memory tile that the P.V MMA reads, rescale O in TMEM when
//             the running max moved by more than 2^8, final O/l and L store.
// The running max used for the exponentials is only advanced when it grew by
// more than 8 (in log2 units), which keeps P <= 256 and makes most iterations
// skip the O rescale; O/l at the end is exact either way.
//
// HBM layout: Q, K, V, O [BH, S, D] with D contiguous (stride_seq == D),
// L [BH, S] fp32.

#include "sm100_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

namespace tmc {
namespace {

using namespace ptx;

constexpr int BLOCK_M = 128, BLOCK_N = 128;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int S_COL0 = 0, S_COL1 = 128, O_COL = 256;
constexpr float kLog2e = 1.44269504088896340736f;
constexpr float kRescaleThreshold = 8.0f;

enum Site : uint32_t {
  kLoadKEmpty = 11, kLoadVEmpty = 12, kMmaQ = 13, kMmaK = 14, kMmaV = 15, kMmaP = 16,
  kSoftS = 17, kSoftPv = 18, kSoftFinal = 19, kDrainLoad = 20
};

struct Shared {
  alignas(8) uint64_t q_full;
  alignas(8) uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  alignas(8) uint64_t s_full[2];
  alignas(8) uint64_t p_full;
  alignas(8) uint64_t pv_done;
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

template <typename T, int D, uint32_t FMT, bool P_TMEM>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, Params prm, DeviceStatus* status) {
  constexpr int HALVES = D / 64;                        // 64-column swizzle atoms per row
  constexpr int TILE_BYTES = BLOCK_M * D * 2;           // Q, K, V tiles: 128 rows x D
  constexpr int HALF_BYTES = BLOCK_M * 128;             // one [128 x 64] swizzled box
  constexpr int P_BYTES = BLOCK_M * BLOCK_N * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // layout: Q | K0 K1 | V0 V1 | P | barriers
  const uint32_t q_addr = smem_u32(smem);
  const uint32_t k_addr = q_addr + TILE_BYTES;
  const uint32_t v_addr = k_addr + 2 * TILE_BYTES;
  const uint32_t p_addr = v_addr + 2 * TILE_BYTES;
  uint8_t* p_ptr = smem + 5 * TILE_BYTES;
  Shared& ss = *reinterpret_cast<Shared*>(smem + 5 * TILE_BYTES + P_BYTES);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  WaitCtx wc{&ss.abort_flag, status};

  // heavy (late) query tiles first under a causal mask
  const int m_tile = prm.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int bh = blockIdx.y;
  const int m0 = m_tile * BLOCK_M;
  int key_end = prm.n_ctx;
  if (prm.causal) key_end = min(prm.n_ctx, m0 + BLOCK_M);
  const int n_blocks = (key_end + BLOCK_N - 1) / BLOCK_N;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ss.q_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&ss.k_full[s]), 1);
      mbar_init(smem_u32(&ss.k_empty[s]), 1);
      mbar_init(smem_u32(&ss.v_full[s]), 1);
      mbar_init(smem_u32(&ss.v_empty[s]), 1);
      mbar_init(smem_u32(&ss.s_full[s]), 1);
    }
    mbar_init(smem_u32(&ss.p_full), 128);
    mbar_init(smem_u32(&ss.pv_done), 1);
    ss.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&ss.tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ss.tmem_base;

  if (warp == 4) {
    // ---------------------------------------------------------------- loads
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      mbar_expect_tx(smem_u32(&ss.q_full), TILE_BYTES);
#pragma unroll
      for (int h = 0; h < HALVES; ++h)
        tma_load_3d(q_addr + h * HALF_BYTES, &map_q, smem_u32(&ss.q_full), h * 64, m0, bh);
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&ss.k_empty[s]), ph ^ 1, wc, kLoadKEmpty)) { ok = false; break; }
        mbar_expect_tx(smem_u32(&ss.k_full[s]), TILE_BYTES);
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          tma_load_3d(k_addr + s * TILE_BYTES + h * HALF_BYTES, &map_k, smem_u32(&ss.k_full[s]), h * 64,
                      j * BLOCK_N, bh);
        if (!mbar_wait(smem_u32(&ss.v_empty[s]), ph ^ 1, wc, kLoadVEmpty)) { ok = false; ++issued; break; }
        mbar_expect_tx(smem_u32(&ss.v_full[s]), TILE_BYTES);
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          tma_load_3d(v_addr + s * TILE_BYTES + h * HALF_BYTES, &map_v, smem_u32(&ss.v_full[s]), h * 64,
                      j * BLOCK_N, bh);
        ++issued;
      }
      // every copy started here must have landed before the CTA exits
      {
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(&ss.q_full), 0)) {
          if (clock64() - t0 > kWaitCycles) { report_timeout(wc, kDrainLoad, 0); break; }
        }
        for (int j = max(0, issued - 2); j < issued; ++j) {
          const int s = j & 1;
          const uint32_t ph = (j >> 1) & 1;
          const long long t1 = clock64();
          while (!(mbar_try_wait(smem_u32(&ss.k_full[s]), ph) && mbar_try_wait(smem_u32(&ss.v_full[s]), ph))) {
            if (clock64() - t1 > kWaitCycles) { report_timeout(wc, kDrainLoad, j + 1); break; }
          }
        }
      }
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(FMT, BLOCK_M, BLOCK_N, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(FMT, BLOCK_M, D, 0, 1);
      bool ok = mbar_wait(smem_u32(&ss.q_full), 0, wc, kMmaQ);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(smem_u32(&ss.k_full[s]), (j >> 1) & 1, wc, kMmaK)) return false;
        tc_fence_after();
        const uint32_t kb = k_addr + s * TILE_BYTES;
        const uint32_t d_tmem = tmem + (s ? S_COL1 : S_COL0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * HALF_BYTES + (kk % 4) * 32;
          mma_f16_ss(d_tmem, smem_desc_sw128(q_addr + off, 0, 1024), smem_desc_sw128(kb + off, 0, 1024),
                     idesc_qk, kk != 0);
        }
        mma_commit(smem_u32(&ss.k_empty[s]));
        mma_commit(smem_u32(&ss.s_full[s]));
        return true;
      };
      if (ok && n_blocks > 0) ok = issue_qk(0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks && !issue_qk(j + 1)) { ok = false; break; }
        const int s = j & 1;
        if (!mbar_wait(smem_u32(&ss.v_full[s]), (j >> 1) & 1, wc, kMmaV)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&ss.p_full), j & 1, wc, kMmaP)) { ok = false; break; }
        tc_fence_after();
        const uint32_t vb = v_addr + s * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
          // P: K-major, 64-key halves 16 KiB apart.  V: MN-major, 16 keys = 2048 bytes
          // further, 64-column halves HALF_BYTES apart.
          if constexpr (P_TMEM) {
            // P as a TMEM operand: 16 keys = 8 packed 32-bit columns of the score buffer
            mma_f16_ts(tmem + O_COL, tmem + (s ? S_COL1 : S_COL0) + kk * 8,
                       smem_desc_sw128(vb + kk * 2048, HALF_BYTES, 1024), idesc_pv, (j | kk) != 0);
          } else {
            const uint32_t p_off = (kk / 4) * (BLOCK_M * 128) + (kk % 4) * 32;
            mma_f16_ss(tmem + O_COL, smem_desc_sw128(p_addr + p_off, 0, 1024),
                       smem_desc_sw128(vb + kk * 2048, HALF_BYTES, 1024), idesc_pv, (j | kk) != 0);
          }
        }
        mma_commit(smem_u32(&ss.v_empty[s]));
        mma_commit(smem_u32(&ss.pv_done));
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax
    const int row_in_tile = warp * 32 + lane;
    const int q_row = m0 + row_in_tile;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    const float qk_scale = prm.sm_scale * kLog2e;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int s = j & 1;
      if (!mbar_wait(smem_u32(&ss.s_full[s]), (j >> 1) & 1, wc, kSoftS)) { ok = false; break; }
      tc_fence_after();
      float x[BLOCK_N];
      {
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld_32x32(tmem + lane_addr + (s ? S_COL1 : S_COL0) + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) x[c * 32 + i] = __uint_as_float(r[i]) * qk_scale;
        }
      }
      const int n0 = j * BLOCK_N;
      const bool boundary = (n0 + BLOCK_N > prm.n_ctx) || (prm.causal && n0 + BLOCK_N > m0);
      if (boundary) {
#pragma unroll
        for (int i = 0; i < BLOCK_N; ++i) {
          const int key = n0 + i;
          if (key >= prm.n_ctx || (prm.causal && key > q_row)) x[i] = -INFINITY;
        }
      }
      float mx = x[0];
#pragma unroll
      for (int i = 1; i < BLOCK_N; ++i) mx = fmaxf(mx, x[i]);
      // advance the working max only when it moved far (or on the first block)
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_used + kRescaleThreshold) {
        alpha = fast_exp2(m_used - mx);      // 0 on the first block (m_used = -inf)
        m_used = mx;
        rescale = j > 0;
      }
      const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
      float sum = 0.f;
      uint32_t packed[BLOCK_N / 2];
#pragma unroll
      for (int i = 0; i < BLOCK_N; i += 2) {
        const float p0 = fast_exp2(x[i] + neg_m);
        const float p1 = fast_exp2(x[i + 1] + neg_m);
        sum += p0 + p1;
        packed[i / 2] = pack2<T>(p0, p1);
      }
      l = l * alpha + sum;
      // P(j) may only replace P(j-1) once the P.V MMA of block j-1 has finished; the
      // same event makes O safe to rescale.
      const bool any_rescale = __any_sync(0xffffffffu, rescale);
      if (j > 0 && (!P_TMEM || any_rescale) &&
          !mbar_wait(smem_u32(&ss.pv_done), (j - 1) & 1, wc, kSoftPv)) { ok = false; break; }
      tc_fence_after();
      if (any_rescale) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem + lane_addr + O_COL + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32(tmem + lane_addr + O_COL + c * 32, r);
        }
        tmem_st_wait();
      }
      if constexpr (P_TMEM) {
        // P replaces the first 64 columns of the score buffer it was computed from
        // (two 16-bit values per 32-bit column, even key in the low half).
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = packed[c * 32 + i];
          tmem_st_32x32(tmem + lane_addr + (s ? S_COL1 : S_COL0) + c * 32, r);
        }
        tmem_st_wait();
      } else {
      // P tile: K-major, 128-byte swizzle; row r, 16-byte chunk c at (c ^ (r & 7)).
        uint8_t* prow = p_ptr + row_in_tile * 128;
        const int sw = row_in_tile & 7;
#pragma unroll
        for (int c = 0; c < BLOCK_N / 8; ++c) {
          uint4 v = make_uint4(packed[c * 4 + 0], packed[c * 4 + 1], packed[c * 4 + 2], packed[c * 4 + 3]);
          *reinterpret_cast<uint4*>(prow + (c / 8) * (BLOCK_M * 128) + (((c % 8) ^ sw) * 16)) = v;
        }
      fence_proxy_async();
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&ss.p_full));
    }
    // ---- epilogue: O / l and the row statistic
    if (ok && n_blocks > 0) ok = mbar_wait(smem_u32(&ss.pv_done), (n_blocks - 1) & 1, wc, kSoftFinal);
    tc_fence_after();
    if (ok && n_blocks > 0) {
      const float inv_l = 1.f / l;
      const bool live = q_row < prm.rows;
      T* orow = (T*)prm.o + (int64_t)bh * prm.stride_head + (int64_t)q_row * prm.stride_seq;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem + lane_addr + O_COL + c * 32, r);
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 out;
            out.x = pack2<T>(__uint_as_float(r[v * 8 + 0]) * inv_l, __uint_as_float(r[v * 8 + 1]) * inv_l);
            out.y = pack2<T>(__uint_as_float(r[v * 8 + 2]) * inv_l, __uint_as_float(r[v * 8 + 3]) * inv_l);
            out.z = pack2<T>(__uint_as_float(r[v * 8 + 4]) * inv_l, __uint_as_float(r[v * 8 + 5]) * inv_l);
            out.w = pack2<T>(__uint_as_float(r[v * 8 + 6]) * inv_l, __uint_as_float(r[v * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = out;
          }
        }
      }
      if (live && prm.lse) prm.lse[(int64_t)bh * prm.stride_lse + q_row] = m_used + log2f(l);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <typename T, int D, uint32_t FMT, bool P_TMEM>
std::string launch_typed_p(const AttnProblem& p, const LaunchCtx& ctx, CUtensorMapDataType type) {
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
  size_t smem = 5 * (BLOCK_M * D * 2) + BLOCK_M * BLOCK_N * 2 + sizeof(Shared) + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;
  auto kernel = attn_fwd_tc_kernel<T, D, FMT, P_TMEM>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return std::string("attn_fwd: ") + cudaGetErrorString(e);
  dim3 grid((unsigned)((p.rows + BLOCK_M - 1) / BLOCK_M), (unsigned)p.bh, 1);
  kernel<<<grid, NUM_THREADS, smem, ctx.stream>>>(maps[0], maps[1], maps[2], prm, ctx.status);
  ++*ctx.launches;
  e = cudaGetLastError();
  if (e != cudaSuccess) return std::string("attn_fwd launch failed: ") + cudaGetErrorString(e);
  return std::string();
}

template <typename T, int D, uint32_t FMT>
std::string launch_typed(const AttnProblem& p, const LaunchCtx& ctx, CUtensorMapDataType type) {
  // $TMCUDA_ATTN_P=smem keeps P in shared memory (the first, conservative form).
  static const bool p_smem = [] {
    const char* e = std::getenv("TMCUDA_ATTN_P");
    return e && std::string(e) == "smem";
  }();
  return p_smem ? launch_typed_p<T, D, FMT, false>(p, ctx, type)
                : launch_typed_p<T, D, FMT, true>(p, ctx, type);
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
  if (p.n_ctx > 0x7fffffff / 256 || p.bh > 65535) return no("extent out of range");
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
