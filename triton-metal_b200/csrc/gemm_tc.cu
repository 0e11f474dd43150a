// matmul_kernel on the 5th-generation tensor cores (tcgen05 + TMEM), bf16 / f16
// operands with fp32 accumulation.
//
// Semantics: Sources/TritonMetalBench/GEMMKernel.swift:28-174 - C = A @ B from a
// zero accumulator, fp32 accumulate, result rounded to the element type on store.
//
// Shape of the kernel (one CTA per SM, persistent over output tiles):
//   warp 4   TMA producer: A tile [128 x 64] (K-major) and B tile [64 x 256]
//            (row-major B is an MN-major operand) into a 4-stage shared-memory ring
//   warp 5   MMA issuer: tcgen05.mma 128x256x16 into one of two 256-column TMEM
//            accumulators; tcgen05.commit releases ring stages and publishes tiles
//   warps 0-3 epilogue: tcgen05.ld the finished accumulator (thread = row),
//            round, store; overlaps the next tile's main loop
// Tiles are walked in groups of row blocks, column by column and back, so that the CTAs
// running at the same time share B column blocks and A row blocks through L2.
//
// HBM layout: A [M,K] row-major, B [K,N] row-major, C [M,N] row-major, element
// strides multiples of 8 (16 bytes); ragged M, N, K edges are handled by TMA
// zero fill on loads and by masks on stores.
//
// Gathered form (row-sharded GEMM over several GPUs, one process per GPU): the same kernel
// with an epilogue that writes every finished tile of this rank's rows into every rank's
// copy of the whole C - its own and, through peer-mapped memory, the others' - so the exchange
// that replicates C runs tile by tile under the main loop instead of as a collective behind
// it.  Each epilogue warp stages its 32 rows of a 128-column half in shared memory, as two
// 64-column boxes in the swizzled layout of a loaded tile, and hands them to the TMA: one
// tile-mode store per box and copy of C (per-CTA stores, no multicast; edges are clipped by
// the tensor map).  A second form sends the staged rows with plain 16-byte global stores, a
// warp instruction covering two 256-byte row segments; measured on eight GPUs the TMA form is
// 3 % faster (both are bound by what the links deliver: 117 MB into every GPU per step).
// When a rank's last tile is out (bulk groups complete, system-scope fence) it raises one
// flag per peer (release, system scope); the last CTA then waits - bounded - until every
// peer's flag for this launch has arrived, so that when the kernel completes this rank's copy
// of C is whole.  No TMA load and no library call ever touches a peer's memory.

#include "sm100_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

namespace tmc {

// ---------------------------------------------------------------------------
// Tensor map helper (driver entry point resolved at run time: the library does
// not link against libcuda)
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

std::string make_tensor_map(CUtensorMap* out, CUtensorMapDataType type, int rank, const void* base,
                            const uint64_t* dims, const uint64_t* strides_bytes,
                            const uint32_t* box) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return "cuTensorMapEncodeTiled is not available from this driver";
  cuuint64_t gdim[5];
  cuuint64_t gstride[5];
  cuuint32_t bdim[5];
  cuuint32_t estride[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estride[i] = 1;
    if (i > 0) gstride[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(out, type, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, bdim, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r);
  return std::string();
}

namespace {

using namespace ptx;

constexpr int BM = 128, BN = 256, BK = 64;      // CTA tile (elements)
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;            // 16 KiB
constexpr int B_BOX_BYTES = BK * 64 * 2;        // one [64 k x 64 n] box: 8 KiB
constexpr int B_BYTES = B_BOX_BYTES * (BN / 64);
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 48 KiB
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int MAX_RANKS = 8;                    // copies of C a gathered launch can feed
constexpr int STAGING_COLS = 128;               // columns staged per pass: 256-byte row segments
constexpr int STAGING_BYTES = 4 * 32 * STAGING_COLS * 2;   // four epilogue warps x 32 rows

// What a gathered launch adds to the plain one.
struct GatherArgs {
  void* replica[MAX_RANKS];        // rank r's copy of the whole C (own memory or peer-mapped)
  uint32_t* flags[MAX_RANKS];      // rank r's flag array: word slot*MAX_RANKS + s is raised by rank s
  unsigned int* finished;          // this rank's counter of CTAs that have stored their last tile
  int world, rank, slot;
  uint32_t epoch;                  // value the flags take for this launch (grows launch by launch)
  int wait_for_peers;
  long long wait_budget;           // cycles the final wait may take
  int tma_store;                   // 1: tiles leave through TMA stores (GatherMaps), 0: through st.global
};

// One tensor map per copy of C (rows up to the end of this rank's block, 64-column x 32-row boxes
// with the 128-byte swizzle of a loaded tile), for the TMA-store form of the gathered epilogue.
struct alignas(64) GatherMaps {
  CUtensorMap replica[MAX_RANKS];
};

// site codes reported by bounded waits
enum Site : uint32_t { kProdEmpty = 1, kMmaFull = 2, kMmaAccEmpty = 3, kEpiAccFull = 4, kDrain = 5, kPeerFlag = 6 };

struct SharedStorage {
  alignas(8) uint64_t full[STAGES];
  alignas(8) uint64_t empty[STAGES];
  alignas(8) uint64_t acc_full[2];
  alignas(8) uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Tiles are walked in groups of `group_m` row blocks, column by column inside a group, so that
// the CTAs running at the same time share a few B column panels and the group's A row panels
// stay in L2 for the whole group; odd groups walk the columns backwards, so that the B panels a
// group ends on are the ones the next group starts with.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int rows = min(tiles_m - first_m, group_m);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
  if (group & 1) tn = tiles_n - 1 - tn;
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <typename T, uint32_t FMT, bool GATHER>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               T* __restrict__ C, int M, int N, int K, int64_t scm, int group_m, DeviceStatus* status,
               const __grid_constant__ GatherArgs gather, const __grid_constant__ GatherMaps gather_maps) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128-byte swizzle atoms
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  SharedStorage& ss = *reinterpret_cast<SharedStorage*>(smem + STAGES * STAGE_BYTES);
  const uint32_t smem_base = smem_u32(smem);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  WaitCtx wc{&ss.abort_flag, status};

  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ss.full[s]), 1);
      mbar_init(smem_u32(&ss.empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ss.acc_full[a]), 1);
      mbar_init(smem_u32(&ss.acc_empty[a]), 4);
    }
    ss.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&ss.tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss.tmem_base;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, group_m, tm, tn);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(smem_u32(&ss.empty[stage]), phase ^ 1, wc, kProdEmpty)) { ok = false; break; }
          const uint32_t bar = smem_u32(&ss.full[stage]);
          const uint32_t dst = smem_base + stage * STAGE_BYTES;
          mbar_expect_tx(bar, STAGE_BYTES);
          tma_load_2d(dst, &map_a, bar, kb * BK, tm * BM);
#pragma unroll
          for (int b = 0; b < BN / 64; ++b)
            tma_load_2d(dst + A_BYTES + b * B_BOX_BYTES, &map_b, bar, tn * BN + b * 64, kb * BK);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // Before leaving, every copy this thread started must have landed: wait for
      // the last `min(issued, STAGES)` stages (bounded).
      uint32_t pending = issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES;
      int s = stage;
      uint32_t ph = phase;
      for (uint32_t i = 0; i < pending; ++i) {
        if (--s < 0) { s = STAGES - 1; ph ^= 1; }
        // the stage's most recent fill completes the phase with parity `ph`
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(&ss.full[s]), ph)) {
          if (clock64() - t0 > kWaitCycles) { report_timeout(wc, kDrain, s); break; }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer
    // the whole warp runs this loop, converged; one elected lane issues (see mma_f16_ss_elect)
    {
      constexpr uint32_t idesc = make_idesc(FMT, BM, BN, 0, 1);
      const SmemDesc a_base = make_desc_sw128(smem_base, 0, 1024);
      const SmemDesc b_base = make_desc_sw128(smem_base + A_BYTES, B_BOX_BYTES, 1024);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait_warp(smem_u32(&ss.acc_empty[acc]), acc_phase ^ 1, wc, kMmaAccEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_warp(smem_u32(&ss.full[stage]), phase, wc, kMmaFull)) { ok = false; break; }
          tc_fence_after();
          const SmemDesc a_desc = a_base.advanced(stage * STAGE_BYTES);
          const SmemDesc b_desc = b_base.advanced(stage * STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // A: K-major, 16 elements = 32 bytes further along the 128-byte row.
            // B: MN-major, 16 K rows = 2048 bytes further; 64-column blocks 8 KiB apart.
            mma_f16_ss_elect(d_tmem, a_desc.at(k * 32), b_desc.at(k * 2048), idesc, (kb | k) != 0);
          }
          mma_commit_elect(smem_u32(&ss.empty[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) mma_commit_elect(smem_u32(&ss.acc_full[acc]));
      }
      // All MMAs must have retired before TMEM is released: commit to a drained
      // barrier slot and wait for it (bounded).  acc_full[0..1] may still be in use
      // by the epilogue, so a dedicated wait on the last committed stage is used:
      // the epilogue's own wait on acc_full already orders the final tile.
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 0-3)
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, group_m, tm, tn);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(smem_u32(&ss.acc_full[acc]), acc_phase, wc, kEpiAccFull)) { ok = false; break; }
      tc_fence_after();
      if constexpr (GATHER) {
        // C is this rank's first row inside a copy of the whole matrix: the same element offset
        // holds in every copy.  128 columns at a time go through this warp's staging rows
        // (16-byte chunks XORed with the row so that neither side of the exchange conflicts on
        // banks), then out to every copy, two 256-byte row segments per store instruction.
        const uint32_t stage_addr = smem_base + STAGES * STAGE_BYTES + 1024 + warp * (32 * STAGING_COLS * 2);
        const int64_t base_off = C - (T*)gather.replica[gather.rank];
        const int cols_left = N - tn * BN;
        if (gather.tma_store) {
          // Each warp stages its 32 rows of a 128-column half as two 64-column boxes in the
          // 128-byte-swizzled layout of a loaded tile and hands them to the TMA, one store per
          // box and copy of C (the TMA clips rows and columns past the edges); the boxes are
          // reused once the TMA has read them.
          const int row0 = (int)(base_off / scm) + tm * BM + warp * 32;      // row in the whole C
#pragma unroll 1
          for (int h = 0; h < BN / STAGING_COLS; ++h) {
            if (h * STAGING_COLS >= cols_left) break;
#pragma unroll 1
            for (int c4 = 0; c4 < STAGING_COLS / 32; ++c4) {
              uint32_t r[32];
              tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + acc * BN + h * STAGING_COLS + c4 * 32, r);
              tmem_ld_wait();
              const uint32_t box = stage_addr + (c4 / 2) * 4096 + lane * 128;
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                const uint32_t chunk = (uint32_t)((c4 % 2) * 4 + v) ^ (uint32_t)(lane & 7);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(box + chunk * 16),
                             "r"(pack2<T>(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]))),
                             "r"(pack2<T>(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]))),
                             "r"(pack2<T>(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]))),
                             "r"(pack2<T>(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7])))
                             : "memory");
              }
            }
            fence_proxy_async();          // the TMA reads shared memory through the async proxy
            __syncwarp();
            if (lane == 0) {
              const int col0 = tn * BN + h * STAGING_COLS;
              // peers first, each rank starting with a different one, the local copy last
              for (int p = 1; p <= gather.world; ++p) {
                int dst = gather.rank + p;
                if (dst >= gather.world) dst -= gather.world;
                tma_store_2d(&gather_maps.replica[dst], stage_addr, col0, row0);
                if (col0 + 64 < N) tma_store_2d(&gather_maps.replica[dst], stage_addr + 4096, col0 + 64, row0);
              }
              tma_store_commit();
              tma_store_wait_read();
            }
            __syncwarp();
          }
        } else
#pragma unroll 1
        for (int h = 0; h < BN / STAGING_COLS; ++h) {
#pragma unroll 1
          for (int c4 = 0; c4 < STAGING_COLS / 32; ++c4) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + acc * BN + h * STAGING_COLS + c4 * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const uint32_t chunk = (uint32_t)(c4 * 4 + v) ^ (uint32_t)(lane & 15);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_addr + lane * 256 + chunk * 16),
                           "r"(pack2<T>(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]))),
                           "r"(pack2<T>(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]))),
                           "r"(pack2<T>(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]))),
                           "r"(pack2<T>(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7])))
                           : "memory");
            }
          }
          __syncwarp();
          const int chunk = lane & 15;                         // 16-byte piece of a 256-byte segment
          const int col = h * STAGING_COLS + chunk * 8;
          const bool col_ok = col + 8 <= cols_left;
#pragma unroll 1
          for (int it = 0; it < 16; ++it) {
            const int r_in = it * 2 + (lane >> 4);
            const int row = tm * BM + warp * 32 + r_in;
            uint4 val;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                         : "r"(stage_addr + r_in * 256 + ((chunk ^ (r_in & 15)) * 16)));
            if (row < M && col_ok) {
              const int64_t off = base_off + (int64_t)row * scm + (int64_t)tn * BN + col;
              // peers first, each rank starting with a different one, the local copy last
              for (int p = 1; p <= gather.world; ++p) {
                int dst = gather.rank + p;
                if (dst >= gather.world) dst -= gather.world;
                *reinterpret_cast<uint4*>((T*)gather.replica[dst] + off) = val;
              }
            }
          }
          __syncwarp();
        }
      } else {
        const int row = tm * BM + warp * 32 + lane;
        T* crow = C + (int64_t)row * scm + (int64_t)tn * BN;
        const int cols_left = N - tn * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + acc * BN + c0, r);
          tmem_ld_wait();
          if (row < M) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = c0 + v * 8;
              if (col + 8 <= cols_left) {
                uint4 out;
                out.x = pack2<T>(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                out.y = pack2<T>(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                out.z = pack2<T>(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                out.w = pack2<T>(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                *reinterpret_cast<uint4*>(crow + col) = out;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ss.acc_empty[acc]));
    }
    if constexpr (GATHER) {
      // Every store of this CTA is out (the TMA's included, once their groups have completed).
      // Make them visible to the other GPUs, count the CTA, and let the last one of this rank
      // tell the peers - then wait for what they have to tell.
      if (gather.tma_store && lane == 0) tma_store_wait_all();
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");          // the four epilogue warps
      if (threadIdx.x == 0) {
        const unsigned int before = atomicAdd(gather.finished, 1u);
        if (before == gridDim.x - 1) {
          *gather.finished = 0;                                // ready for the next launch
          __threadfence_system();
          const int word = gather.slot * MAX_RANKS;
          for (int p = 1; p < gather.world; ++p) {
            int dst = gather.rank + p;
            if (dst >= gather.world) dst -= gather.world;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(gather.flags[dst] + word + gather.rank),
                         "r"(gather.epoch)
                         : "memory");
          }
          if (gather.wait_for_peers) {
            const long long start = clock64();
            for (int r = 0; r < gather.world; ++r) {
              if (r == gather.rank) continue;
              const uint32_t* flag = gather.flags[gather.rank] + word + r;
              for (;;) {
                uint32_t seen;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
                if ((int32_t)(seen - gather.epoch) >= 0) break;      // this launch's flag, or a later one
                if (clock64() - start > gather.wait_budget) {
                  report_timeout(wc, kPeerFlag, (uint32_t)r);
                  r = gather.world;                                  // give up on the others as well
                  break;
                }
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <typename T, uint32_t FMT>
std::string launch_typed(const GemmProblem& p, const LaunchCtx& ctx, CUtensorMapDataType type,
                         const GatherArgs* gather, int64_t row0 = 0) {
  CUtensorMap map_a, map_b;
  {
    uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.M};
    uint64_t strides[1] = {(uint64_t)p.sam * 2};
    uint32_t box[2] = {(uint32_t)BK, (uint32_t)BM};
    std::string e = make_tensor_map(&map_a, type, 2, p.a, dims, strides, box);
    if (!e.empty()) return e;
  }
  {
    uint64_t dims[2] = {(uint64_t)p.N, (uint64_t)p.K};
    uint64_t strides[1] = {(uint64_t)p.sbk * 2};
    uint32_t box[2] = {64u, (uint32_t)BK};
    std::string e = make_tensor_map(&map_b, type, 2, p.b, dims, strides, box);
    if (!e.empty()) return e;
  }
  const size_t smem = STAGES * STAGE_BYTES + 1024 + 1024 + (gather ? STAGING_BYTES : 0);
  auto kernel = gather ? gemm_tc_kernel<T, FMT, true> : gemm_tc_kernel<T, FMT, false>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return std::string("matmul_kernel: ") + cudaGetErrorString(e);
  const int tiles = (int)(((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN));
  const int grid = tiles < ctx.sm_count ? tiles : ctx.sm_count;
  GatherArgs none{};
  static const GatherMaps no_maps{};
  GatherMaps maps{};
  if (gather && gather->tma_store) {
    for (int r = 0; r < gather->world; ++r) {
      uint64_t dims[2] = {(uint64_t)p.N, (uint64_t)(row0 + p.M)};
      uint64_t strides[1] = {(uint64_t)p.scm * 2};
      uint32_t box[2] = {64u, 32u};
      std::string e2 = make_tensor_map(&maps.replica[r], type, 2, gather->replica[r], dims, strides, box);
      if (!e2.empty()) return e2;
    }
  }
  // Measured on 8192^3 (B200): groups of 16 row blocks beat 4, 8, 12, 24, 32 and 64 in time,
  // sustained throughput and clock under the power cap alike; a wave of 148 tiles then spans
  // about 16 x 9 tiles, close to the squarest footprint (least A + B bytes) a wave can have.
  constexpr int group_m = 16;
  kernel<<<grid, NUM_THREADS, smem, ctx.stream>>>(map_a, map_b, (T*)p.c, (int)p.M, (int)p.N, (int)p.K,
                                                 p.scm, group_m, ctx.status, gather ? *gather : none,
                                                 gather && gather->tma_store ? maps : no_maps);
  ++*ctx.launches;
  e = cudaGetLastError();
  if (e != cudaSuccess) return std::string("matmul_kernel launch failed: ") + cudaGetErrorString(e);
  return std::string();
}

}  // namespace

bool gemm_tc_eligible(const GemmProblem& p, std::string* why) {
  auto no = [&](const char* m) {
    if (why) *why = m;
    return false;
  };
  if (p.elt == Elt::F32) return no("fp32 operands take the 3xTF32 kernel");
  if (p.sak != 1 || p.sbn != 1 || p.scn != 1) return no("operands are not row-major with unit inner stride");
  if (p.sam % 8 || p.sbk % 8 || p.scm % 8) return no("row strides are not multiples of 16 bytes");
  if (((uintptr_t)p.a | (uintptr_t)p.b | (uintptr_t)p.c) % 16) return no("base pointers are not 16-byte aligned");
  if (p.M < BM || p.N < 64 || p.K < BK) return no("problem smaller than one tile");
  if (p.N % 8) return no("N is not a multiple of 8");
  if (p.M > 0x7fffffff || p.N > 0x7fffffff || p.K > 0x7fffffff) return no("extent above 2^31");
  if (p.sam < p.K || p.sbk < p.N || p.scm < p.N) return no("rows overlap");
  return true;
}

std::string launch_gemm_tc(const GemmProblem& p, const LaunchCtx& ctx) {
  if (p.elt == Elt::BF16)
    return launch_typed<__nv_bfloat16, 1>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, nullptr);
  return launch_typed<__half, 0>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, nullptr);
}

// The gathered form: p.c points at this rank's first row inside its own copy of the whole C
// (g.replica[g.rank] + row0 * stride_cm); every finished tile also goes to the same place in
// the other copies.
std::string launch_gemm_tc_gathered(const GemmProblem& p, const GemmGather& g, const LaunchCtx& ctx) {
  if (g.world < 1 || g.world > MAX_RANKS || g.rank < 0 || g.rank >= g.world) return "rank / world out of range";
  GatherArgs a{};
  for (int r = 0; r < g.world; ++r) {
    a.replica[r] = g.replica[r];
    a.flags[r] = g.flags[r];
  }
  a.finished = g.finished;
  a.world = g.world;
  a.rank = g.rank;
  a.slot = g.slot;
  a.epoch = g.epoch;
  a.wait_for_peers = g.wait_for_peers;
  a.wait_budget = g.wait_budget_cycles > 0 ? g.wait_budget_cycles : ptx::kWaitCycles;
  a.tma_store = g.tma_store;
  // first row of this rank's block inside a copy of C
  const int64_t row0 = ((const char*)p.c - (const char*)g.replica[g.rank]) / (p.scm * 2);
  if (p.elt == Elt::BF16)
    return launch_typed<__nv_bfloat16, 1>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, &a, row0);
  return launch_typed<__half, 0>(p, ctx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, &a, row0);
}

}  // namespace tmc
