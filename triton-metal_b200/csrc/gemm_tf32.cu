// matmul_kernel for fp32 operands on the tensor cores: 3xTF32.
//
// Semantics: Sources/TritonMetalBench/GEMMKernel.swift:28-174 with element f32 - the
// reference computes true fp32 products (Metal has one precision).  A TF32 MMA keeps
// 10 mantissa bits of each operand, so every operand is split once into
//     hi = tf32(x),  lo = tf32(x - hi)            (x = hi + lo up to 2^-22 |x|)
// and each K step issues three kind::tf32 MMAs into the same fp32 TMEM accumulator:
//     C += A_lo*B_hi + A_hi*B_lo + A_hi*B_hi       (the lo*lo term, ~2^-22, is dropped)
//
// Two kernels:
//   split_tf32_kernel   reads A[M,K] and B[K,N] with their own strides and writes
//                       A_hi, A_lo as [M, Kp] and B_hi, B_lo TRANSPOSED as [N, Kp]
//                       (Kp = K rounded up to 4, zero padded) into scratch memory, so
//                       both MMA operands are K-major and any input stride is accepted;
//   gemm_tf32_kernel    the same persistent, warp-specialised pipeline as the 16-bit
//                       kernel (gemm_tc.cu): tile 128x256x32, 2 stages of
//                       {A_hi, A_lo, B_hi, B_lo} = 96 KiB each, two 256-column TMEM
//                       accumulators, fp32 epilogue.
// The tensor core's fp32 accumulator does not round to nearest: the error of one long
// accumulation grows linearly with K (6e-5 relative at K = 8192, measured).  The K loop
// is therefore cut into chunks of 256: each chunk accumulates in TMEM from zero, and the
// epilogue warps add the finished chunks in registers with ordinary round-to-nearest
// fp32 adds while the next chunk runs in the other TMEM accumulator.  The error then
// stays at the level of one chunk (about 2e-6) for every K.
//
// The scratch is global memory beyond the caller's inputs and outputs:
// 8 * (M + N) * Kp bytes.  tm_launch takes it from a workspace the library grows on
// demand (cudaMalloc); tmx_matmul_f32_static uses a fixed device array instead.

#include "sm100_ptx.cuh"

#include <mutex>

namespace tmc {
namespace {

using namespace ptx;

constexpr int BM = 128, BN = 256, BK = 32;       // CTA tile (fp32 elements)
constexpr int STAGES = 2;
constexpr int A_BYTES = BM * BK * 4;             // 16 KiB
constexpr int B_BYTES = BN * BK * 4;             // 32 KiB
constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;   // 96 KiB
constexpr int GROUP_M = 16;
constexpr int NUM_THREADS = 320;         // warps 0-3, 6-9 epilogue; 4 TMA; 5 MMA
constexpr int CHUNK_KB = 8;              // K blocks (of 32) accumulated in TMEM before a read-out
constexpr int TMEM_COLS = 512;

struct SharedStorage {
  alignas(8) uint64_t full[STAGES];
  alignas(8) uint64_t empty[STAGES];
  alignas(8) uint64_t acc_full[2];
  alignas(8) uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// One 32x32 tile per CTA iteration; `transpose` writes out[c, r] instead of out[r, c].
// src is [rows, cols] with element strides (sr, sc); outputs are dense with leading
// dimension `ld` (zero padded up to `ld` along the inner axis).
__global__ void __launch_bounds__(256)
split_tf32_kernel(const float* __restrict__ src, int64_t rows, int64_t cols, int64_t sr, int64_t sc,
                  float* __restrict__ hi, float* __restrict__ lo, int64_t ld, int transpose) {
  __shared__ float th[32][33], tl[32][33];
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;   // 32 x 8
  const int64_t r0 = (int64_t)blockIdx.y * 32, c0 = (int64_t)blockIdx.x * 32;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = r0 + ty + i * 8, c = c0 + tx;
    float x = 0.f;
    if (r < rows && c < cols) x = src[r * sr + c * sc];
    const float h = to_tf32(x);
    const float l = to_tf32(x - h);
    if (transpose) {
      th[ty + i * 8][tx] = h;
      tl[ty + i * 8][tx] = l;
    } else if (r < rows && c < ld) {
      hi[r * ld + c] = h;
      lo[r * ld + c] = l;
    }
  }
  if (transpose) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // output row = source column, output column = source row
      const int64_t orow = c0 + ty + i * 8, ocol = r0 + tx;
      if (orow < cols && ocol < ld) {
        hi[orow * ld + ocol] = th[tx][ty + i * 8];
        lo[orow * ld + ocol] = tl[tx][ty + i * 8];
      }
    }
  }
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = GROUP_M * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(tiles_m - first_m, GROUP_M);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
                 const __grid_constant__ CUtensorMap map_bhi, const __grid_constant__ CUtensorMap map_blo,
                 float* __restrict__ C, int M, int N, int K, int64_t scm, int64_t scn, int vec_store,
                 const float* __restrict__ bias, int relu, DeviceStatus* status) {
  extern __shared__ uint8_t smem_raw[];
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
      mbar_init(smem_u32(&ss.acc_empty[a]), 8);
    }
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
  const uint32_t tmem_base = ss.tmem_base;

  if (warp == 4) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(smem_u32(&ss.empty[stage]), phase ^ 1, wc, 71)) { ok = false; break; }
          const uint32_t bar = smem_u32(&ss.full[stage]);
          const uint32_t dst = smem_base + stage * STAGE_BYTES;
          mbar_expect_tx(bar, STAGE_BYTES);
          tma_load_2d(dst, &map_ahi, bar, kb * BK, tm * BM);
          tma_load_2d(dst + A_BYTES, &map_alo, bar, kb * BK, tm * BM);
          tma_load_2d(dst + 2 * A_BYTES, &map_bhi, bar, kb * BK, tn * BN);
          tma_load_2d(dst + 2 * A_BYTES + B_BYTES, &map_blo, bar, kb * BK, tn * BN);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      uint32_t pending = issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES;
      int s = stage;
      uint32_t ph = phase;
      for (uint32_t i = 0; i < pending; ++i) {
        if (--s < 0) { s = STAGES - 1; ph ^= 1; }
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(&ss.full[s]), ph)) {
          if (clock64() - t0 > kWaitCycles) { report_timeout(wc, 75, s); break; }
        }
      }
    }
  } else if (warp == 5) {
    // the whole warp runs this loop, converged; one elected lane issues (see mma_f16_ss_elect)
    {
      constexpr uint32_t idesc = make_idesc(2, BM, BN, 0, 0);     // tf32, both operands K-major
      int stage = 0;
      uint32_t phase = 0;
      const SmemDesc stage_base = make_desc_sw128(smem_base, 0, 1024);
      int local = 0;                       // chunks issued so far (selects the accumulator)
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb0 = 0; kb0 < k_blocks && ok; kb0 += CHUNK_KB, ++local) {
          const int acc = local & 1;
          const uint32_t acc_phase = (local >> 1) & 1;
          if (!mbar_wait_warp(smem_u32(&ss.acc_empty[acc]), acc_phase ^ 1, wc, 73)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          const int kb_end = min(k_blocks, kb0 + CHUNK_KB);
          for (int kb = kb0; kb < kb_end; ++kb) {
            if (!mbar_wait_warp(smem_u32(&ss.full[stage]), phase, wc, 72)) { ok = false; break; }
            tc_fence_after();
            // operands of a stage: A hi | A lo | B hi | B lo
            const SmemDesc ahi = stage_base.advanced(stage * STAGE_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 8; ++k) {
              // 8 fp32 = 32 bytes further along the 128-byte row, for every operand
              const uint64_t d_ahi = ahi.at(k * 32);
              const uint64_t d_alo = ahi.at(A_BYTES + k * 32);
              const uint64_t d_bhi = ahi.at(2 * A_BYTES + k * 32);
              const uint64_t d_blo = ahi.at(2 * A_BYTES + B_BYTES + k * 32);
              mma_tf32_ss_elect(d_tmem, d_alo, d_bhi, idesc, (kb != kb0) || k != 0);
              mma_tf32_ss_elect(d_tmem, d_ahi, d_blo, idesc, 1);
              mma_tf32_ss_elect(d_tmem, d_ahi, d_bhi, idesc, 1);
            }
            mma_commit_elect(smem_u32(&ss.empty[stage]));
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (ok) mma_commit_elect(smem_u32(&ss.acc_full[acc]));
        }
      }
    }
  } else {
    // Epilogue: warps 0-3 own columns [0,128) of the tile, warps 6-9 columns [128,256);
    // (warp % 4) selects the 32 TMEM lanes (rows) a warp may read.
    const int half = warp >= 6 ? 1 : 0;
    const int quarter = warp % 4;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      float sums[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) sums[i] = 0.f;
      for (int kb0 = 0; kb0 < k_blocks && ok; kb0 += CHUNK_KB, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(smem_u32(&ss.acc_full[acc]), acc_phase, wc, 74)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + half * 128 + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) sums[c * 32 + i] += __uint_as_float(r[i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ss.acc_empty[acc]));
      }
      if (!ok) break;
      const int row = tm * BM + quarter * 32 + lane;
      const int col_base = tn * BN + half * 128;
      float* crow = C + (int64_t)row * scm + (int64_t)col_base * scn;
      const int cols_left = N - col_base;
      if (bias || relu) {
        // fused epilogue on the summed accumulator: + bias[column], then max(., 0)
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          float v = sums[i];
          if (bias && i < cols_left) v += __ldg(bias + col_base + i);
          sums[i] = relu ? fmaxf(v, 0.f) : v;
        }
      }
      if (row < M) {
        if (vec_store) {
#pragma unroll
          for (int v = 0; v < 32; ++v) {
            const int col = v * 4;
            if (col + 4 <= cols_left) {
              *reinterpret_cast<float4*>(crow + col) =
                  make_float4(sums[col], sums[col + 1], sums[col + 2], sums[col + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                if (col + i < cols_left) crow[col + i] = sums[col + i];
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i < cols_left) crow[(int64_t)i * scn] = sums[i];
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

// Fixed scratch for tmx_matmul_f32_static: lives in the library image, so every GPU that
// loads the library holds these 8 MiB until the process exits.  In host code the name
// `g_static_scratch` is only a stand-in for the symbol; the device address is obtained
// with cudaGetSymbolAddress below and that address is what the kernels receive.
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;

// Workspace the library owns for tm_launch (grown on demand, never shrunk).
struct Workspace {
  std::mutex lock;
  void* ptr = nullptr;
  size_t bytes = 0;
};
Workspace g_workspace;

}  // namespace

size_t gemm_tf32_scratch_bytes(int64_t M, int64_t N, int64_t K) {
  // in 128 bits: absurd extents must read as "too large", not wrap to something small
  const __int128 kp = ((__int128)K + 3) / 4 * 4;
  const __int128 need = 8 * ((__int128)M + (__int128)N) * kp;
  if (M < 0 || N < 0 || K < 0 || need > (__int128)(SIZE_MAX / 2)) return SIZE_MAX / 2;
  return (size_t)need;
}

// Runs split + GEMM with `scratch` (device pointer, at least gemm_tf32_scratch_bytes).
std::string run_gemm_tf32(const GemmProblem& p, const LaunchCtx& ctx, void* scratch) {
  const int64_t M = p.M, N = p.N, K = p.K;
  const int64_t kp = (K + 3) / 4 * 4;
  float* a_hi = (float*)scratch;
  float* a_lo = a_hi + M * kp;
  float* b_hi = a_lo + M * kp;
  float* b_lo = b_hi + N * kp;
  {
    dim3 grid((unsigned)((kp + 31) / 32), (unsigned)((M + 31) / 32), 1);
    split_tf32_kernel<<<grid, 256, 0, ctx.stream>>>((const float*)p.a, M, K, p.sam, p.sak, a_hi, a_lo, kp, 0);
    ++*ctx.launches;
  }
  {
    // B[K,N] -> transposed [N, Kp]
    dim3 grid((unsigned)((N + 31) / 32), (unsigned)((kp + 31) / 32), 1);
    split_tf32_kernel<<<grid, 256, 0, ctx.stream>>>((const float*)p.b, K, N, p.sbk, p.sbn, b_hi, b_lo, kp, 1);
    ++*ctx.launches;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return std::string("matmul_kernel (split) launch failed: ") + cudaGetErrorString(e);
  CUtensorMap maps[4];
  const float* bases[4] = {a_hi, a_lo, b_hi, b_lo};
  for (int i = 0; i < 4; ++i) {
    const bool is_a = i < 2;
    uint64_t dims[2] = {(uint64_t)kp, (uint64_t)(is_a ? M : N)};
    uint64_t strides[1] = {(uint64_t)kp * 4};
    uint32_t box[2] = {(uint32_t)BK, (uint32_t)(is_a ? BM : BN)};
    std::string err = make_tensor_map(&maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, bases[i], dims, strides, box);
    if (!err.empty()) return err;
  }
  const size_t smem = STAGES * STAGE_BYTES + sizeof(SharedStorage) + 1024;
  e = cudaFuncSetAttribute(gemm_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return std::string("matmul_kernel: ") + cudaGetErrorString(e);
  const int tiles = (int)(((M + BM - 1) / BM) * ((N + BN - 1) / BN));
  const int grid = tiles < ctx.sm_count ? tiles : ctx.sm_count;
  const int vec = p.scn == 1 && p.scm % 4 == 0 && ((uintptr_t)p.c % 16 == 0);
  gemm_tf32_kernel<<<grid, NUM_THREADS, smem, ctx.stream>>>(maps[0], maps[1], maps[2], maps[3], (float*)p.c,
                                                           (int)M, (int)N, (int)kp, p.scm, p.scn, vec,
                                                           p.bias, p.relu, ctx.status);
  ++*ctx.launches;
  e = cudaGetLastError();
  if (e != cudaSuccess) return std::string("matmul_kernel launch failed: ") + cudaGetErrorString(e);
  return std::string();
}

bool gemm_tf32_eligible(const GemmProblem& p, std::string* why) {
  auto no = [&](const char* m) {
    if (why) *why = m;
    return false;
  };
  if (p.elt != Elt::F32) return no("not fp32");
  if (p.M < 128 || p.N < 64 || p.K < 32) return no("problem smaller than one tile");
  if ((double)p.M * (double)p.N * (double)p.K < 4194304.0) return no("problem too small to amortise the operand split");
  if (p.M > 0x7fffffff || p.N > 0x7fffffff || p.K > 0x7ffffff0) return no("extent above 2^31");
  return true;
}

std::string launch_gemm_tf32(const GemmProblem& p, const LaunchCtx& ctx) {
  const size_t need = gemm_tf32_scratch_bytes(p.M, p.N, p.K);
  std::lock_guard<std::mutex> guard(g_workspace.lock);
  if (g_workspace.bytes < need) {
    // the stream may still be using the old workspace
    cudaStreamSynchronize(ctx.stream);
    if (g_workspace.ptr) cudaFree(g_workspace.ptr);
    g_workspace.ptr = nullptr;
    g_workspace.bytes = 0;
    cudaError_t e = cudaMalloc(&g_workspace.ptr, need);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return "could not allocate " + std::to_string(need) + " bytes of scratch for the 3xTF32 operand split: " +
             cudaGetErrorString(e);
    }
    g_workspace.bytes = need;
  }
  return run_gemm_tf32(p, ctx, g_workspace.ptr);
}

}  // namespace tmc

namespace tmc {

size_t gemm_tf32_static_capacity() { return kStaticScratchBytes; }

// The 3xTF32 GEMM with its operand split in the fixed device array instead of an allocated
// workspace.  The first call on a device resolves the array's device address (with that
// device current); nothing here allocates or frees device memory.  Every call uses the same
// array: the split kernels rewrite every word the GEMM will read (including the zero padding
// of K up to a multiple of 4), so nothing left by an earlier call is ever consumed.
// Device address of the fixed array on `device` (which must be current): looked up once per
// device with cudaGetSymbolAddress and cached.  With CUDA's lazy module loading this lookup is
// also what loads this translation unit's module, i.e. the moment the driver reserves the
// array's 8 MiB and the kernel images on that GPU.
static std::string static_scratch_address(int device, void** out) {
  static std::mutex lock;
  static void* address[kMaxDevices] = {};
  if (device < 0 || device >= kMaxDevices) return "device ordinal outside 0..63";
  std::lock_guard<std::mutex> guard(lock);
  if (!address[device]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr) {
      cudaGetLastError();
      return std::string("could not resolve the fixed scratch array on this device: ") + cudaGetErrorString(e);
    }
    address[device] = ptr;
  }
  *out = address[device];
  return std::string();
}

std::string prepare_gemm_tf32_static(int device) {
  void* scratch = nullptr;
  return static_scratch_address(device, &scratch);
}

std::string run_gemm_tf32_static(const GemmProblem& p, const LaunchCtx& ctx, int device) {
  const size_t need = gemm_tf32_scratch_bytes(p.M, p.N, p.K);
  if (need > kStaticScratchBytes) {
    return "the operand split needs " + std::to_string(need) + " bytes of scratch (8*(M+N)*roundup(K,4)), more than the " +
           std::to_string(kStaticScratchBytes) + "-byte fixed array; use tm_launch for this size";
  }
  void* scratch = nullptr;
  std::string e = static_scratch_address(device, &scratch);
  if (!e.empty()) return e;
  return run_gemm_tf32(p, ctx, scratch);
}

}  // namespace tmc
