// Generic SIMT kernels: every dtype, every stride, ragged edges, any head
// dimension up to 256.  They are the correctness floor of the library - the
// shapes the tcgen05 kernels do not take (non-contiguous operands, ragged or
// tiny problems, head dimensions other than 64/128) run here - and they follow
// the reference kernels' arithmetic step by step:
//
//   matmul_kernel        Sources/TritonMetalBench/GEMMKernel.swift:28-174
//   attn_fwd             Sources/TritonMetalBench/AttentionKernel.swift:40-250
//   attn_bwd_preprocess  Sources/TritonMetalBench/AttentionBackwardKernel.swift:53-136
//   attn_bwd_dq          Sources/TritonMetalBench/AttentionBackwardKernel.swift:151-344
//   attn_bwd_dkdv        Sources/TritonMetalBench/AttentionBackwardKernel.swift:354-575
//
// All products accumulate in fp32; 16-bit kernels round P / dS to the element
// type before the second contraction and round the result on store, as the
// reference's f16 forms do with arith.truncf.

#include "tm_core.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tmc {

namespace {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
// Round through the element type (identity for fp32).
template <typename T> __device__ __forceinline__ float round_to(float v) {
  return to_f32(from_f32<T>(v));
}

constexpr float kLog2e = 1.44269504088896340736f;

// ---------------------------------------------------------------------------
// Probe
// ---------------------------------------------------------------------------
__global__ void probe_kernel(int* out) {
  if (threadIdx.x == 0) *out = 0x7a11;
}

// ---------------------------------------------------------------------------
// GEMM: 64x64 output tile per CTA, 16-deep K steps, 4x4 outputs per thread.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, int64_t M,
                 int64_t N, int64_t K, int64_t sam, int64_t sak, int64_t sbk, int64_t sbn,
                 int64_t scm, int64_t scn, const float* __restrict__ bias, int relu) {
  __shared__ float As[16][64 + 4];
  __shared__ float Bs[16][64 + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int64_t m0 = (int64_t)blockIdx.x * 64, n0 = (int64_t)blockIdx.y * 64;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int64_t k0 = 0; k0 < K; k0 += 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int idx = tid + i * 256;
      int m = idx / 16, k = idx % 16;
      float v = 0.f;
      if (m0 + m < M && k0 + k < K) v = to_f32(A[(m0 + m) * sam + (k0 + k) * sak]);
      As[k][m] = v;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int idx = tid + i * 256;
      int k = idx / 64, n = idx % 64;
      float v = 0.f;
      if (n0 + n < N && k0 + k < K) v = to_f32(B[(k0 + k) * sbk + (n0 + n) * sbn]);
      Bs[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t n = n0 + tx * 4 + j;
      if (n < N) {
        // optional fused epilogue: + bias[n], then max(., 0), on the accumulator
        float v = acc[i][j];
        if (bias) v += bias[n];
        if (relu) v = fmaxf(v, 0.f);
        C[m * scm + n * scn] = from_f32<T>(v);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Attention tiles.  One CTA owns 32 "resident" rows (queries for fwd/dq, keys
// for dkdv) and streams 32-row tiles of the other side through shared memory.
// Four threads (a quad) share one resident row: each computes 8 of the 32
// scores of a tile, row statistics are combined with warp shuffles inside the
// quad, and each thread accumulates every fourth output column.
// ---------------------------------------------------------------------------
constexpr int kRows = 32;     // resident rows per CTA
constexpr int kTile = 32;     // streamed rows per step
constexpr int kThreads = 128;

struct AttnArgs {
  const void *q, *k, *v, *d_o;
  void *out0, *out1;
  float* lse_out;
  const float *lse, *delta;
  float sm_scale;
  int64_t stride_head, stride_seq, stride_lse, n_ctx, rows;
  int D, causal;
};

// Load `kTile` rows x D of a [*, D]-contiguous tensor starting at row0 into
// shared memory as fp32 (row stride D+1), zero beyond `limit`.
template <typename T>
__device__ __forceinline__ void load_rows(float* dst, const T* base, int64_t stride_seq,
                                          int64_t row0, int64_t limit, int D) {
  const int ld = D + 1;
  for (int idx = threadIdx.x; idx < kTile * D; idx += kThreads) {
    int r = idx / D, d = idx - r * D;
    float v = 0.f;
    if (row0 + r < limit) v = to_f32(base[(row0 + r) * stride_seq + d]);
    dst[r * ld + d] = v;
  }
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  return v;
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(kThreads) attn_fwd_simt_kernel(AttnArgs a) {
  extern __shared__ float smem[];
  const int D = a.D, ld = D + 1;
  float* Qs = smem;
  float* Ks = Qs + kRows * ld;
  float* Vs = Ks + kTile * ld;
  float* Ps = Vs + kTile * ld;   // [kRows][kTile+1]
  const int r = threadIdx.x / 4, c = threadIdx.x % 4;
  const int64_t bh = blockIdx.y;
  const int64_t m0 = (int64_t)blockIdx.x * kRows;
  const T* Q = (const T*)a.q + bh * a.stride_head;
  const T* Kp = (const T*)a.k + bh * a.stride_head;
  const T* Vp = (const T*)a.v + bh * a.stride_head;
  T* O = (T*)a.out0 + bh * a.stride_head;
  const float qk_scale = a.sm_scale * kLog2e;

  load_rows<T>(Qs, Q, a.stride_seq, m0, a.n_ctx, D);
  float m_i = -INFINITY, l_i = 0.f;
  float acc[DMAX / 4];
#pragma unroll
  for (int i = 0; i < DMAX / 4; ++i) acc[i] = 0.f;

  int64_t key_end = a.n_ctx;
  if (a.causal) key_end = min(a.n_ctx, m0 + kRows);
  const int64_t q_row = m0 + r;
  for (int64_t n0 = 0; n0 < key_end; n0 += kTile) {
    __syncthreads();
    load_rows<T>(Ks, Kp, a.stride_seq, n0, a.n_ctx, D);
    load_rows<T>(Vs, Vp, a.stride_seq, n0, a.n_ctx, D);
    __syncthreads();
    float s[kTile / 4];
    float row_max = -INFINITY;
#pragma unroll
    for (int t = 0; t < kTile / 4; ++t) {
      const int j = c + 4 * t;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(Qs[r * ld + d], Ks[j * ld + d], dot);
      float v = dot * qk_scale;
      const int64_t key = n0 + j;
      if (key >= a.n_ctx || (a.causal && key > q_row)) v = -INFINITY;
      s[t] = v;
      row_max = fmaxf(row_max, v);
    }
    row_max = quad_max(row_max);
    const float m_new = fmaxf(m_i, row_max);
    float sum = 0.f;
#pragma unroll
    for (int t = 0; t < kTile / 4; ++t) {
      float p = m_new == -INFINITY ? 0.f : exp2f(s[t] - m_new);
      sum += p;
      Ps[r * (kTile + 1) + c + 4 * t] = round_to<T>(p);
    }
    sum = quad_sum(sum);
    const float alpha = m_new == -INFINITY ? 1.f : exp2f(m_i - m_new);
    l_i = l_i * alpha + sum;
    m_i = m_new;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < DMAX / 4; ++i) {
      const int d = c + 4 * i;
      if (d < D) {
        float o = acc[i] * alpha;
        for (int j = 0; j < kTile; ++j) o = fmaf(Ps[r * (kTile + 1) + j], Vs[j * ld + d], o);
        acc[i] = o;
      }
    }
  }
  if (q_row < a.rows) {
#pragma unroll
    for (int i = 0; i < DMAX / 4; ++i) {
      const int d = c + 4 * i;
      if (d < D) O[q_row * a.stride_seq + d] = from_f32<T>(acc[i] / l_i);
    }
    if (a.lse_out && c == 0) a.lse_out[bh * a.stride_lse + q_row] = m_i + log2f(l_i);
  }
}

// Delta_i = sum_d O[i,d] * dO[i,d]; one warp per row.
template <typename T>
__global__ void __launch_bounds__(256) attn_bwd_preprocess_kernel(AttnArgs a) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  const int64_t bh = blockIdx.y;
  if (row >= a.rows) return;
  const T* O = (const T*)a.q + bh * a.stride_head + row * a.stride_seq;     // q slot carries O
  const T* dO = (const T*)a.d_o + bh * a.stride_head + row * a.stride_seq;
  float sum = 0.f;
  for (int d = lane; d < a.D; d += 32) sum = fmaf(to_f32(O[d]), to_f32(dO[d]), sum);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) ((float*)a.out0)[bh * a.stride_lse + row] = sum;
}

// 16-bit, 16-byte aligned rows: LPR lanes of a warp share one row, each loading
// 16-byte chunks - the HBM-bound form used by the benchmark shapes.
template <typename T, int LPR>
__global__ void __launch_bounds__(256) attn_bwd_preprocess_vec_kernel(AttnArgs a) {
  constexpr int kRowsPerWarp = 32 / LPR;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int sub = lane / LPR, l = lane % LPR;
  const int64_t row = ((int64_t)blockIdx.x * 8 + warp) * kRowsPerWarp + sub;
  const int64_t bh = blockIdx.y;
  float sum = 0.f;
  if (row < a.rows) {
    const uint4* O = (const uint4*)((const T*)a.q + bh * a.stride_head + row * a.stride_seq);
    const uint4* dO = (const uint4*)((const T*)a.d_o + bh * a.stride_head + row * a.stride_seq);
    const int chunks = a.D / 8;
    for (int ch = l; ch < chunks; ch += LPR) {
      uint4 x = __ldg(O + ch), y = __ldg(dO + ch);
      const T* xs = (const T*)&x;
      const T* ys = (const T*)&y;
#pragma unroll
      for (int i = 0; i < 8; ++i) sum = fmaf(to_f32(xs[i]), to_f32(ys[i]), sum);
    }
  }
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (row < a.rows && l == 0) ((float*)a.out0)[bh * a.stride_lse + row] = sum;
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(kThreads) attn_bwd_dq_simt_kernel(AttnArgs a) {
  extern __shared__ float smem[];
  const int D = a.D, ld = D + 1;
  float* Qs = smem;
  float* dOs = Qs + kRows * ld;
  float* Ks = dOs + kRows * ld;
  float* Vs = Ks + kTile * ld;
  float* dSs = Vs + kTile * ld;   // [kRows][kTile+1]
  const int r = threadIdx.x / 4, c = threadIdx.x % 4;
  const int64_t bh = blockIdx.y;
  const int64_t m0 = (int64_t)blockIdx.x * kRows;
  const int64_t head = bh * a.stride_head;
  const float qk_scale = a.sm_scale * kLog2e;
  load_rows<T>(Qs, (const T*)a.q + head, a.stride_seq, m0, a.n_ctx, D);
  load_rows<T>(dOs, (const T*)a.d_o + head, a.stride_seq, m0, a.n_ctx, D);
  const int64_t q_row = m0 + r;
  float lse = 0.f, delta = 0.f;
  if (q_row < a.n_ctx) {
    lse = a.lse[bh * a.stride_lse + q_row];
    delta = a.delta[bh * a.stride_lse + q_row];
  }
  float acc[DMAX / 4];
#pragma unroll
  for (int i = 0; i < DMAX / 4; ++i) acc[i] = 0.f;
  int64_t key_end = a.n_ctx;
  if (a.causal) key_end = min(a.n_ctx, m0 + kRows);
  for (int64_t n0 = 0; n0 < key_end; n0 += kTile) {
    __syncthreads();
    load_rows<T>(Ks, (const T*)a.k + head, a.stride_seq, n0, a.n_ctx, D);
    load_rows<T>(Vs, (const T*)a.v + head, a.stride_seq, n0, a.n_ctx, D);
    __syncthreads();
#pragma unroll
    for (int t = 0; t < kTile / 4; ++t) {
      const int j = c + 4 * t;
      float qk = 0.f, dp = 0.f;
      for (int d = 0; d < D; ++d) {
        qk = fmaf(Qs[r * ld + d], Ks[j * ld + d], qk);
        dp = fmaf(dOs[r * ld + d], Vs[j * ld + d], dp);
      }
      const int64_t key = n0 + j;
      float p = 0.f;
      if (key < a.n_ctx && !(a.causal && key > q_row)) p = exp2f(qk * qk_scale - lse);
      dSs[r * (kTile + 1) + j] = round_to<T>(p * (dp - delta));
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < DMAX / 4; ++i) {
      const int d = c + 4 * i;
      if (d < D) {
        float o = acc[i];
        for (int j = 0; j < kTile; ++j) o = fmaf(dSs[r * (kTile + 1) + j], Ks[j * ld + d], o);
        acc[i] = o;
      }
    }
  }
  if (q_row < a.rows) {
    T* dQ = (T*)a.out0 + head;
#pragma unroll
    for (int i = 0; i < DMAX / 4; ++i) {
      const int d = c + 4 * i;
      if (d < D) dQ[q_row * a.stride_seq + d] = from_f32<T>(acc[i] * a.sm_scale);
    }
  }
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(kThreads) attn_bwd_dkdv_simt_kernel(AttnArgs a) {
  extern __shared__ float smem[];
  const int D = a.D, ld = D + 1;
  float* Ks = smem;
  float* Vs = Ks + kRows * ld;
  float* Qs = Vs + kRows * ld;
  float* dOs = Qs + kTile * ld;
  float* Ps = dOs + kTile * ld;            // [kRows][kTile+1]  P^T
  float* dSs = Ps + kRows * (kTile + 1);   // [kRows][kTile+1]  dS^T
  float* stats = dSs + kRows * (kTile + 1);  // lse[kTile], delta[kTile]
  const int r = threadIdx.x / 4, c = threadIdx.x % 4;
  const int64_t bh = blockIdx.y;
  const int64_t n0 = (int64_t)blockIdx.x * kRows;
  const int64_t head = bh * a.stride_head;
  const float qk_scale = a.sm_scale * kLog2e;
  load_rows<T>(Ks, (const T*)a.k + head, a.stride_seq, n0, a.n_ctx, D);
  load_rows<T>(Vs, (const T*)a.v + head, a.stride_seq, n0, a.n_ctx, D);
  const int64_t k_row = n0 + r;
  float dk[DMAX / 4], dv[DMAX / 4];
#pragma unroll
  for (int i = 0; i < DMAX / 4; ++i) { dk[i] = 0.f; dv[i] = 0.f; }
  // Under a causal mask, queries before this key block never attend to it.
  int64_t q_begin = a.causal ? (n0 / kTile) * kTile : 0;
  for (int64_t m0 = q_begin; m0 < a.n_ctx; m0 += kTile) {
    __syncthreads();
    load_rows<T>(Qs, (const T*)a.q + head, a.stride_seq, m0, a.n_ctx, D);
    load_rows<T>(dOs, (const T*)a.d_o + head, a.stride_seq, m0, a.n_ctx, D);
    if (threadIdx.x < kTile) {
      int64_t q = m0 + threadIdx.x;
      stats[threadIdx.x] = q < a.n_ctx ? a.lse[bh * a.stride_lse + q] : 0.f;
      stats[kTile + threadIdx.x] = q < a.n_ctx ? a.delta[bh * a.stride_lse + q] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < kTile / 4; ++t) {
      const int i = c + 4 * t;
      float qk = 0.f, dp = 0.f;
      for (int d = 0; d < D; ++d) {
        qk = fmaf(Ks[r * ld + d], Qs[i * ld + d], qk);
        dp = fmaf(Vs[r * ld + d], dOs[i * ld + d], dp);
      }
      const int64_t q = m0 + i;
      float p = 0.f;
      if (q < a.n_ctx && !(a.causal && k_row > q)) p = exp2f(qk * qk_scale - stats[i]);
      Ps[r * (kTile + 1) + i] = round_to<T>(p);
      dSs[r * (kTile + 1) + i] = round_to<T>(p * (dp - stats[kTile + i]));
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < DMAX / 4; ++i) {
      const int d = c + 4 * i;
      if (d < D) {
        float x = dv[i], y = dk[i];
        for (int j = 0; j < kTile; ++j) {
          x = fmaf(Ps[r * (kTile + 1) + j], dOs[j * ld + d], x);
          y = fmaf(dSs[r * (kTile + 1) + j], Qs[j * ld + d], y);
        }
        dv[i] = x;
        dk[i] = y;
      }
    }
  }
  if (k_row < a.rows) {
    T* dK = (T*)a.out0 + head;
    T* dV = (T*)a.out1 + head;
#pragma unroll
    for (int i = 0; i < DMAX / 4; ++i) {
      const int d = c + 4 * i;
      if (d < D) {
        dK[k_row * a.stride_seq + d] = from_f32<T>(dk[i] * a.sm_scale);
        dV[k_row * a.stride_seq + d] = from_f32<T>(dv[i]);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Host-side launch helpers
// ---------------------------------------------------------------------------
std::string check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return std::string(what) + " launch failed: " + cudaGetErrorString(e);
  return std::string();
}

AttnArgs make_args(const AttnProblem& p) {
  AttnArgs a{};
  a.q = p.q; a.k = p.k; a.v = p.v; a.d_o = p.d_o;
  a.out0 = p.out0; a.out1 = p.out1;
  a.lse_out = p.lse; a.lse = p.lse; a.delta = p.delta;
  a.sm_scale = p.sm_scale;
  a.stride_head = p.stride_head; a.stride_seq = p.stride_seq; a.stride_lse = p.stride_lse;
  a.n_ctx = p.n_ctx; a.rows = p.rows; a.D = p.head_dim; a.causal = p.causal;
  return a;
}

template <typename K>
std::string launch_tiles(K kernel, const AttnProblem& p, const LaunchCtx& ctx, size_t smem_floats,
                         const char* what) {
  if (p.bh > 65535) return std::string(what) + ": batch*heads above 65535 is not supported";
  size_t bytes = smem_floats * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return std::string(what) + ": " + cudaGetErrorString(e);
  dim3 grid((unsigned)((p.rows + kRows - 1) / kRows), (unsigned)p.bh, 1);
  kernel<<<grid, kThreads, bytes, ctx.stream>>>(make_args(p));
  ++*ctx.launches;
  return check_launch(what);
}

#define TM_DISPATCH_ELT(ELT, CALL)                                 \
  switch (ELT) {                                                   \
    case Elt::F32: { using T = float; CALL; } break;               \
    case Elt::F16: { using T = __half; CALL; } break;              \
    default: { using T = __nv_bfloat16; CALL; } break;             \
  }

#define TM_DISPATCH_D(D, CALL)                                     \
  if ((D) <= 64) { constexpr int DMAX = 64; CALL; }                \
  else if ((D) <= 128) { constexpr int DMAX = 128; CALL; }         \
  else { constexpr int DMAX = 256; CALL; }

}  // namespace

std::string launch_probe(const LaunchCtx& ctx, int* out_host) {
  int* dev = nullptr;
  cudaError_t e = cudaMalloc(&dev, sizeof(int));
  if (e != cudaSuccess) return cudaGetErrorString(e);
  cudaMemsetAsync(dev, 0, sizeof(int), ctx.stream);
  probe_kernel<<<1, 32, 0, ctx.stream>>>(dev);
  e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpyAsync(out_host, dev, sizeof(int), cudaMemcpyDeviceToHost, ctx.stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx.stream);
  cudaFree(dev);
  if (e != cudaSuccess) return cudaGetErrorString(e);
  return std::string();
}

std::string launch_gemm_simt(const GemmProblem& p, const LaunchCtx& ctx) {
  int64_t gm = (p.M + 63) / 64, gn = (p.N + 63) / 64;
  if (gn > 65535) return "matmul_kernel: N above 4194240 is not supported by the generic kernel";
  dim3 grid((unsigned)gm, (unsigned)gn, 1);
  TM_DISPATCH_ELT(p.elt, (gemm_simt_kernel<T><<<grid, 256, 0, ctx.stream>>>(
                             (const T*)p.a, (const T*)p.b, (T*)p.c, p.M, p.N, p.K, p.sam, p.sak,
                             p.sbk, p.sbn, p.scm, p.scn, p.bias, p.relu)));
  ++*ctx.launches;
  return check_launch("matmul_kernel");
}

std::string launch_attn_fwd_simt(const AttnProblem& p, const LaunchCtx& ctx) {
  const int ld = p.head_dim + 1;
  size_t floats = (size_t)(kRows + 2 * kTile) * ld + kRows * (kTile + 1);
  std::string e;
  TM_DISPATCH_ELT(p.elt, TM_DISPATCH_D(p.head_dim, (e = launch_tiles(attn_fwd_simt_kernel<T, DMAX>, p,
                                                                     ctx, floats, "attn_fwd"))));
  return e;
}

std::string launch_attn_bwd_preprocess(const AttnProblem& p, const LaunchCtx& ctx) {
  if (p.bh > 65535) return "attn_bwd_preprocess: batch*heads above 65535 is not supported";
  AttnArgs a = make_args(p);
  a.q = p.o;   // the kernel reads O through the q slot
  const int eb = elt_size(p.elt);
  const bool vec = eb == 2 && (p.head_dim == 64 || p.head_dim == 128) && p.stride_seq % 8 == 0 &&
                   p.stride_head % 8 == 0 && ((uintptr_t)p.o % 16 == 0) && ((uintptr_t)p.d_o % 16 == 0);
  if (vec) {
    if (p.head_dim == 64) {
      dim3 grid((unsigned)((p.rows + 31) / 32), (unsigned)p.bh, 1);
      if (p.elt == Elt::F16) attn_bwd_preprocess_vec_kernel<__half, 8><<<grid, 256, 0, ctx.stream>>>(a);
      else attn_bwd_preprocess_vec_kernel<__nv_bfloat16, 8><<<grid, 256, 0, ctx.stream>>>(a);
    } else {
      dim3 grid((unsigned)((p.rows + 15) / 16), (unsigned)p.bh, 1);
      if (p.elt == Elt::F16) attn_bwd_preprocess_vec_kernel<__half, 16><<<grid, 256, 0, ctx.stream>>>(a);
      else attn_bwd_preprocess_vec_kernel<__nv_bfloat16, 16><<<grid, 256, 0, ctx.stream>>>(a);
    }
  } else {
    dim3 grid((unsigned)((p.rows + 7) / 8), (unsigned)p.bh, 1);
    TM_DISPATCH_ELT(p.elt, (attn_bwd_preprocess_kernel<T><<<grid, 256, 0, ctx.stream>>>(a)));
  }
  ++*ctx.launches;
  return check_launch("attn_bwd_preprocess");
}

std::string launch_attn_bwd_dq_simt(const AttnProblem& p, const LaunchCtx& ctx) {
  const int ld = p.head_dim + 1;
  size_t floats = (size_t)(2 * kRows + 2 * kTile) * ld + kRows * (kTile + 1);
  std::string e;
  TM_DISPATCH_ELT(p.elt, TM_DISPATCH_D(p.head_dim, (e = launch_tiles(attn_bwd_dq_simt_kernel<T, DMAX>,
                                                                     p, ctx, floats, "attn_bwd_dq"))));
  return e;
}

std::string launch_attn_bwd_dkdv_simt(const AttnProblem& p, const LaunchCtx& ctx) {
  const int ld = p.head_dim + 1;
  size_t floats = (size_t)(2 * kRows + 2 * kTile) * ld + 2 * kRows * (kTile + 1) + 2 * kTile;
  std::string e;
  TM_DISPATCH_ELT(p.elt, TM_DISPATCH_D(p.head_dim, (e = launch_tiles(attn_bwd_dkdv_simt_kernel<T, DMAX>,
                                                                     p, ctx, floats, "attn_bwd_dkdv"))));
  return e;
}

}  // namespace tmc
