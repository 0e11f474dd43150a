// fp32 attention for long sequences on the tensor cores: every contraction of attn_fwd,
// attn_bwd_dq and attn_bwd_dkdv runs as a 3xTF32 GEMM (gemm_tf32.cu), the softmax and the
// dS = P (dP - Delta) products in between run as row-wise fp32 kernels over a materialised
// score matrix.
//
// Semantics: Sources/TritonMetalBench/AttentionKernel.swift:40-250 (forward, f32 path) and
// Sources/TritonMetalBench/AttentionBackwardKernel.swift:151-575 (dq, dkdv): scores scaled by
// sm_scale * log2 e, the row statistic L = m + log2 l in log2 units, P rebuilt from L in the
// backward, dQ and dK scaled by sm_scale.  fp32 accuracy (1e-5 with the reference's
// relative_error) is what the split buys: a single tf32 product would give 1e-3.
//
// This is the unfused form - one (batch, head) slice at a time, S [rows x n_ctx] written to a
// workspace between the GEMMs - which is what fp32 allows without a second family of fused
// kernels: an fp32 score tile with its hi / lo halves takes the TMEM the fused 16-bit kernels
// use for two tiles.  It is chosen for sequences of 1024 rows and more, where the exact-FMA
// SIMT kernels (which stay for short sequences such as the h2 s96 d64 training configuration,
// launch-latency bound) fall an order of magnitude behind; `path = 2` asks for it from 256.
//
// HBM layout: Q, K, V, O, dO, dQ, dK, dV [BH, S, D] fp32 with any row stride; L, Delta [BH, S].

#include "tm_core.h"

#include <cuda_runtime.h>

#include <mutex>

namespace tmc {
namespace {

constexpr float kLog2e = 1.44269504088896340736f;

// One block per score row: P = softmax over the row's keys (scores scaled by qk_scale, base 2),
// written over the scores; L = m + log2 l.  Keys past n_ctx never exist in the row; under a
// causal mask key > row gives P = 0.
__global__ void __launch_bounds__(256) softmax_scores_kernel(float* s, float* lse, int64_t ld, int n_ctx,
                                                             float qk_scale, int causal) {
  __shared__ float red[8];
  const int row = blockIdx.x;
  float* srow = s + (int64_t)row * ld;
  const int keys = causal ? min(n_ctx, row + 1) : n_ctx;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float m = -INFINITY;
  for (int j = threadIdx.x; j < keys; j += 256) m = fmaxf(m, srow[j]);
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = red[0];
  for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
  __syncthreads();
  const float m2 = m * qk_scale;
  float sum = 0.f;
  for (int j = threadIdx.x; j < keys; j += 256) {
    const float p = exp2f(fmaf(srow[j], qk_scale, -m2));
    srow[j] = p;
    sum += p;
  }
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = 0.f;
  for (int w = 0; w < 8; ++w) sum += red[w];
  const float inv = 1.f / sum;
  for (int j = threadIdx.x; j < n_ctx; j += 256) srow[j] = j < keys ? srow[j] * inv : 0.f;
  if (threadIdx.x == 0 && lse) lse[row] = m2 + log2f(sum);
}

// Backward, one block per query row: P = exp2(S * qk_scale - L[row]) over the scores (masked
// keys give 0) and dS = sm_scale * P * (dP - Delta[row]) over dP, both in place.
__global__ void __launch_bounds__(256) p_and_ds_kernel(float* s, float* dp, const float* lse, const float* delta,
                                                       int64_t ld, int n_ctx, float qk_scale, float sm_scale,
                                                       int causal) {
  const int row = blockIdx.x;
  float* srow = s + (int64_t)row * ld;
  float* drow = dp + (int64_t)row * ld;
  const float l = lse[row], dl = delta[row];
  const int keys = causal ? min(n_ctx, row + 1) : n_ctx;
  for (int j = threadIdx.x; j < n_ctx; j += 256) {
    const float p = j < keys ? exp2f(fmaf(srow[j], qk_scale, -l)) : 0.f;
    srow[j] = p;
    drow[j] = sm_scale * p * (drow[j] - dl);
  }
}

// Workspace for the score matrices (grown on demand, never shrunk).
struct Workspace {
  std::mutex lock;
  float* ptr = nullptr;
  size_t bytes = 0;
};
Workspace g_scores;

std::string reserve(size_t bytes, cudaStream_t stream, float** out) {
  std::lock_guard<std::mutex> guard(g_scores.lock);
  if (g_scores.bytes < bytes) {
    cudaStreamSynchronize(stream);        // the stream may still be using the old one
    if (g_scores.ptr) cudaFree(g_scores.ptr);
    g_scores.ptr = nullptr;
    g_scores.bytes = 0;
    cudaError_t e = cudaMalloc((void**)&g_scores.ptr, bytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return "could not allocate " + std::to_string(bytes) + " bytes for the fp32 score matrices: " +
             cudaGetErrorString(e);
    }
    g_scores.bytes = bytes;
  }
  *out = g_scores.ptr;
  return std::string();
}

// C[M,N] = A[M,K] @ B[K,N] in fp32 as 3xTF32, any strides.
std::string gemm(const LaunchCtx& ctx, const float* a, const float* b, float* c, int64_t M, int64_t N, int64_t K,
                 int64_t sam, int64_t sak, int64_t sbk, int64_t sbn, int64_t scm) {
  GemmProblem g{};
  g.elt = Elt::F32;
  g.a = a; g.b = b; g.c = c;
  g.M = M; g.N = N; g.K = K;
  g.sam = sam; g.sak = sak; g.sbk = sbk; g.sbn = sbn; g.scm = scm; g.scn = 1;
  return launch_gemm_tf32(g, ctx);
}

std::string check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return std::string(what) + " launch failed: " + cudaGetErrorString(e);
  return std::string();
}

}  // namespace

bool attn_f32_tc_eligible(const AttnProblem& p, bool forced, std::string* why) {
  auto no = [&](const char* m) {
    if (why) *why = m;
    return false;
  };
  if (p.elt != Elt::F32) return no("not fp32");
  if (p.head_dim < 64 || p.head_dim > 256) return no("head dimension outside 64...256");
  if (p.n_ctx < 256 || p.rows < 128) return no("sequence shorter than 256 rows");
  if (!forced && p.n_ctx < 1024) return no("below 1024 rows the exact-FMA kernels are at least as fast");
  if (p.n_ctx > 65536) return no("sequence above 65536 rows");
  if (!(p.sm_scale > 0.f)) return no("softmax scale is not positive");
  return true;
}

std::string launch_attn_fwd_f32_tc(const AttnProblem& p, const LaunchCtx& ctx) {
  const int64_t S = p.n_ctx, R = p.rows, D = p.head_dim, ld = (S + 3) / 4 * 4;
  float* scores = nullptr;
  std::string e = reserve((size_t)R * ld * sizeof(float), ctx.stream, &scores);
  if (!e.empty()) return e;
  const float qk_scale = p.sm_scale * kLog2e;
  for (int64_t h = 0; h < p.bh; ++h) {
    const float* q = (const float*)p.q + h * p.stride_head;
    const float* k = (const float*)p.k + h * p.stride_head;
    const float* v = (const float*)p.v + h * p.stride_head;
    float* o = (float*)p.out0 + h * p.stride_head;
    // S = Q K^T: B[d, key] = K[key, d]
    e = gemm(ctx, q, k, scores, R, S, D, p.stride_seq, 1, 1, p.stride_seq, ld);
    if (!e.empty()) return e;
    softmax_scores_kernel<<<(unsigned)R, 256, 0, ctx.stream>>>(scores, p.lse ? p.lse + h * p.stride_lse : nullptr, ld,
                                                               (int)S, qk_scale, p.causal);
    ++*ctx.launches;
    e = check_launch("attn_fwd (softmax)");
    if (!e.empty()) return e;
    // O = P V
    e = gemm(ctx, scores, v, o, R, D, S, ld, 1, p.stride_seq, 1, p.stride_seq);
    if (!e.empty()) return e;
  }
  return std::string();
}

// P (over S) and sm_scale * dS (over dP) of one head, all n_ctx query rows, in the workspace.
static std::string p_and_ds(const AttnProblem& p, const LaunchCtx& ctx, int64_t h, int64_t q_rows, float* scores,
                            float* dscores, int64_t ld) {
  const int64_t S = p.n_ctx, D = p.head_dim;
  const float* q = (const float*)p.q + h * p.stride_head;
  const float* k = (const float*)p.k + h * p.stride_head;
  const float* v = (const float*)p.v + h * p.stride_head;
  const float* d_o = (const float*)p.d_o + h * p.stride_head;
  std::string e = gemm(ctx, q, k, scores, q_rows, S, D, p.stride_seq, 1, 1, p.stride_seq, ld);       // S = Q K^T
  if (!e.empty()) return e;
  e = gemm(ctx, d_o, v, dscores, q_rows, S, D, p.stride_seq, 1, 1, p.stride_seq, ld);               // dP = dO V^T
  if (!e.empty()) return e;
  p_and_ds_kernel<<<(unsigned)q_rows, 256, 0, ctx.stream>>>(scores, dscores, p.lse + h * p.stride_lse,
                                                            p.delta + h * p.stride_lse, ld, (int)S,
                                                            p.sm_scale * kLog2e, p.sm_scale, p.causal);
  ++*ctx.launches;
  return check_launch("attn_bwd (dS)");
}

std::string launch_attn_bwd_dq_f32_tc(const AttnProblem& p, const LaunchCtx& ctx) {
  const int64_t S = p.n_ctx, R = p.rows, D = p.head_dim, ld = (S + 3) / 4 * 4;
  float* ws = nullptr;
  std::string e = reserve((size_t)2 * R * ld * sizeof(float), ctx.stream, &ws);
  if (!e.empty()) return e;
  float *scores = ws, *dscores = ws + R * ld;
  for (int64_t h = 0; h < p.bh; ++h) {
    e = p_and_ds(p, ctx, h, R, scores, dscores, ld);
    if (!e.empty()) return e;
    // dQ = (sm_scale dS) K
    e = gemm(ctx, dscores, (const float*)p.k + h * p.stride_head, (float*)p.out0 + h * p.stride_head, R, D, S, ld, 1,
             p.stride_seq, 1, p.stride_seq);
    if (!e.empty()) return e;
  }
  return std::string();
}

std::string launch_attn_bwd_dkdv_f32_tc(const AttnProblem& p, const LaunchCtx& ctx) {
  // p.rows bounds the key rows that are written; every query row contributes to them
  const int64_t S = p.n_ctx, R = p.rows, D = p.head_dim, ld = (S + 3) / 4 * 4;
  float* ws = nullptr;
  std::string e = reserve((size_t)2 * S * ld * sizeof(float), ctx.stream, &ws);
  if (!e.empty()) return e;
  float *scores = ws, *dscores = ws + S * ld;
  for (int64_t h = 0; h < p.bh; ++h) {
    e = p_and_ds(p, ctx, h, S, scores, dscores, ld);
    if (!e.empty()) return e;
    // dV = P^T dO and dK = (sm_scale dS)^T Q: A[key, query] = X[query, key]
    e = gemm(ctx, scores, (const float*)p.d_o + h * p.stride_head, (float*)p.out1 + h * p.stride_head, R, D, S, 1, ld,
             p.stride_seq, 1, p.stride_seq);
    if (!e.empty()) return e;
    e = gemm(ctx, dscores, (const float*)p.q + h * p.stride_head, (float*)p.out0 + h * p.stride_head, R, D, S, 1, ld,
             p.stride_seq, 1, p.stride_seq);
    if (!e.empty()) return e;
  }
  return std::string();
}

}  // namespace tmc
