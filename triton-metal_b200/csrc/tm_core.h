// Internal declarations shared by the translation units of libtmcuda.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>
#include <string>
#include <vector>

namespace tmc {

// ---------------------------------------------------------------------------
// Element types and kernel identities
// ---------------------------------------------------------------------------

enum class Elt : int { F32 = 0, F16 = 1, BF16 = 2 };

inline int elt_size(Elt e) { return e == Elt::F32 ? 4 : 2; }
inline const char* elt_name(Elt e) {
  return e == Elt::F32 ? "f32" : (e == Elt::F16 ? "f16" : "bf16");
}

enum class KernelId : int {
  Matmul = 0,
  AttnFwd = 1,
  AttnBwdPreprocess = 2,
  AttnBwdDq = 3,
  AttnBwdDkdv = 4,
  // The one-dimensional kernels the reference's own ABI tests launch
  // (Tests/TritonMetalCoreTests/Fixtures.swift, python/tests/test_plugin_shape.py).
  VecCopy = 5,       // copy_kernel(in, out, n)
  VecAdd = 6,        // add_kernel(a, b, out, n)
  VecMul = 7,        // mul_kernel(a, b, out, n)
  ScaleBias = 8,     // scale_bias_kernel(in, out, scale, bias, n)
  Softmax = 9,       // softmax_kernel(in, out, in_row_stride, out_row_stride, n_cols)
  // The fused sparse-autoencoder encoder, out = relu(x @ w + bias), fp32, row-major
  // (Sources/TritonMetalMLX/SAEEncoder.swift:40-200): the matmul with an epilogue.
  SaeEncode = 10,    // sae_encode_kernel(x, w, bias, out, M, D, F)
  Count = 11
};
inline bool is_rowwise(KernelId id) {
  return (int)id >= (int)KernelId::VecCopy && (int)id <= (int)KernelId::Softmax;
}

const char* kernel_entry_name(KernelId id);

// The role of one tt.func argument, resolved from its name or position.
enum class Role : int {
  Unknown = 0,
  // matmul_kernel
  A, B, C, M, N, K, StrideAm, StrideAk, StrideBk, StrideBn, StrideCm, StrideCn,
  // attention kernels
  Q, Kt, V, O, DO, DQ, DK, DV, L, Delta, SmScale, StrideHead, StrideSeq, StrideLse, NCtx,
  // one-dimensional kernels
  In0, In1, Out, Count, Scale, Bias, StrideIn, StrideOut, NCols,
  // sae_encode_kernel (x, w, out, M, D, F reuse A, B, C, M, K, N)
  BiasVec,
  Last = BiasVec
};

struct ArgInfo {
  int index = 0;
  bool is_pointer = false;
  std::string dtype;   // "f32" "f16" "bf16" "i32" "i64" "i1" ...
  std::string name;    // without the leading '%'
  Role role = Role::Unknown;
};

// What tm_emit_msl extracts from a module and what a "library" holds.
struct KernelDesc {
  KernelId id = KernelId::Matmul;
  Elt elt = Elt::F32;
  int block_m = 0, block_n = 0, block_k = 0, head_dim = 0;
  int threads = 128;
  int causal = 0;
  std::vector<ArgInfo> args;
};

// ir_scan.cpp -----------------------------------------------------------------
// Scan Triton IR text.  On failure returns false and fills `error` with a
// message in the reference's CoreError wording.
bool scan_module(const std::string& ttir, int num_simdgroups,
                 std::vector<KernelDesc>& out, std::string& error);
std::string descriptor_text(const std::vector<KernelDesc>& kernels);
bool parse_descriptor(const std::string& text, std::vector<KernelDesc>& out, std::string& error);
std::string kernel_info_json(const std::vector<KernelDesc>& kernels);

// ---------------------------------------------------------------------------
// Problem descriptions handed to the kernel launchers (device pointers)
// ---------------------------------------------------------------------------

struct GemmProblem {
  Elt elt;
  const void* a; const void* b; void* c;
  int64_t M, N, K;                 // effective extents (already clamped by the grid)
  int64_t sam, sak, sbk, sbn, scm, scn;   // strides in elements
  // fused epilogue (fp32 kernels only): C = max(acc + bias[n], 0) when `relu`; bias may be null
  const float* bias = nullptr;
  int relu = 0;
};

struct AttnProblem {
  Elt elt;
  const void* q; const void* k; const void* v; const void* o; const void* d_o;
  void* out0;       // O (fwd), Delta (preprocess), dQ (dq), dK (dkdv)
  void* out1;       // dV (dkdv) or nullptr
  float* lse;       // L: written by fwd (may be null), read by bwd
  const float* delta;
  float sm_scale;
  int64_t stride_head, stride_seq, stride_lse;
  int64_t n_ctx;
  int64_t rows;     // query rows (fwd, preprocess, dq) or key rows (dkdv) covered by the grid
  int64_t bh;       // batch*heads = grid_y
  int head_dim;
  int causal;
};

// One launch of a one-dimensional kernel: `limit` elements (already clamped by the grid) for
// the element-wise kernels; `rows` rows of `cols` columns (already clamped by BLOCK) for softmax.
struct RowProblem {
  KernelId id;
  const float* in0; const float* in1; float* out;
  int64_t limit;
  float scale, bias;
  int64_t rows, cols, stride_in, stride_out;
};

// Device status word: non-zero after a bounded wait inside a kernel gave up.
struct DeviceStatus {
  unsigned int code;      // 0 ok
  unsigned int where;     // role / barrier id that gave up
  unsigned int block;
  unsigned int extra;
};

struct LaunchCtx {
  cudaStream_t stream;
  int sm_count;
  DeviceStatus* status;   // device pointer
  int64_t* launches;      // incremented by each launcher per kernel launched
};

// Launchers.  Return nullptr on success or a static/owned error string.
// path_used: 1 SIMT, 2 tcgen05.
std::string launch_gemm_simt(const GemmProblem& p, const LaunchCtx& ctx);
std::string launch_attn_fwd_simt(const AttnProblem& p, const LaunchCtx& ctx);
std::string launch_attn_bwd_preprocess(const AttnProblem& p, const LaunchCtx& ctx);
std::string launch_attn_bwd_dq_simt(const AttnProblem& p, const LaunchCtx& ctx);
std::string launch_attn_bwd_dkdv_simt(const AttnProblem& p, const LaunchCtx& ctx);

// tcgen05 paths: `eligible` says whether the shape can take the path.
bool gemm_tc_eligible(const GemmProblem& p, std::string* why);
std::string launch_gemm_tc(const GemmProblem& p, const LaunchCtx& ctx);
// Row-sharded GEMM whose epilogue replicates C: every rank's copy of the whole C (device
// pointers: this rank's own memory at [rank], peer-mapped memory elsewhere), one flag array
// per rank (FLAG_SLOTS x 8 words; word slot*8 + s is raised by rank s), a counter in this
// rank's memory.
constexpr int kGatherMaxRanks = 8;
constexpr int kGatherFlagSlots = 64;
struct GemmGather {
  void* replica[kGatherMaxRanks];
  uint32_t* flags[kGatherMaxRanks];
  unsigned int* finished;
  int world, rank, slot;
  uint32_t epoch;
  int wait_for_peers;
  long long wait_budget_cycles;   // 0: the library's default (about a second)
  int tma_store;                  // tiles leave through TMA stores instead of st.global
};
std::string launch_gemm_tc_gathered(const GemmProblem& p, const GemmGather& g, const LaunchCtx& ctx);
// fp32 operands: 3xTF32 on the tensor cores, operands split into scratch memory.
bool gemm_tf32_eligible(const GemmProblem& p, std::string* why);
std::string launch_gemm_tf32(const GemmProblem& p, const LaunchCtx& ctx);           // library workspace
size_t gemm_tf32_scratch_bytes(int64_t M, int64_t N, int64_t K);
std::string run_gemm_tf32(const GemmProblem& p, const LaunchCtx& ctx, void* scratch);  // caller's scratch
std::string run_gemm_tf32_static(const GemmProblem& p, const LaunchCtx& ctx, int device);  // fixed device array
size_t gemm_tf32_static_capacity();
std::string prepare_gemm_tf32_static(int device);   // resolves the array's address (loads the module)
bool attn_fwd_tc_eligible(const AttnProblem& p, std::string* why);
std::string launch_attn_fwd_tc(const AttnProblem& p, const LaunchCtx& ctx);
bool attn_bwd_tc_eligible(const AttnProblem& p, std::string* why);
std::string launch_attn_bwd_dq_tc(const AttnProblem& p, const LaunchCtx& ctx);
std::string launch_attn_bwd_dkdv_tc(const AttnProblem& p, const LaunchCtx& ctx);

// fp32 attention with every contraction as a 3xTF32 GEMM over a materialised score matrix (long
// sequences); `forced`: the caller asked for the tensor-core path, so the lower length bound applies.
bool attn_f32_tc_eligible(const AttnProblem& p, bool forced, std::string* why);
std::string launch_attn_fwd_f32_tc(const AttnProblem& p, const LaunchCtx& ctx);
std::string launch_attn_bwd_dq_f32_tc(const AttnProblem& p, const LaunchCtx& ctx);
std::string launch_attn_bwd_dkdv_f32_tc(const AttnProblem& p, const LaunchCtx& ctx);

std::string launch_rowwise(const RowProblem& p, const LaunchCtx& ctx);

std::string launch_probe(const LaunchCtx& ctx, int* out_host);
// A kernel that waits, with the library's bounded waits and `budget_cycles`, on a barrier nothing
// arrives on; results_host[0..1]: 1 = the wait gave up (expected), 2 = it claimed success.
std::string launch_bounded_wait_selftest(const LaunchCtx& ctx, long long budget_cycles, int* results_host);

}  // namespace tmc
