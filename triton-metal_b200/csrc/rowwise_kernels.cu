// The one-dimensional kernels the reference's ABI tests launch (vector copy / add / multiply,
// scale-and-bias, row softmax: Tests/TritonMetalCoreTests/Fixtures.swift:8-125,
// python/tests/test_plugin_shape.py:24-90), fp32.  All are HBM-bound: 16-byte accesses when
// the pointers allow, a grid that is a multiple of the SM count, nothing staged on chip.
//
// Semantics kept from the Triton programs: program p covers elements [p*BLOCK, (p+1)*BLOCK)
// masked by i < n, so nothing beyond min(n, grid*BLOCK) is read or written (the host clamps
// `limit`); softmax_kernel's program r covers row r, columns < min(n_cols, BLOCK), and takes
// exp(x - max) / sum in fp32.

#include "tm_core.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

namespace tmc {
namespace {

enum class Op : int { Copy, Add, Mul, ScaleBias };

template <Op OP>
__device__ __forceinline__ float apply(float a, float b, float scale, float bias) {
  if (OP == Op::Copy) return a;
  if (OP == Op::Add) return a + b;
  if (OP == Op::Mul) return a * b;
  return __fadd_rn(__fmul_rn(a, scale), bias);     // a multiply then an add, as the program says
}

template <Op OP, bool VEC>
__global__ void __launch_bounds__(256) vec_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                  float* __restrict__ out, int64_t limit, float scale,
                                                  float bias) {
  constexpr bool TWO = OP == Op::Add || OP == Op::Mul;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (VEC) {
    const int64_t quads = limit / 4;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    float4* o4 = reinterpret_cast<float4*>(out);
    for (int64_t q = i; q < quads; q += stride) {
      const float4 x = __ldcs(a4 + q);
      float4 y = x;
      if (TWO) y = __ldcs(b4 + q);
      float4 r;
      r.x = apply<OP>(x.x, y.x, scale, bias);
      r.y = apply<OP>(x.y, y.y, scale, bias);
      r.z = apply<OP>(x.z, y.z, scale, bias);
      r.w = apply<OP>(x.w, y.w, scale, bias);
      __stcs(o4 + q, r);
    }
    for (int64_t t = quads * 4 + i; t < limit; t += stride) out[t] = apply<OP>(a[t], TWO ? b[t] : 0.f, scale, bias);
  } else {
    for (; i < limit; i += stride) out[i] = apply<OP>(a[i], TWO ? b[i] : 0.f, scale, bias);
  }
}

// One warp per row; a row is at most 65536 columns and is read twice from L1/L2 when it does
// not fit the 32 values a lane keeps in registers.
__global__ void __launch_bounds__(256) softmax_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                      int64_t rows, int64_t cols, int64_t stride_in,
                                                      int64_t stride_out) {
  const int lane = threadIdx.x % 32;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x / 32);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32; row < rows; row += warps) {
    const float* x = in + row * stride_in;
    float* y = out + row * stride_out;
    float m = -INFINITY;
    for (int64_t c = lane; c < cols; c += 32) m = fmaxf(m, x[c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
    for (int64_t c = lane; c < cols; c += 32) sum += expf(x[c] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    for (int64_t c = lane; c < cols; c += 32) y[c] = expf(x[c] - m) / sum;
  }
}

template <Op OP>
void launch_vec(const RowProblem& p, const LaunchCtx& ctx) {
  const bool two = OP == Op::Add || OP == Op::Mul;
  const bool aligned = (((uintptr_t)p.in0 | (uintptr_t)p.out | (two ? (uintptr_t)p.in1 : 0)) % 16) == 0;
  const int64_t work = aligned ? (p.limit + 3) / 4 : p.limit;
  int64_t blocks = (work + 255) / 256;
  const int64_t cap = (int64_t)ctx.sm_count * 8;       // 8 resident CTAs of 256 threads per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (aligned)
    vec_kernel<OP, true><<<(unsigned)blocks, 256, 0, ctx.stream>>>(p.in0, p.in1, p.out, p.limit, p.scale, p.bias);
  else
    vec_kernel<OP, false><<<(unsigned)blocks, 256, 0, ctx.stream>>>(p.in0, p.in1, p.out, p.limit, p.scale, p.bias);
}

}  // namespace

std::string launch_rowwise(const RowProblem& p, const LaunchCtx& ctx) {
  switch (p.id) {
    case KernelId::VecCopy: launch_vec<Op::Copy>(p, ctx); break;
    case KernelId::VecAdd: launch_vec<Op::Add>(p, ctx); break;
    case KernelId::VecMul: launch_vec<Op::Mul>(p, ctx); break;
    case KernelId::ScaleBias: launch_vec<Op::ScaleBias>(p, ctx); break;
    case KernelId::Softmax: {
      int64_t blocks = (p.rows + 7) / 8;
      const int64_t cap = (int64_t)ctx.sm_count * 8;
      if (blocks > cap) blocks = cap;
      softmax_kernel<<<(unsigned)blocks, 256, 0, ctx.stream>>>(p.in0, p.out, p.rows, p.cols, p.stride_in,
                                                              p.stride_out);
      break;
    }
    default: return "not a one-dimensional kernel";
  }
  ++*ctx.launches;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return std::string(kernel_entry_name(p.id)) + " launch failed: " + cudaGetErrorString(e);
  return std::string();
}

}  // namespace tmc
