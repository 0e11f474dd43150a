// Self-test of the bounded-wait machinery every tcgen05 kernel of this library relies on.
//
// The kernels wait on mbarriers with a cycle budget; when it runs out they record where in a
// host-visible status word, raise the CTA's abort flag and return, and the next host-side
// synchronisation reports the launch as failed.  That path cannot be reached through the
// real kernels without breaking one of them, so this file holds a tiny kernel that waits -
// with the same mbar_wait / mbar_wait_warp the real kernels use and a short budget - on a
// barrier nothing ever arrives on.  The wait runs out, the status is written and the kernel
// returns normally: no trap, no fault, the context stays usable.

#include "sm100_ptx.cuh"

namespace tmc {
namespace {

using namespace ptx;

constexpr uint32_t kSelfTestThreadSite = 90, kSelfTestWarpSite = 91;

// Block of 64 threads.  Warp 0: lane 0 waits alone (the form the TMA and element-wise roles
// use).  Warp 1: the whole warp waits by vote (the form the MMA issuer uses).  results[0..1]
// get 1 when the wait came back "gave up" as it must, 2 if it claimed success.
__global__ void bounded_wait_selftest_kernel(DeviceStatus* status, long long budget, int* results) {
  __shared__ alignas(8) uint64_t never;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&never), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  WaitCtx wc{&abort_flag, status, budget};
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  if (warp == 0) {
    if (lane == 0) results[0] = mbar_wait(smem_u32(&never), 0, wc, kSelfTestThreadSite) ? 2 : 1;
  } else {
    const bool got = mbar_wait_warp(smem_u32(&never), 0, wc, kSelfTestWarpSite);
    if (lane == 0) results[1] = got ? 2 : 1;
  }
  __syncthreads();
}

}  // namespace

// Runs the self-test on the library's stream.  `results_host` (two ints) receives what the two
// waits returned; the status word is left for the caller's synchronisation to pick up.
std::string launch_bounded_wait_selftest(const LaunchCtx& ctx, long long budget_cycles, int* results_host) {
  int* dev = nullptr;
  cudaError_t e = cudaMalloc(&dev, 2 * sizeof(int));
  if (e != cudaSuccess) return cudaGetErrorString(e);
  cudaMemsetAsync(dev, 0, 2 * sizeof(int), ctx.stream);
  bounded_wait_selftest_kernel<<<1, 64, 0, ctx.stream>>>(ctx.status, budget_cycles, dev);
  ++*ctx.launches;
  e = cudaGetLastError();
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(results_host, dev, 2 * sizeof(int), cudaMemcpyDeviceToHost, ctx.stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx.stream);
  cudaFree(dev);
  if (e != cudaSuccess) return cudaGetErrorString(e);
  return std::string();
}

}  // namespace tmc
