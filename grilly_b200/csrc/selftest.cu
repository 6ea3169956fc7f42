// Self-test of the bounded-wait path: a one-CTA kernel waits, with the same helper the tcgen05 kernels use, on an
// mbarrier that nothing ever arrives on. The wait gives up after the given budget, the kernel records a status
// code and returns normally, so the host sees GRILLY_ERR_TIMEOUT at the next sync and the context stays usable.
// Nothing here traps, faults or spins without a limit.
#include "ptx.cuh"
#include "internal.h"

namespace gb {

__global__ void wait_timeout_selftest_kernel(int* err, unsigned long long budget_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!mbar_wait(&bar, 0, &abort_flag, budget_ns)) atomicCAS(err, 0, ERR_WAIT_FULL);
  }
}

}  // namespace gb

extern "C" int grilly_selftest_wait_timeout(grilly_ctx* ctx, int budget_ms) {
  if (!ctx) return GRILLY_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (cudaSetDevice(ctx->device) != cudaSuccess) return gb::set_error(ctx, GRILLY_ERR_CUDA, "cudaSetDevice failed");
  if (budget_ms < 1 || budget_ms > 1000) return gb::set_error(ctx, GRILLY_ERR_INVALID_ARG, "selftest: budget must be 1..1000 ms");
  gb::wait_timeout_selftest_kernel<<<1, 32, 0, ctx->stream>>>(ctx->err_dev, static_cast<unsigned long long>(budget_ms) * 1000000ull);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}
