// grilly_layernorm_linear_noalloc: Linear(LayerNorm(x)) for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc when they run an op: a serving thread that has promised
// its scheduler a fixed memory footprint, or a process whose whole device memory has already been handed to
// another allocator (a framework's caching pool), where a late cudaMalloc can fail or stall the device while
// the driver maps memory. grilly_layernorm_linear needs scratch for the per-row mean and 1/std; this variant
// keeps that scratch inside the library image instead: a fixed array in device memory that every GPU which
// loads the library holds from load time until the process exits (512 KiB).
//
// Consequences the caller has to know:
//  * at most GRILLY_NOALLOC_MAX_ROWS rows per call; more is rejected with GRILLY_ERR_INVALID_ARG;
//  * all calls on a device share the one array, so two calls that overlap on the GPU (different streams or
//    contexts on the same device) race on it; calls issued on one stream are ordered and safe;
//  * the array keeps whatever the previous call left. Nothing here relies on it starting at zero: the
//    statistics kernel writes rows [0, M) before the GEMM reads exactly those rows;
//  * in LayerNorm mode the result is computed by the folded form only (GEMM on the raw rows, normalisation finished
//    in the epilogue), which is accurate while no row mean is more than GRILLY_LNLINEAR_MAX_MEAN_OVER_STD standard
//    deviations from zero. The allocating entry point switches to normalise-then-GEMM beyond that, which needs
//    M x K scratch; this one cannot, and returns GRILLY_ERR_UNSUPPORTED for such inputs (y is not written);
//  * the first launch of each kernel variant makes the CUDA runtime load its code, which takes device memory for
//    the code itself; a caller that must not see any allocation issues one warm-up call per shape class first;
//  * the first call on each device looks up the array's device address (cudaGetSymbolAddress). Make that first
//    call before any stream capture is started on the stream.
#include "args.h"
#include "internal.h"

namespace {

constexpr int kMaxRows = GRILLY_NOALLOC_MAX_ROWS;
constexpr int kMaxDevices = 64;

// mean[0 .. kMaxRows) followed by rstd[0 .. kMaxRows). In host code this name is only a handle for the
// runtime's symbol lookup, not a device address: kernels get the pointer returned by cudaGetSymbolAddress.
static __device__ __align__(256) float g_norm_stats_scratch[2 * kMaxRows];

// One resolved address per device for the whole process. Contexts of different devices run under different context
// mutexes, so the table has a lock of its own.
float* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mu;

int scratch_for_device(grilly_ctx* ctx, float** out) {
  if (ctx->device < 0 || ctx->device >= kMaxDevices)
    return gb::set_error(ctx, GRILLY_ERR_UNSUPPORTED, "layernorm_linear_noalloc: device index out of range");
  std::lock_guard<std::mutex> table_lock(g_scratch_mu);
  if (!g_scratch_addr[ctx->device]) {
    // once per device, with that device current (the caller has already made it current)
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_norm_stats_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      return gb::set_error(ctx, GRILLY_ERR_CUDA,
                           std::string("layernorm_linear_noalloc: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
    }
    g_scratch_addr[ctx->device] = static_cast<float*>(p);
  }
  *out = g_scratch_addr[ctx->device];
  return GRILLY_OK;
}

}  // namespace

extern "C" int grilly_layernorm_linear_noalloc(grilly_ctx* ctx, const float* x_dev, const void* wf_dev,
                                               const float* col_sum_dev, const float* bias_f_dev, void* y_dev, int M,
                                               int N, int K, float eps, int norm_mode, int act, int precision, int flags) {
  if (!ctx) return GRILLY_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (cudaSetDevice(ctx->device) != cudaSuccess) return gb::set_error(ctx, GRILLY_ERR_CUDA, "cudaSetDevice failed");
  if (precision != GRILLY_PREC_TF32 && precision != GRILLY_PREC_BF16)
    return gb::set_error(ctx, GRILLY_ERR_INVALID_ARG, "precision must be GRILLY_PREC_TF32 or GRILLY_PREC_BF16");
  if (!x_dev || !wf_dev || !y_dev) return gb::set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_linear_noalloc: null operand");
  if (M <= 0 || N <= 0 || K <= 0) return gb::set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_linear_noalloc: M, N, K must be positive");
  if (M > kMaxRows)
    return gb::set_error(ctx, GRILLY_ERR_INVALID_ARG,
                         "layernorm_linear_noalloc: " + std::to_string(M) + " rows exceed the built-in scratch of " +
                             std::to_string(kMaxRows) + " rows; split the call or use grilly_layernorm_linear");
  if (precision != GRILLY_PREC_TF32)
    return gb::set_error(ctx, GRILLY_ERR_UNSUPPORTED, "layernorm_linear_noalloc: x is fp32, so only GRILLY_PREC_TF32 is supported");
  if (norm_mode != GRILLY_NORM_LAYER && norm_mode != GRILLY_NORM_RMS)
    return gb::set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_linear_noalloc: unknown norm mode");
  if (norm_mode == GRILLY_NORM_LAYER && !col_sum_dev)
    return gb::set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_linear_noalloc: col_sum is required for LayerNorm");
  if (act < GRILLY_ACT_NONE || act > GRILLY_ACT_RELU)
    return gb::set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_linear_noalloc: unknown activation");
  float* stats = nullptr;
  int rc = scratch_for_device(ctx, &stats);
  if (rc) return rc;

  return gb::layernorm_linear_impl(ctx, x_dev, wf_dev, col_sum_dev, bias_f_dev, y_dev, stats, stats + kMaxRows, M, N, K, eps,
                                   norm_mode, act, precision, flags, /*may_allocate=*/false);
}
