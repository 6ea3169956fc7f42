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

  gb::NormArgs n{};
  n.x = x_dev; n.rows = M; n.F = K; n.eps = eps; n.mode = norm_mode;
  n.mean_out = stats; n.rstd_out = stats + kMaxRows;
  if ((rc = gb::launch_norm(ctx, n))) return rc;
  gb::GemmArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.bias = bias_f_dev;
  a.out = y_dev; a.ld_out = N;
  a.out_bf16 = (flags & GRILLY_FLAG_OUT_BF16) ? 1 : 0;
  a.round_tf32 = (flags & GRILLY_FLAG_ROUND_TF32) ? 1 : 0;
  a.act = act;
  a.row_rstd = stats + kMaxRows;
  a.row_mean = norm_mode == GRILLY_NORM_LAYER ? stats : nullptr;
  a.col_sum = col_sum_dev;
  return gb::launch_gemm(ctx, false, false, x_dev, wf_dev, a, 0);
}
