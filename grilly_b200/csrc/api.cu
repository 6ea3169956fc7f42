// C ABI of libgrilly_b200.so: context, stream-ordered device pool, tensor-map
// cache and the operator entry points declared in include/grilly_b200.h.
#include "internal.h"
#include "args.h"
#include <cudaTypedefs.h>
#include <cstdlib>

namespace gb {

int set_error(grilly_ctx* ctx, int code, const std::string& msg) {
  if (ctx) ctx->last_error = msg;
  return code;
}

int prof_begin(grilly_ctx* ctx, int cls, double flops, double bytes) {
  if (!ctx->profiling) return -1;
  grilly_ctx::ProfRec r{cls, nullptr, nullptr, flops, bytes};
  if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return -1;
  cudaEventRecord(r.a, ctx->stream);
  ctx->prof.push_back(r);
  return static_cast<int>(ctx->prof.size()) - 1;
}
void prof_end(grilly_ctx* ctx, int idx) {
  if (idx >= 0) cudaEventRecord(ctx->prof[idx].b, ctx->stream);
}

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

static int load_encode(grilly_ctx* ctx) {
  if (g_encode) return GRILLY_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
    return set_error(ctx, GRILLY_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  return GRILLY_OK;
}

int get_tmap_2d(grilly_ctx* ctx, int dtype, const void* ptr, uint64_t inner, uint64_t outer, uint64_t stride_bytes,
                uint32_t box_inner, uint32_t box_outer, CUtensorMap* out, int swizzle) {
  TmapKey key{ptr, inner, outer, stride_bytes, box_inner, box_outer, dtype, swizzle};
  auto it = ctx->tmaps.find(key);
  if (it != ctx->tmaps.end()) {
    ctx->tmap_hits++;
    *out = it->second;
    return GRILLY_OK;
  }
  int rc = load_encode(ctx);
  if (rc) return rc;
  if (box_inner > 256 || box_outer > 256) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "tensor map: box dimension above 256");
  if (stride_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(ptr) & 15))
    return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "tensor map: base and row pitch must be multiples of 16 bytes");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = g_encode(&m, dtype == TM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                        const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle == TM_SW128_ATOM32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : swizzle == TM_SWNONE ? CU_TENSOR_MAP_SWIZZLE_NONE
                        : swizzle == TM_SW64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(ctx, GRILLY_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
  ctx->tmap_misses++;
  if (ctx->tmaps.size() > 4096) ctx->tmaps.clear();
  ctx->tmaps.emplace(key, m);
  *out = m;
  return GRILLY_OK;
}

}  // namespace gb

using namespace gb;

#define CTX_GUARD(ctx)                                  \
  if (!(ctx)) return GRILLY_ERR_INVALID_ARG;            \
  std::lock_guard<std::mutex> lock__((ctx)->mu);        \
  if (cudaSetDevice((ctx)->device) != cudaSuccess) return set_error(ctx, GRILLY_ERR_CUDA, "cudaSetDevice failed")

extern "C" {

int grilly_device_count(int* count) {
  if (!count) return GRILLY_ERR_INVALID_ARG;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) { *count = 0; cudaGetLastError(); return GRILLY_ERR_CUDA; }
  *count = n;
  return GRILLY_OK;
}

int grilly_init(int device, grilly_ctx** out) {
  if (!out) return GRILLY_ERR_INVALID_ARG;
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { cudaGetLastError(); return GRILLY_ERR_CUDA; }
  if (device < 0 || device >= n) return GRILLY_ERR_INVALID_ARG;
  if (cudaSetDevice(device) != cudaSuccess) return GRILLY_ERR_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return GRILLY_ERR_CUDA;
  if (prop.major != 10) return GRILLY_ERR_UNSUPPORTED;  // the kernels are sm_100a only
  grilly_ctx* ctx = new grilly_ctx();
  ctx->device = device;
  ctx->num_sms = prop.multiProcessorCount;
  bool ok = cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) == cudaSuccess;
  ctx->stream = ctx->own_stream;
  ok = ok && cudaDeviceGetDefaultMemPool(&ctx->pool, device) == cudaSuccess;
  if (ok) {
    // keep freed blocks in the pool instead of returning them to the driver (buffer reuse across calls)
    uint64_t thresh = UINT64_MAX;
    ok = cudaMemPoolSetAttribute(ctx->pool, cudaMemPoolAttrReleaseThreshold, &thresh) == cudaSuccess;
  }
  ok = ok && cudaMalloc(&ctx->err_dev, 4 * sizeof(int)) == cudaSuccess;  // [0] status word, [1] attention work counter, [2] layernorm_linear's max |mean|/std
  ok = ok && cudaMemset(ctx->err_dev, 0, 4 * sizeof(int)) == cudaSuccess;
  ok = ok && cudaMallocHost(&ctx->err_host, 2 * sizeof(int)) == cudaSuccess;   // [0] status, [1] mirror of word [2]
  if (!ok) {
    cudaGetLastError();
    delete ctx;
    return GRILLY_ERR_CUDA;
  }
  *ctx->err_host = 0;
  // tuning/debug overrides: read here once, never on the launch path
  auto env_int = [](const char* name, int fallback) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : fallback;
  };
  ctx->tune.gemm_group = env_int("GRILLY_GEMM_GROUP", 0);
  ctx->tune.gemm_bn = env_int("GRILLY_GEMM_BN", 0);
  ctx->tune.gemm_pair = env_int("GRILLY_GEMM_PAIR", -1);
  ctx->tune.gemm_swap = env_int("GRILLY_GEMM_SWAP", -1);
  ctx->tune.attn_hpc = env_int("GRILLY_ATTN_HPC", 0);
  ctx->tune.attn_general = getenv("GRILLY_ATTN_GENERAL") != nullptr ? 1 : 0;
  ctx->tune.fused_ln = env_int("GRILLY_FUSED_LN", 1);
  *out = ctx;
  return GRILLY_OK;
}

int grilly_shutdown(grilly_ctx* ctx) {
  if (!ctx) return GRILLY_ERR_INVALID_ARG;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  for (auto& kv : ctx->live) cudaFreeAsync(kv.first, ctx->own_stream);
  for (auto& t : ctx->rope_tables) { cudaFree(t.cos_t); cudaFree(t.sin_t); }
  if (ctx->timer_a) { cudaEventDestroy(ctx->timer_a); cudaEventDestroy(ctx->timer_b); }
  cudaStreamSynchronize(ctx->own_stream);
  cudaFree(ctx->err_dev);
  cudaFreeHost(ctx->err_host);
  cudaStreamDestroy(ctx->own_stream);
  delete ctx;
  return GRILLY_OK;
}

const char* grilly_last_error(grilly_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

int grilly_set_stream(grilly_ctx* ctx, void* cuda_stream) {
  CTX_GUARD(ctx);
  ctx->stream = cuda_stream ? reinterpret_cast<cudaStream_t>(cuda_stream) : ctx->own_stream;
  return GRILLY_OK;
}

int grilly_set_tuning(grilly_ctx* ctx, const char* name, int value) {
  CTX_GUARD(ctx);
  if (!name) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "set_tuning: null name");
  const std::string n(name);
  if (n == "gemm_group") ctx->tune.gemm_group = value;
  else if (n == "gemm_bn") ctx->tune.gemm_bn = value;
  else if (n == "gemm_pair") ctx->tune.gemm_pair = value;
  else if (n == "gemm_swap") ctx->tune.gemm_swap = value;
  else if (n == "attn_hpc") ctx->tune.attn_hpc = value;
  else if (n == "attn_general") ctx->tune.attn_general = value;
  else if (n == "fused_ln") ctx->tune.fused_ln = value;
  else return set_error(ctx, GRILLY_ERR_INVALID_ARG, "set_tuning: unknown knob '" + n + "'");
  return GRILLY_OK;
}

static int check_device_status(grilly_ctx* ctx) {
  // read back the status word the bounded waits write
  GB_CUDA_CHECK(ctx, cudaMemcpyAsync(ctx->err_host, ctx->err_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  GB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
  if (*ctx->err_host != 0) {
    const int code = *ctx->err_host;
    *ctx->err_host = 0;
    cudaMemsetAsync(ctx->err_dev, 0, sizeof(int), ctx->stream);
    return set_error(ctx, GRILLY_ERR_TIMEOUT, "a device-side wait gave up (kernel status " + std::to_string(code) + ")");
  }
  return GRILLY_OK;
}

int grilly_sync(grilly_ctx* ctx) {
  CTX_GUARD(ctx);
  return check_device_status(ctx);
}

int grilly_launch_count(grilly_ctx* ctx, uint64_t* count) {
  if (!ctx || !count) return GRILLY_ERR_INVALID_ARG;
  *count = ctx->launches;
  return GRILLY_OK;
}

int grilly_timer_start(grilly_ctx* ctx) {
  CTX_GUARD(ctx);
  if (!ctx->timer_a) {
    GB_CUDA_CHECK(ctx, cudaEventCreate(&ctx->timer_a));
    GB_CUDA_CHECK(ctx, cudaEventCreate(&ctx->timer_b));
  }
  GB_CUDA_CHECK(ctx, cudaEventRecord(ctx->timer_a, ctx->stream));
  return GRILLY_OK;
}

int grilly_timer_stop(grilly_ctx* ctx, float* ms) {
  CTX_GUARD(ctx);
  if (!ms || !ctx->timer_a) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "timer_stop: no timer running or null output");
  GB_CUDA_CHECK(ctx, cudaEventRecord(ctx->timer_b, ctx->stream));
  GB_CUDA_CHECK(ctx, cudaEventSynchronize(ctx->timer_b));
  GB_CUDA_CHECK(ctx, cudaEventElapsedTime(ms, ctx->timer_a, ctx->timer_b));
  return GRILLY_OK;
}

int grilly_profile_begin(grilly_ctx* ctx) {
  CTX_GUARD(ctx);
  for (auto& r : ctx->prof) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  ctx->prof.clear();
  ctx->profiling = true;
  return GRILLY_OK;
}

int grilly_profile_end(grilly_ctx* ctx, double* out) {
  CTX_GUARD(ctx);
  if (!out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "profile_end: null output");
  ctx->profiling = false;
  GB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
  for (int i = 0; i < PROF_NCLASS * 4; ++i) out[i] = 0.0;
  for (auto& r : ctx->prof) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
      out[r.cls * 4 + 0] += 1.0;
      out[r.cls * 4 + 1] += ms;
      out[r.cls * 4 + 2] += r.flops;
      out[r.cls * 4 + 3] += r.bytes;
    }
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
  }
  ctx->prof.clear();
  cudaGetLastError();
  return GRILLY_OK;
}

int grilly_alloc(grilly_ctx* ctx, size_t bytes, void** dptr) {
  CTX_GUARD(ctx);
  if (!dptr) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "alloc: null output pointer");
  if (bytes == 0) bytes = 16;
  void* p = nullptr;
  // a "hit" in the sense of BufferPool.acquire (backend/buffer_pool.py:534-562): the pool served the request from
  // memory it already held, i.e. its reserved size did not grow
  uint64_t reserved_before = 0, reserved_after = 0;
  cudaMemPoolGetAttribute(ctx->pool, cudaMemPoolAttrReservedMemCurrent, &reserved_before);
  cudaError_t e = cudaMallocAsync(&p, bytes, ctx->stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return set_error(ctx, e == cudaErrorMemoryAllocation ? GRILLY_ERR_OOM : GRILLY_ERR_CUDA,
                     std::string("cudaMallocAsync: ") + cudaGetErrorString(e));
  }
  cudaMemPoolGetAttribute(ctx->pool, cudaMemPoolAttrReservedMemCurrent, &reserved_after);
  if (reserved_after <= reserved_before) ctx->pool_hits++;
  ctx->live[p] = bytes;
  ctx->n_alloc++;
  ctx->bytes_in_use += bytes;
  if (ctx->bytes_in_use > ctx->peak_bytes) ctx->peak_bytes = ctx->bytes_in_use;
  *dptr = p;
  return GRILLY_OK;
}

int grilly_free(grilly_ctx* ctx, void* dptr) {
  CTX_GUARD(ctx);
  if (!dptr) return GRILLY_OK;
  auto it = ctx->live.find(dptr);
  if (it == ctx->live.end()) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "free: pointer was not allocated by this context");
  ctx->bytes_in_use -= it->second;
  ctx->live.erase(it);
  ctx->n_free++;
  // descriptors built over this buffer must not outlive it
  for (auto t = ctx->tmaps.begin(); t != ctx->tmaps.end();) {
    if (t->first.ptr == dptr) t = ctx->tmaps.erase(t); else ++t;
  }
  GB_CUDA_CHECK(ctx, cudaFreeAsync(dptr, ctx->stream));
  return GRILLY_OK;
}

int grilly_upload(grilly_ctx* ctx, void* dst, const void* src, size_t bytes) {
  CTX_GUARD(ctx);
  if (!dst || !src) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "upload: null pointer");
  GB_CUDA_CHECK(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  // pageable sources are staged by the runtime before the call returns; pinned ones must stay valid until sync
  return GRILLY_OK;
}

int grilly_download(grilly_ctx* ctx, void* dst, const void* src, size_t bytes) {
  CTX_GUARD(ctx);
  if (!dst || !src) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "download: null pointer");
  GB_CUDA_CHECK(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return check_device_status(ctx);
}

int grilly_memset(grilly_ctx* ctx, void* dst, int byte_value, size_t nbytes) {
  CTX_GUARD(ctx);
  if (!dst && nbytes) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "memset: null destination");
  if (nbytes) GB_CUDA_CHECK(ctx, cudaMemsetAsync(dst, byte_value, nbytes, ctx->stream));
  return GRILLY_OK;
}

int grilly_copy_2d(grilly_ctx* ctx, void* dst_dev, size_t dst_pitch, const void* src_dev, size_t src_pitch, size_t width_bytes,
                   size_t rows) {
  CTX_GUARD(ctx);
  if (!dst_dev || !src_dev) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "copy_2d: null pointer");
  if (width_bytes > dst_pitch || width_bytes > src_pitch) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "copy_2d: width exceeds a pitch");
  if (width_bytes == 0 || rows == 0) return GRILLY_OK;
  // cudaMemcpyDefault: either side may be memory of another GPU mapped into this process; the copy engines move it
  GB_CUDA_CHECK(ctx, cudaMemcpy2DAsync(dst_dev, dst_pitch, src_dev, src_pitch, width_bytes, rows, cudaMemcpyDefault, ctx->stream));
  return GRILLY_OK;
}

int grilly_host_alloc(grilly_ctx* ctx, size_t bytes, void** hptr) {
  CTX_GUARD(ctx);
  if (!hptr) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "host_alloc: null output pointer");
  GB_CUDA_CHECK(ctx, cudaMallocHost(hptr, bytes ? bytes : 16));
  return GRILLY_OK;
}
int grilly_host_free(grilly_ctx* ctx, void* hptr) {
  CTX_GUARD(ctx);
  if (hptr) GB_CUDA_CHECK(ctx, cudaFreeHost(hptr));
  return GRILLY_OK;
}

int grilly_pool_stats(grilly_ctx* ctx, uint64_t out[8]) {
  CTX_GUARD(ctx);
  if (!out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "pool_stats: null output");
  uint64_t reserved = 0;
  cudaMemPoolGetAttribute(ctx->pool, cudaMemPoolAttrReservedMemCurrent, &reserved);
  out[0] = ctx->n_alloc; out[1] = ctx->n_free; out[2] = ctx->bytes_in_use; out[3] = ctx->peak_bytes;
  out[4] = reserved; out[5] = ctx->tmap_hits; out[6] = ctx->tmap_misses; out[7] = ctx->pool_hits;
  return GRILLY_OK;
}

int grilly_round_tf32(grilly_ctx* ctx, const float* x, float* y, long long n) {
  CTX_GUARD(ctx);
  return launch_round_tf32(ctx, x, y, n);
}
int grilly_cast_f32_to_bf16(grilly_ctx* ctx, const float* x, void* y, long long n) {
  CTX_GUARD(ctx);
  return launch_f32_to_bf16(ctx, x, y, n);
}
int grilly_cast_bf16_to_f32(grilly_ctx* ctx, const void* x, float* y, long long n) {
  CTX_GUARD(ctx);
  return launch_bf16_to_f32(ctx, x, y, n);
}

static int check_prec(grilly_ctx* ctx, int precision, bool x3_ok = false) {
  if (precision == GRILLY_PREC_TF32X3 && x3_ok) return GRILLY_OK;
  if (precision == GRILLY_PREC_TF32X3)
    return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "GRILLY_PREC_TF32X3 is offered by linear, fused_qkv_projection and gemm_mnk only");
  if (precision != GRILLY_PREC_TF32 && precision != GRILLY_PREC_BF16)
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "precision must be GRILLY_PREC_TF32, GRILLY_PREC_BF16 or GRILLY_PREC_TF32X3");
  return GRILLY_OK;
}

static int linear_nolock(grilly_ctx* ctx, const void* x, const void* w, const float* bias, const float* residual, void* y,
                         int M, int N, int K, int act, int precision, int flags) {
  int rc = check_prec(ctx, precision, true);
  if (rc) return rc;
  if (!x || !w || !y) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "linear: null operand");
  if (act < GRILLY_ACT_NONE || act > GRILLY_ACT_RELU) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "linear: unknown activation");
  GemmArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.bias = bias; a.residual = residual;
  a.swiglu_pairs = (flags & GRILLY_FLAG_SWIGLU_PAIRS) ? 1 : 0;
  a.ld_res = a.swiglu_pairs ? N / 2 : N;
  a.out = y; a.ld_out = a.swiglu_pairs ? N / 2 : N;
  a.out_bf16 = (flags & GRILLY_FLAG_OUT_BF16) ? 1 : 0;
  a.round_tf32 = (flags & GRILLY_FLAG_ROUND_TF32) ? 1 : 0;
  a.act = act;
  if (a.swiglu_pairs && residual) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "linear: SwiGLU pairs with a residual is not supported");
  if (precision == GRILLY_PREC_TF32X3) {
    if (M <= 0 || N <= 0 || K <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "gemm: M, N, K must be positive");
    return linear_tf32x3(ctx, static_cast<const float*>(x), static_cast<const float*>(w), a);
  }
  return launch_gemm(ctx, precision == GRILLY_PREC_BF16, false, x, w, a, 0);
}

int grilly_linear(grilly_ctx* ctx, const void* x, const void* w, const float* bias, const float* residual, void* y, int M,
                  int N, int K, int act, int precision, int flags) {
  CTX_GUARD(ctx);
  return linear_nolock(ctx, x, w, bias, residual, y, M, N, K, act, precision, flags);
}

int grilly_fused_qkv_projection(grilly_ctx* ctx, const void* x, const void* w_qkv, const float* b_qkv, void* qkv, int rows,
                                int hidden, int num_heads, int head_dim, int precision, int flags) {
  CTX_GUARD(ctx);
  if (num_heads <= 0 || head_dim <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "qkv: heads and head_dim must be positive");
  return linear_nolock(ctx, x, w_qkv, b_qkv, nullptr, qkv, rows, 3 * num_heads * head_dim, hidden, GRILLY_ACT_NONE, precision, flags);
}

int grilly_fold_layernorm_weights(grilly_ctx* ctx, const float* w, const float* gamma, const float* beta, const float* bias,
                                  void* wf, float* col_sum, float* bias_f, int N, int K, int precision) {
  CTX_GUARD(ctx);
  int rc = check_prec(ctx, precision);
  if (rc) return rc;
  if (!w || !wf || !col_sum || !bias_f) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "fold_layernorm_weights: null operand");
  return launch_fold_ln(ctx, w, gamma, beta, bias, wf, col_sum, bias_f, N, K, precision == GRILLY_PREC_BF16);
}

}  // extern "C"

namespace gb {
// Linear(Norm(x)) shared by grilly_layernorm_linear and its no-allocation variant. mean / rstd: scratch for M floats
// each. The folded form runs the GEMM on the RAW rows and finishes y = rstd (acc - mean col_sum) + bias' in the
// epilogue; its rounding error grows with |row mean| / (row std), so in LayerNorm mode the statistics kernel also
// reports the largest such ratio and beyond GRILLY_LNLINEAR_MAX_MEAN_OVER_STD the rows are normalised first
// (x^ = (x - mean) rstd, rounded for the MMA, into scratch of M x K elements) and the GEMM runs on x^ with the same
// folded weights: y = x^ W'^T + bias'. RMSNorm has no mean term and always takes the folded form.
int layernorm_linear_impl(grilly_ctx* ctx, const void* x, const void* wf, const float* col_sum, const float* bias_f, void* y,
                          float* mean, float* rstd, int M, int N, int K, float eps, int norm_mode, int act, int precision,
                          int flags, bool may_allocate) {
  const bool bf16 = precision == GRILLY_PREC_BF16;
  if (M <= 0 || N <= 0 || K <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_linear: M, N, K must be positive");
  if (act < GRILLY_ACT_NONE || act > GRILLY_ACT_RELU) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_linear: unknown activation");
  if (norm_mode != GRILLY_NORM_LAYER && norm_mode != GRILLY_NORM_RMS) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_linear: unknown norm mode");
  unsigned* ratio_dev = reinterpret_cast<unsigned*>(ctx->err_dev + 2);
  const bool layer = norm_mode == GRILLY_NORM_LAYER;
  if (layer) GB_CUDA_CHECK(ctx, cudaMemsetAsync(ratio_dev, 0, sizeof(unsigned), ctx->stream));
  NormArgs n{};
  n.x = static_cast<const float*>(x); n.x_bf16 = bf16 ? 1 : 0; n.rows = M; n.F = K; n.eps = eps; n.mode = norm_mode;
  n.mean_out = mean; n.rstd_out = rstd; n.ratio_max = layer ? ratio_dev : nullptr;
  int rc = launch_norm(ctx, n);
  if (rc) return rc;
  GemmArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.bias = bias_f;
  a.out = y; a.ld_out = N;
  a.out_bf16 = (flags & GRILLY_FLAG_OUT_BF16) ? 1 : 0;
  a.round_tf32 = (flags & GRILLY_FLAG_ROUND_TF32) ? 1 : 0;
  a.act = act;
  if (layer) {
    // one small read-back decides the form (the only synchronisation of this entry point; RMS mode has none)
    int* mirror = ctx->err_host + 1;
    GB_CUDA_CHECK(ctx, cudaMemcpyAsync(mirror, ratio_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    GB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    float ratio;
    std::memcpy(&ratio, mirror, sizeof(float));
    if (!(ratio <= GRILLY_LNLINEAR_MAX_MEAN_OVER_STD)) {   // also taken for NaN statistics
      if (!may_allocate)
        return set_error(ctx, GRILLY_ERR_UNSUPPORTED,
                         "layernorm_linear_noalloc: a row mean is " + std::to_string(ratio) + " standard deviations from zero, beyond the "
                         "folded form's accuracy envelope; grilly_layernorm_linear handles such rows (it normalises them into scratch first)");
      const size_t elt = bf16 ? 2 : 4;
      void* xn = nullptr;
      if (cudaMallocAsync(&xn, static_cast<size_t>(M) * K * elt, ctx->stream) != cudaSuccess) {
        cudaGetLastError();
        return set_error(ctx, GRILLY_ERR_OOM, "layernorm_linear: no memory for the normalised rows");
      }
      NormArgs m = n;
      m.mean_out = nullptr; m.rstd_out = nullptr; m.ratio_max = nullptr;
      m.y = xn; m.out_bf16 = bf16 ? 1 : 0; m.round_tf32 = bf16 ? 0 : 1;   // gamma and beta already live in the folded weights
      rc = launch_norm(ctx, m);
      if (!rc) rc = launch_gemm(ctx, bf16, false, xn, wf, a, 0);
      cudaFreeAsync(xn, ctx->stream);
      return rc;
    }
  }
  a.row_rstd = rstd;
  a.row_mean = layer ? mean : nullptr;
  a.col_sum = col_sum;
  return launch_gemm(ctx, bf16, false, x, wf, a, 0);
}
}  // namespace gb

extern "C" {

int grilly_layernorm_linear(grilly_ctx* ctx, const void* x, const void* wf, const float* col_sum, const float* bias_f,
                            void* y, float* stats, int M, int N, int K, float eps, int norm_mode, int act, int precision,
                            int flags) {
  CTX_GUARD(ctx);
  int rc = check_prec(ctx, precision);
  if (rc) return rc;
  if (!x || !wf || !y || !stats) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_linear: null operand");
  if (norm_mode == GRILLY_NORM_LAYER && !col_sum) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_linear: col_sum is required");
  return layernorm_linear_impl(ctx, x, wf, col_sum, bias_f, y, stats, stats + M, M, N, K, eps, norm_mode, act, precision, flags, true);
}

int grilly_linear_layernorm(grilly_ctx* ctx, const void* x, const void* w, const float* bias, const void* residual,
                            const float* gamma, const float* beta, void* y, float* scratch, int M, int N, int K, float eps,
                            int precision, int flags) {
  CTX_GUARD(ctx);
  int rc = check_prec(ctx, precision);
  if (rc) return rc;
  if (!x || !w || !y) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "linear_layernorm: null operand");
  const bool bf16 = precision == GRILLY_PREC_BF16;
  GemmLnArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.bias = bias; a.residual = residual; a.ld_res = N; a.gamma = gamma; a.beta = beta; a.eps = eps;
  a.out = y; a.ld_out = N;
  a.out_bf16 = (flags & GRILLY_FLAG_OUT_BF16) ? 1 : 0;
  a.round_tf32 = (flags & GRILLY_FLAG_ROUND_TF32) ? 1 : 0;
  if (ctx->tune.fused_ln && M > 0 && K > 0 && gemm_ln_supported(bf16, N, K, a)) return launch_gemm_ln(ctx, bf16, x, w, a);
  // other widths: the GEMM writes the fp32 sum (bias and residual in its epilogue), the row kernel normalises it
  if (!scratch) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "linear_layernorm: this shape needs the M x N fp32 scratch");
  GemmArgs g{};
  g.M = M; g.N = N; g.K = K;
  g.bias = bias; g.residual = static_cast<const float*>(residual); g.ld_res = N; g.residual_bf16 = (residual && bf16) ? 1 : 0;
  g.out = scratch; g.ld_out = N;
  if ((rc = launch_gemm(ctx, bf16, false, x, w, g, 0))) return rc;
  NormArgs n{};
  n.x = scratch; n.gamma = gamma; n.beta = beta; n.y = y; n.rows = M; n.F = N; n.eps = eps; n.mode = NORM_LAYER;
  n.out_bf16 = a.out_bf16; n.round_tf32 = a.round_tf32;
  return launch_norm(ctx, n);
}

int grilly_gemm_mnk(grilly_ctx* ctx, const void* a_dev, const void* b_dev, void* c_dev, int M, int K, int N, int precision,
                    int flags) {
  CTX_GUARD(ctx);
  int rc = check_prec(ctx, precision, true);
  if (rc) return rc;
  if (!a_dev || !b_dev || !c_dev) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "gemm_mnk: null operand");
  GemmArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.out = c_dev; a.ld_out = N;
  a.out_bf16 = (flags & GRILLY_FLAG_OUT_BF16) ? 1 : 0;
  a.round_tf32 = (flags & GRILLY_FLAG_ROUND_TF32) ? 1 : 0;
  if (precision == GRILLY_PREC_TF32X3) {
    if (M <= 0 || N <= 0 || K <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "gemm: M, N, K must be positive");
    if (N % 4) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "gemm_mnk: N * element size must be a multiple of 16 bytes (pad N)");
    return gemm_mnk_tf32x3(ctx, static_cast<const float*>(a_dev), static_cast<const float*>(b_dev), a);
  }
  return launch_gemm(ctx, precision == GRILLY_PREC_BF16, true, a_dev, b_dev, a, 0);
}

int grilly_gemm_mnk_multi(grilly_ctx* ctx, const void* a_dev, const void* b_dev, void* const* c_ptrs, int num_outputs, int M,
                          int K, int N, long long ld_c, int precision) {
  CTX_GUARD(ctx);
  int rc = check_prec(ctx, precision);
  if (rc) return rc;
  if (!a_dev || !b_dev || !c_ptrs || num_outputs < 1 || num_outputs > 8)
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "gemm_mnk_multi: null operand or destination count outside [1, 8]");
  for (int i = 0; i < num_outputs; ++i)
    if (!c_ptrs[i]) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "gemm_mnk_multi: null destination");
  if (ld_c < N) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "gemm_mnk_multi: ld_c is smaller than N");
  GemmArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.out = c_ptrs[0]; a.ld_out = ld_c;
  return launch_gemm_multi(ctx, precision == GRILLY_PREC_BF16, a_dev, b_dev, a, c_ptrs + 1, num_outputs - 1);
}

int grilly_flash_attention(grilly_ctx* ctx, const void* q, const void* k, const void* v, void* out, int B, int S, int H,
                           int D, long long ld_qkv, long long ld_out, const int* cu_seqlens, long long total_rows,
                           const float* key_mask, float scale, int causal, int rope_style, float rope_base,
                           float rope_scaling, int precision, int flags) {
  CTX_GUARD(ctx);
  int rc = check_prec(ctx, precision);
  if (rc) return rc;
  if (!q || !k || !v || !out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "flash_attention: null operand");
  if (cu_seqlens && key_mask) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "flash_attention: key_mask applies to the padded layout only");
  if (!cu_seqlens) total_rows = static_cast<long long>(B) * S;
  if (total_rows <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "flash_attention: no rows");
  AttnArgs a{};
  a.B = B; a.S = S; a.H = H; a.D = D;
  a.cu_seqlens = cu_seqlens; a.key_mask = key_mask;
  a.scale = scale; a.causal = causal ? 1 : 0;
  a.out = out; a.ld_out = ld_out;
  a.out_bf16 = (flags & GRILLY_FLAG_OUT_BF16) ? 1 : 0;
  a.round_tf32 = (flags & GRILLY_FLAG_ROUND_TF32) ? 1 : 0;
  a.rope_style = rope_style;
  if (rope_style != GRILLY_ROPE_NONE) {
    if (rope_style != GRILLY_ROPE_INTERLEAVED && rope_style != GRILLY_ROPE_ROTATE_HALF)
      return set_error(ctx, GRILLY_ERR_INVALID_ARG, "flash_attention: unknown rope style");
    if (rope_scaling == 0.f) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "flash_attention: rope scaling must be non-zero");
    rc = get_rope_table(ctx, S, D, rope_base, rope_scaling, &a.rope_cos, &a.rope_sin);
    if (rc) return rc;
  }
  const bool bf16 = precision == GRILLY_PREC_BF16;
  if (rope_style != GRILLY_ROPE_NONE && S > 2 * 128) {
    // Long sequences: every 128-query CTA would rotate all of its key tiles again. Rotate K once into pool scratch
    // instead; Q is still rotated in shared memory by the CTA that loads it (once per tile either way).
    const size_t bytes = static_cast<size_t>(total_rows) * H * D * (bf16 ? 2 : 4);
    void* kr = nullptr;
    cudaError_t e2 = cudaMallocAsync(&kr, bytes, ctx->stream);
    if (e2 != cudaSuccess) { cudaGetLastError(); return set_error(ctx, GRILLY_ERR_OOM, "flash_attention: no memory for the rotated K copy"); }
    rc = launch_rope_rows(ctx, bf16, k, kr, total_rows, ld_qkv, H, D, S, cu_seqlens, B, a.rope_cos, a.rope_sin, rope_style);
    a.rope_k_done = 1;
    if (!rc) rc = launch_attention(ctx, bf16, q, kr, v, ld_qkv, static_cast<long long>(H) * D, ld_qkv, total_rows, a);
    cudaFreeAsync(kr, ctx->stream);
    return rc;
  }
  return launch_attention(ctx, bf16, q, k, v, ld_qkv, ld_qkv, ld_qkv, total_rows, a);
}

int grilly_attention_scores(grilly_ctx* ctx, const float* q, const float* k, float* scores, int B, int S, int H, int D, float scale) {
  CTX_GUARD(ctx);
  if (!q || !k || !scores) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention_scores: null operand");
  return launch_attn_scores(ctx, q, k, scores, B, S, H, D, scale);
}

int grilly_attention_mask(grilly_ctx* ctx, float* scores, const float* mask, int B, int H, int S, int use_causal, float mask_value) {
  CTX_GUARD(ctx);
  if (!scores) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention_mask: null operand");
  return launch_attn_mask(ctx, scores, mask, B, H, S, use_causal ? 1 : 0, mask_value);
}

int grilly_attention_output(grilly_ctx* ctx, const float* weights, const float* v, float* out, int B, int S, int H, int D) {
  return grilly_attention_output_ex(ctx, weights, v, out, B, S, S, H, D, 0);
}

int grilly_attention_output_ex(grilly_ctx* ctx, const float* weights, const float* v, float* out, int B, int Sq, int Sk, int H, int D,
                               int causal) {
  CTX_GUARD(ctx);
  if (!weights || !v || !out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention_output: null operand");
  return launch_attn_output(ctx, weights, v, out, B, Sq, Sk, H, D, causal ? 1 : 0);
}

int grilly_apply_rope(grilly_ctx* ctx, const float* x, float* y, const int* position_ids, int B, int S, int H, int D,
                      int max_pos, float base, float scaling, int rope_style) {
  CTX_GUARD(ctx);
  if (!x || !y) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "apply_rope: null operand");
  if (D % 2) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "apply_rope: head_dim must be even");
  if (rope_style != GRILLY_ROPE_INTERLEAVED && rope_style != GRILLY_ROPE_ROTATE_HALF)
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "apply_rope: unknown rope style");
  const float *c, *s;
  int rc = get_rope_table(ctx, max_pos > S ? max_pos : S, D, base, scaling, &c, &s);
  if (rc) return rc;
  return launch_rope_apply(ctx, x, y, c, s, position_ids, B, S, H, D, rope_style);
}

int grilly_layernorm(grilly_ctx* ctx, const float* x, const float* residual, const float* gamma, const float* beta, void* y,
                     long long rows, int F, float eps, int norm_mode, int flags) {
  CTX_GUARD(ctx);
  if (!x || !y) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm: null operand");
  if (rows > 0x7fffffffLL) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "layernorm: too many rows");
  NormArgs n{};
  n.x = x; n.residual = residual; n.gamma = gamma; n.beta = beta; n.y = y;
  n.rows = static_cast<int>(rows); n.F = F; n.eps = eps; n.mode = norm_mode;
  n.out_bf16 = (flags & GRILLY_FLAG_OUT_BF16) ? 1 : 0;
  n.round_tf32 = (flags & GRILLY_FLAG_ROUND_TF32) ? 1 : 0;
  return launch_norm(ctx, n);
}

int grilly_softmax(grilly_ctx* ctx, const float* x, float* y, long long rows, int cols) {
  CTX_GUARD(ctx);
  if (!x || !y) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "softmax: null operand");
  return launch_softmax(ctx, x, y, rows, cols);
}

int grilly_eltwise(grilly_ctx* ctx, int op, const float* a, const float* b, float* y, long long n, int half) {
  CTX_GUARD(ctx);
  if (!a || !y) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "eltwise: null operand");
  if (op < GRILLY_ELT_GELU || op > GRILLY_ELT_SWIGLU) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "eltwise: unknown op");
  return launch_eltwise(ctx, op, a, b, y, n, half);
}

int grilly_activation_params(grilly_ctx* ctx, int op, const float* x, float* y, long long n, float p0, float p1) {
  CTX_GUARD(ctx);
  if (!x || !y) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "activation: null operand");
  if (op != GRILLY_ELT_GCU && op != GRILLY_ELT_ROSWISH) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "activation: op must be GRILLY_ELT_GCU or GRILLY_ELT_ROSWISH");
  return launch_act_params(ctx, op, x, y, n, p0, p1);
}

int grilly_embedding_lookup(grilly_ctx* ctx, const int* ids, const float* table, float* out, long long n_tokens, int vocab,
                            int F) {
  CTX_GUARD(ctx);
  if (!ids || !table || !out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "embedding_lookup: null operand");
  return launch_gather(ctx, ids, table, out, n_tokens, vocab, F);
}

int grilly_embed_layernorm(grilly_ctx* ctx, const int* ids, const int* cu_seqlens, const float* word, const float* pos,
                           const float* type0, const float* gamma, const float* beta, float* out, int B, int S, int F,
                           int vocab, int max_pos, float eps, int flags) {
  CTX_GUARD(ctx);
  if (!ids || !word || !out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "embed_layernorm: null operand");
  EmbedArgs e{};
  e.ids = ids; e.cu_seqlens = cu_seqlens; e.word = word; e.pos = pos; e.type0 = type0; e.gamma = gamma; e.beta = beta;
  e.out = out; e.B = B; e.S = S; e.F = F; e.vocab = vocab; e.max_pos = max_pos; e.eps = eps;
  e.round_tf32 = (flags & GRILLY_FLAG_ROUND_TF32) ? 1 : 0;
  return launch_embed(ctx, e);
}

int grilly_mean_pool(grilly_ctx* ctx, const float* x, const float* mask, const int* cu_seqlens, float* out, int B, int S,
                     int F, int normalize) {
  CTX_GUARD(ctx);
  if (!x || !out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "mean_pool: null operand");
  if (mask && cu_seqlens) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "mean_pool: give a mask (padded rows) or cu_seqlens (packed rows), not both");
  PoolArgs p{};
  p.x = x; p.mask = mask; p.cu_seqlens = cu_seqlens; p.out = out; p.B = B; p.S = S; p.F = F; p.normalize = normalize ? 1 : 0;
  return launch_pool(ctx, p);
}

}  // extern "C"
