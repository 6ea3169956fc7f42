// Host launchers for the HBM-bound row kernels.
#include "rowops.cuh"
#include "internal.h"

namespace gb {

static inline int grid_for(long long work_items, int per_block, int num_sms, int blocks_per_sm = 8) {
  long long g = (work_items + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(num_sms) * blocks_per_sm;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

int launch_norm(grilly_ctx* ctx, const NormArgs& a) {
  if (a.rows <= 0 || a.F <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm: rows and features must be positive");
  const int grid = grid_for(a.rows, 8, ctx->num_sms);
  const bool aligned = !a.x_bf16 && (a.F % 4 == 0) && !(reinterpret_cast<uintptr_t>(a.x) & 15) && !(reinterpret_cast<uintptr_t>(a.y) & 15) &&
                       !(reinterpret_cast<uintptr_t>(a.residual) & 15) && !(reinterpret_cast<uintptr_t>(a.gamma) & 15) &&
                       !(reinterpret_cast<uintptr_t>(a.beta) & 15);
  const double in_elt = a.x_bf16 ? 2.0 : 4.0;
  const double nbytes = static_cast<double>(a.rows) * a.F * (in_elt + (a.residual ? in_elt : 0.0) + (a.y ? (a.out_bf16 ? 2.0 : 4.0) : 0.0));
  const int pi = prof_begin(ctx, PROF_NORM, 8.0 * a.rows * a.F, nbytes);
  if (aligned && a.F <= 128 * 3) norm_rows_kernel<3><<<grid, 256, 0, ctx->stream>>>(a);
  else if (aligned && a.F <= 128 * 8) norm_rows_kernel<8><<<grid, 256, 0, ctx->stream>>>(a);
  else if (aligned && a.F <= 128 * 16) norm_rows_kernel<16><<<grid, 256, 0, ctx->stream>>>(a);
  else norm_rows_generic_kernel<<<grid, 256, 0, ctx->stream>>>(a);
  prof_end(ctx, pi);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int launch_softmax(grilly_ctx* ctx, const float* x, float* y, long long rows, int cols) {
  if (rows <= 0 || cols <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "softmax: rows and cols must be positive");
  softmax_rows_kernel<<<grid_for(rows, 8, ctx->num_sms), 256, 0, ctx->stream>>>(x, y, rows, cols);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int launch_eltwise(grilly_ctx* ctx, int op, const float* a, const float* b, float* y, long long n, int half) {
  if (n <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "eltwise: n must be positive");
  if (op == ELT_ADD && !b) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "eltwise add: second operand missing");
  if (op == ELT_SWIGLU && half <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "swiglu: half width must be positive");
  eltwise_kernel<<<grid_for(n, 256 * 4, ctx->num_sms, 16), 256, 0, ctx->stream>>>(op, a, b, y, n, half > 0 ? half : 1);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int launch_act_params(grilly_ctx* ctx, int op, const float* a, float* y, long long n, float p0, float p1) {
  if (n <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "activation: n must be positive");
  act_params_kernel<<<grid_for(n, 256 * 4, ctx->num_sms, 16), 256, 0, ctx->stream>>>(op, a, y, n, p0, p1);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int launch_round_tf32(grilly_ctx* ctx, const float* x, float* y, long long n) {
  if (n <= 0) return GRILLY_OK;
  round_tf32_kernel<<<grid_for(n, 256 * 4, ctx->num_sms, 16), 256, 0, ctx->stream>>>(x, y, n);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}
int launch_f32_to_bf16(grilly_ctx* ctx, const float* x, void* y, long long n) {
  if (n <= 0) return GRILLY_OK;
  f32_to_bf16_kernel<<<grid_for(n, 256 * 4, ctx->num_sms, 16), 256, 0, ctx->stream>>>(x, reinterpret_cast<__nv_bfloat16*>(y), n);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}
int launch_bf16_to_f32(grilly_ctx* ctx, const void* x, float* y, long long n) {
  if (n <= 0) return GRILLY_OK;
  bf16_to_f32_kernel<<<grid_for(n, 256 * 4, ctx->num_sms, 16), 256, 0, ctx->stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), y, n);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int launch_gather(grilly_ctx* ctx, const int* ids, const float* table, float* out, long long n, int vocab, int F) {
  if (n <= 0 || F <= 0 || vocab <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "embedding_lookup: sizes must be positive");
  gather_rows_kernel<<<grid_for(n, 8, ctx->num_sms), 256, 0, ctx->stream>>>(ids, table, out, n, vocab, F);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int launch_embed(grilly_ctx* ctx, const EmbedArgs& a) {
  if (a.B <= 0 || a.S <= 0 || a.F <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "embed: sizes must be positive");
  if (a.F % 4 != 0 || a.F > 128 * 8) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "embed: hidden size must be a multiple of 4 and at most 1024");
  const int grid = grid_for(static_cast<long long>(a.B) * a.S, 8, ctx->num_sms);
  // ids of every position, one table row read and one row written per valid token (the position table stays in L2)
  const double tokens = a.rows_hint > 0 ? static_cast<double>(a.rows_hint) : static_cast<double>(a.B) * a.S;
  const int pi = prof_begin(ctx, PROF_EMBED, 0.0, static_cast<double>(a.B) * a.S * 4.0 + tokens * 8.0 * a.F);
  if (a.F <= 128 * 3) embed_ln_kernel<3><<<grid, 256, 0, ctx->stream>>>(a);
  else embed_ln_kernel<8><<<grid, 256, 0, ctx->stream>>>(a);
  prof_end(ctx, pi);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int launch_pool(grilly_ctx* ctx, const PoolArgs& a) {
  if (a.B <= 0 || a.S <= 0 || a.F <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "mean_pool: sizes must be positive");
  const size_t smem = (static_cast<size_t>(a.F) + 8) * sizeof(float);
  if (smem > 48 * 1024) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "mean_pool: feature size too large");
  const double tokens = a.rows_hint > 0 ? static_cast<double>(a.rows_hint) : static_cast<double>(a.B) * a.S;
  const int pi = prof_begin(ctx, PROF_POOL, 0.0, tokens * a.F * 4.0 + static_cast<double>(a.B) * a.F * 4.0);
  const bool vec = a.F % 4 == 0 && ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.out)) & 15) == 0;
  if (vec && a.F <= 128 * 3) pool_normalize_vec_kernel<3><<<a.B, 128, 0, ctx->stream>>>(a);
  else if (vec && a.F <= 128 * 8) pool_normalize_vec_kernel<8><<<a.B, 128, 0, ctx->stream>>>(a);
  else pool_normalize_kernel<<<a.B, 128, smem, ctx->stream>>>(a);
  prof_end(ctx, pi);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

// Wf = W diag(gamma) rounded to the GEMM's operand precision, col_sum = row sums of the rounded Wf,
// bias_f = bias + W beta. One warp per output feature.
__global__ void __launch_bounds__(256) fold_ln_kernel(const float* __restrict__ w, const float* __restrict__ gamma,
                                                      const float* __restrict__ beta, const float* __restrict__ bias,
                                                      void* __restrict__ wf, float* __restrict__ col_sum,
                                                      float* __restrict__ bias_f, int N, int K, int bf16) {
  const int lane = threadIdx.x & 31;
  const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (c >= N) return;
  float cs = 0.f, bs = 0.f;
  for (int k = lane; k < K; k += 32) {
    const float wv = w[static_cast<long long>(c) * K + k];
    float f = wv * (gamma ? gamma[k] : 1.f);
    if (bf16) {
      const __nv_bfloat16 h = __float2bfloat16(f);
      reinterpret_cast<__nv_bfloat16*>(wf)[static_cast<long long>(c) * K + k] = h;
      f = __bfloat162float(h);
    } else {
      f = round_to_tf32(f);
      reinterpret_cast<float*>(wf)[static_cast<long long>(c) * K + k] = f;
    }
    cs += f;
    if (beta) bs += wv * beta[k];
  }
  cs = warp_sum(cs);
  bs = warp_sum(bs);
  if (lane == 0) {
    col_sum[c] = cs;
    bias_f[c] = (bias ? bias[c] : 0.f) + bs;
  }
}

int launch_fold_ln(grilly_ctx* ctx, const float* w, const float* gamma, const float* beta, const float* bias, void* wf,
                   float* col_sum, float* bias_f, int N, int K, bool bf16) {
  if (N <= 0 || K <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "fold_layernorm_weights: sizes must be positive");
  fold_ln_kernel<<<(N + 7) / 8, 256, 0, ctx->stream>>>(w, gamma, beta, bias, wf, col_sum, bias_f, N, K, bf16 ? 1 : 0);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int get_rope_table(grilly_ctx* ctx, int S, int D, float base, float scaling, const float** cos_t, const float** sin_t) {
  for (auto& t : ctx->rope_tables) {
    if (t.S >= S && t.D == D && t.base == base && t.scaling == scaling) {
      *cos_t = t.cos_t;
      *sin_t = t.sin_t;
      return GRILLY_OK;
    }
  }
  grilly_ctx::RopeTable t{S, D, base, scaling, nullptr, nullptr};
  const size_t bytes = static_cast<size_t>(S) * (D / 2) * sizeof(float);
  GB_CUDA_CHECK(ctx, cudaMalloc(&t.cos_t, bytes));
  GB_CUDA_CHECK(ctx, cudaMalloc(&t.sin_t, bytes));
  const long long n = static_cast<long long>(S) * (D / 2);
  rope_table_kernel<<<grid_for(n, 256, ctx->num_sms), 256, 0, ctx->stream>>>(t.cos_t, t.sin_t, S, D, base, scaling);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  ctx->rope_tables.push_back(t);
  *cos_t = t.cos_t;
  *sin_t = t.sin_t;
  return GRILLY_OK;
}

int launch_attn_scores(grilly_ctx* ctx, const float* q, const float* k, float* scores, int B, int S, int H, int D, float scale) {
  if (B <= 0 || S <= 0 || H <= 0 || D <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention_scores: sizes must be positive");
  attn_scores_kernel<<<grid_for(static_cast<long long>(B) * H * S, 8, ctx->num_sms), 256, 0, ctx->stream>>>(q, k, scores, B, S, H, D, scale);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}
int launch_attn_mask(grilly_ctx* ctx, float* scores, const float* mask, int B, int H, int S, int use_causal, float mask_value) {
  const long long n = static_cast<long long>(B) * H * S * S;
  if (n <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention_mask: sizes must be positive");
  if (!use_causal && !mask) return GRILLY_OK;  // nothing to apply (backend/attention.py:157-160)
  attn_mask_kernel<<<grid_for(n, 256 * 4, ctx->num_sms, 16), 256, 0, ctx->stream>>>(scores, mask, n, H, S, use_causal, mask_value);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}
int launch_attn_output(grilly_ctx* ctx, const float* w, const float* v, float* out, int B, int Sq, int Sk, int H, int D, int causal) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || H <= 0 || D <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention_output: sizes must be positive");
  attn_output_kernel<<<grid_for(static_cast<long long>(B) * H * Sq, 8, ctx->num_sms), 256, 0, ctx->stream>>>(w, v, out, B, Sq, Sk, H, D, causal);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int launch_rope_rows(grilly_ctx* ctx, bool bf16, const void* src, void* dst, long long rows, long long pitch, int H, int D,
                     int S, const int* cu_seqlens, int B, const float* cos_t, const float* sin_t, int style) {
  const int elt = bf16 ? 2 : 4;
  const int pieces = D / (16 / elt);
  const long long total = rows * H * (style == 1 ? pieces : pieces / 2);
  if (total <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "rope: sizes must be positive");
  const int grid = grid_for(total, 256, ctx->num_sms, 16);
  const int pi = prof_begin(ctx, PROF_OTHER, 0.0, 2.0 * rows * H * D * elt);
  if (bf16) rope_rows_kernel<true><<<grid, 256, 0, ctx->stream>>>(src, dst, rows, pitch, H, D, S, cu_seqlens, B, cos_t, sin_t, style);
  else rope_rows_kernel<false><<<grid, 256, 0, ctx->stream>>>(src, dst, rows, pitch, H, D, S, cu_seqlens, B, cos_t, sin_t, style);
  prof_end(ctx, pi);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int launch_rope_apply(grilly_ctx* ctx, const float* x, float* y, const float* cos_t, const float* sin_t,
                      const int* position_ids, int B, int S, int H, int D, int style) {
  const long long n_pairs = static_cast<long long>(B) * S * H * (D / 2);
  if (n_pairs <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "apply_rope: sizes must be positive");
  rope_apply_kernel<<<grid_for(n_pairs, 256 * 2, ctx->num_sms, 16), 256, 0, ctx->stream>>>(x, y, cos_t, sin_t, position_ids,
                                                                                         n_pairs, S, H, D, style);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

}  // namespace gb
