// Device-resident post-LN BERT/MiniLM sentence encoder built from the hot-path
// kernels. Weights are uploaded once; a forward uploads token ids, runs on
// packed (padding-free) token rows and downloads one pooled vector per sentence.
//
// Per layer (T = packed token rows, F = hidden):
//   qkv  = x Wqkv^T + bqkv                      tcgen05 GEMM            [T, 3F]
//   attn = softmax(q k^T / sqrt(d)) v           tcgen05 flash-attention [T, F]
//   x2   = LayerNorm(attn Wo^T + bo + x)        GEMM with residual + LayerNorm epilogue [T, F]
//   h    = gelu(x2 W1^T + b1)                   GEMM, GELU epilogue     [T, ffn]
//   x    = LayerNorm(h W2^T + b2 + x2)          GEMM with residual + LayerNorm epilogue
// (hidden sizes other than 128/256/384/512 run each of the two fused steps as GEMM + row kernel)
// Sentences are processed in chunks of at most `chunk_tokens` rows through all
// layers, reusing one set of activation buffers, so a chunk's activations stay
// in the 126 MB L2 between producer and consumer kernels.
#include "internal.h"
#include <cstdlib>
#include "args.h"
#include <algorithm>
#include <cmath>

using namespace gb;

struct EncLayer {
  float *wqkv = nullptr, *bqkv = nullptr, *wo = nullptr, *bo = nullptr, *ln1_g = nullptr, *ln1_b = nullptr;
  float *w1 = nullptr, *b1 = nullptr, *w2 = nullptr, *b2 = nullptr, *ln2_g = nullptr, *ln2_b = nullptr;
  float *wgu = nullptr, *bgu = nullptr;   // pre-norm GeGLU layers: (2 ffn, hidden) rows (up_j, gate_j) and the bias alike
  // bf16 mode: the GEMM weights as bf16 (the fp32 slots above are then only the upload staging)
  void *wqkv_h = nullptr, *wo_h = nullptr, *w1_h = nullptr, *w2_h = nullptr;
};

struct grilly_encoder {
  grilly_ctx* ctx = nullptr;
  grilly_encoder_config cfg{};
  float *word = nullptr, *pos = nullptr, *type = nullptr, *emb_g = nullptr, *emb_b = nullptr;
  float *final_g = nullptr, *final_b = nullptr;   // pre-norm models: the LayerNorm after the last layer
  std::vector<EncLayer> layers;
  // activation workspace for one chunk
  long long cap_rows = 0;
  // tf32 mode: all fp32. bf16 mode: x, x2, attn, qkv, h are bf16 (MMA operands and the residual they carry), the
  // pre-LayerNorm sums t and the final hidden states xf stay fp32.
  void *x = nullptr, *x2 = nullptr, *attn = nullptr, *qkv = nullptr, *h = nullptr;
  float *t = nullptr, *xf = nullptr;
  bool bf16 = false;
  // per-call buffers
  int cap_B = 0, cap_S = 0;
  int* ids_dev = nullptr;      // [B][S]
  int* cu_dev = nullptr;       // chunk-relative row offsets, one [Bc+1] segment per chunk
  float* out_dev = nullptr;    // [B][F]
  int* ids_pin = nullptr;      // pinned staging
  int* cu_pin = nullptr;
  float* out_pin = nullptr;
  float* mask_dev = nullptr;   // padded-layout fallback for masks that are not prefixes
  // optional copy of the final hidden states (packed rows) for parity checks
  bool keep_hidden = false;
  float* hidden_all = nullptr;
  long long hidden_cap = 0, last_rows = 0;
  std::vector<void*> owned;
};

static int enc_alloc(grilly_encoder* e, size_t bytes, void** p) {
  cudaError_t err = cudaMalloc(p, bytes ? bytes : 16);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return set_error(e->ctx, err == cudaErrorMemoryAllocation ? GRILLY_ERR_OOM : GRILLY_ERR_CUDA,
                     std::string("encoder allocation: ") + cudaGetErrorString(err));
  }
  e->owned.push_back(*p);
  return GRILLY_OK;
}
static void enc_release(grilly_encoder* e, void* p) {
  if (!p) return;
  cudaFree(p);
  e->owned.erase(std::remove(e->owned.begin(), e->owned.end(), p), e->owned.end());
}

static int ensure_workspace(grilly_encoder* e, long long rows) {
  if (rows <= e->cap_rows) return GRILLY_OK;
  const int F = e->cfg.hidden, ffn = e->cfg.ffn;
  const size_t act = e->bf16 ? 2 : 4;  // bytes per activation element that feeds an MMA
  void** bufs[7] = {&e->x, &e->x2, reinterpret_cast<void**>(&e->t), &e->attn, &e->qkv, &e->h, reinterpret_cast<void**>(&e->xf)};
  const size_t row_bytes[7] = {F * act, F * act, F * sizeof(float), F * act, 3 * F * act, ffn * act, e->bf16 ? F * sizeof(float) : 0};
  for (int i = 0; i < 7; ++i) {
    enc_release(e, *bufs[i]);
    *bufs[i] = nullptr;
    if (row_bytes[i] == 0) continue;
    int rc = enc_alloc(e, static_cast<size_t>(rows) * row_bytes[i], bufs[i]);
    if (rc) { e->cap_rows = 0; return rc; }
  }
  e->cap_rows = rows;
  return GRILLY_OK;
}

static int ensure_io(grilly_encoder* e, int B, int S) {
  if (B <= e->cap_B && S <= e->cap_S) return GRILLY_OK;
  const int nB = std::max(B, e->cap_B), nS = std::max(S, e->cap_S);
  enc_release(e, e->ids_dev); enc_release(e, e->cu_dev); enc_release(e, e->out_dev); enc_release(e, e->mask_dev);
  e->ids_dev = nullptr; e->cu_dev = nullptr; e->out_dev = nullptr; e->mask_dev = nullptr;
  if (e->ids_pin) cudaFreeHost(e->ids_pin);
  if (e->cu_pin) cudaFreeHost(e->cu_pin);
  if (e->out_pin) cudaFreeHost(e->out_pin);
  e->ids_pin = nullptr; e->cu_pin = nullptr; e->out_pin = nullptr;
  e->cap_B = e->cap_S = 0;
  int rc;
  if ((rc = enc_alloc(e, static_cast<size_t>(nB) * nS * sizeof(int), reinterpret_cast<void**>(&e->ids_dev)))) return rc;
  if ((rc = enc_alloc(e, static_cast<size_t>(2 * nB + 2) * sizeof(int), reinterpret_cast<void**>(&e->cu_dev)))) return rc;
  if ((rc = enc_alloc(e, static_cast<size_t>(nB) * e->cfg.hidden * sizeof(float), reinterpret_cast<void**>(&e->out_dev)))) return rc;
  if ((rc = enc_alloc(e, static_cast<size_t>(nB) * nS * sizeof(float), reinterpret_cast<void**>(&e->mask_dev)))) return rc;
  GB_CUDA_CHECK(e->ctx, cudaMallocHost(&e->ids_pin, static_cast<size_t>(nB) * nS * sizeof(int)));
  GB_CUDA_CHECK(e->ctx, cudaMallocHost(&e->cu_pin, static_cast<size_t>(2 * nB + 2) * sizeof(int)));
  GB_CUDA_CHECK(e->ctx, cudaMallocHost(&e->out_pin, static_cast<size_t>(nB) * e->cfg.hidden * sizeof(float)));
  e->cap_B = nB; e->cap_S = nS;
  return GRILLY_OK;
}

static int enc_linear(grilly_encoder* e, const void* x, const void* w, const float* bias, const void* residual, void* y,
                      int M, int N, int K, int act, bool out_fp32, bool glu_pairs = false) {
  GemmArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.bias = bias; a.residual = reinterpret_cast<const float*>(residual); a.ld_res = N;
  a.residual_bf16 = (residual && e->bf16) ? 1 : 0;
  a.out = y; a.ld_out = glu_pairs ? N / 2 : N;
  a.swiglu_pairs = glu_pairs ? 1 : 0;   // weight rows come as (multiplier_j, activated_j) pairs: out[:, j] = first * act(second)
  a.act = act;
  a.out_bf16 = (e->bf16 && !out_fp32) ? 1 : 0;
  // tf32 mode: outputs that feed an MMA directly are rounded to tf32; pre-LayerNorm sums stay full fp32
  a.round_tf32 = (!e->bf16 && !out_fp32) ? 1 : 0;
  return launch_gemm(e->ctx, e->bf16, false, x, w, a, 0);
}

// y = LayerNorm(x W^T + bias + residual): one kernel where the width allows it, else GEMM into t + row kernel
static int enc_linear_norm(grilly_encoder* e, const void* x, const void* w, const float* bias, const void* residual,
                           const float* g, const float* b, void* y, int M, int N, int K, bool out_fp32);

static int enc_norm(grilly_encoder* e, const float* x, const float* g, const float* b, void* y, int rows, bool out_fp32,
                    float eps = -1.f) {
  NormArgs n{};
  n.x = x; n.gamma = g; n.beta = b; n.y = y; n.rows = rows; n.F = e->cfg.hidden; n.eps = eps >= 0.f ? eps : e->cfg.layer_ln_eps;
  n.mode = NORM_LAYER;
  n.out_bf16 = (e->bf16 && !out_fp32) ? 1 : 0;
  n.round_tf32 = (e->bf16 || out_fp32) ? 0 : 1;
  n.reverse = 1;   // the GEMM before it wrote the last rows last: start where L2 still holds them (about 4 % of this kernel)
  return launch_norm(e->ctx, n);
}

static int enc_linear_norm(grilly_encoder* e, const void* x, const void* w, const float* bias, const void* residual,
                           const float* g, const float* b, void* y, int M, int N, int K, bool out_fp32) {
  GemmLnArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.bias = bias; a.residual = residual; a.ld_res = N; a.gamma = g; a.beta = b; a.eps = e->cfg.layer_ln_eps;
  a.out = y; a.ld_out = N;
  a.out_bf16 = (e->bf16 && !out_fp32) ? 1 : 0;
  a.round_tf32 = e->bf16 ? 0 : 1;
  if (e->ctx->tune.fused_ln && gemm_ln_supported(e->bf16, N, K, a)) return launch_gemm_ln(e->ctx, e->bf16, x, w, a);
  int rc = enc_linear(e, x, w, bias, residual, e->t, M, N, K, ACT_NONE, true);
  if (rc) return rc;
  return enc_norm(e, e->t, g, b, y, M, out_fp32);
}

// Runs one chunk: sequences [b0, b1) whose packed rows are [0, rows) of the workspace.
static int run_chunk(grilly_encoder* e, const int* ids_dev, const int* cu_chunk_dev, int b0, int b1, int S, int rows,
                     int max_len, float* out_dev, long long hidden_row0, double sum_len2,
                     const float* key_mask_dev = nullptr) {
  grilly_ctx* ctx = e->ctx;
  const auto& c = e->cfg;
  const int F = c.hidden, H = c.num_heads, D = F / H, Bc = b1 - b0;
  int rc;
  const size_t act = e->bf16 ? 2 : 4;
  const bool prenorm = c.arch == GRILLY_ARCH_MODERNBERT;
  EmbedArgs em{};
  em.ids = ids_dev + static_cast<long long>(b0) * S; em.cu_seqlens = cu_chunk_dev; em.word = e->word;
  em.pos = prenorm ? nullptr : e->pos;   // pre-norm models carry positions as RoPE inside attention (:1147-1155)
  em.type0 = (c.has_token_type && !prenorm) ? e->type : nullptr; em.gamma = e->emb_g; em.beta = e->emb_b; em.out = reinterpret_cast<float*>(e->x);
  em.B = Bc; em.S = S; em.F = F; em.vocab = c.vocab; em.max_pos = c.max_pos; em.eps = c.embed_ln_eps;
  em.round_tf32 = e->bf16 ? 0 : 1; em.out_bf16 = e->bf16 ? 1 : 0; em.rows_hint = rows;
  if ((rc = launch_embed(ctx, em))) return rc;
  float* final_hidden = e->bf16 ? e->xf : reinterpret_cast<float*>(e->x);
  if (prenorm) {
    // ---- ModernBERT branch of _forward_layer (utils/vulkan_sentence_transformer.py:799-970), fp32 storage / tf32 MMAs.
    // The residual stream x is kept tf32-rounded: it is the QKV GEMM's operand as it stands (the attention norm is the
    // identity), so rounding it where it is produced keeps the MMA from truncating it.
    const float* cos_t = nullptr; const float* sin_t = nullptr;
    if ((rc = get_rope_table(ctx, max_len, D, c.rope_base, 1.0f, &cos_t, &sin_t))) return rc;
    for (int l = 0; l < c.num_layers; ++l) {
      const EncLayer& L = e->layers[l];
      if ((rc = enc_linear(e, e->x, L.wqkv, L.bqkv, nullptr, e->qkv, rows, 3 * F, F, ACT_NONE, false))) return rc;
      AttnArgs at{};
      at.B = Bc; at.S = max_len; at.H = H; at.D = D; at.cu_seqlens = cu_chunk_dev; at.scale = 1.0f / sqrtf(static_cast<float>(D));
      at.out = e->attn; at.ld_out = F; at.round_tf32 = 1; at.key_mask = key_mask_dev;
      at.rope_style = ROPE_ROTATE_HALF; at.rope_cos = cos_t; at.rope_sin = sin_t;
      ctx->attn_flops_hint = 4.0 * H * D * sum_len2;
      const char* qkv = reinterpret_cast<const char*>(e->qkv);
      if ((rc = launch_attention(ctx, false, qkv, qkv + F * act, qkv + 2 * F * act, 3LL * F, 3LL * F, 3LL * F, rows, at))) return rc;
      // x2 = x + attn Wo^T + bo (no norm after it); the MLP's LayerNorm reads it, the MLP's residual is it
      if ((rc = enc_linear(e, e->attn, L.wo, L.bo, e->x, e->x2, rows, F, F, ACT_NONE, false))) return rc;
      if ((rc = enc_norm(e, reinterpret_cast<const float*>(e->x2), L.ln2_g, L.ln2_b, e->attn, rows, false))) return rc;
      // GeGLU: h[:, j] = (n Wup_j + bup_j) * gelu(n Wgate_j + bgate_j), one GEMM over the interleaved rows
      if ((rc = enc_linear(e, e->attn, L.wgu, L.bgu, nullptr, e->h, rows, 2 * c.ffn, F, ACT_GELU_TANH, false, true))) return rc;
      if ((rc = enc_linear(e, e->h, L.w2, L.b2, e->x2, e->x, rows, F, c.ffn, ACT_NONE, false))) return rc;
    }
    // final LayerNorm (:1166-1177), then CLS pooling (:1181-1183) and L2 normalisation
    if ((rc = enc_norm(e, reinterpret_cast<const float*>(e->x), e->final_g, e->final_b, e->t, rows, true, c.final_ln_eps))) return rc;
    final_hidden = e->t;
  }
  for (int l = 0; !prenorm && l < c.num_layers; ++l) {
    const EncLayer& L = e->layers[l];
    const bool last = l + 1 == c.num_layers;
    const void* wqkv = e->bf16 ? L.wqkv_h : static_cast<const void*>(L.wqkv);
    const void* wo = e->bf16 ? L.wo_h : static_cast<const void*>(L.wo);
    const void* w1 = e->bf16 ? L.w1_h : static_cast<const void*>(L.w1);
    const void* w2 = e->bf16 ? L.w2_h : static_cast<const void*>(L.w2);
    if ((rc = enc_linear(e, e->x, wqkv, L.bqkv, nullptr, e->qkv, rows, 3 * F, F, ACT_NONE, false))) return rc;
    AttnArgs at{};
    at.B = Bc; at.S = max_len; at.H = H; at.D = D; at.cu_seqlens = cu_chunk_dev; at.scale = 1.0f / sqrtf(static_cast<float>(D));
    at.out = e->attn; at.ld_out = F; at.round_tf32 = e->bf16 ? 0 : 1; at.out_bf16 = e->bf16 ? 1 : 0;
    at.key_mask = key_mask_dev;   // padded layout only (cu_chunk_dev is null then)
    ctx->attn_flops_hint = 4.0 * H * D * sum_len2;  // valid (query, key) pairs only
    const char* qkv = reinterpret_cast<const char*>(e->qkv);
    if ((rc = launch_attention(ctx, e->bf16, qkv, qkv + F * act, qkv + 2 * F * act, 3LL * F, 3LL * F, 3LL * F, rows, at))) return rc;
    if ((rc = enc_linear_norm(e, e->attn, wo, L.bo, e->x, L.ln1_g, L.ln1_b, e->x2, rows, F, F, false))) return rc;
    if ((rc = enc_linear(e, e->x2, w1, L.b1, nullptr, e->h, rows, c.ffn, F, ACT_GELU_TANH, false))) return rc;
    // the last LayerNorm of the model feeds the pooling, which reads fp32
    if ((rc = enc_linear_norm(e, e->h, w2, L.b2, e->x2, L.ln2_g, L.ln2_b, (last && e->bf16) ? static_cast<void*>(e->xf) : e->x, rows, F,
                              c.ffn, last && e->bf16))) return rc;
  }
  PoolArgs p{};
  p.x = final_hidden; p.cu_seqlens = cu_chunk_dev; p.mask = key_mask_dev; p.out = out_dev + static_cast<long long>(b0) * F; p.B = Bc; p.S = S; p.F = F; p.normalize = 1; p.rows_hint = rows;
  p.cls = prenorm ? 1 : 0;
  if ((rc = launch_pool(ctx, p))) return rc;
  if (e->keep_hidden && e->hidden_all)
    GB_CUDA_CHECK(ctx, cudaMemcpyAsync(e->hidden_all + hidden_row0 * F, final_hidden, static_cast<size_t>(rows) * F * sizeof(float),
                                       cudaMemcpyDeviceToDevice, ctx->stream));
  return GRILLY_OK;
}

struct ChunkPlan { int b0, b1, rows, max_len, cu_off; double sum_len2; };

// Splits the batch into chunks of consecutive sentences and writes chunk-relative row offsets to cu_host.
static void plan_chunks(const int* lengths, int B, int chunk_tokens, std::vector<ChunkPlan>& plan, int* cu_host, long long* total) {
  plan.clear();
  long long tot = 0;
  int b = 0, off = 0;
  while (b < B) {
    ChunkPlan c{b, b, 0, 0, off, 0.0};
    cu_host[off] = 0;
    while (c.b1 < B) {
      const int len = lengths[c.b1];
      if (chunk_tokens > 0 && c.b1 > c.b0 && c.rows + len > chunk_tokens) break;
      c.rows += len;
      c.max_len = std::max(c.max_len, len);
      c.sum_len2 += static_cast<double>(len) * len;
      c.b1++;
      cu_host[off + (c.b1 - c.b0)] = c.rows;
    }
    off += (c.b1 - c.b0) + 1;
    tot += c.rows;
    b = c.b1;
    plan.push_back(c);
  }
  *total = tot;
}

extern "C" int grilly_plan_chunks(const int* lengths, int B, int chunk_tokens, int* chunk_bounds_out, int* cu_out,
                                  long long* total_rows_out) {
  if (!lengths || B <= 0 || !chunk_bounds_out || !cu_out) return GRILLY_ERR_INVALID_ARG;
  for (int b = 0; b < B; ++b)
    if (lengths[b] < 0) return GRILLY_ERR_INVALID_ARG;
  std::vector<ChunkPlan> plan;
  long long total = 0;
  plan_chunks(lengths, B, chunk_tokens, plan, cu_out, &total);
  for (size_t i = 0; i < plan.size(); ++i) chunk_bounds_out[i] = plan[i].b0;
  chunk_bounds_out[plan.size()] = B;
  if (total_rows_out) *total_rows_out = total;
  return static_cast<int>(plan.size());
}

static int forward_device_nolock(grilly_encoder* e, const int* ids_dev, const int* lengths, int B, int S, float* out_dev,
                                 int* cu_host_staging) {
  grilly_ctx* ctx = e->ctx;
  if (e->cfg.arch == GRILLY_ARCH_POST_LN && S > e->cfg.max_pos) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder: sequence length exceeds the position table");
  for (int b = 0; b < B; ++b)
    if (lengths[b] < 0 || lengths[b] > S) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder: a valid length is outside [0, S]");
  std::vector<ChunkPlan> plan;
  long long total = 0;
  plan_chunks(lengths, B, e->cfg.chunk_tokens, plan, cu_host_staging, &total);
  int max_rows = 1;
  for (auto& c : plan) max_rows = std::max(max_rows, c.rows);
  int rc = ensure_workspace(e, max_rows);
  if (rc) return rc;
  if (e->keep_hidden && total > e->hidden_cap) {
    enc_release(e, e->hidden_all);
    e->hidden_all = nullptr;
    if ((rc = enc_alloc(e, static_cast<size_t>(total) * e->cfg.hidden * sizeof(float), reinterpret_cast<void**>(&e->hidden_all)))) return rc;
    e->hidden_cap = total;
  }
  const int n_cu = plan.back().cu_off + (plan.back().b1 - plan.back().b0) + 1;
  GB_CUDA_CHECK(ctx, cudaMemcpyAsync(e->cu_dev, cu_host_staging, static_cast<size_t>(n_cu) * sizeof(int), cudaMemcpyHostToDevice, ctx->stream));
  long long row0 = 0;
  for (auto& c : plan) {
    if (c.rows == 0) {
      // only empty sentences: their pooled vectors are zero
      GB_CUDA_CHECK(ctx, cudaMemsetAsync(out_dev + static_cast<long long>(c.b0) * e->cfg.hidden, 0,
                                         static_cast<size_t>(c.b1 - c.b0) * e->cfg.hidden * sizeof(float), ctx->stream));
      continue;
    }
    if ((rc = run_chunk(e, ids_dev, e->cu_dev + c.cu_off, c.b0, c.b1, S, c.rows, std::max(c.max_len, 1), out_dev, row0, c.sum_len2))) return rc;
    row0 += c.rows;
  }
  e->last_rows = total;
  return GRILLY_OK;
}

// Masks that are not a run of ones followed by zeros cannot be packed: run on the padded layout (B*S rows) with the
// mask applied as a key mask in attention and as the pooling mask, exactly as the reference does.
static int forward_padded_nolock(grilly_encoder* e, const int* ids_dev, const float* mask_dev, int B, int S, float* out_dev) {
  grilly_ctx* ctx = e->ctx;
  if (e->cfg.arch == GRILLY_ARCH_POST_LN && S > e->cfg.max_pos) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder: sequence length exceeds the position table");
  int per_chunk = B;
  if (e->cfg.chunk_tokens > 0) per_chunk = std::max(1, e->cfg.chunk_tokens / S);
  int rc = ensure_workspace(e, static_cast<long long>(std::min(per_chunk, B)) * S);
  if (rc) return rc;
  const long long total = static_cast<long long>(B) * S;
  if (e->keep_hidden && total > e->hidden_cap) {
    enc_release(e, e->hidden_all);
    e->hidden_all = nullptr;
    if ((rc = enc_alloc(e, static_cast<size_t>(total) * e->cfg.hidden * sizeof(float), reinterpret_cast<void**>(&e->hidden_all)))) return rc;
    e->hidden_cap = total;
  }
  for (int b0 = 0; b0 < B; b0 += per_chunk) {
    const int b1 = std::min(B, b0 + per_chunk);
    const int rows = (b1 - b0) * S;
    if ((rc = run_chunk(e, ids_dev, nullptr, b0, b1, S, rows, S, out_dev, static_cast<long long>(b0) * S,
                        static_cast<double>(b1 - b0) * S * S, mask_dev + static_cast<long long>(b0) * S))) return rc;
  }
  e->last_rows = total;
  return GRILLY_OK;
}

extern "C" {

int grilly_encoder_create(grilly_ctx* ctx, const grilly_encoder_config* cfg, grilly_encoder** out) {
  if (!ctx || !cfg || !out) return GRILLY_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(ctx->mu);
  *out = nullptr;
  if (cfg->precision != GRILLY_PREC_TF32 && cfg->precision != GRILLY_PREC_BF16) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder: precision must be GRILLY_PREC_TF32 or GRILLY_PREC_BF16");
  if (cfg->num_layers <= 0 || cfg->hidden <= 0 || cfg->num_heads <= 0 || cfg->ffn <= 0 || cfg->vocab <= 0 || cfg->max_pos <= 0)
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder: sizes must be positive");
  if (cfg->hidden % cfg->num_heads) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder: hidden must be divisible by num_heads");
  const int D = cfg->hidden / cfg->num_heads;
  // head dims the attention kernels are instantiated for (bf16 head_dim 32 only while every sentence fits one key tile)
  const bool d_ok = cfg->precision == GRILLY_PREC_BF16 ? (D == 32 || D == 64 || D == 128) : (D == 32 || D == 64 || D == 96 || D == 128);
  if (!d_ok) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "encoder: head_dim must be 32, 64, 96 or 128 (tf32) / 32, 64 or 128 (bf16)");
  if (cfg->precision == GRILLY_PREC_BF16 && (cfg->hidden % 8 || cfg->ffn % 8))
    return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "encoder: bf16 mode needs hidden and ffn to be multiples of 8");
  if (cfg->hidden % 4 || cfg->ffn % 4 || cfg->hidden > 1024) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "encoder: hidden and ffn must be multiples of 4, hidden at most 1024");
  if (cfg->arch != GRILLY_ARCH_POST_LN && cfg->arch != GRILLY_ARCH_MODERNBERT) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder: unknown architecture");
  if (cfg->arch == GRILLY_ARCH_MODERNBERT && cfg->precision != GRILLY_PREC_TF32)
    return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "encoder: the pre-norm (ModernBERT) architecture runs in tf32 mode");
  if (cfg->arch == GRILLY_ARCH_MODERNBERT && !(cfg->rope_base > 0.f)) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder: rope_base must be positive");
  cudaSetDevice(ctx->device);
  grilly_encoder* e = new grilly_encoder();
  e->ctx = ctx;
  e->cfg = *cfg;
  e->bf16 = cfg->precision == GRILLY_PREC_BF16;
  e->layers.resize(cfg->num_layers);
  const size_t F = cfg->hidden, ffn = cfg->ffn;
  int rc = 0;
  auto A = [&](float** p, size_t n) { if (!rc) rc = enc_alloc(e, n * sizeof(float), reinterpret_cast<void**>(p)); };
  A(&e->word, static_cast<size_t>(cfg->vocab) * F); A(&e->pos, static_cast<size_t>(cfg->max_pos) * F); A(&e->type, 2 * F);
  A(&e->emb_g, F); A(&e->emb_b, F);
  if (cfg->arch == GRILLY_ARCH_MODERNBERT) { A(&e->final_g, F); A(&e->final_b, F); }
  for (auto& L : e->layers) {
    if (cfg->arch == GRILLY_ARCH_MODERNBERT) { A(&L.wgu, 2 * ffn * F); A(&L.bgu, 2 * ffn); }
    A(&L.wqkv, 3 * F * F); A(&L.bqkv, 3 * F); A(&L.wo, F * F); A(&L.bo, F); A(&L.ln1_g, F); A(&L.ln1_b, F);
    A(&L.w1, ffn * F); A(&L.b1, ffn); A(&L.w2, F * ffn); A(&L.b2, F); A(&L.ln2_g, F); A(&L.ln2_b, F);
    if (e->bf16) {
      auto Hh = [&](void** p, size_t n) { if (!rc) rc = enc_alloc(e, n * 2, p); };
      Hh(&L.wqkv_h, 3 * F * F); Hh(&L.wo_h, F * F); Hh(&L.w1_h, ffn * F); Hh(&L.w2_h, F * ffn);
    }
  }
  if (rc) {
    for (void* p : e->owned) cudaFree(p);
    delete e;
    return rc;
  }
  *out = e;
  return GRILLY_OK;
}

int grilly_encoder_set_weight(grilly_encoder* e, const char* name, int layer, const float* data, size_t count) {
  if (!e || !name || !data) return GRILLY_ERR_INVALID_ARG;
  grilly_ctx* ctx = e->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  cudaSetDevice(ctx->device);
  const size_t F = e->cfg.hidden, ffn = e->cfg.ffn;
  float* dst = nullptr;
  void* dst_h = nullptr;   // bf16 copy of a GEMM weight (bf16 mode)
  size_t expect = 0;
  bool is_gemm_weight = false;
  const std::string n(name);
  if (layer < 0) {
    if (n == "word") { dst = e->word; expect = static_cast<size_t>(e->cfg.vocab) * F; }
    else if (n == "pos") { dst = e->pos; expect = static_cast<size_t>(e->cfg.max_pos) * F; }
    else if (n == "type") { dst = e->type; expect = 2 * F; }
    else if (n == "emb_ln_g") { dst = e->emb_g; expect = F; }
    else if (n == "emb_ln_b") { dst = e->emb_b; expect = F; }
    else if (n == "final_g") { dst = e->final_g; expect = F; }
    else if (n == "final_b") { dst = e->final_b; expect = F; }
  } else if (layer < e->cfg.num_layers) {
    EncLayer& L = e->layers[layer];
    if (n == "wqkv") { dst = L.wqkv; dst_h = L.wqkv_h; expect = 3 * F * F; is_gemm_weight = true; }
    else if (n == "bqkv") { dst = L.bqkv; expect = 3 * F; }
    else if (n == "wo") { dst = L.wo; dst_h = L.wo_h; expect = F * F; is_gemm_weight = true; }
    else if (n == "bo") { dst = L.bo; expect = F; }
    else if (n == "ln1_g") { dst = L.ln1_g; expect = F; }
    else if (n == "ln1_b") { dst = L.ln1_b; expect = F; }
    else if (n == "w1") { dst = L.w1; dst_h = L.w1_h; expect = ffn * F; is_gemm_weight = true; }
    else if (n == "b1") { dst = L.b1; expect = ffn; }
    else if (n == "w2") { dst = L.w2; dst_h = L.w2_h; expect = F * ffn; is_gemm_weight = true; }
    else if (n == "b2") { dst = L.b2; expect = F; }
    else if (n == "ln2_g") { dst = L.ln2_g; expect = F; }
    else if (n == "ln2_b") { dst = L.ln2_b; expect = F; }
    else if (n == "wgu") { dst = L.wgu; expect = 2 * ffn * F; is_gemm_weight = true; }
    else if (n == "bgu") { dst = L.bgu; expect = 2 * ffn; }
  }
  if (!dst) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder_set_weight: unknown weight name '" + n + "' or layer");
  if (count != expect) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder_set_weight: '" + n + "' expects " + std::to_string(expect) + " values");
  GB_CUDA_CHECK(ctx, cudaMemcpyAsync(dst, data, count * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  int rc = GRILLY_OK;
  // GEMM weights are consumed as tf32: round them to nearest once here instead of letting the MMA truncate
  if (is_gemm_weight && e->bf16) rc = launch_f32_to_bf16(ctx, dst, dst_h, static_cast<long long>(count));
  else if (is_gemm_weight) rc = launch_round_tf32(ctx, dst, dst, static_cast<long long>(count));
  GB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));  // the host array may be freed by the caller
  return rc;
}

int grilly_encoder_keep_hidden(grilly_encoder* e, int on) {
  if (!e) return GRILLY_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(e->ctx->mu);
  e->keep_hidden = on != 0;
  return GRILLY_OK;
}

int grilly_encoder_forward_device(grilly_encoder* e, const int* ids_dev, const int* lengths_host, int B, int S, float* out_dev) {
  if (!e) return GRILLY_ERR_INVALID_ARG;
  grilly_ctx* ctx = e->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  cudaSetDevice(ctx->device);
  if (!ids_dev || !lengths_host || !out_dev || B <= 0 || S <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder_forward_device: bad arguments");
  int rc = ensure_io(e, B, S);
  if (rc) return rc;
  // the staging array is reused by the next call: wait for the previous upload of it to finish
  GB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
  return forward_device_nolock(e, ids_dev, lengths_host, B, S, out_dev, e->cu_pin);
}

int grilly_encoder_forward(grilly_encoder* e, const int* ids_host, const float* mask_host, int B, int S, float* out_host) {
  if (!e) return GRILLY_ERR_INVALID_ARG;
  grilly_ctx* ctx = e->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  cudaSetDevice(ctx->device);
  if (!ids_host || !out_host || B <= 0 || S <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder_forward: bad arguments");
  int rc = ensure_io(e, B, S);
  if (rc) return rc;
  // the ids go on their way first: the copy runs while the host reads the mask
  const size_t n_ids = static_cast<size_t>(B) * S;
  if (ids_host != e->ids_pin) std::memcpy(e->ids_pin, ids_host, n_ids * sizeof(int));   // already staged by the caller otherwise
  GB_CUDA_CHECK(ctx, cudaMemcpyAsync(e->ids_dev, e->ids_pin, n_ids * sizeof(int), cudaMemcpyHostToDevice, ctx->stream));
  // valid lengths from the mask; the packed path needs every mask row to be a prefix of ones
  std::vector<int> lengths(B);
  bool holes = false;
  for (int b = 0; b < B && !holes; ++b) {
    int len = S;
    if (mask_host) {
      // branch-free counts (the compiler vectorises them): the row is a prefix of ones exactly when its first
      // `count` entries are all ones
      const float* m = mask_host + static_cast<size_t>(b) * S;
      int count = 0, head = 0;
      for (int s = 0; s < S; ++s) count += m[s] > 0.5f ? 1 : 0;
      for (int s = 0; s < count; ++s) head += m[s] > 0.5f ? 1 : 0;
      holes = head != count;
      len = count;
    }
    lengths[b] = len;
  }
  if (holes) {
    GB_CUDA_CHECK(ctx, cudaMemcpyAsync(e->mask_dev, mask_host, n_ids * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    rc = forward_padded_nolock(e, e->ids_dev, e->mask_dev, B, S, e->out_dev);
  } else {
    rc = forward_device_nolock(e, e->ids_dev, lengths.data(), B, S, e->out_dev, e->cu_pin);
  }
  if (rc) return rc;
  const size_t out_bytes = static_cast<size_t>(B) * e->cfg.hidden * sizeof(float);
  GB_CUDA_CHECK(ctx, cudaMemcpyAsync(e->out_pin, e->out_dev, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
  GB_CUDA_CHECK(ctx, cudaMemcpyAsync(ctx->err_host, ctx->err_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  GB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
  if (*ctx->err_host != 0) {
    const int code = *ctx->err_host;
    *ctx->err_host = 0;
    cudaMemsetAsync(ctx->err_dev, 0, sizeof(int), ctx->stream);
    return set_error(ctx, GRILLY_ERR_TIMEOUT, "a device-side wait gave up (kernel status " + std::to_string(code) + ")");
  }
  if (out_host != e->out_pin) std::memcpy(out_host, e->out_pin, out_bytes);
  return GRILLY_OK;
}

int grilly_encoder_io_buffers(grilly_encoder* e, int B, int S, int** ids_pinned, float** out_pinned) {
  if (!e || B <= 0 || S <= 0) return GRILLY_ERR_INVALID_ARG;
  grilly_ctx* ctx = e->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  cudaSetDevice(ctx->device);
  const int rc = ensure_io(e, B, S);
  if (rc) return rc;
  if (ids_pinned) *ids_pinned = e->ids_pin;
  if (out_pinned) *out_pinned = e->out_pin;
  return GRILLY_OK;
}

int grilly_encoder_last_hidden(grilly_encoder* e, float* out_host, long long max_rows, long long* rows) {
  if (!e || !rows) return GRILLY_ERR_INVALID_ARG;
  grilly_ctx* ctx = e->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  cudaSetDevice(ctx->device);
  if (!e->keep_hidden || !e->hidden_all) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "encoder_last_hidden: enable grilly_encoder_keep_hidden before the forward");
  *rows = e->last_rows;
  if (!out_host) return GRILLY_OK;
  const long long n = std::min(max_rows, e->last_rows);
  GB_CUDA_CHECK(ctx, cudaMemcpyAsync(out_host, e->hidden_all, static_cast<size_t>(n) * e->cfg.hidden * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  GB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
  return GRILLY_OK;
}

int grilly_encoder_destroy(grilly_encoder* e) {
  if (!e) return GRILLY_ERR_INVALID_ARG;
  {
    std::lock_guard<std::mutex> lock(e->ctx->mu);
    cudaSetDevice(e->ctx->device);
    cudaStreamSynchronize(e->ctx->stream);
    for (void* p : e->owned) cudaFree(p);
    if (e->ids_pin) cudaFreeHost(e->ids_pin);
    if (e->cu_pin) cudaFreeHost(e->cu_pin);
    if (e->out_pin) cudaFreeHost(e->out_pin);
  }
  delete e;
  return GRILLY_OK;
}

}  // extern "C"
