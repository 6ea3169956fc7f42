/*
 * grilly_b200 -- C ABI of the CUDA (sm_100a) implementation of grilly's dense
 * transformer hot path.  Plain pointers and sizes only; every function returns
 * a status code (0 = GRILLY_OK, negative = error) and grilly_last_error() gives
 * the message.  Pointers named *_dev are device addresses on the context's GPU;
 * pointers named *_host are host addresses.  All work is issued on the
 * context's stream; calls taking host output buffers return after the data has
 * arrived, the others are asynchronous until grilly_sync().
 *
 * File:line citations name the reference (grilly 0.1.0) interface each entry
 * point replaces; paths are relative to the reference's project root.
 */
#ifndef GRILLY_B200_H
#define GRILLY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct grilly_ctx grilly_ctx;
typedef struct grilly_encoder grilly_encoder;

enum {
  GRILLY_OK = 0,
  GRILLY_ERR_INVALID_ARG = -1,
  GRILLY_ERR_OOM = -2,
  GRILLY_ERR_CUDA = -3,
  GRILLY_ERR_NCCL = -4,
  GRILLY_ERR_TIMEOUT = -5,     /* a bounded device-side wait gave up */
  GRILLY_ERR_UNSUPPORTED = -6
};

/* GRILLY_PREC_TF32X3 (grilly_linear, grilly_fused_qkv_projection, grilly_gemm_mnk only): operands are raw fp32; every
 * value is split into tf32 hi + lo and the product runs over 3K (hi.hi + lo.hi + hi.lo, fp32 accumulate), which gives
 * fp32-level results (rel-L2 about 3e-6), so that argmax / top-k indices taken from the output agree with the
 * reference's fp32 arithmetic (fnn-linear.glsl:43-57, gemm_mnk.glsl:48-87). Three times the MMAs, scratch of 3 x the
 * operand bytes from the context's pool. */
enum { GRILLY_PREC_TF32 = 0, GRILLY_PREC_BF16 = 1, GRILLY_PREC_TF32X3 = 2 };
enum { GRILLY_ACT_NONE = 0, GRILLY_ACT_GELU = 1, GRILLY_ACT_SILU = 2, GRILLY_ACT_RELU = 3 };
enum { GRILLY_NORM_LAYER = 0, GRILLY_NORM_RMS = 1 };
enum { GRILLY_ELT_GELU = 1, GRILLY_ELT_SILU = 2, GRILLY_ELT_RELU = 3, GRILLY_ELT_ADD = 4, GRILLY_ELT_SWIGLU = 5,
       GRILLY_ELT_GCU = 6, GRILLY_ELT_ROSWISH = 7 };
enum { GRILLY_ROPE_NONE = 0, GRILLY_ROPE_INTERLEAVED = 1, GRILLY_ROPE_ROTATE_HALF = 2 };
enum { GRILLY_DIST_L2 = 1, GRILLY_DIST_COSINE = 2, GRILLY_DIST_DOT = 3 };  /* faiss-distance.glsl:25 (there 0, 1, 2) */

/* flags for the GEMM family, attention and the norms */
enum {
  GRILLY_FLAG_OUT_BF16 = 1,     /* store the result as bf16 instead of fp32 */
  GRILLY_FLAG_ROUND_TF32 = 2,   /* round fp32 results to the nearest tf32 value (they feed a tf32 GEMM next) */
  GRILLY_FLAG_SWIGLU_PAIRS = 4  /* weight rows interleaved (gate_j, up_j): y[:, j] = gate_j * silu(up_j), N/2 columns out;
                                   with act = GRILLY_ACT_GELU the gate is gate_j * gelu(up_j) (GeGLU) */
};

/* ---- context, replaces VulkanCore (backend/core.py:14-439) ------------------------------- */
int grilly_device_count(int* count);
/* backend/core.py:17-33,57-166: instance + device + queue creation -> one context per (process, GPU) */
int grilly_init(int device, grilly_ctx** ctx);
/* backend/core.py:423-439 cleanup(), backend/compute.py:56-68 */
int grilly_shutdown(grilly_ctx* ctx);
const char* grilly_last_error(grilly_ctx* ctx);
/* run on a caller-owned CUDA stream (e.g. torch's current stream); NULL restores the context's own stream */
int grilly_set_stream(grilly_ctx* ctx, void* cuda_stream);
/* backend/core.py:417-418 vkQueueWaitIdle; also reports a device-side wait that gave up as GRILLY_ERR_TIMEOUT */
int grilly_sync(grilly_ctx* ctx);
/* Tuning / debug knobs of the kernel selection, normally left alone. They are read from the environment once in
 * grilly_init (GRILLY_GEMM_GROUP, GRILLY_GEMM_BN, GRILLY_GEMM_PAIR, GRILLY_GEMM_SWAP, GRILLY_ATTN_HPC,
 * GRILLY_ATTN_GENERAL, GRILLY_FUSED_LN) and can be changed here per context: name in {gemm_group, gemm_bn, gemm_pair, gemm_swap,
 * attn_hpc, attn_general, fused_ln}; value 0 (gemm_pair, gemm_swap: -1) restores the default choice. The reference has no
 * counterpart (its shaders have fixed workgroup sizes, backend/fnn.py:1465-1470). */
int grilly_set_tuning(grilly_ctx* ctx, const char* name, int value);
/* number of kernels this context has launched (monotonic) */
int grilly_launch_count(grilly_ctx* ctx, uint64_t* count);

/* Per-kernel-class timing with CUDA events on the launching stream (the reference has no profiler; its
 * tutorials time with perf_counter, tutorials/02_fused_operations.py:29-39). Between begin and end every launch is
 * bracketed by an event pair. out has 6 classes x 4 doubles: {launches, milliseconds, algorithmic FLOPs,
 * algorithmic bytes} for class 0 GEMM, 1 attention, 2 norm, 3 embedding, 4 pooling, 5 other. */
/* Failure-detection self-test: launches a kernel whose only wait (on a barrier nothing signals) runs out after
 * budget_ms (1..1000). The kernel returns normally; the next grilly_sync() reports GRILLY_ERR_TIMEOUT once and the
 * context keeps working. The reference has no counterpart (its dispatch blocks in vkQueueWaitIdle, backend/core.py:418). */
int grilly_selftest_wait_timeout(grilly_ctx* ctx, int budget_ms);
/* Device-side stopwatch: start records an event on the context's stream, stop records a second one, waits for it
 * and returns the milliseconds between the two. */
int grilly_timer_start(grilly_ctx* ctx);
int grilly_timer_stop(grilly_ctx* ctx, float* ms);
int grilly_profile_begin(grilly_ctx* ctx);
int grilly_profile_end(grilly_ctx* ctx, double* out);

/* ---- device pool, replaces BufferPool / VMABufferPool (backend/buffer_pool.py:466-651, 120-462;
 *      backend/vma_wrapper.py:268-437) with a stream-ordered cudaMallocAsync pool ------------- */
/* backend/buffer_pool.py:534-562 acquire() */
int grilly_alloc(grilly_ctx* ctx, size_t bytes, void** dptr);
/* backend/buffer_pool.py:564-579 release() */
int grilly_free(grilly_ctx* ctx, void* dptr);
/* backend/core.py:345-350 _upload_buffer */
int grilly_upload(grilly_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
/* backend/core.py:352-360 _download_buffer (returns after the copy has completed) */
int grilly_download(grilly_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
/* Strided device-to-device copy of `rows` rows of `width_bytes` on the context's stream (cudaMemcpy2DAsync); dst or
 * src may be peer-mapped memory of another GPU. Used to move row slabs of a column block of C between GPUs without
 * handing peer memory to any kernel. No counterpart in the reference (no multi-GPU code, CHANGELOG.md:75). */
int grilly_copy_2d(grilly_ctx* ctx, void* dst_dev, size_t dst_pitch, const void* src_dev, size_t src_pitch, size_t width_bytes,
                   size_t rows);
/* Fills nbytes at dst_dev with a byte value on the context's stream (cudaMemsetAsync). */
int grilly_memset(grilly_ctx* ctx, void* dst_dev, int byte_value, size_t nbytes);
/* pinned host staging memory for the two calls above */
int grilly_host_alloc(grilly_ctx* ctx, size_t bytes, void** hptr);
int grilly_host_free(grilly_ctx* ctx, void* hptr);
/* backend/buffer_pool.py:627-640 get_stats(): out[0]=allocs out[1]=frees out[2]=bytes_in_use
 * out[3]=peak_bytes out[4]=pool_reserved_bytes out[5]=tensor_map_cache_hits out[6]=tensor_map_cache_misses
 * out[7]=pool_hits (allocations the pool served from memory it already held; misses = allocs - hits) */
int grilly_pool_stats(grilly_ctx* ctx, uint64_t out[8]);

/* ---- conversions used when operands enter from NumPy ------------------------------------ */
int grilly_round_tf32(grilly_ctx* ctx, const float* x_dev, float* y_dev, long long n);
int grilly_cast_f32_to_bf16(grilly_ctx* ctx, const float* x_dev, void* y_dev, long long n);
int grilly_cast_bf16_to_f32(grilly_ctx* ctx, const void* x_dev, float* y_dev, long long n);

/* ---- GEMM family ------------------------------------------------------------------------- */
/* y[M,N] = act(x[M,K] * W[N,K]^T + bias) (+ residual).  W is (out, in) row-major.
 * VulkanFNN.linear backend/fnn.py:1394-1496 (shader fnn-linear.glsl:33-58);
 * fused_linear_gelu/relu/silu backend/fnn.py:2022-2303 (fused-linear-{gelu,relu,silu}.glsl);
 * GRILLY_FLAG_SWIGLU_PAIRS: fused-swiglu.glsl:48-79, backend/_glu_append.py:47-60; with GRILLY_ACT_GELU
 * fused-geglu.glsl:53-84, backend/_glu_append.py:224-262.
 * x and W are fp32 (precision TF32) or bf16 (precision BF16); bias and residual are fp32. */
int grilly_linear(grilly_ctx* ctx, const void* x_dev, const void* w_dev, const float* bias_dev,
                  const float* residual_dev, void* y_dev, int M, int N, int K, int act, int precision, int flags);
/* QKV = x * [Wq;Wk;Wv]^T + [bq;bk;bv], output (rows, 3*H*D) with column blocks Q,K,V.
 * fused-qkv-projection.glsl:48-74 (no Python wrapper in the reference). */
int grilly_fused_qkv_projection(grilly_ctx* ctx, const void* x_dev, const void* w_qkv_dev, const float* b_qkv_dev,
                                void* qkv_dev, int rows, int hidden, int num_heads, int head_dim, int precision,
                                int flags);
/* One-time fold for the call below: Wf = W * diag(gamma), col_sum[c] = sum_k Wf[c,k] (of the tf32/bf16-rounded
 * values the GEMM will consume), bias_f = bias + W * beta.  Outputs: wf_dev (N*K, fp32 or bf16), col_sum_dev (N),
 * bias_f_dev (N). */
int grilly_fold_layernorm_weights(grilly_ctx* ctx, const float* w_dev, const float* gamma_dev, const float* beta_dev,
                                  const float* bias_dev, void* wf_dev, float* col_sum_dev, float* bias_f_dev, int N,
                                  int K, int precision);
/* y = Linear(Norm(x)): row statistics kernel + GEMM with the normalisation finished in the epilogue.
 * fused-layernorm-linear.glsl:67-128 (mode GRILLY_NORM_LAYER); snn-rmsnorm.glsl:34-75 then fnn-linear (GRILLY_NORM_RMS).
 * x [M,K] is fp32 (precision TF32) or bf16 (precision BF16; fold the weights with the same precision); stats_dev is
 * scratch for 2*M floats (mean, rstd).
 * Accuracy envelope: the GEMM consumes the RAW rows and the epilogue computes rstd * (acc - mean * col_sum), which
 * loses accuracy by cancellation when a row's mean is large against its standard deviation (rel-L2 grows like
 * sqrt(1 + (mean/std)^2) times the plain product's error). In LayerNorm mode the statistics kernel therefore also
 * reports the largest |mean|/std of the call; the entry point reads it back (ONE stream synchronisation) and, above
 * GRILLY_LNLINEAR_MAX_MEAN_OVER_STD, normalises the rows into pool scratch (M x K elements) and runs the GEMM on
 * those instead, as fused-layernorm-linear.glsl:102-126 orders the operations. Either way the result is within the
 * precision's tolerance (2e-3 tf32, 1e-2 bf16). RMS mode has no mean term: always the folded form, no
 * synchronisation. */
#define GRILLY_LNLINEAR_MAX_MEAN_OVER_STD 1.5f
int grilly_layernorm_linear(grilly_ctx* ctx, const void* x_dev, const void* wf_dev, const float* col_sum_dev,
                            const float* bias_f_dev, void* y_dev, float* stats_dev, int M, int N, int K, float eps,
                            int norm_mode, int act, int precision, int flags);
/* Same result as grilly_layernorm_linear, for callers that cannot allocate device memory while they run an op
 * (a serving thread with a fixed memory budget, or a process whose device memory is owned by another allocator):
 * the statistics scratch is a 512 KiB array built into the library image, resident on every GPU that loads the
 * library. No counterpart in the reference. Limits: M <= GRILLY_NOALLOC_MAX_ROWS (more is rejected with
 * GRILLY_ERR_INVALID_ARG); tf32 mode only; all calls on a device share the array, so calls that overlap on the
 * GPU race (calls on one stream are ordered); the first call on a device resolves the array's address and should
 * come before any stream capture. Allocates nothing on the device and frees nothing. */
#define GRILLY_NOALLOC_MAX_ROWS 65536
int grilly_layernorm_linear_noalloc(grilly_ctx* ctx, const float* x_dev, const void* wf_dev, const float* col_sum_dev,
                                    const float* bias_f_dev, void* y_dev, int M, int N, int K, float eps, int norm_mode,
                                    int act, int precision, int flags);
/* y = LayerNorm(x W^T + bias + residual) * gamma + beta: the post-LN step of a BERT layer, which the reference
 * runs as linear, add, layer_norm (utils/vulkan_sentence_transformer.py:997-1011 and 1018-1033; fnn-linear.glsl,
 * fnn-residual.glsl, fnn-layernorm.glsl:44-103; biased variance, eps inside the square root).
 * x [M,K] and W [N,K] are fp32 (TF32) or bf16 (BF16); residual [M,N] has the operands' type; bias, gamma, beta fp32
 * (each may be NULL). For N in {128, 256, 384, 512} this is ONE kernel (a 128-row tile holds whole output rows in
 * tensor memory, the statistics are taken in the GEMM's epilogue and the pre-norm sum never reaches memory);
 * scratch_dev may then be NULL. Other widths run the GEMM into scratch_dev (M*N floats) and the row kernel after it.
 * Flags: GRILLY_FLAG_ROUND_TF32, GRILLY_FLAG_OUT_BF16 (BF16 mode only). Asynchronous. */
int grilly_linear_layernorm(grilly_ctx* ctx, const void* x_dev, const void* w_dev, const float* bias_dev, const void* residual_dev,
                            const float* gamma_dev, const float* beta_dev, void* y_dev, float* scratch_dev, int M, int N, int K,
                            float eps, int precision, int flags);
/* C[M,N] = A[M,K] * B[K,N], all row-major.  VulkanFNN.gemm backend/fnn.py:104-166 (gemm_mnk.glsl:35-88). */
int grilly_gemm_mnk(grilly_ctx* ctx, const void* a_dev, const void* b_dev, void* c_dev, int M, int K, int N,
                    int precision, int flags);

/* ---- attention --------------------------------------------------------------------------- */
/* out = softmax(scale * Q K^T + mask) V per (sequence, head); Q/K/V/out are 2-D row-major views
 * [rows][ld] with head h in columns [h*D, (h+1)*D)  (the (B,S,H,D) layout of
 * VulkanAttention.flash_attention2 backend/attention.py:361-597, flash-attention2.glsl:81-219;
 * RoPE variant flash-attention2-rope.glsl:74-149,165-247; rotate-half pairing rope.glsl:52-126).
 * cu_seqlens_dev == NULL: padded layout, sequence b = rows [b*S,(b+1)*S), optional key_mask_dev [B][S] (1 = keep).
 * cu_seqlens_dev != NULL: packed layout, int32 [B+1] row offsets, S = longest sequence, total_rows = cu_seqlens[B].
 * Causal rule: key position > query position is masked (attention-mask.glsl:42-46). */
int grilly_flash_attention(grilly_ctx* ctx, const void* q_dev, const void* k_dev, const void* v_dev, void* out_dev,
                           int B, int S, int H, int D, long long ld_qkv, long long ld_out, const int* cu_seqlens_dev,
                           long long total_rows, const float* key_mask_dev, float scale, int causal, int rope_style,
                           float rope_base, float rope_scaling, int precision, int flags);
/* The unfused pipeline the reference's encoder calls today (utils/vulkan_sentence_transformer.py:1037-1067), kept so
 * that code runs unchanged; it materialises (B,H,S,S) like the reference does. fp32 FMAs, no tensor cores.
 * VulkanAttention.attention_scores backend/attention.py:41-126 (attention-scores.glsl:33-65): q,k (B,S,H,D) ->
 * scores (B,H,S,S) = scale * Q K^T. */
int grilly_attention_scores(grilly_ctx* ctx, const float* q_dev, const float* k_dev, float* scores_dev, int B, int S, int H,
                            int D, float scale);
/* attention_mask backend/attention.py:128-203 (attention-mask.glsl:26-55), in place: use_causal -> key > query gets
 * mask_value; else key-padding mask_dev (B,S), < 0.5 gets mask_value (NULL = no change). */
int grilly_attention_mask(grilly_ctx* ctx, float* scores_dev, const float* mask_dev, int B, int H, int S, int use_causal,
                          float mask_value);
/* attention_output backend/attention.py:205-300 (attention-output.glsl:28-70): weights (B,H,S,S), v (B,S,H,D) -> (B,S,H,D) */
int grilly_attention_output(grilly_ctx* ctx, const float* weights_dev, const float* v_dev, float* out_dev, int B, int S,
                            int H, int D);
/* The architecture-specific forms the reference's registry selects for attention_output (backend/shader_registry.py:154-156,
 * backend/attention.py:226-229): causal != 0 sums keys k <= q only (attention-output-gpt.glsl, also used for 'granite');
 * Sq != Sk is the decoder-over-encoder form (attention-output-t5.glsl): weights (B,H,Sq,Sk), v (B,Sk,H,D) -> (B,Sq,H,D). */
int grilly_attention_output_ex(grilly_ctx* ctx, const float* weights_dev, const float* v_dev, float* out_dev, int B, int Sq,
                               int Sk, int H, int D, int causal);
/* stand-alone RoPE on (B,S,H,D) fp32, VulkanAttention.apply_rope backend/attention.py:599-676 (rope.glsl:52-126);
 * position_ids_dev int32 [B][S] or NULL for 0..S-1; max_pos = number of table rows to build. */
int grilly_apply_rope(grilly_ctx* ctx, const float* x_dev, float* y_dev, const int* position_ids_dev, int B, int S,
                      int H, int D, int max_pos, float base, float scaling, int rope_style);

/* ---- row kernels ------------------------------------------------------------------------- */
/* y = Norm(x (+ residual)); VulkanFNN.layernorm backend/fnn.py:1285-1389 (fnn-layernorm.glsl:44-103);
 * RMS mode snn-rmsnorm.glsl:34-75.  gamma/beta may be NULL. */
int grilly_layernorm(grilly_ctx* ctx, const float* x_dev, const float* residual_dev, const float* gamma_dev,
                     const float* beta_dev, void* y_dev, long long rows, int F, float eps, int norm_mode, int flags);
/* VulkanFNN.activation_softmax backend/fnn.py:574-663 (activation-softmax.glsl:34-84) */
int grilly_softmax(grilly_ctx* ctx, const float* x_dev, float* y_dev, long long rows, int cols);
/* activation_gelu/silu/relu, residual, activation_swiglu: backend/fnn.py:232-572,1950-2014
 * (activation-{gelu,silu,relu,swiglu}.glsl, fnn-residual.glsl).  n = number of OUTPUT elements;
 * half = output width for GRILLY_ELT_SWIGLU (input rows are 2*half wide). */
int grilly_eltwise(grilly_ctx* ctx, int op, const float* a_dev, const float* b_dev, float* y_dev, long long n,
                   int half);
/* activation_gcu backend/fnn.py:385-440 (x cos x; op GRILLY_ELT_GCU, p0 and p1 unused) and activation_roswish
 * backend/fnn.py:442-497 ((x + alpha) sigmoid(beta x) - alpha / 2; op GRILLY_ELT_ROSWISH, p0 = alpha, p1 = beta). May run
 * in place (y == x): fused_linear_gcu / fused_linear_roswish (backend/fnn.py:2307-2463) are grilly_linear followed by
 * this on the result, on the device. */
int grilly_activation_params(grilly_ctx* ctx, int op, const float* x_dev, float* y_dev, long long n, float p0, float p1);
/* VulkanLearning.embedding_lookup backend/learning.py:811-877 (embedding-lookup.glsl:28-55) */
int grilly_embedding_lookup(grilly_ctx* ctx, const int* ids_dev, const float* table_dev, float* out_dev,
                            long long n_tokens, int vocab, int F);
/* word[id] + type[0] + pos[s] -> LayerNorm, written to padded rows (cu_seqlens_dev NULL) or packed rows.
 * utils/vulkan_sentence_transformer.py:563-747 */
int grilly_embed_layernorm(grilly_ctx* ctx, const int* ids_dev, const int* cu_seqlens_dev, const float* word_dev,
                           const float* pos_dev, const float* type0_dev, const float* gamma_dev, const float* beta_dev,
                           float* out_dev, int B, int S, int F, int vocab, int max_pos, float eps, int flags);
/* masked mean over tokens then optional x/(||x||+1e-8): VulkanPooling.mean_pool backend/pooling.py:22-142
 * (embedding-pool.glsl:61-81) + functional.embedding_normalize functional/embedding.py:42-68 */
int grilly_mean_pool(grilly_ctx* ctx, const float* x_dev, const float* mask_dev, const int* cu_seqlens_dev,
                     float* out_dev, int B, int S, int F, int normalize);

/* ---- backward pass and optimiser step (the training-side callers of the same tensors) ------------------------ */
/* VulkanFNN.layernorm_backward backend/fnn.py:1701-1847 (fnn-layernorm-backward.glsl): grad_in [rows][F],
 * grad_gamma [F] = sum_rows grad_out * x_norm, grad_beta [F] = sum_rows grad_out. gamma may be NULL (= 1); mean_dev /
 * var_dev [rows] are the forward pass's statistics or NULL (then computed: biased variance). Deterministic (no
 * atomics); scratch from the context's pool. */
int grilly_layernorm_backward(grilly_ctx* ctx, const float* grad_out_dev, const float* x_dev, const float* gamma_dev,
                              const float* mean_dev, const float* var_dev, float* grad_in_dev, float* grad_gamma_dev,
                              float* grad_beta_dev, long long rows, int F, float eps);
/* VulkanFNN.softmax_backward backend/fnn.py:1849-1933 (activation-softmax-backward.glsl): grad_in = y * (grad_out -
 * sum(grad_out * y)) over the last dimension. */
int grilly_softmax_backward(grilly_ctx* ctx, const float* grad_out_dev, const float* softmax_out_dev, float* grad_in_dev,
                            long long rows, int cols);
/* VulkanBackwardOps.attention_backward backend/autograd_core.py:609-646 (attention-backward.glsl): all tensors in the
 * (B, H, S, D) layout that function uses, attn_weights (B, H, S, S) from the forward pass:
 *   grad_v = A^T dO; grad_scores = softmax_backward(dO V^T, A) * scale; grad_q = grad_scores K; grad_k = grad_scores^T Q.
 * fp32 products (batched, shared-memory tiled); scratch of B*H*S*S floats from the context's pool. */
int grilly_attention_backward(grilly_ctx* ctx, const float* grad_out_dev, const float* q_dev, const float* k_dev, const float* v_dev,
                              const float* attn_weights_dev, float* grad_q_dev, float* grad_k_dev, float* grad_v_dev, int B, int H,
                              int S, int D, float scale);
/* VulkanLearning.adam_update backend/learning.py:967-1077 (adam-update.glsl), in place on the device:
 * m = b1 m + (1-b1) g; v = b2 v + (1-b2) g^2; w -= lr (m / (1 - b1^t)) / (sqrt(v / (1 - b2^t)) + eps); the bias
 * corrections are skipped when beta^t >= 1, as in the reference's CPU branch; clear_grad zeroes g. */
int grilly_adam_update(grilly_ctx* ctx, float* weights_dev, float* gradients_dev, float* moment1_dev, float* moment2_dev, long long n,
                       float learning_rate, float beta1, float beta2, float epsilon, float beta1_t, float beta2_t, int clear_grad);
/* out[c][r] = in[r][c] on the device: the grad_output^T operand of VulkanFNN.linear_backward's weight gradient
 * (backend/fnn.py:1548-1573 transposes on the host). */
int grilly_transpose_2d(grilly_ctx* ctx, const float* in_dev, float* out_dev, int rows, int cols);

/* ---- resident sentence encoder ---------------------------------------------------------------- */
/* VulkanSentenceTransformer.encode utils/vulkan_sentence_transformer.py:1109-1219; weights live on the device between
 * calls. Two layer architectures, as _forward_layer has them:
 *   GRILLY_ARCH_POST_LN   the BERT / DistilBERT / MiniLM branch (:972-1033): attention, LayerNorm(x + attn), GELU FFN,
 *                         LayerNorm(x + ffn); learned positions and token type added to the embeddings; masked mean pool.
 *   GRILLY_ARCH_MODERNBERT the pre-norm branch (:799-970): q/k/v from x itself (the attention norm is the identity),
 *                         rotate-half RoPE on q and k, x += attn, LayerNorm before a GeGLU MLP
 *                         (gelu(x Wgate^T) * (x Wup^T)) Wo), x += mlp; no position table; a final LayerNorm after the
 *                         last layer and CLS pooling (first token) as encode() does for this model type (:1150-1181). */
enum { GRILLY_ARCH_POST_LN = 0, GRILLY_ARCH_MODERNBERT = 1 };
typedef struct grilly_encoder_config {
  int num_layers, hidden, num_heads, ffn, vocab, max_pos;
  float embed_ln_eps, layer_ln_eps;
  int has_token_type;   /* add token-type row 0 (BERT) */
  int precision;        /* GRILLY_PREC_TF32 or GRILLY_PREC_BF16 */
  int chunk_tokens;     /* process at most this many tokens at once so activations stay L2-resident; 0 = all */
  int arch;             /* GRILLY_ARCH_POST_LN or GRILLY_ARCH_MODERNBERT (tf32 mode only) */
  float rope_base;      /* MODERNBERT: RoPE base (local_rope_theta, :843-846) */
  float final_ln_eps;   /* MODERNBERT: epsilon of the final LayerNorm */
} grilly_encoder_config;

int grilly_encoder_create(grilly_ctx* ctx, const grilly_encoder_config* cfg, grilly_encoder** enc);
/* name in {word, pos, type, emb_ln_g, emb_ln_b, final_g, final_b} (layer = -1) or {wqkv, bqkv, wo, bo, ln1_g, ln1_b, w1,
 * b1, w2, b2, ln2_g, ln2_b, wgu, bgu} (layer >= 0); data are fp32 host arrays in the reference's (out, in) layout.
 * MODERNBERT uses wqkv, bqkv, wo, bo, ln2_g/ln2_b (the MLP norm), w2/b2 (the MLP's output projection) and wgu / bgu:
 * the (2 ffn, hidden) matrix whose rows alternate (up_j, gate_j) -- the row that multiplies first, the row that goes
 * through GELU second -- and the bias interleaved the same way; final_g / final_b are the final LayerNorm. */
int grilly_encoder_set_weight(grilly_encoder* enc, const char* name, int layer, const float* data_host, size_t count);
/* ids_host int32 [B][S]; mask_host fp32 [B][S] (1 = token, 0 = padding) or NULL; out_host fp32 [B][hidden]:
 * mean-pooled, L2-normalised embeddings.  Includes the host->device and device->host copies.  Rows of ones followed
 * by zeros run packed (padding rows never exist on the device); a mask with holes runs the whole batch on the padded
 * layout with the mask as attention key mask and pooling mask. */
int grilly_encoder_forward(grilly_encoder* enc, const int* ids_host, const float* mask_host, int B, int S,
                           float* out_host);
/* The encoder's own page-locked staging buffers, sized for at least B x S ids and B x hidden outputs: a caller that
 * writes its ids there and passes these same pointers to grilly_encoder_forward has its copies to and from the device
 * start from / end in page-locked memory without the staging memcpy on either side. The pointers stay valid until a
 * forward or a call of this function with a larger B or S, or grilly_encoder_destroy. No counterpart in the reference
 * (its staging is Vulkan-mapped memory inside every op, backend/fnn.py:1437-1489). */
int grilly_encoder_io_buffers(grilly_encoder* enc, int B, int S, int** ids_pinned, float** out_pinned);
/* same with device buffers and no copies: ids_dev int32 [B][S], lengths_host int32 [B] valid prefix lengths,
 * out_dev fp32 [B][hidden].  Asynchronous. */
int grilly_encoder_forward_device(grilly_encoder* enc, const int* ids_dev, const int* lengths_host, int B, int S,
                                  float* out_dev);
/* keep a copy of the final hidden states of each forward (off by default; costs one device copy per chunk) */
int grilly_encoder_keep_hidden(grilly_encoder* enc, int on);
/* final hidden states of the last forward (packed rows, fp32 [total_tokens][hidden]) for parity checks */
int grilly_encoder_last_hidden(grilly_encoder* enc, float* out_host, long long max_rows, long long* rows);
int grilly_encoder_destroy(grilly_encoder* enc);

/* C = A B like grilly_gemm_mnk, with the fp32 result stored to num_outputs (1..8) matrices c_ptrs[i] (host array of
 * device pointers), all with row pitch ld_c >= N elements; N must be a multiple of 32. The destinations may be
 * peer-mapped memory of other GPUs (plain stores only): with each GPU computing one column block of a product and
 * writing it into every GPU's C at its column offset, the exchange of a column-split GEMM happens inside the kernel,
 * tile by tile, instead of in an all-gather after it. No counterpart in the reference, which has no multi-GPU code
 * (CHANGELOG.md:75). One launch of THIS entry point at a time per GPU: the destination list lives in constant memory
 * of the library and is rewritten in stream order by every call, so two contexts or streams that overlap such
 * launches on one GPU would mix their lists. Other GEMM launches never read the list (the multi-destination epilogue
 * is selected by an argument of this launch alone) and may overlap freely. Asynchronous. */
int grilly_gemm_mnk_multi(grilly_ctx* ctx, const void* a_dev, const void* b_dev, void* const* c_ptrs, int num_outputs, int M,
                          int K, int N, long long ld_c, int precision);

/* ---- vector search over the embeddings ---------------------------------------------------------------------- */
/* Replaces VulkanFAISS.compute_distances (backend/faiss.py:25-104; shader faiss-distance.glsl:29-83):
 * out[q][d] for queries fp32 [num_queries][dim] and database fp32 [num_database][dim], all device pointers.
 *   GRILLY_DIST_L2     sqrt(sum (q - d)^2), evaluated as sqrt(max(|q|^2 + |d|^2 - 2 q.d, 0))
 *   GRILLY_DIST_COSINE 1 - q.d / (|q| |d| + 1e-8)
 *   GRILLY_DIST_DOT    -(q.d)
 * The dot products come from one tensor-core GEMM over tf32 hi/lo splits of both operands (fp32-level accuracy);
 * scratch of 3 x the operand bytes is taken from the context's pool for the duration of the call. Asynchronous. */
int grilly_faiss_distances(grilly_ctx* ctx, const float* queries, const float* database, float* out, int num_queries,
                           int num_database, int dim, int distance_type);
/* Replaces VulkanFAISS.topk (backend/faiss.py:120-195; shader faiss-topk.glsl): for each of num_queries rows of
 * distances fp32 [num_queries][num_database], the k smallest values in ascending order (equal values by ascending
 * index) and their column indices. Exact selection; 1 <= k <= min(num_database, 1024). Asynchronous. */
int grilly_faiss_topk(grilly_ctx* ctx, const float* distances, int num_queries, int num_database, int k,
                      unsigned int* indices_out, float* distances_out);

/* compute_distances followed by topk (backend/faiss.py:25-104 then :120-195, the two calls of the reference's search
 * examples, README.md:117-122) without the (num_queries, num_database) matrix: the database is walked in chunks whose
 * distance block stays in L2, each block is reduced to its k best per query at once, and the chunks' winners are
 * merged. Same values, indices and tie order as grilly_faiss_distances + grilly_faiss_topk. 1 <= k <= min(num_database,
 * 1024). Scratch (one chunk's split operands, one block, the candidates) from the context's pool. Asynchronous. */
int grilly_faiss_search(grilly_ctx* ctx, const float* queries, const float* database, int num_queries, int num_database, int dim,
                        int k, int distance_type, unsigned int* indices_out, float* distances_out);

/* ---- host-side planning helpers (no GPU needed; exposed so the host logic can be tested on CPU) ------------- */
/* N-tile (64/128/192/256) the GEMM launcher picks for an M x N output on a GPU with num_sms SMs. */
int grilly_gemm_pick_tile(int M, int N, int num_sms);
/* Splits B sentences with the given valid lengths into chunks of consecutive sentences of at most chunk_tokens
 * packed rows (0 = one chunk; a single sentence longer than the limit gets a chunk of its own).
 * chunk_bounds_out receives n_chunks+1 sentence indices, cu_out one run of chunk-relative row offsets per chunk
 * (B + n_chunks ints in total). Returns the number of chunks, or a negative status. */
int grilly_plan_chunks(const int* lengths, int B, int chunk_tokens, int* chunk_bounds_out, int* cu_out,
                       long long* total_rows_out);

#ifdef __cplusplus
}
#endif
#endif /* GRILLY_B200_H */
