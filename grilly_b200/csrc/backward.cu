// Backward-pass and optimiser kernels next to the forward hot path: LayerNorm backward, softmax backward, attention
// backward and the Adam update. These are the reference's training-side callers of the same tensors
// (backend/fnn.py:1701-1847 layernorm_backward, :1849-1933 softmax_backward; backend/autograd_core.py:609-646 and
// shaders/attention-backward.glsl attention_backward; backend/learning.py:967-1077 and shaders/adam-update.glsl
// adam_update). They are HBM-bound row / element kernels in fp32 plus small batched products; none of them is on the
// inference hot path, so they are written for correctness and coalesced access, not tuned further.
#include "internal.h"
#include <algorithm>

namespace gb {

namespace {
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
}  // namespace

// ---------------------------------------------------------------- LayerNorm backward
// One warp per row. mean/var are taken from the caller when given (the reference accepts the forward pass's values),
// else computed (biased variance). Writes grad_input and the row's (mean, 1/std) for the column reductions.
//   dxn = go * gamma;  dvar = sum(dxn (x - mean)) * -0.5 (var + eps)^-1.5
//   dmean = -sum(dxn) / std + dvar * mean(-2 (x - mean));  gi = dxn / std + dvar * 2 (x - mean) / F + dmean / F
__global__ void __launch_bounds__(256) layernorm_bwd_rows_kernel(const float* __restrict__ go, const float* __restrict__ x,
                                                                 const float* __restrict__ gamma, const float* __restrict__ mean_in,
                                                                 const float* __restrict__ var_in, float* __restrict__ gi,
                                                                 float* __restrict__ stats, long long rows, int F, float eps) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (long long row = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5); row < rows;
       row += static_cast<long long>(gridDim.x) * wpb) {
    const float* xp = x + row * F;
    const float* gp = go + row * F;
    float mean, var;
    if (mean_in) {
      mean = __ldg(mean_in + row);
    } else {
      float s = 0.f;
      for (int i = lane; i < F; i += 32) s += xp[i];
      mean = warp_sum(s) / static_cast<float>(F);
    }
    if (var_in) {
      var = __ldg(var_in + row);
    } else {
      float sq = 0.f;
      for (int i = lane; i < F; i += 32) { const float d = xp[i] - mean; sq += d * d; }
      var = warp_sum(sq) / static_cast<float>(F);
    }
    const float std_ = sqrtf(var + eps);
    const float inv_std = 1.f / std_;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = lane; i < F; i += 32) {
      const float d = xp[i] - mean;
      const float dxn = gp[i] * (gamma ? __ldg(gamma + i) : 1.f);
      s1 = fmaf(dxn, d, s1);
      s2 += dxn;
      s3 += d;
    }
    s1 = warp_sum(s1); s2 = warp_sum(s2); s3 = warp_sum(s3);
    const float invF = 1.f / static_cast<float>(F);
    const float dvar = s1 * -0.5f * inv_std * inv_std * inv_std;
    const float dmean = -s2 * inv_std + dvar * (-2.f * s3 * invF);
    for (int i = lane; i < F; i += 32) {
      const float d = xp[i] - mean;
      const float dxn = gp[i] * (gamma ? __ldg(gamma + i) : 1.f);
      gi[row * F + i] = dxn * inv_std + dvar * 2.f * d * invF + dmean * invF;
    }
    if (lane == 0) { stats[2 * row] = mean; stats[2 * row + 1] = inv_std; }
  }
}

// Column sums over a slab of rows: partial[block][0][f] = sum go * x_norm, partial[block][1][f] = sum go.
// Threads own feature columns, so every load is coalesced and the result does not depend on the launch's timing.
__global__ void __launch_bounds__(256) layernorm_bwd_cols_kernel(const float* __restrict__ go, const float* __restrict__ x,
                                                                 const float* __restrict__ stats, float* __restrict__ partial,
                                                                 long long rows, int F, long long rows_per_block) {
  const long long r0 = static_cast<long long>(blockIdx.x) * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    float gg = 0.f, gb_ = 0.f;
    for (long long r = r0; r < r1; ++r) {
      const float g = go[r * F + f];
      gg = fmaf(g, (x[r * F + f] - stats[2 * r]) * stats[2 * r + 1], gg);
      gb_ += g;
    }
    partial[(static_cast<long long>(blockIdx.x) * 2) * F + f] = gg;
    partial[(static_cast<long long>(blockIdx.x) * 2 + 1) * F + f] = gb_;
  }
}
__global__ void layernorm_bwd_final_kernel(const float* __restrict__ partial, float* __restrict__ grad_gamma,
                                           float* __restrict__ grad_beta, int nblocks, int F) {
  const int f = blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= F) return;
  float gg = 0.f, gb_ = 0.f;
  for (int b = 0; b < nblocks; ++b) {
    gg += partial[(static_cast<long long>(b) * 2) * F + f];
    gb_ += partial[(static_cast<long long>(b) * 2 + 1) * F + f];
  }
  grad_gamma[f] = gg;
  grad_beta[f] = gb_;
}

// ---------------------------------------------------------------- softmax backward: gi = y (go - sum(go y)), one warp per row
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const float* __restrict__ go, const float* __restrict__ y,
                                                          float* __restrict__ gi, long long rows, int cols, float scale) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (long long row = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5); row < rows;
       row += static_cast<long long>(gridDim.x) * wpb) {
    const float* gp = go + row * cols;
    const float* yp = y + row * cols;
    float s = 0.f;
    for (int i = lane; i < cols; i += 32) s = fmaf(gp[i], yp[i], s);
    s = warp_sum(s);
    for (int i = lane; i < cols; i += 32) gi[row * cols + i] = yp[i] * (gp[i] - s) * scale;
  }
}

// ---------------------------------------------------------------- batched fp32 products for the attention backward
// C[b] = alpha * op(A[b]) op(B[b]) with row-major matrices, 32 x 32 tiles through shared memory (padded against bank
// conflicts); op = transpose when the flag is set. A[b] is (M x K) or, transposed, stored as (K x M).
__global__ void __launch_bounds__(256) bmm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                                                      int M, int N, int K, int trans_a, int trans_b, float alpha) {
  __shared__ float sa[32][33], sb[32][33];
  const long long batch = blockIdx.z;
  const float* a = A + batch * static_cast<long long>(M) * K;
  const float* bm = B + batch * static_cast<long long>(K) * N;
  float* c = C + batch * static_cast<long long>(M) * N;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8 threads, 4 outputs each
  const int m0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < K; k0 += 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty + 8 * i;
      // sa[m][k]
      {
        const int m = m0 + (trans_a ? tx : r), k = k0 + (trans_a ? r : tx);
        const float v = (m < M && k < K) ? (trans_a ? a[static_cast<long long>(k) * M + m] : a[static_cast<long long>(m) * K + k]) : 0.f;
        if (trans_a) sa[tx][r] = v; else sa[r][tx] = v;
      }
      // sb[k][n]
      {
        const int k = k0 + (trans_b ? tx : r), n = n0 + (trans_b ? r : tx);
        const float v = (k < K && n < N) ? (trans_b ? bm[static_cast<long long>(n) * K + k] : bm[static_cast<long long>(k) * N + n]) : 0.f;
        if (trans_b) sb[tx][r] = v; else sb[r][tx] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) {
      const float bv = sb[kk][tx];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(sa[ty + 8 * i][kk], bv, acc[i]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty + 8 * i, n = n0 + tx;
    if (m < M && n < N) c[static_cast<long long>(m) * N + n] = alpha * acc[i];
  }
}

static int launch_bmm(grilly_ctx* ctx, const float* A, const float* B, float* C, int batch, int M, int N, int K, bool ta, bool tb,
                      float alpha) {
  if (batch > 65535) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "attention_backward: batch x heads is limited to 65535");
  dim3 grid((N + 31) / 32, (M + 31) / 32, batch);
  bmm_f32_kernel<<<grid, 256, 0, ctx->stream>>>(A, B, C, M, N, K, ta ? 1 : 0, tb ? 1 : 0, alpha);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

// ---------------------------------------------------------------- Adam update, in place
__global__ void __launch_bounds__(256) adam_update_kernel(float* __restrict__ w, float* __restrict__ g, float* __restrict__ m,
                                                          float* __restrict__ v, long long n, float lr, float beta1, float beta2,
                                                          float eps, float c1, float c2, int clear_grad) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float gr = g[i];
    const float m_new = beta1 * m[i] + (1.f - beta1) * gr;
    const float v_new = beta2 * v[i] + (1.f - beta2) * gr * gr;
    m[i] = m_new;
    v[i] = v_new;
    w[i] -= lr * (m_new * c1) / (sqrtf(v_new * c2) + eps);
    if (clear_grad) g[i] = 0.f;
  }
}

// 2-D transpose through a padded shared-memory tile: out[c][r] = in[r][c]
__global__ void __launch_bounds__(256) transpose_kernel(const float* __restrict__ in, float* __restrict__ out, int rows, int cols) {
  __shared__ float t[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty + 8 * i, c = c0 + tx;
    if (r < rows && c < cols) t[ty + 8 * i][tx] = in[static_cast<long long>(r) * cols + c];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty + 8 * i, r = r0 + tx;
    if (r < rows && c < cols) out[static_cast<long long>(c) * rows + r] = t[tx][ty + 8 * i];
  }
}

}  // namespace gb

using namespace gb;

#define BWD_GUARD(ctx)                                                                             \
  if (!(ctx)) return GRILLY_ERR_INVALID_ARG;                                                       \
  std::lock_guard<std::mutex> lock__((ctx)->mu);                                                   \
  if (cudaSetDevice((ctx)->device) != cudaSuccess) return set_error(ctx, GRILLY_ERR_CUDA, "cudaSetDevice failed")

extern "C" {

int grilly_layernorm_backward(grilly_ctx* ctx, const float* grad_out, const float* x, const float* gamma, const float* mean,
                              const float* var, float* grad_in, float* grad_gamma, float* grad_beta, long long rows, int F,
                              float eps) {
  BWD_GUARD(ctx);
  if (!grad_out || !x || !grad_in || !grad_gamma || !grad_beta) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_backward: null operand");
  if (rows <= 0 || F <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "layernorm_backward: rows and features must be positive");
  const int nblocks = static_cast<int>(std::min<long long>((rows + 63) / 64, 2LL * ctx->num_sms));
  const long long rows_per_block = (rows + nblocks - 1) / nblocks;
  float* scratch = nullptr;   // (mean, 1/std) per row, then the per-block column sums
  const size_t bytes = (static_cast<size_t>(rows) * 2 + static_cast<size_t>(nblocks) * 2 * F) * sizeof(float);
  if (cudaMallocAsync(&scratch, bytes, ctx->stream) != cudaSuccess) { cudaGetLastError(); return set_error(ctx, GRILLY_ERR_OOM, "layernorm_backward: no memory for the scratch"); }
  float* partial = scratch + rows * 2;
  const int grid_rows = static_cast<int>(std::min<long long>((rows + 7) / 8, 8LL * ctx->num_sms));
  layernorm_bwd_rows_kernel<<<grid_rows, 256, 0, ctx->stream>>>(grad_out, x, gamma, mean, var, grad_in, scratch, rows, F, eps);
  layernorm_bwd_cols_kernel<<<nblocks, 256, 0, ctx->stream>>>(grad_out, x, scratch, partial, rows, F, rows_per_block);
  layernorm_bwd_final_kernel<<<(F + 255) / 256, 256, 0, ctx->stream>>>(partial, grad_gamma, grad_beta, nblocks, F);
  ctx->launches += 3;
  cudaError_t e = cudaGetLastError();
  cudaFreeAsync(scratch, ctx->stream);
  if (e != cudaSuccess) return set_error(ctx, GRILLY_ERR_CUDA, std::string("layernorm_backward: ") + cudaGetErrorString(e));
  return GRILLY_OK;
}

int grilly_softmax_backward(grilly_ctx* ctx, const float* grad_out, const float* softmax_out, float* grad_in, long long rows,
                            int cols) {
  BWD_GUARD(ctx);
  if (!grad_out || !softmax_out || !grad_in) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "softmax_backward: null operand");
  if (rows <= 0 || cols <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "softmax_backward: rows and cols must be positive");
  const int grid = static_cast<int>(std::min<long long>((rows + 7) / 8, 8LL * ctx->num_sms));
  softmax_bwd_kernel<<<grid, 256, 0, ctx->stream>>>(grad_out, softmax_out, grad_in, rows, cols, 1.f);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int grilly_attention_backward(grilly_ctx* ctx, const float* grad_out, const float* q, const float* k, const float* v,
                              const float* attn_weights, float* grad_q, float* grad_k, float* grad_v, int B, int H, int S, int D,
                              float scale) {
  BWD_GUARD(ctx);
  if (!grad_out || !q || !k || !v || !attn_weights || !grad_q || !grad_k || !grad_v)
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention_backward: null operand");
  if (B <= 0 || H <= 0 || S <= 0 || D <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention_backward: sizes must be positive");
  const long long bh = static_cast<long long>(B) * H;
  if (bh > 65535) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "attention_backward: batch x heads is limited to 65535");
  float* gs = nullptr;   // grad_attn, then grad_scores in place: (B, H, S, S)
  if (cudaMallocAsync(&gs, static_cast<size_t>(bh) * S * S * sizeof(float), ctx->stream) != cudaSuccess) {
    cudaGetLastError();
    return set_error(ctx, GRILLY_ERR_OOM, "attention_backward: no memory for the score gradients");
  }
  const int nb = static_cast<int>(bh);
  int rc = launch_bmm(ctx, attn_weights, grad_out, grad_v, nb, S, D, S, true, false, 1.f);       // grad_v = A^T dO
  if (!rc) rc = launch_bmm(ctx, grad_out, v, gs, nb, S, S, D, false, true, 1.f);                 // grad_attn = dO V^T
  if (!rc) {
    const long long rows = bh * S;
    const int grid = static_cast<int>(std::min<long long>((rows + 7) / 8, 8LL * ctx->num_sms));
    softmax_bwd_kernel<<<grid, 256, 0, ctx->stream>>>(gs, attn_weights, gs, rows, S, scale);     // grad_scores, scaled
    ctx->launches++;
    if (cudaGetLastError() != cudaSuccess) rc = set_error(ctx, GRILLY_ERR_CUDA, "attention_backward: launch failed");
  }
  if (!rc) rc = launch_bmm(ctx, gs, k, grad_q, nb, S, D, S, false, false, 1.f);                   // grad_q = dS K
  if (!rc) rc = launch_bmm(ctx, gs, q, grad_k, nb, S, D, S, true, false, 1.f);                    // grad_k = dS^T Q
  cudaFreeAsync(gs, ctx->stream);
  return rc;
}

int grilly_adam_update(grilly_ctx* ctx, float* weights, float* gradients, float* moment1, float* moment2, long long n,
                       float learning_rate, float beta1, float beta2, float epsilon, float beta1_t, float beta2_t,
                       int clear_grad) {
  BWD_GUARD(ctx);
  if (!weights || !gradients || !moment1 || !moment2) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "adam_update: null operand");
  if (n <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "adam_update: n must be positive");
  // bias corrections as the reference's CPU branch applies them (none once beta^t has reached 1)
  const float c1 = beta1_t < 1.f ? 1.f / (1.f - beta1_t) : 1.f;
  const float c2 = beta2_t < 1.f ? 1.f / (1.f - beta2_t) : 1.f;
  const int grid = static_cast<int>(std::min<long long>((n + 255) / 256, 16LL * ctx->num_sms));
  adam_update_kernel<<<grid, 256, 0, ctx->stream>>>(weights, gradients, moment1, moment2, n, learning_rate, beta1, beta2, epsilon, c1,
                                                    c2, clear_grad ? 1 : 0);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int grilly_transpose_2d(grilly_ctx* ctx, const float* in, float* out, int rows, int cols) {
  BWD_GUARD(ctx);
  if (!in || !out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "transpose_2d: null operand");
  if (rows <= 0 || cols <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "transpose_2d: sizes must be positive");
  dim3 grid((cols + 31) / 32, (rows + 31) / 32, 1);
  if (grid.y > 65535) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "transpose_2d: more than 2 097 120 rows");
  transpose_kernel<<<grid, 256, 0, ctx->stream>>>(in, out, rows, cols);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

}  // extern "C"
