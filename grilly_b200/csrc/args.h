// Plain argument structs shared by the kernels and the host code that launches them.
#pragma once

namespace gb {

enum : int { ACT_NONE = 0, ACT_GELU_TANH = 1, ACT_SILU = 2, ACT_RELU = 3 };
enum : int { ROPE_NONE = 0, ROPE_INTERLEAVED = 1, ROPE_ROTATE_HALF = 2 };
enum : int { NORM_LAYER = 0, NORM_RMS = 1 };
enum : int { DIST_NONE = 0, DIST_L2 = 1, DIST_COSINE = 2, DIST_DOT = 3 };
enum : int { ELT_GELU = 1, ELT_SILU = 2, ELT_RELU = 3, ELT_ADD = 4, ELT_SWIGLU = 5, ELT_GCU = 6, ELT_ROSWISH = 7 };

struct GemmArgs {
  int M, N, K;
  int num_m_tiles, num_n_tiles, num_k_blocks;
  int tile_group;         // fast-dimension blocks per group of the tile order (see tile_coords)
  int multi_out;          // gemm_mnk only: number of FURTHER destinations (in g_gemm_extra_out) this launch stores to;
                          // 0 for every other launch. Sits in the padding before the pointers: the struct does not grow.
  const float* bias;      // [N] (pre-activation) or null
  const float* residual;  // [M][ld_res] fp32, added after the activation, or null
  long long ld_res;
  int residual_bf16;      // the residual tensor is bf16 instead of fp32
  void* out;              // [M][ld_out] fp32 or bf16
  long long ld_out;
  int out_bf16;
  int act;
  int round_tf32;         // round fp32 results to the nearest tf32 value before storing
  int swiglu_pairs;       // columns come as (gate, up) pairs: out[:, c/2] = gate * silu(up)
  // LayerNorm folded into the GEMM (weights pre-scaled by gamma):
  //   y = rstd[r] * (acc - mean[r] * col_sum[c]) + bias[c]
  const float* row_mean;  // null for RMSNorm (no mean term)
  const float* row_rstd;  // null when no normalisation is folded in
  const float* col_sum;
  int* err;               // device status word
};

// y = LayerNorm(x W^T + bias + residual) * gamma + beta in one kernel (gemm_ln_pair.cuh)
struct GemmLnArgs {
  int M, N, K;
  int num_tiles, num_k_blocks;
  const float* bias;       // [N] or null
  const void* residual;    // [M][ld_res] fp32 (tf32 mode) or bf16 (bf16 mode), or null
  long long ld_res;
  const float* gamma;      // [N] or null (= 1)
  const float* beta;       // [N] or null (= 0)
  float eps;
  void* out;               // [M][ld_out] fp32 or bf16
  long long ld_out;
  int out_bf16;            // bf16 mode only
  int round_tf32;
  int* err;
};

struct AttnArgs {
  int B, S, H, D;
  const int* cu_seqlens;   // [B+1] packed rows, or null for the padded layout
  const float* key_mask;   // [B][S], 1 = keep (< 0.5 = masked), padded layout only, or null
  float scale;
  int causal;
  void* out;               // [rows][ld_out], fp32 or bf16
  long long ld_out;
  int out_bf16;
  int round_tf32;
  int rope_style;
  const float* rope_cos;   // [S][D/2] tables (position-major), or null
  const float* rope_sin;
  int rope_k_done;         // K is already rotated (pre-pass): the kernel rotates Q only
  int* err;
};

struct NormArgs {
  const float* x;         // [rows][F]
  const float* residual;  // [rows][F] added to x before normalising, or null
  const float* gamma;     // [F] or null (= 1)
  const float* beta;      // [F] or null (= 0)
  void* y;                // [rows][F] fp32 or bf16, may be null (statistics only)
  float* mean_out;        // [rows] or null
  float* rstd_out;        // [rows] or null
  int rows, F;
  float eps;
  int mode;               // NORM_LAYER: gamma (x-mean) rstd + beta (biased variance); NORM_RMS: x / sqrt(mean(x^2)+eps) gamma
  int out_bf16;
  int round_tf32;
  int reverse;            // walk the rows from the last to the first (the rows a producer wrote last are still in L2)
  int x_bf16;             // x (and residual) are bf16 instead of fp32
  unsigned* ratio_max;    // optional: atomic max over rows of |mean| * rstd as fp32 bits (the cancellation measure of
                          // the folded LayerNorm->linear form); the caller zeroes it first
};

struct EmbedArgs {
  const int* ids;          // [B][S] token ids
  const int* cu_seqlens;   // [B+1]: packed output row of sequence b's first token; null = padded output (row b*S+s)
  const float* word;       // [vocab][F]
  const float* pos;        // [max_pos][F] or null
  const float* type0;      // [F] token-type row 0 or null
  const float* gamma;      // embedding LayerNorm, or null to skip the norm
  const float* beta;
  float* out;              // [rows][F]
  int B, S, F, vocab, max_pos;
  float eps;
  int round_tf32;
  int out_bf16;            // write bf16 rows (bf16 encoder mode)
  long long rows_hint;     // valid tokens of the batch if the caller knows them (for the byte count of the profile), else 0
};

struct PoolArgs {
  const float* x;         // [rows][F]
  const float* mask;      // [B][S] (padded layout): position counts when mask > 0.5; or null
  const int* cu_seqlens;  // [B+1] (packed layout): all rows of the sequence count; or null
  float* out;             // [B][F]
  int B, S, F;
  int normalize;          // 1: divide the pooled vector by (||v||_2 + 1e-8)
  int cls;                // 1: take the sequence's first token instead of the mean (CLS pooling)
  long long rows_hint;    // valid tokens of the batch if the caller knows them (for the byte count of the profile), else 0
};

}  // namespace gb
