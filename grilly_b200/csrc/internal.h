// Host-side internals shared by the translation units of libgrilly_b200.so:
// the context (device, stream, stream-ordered pool, tensor-map cache, status
// word) and the kernel launchers.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/grilly_b200.h"

struct TmapKey {
  const void* ptr;
  uint64_t inner, outer, stride_bytes;
  uint32_t box_inner, box_outer;
  int dtype;
  int swizzle;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && inner == o.inner && outer == o.outer && stride_bytes == o.stride_bytes &&
           box_inner == o.box_inner && box_outer == o.box_outer && dtype == o.dtype && swizzle == o.swizzle;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.ptr);
    auto mix = [&](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix(k.inner); mix(k.outer); mix(k.stride_bytes); mix(k.box_inner); mix(k.box_outer); mix(static_cast<uint64_t>(k.dtype)); mix(static_cast<uint64_t>(k.swizzle));
    return static_cast<size_t>(h);
  }
};

struct grilly_ctx {
  int device = 0;
  int num_sms = 148;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  cudaMemPool_t pool = nullptr;
  int* err_dev = nullptr;       // device status word written by bounded waits
  int* err_host = nullptr;      // pinned mirror
  std::mutex mu;
  std::string last_error;
  // pool statistics
  uint64_t n_alloc = 0, n_free = 0, bytes_in_use = 0, peak_bytes = 0;
  uint64_t pool_hits = 0;       // allocations served without the pool's reserved size growing
  std::unordered_map<void*, size_t> live;
  // tensor-map cache
  std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> tmaps;
  uint64_t tmap_hits = 0, tmap_misses = 0;
  uint64_t launches = 0;
  std::unordered_set<const void*> smem_attr_done;  // kernels whose dynamic-smem limit is already raised
  std::unordered_map<const void*, int> max_clusters;  // CTA-pair kernels: co-resident clusters of 2 on this GPU
  // optional per-kernel-class timing (CUDA events on the launching stream), see grilly_profile_begin/end
  struct ProfRec { int cls; cudaEvent_t a, b; double flops, bytes; };
  cudaEvent_t timer_a = nullptr, timer_b = nullptr;  // grilly_timer_start / grilly_timer_stop
  bool profiling = false;
  std::vector<ProfRec> prof;
  double attn_flops_hint = -1.0;  // set by a caller that knows the true sequence lengths
  // Tuning/debug overrides, read from the environment ONCE in grilly_init (GRILLY_GEMM_GROUP, GRILLY_GEMM_BN,
  // GRILLY_GEMM_PAIR, GRILLY_GEMM_SWAP, GRILLY_ATTN_HPC, GRILLY_ATTN_GENERAL); 0 / -1 = not set
  struct Tuning {
    int gemm_group = 0;      // fast-dimension blocks per group of the tile order
    int gemm_bn = 0;         // forced N tile (64, 128, 192, 256); also rules out the pair kernel
    int gemm_pair = -1;      // 0/1: never/always the CTA-pair kernel
    int gemm_swap = -1;      // 0/1: never/always the swapped orientation for `linear`
    int attn_hpc = 0;        // heads per work unit of the short attention kernel
    int attn_general = 0;    // 1: always the general attention kernel
    int fused_ln = 1;        // 0: linear + LayerNorm as two launches even where the one-kernel form exists
  } tune;
  // RoPE tables, keyed by (S, D, base, scaling)
  struct RopeTable { int S, D; float base, scaling; float* cos_t; float* sin_t; };
  std::vector<RopeTable> rope_tables;
};

namespace gb {

int set_error(grilly_ctx* ctx, int code, const std::string& msg);
#define GB_CUDA_CHECK(ctx, expr)                                                                  \
  do {                                                                                            \
    cudaError_t e__ = (expr);                                                                     \
    if (e__ != cudaSuccess)                                                                       \
      return gb::set_error(ctx, e__ == cudaErrorMemoryAllocation ? GRILLY_ERR_OOM : GRILLY_ERR_CUDA, \
                           std::string(#expr) + ": " + cudaGetErrorString(e__));                  \
  } while (0)

enum { PROF_GEMM = 0, PROF_ATTN = 1, PROF_NORM = 2, PROF_EMBED = 3, PROF_POOL = 4, PROF_OTHER = 5, PROF_NCLASS = 6 };
// Brackets one launch with events when profiling is on; algorithmic FLOPs / bytes are recorded with it.
int prof_begin(grilly_ctx* ctx, int cls, double flops, double bytes);
void prof_end(grilly_ctx* ctx, int idx);

enum { TM_F32 = 0, TM_BF16 = 1 };
enum { TM_SW128 = 0, TM_SW128_ATOM32 = 1, TM_SWNONE = 2, TM_SW64 = 3 };  // 128-byte swizzle of 16-byte chunks, or of 32-byte chunks (tf32 MN-major), none, or the 64-byte swizzle
// 2-D row-major tensor [outer][inner] with a row pitch, 128-byte swizzle, zero fill out of bounds.
int get_tmap_2d(grilly_ctx* ctx, int dtype, const void* ptr, uint64_t inner, uint64_t outer, uint64_t stride_bytes,
                uint32_t box_inner, uint32_t box_outer, CUtensorMap* out, int swizzle = TM_SW128);

struct GemmArgs;
struct GemmLnArgs;
struct AttnArgs;
struct NormArgs;
struct EmbedArgs;
struct PoolArgs;

// gemm.cu
int launch_gemm(grilly_ctx* ctx, bool bf16, bool b_mn_major, const void* a, const void* b, GemmArgs& args, int force_bn);
int launch_gemm_multi(grilly_ctx* ctx, bool bf16, const void* a, const void* b, GemmArgs& args, void* const* extra, int n_extra);
// y = LayerNorm(x W^T + bias + residual) in one kernel (csrc/gemm_ln_pair.cuh); supported for out_features in
// {128, 256, 384, 512}
bool gemm_ln_supported(bool bf16, int N, int K, const GemmLnArgs& a);
int launch_gemm_ln(grilly_ctx* ctx, bool bf16, const void* x, const void* w, GemmLnArgs& args);
// tf32x3.cu: fp32-accurate products through tf32 hi/lo splits (K' = 3K)
int launch_split_rows(grilly_ctx* ctx, const float* x, float* out, float* norm2, long long rows, int dim, int dim_pad,
                      bool lo_second);
int linear_tf32x3(grilly_ctx* ctx, const float* x, const float* w, GemmArgs& args);
int gemm_mnk_tf32x3(grilly_ctx* ctx, const float* a, const float* b, GemmArgs& args);
// api.cu: Linear(Norm(x)) shared by the allocating and the no-allocation entry points
int layernorm_linear_impl(grilly_ctx* ctx, const void* x, const void* wf, const float* col_sum, const float* bias_f, void* y,
                          float* mean, float* rstd, int M, int N, int K, float eps, int norm_mode, int act, int precision,
                          int flags, bool may_allocate);
// attention.cu
int launch_attention(grilly_ctx* ctx, bool bf16, const void* q, const void* k, const void* v, long long ld_q, long long ld_k,
                     long long ld_v, long long total_rows, AttnArgs& args);
// rowops.cu
int launch_norm(grilly_ctx* ctx, const NormArgs& a);
int launch_softmax(grilly_ctx* ctx, const float* x, float* y, long long rows, int cols);
int launch_eltwise(grilly_ctx* ctx, int op, const float* a, const float* b, float* y, long long n, int half);
int launch_act_params(grilly_ctx* ctx, int op, const float* a, float* y, long long n, float p0, float p1);
int launch_round_tf32(grilly_ctx* ctx, const float* x, float* y, long long n);
int launch_f32_to_bf16(grilly_ctx* ctx, const float* x, void* y, long long n);
int launch_bf16_to_f32(grilly_ctx* ctx, const void* x, float* y, long long n);
int launch_gather(grilly_ctx* ctx, const int* ids, const float* table, float* out, long long n, int vocab, int F);
int launch_embed(grilly_ctx* ctx, const EmbedArgs& a);
int launch_pool(grilly_ctx* ctx, const PoolArgs& a);
int launch_fold_ln(grilly_ctx* ctx, const float* w, const float* gamma, const float* beta, const float* bias, void* wf,
                   float* col_sum, float* bias_f, int N, int K, bool bf16);
int get_rope_table(grilly_ctx* ctx, int S, int D, float base, float scaling, const float** cos_t, const float** sin_t);
int launch_attn_scores(grilly_ctx* ctx, const float* q, const float* k, float* scores, int B, int S, int H, int D, float scale);
int launch_attn_mask(grilly_ctx* ctx, float* scores, const float* mask, int B, int H, int S, int use_causal, float mask_value);
int launch_attn_output(grilly_ctx* ctx, const float* w, const float* v, float* out, int B, int Sq, int Sk, int H, int D, int causal);
int launch_rope_rows(grilly_ctx* ctx, bool bf16, const void* src, void* dst, long long rows, long long pitch, int H, int D,
                     int S, const int* cu_seqlens, int B, const float* cos_t, const float* sin_t, int style);
int launch_rope_apply(grilly_ctx* ctx, const float* x, float* y, const float* cos_t, const float* sin_t,
                      const int* position_ids, int B, int S, int H, int D, int style);

}  // namespace gb
