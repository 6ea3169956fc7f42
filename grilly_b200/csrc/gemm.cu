// Host launcher for the tcgen05 GEMM: picks the N tile, builds (or reuses) the
// TMA descriptors and launches one persistent CTA per SM.
#include "gemm.cuh"
#include "gemm_pair.cuh"
#include "gemm_ln_pair.cuh"
#include "internal.h"

namespace gb {

template <int BN, bool kBf16, bool kBMn, bool kSwap>
static int launch_one(grilly_ctx* ctx, const void* a, const void* b, GemmArgs& args) {
  using Cfg = GemmCfg<BN>;
  constexpr int ELT = kBf16 ? 2 : 4;
  constexpr int BK = 128 / ELT;
  static_assert(!(kBMn && kSwap), "the swapped orientation is for the K-major weight layout only");
  const int dtype = kBf16 ? TM_BF16 : TM_F32;
  CUtensorMap ta, tb;
  int rc;
  if (kSwap) {
    // 128-row operand = weights W[N][K]; BN-row operand = activations x[M][K]
    if ((rc = get_tmap_2d(ctx, dtype, b, args.K, args.N, static_cast<uint64_t>(args.K) * ELT, BK, 128, &ta))) return rc;
    if ((rc = get_tmap_2d(ctx, dtype, a, args.K, args.M, static_cast<uint64_t>(args.K) * ELT, BK, BN, &tb))) return rc;
    args.num_m_tiles = (args.N + 127) / 128;
    args.num_n_tiles = (args.M + BN - 1) / BN;
  } else {
    if ((rc = get_tmap_2d(ctx, dtype, a, args.K, args.M, static_cast<uint64_t>(args.K) * ELT, BK, 128, &ta))) return rc;
    if (kBMn) {
      // B is [K][N] row-major: boxes of 128 B along N by BK k-rows
      rc = get_tmap_2d(ctx, dtype, b, args.N, args.K, static_cast<uint64_t>(args.N) * ELT, 128 / ELT, BK, &tb,
                       kBf16 ? TM_SW128 : TM_SW128_ATOM32);
    } else {
      // B is [N][K] row-major: boxes of 128 B along K by BN rows
      rc = get_tmap_2d(ctx, dtype, b, args.K, args.N, static_cast<uint64_t>(args.K) * ELT, BK, BN, &tb);
    }
    if (rc) return rc;
    args.num_m_tiles = (args.M + 127) / 128;
    args.num_n_tiles = (args.N + BN - 1) / BN;
  }
  args.num_k_blocks = (args.K + BK - 1) / BK;
  // co-running tiles (one per SM) load group*fast_rows + (SMs/group)*slow_rows operand rows per k-block: smallest
  // near group = sqrt(SMs * slow_rows / fast_rows)
  args.tile_group = ctx->tune.gemm_group > 0 ? ctx->tune.gemm_group : (kSwap ? 16 : 8);
  args.err = ctx->err_dev;
  auto kern = gemm_tcgen05_kernel<BN, kBf16, kBMn, kSwap>;
  if (!ctx->smem_attr_done.count(reinterpret_cast<const void*>(kern))) {
    GB_CUDA_CHECK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    ctx->smem_attr_done.insert(reinterpret_cast<const void*>(kern));
  }
  const int tiles = args.num_m_tiles * args.num_n_tiles;
  const int grid = tiles < ctx->num_sms ? tiles : ctx->num_sms;
  const double out_cols = args.swiglu_pairs ? args.N / 2.0 : args.N;
  const double bytes = static_cast<double>(ELT) * (static_cast<double>(args.M) * args.K + static_cast<double>(args.N) * args.K) +
                       (args.bias ? 4.0 * args.N : 0.0) + static_cast<double>(args.M) * out_cols * (args.out_bf16 ? 2.0 : 4.0) +
                       (args.residual ? 4.0 * args.M * out_cols : 0.0);
  const int pi = prof_begin(ctx, PROF_GEMM, 2.0 * args.M * static_cast<double>(args.N) * args.K, bytes);
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, ctx->stream>>>(ta, tb, args);
  prof_end(ctx, pi);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

// CTA-pair variant (gemm_pair.cuh), tiles of 256 x 256. kBMn = false: `linear`, x = tokens [M][K], w = weights [N][K],
// both K-major. kBMn = true: `gemm_mnk`, x = A [M][K], w = B [K][N] row-major.
template <bool kBf16, bool kBMn>
static int launch_pair(grilly_ctx* ctx, const void* x, const void* w, GemmArgs& args) {
  using Cfg = GemmPairCfg;
  constexpr int ELT = kBf16 ? 2 : 4;
  constexpr int BK = 128 / ELT;
  const int dtype = kBf16 ? TM_BF16 : TM_F32;
  CUtensorMap tw, tx;   // tw: the MMA's M operand, tx: its N operand
  int rc;
  if (kBMn) {
    if ((rc = get_tmap_2d(ctx, dtype, x, args.K, args.M, static_cast<uint64_t>(args.K) * ELT, BK, 128, &tw))) return rc;
    if ((rc = get_tmap_2d(ctx, dtype, w, args.N, args.K, static_cast<uint64_t>(args.N) * ELT, 128 / ELT, BK, &tx,
                          kBf16 ? TM_SW128 : TM_SW128_ATOM32))) return rc;
    args.num_m_tiles = (args.M + Cfg::TILE - 1) / Cfg::TILE;
    args.num_n_tiles = (args.N + Cfg::TILE - 1) / Cfg::TILE;
  } else {
    if ((rc = get_tmap_2d(ctx, dtype, w, args.K, args.N, static_cast<uint64_t>(args.K) * ELT, BK, 128, &tw))) return rc;
    if ((rc = get_tmap_2d(ctx, dtype, x, args.K, args.M, static_cast<uint64_t>(args.K) * ELT, BK, 128, &tx))) return rc;
    args.num_m_tiles = (args.N + Cfg::TILE - 1) / Cfg::TILE;
    args.num_n_tiles = (args.M + Cfg::TILE - 1) / Cfg::TILE;
  }
  args.num_k_blocks = (args.K + BK - 1) / BK;
  args.tile_group = ctx->tune.gemm_group > 0 ? ctx->tune.gemm_group : 8;
  args.err = ctx->err_dev;
  auto kern = gemm_tcgen05_pair_kernel<kBf16, kBMn>;
  const void* key = reinterpret_cast<const void*>(kern);
  if (!ctx->smem_attr_done.count(key)) {
    GB_CUDA_CHECK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    ctx->smem_attr_done.insert(key);
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(GEMM_PAIR_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = ctx->stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  auto found = ctx->max_clusters.find(key);
  if (found == ctx->max_clusters.end()) {
    int n = 0;
    cfg.gridDim = dim3(2 * (ctx->num_sms / 2), 1, 1);
    GB_CUDA_CHECK(ctx, cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    if (n <= 0) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "gemm: no CTA pair fits on this GPU");
    found = ctx->max_clusters.emplace(key, n).first;
  }
  const int tiles = args.num_m_tiles * args.num_n_tiles;
  const int pairs = tiles < found->second ? tiles : found->second;
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  const double out_cols = args.swiglu_pairs ? args.N / 2.0 : args.N;
  const double bytes = static_cast<double>(ELT) * (static_cast<double>(args.M) * args.K + static_cast<double>(args.N) * args.K) +
                       (args.bias ? 4.0 * args.N : 0.0) + static_cast<double>(args.M) * out_cols * (args.out_bf16 ? 2.0 : 4.0) +
                       (args.residual ? 4.0 * args.M * out_cols : 0.0);
  const int pi = prof_begin(ctx, PROF_GEMM, 2.0 * args.M * static_cast<double>(args.N) * args.K, bytes);
  GB_CUDA_CHECK(ctx, cudaLaunchKernelEx(&cfg, kern, tw, tx, args));
  prof_end(ctx, pi);
  ctx->launches++;
  return GRILLY_OK;
}

// A pair tile covers 256 features: worth it when the GEMM is large enough to be bound by operand traffic and the
// last feature block is not mostly padding (384 features would waste a quarter of the MMAs).
static bool pick_pair(int M, int N, bool b_mn_major) {
  if (M < 1024 || N < 256) return false;
  const int padded = (N + 255) / 256 * 256;
  if (padded * 8 > N * 9) return false;
  // gemm_mnk tiles the rows of C in 256s as well
  return !b_mn_major || ((M + 255) / 256 * 256) * 8 <= M * 9;
}

// One tcgen05.mma takes about the same time for any N up to 256, so a tile costs the same whatever its width:
// take the widest tile that is not mostly padding. The swapped orientation (weights as the 128-row operand,
// tokens as the MMA's N) is used for `linear` whenever the output is wide enough to fill 128 feature rows.
static bool pick_swap(int N, bool b_mn_major) { return !b_mn_major && N >= 96; }
static int pick_bn(int cols) { return cols <= 64 ? 64 : cols <= 128 ? 128 : cols <= 192 ? 192 : 256; }

}  // namespace gb
extern "C" int grilly_gemm_pick_tile(int M, int N, int num_sms) {
  if (M <= 0 || N <= 0 || num_sms <= 0) return GRILLY_ERR_INVALID_ARG;
  return gb::pick_bn(gb::pick_swap(N, false) ? M : N);
}
namespace gb {

template <bool kBf16, bool kBMn, bool kSwap>
static int dispatch_bn(grilly_ctx* ctx, int bn, const void* a, const void* b, GemmArgs& args) {
  switch (bn) {
    case 256: return launch_one<256, kBf16, kBMn, kSwap>(ctx, a, b, args);
    case 192: return launch_one<192, kBf16, kBMn, kSwap>(ctx, a, b, args);
    case 128: return launch_one<128, kBf16, kBMn, kSwap>(ctx, a, b, args);
    case 64: return launch_one<64, kBf16, kBMn, kSwap>(ctx, a, b, args);
    default: return set_error(ctx, GRILLY_ERR_INVALID_ARG, "gemm: N tile must be 64, 128, 192 or 256");
  }
}

int launch_gemm(grilly_ctx* ctx, bool bf16, bool b_mn_major, const void* a, const void* b, GemmArgs& args, int force_bn) {
  if (args.M <= 0 || args.N <= 0 || args.K <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "gemm: M, N, K must be positive");
  const int elt = bf16 ? 2 : 4;
  if ((static_cast<long long>(args.K) * elt) % 16 != 0)
    return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "gemm: K * element size must be a multiple of 16 bytes (pad K)");
  if (b_mn_major && (static_cast<long long>(args.N) * elt) % 16 != 0)
    return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "gemm_mnk: N * element size must be a multiple of 16 bytes (pad N)");
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15))
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "gemm: operands must be 16-byte aligned");
  if (args.swiglu_pairs && (args.N & 1)) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "gemm: SwiGLU pairs need an even N");
  // tuning/debug override of the tile width (64, 128, 192 or 256); a forced width also rules out the pair kernel
  if (force_bn <= 0) force_bn = ctx->tune.gemm_bn;
  bool pair = pick_pair(args.M, args.N, b_mn_major);
  if (ctx->tune.gemm_pair >= 0) pair = ctx->tune.gemm_pair != 0;
  if (pair && force_bn <= 0) {
    if (b_mn_major) return bf16 ? launch_pair<true, true>(ctx, a, b, args) : launch_pair<false, true>(ctx, a, b, args);
    return bf16 ? launch_pair<true, false>(ctx, a, b, args) : launch_pair<false, false>(ctx, a, b, args);
  }
  bool swap = pick_swap(args.N, b_mn_major);
  if (ctx->tune.gemm_swap >= 0) swap = !b_mn_major && ctx->tune.gemm_swap != 0;
  const int bn = force_bn > 0 ? force_bn : pick_bn(swap ? args.M : args.N);
  if (bf16) {
    if (b_mn_major) return dispatch_bn<true, true, false>(ctx, bn, a, b, args);
    return swap ? dispatch_bn<true, false, true>(ctx, bn, a, b, args) : dispatch_bn<true, false, false>(ctx, bn, a, b, args);
  }
  if (b_mn_major) return dispatch_bn<false, true, false>(ctx, bn, a, b, args);
  return swap ? dispatch_bn<false, false, true>(ctx, bn, a, b, args) : dispatch_bn<false, false, false>(ctx, bn, a, b, args);
}

// gemm_mnk whose fp32 result goes to args.out and to n_extra further matrices of the same pitch (device pointers,
// possibly peer-mapped). The list is placed in constant memory in stream order before the launch; the launch is
// marked (GemmArgs::multi_out) as the one that reads it.
int launch_gemm_multi(grilly_ctx* ctx, bool bf16, const void* a, const void* b, GemmArgs& args, void* const* extra, int n_extra) {
  if (n_extra < 0 || n_extra > 7) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "gemm_mnk_multi: at most 8 destinations");
  if (n_extra > 0 && (args.N % 32 != 0 || args.out_bf16))
    return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "gemm_mnk_multi: fp32 output and N a multiple of 32 are required");
  GemmExtraOut h{};
  h.n = n_extra;
  for (int i = 0; i < n_extra; ++i) h.p[i] = extra[i];
  if (n_extra > 0) GB_CUDA_CHECK(ctx, cudaMemcpyToSymbolAsync(g_gemm_extra_out, &h, sizeof(h), 0, cudaMemcpyHostToDevice, ctx->stream));
  args.multi_out = n_extra;   // only this launch reads the list
  return launch_gemm(ctx, bf16, true, a, b, args, 0);
}

// ---- y = LayerNorm(x W^T + bias + residual) in one kernel (gemm_ln_pair.cuh)
bool gemm_ln_supported(bool bf16, int N, int K, const GemmLnArgs& a) {
  const int elt = bf16 ? 2 : 4;
  if (N != 128 && N != 256 && N != 384 && N != 512) return false;          // whole rows in one CTA's tensor memory
  if ((static_cast<long long>(K) * elt) % 16 != 0) return false;
  if (a.out_bf16 && !bf16) return false;
  if (a.residual && ((a.ld_res * elt) % 16 != 0 || (reinterpret_cast<uintptr_t>(a.residual) & 15))) return false;
  if ((reinterpret_cast<uintptr_t>(a.out) & 15) || (a.ld_out * (a.out_bf16 ? 2 : 4)) % 16 != 0) return false;
  return true;
}

// The shared-MMA form (gemm_ln_pair.cuh): 256 token rows per CTA pair, whole rows per CTA.
template <int N, int SUB, int BUFS, bool kBf16>
static int launch_ln_pair_cfg(grilly_ctx* ctx, const void* x, const void* w, GemmLnArgs& args) {
  using Cfg = GemmLnPairCfg<N, SUB, BUFS, kBf16>;
  constexpr int ELT = kBf16 ? 2 : 4;
  constexpr int BK = 128 / ELT;
  const int dtype = kBf16 ? TM_BF16 : TM_F32;
  CUtensorMap ta, tb, tr, to;
  int rc;
  if ((rc = get_tmap_2d(ctx, dtype, x, args.K, args.M, static_cast<uint64_t>(args.K) * ELT, BK, 128, &ta))) return rc;
  if ((rc = get_tmap_2d(ctx, dtype, w, args.K, args.N, static_cast<uint64_t>(args.K) * ELT, BK, Cfg::BH, &tb))) return rc;
  // residual boxes of 32 rows x 32 columns: fp32 rows are 128 bytes (swizzled like the output), bf16 rows 64 bytes (plain)
  if (!args.residual) tr = ta;
  else if ((rc = get_tmap_2d(ctx, dtype, args.residual, args.N, args.M, static_cast<uint64_t>(args.ld_res) * ELT, 32, 32, &tr,
                             kBf16 ? TM_SWNONE : TM_SW128))) return rc;
  // output boxes of 32 rows x 32 columns: fp32 rows are 128 bytes (128-byte swizzle), bf16 rows 64 bytes (64-byte swizzle)
  if (args.out_bf16) {
    if ((rc = get_tmap_2d(ctx, TM_BF16, args.out, args.N, args.M, static_cast<uint64_t>(args.ld_out) * 2, 32, 32, &to, TM_SW64))) return rc;
  } else if ((rc = get_tmap_2d(ctx, TM_F32, args.out, args.N, args.M, static_cast<uint64_t>(args.ld_out) * 4, 32, 32, &to))) return rc;
  args.num_tiles = (args.M + 255) / 256;
  args.num_k_blocks = (args.K + BK - 1) / BK;
  args.err = ctx->err_dev;
  auto kern = gemm_rowln_pair_kernel<N, SUB, BUFS, kBf16>;
  const void* key = reinterpret_cast<const void*>(kern);
  if (!ctx->smem_attr_done.count(key)) {
    GB_CUDA_CHECK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    ctx->smem_attr_done.insert(key);
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = ctx->stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  auto found = ctx->max_clusters.find(key);
  if (found == ctx->max_clusters.end()) {
    int n = 0;
    cfg.gridDim = dim3(2 * (ctx->num_sms / 2), 1, 1);
    GB_CUDA_CHECK(ctx, cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    if (n <= 0) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "linear_layernorm: no CTA pair fits on this GPU");
    found = ctx->max_clusters.emplace(key, n).first;
  }
  const int pairs = args.num_tiles < found->second ? args.num_tiles : found->second;
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  const double mn = static_cast<double>(args.M) * args.N;
  const double bytes = static_cast<double>(ELT) * (static_cast<double>(args.M) * args.K + static_cast<double>(args.N) * args.K) +
                       12.0 * args.N + mn * (args.out_bf16 ? 2.0 : 4.0) + (args.residual ? mn * ELT : 0.0);
  const int pi = prof_begin(ctx, PROF_GEMM, 2.0 * mn * args.K, bytes);
  GB_CUDA_CHECK(ctx, cudaLaunchKernelEx(&cfg, kern, ta, tb, tr, to, args));
  prof_end(ctx, pi);
  ctx->launches++;
  return GRILLY_OK;
}

template <bool kBf16>
static int launch_ln_pair(grilly_ctx* ctx, const void* x, const void* w, GemmLnArgs& args) {
  // 384 features: three epilogue warps per TMEM lane quadrant with one staging buffer each leave room for a fourth
  // operand stage (measured best for K = 384 and K = 1536 alike)
  switch (args.N) {
    case 128: return launch_ln_pair_cfg<128, 2, 2, kBf16>(ctx, x, w, args);
    case 256: return launch_ln_pair_cfg<256, 2, 2, kBf16>(ctx, x, w, args);
    case 384: return launch_ln_pair_cfg<384, 3, 1, kBf16>(ctx, x, w, args);
    default: return launch_ln_pair_cfg<512, 2, 2, kBf16>(ctx, x, w, args);
  }
}

int launch_gemm_ln(grilly_ctx* ctx, bool bf16, const void* x, const void* w, GemmLnArgs& args) {
  if (args.M <= 0 || args.N <= 0 || args.K <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "linear_layernorm: M, N, K must be positive");
  if (!gemm_ln_supported(bf16, args.N, args.K, args))
    return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "linear_layernorm: the one-kernel form needs out_features in {128, 256, 384, 512} and 16-byte aligned rows");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "linear_layernorm: operands must be 16-byte aligned");
  return bf16 ? launch_ln_pair<true>(ctx, x, w, args) : launch_ln_pair<false>(ctx, x, w, args);
}

}  // namespace gb
