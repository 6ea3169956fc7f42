// Host launcher for the tcgen05 GEMM: picks the N tile, builds (or reuses) the
// TMA descriptors and launches one persistent CTA per SM.
#include "gemm.cuh"
#include "internal.h"
#include <cstdlib>

namespace gb {

template <int BN, bool kBf16, bool kBMn>
static int launch_one(grilly_ctx* ctx, const void* a, const void* b, GemmArgs& args) {
  using Cfg = GemmCfg<BN>;
  constexpr int ELT = kBf16 ? 2 : 4;
  constexpr int BK = 128 / ELT;
  const int dtype = kBf16 ? TM_BF16 : TM_F32;
  CUtensorMap ta, tb;
  int rc = get_tmap_2d(ctx, dtype, a, args.K, args.M, static_cast<uint64_t>(args.K) * ELT, BK, 128, &ta);
  if (rc) return rc;
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
  args.num_k_blocks = (args.K + BK - 1) / BK;
  args.err = ctx->err_dev;
  auto kern = gemm_tcgen05_kernel<BN, kBf16, kBMn>;
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

// Wave-quantisation estimate: time ~ waves * (tile cost), tile cost ~ BN columns + fixed overhead.
static int pick_bn(int M, int N, int num_sms) {
  const int cands[4] = {256, 192, 128, 64};
  const long long m_tiles = (M + 127) / 128;
  double best = 1e300;
  int best_bn = 128;
  for (int i = 0; i < 4; ++i) {
    const int bn = cands[i];
    const long long n_tiles = (N + bn - 1) / bn;
    const long long tiles = m_tiles * n_tiles;
    const long long waves = (tiles + num_sms - 1) / num_sms;
    const double cost = static_cast<double>(waves) * (bn + 24);
    if (cost < best - 1e-9) { best = cost; best_bn = bn; }
  }
  return best_bn;
}

}  // namespace gb
extern "C" int grilly_gemm_pick_tile(int M, int N, int num_sms) {
  if (M <= 0 || N <= 0 || num_sms <= 0) return GRILLY_ERR_INVALID_ARG;
  return gb::pick_bn(M, N, num_sms);
}
namespace gb {

template <bool kBf16, bool kBMn>
static int dispatch_bn(grilly_ctx* ctx, int bn, const void* a, const void* b, GemmArgs& args) {
  switch (bn) {
    case 256: return launch_one<256, kBf16, kBMn>(ctx, a, b, args);
    case 192: return launch_one<192, kBf16, kBMn>(ctx, a, b, args);
    case 128: return launch_one<128, kBf16, kBMn>(ctx, a, b, args);
    case 64: return launch_one<64, kBf16, kBMn>(ctx, a, b, args);
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
  if (force_bn <= 0) {
    // tuning/debug override of the N tile (64, 128, 192 or 256)
    if (const char* env = getenv("GRILLY_GEMM_BN")) force_bn = atoi(env);
  }
  const int bn = force_bn > 0 ? force_bn : pick_bn(args.M, args.N, ctx->num_sms);
  if (bf16) {
    return b_mn_major ? dispatch_bn<true, true>(ctx, bn, a, b, args) : dispatch_bn<true, false>(ctx, bn, a, b, args);
  }
  return b_mn_major ? dispatch_bn<false, true>(ctx, bn, a, b, args) : dispatch_bn<false, false>(ctx, bn, a, b, args);
}

}  // namespace gb
