// Host launcher for the tcgen05 GEMM: picks the N tile, builds (or reuses) the
// TMA descriptors and launches one persistent CTA per SM.
#include "gemm.cuh"
#include "internal.h"
#include <cstdlib>

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
  bool swap = pick_swap(args.N, b_mn_major);
  if (const char* env = getenv("GRILLY_GEMM_SWAP")) swap = !b_mn_major && atoi(env) != 0;  // tuning/debug override
  if (force_bn <= 0) {
    // tuning/debug override of the tile width (64, 128, 192 or 256)
    if (const char* env = getenv("GRILLY_GEMM_BN")) force_bn = atoi(env);
  }
  const int bn = force_bn > 0 ? force_bn : pick_bn(swap ? args.M : args.N);
  if (bf16) {
    if (b_mn_major) return dispatch_bn<true, true, false>(ctx, bn, a, b, args);
    return swap ? dispatch_bn<true, false, true>(ctx, bn, a, b, args) : dispatch_bn<true, false, false>(ctx, bn, a, b, args);
  }
  if (b_mn_major) return dispatch_bn<false, true, false>(ctx, bn, a, b, args);
  return swap ? dispatch_bn<false, false, true>(ctx, bn, a, b, args) : dispatch_bn<false, false, false>(ctx, bn, a, b, args);
}

}  // namespace gb
