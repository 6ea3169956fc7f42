// Host launcher for the tcgen05 flash-attention kernel.
#include <algorithm>
#include "attention.cuh"
#include "attention_short.cuh"
#include "internal.h"

namespace gb {

template <int D, bool kBf16>
static int launch_one(grilly_ctx* ctx, const void* q, const void* k, const void* v, long long ld_q, long long ld_k,
                      long long ld_v, long long total_rows, AttnArgs& args) {
  using Cfg = AttnCfg<D, kBf16>;
  constexpr int ELT = kBf16 ? 2 : 4;
  const int dtype = kBf16 ? TM_BF16 : TM_F32;
  const uint64_t width = static_cast<uint64_t>(args.H) * D;  // columns reachable from each base pointer
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = get_tmap_2d(ctx, dtype, q, width, total_rows, ld_q * ELT, 128 / ELT, ATTN_TILE, &tq))) return rc;
  if ((rc = get_tmap_2d(ctx, dtype, k, width, total_rows, ld_k * ELT, 128 / ELT, ATTN_TILE, &tk))) return rc;
  // V is consumed as the MN-major operand of P V: tf32 needs the 32-byte-atom swizzle
  if ((rc = get_tmap_2d(ctx, dtype, v, width, total_rows, ld_v * ELT, 128 / ELT, ATTN_TILE, &tv,
                        kBf16 ? TM_SW128 : TM_SW128_ATOM32))) return rc;
  args.err = ctx->err_dev;
  auto kern = flash_attn_tcgen05_kernel<D, kBf16>;
  if (!ctx->smem_attr_done.count(reinterpret_cast<const void*>(kern))) {
    GB_CUDA_CHECK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    ctx->smem_attr_done.insert(reinterpret_cast<const void*>(kern));
  }
  dim3 grid((args.S + ATTN_TILE - 1) / ATTN_TILE, args.H, args.B);
  // algorithmic work: 4*D FLOPs per (query, key) pair (half under a causal mask), q/k/v read + out written once
  double flops = ctx->attn_flops_hint >= 0.0 ? ctx->attn_flops_hint
                                             : 4.0 * args.B * args.H * static_cast<double>(args.S) * args.S * D * (args.causal ? 0.5 : 1.0);
  ctx->attn_flops_hint = -1.0;
  const double bytes = static_cast<double>(total_rows) * args.H * D * (3.0 * ELT + (args.out_bf16 ? 2.0 : 4.0));
  const int pi = prof_begin(ctx, PROF_ATTN, flops, bytes);
  kern<<<grid, ATTN_THREADS, Cfg::SMEM_BYTES, ctx->stream>>>(tq, tk, tv, args);
  prof_end(ctx, pi);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

template <int D, bool kBf16>
static int launch_short(grilly_ctx* ctx, const void* q, const void* k, const void* v, long long ld_q, long long ld_k,
                        long long ld_v, long long total_rows, AttnArgs& args) {
  using Cfg = AttnShortCfg<D, kBf16>;
  constexpr int ELT = kBf16 ? 2 : 4;
  const int dtype = kBf16 ? TM_BF16 : TM_F32;
  const uint64_t width = static_cast<uint64_t>(args.H) * D;
  AttnShortMaps maps;
  int rc;
  for (int i = 0; i < 4; ++i) {
    const uint32_t rows = 32u * (i + 1);
    if ((rc = get_tmap_2d(ctx, dtype, q, width, total_rows, ld_q * ELT, 128 / ELT, rows, &maps.q[i]))) return rc;
    if ((rc = get_tmap_2d(ctx, dtype, k, width, total_rows, ld_k * ELT, 128 / ELT, rows, &maps.k[i]))) return rc;
    if ((rc = get_tmap_2d(ctx, dtype, v, width, total_rows, ld_v * ELT, 128 / ELT, rows, &maps.v[i],
                          kBf16 ? TM_SW128 : TM_SW128_ATOM32))) return rc;
  }
  args.err = ctx->err_dev;
  auto kern = flash_attn_short_kernel<D, kBf16>;
  if (!ctx->smem_attr_done.count(reinterpret_cast<const void*>(kern))) {
    GB_CUDA_CHECK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    ctx->smem_attr_done.insert(reinterpret_cast<const void*>(kern));
  }
  // a unit is one sequence with all its heads, split into head groups while there are fewer than about six units per
  // slot (sequences differ in length, so a slot's last unit decides how long the tail of the launch is)
  int hpc = args.H;
  while (hpc > 1 && static_cast<long long>(args.B) * ((args.H + hpc - 1) / hpc) < 6LL * Cfg::NSLOT * ctx->num_sms) hpc = (hpc + 1) / 2;
  if (ctx->tune.attn_hpc > 0) hpc = ctx->tune.attn_hpc;   // heads per unit, for tuning runs
  hpc = (hpc + Cfg::HPR - 1) / Cfg::HPR * Cfg::HPR;   // heads that share a loaded row chunk stay in one unit
  const int head_groups = (args.H + hpc - 1) / hpc;
  const long long units = static_cast<long long>(args.B) * head_groups;
  if (units > 2147483647LL) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "attention: too many (sequence, head group) units");
  const int ctas = static_cast<int>(std::min<long long>(ctx->num_sms, (units + Cfg::NSLOT - 1) / Cfg::NSLOT));
  double flops = ctx->attn_flops_hint >= 0.0 ? ctx->attn_flops_hint : 4.0 * args.B * args.H * static_cast<double>(args.S) * args.S * D;
  ctx->attn_flops_hint = -1.0;
  const double bytes = static_cast<double>(total_rows) * args.H * D * (3.0 * ELT + (args.out_bf16 ? 2.0 : 4.0));
  int* counter = ctx->err_dev + 1;                     // the slots of all CTAs take their units from this counter
  GB_CUDA_CHECK(ctx, cudaMemsetAsync(counter, 0, sizeof(int), ctx->stream));
  const int pi = prof_begin(ctx, PROF_ATTN, flops, bytes);
  kern<<<ctas, Cfg::THREADS, Cfg::SMEM_BYTES, ctx->stream>>>(maps, args, hpc, head_groups, static_cast<int>(units), counter);
  prof_end(ctx, pi);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

int launch_attention(grilly_ctx* ctx, bool bf16, const void* q, const void* k, const void* v, long long ld_q, long long ld_k,
                     long long ld_v, long long total_rows, AttnArgs& args) {
  const int elt = bf16 ? 2 : 4;
  if (args.B <= 0 || args.S <= 0 || args.H <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention: B, S, H must be positive");
  if ((ld_q * elt) % 16 != 0 || (ld_k * elt) % 16 != 0 || (ld_v * elt) % 16 != 0) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "attention: row pitch must be a multiple of 16 bytes");
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15))
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention: q, k, v must be 16-byte aligned");
  // the kernels store bf16 results as 32-bit pairs and fp32 results as 16-byte vectors where the pitch allows it
  if (!args.out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention: null output");
  if (args.out_bf16 && ((args.ld_out & 1) || (reinterpret_cast<uintptr_t>(args.out) & 3)))
    return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "attention: a bf16 output needs an even row pitch and a 4-byte aligned base");
  if (!args.out_bf16 && (reinterpret_cast<uintptr_t>(args.out) & 3))
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "attention: the output must be 4-byte aligned");
  // every sequence fits one key tile and nothing needs per-tile state: the multi-head kernel
  const bool short_ok = args.S <= ATTN_TILE && !args.causal && args.rope_style == ROPE_NONE && args.scale > 0.f &&
                        args.B <= 2147483647 && !ctx->tune.attn_general;
  if (short_ok) {
    if (!bf16 && args.D == 32) return launch_short<32, false>(ctx, q, k, v, ld_q, ld_k, ld_v, total_rows, args);
    if (!bf16 && args.D == 64) return launch_short<64, false>(ctx, q, k, v, ld_q, ld_k, ld_v, total_rows, args);
    if (bf16 && args.D == 32) return launch_short<32, true>(ctx, q, k, v, ld_q, ld_k, ld_v, total_rows, args);
    if (bf16 && args.D == 64) return launch_short<64, true>(ctx, q, k, v, ld_q, ld_k, ld_v, total_rows, args);
    if (bf16 && args.D == 128) return launch_short<128, true>(ctx, q, k, v, ld_q, ld_k, ld_v, total_rows, args);
  }
  if (args.H > 65535 || args.B > 65535) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "attention: B and H are limited to 65535 for sequences longer than 128");
  if (!bf16 && args.D == 32) return launch_one<32, false>(ctx, q, k, v, ld_q, ld_k, ld_v, total_rows, args);
  if (!bf16 && args.D == 64) return launch_one<64, false>(ctx, q, k, v, ld_q, ld_k, ld_v, total_rows, args);
  if (!bf16 && args.D == 96) return launch_one<96, false>(ctx, q, k, v, ld_q, ld_k, ld_v, total_rows, args);
  if (!bf16 && args.D == 128) return launch_one<128, false>(ctx, q, k, v, ld_q, ld_k, ld_v, total_rows, args);
  if (bf16 && args.D == 64) return launch_one<64, true>(ctx, q, k, v, ld_q, ld_k, ld_v, total_rows, args);
  if (bf16 && args.D == 128) return launch_one<128, true>(ctx, q, k, v, ld_q, ld_k, ld_v, total_rows, args);
  return set_error(ctx, GRILLY_ERR_UNSUPPORTED,
                   "attention: head_dim must be 32, 64, 96 or 128 (tf32 mode), 64 or 128 (bf16 mode), or 32 in bf16 mode for sequences up to 128");
}

}  // namespace gb
