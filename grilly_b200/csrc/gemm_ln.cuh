// y = LayerNorm(x W^T + bias + residual) * gamma + beta in ONE kernel: the post-LN step of a BERT layer
// (utils/vulkan_sentence_transformer.py:997-1011 and 1018-1033 in the reference: linear, add the residual, LayerNorm)
// without the pre-norm sum ever reaching memory.
//
// The row statistics need whole output rows, and the epilogue that takes them has to run UNDER the next tile's main
// loop or it adds to every tile. Both together fit like this: a cluster of two CTAs owns a tile of 128 token rows
// x all N features (N in {128, 256, 384, 512}); CTA r of the pair computes features [r N/2, (r+1) N/2) of those
// rows. Its accumulator is N/2 TMEM columns wide, so two accumulators fit (2 x N/2 <= 512 columns) and the epilogue
// of tile i overlaps the MMAs of tile i+1, as in gemm.cuh. One epilogue thread owns one token row of its CTA's
// half:
//   pass 1: v = acc + bias + residual, written back to TMEM; mean and sum of squared deviations of the half row
//   exchange: (mean, M2) go to the same row's thread in the other CTA through distributed shared memory; both
//           merge the two halves with the pairwise formula (M2 = M2a + M2b + (mean_a - mean_b)^2 n / 2) and get the
//           same row statistics bit for bit
//   pass 2: (v - mean) * rstd * gamma + beta, optional tf32 rounding, staged in swizzled shared memory and stored
//           with cp.async.bulk.tensor (fp32 output: whole 128-byte lines leave the SM, ragged last rows are clipped
//           by the copy engine) or with 8-byte vector stores (bf16 output).
// The residual comes in through TMA as well (a ring of [128 rows x 32 columns] boxes filled by a warp of its own that
// runs ahead of the epilogue), because a thread that owns a row would otherwise fetch 32 different cache lines per
// load instruction and wait for each of them.
//
// Roles per CTA: warp 0 operand TMA producer, warp 1 MMA issuer + TMEM allocation, warp 2 residual TMA producer,
// warps 3..6 epilogue (one per TMEM lane quadrant). Every wait is bounded (ptx.cuh); a wait that gives up records a
// status, raises the abort flag of both CTAs and the pair drains. Every load is a per-CTA load of this GPU's own
// memory.
#pragma once
#include "gemm.cuh"

namespace gb {

constexpr int GEMM_LN_THREADS = 224;       // warp 0 TMA, warp 1 MMA, warp 2 residual TMA, warps 3..6 epilogue

// kDeep trades epilogue buffers for one more operand stage: with a long K loop the main loop is bound by the bytes
// that are in flight from L2 and the epilogue has time to spare under it; with a short K loop it is the other way round.
template <int NCHUNK, bool kBf16, bool kDeep>   // NCHUNK = 32-column chunks per CTA (N / 64)
struct GemmLnCfg {
  static constexpr int OUT_BUFS = kDeep ? 1 : 2;             // output staging buffers per epilogue warp (32 rows x 128 B each)
  static constexpr int NHALF = NCHUNK * 32;                  // features per CTA
  static constexpr int N = 2 * NHALF;
  static constexpr int ELT = kBf16 ? 2 : 4;
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = NHALF * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int RES_BUFS = (kDeep || NCHUNK >= 8) ? 2 : 3;   // residual ring depth (boxes of 128 rows x 32 columns)
  static constexpr int RES_BUF_BYTES = 128 * 32 * ELT;       // one residual box
  static constexpr int RES_BYTES = RES_BUFS * 128 * 32 * 4;  // sized for fp32 so that what follows stays 1024-byte aligned
  static constexpr int OUT_BYTES = 4 * OUT_BUFS * 4096;
  static constexpr int PARAM_BYTES = 3 * NHALF * 4;          // bias, gamma, beta of this CTA's half
  static constexpr int STATS_BYTES = 2 * 128 * 8;            // (mean, M2) of the peer's half rows, two tiles in flight
  static constexpr int CTRL_BYTES = 512;                     // barriers, TMEM address, abort flag
  static constexpr int FIXED = RES_BYTES + OUT_BYTES + PARAM_BYTES + STATS_BYTES + CTRL_BYTES + 1024 /*align slack*/;
  static constexpr int MAX_SMEM = 227 * 1024;
  static constexpr int STAGES_RAW = (MAX_SMEM - FIXED) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + FIXED;
  static constexpr int TMEM_COLS = N <= 32 ? 32 : N <= 64 ? 64 : N <= 128 ? 128 : N <= 256 ? 256 : 512;
  static_assert(N <= 512, "two accumulators of N/2 columns must fit TMEM");
  static_assert(NHALF % 16 == 0 && NHALF <= 256, "each CTA's half is one tcgen05.mma wide");
  static_assert(NCHUNK % 2 == 0, "the epilogue walks the chunks in pairs");
  static_assert(STAGES >= 3, "the operand ring needs at least three stages");
};

template <int NCHUNK, bool kBf16, bool kDeep>
__global__ void __launch_bounds__(GEMM_LN_THREADS, 1)
gemm_rowln_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ CUtensorMap tmap_res, const __grid_constant__ CUtensorMap tmap_out,
                          const GemmLnArgs args) {
  using Cfg = GemmLnCfg<NCHUNK, kBf16, kDeep>;
  constexpr int OB = Cfg::OUT_BUFS;
  constexpr int NHALF = Cfg::NHALF;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ELT = Cfg::ELT;
  constexpr int BK = 128 / ELT;
  constexpr int KSTEPS = 4;
  constexpr int RB = Cfg::RES_BUFS;
  constexpr uint32_t IDESC = make_idesc(kBf16, 128, NHALF, false, false);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* res_ring = smem + STAGES * Cfg::STAGE_BYTES;             // 1024-byte aligned: every size before it is
  uint8_t* out_stage = res_ring + Cfg::RES_BYTES;                   // 1024-byte aligned
  float* s_bias = reinterpret_cast<float*>(out_stage + Cfg::OUT_BYTES);
  float* s_gamma = s_bias + NHALF;
  float* s_beta = s_gamma + NHALF;
  float2* s_peer = reinterpret_cast<float2*>(s_beta + NHALF);        // [2][128] written by the OTHER CTA
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s_peer) + Cfg::STATS_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;        // [2]
  uint64_t* tmem_empty = tmem_full + 2;            // [2]
  uint64_t* res_full = tmem_empty + 2;             // [RB]
  uint64_t* res_empty = res_full + RB;             // [RB]
  uint64_t* stats_bar = res_empty + RB;            // [2]: the peer's 128 epilogue threads arrive
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(stats_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();         // which half of the features this CTA owns
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int col_base = static_cast<int>(rank) * NHALF;
  const bool has_res = args.residual != nullptr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
      mbar_init(&stats_bar[a], 128);
    }
    for (int b = 0; b < RB; ++b) {
      mbar_init(&res_full[b], 1);
      mbar_init(&res_empty[b], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_res);
    prefetch_tmap(&tmap_out);
  }
  // this CTA's slice of the per-feature parameters (missing ones become the neutral value)
  for (int i = threadIdx.x; i < NHALF; i += GEMM_LN_THREADS) {
    s_bias[i] = args.bias ? __ldg(args.bias + col_base + i) : 0.f;
    s_gamma[i] = args.gamma ? __ldg(args.gamma + col_base + i) : 1.f;
    s_beta[i] = args.beta ? __ldg(args.beta + col_base + i) : 0.f;
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                                  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // a failed wait stops both CTAs: the peer's waits poll its own flag
  auto fail = [&](int code) {
    if (!*abort_flag) atomicCAS(args.err, 0, code);
    *abort_flag = 1;
    st_cluster_u32(map_to_cta(const_cast<int*>(abort_flag), rank ^ 1u), 1u);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ operand TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < args.num_tiles && ok; tile += num_pairs) {
        for (int kb = 0; kb < args.num_k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { fail(ERR_WAIT_EMPTY); ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, tile * 128);                  // 128 token rows
          tma_load_2d(sa + Cfg::A_BYTES, &tmap_b, &full_bar[stage], kb * BK, col_base);     // this CTA's weight rows
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      const uint32_t smem_base = smem_u32(smem);
      const uint64_t a_desc0 = make_smem_desc_sw128(smem_base, 16, 1024);
      const uint64_t b_desc0 = make_smem_desc_sw128(smem_base + Cfg::A_BYTES, 16, 1024);
      const uint32_t a_desc_lo = static_cast<uint32_t>(a_desc0), a_desc_hi = static_cast<uint32_t>(a_desc0 >> 32);
      const uint32_t b_desc_lo = static_cast<uint32_t>(b_desc0), b_desc_hi = static_cast<uint32_t>(b_desc0 >> 32);
      for (int tile = pair; tile < args.num_tiles && ok; tile += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) { fail(ERR_WAIT_TMEM_EMPTY); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * NHALF;
        for (int kb = 0; kb < args.num_k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { fail(ERR_WAIT_FULL); ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_desc_lo + stage * (Cfg::STAGE_BYTES >> 4);
          const uint32_t b_lo = b_desc_lo + stage * (Cfg::STAGE_BYTES >> 4);
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            const uint64_t adesc = (static_cast<uint64_t>(a_desc_hi) << 32) | (a_lo + ks * 2);
            const uint64_t bdesc = (static_cast<uint64_t>(b_desc_hi) << 32) | (b_lo + ks * 2);
            umma_ss<kBf16>(d_tmem, adesc, bdesc, IDESC, (kb | ks) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ residual TMA producer (runs ahead of the epilogue)
    if (lane == 0 && has_res) {
      int buf = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < args.num_tiles && ok; tile += num_pairs) {
        for (int c = 0; c < NCHUNK; ++c) {
          if (!mbar_wait(&res_empty[buf], phase ^ 1u, abort_flag)) { fail(ERR_WAIT_EMPTY); ok = false; break; }
          mbar_expect_tx(&res_full[buf], Cfg::RES_BUF_BYTES);
          tma_load_2d(res_ring + buf * Cfg::RES_BUF_BYTES, &tmap_res, &res_full[buf], col_base + c * 32, tile * 128);
          if (++buf == RB) { buf = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue: one thread = one token row of this half
    const int quad = warp & 3;
    const int trow = quad * 32 + lane;                    // row within the tile = TMEM lane
    uint8_t* my_out = out_stage + (warp - 3) * (OB * 4096);
    const float inv_half = 1.0f / static_cast<float>(NHALF);
    const float inv_n = 1.0f / static_cast<float>(2 * NHALF);
    const uint32_t peer_slot0 = map_to_cta(s_peer, rank ^ 1u);
    const uint32_t peer_stats_bar0 = map_to_cta(stats_bar, rank ^ 1u);
    int it = 0;
    int rbuf = 0;
    uint32_t rphase = 0;
    uint32_t out_count = 0;                               // bulk-store groups committed by this warp's lane 0 so far
    bool ok = true;
    for (int tile = pair; tile < args.num_tiles && ok; tile += num_pairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      const int row0 = tile * 128 + quad * 32;            // first row of this warp's 32
      const int row = row0 + lane;
      const bool row_ok = row < args.M;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag)) { fail(ERR_WAIT_TMEM_FULL); break; }
      tc_fence_after();
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * NHALF;
      uint32_t ra[32], rb[32];
      // ---------------- pass 1: v = acc + bias + residual -> TMEM; shifted sums for the statistics of the half row
      float shift = 0.f, s1 = 0.f, s2 = 0.f;
      __syncwarp();
      tmem_ld_32x32(taddr_row, ra);
      // chunks are walked in pairs (the two register buffers alternate); the pair loop is not unrolled
#pragma unroll 1
      for (int c2 = 0; c2 < NCHUNK && ok; c2 += 2) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int c = c2 + h;
          uint32_t (&cur)[32] = h ? rb : ra;
          uint32_t (&nxt)[32] = h ? ra : rb;
          __syncwarp();
          tmem_ld_wait();
          if (c + 1 < NCHUNK) tmem_ld_32x32(taddr_row + (c + 1) * 32, nxt);
          if (has_res) {
            if (!mbar_wait(&res_full[rbuf], rphase, abort_flag)) { fail(ERR_WAIT_FULL); ok = false; }
            const uint8_t* rp = res_ring + rbuf * Cfg::RES_BUF_BYTES;
            if constexpr (kBf16) {
              // plain row-major box: 64 bytes per row
              const uint4* q4 = reinterpret_cast<const uint4*>(rp + trow * 64);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 w = q4[q];
                const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  cur[8 * q + 2 * u] = __float_as_uint(__uint_as_float(cur[8 * q + 2 * u]) + __uint_as_float(ws[u] << 16));
                  cur[8 * q + 2 * u + 1] = __float_as_uint(__uint_as_float(cur[8 * q + 2 * u + 1]) + __uint_as_float(ws[u] & 0xffff0000u));
                }
              }
            } else {
              // 128-byte swizzle: 16-byte chunk q of row r lives at chunk (q ^ (r & 7))
              const uint8_t* rowp = rp + trow * 128;
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 w = *reinterpret_cast<const float4*>(rowp + ((q ^ (trow & 7)) << 4));
                cur[4 * q] = __float_as_uint(__uint_as_float(cur[4 * q]) + w.x);
                cur[4 * q + 1] = __float_as_uint(__uint_as_float(cur[4 * q + 1]) + w.y);
                cur[4 * q + 2] = __float_as_uint(__uint_as_float(cur[4 * q + 2]) + w.z);
                cur[4 * q + 3] = __float_as_uint(__uint_as_float(cur[4 * q + 3]) + w.w);
              }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&res_empty[rbuf]);   // this warp has read its 32 rows of the box
            if (++rbuf == RB) { rbuf = 0; rphase ^= 1u; }
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 b4 = *reinterpret_cast<const float4*>(s_bias + c * 32 + 4 * q);
            cur[4 * q] = __float_as_uint(__uint_as_float(cur[4 * q]) + b4.x);
            cur[4 * q + 1] = __float_as_uint(__uint_as_float(cur[4 * q + 1]) + b4.y);
            cur[4 * q + 2] = __float_as_uint(__uint_as_float(cur[4 * q + 2]) + b4.z);
            cur[4 * q + 3] = __float_as_uint(__uint_as_float(cur[4 * q + 3]) + b4.w);
          }
          if (c == 0) shift = __uint_as_float(cur[0]);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float d = __uint_as_float(cur[j]) - shift;
            s1 += d;
            s2 = fmaf(d, d, s2);
          }
          tmem_st_32x32(taddr_row + c * 32, cur);
        }
      }
      tmem_st_wait();
      if (!ok) break;
      // ---------------- statistics of the whole row: this half's (mean, M2) meet the other CTA's
      const float md = s1 * inv_half;
      const float mean_a = shift + md;
      const float m2_a = fmaxf(fmaf(-md, s1, s2), 0.f);            // sum (v - mean_a)^2 over this half
      st_cluster_f32x2(peer_slot0 + static_cast<uint32_t>((acc * 128 + trow) * 8), mean_a, m2_a);
      mbar_arrive_release_cluster(peer_stats_bar0 + acc * 8);
      if (!mbar_wait_cluster(&stats_bar[acc], acc_phase, abort_flag)) { fail(ERR_WAIT_TMEM_FULL); break; }
      const float2 other = s_peer[acc * 128 + trow];
      const float mean = 0.5f * (mean_a + other.x);
      const float delta = mean_a - other.x;
      const float m2 = m2_a + other.y + delta * delta * (0.5f * static_cast<float>(NHALF));
      const float var = m2 * inv_n;
      float rstd = rsqrtf(var + args.eps);
      rstd = rstd * (1.5f - 0.5f * (var + args.eps) * rstd * rstd);   // one Newton step: the rounding of 1/sqrt
      // ---------------- pass 2: normalise, scale, shift, store
      const bool bf16_out = kBf16 && args.out_bf16;
      __syncwarp();
      tmem_ld_32x32(taddr_row, ra);
#pragma unroll 1
      for (int c2 = 0; c2 < NCHUNK; c2 += 2) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int c = c2 + h;
          uint32_t (&cur)[32] = h ? rb : ra;
          uint32_t (&nxt)[32] = h ? ra : rb;
          __syncwarp();
          tmem_ld_wait();
          if (c + 1 < NCHUNK) tmem_ld_32x32(taddr_row + (c + 1) * 32, nxt);
          uint8_t* stg = my_out + (out_count & (OB - 1)) * 4096;
          if (!bf16_out) {
            // this staging buffer is free once the bulk store committed OB groups ago has READ it
            if (lane == 0) tma_store_wait_read<OB - 1>();
            __syncwarp();
          }
          uint8_t* rowp = stg + lane * 128;
          // four columns at a time, finished and put away, so that few values are live at once
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 g4 = *reinterpret_cast<const float4*>(s_gamma + c * 32 + 4 * q);
            const float4 b4 = *reinterpret_cast<const float4*>(s_beta + c * 32 + 4 * q);
            float4 o;
            o.x = fmaf((__uint_as_float(cur[4 * q]) - mean) * rstd, g4.x, b4.x);
            o.y = fmaf((__uint_as_float(cur[4 * q + 1]) - mean) * rstd, g4.y, b4.y);
            o.z = fmaf((__uint_as_float(cur[4 * q + 2]) - mean) * rstd, g4.z, b4.z);
            o.w = fmaf((__uint_as_float(cur[4 * q + 3]) - mean) * rstd, g4.w, b4.w);
            if (args.round_tf32) { o.x = round_to_tf32(o.x); o.y = round_to_tf32(o.y); o.z = round_to_tf32(o.z); o.w = round_to_tf32(o.w); }
            if (bf16_out) {
              if (row_ok) {
                uint2 pk;
                pk.x = pack_bf16x2(o.x, o.y);
                pk.y = pack_bf16x2(o.z, o.w);
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(args.out) + static_cast<long long>(row) * args.ld_out +
                                          col_base + c * 32 + 4 * q) = pk;
              }
            } else {
              *reinterpret_cast<float4*>(rowp + ((q ^ (lane & 7)) << 4)) = o;    // the tensor map's 128-byte swizzle
            }
          }
          if (!bf16_out) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (row0 < args.M) tma_store_2d(&tmap_out, stg, col_base + c * 32, row0);   // rows beyond M are clipped
              tma_store_commit();    // an empty group when nothing was stored: the buffer count stays in step
            }
            ++out_count;
          }
        }
      }
      // this warp has finished reading the accumulator
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
    if (lane == 0) tma_store_wait_all<0>();   // staging memory outlives the last bulk store's read; the data has landed
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);   // let copies and MMAs in flight land (about 1 ms)
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                                        // the peer may still write statistics into this CTA
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace gb
