// y[tokens][features] = act(x W^T + b) (+ residual) with ONE tcgen05 MMA shared by a pair of CTAs (cta_group::2).
//
// Why pairs: with one CTA per tile every 128 x 256 output tile reads (128 + 256) operand rows per k-block from L2,
// and at K = 384 the L2 -> shared-memory traffic (about 43 FLOP per byte), not the tensor pipe, sets the speed. A
// pair computes a 256 (features) x 256 (tokens) tile: each CTA loads 128 weight rows and 128 token rows, the MMA
// reads both halves of both operands from the two CTAs' shared memory, and each CTA ends up with 128 feature rows
// x 256 token columns of the accumulator in its own TMEM. Operand traffic per output drops by one third.
//
// Orientation is the "swapped" one of gemm.cuh (weights are the M operand, tokens the MMA's N), both operands
// K-major. Roles per CTA: warp 0 TMA producer (own halves; bytes are counted on the LEADER's full barrier),
// warp 1 MMA issuer (leader CTA only) and TMEM allocation (both CTAs), warps 2.. epilogue (own 128 features).
// Barriers: full[s] lives in the leader; empty[s] and tmem_full[a] exist in both CTAs and the leader's MMA thread
// commits to both; tmem_empty[a] lives in the leader and collects the epilogue warps of both CTAs.
#pragma once
#include "gemm.cuh"

namespace gb {

// Eight epilogue warps (two per TMEM lane quadrant), not the sixteen of the single-CTA kernel: on the K = 384 launches of the
// encoder the MMAs and the epilogue arithmetic slow each other down, and with fewer warps busy beside the issuing
// thread the same launches run 5-7 % faster (QKV 134 -> 128 us, FFN1 + GELU 169 -> 157 us; 8192^3 unchanged; four
// warps are slower again).
constexpr int GEMM_PAIR_EPI_WARPS = 8;
constexpr int GEMM_PAIR_THREADS = 64 + 32 * GEMM_PAIR_EPI_WARPS;   // warp 0 TMA, warp 1 MMA, the rest epilogue

struct GemmPairCfg {
  static constexpr int HALF_BYTES = 128 * 128;                 // 128 rows x 128 B (one operand half)
  static constexpr int STAGE_BYTES = 2 * HALF_BYTES;           // per CTA: weight half + token half
  static constexpr int STAGES = 7;                             // 224 KB of 227: one more than six took QKV from 126 to 120 us
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = 512;                        // two 256-column accumulators
  static constexpr int TILE = 256;                             // features and tokens per pair tile
};

// kBMn = false: `linear` (tmap_w = weights [N][K], the MMA's M operand; tmap_x = tokens [M][K], the MMA's N operand;
// accumulator lanes are features, the swapped epilogue writes y[token][feature]).
// kBMn = true: `gemm_mnk` (tmap_w = A [M][K], the MMA's M operand; tmap_x = B [K][N] row-major, consumed in place as
// an MN-major N operand in 128-byte-wide column chunks; accumulator lanes are rows of C, the plain epilogue writes
// C[row][col]). num_m_tiles / num_n_tiles count 256-blocks of the MMA's M / N operand in both cases.
template <bool kBf16, bool kBMn>
__global__ void __launch_bounds__(GEMM_PAIR_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                         const GemmArgs args) {
  using Cfg = GemmPairCfg;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ELT = kBf16 ? 2 : 4;
  constexpr int BK = 128 / ELT;
  constexpr int CH = 128 / ELT;                                // columns per 128-byte chunk of an MN-major operand
  constexpr int UMMA_K = 32 / ELT;
  constexpr int KSTEPS = 4;                                    // 32-byte k-steps per 128-byte stage row
  constexpr uint32_t IDESC = make_idesc(kBf16, 256, 256, false, kBMn);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                     // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = args.num_m_tiles * args.num_n_tiles;   // m: 256-feature blocks, n: 256-token blocks

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);                              // used in the leader only
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 2 * GEMM_PAIR_EPI_WARPS);      // used in the leader only
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_w);
    prefetch_tmap(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                                              // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // a failed wait stops both CTAs: the peer's waits poll its own flag
  auto fail = [&](int code) {
    if (!*abort_flag) atomicCAS(args.err, 0, code);
    *abort_flag = 1;
    st_cluster_u32(map_to_cta(const_cast<int*>(abort_flag), rank ^ 1u), 1u);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs, own halves)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m_blk, n_blk;                                      // feature blocks fastest: neighbours share the tokens
        tile_coords(tile, args.num_m_tiles, args.num_n_tiles, args.tile_group, m_blk, n_blk);
        const int w_row = m_blk * Cfg::TILE + static_cast<int>(rank) * 128;
        const int x_row = n_blk * Cfg::TILE + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < args.num_k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { fail(ERR_WAIT_EMPTY); ok = false; break; }
          uint8_t* sw = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sx = sw + Cfg::HALF_BYTES;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * Cfg::STAGE_BYTES);   // both CTAs' bytes land on this barrier
          const uint32_t bar = map_to_cta(&full_bar[stage], 0);
          tma_load_2d_pair(sw, &tmap_w, bar, kb * BK, w_row);
          if constexpr (kBMn) {
#pragma unroll
            for (int c = 0; c < 128 / CH; ++c)                 // this CTA's 128 columns, one chunk of CH columns at a time
              tma_load_2d_pair(sx + c * (BK * 128), &tmap_x, bar, x_row + c * CH, kb * BK);
          } else {
            tma_load_2d_pair(sx, &tmap_x, bar, kb * BK, x_row);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      const uint32_t smem_base = smem_u32(smem);
      const uint64_t a_desc0 = make_smem_desc_sw128(smem_base, 16, 1024);
      constexpr uint32_t B_KSTEP_BYTES = kBMn ? UMMA_K * 128 : 32;   // advance of the N operand per 32-byte k-step
      const uint64_t b_desc0 = kBMn ? make_smem_desc_mn<kBf16>(smem_base + Cfg::HALF_BYTES, BK * 128)
                                    : make_smem_desc_sw128(smem_base + Cfg::HALF_BYTES, 16, 1024);
      const uint32_t a_desc_lo = static_cast<uint32_t>(a_desc0), a_desc_hi = static_cast<uint32_t>(a_desc0 >> 32);
      const uint32_t b_desc_lo = static_cast<uint32_t>(b_desc0), b_desc_hi = static_cast<uint32_t>(b_desc0 >> 32);
      const uint32_t peer_empty0 = map_to_cta(&empty_bar[0], 1), own_empty0 = map_to_cta(&empty_bar[0], 0);
      const uint32_t peer_tfull0 = map_to_cta(&tmem_full[0], 1), own_tfull0 = map_to_cta(&tmem_full[0], 0);
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) { fail(ERR_WAIT_TMEM_EMPTY); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * Cfg::TILE;
        for (int kb = 0; kb < args.num_k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { fail(ERR_WAIT_FULL); ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_desc_lo + stage * (Cfg::STAGE_BYTES >> 4);
          const uint32_t b_lo = b_desc_lo + stage * (Cfg::STAGE_BYTES >> 4);
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            const uint64_t adesc = (static_cast<uint64_t>(a_desc_hi) << 32) | (a_lo + ks * 2);
            const uint64_t bdesc = (static_cast<uint64_t>(b_desc_hi) << 32) | (b_lo + ks * (B_KSTEP_BYTES >> 4));
            umma_ss_pair<kBf16>(d_tmem, adesc, bdesc, IDESC, (kb | ks) != 0 ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_pair(own_empty0 + stage * 8);
          umma_commit_pair(peer_empty0 + stage * 8);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          umma_commit_pair(own_tfull0 + acc * 8);
          umma_commit_pair(peer_tfull0 + acc * 8);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 features)
    constexpr int NCHUNK = Cfg::TILE / 32;
    constexpr int G = GEMM_PAIR_EPI_WARPS / 4;
    constexpr int MAXIT = (NCHUNK + G - 1) / G;
    const int quad = warp & 3;
    const int group = (warp - 2) >> 2;
    const uint32_t leader_tempty0 = map_to_cta(&tmem_empty[0], 0);
    int it = 0;
    EpiFlags f;
    const bool out_al16 = (reinterpret_cast<uintptr_t>(args.out) & 15) == 0;
    f.vec_ok = !args.out_bf16 && (args.ld_out % 4 == 0) && out_al16;
    f.vec8_ok = args.out_bf16 && (args.ld_out % 8 == 0) && out_al16;
    f.res_vec_ok = args.residual && (args.ld_res % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.residual) & 15) == 0);
    f.bias_vec_ok = args.bias && ((reinterpret_cast<uintptr_t>(args.bias) & 15) == 0);
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
      int m_blk, n_blk;
      tile_coords(tile, args.num_m_tiles, args.num_n_tiles, args.tile_group, m_blk, n_blk);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag)) { fail(ERR_WAIT_TMEM_FULL); break; }
      tc_fence_after();
      const int feat = m_blk * Cfg::TILE + static_cast<int>(rank) * 128 + quad * 32 + lane;
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * Cfg::TILE;
      uint32_t ra[32], rb[32];
      __syncwarp();
      if (group < NCHUNK) tmem_ld_32x32(taddr_row + group * 32, ra);
#pragma unroll
      for (int i = 0; i < MAXIT; ++i) {
        const int c = group + i * G;
        uint32_t (&cur)[32] = (i & 1) ? rb : ra;
        uint32_t (&nxt)[32] = (i & 1) ? ra : rb;
        __syncwarp();
        if (c < NCHUNK) tmem_ld_wait();
        if (c + G < NCHUNK) tmem_ld_32x32(taddr_row + (c + G) * 32, nxt);
        const int tok0 = n_blk * Cfg::TILE + c * 32;
        if constexpr (kBMn) {
          // feat is the row of C, tok0 the first of 32 columns
          if (args.multi_out > 0) {   // launcher guarantees fp32 output and N a multiple of 32
            if (c < NCHUNK && tok0 < args.N) epilogue_chunk_multi(args, cur, feat - lane, tok0, lane);
          } else if (c < NCHUNK && feat < args.M && tok0 < args.N) {
            epilogue_chunk(args, f, cur, feat, tok0, 0.f, 1.f);
          }
        } else {
          if (c < NCHUNK && tok0 < args.M) epilogue_chunk_swapped(args, cur, feat, tok0);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tempty0 + acc * 8);
    }
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);          // let copies and MMAs in flight land (about 1 ms)
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                                              // neither CTA frees TMEM or exits while the other still uses it
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace gb
