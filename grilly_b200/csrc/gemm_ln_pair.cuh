// y = LayerNorm(x W^T + bias + residual) * gamma + beta in ONE kernel, with ONE tcgen05 MMA shared by a pair of CTAs
// (cta_group::2): the post-LN step of a BERT layer (utils/vulkan_sentence_transformer.py:997-1011 and 1018-1033 in the
// reference: linear, add the residual, LayerNorm).
//
// A pair owns 256 token rows x all N features (N in {128, 256, 384, 512}). Tokens are the MMA's M operand (each CTA
// loads its own 128 rows), the weights its N operand, in one or two instructions of up to 256 features, of which each
// CTA loads one half. Every CTA ends up with WHOLE rows of its 128 tokens in its own TMEM (N columns), so the row
// statistics need no exchange between the CTAs, and per 128 x N outputs the pair reads (128 + N/2) operand rows from L2
// where a CTA on its own reads (128 + N): with N = 384 and a long K loop that traffic, not the tensor pipe, sets the speed.
//
// With N > 256 the accumulator takes more than half of TMEM and cannot be double-buffered, so the epilogue does not
// overlap the next tile's MMAs; it is made short instead: SUB warps per TMEM lane quadrant split a row's columns
// (SUB x 4 epilogue warps), each thread owns one token row of its column range:
//   pass 1: v = acc + bias + residual, written back to TMEM; mean and sum of squared deviations of the range
//   merge:  the SUB partial results of a row meet in shared memory (an mbarrier per quadrant) and every thread
//           merges them in the same order (M2 = sum M2_i + n_i sum (mean_i - mean)^2), so all agree bit for bit
//   pass 2: (v - mean) * rstd * gamma + beta, optional tf32 rounding, staged in swizzled shared memory and stored with
//           cp.async.bulk.tensor (fp32 boxes under the 128-byte swizzle, bf16 boxes under the 64-byte swizzle).
// The residual comes in through TMA: every epilogue warp fetches [32 rows x 32 columns] boxes of its own rows and
// columns into the buffers it later stages its output in, the first ones of a tile while the tile's MMAs still run.
//
// Roles per CTA: warp 0 operand TMA producer (own halves; bytes are counted on the LEADER's full barrier), warp 1 MMA
// issuer (leader only) + TMEM allocation (both), warp 2 idle, warps 3.. epilogue. Every wait is bounded (ptx.cuh); a
// wait that gives up records a status, raises the abort flag of both CTAs and the pair drains. Every load is a
// per-CTA load of this GPU's own memory.
#pragma once
#include "gemm.cuh"

namespace gb {

template <int N_, int SUB_, int BUFS_, bool kBf16>
struct GemmLnPairCfg {
  static constexpr int N = N_, SUB = SUB_, BUFS = BUFS_;
  static constexpr int ELT = kBf16 ? 2 : 4;
  static constexpr int NI = N > 256 ? 2 : 1;                  // MMA instructions per k-step
  static constexpr int NW = N / NI;                           // features per instruction
  static constexpr int BH = NW / 2;                           // weight rows per instruction that one CTA loads
  static constexpr int NCHUNK = N / 32;                       // 32-column chunks per row
  static constexpr int CPW = NCHUNK / SUB;                    // chunks per epilogue warp
  static constexpr int EPI_WARPS = 4 * SUB;
  static constexpr int THREADS = 96 + 32 * EPI_WARPS;
  static constexpr int ACCS = 2 * N <= 512 ? 2 : 1;           // accumulators that fit TMEM
  static constexpr int TMEM_COLS = ACCS * N <= 128 ? 128 : ACCS * N <= 256 ? 256 : 512;
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = NI * BH * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BUF_BYTES = 4096;                      // one box of 32 rows x 128 bytes
  static constexpr int RES_BOX_BYTES = 32 * 32 * ELT;
  static constexpr int EPI_BYTES = EPI_WARPS * BUFS * BUF_BYTES;
  static constexpr int PARAM_BYTES = 3 * N * 4;               // bias, gamma, beta
  static constexpr int PART_BYTES = ACCS * SUB * 128 * 8;     // (mean, M2) per accumulator, column range and row
  static constexpr int CTRL_BYTES = 1024;                     // barriers, TMEM address, abort flag
  static constexpr int FIXED = EPI_BYTES + PARAM_BYTES + PART_BYTES + CTRL_BYTES + 1024 /*align slack*/;
  static constexpr int MAX_SMEM = 227 * 1024;
  static constexpr int STAGES_RAW = (MAX_SMEM - FIXED) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + FIXED;
  static_assert(NCHUNK % SUB == 0, "the column ranges of a row are equal");
  static_assert(NW % 32 == 0 && NW <= 256 && BH % 8 == 0, "instruction width");
  static_assert(STAGES >= 3, "the operand ring needs at least three stages");
  static_assert(BUFS >= 1 && BUFS <= 4, "buffers per epilogue warp");
  static_assert((2 + 2 * 6 + 2 * 2 + 4 * 4 * 4 + 8) * 8 <= CTRL_BYTES, "control block");
};

template <int N, int SUB, int BUFS, bool kBf16>
__global__ void __launch_bounds__(GemmLnPairCfg<N, SUB, BUFS, kBf16>::THREADS, 1)
gemm_rowln_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_res, const __grid_constant__ CUtensorMap tmap_out,
                       const GemmLnArgs args) {
  using Cfg = GemmLnPairCfg<N, SUB, BUFS, kBf16>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ELT = Cfg::ELT;
  constexpr int BK = 128 / ELT;
  constexpr int KSTEPS = 4;
  constexpr int NI = Cfg::NI, NW = Cfg::NW, BH = Cfg::BH, CPW = Cfg::CPW, ACCS = Cfg::ACCS, EW = Cfg::EPI_WARPS;
  constexpr uint32_t IDESC = make_idesc(kBf16, 256, NW, false, false);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_bufs = smem + STAGES * Cfg::STAGE_BYTES;               // 1024-byte aligned: every size before it is
  float* s_bias = reinterpret_cast<float*>(epi_bufs + Cfg::EPI_BYTES);
  float* s_gamma = s_bias + N;
  float* s_beta = s_gamma + N;
  float2* s_part = reinterpret_cast<float2*>(s_beta + N);              // [ACCS][SUB][128]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s_part) + Cfg::PART_BYTES);   // leader's is used
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;        // [ACCS]
  uint64_t* tmem_empty = tmem_full + 2;            // [ACCS], leader's is used: the epilogue warps of both CTAs arrive
  uint64_t* part_bar = tmem_empty + 2;             // [ACCS][4 quadrants]: 32 * SUB threads arrive
  uint64_t* res_full = part_bar + 8;               // [EW][BUFS]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(res_full + EW * Cfg::BUFS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();         // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const bool has_res = args.residual != nullptr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 2 * EW);
      for (int q = 0; q < 4; ++q) mbar_init(&part_bar[a * 4 + q], 32 * SUB);
    }
    for (int b = 0; b < EW * Cfg::BUFS; ++b) mbar_init(&res_full[b], 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_res);
    prefetch_tmap(&tmap_out);
  }
  for (int i = threadIdx.x; i < N; i += Cfg::THREADS) {   // missing parameters become the neutral value
    s_bias[i] = args.bias ? __ldg(args.bias + i) : 0.f;
    s_gamma[i] = args.gamma ? __ldg(args.gamma + i) : 1.f;
    s_beta[i] = args.beta ? __ldg(args.beta + i) : 0.f;
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, Cfg::TMEM_COLS);
    tmem_relinquish_pair();
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
    // ------------------------------------------------------------ operand TMA producer (both CTAs, own halves)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t bar0 = map_to_cta(&full_bar[0], 0);
      for (int tile = pair; tile < args.num_tiles && ok; tile += num_pairs) {
        const int x_row = tile * 256 + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < args.num_k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { fail(ERR_WAIT_EMPTY); ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * Cfg::STAGE_BYTES);   // both CTAs' bytes land on this barrier
          const uint32_t bar = bar0 + stage * 8;
          tma_load_2d_pair(sa, &tmap_a, bar, kb * BK, x_row);
#pragma unroll
          for (int i = 0; i < NI; ++i)               // this CTA's half of the weight rows of instruction i
            tma_load_2d_pair(sa + Cfg::A_BYTES + i * (BH * 128), &tmap_b, bar, kb * BK, i * NW + static_cast<int>(rank) * BH);
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
      const uint64_t b_desc0 = make_smem_desc_sw128(smem_base + Cfg::A_BYTES, 16, 1024);
      const uint32_t a_desc_lo = static_cast<uint32_t>(a_desc0), a_desc_hi = static_cast<uint32_t>(a_desc0 >> 32);
      const uint32_t b_desc_lo = static_cast<uint32_t>(b_desc0), b_desc_hi = static_cast<uint32_t>(b_desc0 >> 32);
      const uint32_t peer_empty0 = map_to_cta(&empty_bar[0], 1), own_empty0 = map_to_cta(&empty_bar[0], 0);
      const uint32_t peer_tfull0 = map_to_cta(&tmem_full[0], 1), own_tfull0 = map_to_cta(&tmem_full[0], 0);
      for (int tile = pair; tile < args.num_tiles && ok; tile += num_pairs, ++it) {
        const int acc = it % ACCS;
        const uint32_t acc_phase = (it / ACCS) & 1u;
        if (!mbar_wait_cluster(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) { fail(ERR_WAIT_TMEM_EMPTY); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * N;
        for (int kb = 0; kb < args.num_k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { fail(ERR_WAIT_FULL); ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_desc_lo + stage * (Cfg::STAGE_BYTES >> 4);
          const uint32_t b_lo = b_desc_lo + stage * (Cfg::STAGE_BYTES >> 4);
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            const uint64_t adesc = (static_cast<uint64_t>(a_desc_hi) << 32) | (a_lo + ks * 2);
#pragma unroll
            for (int i = 0; i < NI; ++i) {
              const uint64_t bdesc = (static_cast<uint64_t>(b_desc_hi) << 32) | (b_lo + i * ((BH * 128) >> 4) + ks * 2);
              umma_ss_pair<kBf16>(d_tmem + i * NW, adesc, bdesc, IDESC, (kb | ks) != 0 ? 1u : 0u);
            }
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
  } else if (warp >= 3) {
    // ------------------------------------------------------------ epilogue: one thread = one token row, CPW chunks of it
    const int ew = warp - 3;
    const int quad = warp & 3;                            // TMEM lane quadrant this warp can reach
    const int sub = ew >> 2;                              // which column range of the row
    const int trow = quad * 32 + lane;                    // row within this CTA's 128 = TMEM lane
    const int chunk0 = sub * CPW;                         // first 32-column chunk of the range
    uint8_t* my_bufs = epi_bufs + ew * (Cfg::BUFS * Cfg::BUF_BYTES);
    uint64_t* my_res_full = res_full + ew * Cfg::BUFS;
    constexpr float inv_part = 1.0f / static_cast<float>(CPW * 32);
    constexpr float inv_n = 1.0f / static_cast<float>(N);
    const uint32_t leader_tempty0 = map_to_cta(&tmem_empty[0], 0);
    const bool bf16_out = kBf16 && args.out_bf16;
    uint32_t rph = 0;                                     // bit b: parity of the next completion of my_res_full[b]
    int it = 0;
    bool ok = true;
    // residual boxes of a tile: chunk cc of this warp's range goes to buffer cc % BUFS
    auto fetch_res = [&](int tile, int cc) {
      const int b = cc % Cfg::BUFS;
      mbar_expect_tx(&my_res_full[b], Cfg::RES_BOX_BYTES);
      tma_load_2d(my_bufs + b * Cfg::BUF_BYTES, &tmap_res, &my_res_full[b], (chunk0 + cc) * 32,
                  tile * 256 + static_cast<int>(rank) * 128 + quad * 32);
    };
    if (has_res && lane == 0 && pair < args.num_tiles) {
#pragma unroll
      for (int cc = 0; cc < (CPW < Cfg::BUFS ? CPW : Cfg::BUFS); ++cc) fetch_res(pair, cc);
    }
    for (int tile = pair; tile < args.num_tiles && ok; tile += num_pairs, ++it) {
      const int acc = it % ACCS;
      const uint32_t acc_phase = (it / ACCS) & 1u;
      const int row0 = tile * 256 + static_cast<int>(rank) * 128 + quad * 32;   // first row of this warp's 32
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag)) { fail(ERR_WAIT_TMEM_FULL); break; }
      tc_fence_after();
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * N + chunk0 * 32;
      uint32_t ra[32], rb[32];
      // ---------------- pass 1: v = acc + bias + residual -> TMEM; shifted sums for the statistics of the range
      float shift = 0.f, s1 = 0.f, s2 = 0.f;
      __syncwarp();
      tmem_ld_32x32(taddr_row, ra);
#pragma unroll
      for (int cc = 0; cc < CPW; ++cc) {
        uint32_t (&cur)[32] = (cc & 1) ? rb : ra;
        uint32_t (&nxt)[32] = (cc & 1) ? ra : rb;
        __syncwarp();
        tmem_ld_wait();
        if (cc + 1 < CPW) tmem_ld_32x32(taddr_row + (cc + 1) * 32, nxt);
        if (has_res) {
          const int b = cc % Cfg::BUFS;
          if (ok && !mbar_wait(&my_res_full[b], (rph >> b) & 1u, abort_flag)) { fail(ERR_WAIT_FULL); ok = false; }
          rph ^= 1u << b;
          const uint8_t* rp = my_bufs + b * Cfg::BUF_BYTES;
          if constexpr (kBf16) {
            // plain row-major box: 64 bytes per row
            const uint4* q4 = reinterpret_cast<const uint4*>(rp + lane * 64);
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
            // 128-byte swizzle: 16-byte piece q of row r lives at piece (q ^ (r & 7))
            const uint8_t* rowp = rp + lane * 128;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 w = *reinterpret_cast<const float4*>(rowp + ((q ^ (lane & 7)) << 4));
              cur[4 * q] = __float_as_uint(__uint_as_float(cur[4 * q]) + w.x);
              cur[4 * q + 1] = __float_as_uint(__uint_as_float(cur[4 * q + 1]) + w.y);
              cur[4 * q + 2] = __float_as_uint(__uint_as_float(cur[4 * q + 2]) + w.z);
              cur[4 * q + 3] = __float_as_uint(__uint_as_float(cur[4 * q + 3]) + w.w);
            }
          }
          if (cc + Cfg::BUFS < CPW) {                     // the buffer is read: the box after next may land in it
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && ok) fetch_res(tile, cc + Cfg::BUFS);
          }
        }
        const int col = (chunk0 + cc) * 32;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 b4 = *reinterpret_cast<const float4*>(s_bias + col + 4 * q);
          cur[4 * q] = __float_as_uint(__uint_as_float(cur[4 * q]) + b4.x);
          cur[4 * q + 1] = __float_as_uint(__uint_as_float(cur[4 * q + 1]) + b4.y);
          cur[4 * q + 2] = __float_as_uint(__uint_as_float(cur[4 * q + 2]) + b4.z);
          cur[4 * q + 3] = __float_as_uint(__uint_as_float(cur[4 * q + 3]) + b4.w);
        }
        if (cc == 0) shift = __uint_as_float(cur[0]);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float d = __uint_as_float(cur[j]) - shift;
          s1 += d;
          s2 = fmaf(d, d, s2);
        }
        tmem_st_32x32(taddr_row + cc * 32, cur);
      }
      tmem_st_wait();
      if (!ok) break;
      // ---------------- statistics of the whole row: the SUB ranges of a row meet in shared memory
      const float md = s1 * inv_part;
      const float mean_a = shift + md;
      const float m2_a = fmaxf(fmaf(-md, s1, s2), 0.f);            // sum (v - mean_a)^2 over this range
      float2* part = s_part + acc * (SUB * 128);
      part[sub * 128 + trow] = make_float2(mean_a, m2_a);
      mbar_arrive(&part_bar[acc * 4 + quad]);
      if (!mbar_wait(&part_bar[acc * 4 + quad], acc_phase, abort_flag)) { fail(ERR_WAIT_TMEM_FULL); break; }
      float mean = 0.f;
#pragma unroll
      for (int s = 0; s < SUB; ++s) mean += part[s * 128 + trow].x;
      mean *= 1.0f / static_cast<float>(SUB);
      float m2 = 0.f;
#pragma unroll
      for (int s = 0; s < SUB; ++s) {
        const float2 p = part[s * 128 + trow];
        const float dm = p.x - mean;
        m2 += fmaf(dm * dm, static_cast<float>(CPW * 32), p.y);
      }
      const float var = m2 * inv_n;
      float rstd = rsqrtf(var + args.eps);
      rstd = rstd * (1.5f - 0.5f * (var + args.eps) * rstd * rstd);   // one Newton step: the rounding of 1/sqrt
      // ---------------- pass 2: normalise, scale, shift, store
      __syncwarp();
      tmem_ld_32x32(taddr_row, ra);
#pragma unroll
      for (int cc = 0; cc < CPW; ++cc) {
        uint32_t (&cur)[32] = (cc & 1) ? rb : ra;
        uint32_t (&nxt)[32] = (cc & 1) ? ra : rb;
        __syncwarp();
        tmem_ld_wait();
        if (cc + 1 < CPW) tmem_ld_32x32(taddr_row + (cc + 1) * 32, nxt);
        uint8_t* stg = my_bufs + (cc % Cfg::BUFS) * Cfg::BUF_BYTES;
        // this buffer is free once the bulk store committed BUFS groups ago has READ it
        if (lane == 0) tma_store_wait_read<Cfg::BUFS - 1>();
        __syncwarp();
        const int col = (chunk0 + cc) * 32;
        // four columns at a time, finished and put away, so that few values are live at once
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 g4 = *reinterpret_cast<const float4*>(s_gamma + col + 4 * q);
          const float4 b4 = *reinterpret_cast<const float4*>(s_beta + col + 4 * q);
          float4 o;
          o.x = fmaf((__uint_as_float(cur[4 * q]) - mean) * rstd, g4.x, b4.x);
          o.y = fmaf((__uint_as_float(cur[4 * q + 1]) - mean) * rstd, g4.y, b4.y);
          o.z = fmaf((__uint_as_float(cur[4 * q + 2]) - mean) * rstd, g4.z, b4.z);
          o.w = fmaf((__uint_as_float(cur[4 * q + 3]) - mean) * rstd, g4.w, b4.w);
          if (args.round_tf32) { o.x = round_to_tf32(o.x); o.y = round_to_tf32(o.y); o.z = round_to_tf32(o.z); o.w = round_to_tf32(o.w); }
          if (bf16_out) {
            // 64-byte rows under the tensor map's 64-byte swizzle: 16-byte piece p of row r lives at piece p ^ ((r >> 1) & 3)
            uint2 pk;
            pk.x = pack_bf16x2(o.x, o.y);
            pk.y = pack_bf16x2(o.z, o.w);
            *reinterpret_cast<uint2*>(stg + lane * 64 + ((((q >> 1) ^ ((lane >> 1) & 3)) << 4) | ((q & 1) << 3))) = pk;
          } else {
            *reinterpret_cast<float4*>(stg + lane * 128 + ((q ^ (lane & 7)) << 4)) = o;    // the tensor map's 128-byte swizzle
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (row0 < args.M) tma_store_2d(&tmap_out, stg, col, row0);   // rows beyond M are clipped
          tma_store_commit();    // an empty group when nothing was stored: the group count stays in step
        }
      }
      // this warp has finished reading the accumulator
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tempty0 + acc * 8);
      // the next tile's first residual boxes go into the buffers once the bulk stores have read them
      const int next = tile + num_pairs;
      if (has_res && next < args.num_tiles) {
        if (lane == 0) {
          tma_store_wait_read<0>();
#pragma unroll
          for (int cc = 0; cc < (CPW < Cfg::BUFS ? CPW : Cfg::BUFS); ++cc) fetch_res(next, cc);
        }
        __syncwarp();
      }
    }
    if (lane == 0) tma_store_wait_all<0>();   // staging memory outlives the last bulk store's read; the data has landed
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);   // let copies and MMAs in flight land (about 1 ms)
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                                        // neither CTA frees TMEM or exits while the other still uses it
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace gb
