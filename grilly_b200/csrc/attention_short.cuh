// Short-sequence attention (every sequence fits one 128-key tile, no RoPE, no causal mask): the MiniLM encoder case.
//
// The work unit is (sequence, range of heads). For one head the chain  S = Q K^T -> softmax -> O = P V -> store  is a
// string of dependent steps separated by tensor-core completion latencies, so one unit at a time leaves the SM
// mostly waiting. TMEM (512 columns, allocated in powers of two) would let only two independent CTAs of
// 128 + D columns share an SM; instead ONE persistent CTA per SM allocates all 512 columns and runs NSLOT
// independent "slots" (three for head_dim 32 in tf32, four in bf16), each with its own 160 threads (four softmax warps + one issuing
// warp), shared-memory tiles, barriers and TMEM columns. A slot takes the next unit from a global counter, so
// long and short sequences balance out. With a single key tile there is no running-max rescale: row max, exp,
// row sum, P V, divide.
#pragma once
#include "attention.cuh"

namespace gb {

template <int D, bool kBf16>
struct AttnShortCfg {
  static constexpr int ELT = kBf16 ? 2 : 4;
  static constexpr int ROW_BYTES = D * ELT;                       // bytes of one head in a token row
  static_assert(ROW_BYTES == 64 || ROW_BYTES == 128 || ROW_BYTES == 256, "head_dim*elt must be 64, 128 or 256 bytes");
  // A 64-byte head (head_dim 32 in bf16) is loaded together with its neighbour: the 128-byte swizzled row then
  // holds two heads side by side and each head's MMAs start 0 or 64 bytes into the row.
  static constexpr int HPR = ROW_BYTES < 128 ? 128 / ROW_BYTES : 1;   // heads per loaded row chunk
  static constexpr int NCH = ROW_BYTES <= 128 ? 1 : ROW_BYTES / 128;
  static constexpr int TILE_BYTES = NCH * ATTN_CHUNK_BYTES;       // one of Q, K, V
  // TMEM columns of a slot: S/P at [0,128), O at [128,128+D). With bf16 and head_dim <= 64 the packed P fills only
  // [0,64) of the score columns, so O goes to [64,64+D) of the same region, a slot is 128 columns and four fit.
  static constexpr bool SHARE_O = kBf16 && D <= 64;
  static constexpr int SLOT_COLS = SHARE_O ? ATTN_TILE : ATTN_TILE + D;
  static constexpr int O_COL = SHARE_O ? 64 : ATTN_TILE;
  static constexpr int NSLOT = SHARE_O ? 4 : (3 * SLOT_COLS <= 512 ? 3 : 2);
  static_assert(NSLOT * SLOT_COLS <= 512, "slots must fit TMEM");
  static constexpr int SLOT_THREADS = 160;
  static constexpr int THREADS = NSLOT * SLOT_THREADS;
  static constexpr int SLOT_SMEM = 3 * TILE_BYTES;                // Q, K, V of one head (or head pair)
  static constexpr int CTRL_BYTES = 96;                           // per slot: 6 barriers, the unit with its first row and length, key-mask words
  // fp32 rows of 32 features (128 bytes) leave the SM through a staging tile per softmax warp (32 rows x 128 B), so
  // that a store instruction writes four whole rows instead of a 16-byte piece of 32 rows; the other shapes have no
  // shared memory left for it and store from registers
  static constexpr bool STAGE_OUT = !kBf16 && D == 32;
  static constexpr int STAGE_BYTES = STAGE_OUT ? ATTN_TILE * 128 : 0;   // per slot
  static constexpr int STAGE_OFF = NSLOT * SLOT_SMEM;
  static constexpr int CTRL_OFF = STAGE_OFF + NSLOT * STAGE_BYTES;
  static constexpr int SMEM_BYTES = CTRL_OFF + 1024 + NSLOT * CTRL_BYTES + 64;
  static constexpr int TMEM_COLS = 512;
};

// Tensor maps of Q, K and V with boxes of 32, 64, 96 and 128 token rows: a unit fetches only as many rows as its
// sentence has (rounded up to 32), not the whole 128-row tile, so that the copy engine moves about the algorithmic
// bytes and a short sentence's tiles arrive sooner (its chain of dependent steps starts with these loads).
struct AttnShortMaps {
  CUtensorMap q[4], k[4], v[4];
};

// barrier over the `count` threads that name the same id (ids 1..15; 0 is __syncthreads)
__device__ __forceinline__ void named_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(AttnShortCfg<D, kBf16>::THREADS, 1)
flash_attn_short_kernel(const __grid_constant__ AttnShortMaps maps, const AttnArgs args, int heads_per_unit,
                        int head_groups, int total_units, int* work_counter) {
  using Cfg = AttnShortCfg<D, kBf16>;
  constexpr int ELT = Cfg::ELT;
  constexpr int NCH = Cfg::NCH;
  constexpr int HPR = Cfg::HPR;
  constexpr int CHE = 128 / ELT;
  constexpr int UMMA_K = 32 / ELT;
  constexpr int TILE_BYTES = Cfg::TILE_BYTES;
  constexpr uint32_t IDESC_S = make_idesc(kBf16, 128, ATTN_TILE, false, false);
  constexpr uint32_t IDESC_O = make_idesc(kBf16, 128, D, false, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int slot = threadIdx.x / Cfg::SLOT_THREADS;
  const int t = threadIdx.x % Cfg::SLOT_THREADS;            // thread within the slot
  const int warp = t >> 5;                                  // 0..3 softmax (one query row per thread), 4 issuer
  const int lane = t & 31;
  uint8_t* tiles = smem + slot * Cfg::SLOT_SMEM;            // Q | K | V
  uint8_t* ctrl = smem + Cfg::CTRL_OFF + slot * Cfg::CTRL_BYTES;
  uint64_t* bar_qk = reinterpret_cast<uint64_t*>(ctrl);     // Q and K of a head (pair) landed
  uint64_t* bar_v = bar_qk + 1;                             // V landed
  uint64_t* bar_s = bar_qk + 2;                             // S complete
  uint64_t* bar_p = bar_qk + 3;                             // P written (one arrive per softmax warp)
  uint64_t* bar_o = bar_qk + 4;                             // O complete
  uint64_t* bar_or = bar_qk + 5;                            // O read out of TMEM (only when it shares columns with the next S)
  volatile int* slot_unit = reinterpret_cast<volatile int*>(ctrl + 48);   // [0] unit, [1] its first packed row, [2] its length
  uint32_t* s_keep = reinterpret_cast<uint32_t*>(ctrl + 64);   // [4] key-mask bit words of the slot's sequence
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + Cfg::CTRL_OFF + Cfg::NSLOT * Cfg::CTRL_BYTES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  if (t == 0) {
    mbar_init(bar_qk, 1); mbar_init(bar_v, 1); mbar_init(bar_s, 1); mbar_init(bar_p, 4); mbar_init(bar_o, 1);
    mbar_init(bar_or, 4);
    if (slot == 0) {
      *abort_flag = 0;
      for (int i = 0; i < 4; ++i) { prefetch_tmap(&maps.q[i]); prefetch_tmap(&maps.k[i]); prefetch_tmap(&maps.v[i]); }
    }
    fence_mbar_init();
  }
  if (slot == 0 && warp == 4) {
    tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s = tmem_base + slot * Cfg::SLOT_COLS;
  const uint32_t tmem_o = tmem_s + Cfg::O_COL;

#define ATTN_FAIL()                                         \
  do {                                                      \
    if (!*abort_flag) atomicCAS(args.err, 0, ERR_WAIT_ATTN); \
    *abort_flag = 1;                                        \
  } while (0)

  // Barrier phases run on across units: both roles count the heads (and loaded head groups) they have been through.
  uint32_t heads_done = 0, groups_done = 0;

  // The issuing thread knows the slot's units one ahead: while a unit runs it takes the following one from the counter,
  // looks up its rows and, during the unit's last head, sends for the first Q, K and V of the following unit, so that a
  // unit does not start with the round trips of an atomic, two loads and three copies in a row.
  int nx_unit = -1, nx_row0 = 0, nx_L = 0;    // issuing thread only: the unit this slot runs next
  bool nx_loaded = false;                     // ... and whether its first Q, K, V are on their way already
  auto unit_rows = [&](int u, int& r0, int& len) {
    const int bb = u / head_groups;
    if (args.cu_seqlens) {
      r0 = __ldg(args.cu_seqlens + bb);
      len = __ldg(args.cu_seqlens + bb + 1) - r0;
    } else {
      r0 = bb * args.S;
      len = args.S;
    }
  };
  if (t == Cfg::SLOT_THREADS - 32) {
    nx_unit = atomicAdd(work_counter, 1);
    if (nx_unit >= total_units) nx_unit = -1;
    if (nx_unit >= 0) unit_rows(nx_unit, nx_row0, nx_L);
  }

  while (true) {
    // ---- this unit: published by the issuing thread to the slot through shared memory
    if (t == Cfg::SLOT_THREADS - 32) {
      if (*abort_flag) nx_unit = -1;
      slot_unit[0] = nx_unit;
      slot_unit[1] = nx_row0;
      slot_unit[2] = nx_L;
    }
    named_barrier(1 + slot, Cfg::SLOT_THREADS);
    const int unit = slot_unit[0];
    if (unit < 0) break;
    const int row0 = slot_unit[1], L = slot_unit[2];
    const int b = unit / head_groups;
    const int h_begin = (unit % head_groups) * heads_per_unit;
    const int h_end = min(args.H, h_begin + heads_per_unit);
    const bool has_work = L > 0 && h_begin < h_end;          // uniform over the slot
    const int n_s = (L + 31) & ~31;                          // score columns computed (N = 16 mod 32 runs the MMA much slower)
    const int nchunks = (L + 31) >> 5;                       // 32-key chunks with a valid key
    const int ksteps = (L + UMMA_K - 1) / UMMA_K;            // k-steps of P V that cover valid keys

    if (warp == 4) {
      if (lane == 0) {
        // -------------------------------------------------------- TMA + MMA issuer
        const bool loaded = nx_loaded;          // this unit's first Q, K, V were sent for during the previous unit
        int taken = -1;                         // the following unit: the atomic's round trip hides behind this unit's copies
        if (!*abort_flag) taken = atomicAdd(work_counter, 1);
        bool nx_known = false;
        nx_unit = -1;
        nx_loaded = false;
        auto know_next = [&]() {
          if (nx_known) return;
          nx_known = true;
          nx_unit = (taken >= 0 && taken < total_units) ? taken : -1;
          if (nx_unit >= 0) unit_rows(nx_unit, nx_row0, nx_L);
        };
        if (has_work) {
          const uint32_t idesc_s = (IDESC_S & ~(0x3Fu << 17)) | (static_cast<uint32_t>(n_s >> 3) << 17);
          // Q and K of the next head (pair) may be fetched as soon as S is complete, V once P V is complete
          // boxes of n_s rows (32, 64, 96 or 128): rows beyond them keep whatever the slot's previous unit left, which
          // no MMA result that is stored depends on (S columns and P V k-steps stop at n_s, query rows >= L are not stored)
          auto load_qk = [&](int h, int r0, int ns) {
            const int bi = (ns >> 5) - 1;
            mbar_expect_tx(bar_qk, 2u * static_cast<uint32_t>(ns) * 128u * NCH);
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
              tma_load_2d(tiles + c * ATTN_CHUNK_BYTES, &maps.q[bi], bar_qk, h * D + c * CHE, r0);
              tma_load_2d(tiles + TILE_BYTES + c * ATTN_CHUNK_BYTES, &maps.k[bi], bar_qk, h * D + c * CHE, r0);
            }
          };
          auto load_v = [&](int h, int r0, int ns) {
            const int bi = (ns >> 5) - 1;
            mbar_expect_tx(bar_v, static_cast<uint32_t>(ns) * 128u * NCH);
#pragma unroll
            for (int c = 0; c < NCH; ++c)
              tma_load_2d(tiles + 2 * TILE_BYTES + c * ATTN_CHUNK_BYTES, &maps.v[bi], bar_v, h * D + c * CHE, r0);
          };
          if (!loaded) {
            load_qk(h_begin, row0, n_s);
            load_v(h_begin, row0, n_s);
          }
          for (int h = h_begin; h < h_end; ++h) {
            const uint32_t ph = heads_done & 1u;
            const int u = (h - h_begin) % HPR;                 // position of this head inside its loaded group
            const bool last = h + 1 == h_end;
            const bool group_ends = u == HPR - 1 || last;
            if (u == 0 && !mbar_wait(bar_qk, groups_done & 1u, abort_flag)) { ATTN_FAIL(); break; }
            if constexpr (Cfg::SHARE_O) {
              // these scores overwrite the columns that hold O of the slot's previous head: wait until it has been read
              if (heads_done > 0 && !mbar_wait(bar_or, (heads_done - 1) & 1u, abort_flag)) { ATTN_FAIL(); break; }
            }
            tc_fence_after();
            const uint32_t sQ = smem_u32(tiles) + u * Cfg::ROW_BYTES, sK = sQ + TILE_BYTES, sV = sK + TILE_BYTES;
#pragma unroll
            for (int ks = 0; ks < D / UMMA_K; ++ks) {
              const int chunk = (ks * 32) / 128, off = (ks * 32) % 128;
              umma_ss<kBf16>(tmem_s, make_smem_desc_sw128(sQ + chunk * ATTN_CHUNK_BYTES + off, 16, 1024),
                             make_smem_desc_sw128(sK + chunk * ATTN_CHUNK_BYTES + off, 16, 1024), idesc_s, ks != 0 ? 1u : 0u);
            }
            umma_commit(bar_s);
            if (h == h_begin) know_next();   // two loads that are back long before the unit's last head asks for them
            // the following unit's first head group, if it has one: fetched under this unit's last head
            const int nx_h = (nx_unit % head_groups) * heads_per_unit;
            const int nx_ns = (nx_L + 31) & ~31;
            const bool fetch_next = last && nx_unit >= 0 && nx_L > 0 && nx_h < args.H;
            if (group_ends && !last) {
              // S is the last reader of Q and K: fetch the next head's while this head is in its softmax
              if (!mbar_wait(bar_s, ph, abort_flag)) { ATTN_FAIL(); break; }
              load_qk(h + 1, row0, n_s);
            } else if (fetch_next) {
              if (!mbar_wait(bar_s, ph, abort_flag)) { ATTN_FAIL(); break; }
              load_qk(nx_h, nx_row0, nx_ns);
            }
            if (!mbar_wait(bar_p, ph, abort_flag)) { ATTN_FAIL(); break; }
            if (u == 0 && !mbar_wait(bar_v, groups_done & 1u, abort_flag)) { ATTN_FAIL(); break; }
            tc_fence_after();
            for (int ks = 0; ks < ksteps; ++ks)
              umma_ts<kBf16>(tmem_o, tmem_s + ks * 8, make_smem_desc_mn<kBf16>(sV + ks * (UMMA_K * 128), ATTN_CHUNK_BYTES), IDESC_O,
                             ks != 0 ? 1u : 0u);
            umma_commit(bar_o);
            if (!mbar_wait(bar_o, ph, abort_flag)) { ATTN_FAIL(); break; }
            if (group_ends && !last) {
              load_v(h + 1, row0, n_s);
            } else if (fetch_next) {
              load_v(nx_h, nx_row0, nx_ns);
              nx_loaded = true;
            }
            if (group_ends) ++groups_done;
            ++heads_done;
          }
        }
        know_next();
      }
    } else if (has_work) {
      // ---------------------------------------------------------- softmax / output threads (one query row each)
      // a warp reaches only the TMEM lane quadrant given by its warp index in the CTA modulo 4; the four softmax
      // warps of a slot have consecutive indices, so between them they cover the four quadrants (= 128 query rows)
      const int quad = (threadIdx.x >> 5) & 3;
      const int qrow = quad * 32 + lane;                     // this thread's query row within the tile
      const bool warp_active = quad * 32 < L;
      const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
      const float sl2 = args.scale * 1.4426950408889634f;   // scores enter exp2 as s * scale * log2(e)
      const float* kmask = args.key_mask ? args.key_mask + static_cast<long long>(b) * args.S : nullptr;
      if (kmask) {
        if (t < 4) {
          // the key mask is the same for every head and query of the sequence: 4 bit words, built once
          uint32_t w = 0;
          for (int j = 0; j < 32; ++j) {
            const int kidx = t * 32 + j;
            if (kidx < L && __ldg(kmask + kidx) >= 0.5f) w |= 1u << j;
          }
          s_keep[t] = w;
        }
        named_barrier(1 + Cfg::NSLOT + slot, 128);           // the slot's softmax warps only
      }
      for (int h = h_begin; h < h_end; ++h) {
        const uint32_t ph = heads_done & 1u;
        if (!mbar_wait(bar_s, ph, abort_flag)) { ATTN_FAIL(); break; }
        tc_fence_after();
        float l_sum = 0.f;
        // bf16 without a key mask takes one sweep over the scores; tf32 (twice the registers per P chunk: measured slower
        // with one sweep) and masked launches take two
        if (warp_active && (!kBf16 || kmask)) {
          // pass 1: row maximum (scale > 0 is folded in afterwards). Per 32-key chunk two bit words say which columns
          // exist (validw: key < L) and which also pass the key mask (keepw); a full, unmasked chunk takes the plain path.
          float m_raw = -INFINITY;
          bool any_masked = false;
#pragma unroll 1
          for (int c = 0; c < nchunks; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_s + lane_addr + c * 32, r);
            tmem_ld_wait();
            const uint32_t validw = prefix_bits(L - c * 32);
            const uint32_t keepw = kmask ? s_keep[c] : validw;
            if (keepw != 0xffffffffu) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (!((keepw >> j) & 1u)) r[j] = 0xff800000u;   // -inf: absent or masked keys do not set the maximum
              any_masked = any_masked || (validw & ~keepw) != 0u;
            }
            m_raw = fmaxf(m_raw, row_max32(r));
          }
          // masked keys carry the score -1e9 (the reference adds (mask-1)*1e9): they only matter when every key is masked
          float m_sc = m_raw * args.scale;
          if (any_masked) m_sc = fmaxf(m_sc, -1e9f);
          const float m_l2 = m_sc * 1.4426950408889634f;
          const float x_masked = -1e9f * 1.4426950408889634f - m_l2;
          // pass 2: p = exp(s - m), row sum, P written over S
#pragma unroll 1
          for (int c = 0; c < nchunks; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_s + lane_addr + c * 32, r);
            tmem_ld_wait();
            float p[32];
            const uint32_t validw = prefix_bits(L - c * 32);
            const uint32_t keepw = kmask ? s_keep[c] : validw;
            if (keepw != 0xffffffffu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float x = fmaf(__uint_as_float(r[j]), sl2, -m_l2);
                x = ((keepw >> j) & 1u) ? x : (((validw >> j) & 1u) ? x_masked : -INFINITY);
                p[j] = fast_exp2(x);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) p[j] = fast_exp2(fmaf(__uint_as_float(r[j]), sl2, -m_l2));
            }
            if constexpr (kBf16) {
              uint32_t pk[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(p[2 * j], p[2 * j + 1]);
              l_sum += row_sum32(p);
              tmem_st_32x16(tmem_s + lane_addr + c * 16, pk);
            } else {
              uint32_t pk[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                p[j] = round_to_tf32(p[j]);
                pk[j] = __float_as_uint(p[j]);
              }
              l_sum += row_sum32(p);
              tmem_st_32x32(tmem_s + lane_addr + c * 32, pk);
            }
          }
          tmem_st_wait();
        } else if (warp_active) {
          // No key mask: ONE sweep over the scores. The exponentials refer to an integer-valued reference point (log2
          // units, scale folded in) that the first chunk sets and a later chunk moves only if its maximum has outgrown
          // it by more than 2^8; the P chunks and the row sum accumulated so far are then scaled by the exact power of
          // two (rare). The reference point cancels in O / l.
          float m_ref = -INFINITY;
#pragma unroll 1
          for (int c = 0; c < nchunks; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_s + lane_addr + c * 32, r);
            tmem_ld_wait();
            const uint32_t validw = prefix_bits(L - c * 32);
            if (validw != 0xffffffffu) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (!((validw >> j) & 1u)) r[j] = 0xff800000u;   // -inf: absent keys neither set the maximum nor add to the sum
            }
            const float cmax = row_max32(r) * sl2;               // scale > 0 in this kernel
            const bool move = cmax > m_ref + 8.0f || m_ref == -INFINITY;
            if (__any_sync(0xffffffffu, move)) {
              float a = 1.f;
              if (move) {
                const float new_ref = ceilf(cmax);
                const float k = m_ref - new_ref;                 // integer-valued, <= 0 (or -inf)
                a = k < -126.f ? 0.f : __int_as_float((static_cast<int>(k) + 127) << 23);
                m_ref = new_ref;
              }
              tmem_st_wait();
              for (int cc = 0; cc < c; ++cc) {
                if constexpr (kBf16) {
                  uint32_t q[16];
                  tmem_ld_32x16(tmem_s + lane_addr + cc * 16, q);
                  tmem_ld_wait();
#pragma unroll
                  for (int j = 0; j < 16; ++j)
                    q[j] = pack_bf16x2(__uint_as_float(q[j] << 16) * a, __uint_as_float(q[j] & 0xffff0000u) * a);
                  tmem_st_32x16(tmem_s + lane_addr + cc * 16, q);
                } else {
                  uint32_t q[32];
                  tmem_ld_32x32(tmem_s + lane_addr + cc * 32, q);
                  tmem_ld_wait();
#pragma unroll
                  for (int j = 0; j < 32; ++j) q[j] = __float_as_uint(__uint_as_float(q[j]) * a);
                  tmem_st_32x32(tmem_s + lane_addr + cc * 32, q);
                }
              }
              l_sum *= a;
            }
            float p[32];
            const float neg_m = -m_ref;
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float x0, x1;
              fma_f32x2(x0, x1, __uint_as_float(r[j]), __uint_as_float(r[j + 1]), sl2, sl2, neg_m, neg_m);
              p[j] = fast_exp2(x0);
              p[j + 1] = fast_exp2(x1);
            }
            if constexpr (kBf16) {
              uint32_t pk[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(p[2 * j], p[2 * j + 1]);
              l_sum += row_sum32(p);
              tmem_st_32x16(tmem_s + lane_addr + c * 16, pk);
            } else {
              uint32_t pk[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                p[j] = round_to_tf32(p[j]);
                pk[j] = __float_as_uint(p[j]);
              }
              l_sum += row_sum32(p);
              tmem_st_32x32(tmem_s + lane_addr + c * 32, pk);
            }
          }
          tmem_st_wait();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p);

        if (!mbar_wait(bar_o, ph, abort_flag)) { ATTN_FAIL(); break; }
        tc_fence_after();
        if (warp_active) {
          const float inv = 1.f / l_sum;
          const long long orow = static_cast<long long>(row0 + qrow) * args.ld_out + h * D;
          const bool row_ok = qrow < L;
          const bool stage_ok = Cfg::STAGE_OUT && !args.out_bf16 && (args.ld_out % 4 == 0) &&
                                ((reinterpret_cast<uintptr_t>(args.out) & 15) == 0);
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_o + lane_addr + c * 32, r);
            tmem_ld_wait();
            if constexpr (Cfg::STAGE_OUT) {
              if (stage_ok) {
                // lane = row: the row's eight 16-byte pieces go to the warp's staging tile, piece j of row l at
                // position j ^ (l & 7) (no bank conflicts either way); then lane l stores piece l % 8 of rows
                // 4 k + l / 8, so that eight lanes write one whole 128-byte row
                uint8_t* stg = smem + Cfg::STAGE_OFF + slot * Cfg::STAGE_BYTES + quad * 4096;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  float4 q = make_float4(__uint_as_float(r[4 * j]) * inv, __uint_as_float(r[4 * j + 1]) * inv,
                                         __uint_as_float(r[4 * j + 2]) * inv, __uint_as_float(r[4 * j + 3]) * inv);
                  if (args.round_tf32) {
                    q.x = round_to_tf32(q.x); q.y = round_to_tf32(q.y); q.z = round_to_tf32(q.z); q.w = round_to_tf32(q.w);
                  }
                  *reinterpret_cast<float4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = q;
                }
                __syncwarp();
                const int piece = lane & 7;
                float* obase = reinterpret_cast<float*>(args.out) + static_cast<long long>(row0 + quad * 32) * args.ld_out + h * D + piece * 4;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                  const int rr = 4 * k + (lane >> 3);
                  const float4 q = *reinterpret_cast<const float4*>(stg + rr * 128 + ((piece ^ (rr & 7)) << 4));
                  if (quad * 32 + rr < L) *reinterpret_cast<float4*>(obase + static_cast<long long>(rr) * args.ld_out) = q;
                }
                __syncwarp();
                continue;
              }
            }
            if (row_ok) {
              if (args.out_bf16) {
                __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(args.out) + orow + c * 32;
                const bool v8 = (args.ld_out % 8 == 0) && ((reinterpret_cast<uintptr_t>(args.out) & 15) == 0);
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  uint4 q;   // eight bf16 per 16-byte store
                  q.x = pack_bf16x2(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv);
                  q.y = pack_bf16x2(__uint_as_float(r[j + 2]) * inv, __uint_as_float(r[j + 3]) * inv);
                  q.z = pack_bf16x2(__uint_as_float(r[j + 4]) * inv, __uint_as_float(r[j + 5]) * inv);
                  q.w = pack_bf16x2(__uint_as_float(r[j + 6]) * inv, __uint_as_float(r[j + 7]) * inv);
                  if (v8) *reinterpret_cast<uint4*>(op + j) = q;
                  else {
                    uint32_t* o32 = reinterpret_cast<uint32_t*>(op + j);   // head offsets are even: 4-byte aligned
                    o32[0] = q.x; o32[1] = q.y; o32[2] = q.z; o32[3] = q.w;
                  }
                }
              } else {
                float* op = reinterpret_cast<float*>(args.out) + orow + c * 32;
                const bool v4 = (args.ld_out % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.out) & 15) == 0);
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  float4 q = make_float4(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv,
                                         __uint_as_float(r[j + 2]) * inv, __uint_as_float(r[j + 3]) * inv);
                  if (args.round_tf32) {
                    q.x = round_to_tf32(q.x); q.y = round_to_tf32(q.y); q.z = round_to_tf32(q.z); q.w = round_to_tf32(q.w);
                  }
                  if (v4) *reinterpret_cast<float4*>(op + j) = q;
                  else { op[j] = q.x; op[j + 1] = q.y; op[j + 2] = q.z; op[j + 3] = q.w; }
                }
              }
            }
            __syncwarp();
          }
        }
        tc_fence_before();   // O and P of this head are consumed before the next head's MMAs may overwrite them
        if constexpr (Cfg::SHARE_O) {
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_or);
        }
        ++heads_done;
      }
    }
  }
#undef ATTN_FAIL

  if (*abort_flag) {
    for (int k = 0; k < 100; ++k) __nanosleep(10000);   // let copies and MMAs in flight land (about 1 ms)
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (slot == 0 && warp == 4) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace gb
