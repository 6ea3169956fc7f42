// Flash-attention forward on tcgen05 for sm_100a: softmax(scale * Q K^T + mask) V
// without materialising the score matrix.
//
// Data layout: Q, K, V and the output are row-major 2-D views [token rows][width];
// head h of a token occupies columns [h*D, (h+1)*D). That covers the (B,S,H,D)
// layout of flash_attention2 (width = H*D, three tensors) and a packed QKV
// projection output (width = 3*H*D, three base pointers into one buffer).
// Sequences are either padded (batch b owns rows [b*S, (b+1)*S)) or packed
// back to back with cu_seqlens[b] giving the first row of sequence b.
//
// One CTA handles 128 queries of one (sequence, head). Warp 4 (one lane) issues
// TMA loads and tcgen05.mma; warps 0..3 own one query row per thread:
//   S = Q K_j^T  (smem x smem -> TMEM, 128 fp32 columns)
//   row max / exp2 / row sum in registers, P written back over S in TMEM
//   O_j = P V_j  (P read from TMEM, V is the MN-major smem operand, read as loaded) -> TMEM
//   O += O_j with the running-max rescale kept in registers.
// RoPE (interleaved or rotate-half pairs) is applied to the Q and K tiles in
// shared memory right after the TMA load, before the first MMA reads them.
#pragma once
#include "ptx.cuh"
#include "gemm.cuh"  // round_to_tf32
#include <cuda_bf16.h>

namespace gb {



constexpr int ATTN_THREADS = 160;
constexpr int ATTN_TILE = 128;       // queries per CTA and keys per step
constexpr int ATTN_CHUNK_BYTES = ATTN_TILE * 128;  // one 128-row x 128-B swizzled chunk

template <int D, bool kBf16>
struct AttnCfg {
  static constexpr int ELT = kBf16 ? 2 : 4;
  static constexpr int NCH = D * ELT / 128;            // 128-B chunks per Q/K/V row
  static_assert(D * ELT % 128 == 0 && NCH >= 1 && NCH <= 4 && D <= 128, "head_dim*elt must be 128, 256, 384 or 512 bytes");
  static constexpr int Q_BYTES = NCH * ATTN_CHUNK_BYTES;
  static constexpr int SMEM_BYTES = 3 * Q_BYTES + 1024 + 128;
  // TMEM columns: S (fp32 scores, overwritten in place by P in the MMA operand precision) at [0,128),
  // O_j at [128, 128 + D): 256 columns, two CTAs per SM. With bf16 and head_dim <= 64 the packed P fills only
  // columns [0,64) of the score region, so O_j goes to [64, 64 + D) of the same region: 128 columns, and three or
  // four CTAs share an SM (the kernel is bound by the latency of its per-tile chain, so more chains in flight pay).
  static constexpr bool SHARE_O = kBf16 && D <= 64;
  static constexpr int TMEM_COLS = SHARE_O ? 128 : 256;
  static constexpr int O_COL = SHARE_O ? 64 : ATTN_TILE;
  static constexpr int MIN_CTAS = SHARE_O ? 3 : (D <= 64 ? 2 : 1);   // by TMEM columns; four would cap registers at 96 and spill (measured slower)
};

// low n bits set (n <= 0 -> none, n >= 32 -> all)
__device__ __forceinline__ uint32_t prefix_bits(int n) { return n >= 32 ? 0xffffffffu : (n <= 0 ? 0u : ((1u << n) - 1u)); }

// The softmax is bound by the instructions it issues per score. sm_100 has two-lane fp32 forms (one instruction
// multiplies-adds or adds two independent pairs) and a three-input maximum: they halve the multiply-adds and additions
// per score and cut a third of the maxima.
__device__ __forceinline__ void fma_f32x2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
  asm("{ .reg .b64 ra, rb, rc, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mov.b64 rc, {%6, %7};\n"
      " fma.rn.f32x2 rd, ra, rb, rc;\n mov.b64 {%0, %1}, rd; }"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void mul_f32x2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{ .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mul.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd; }"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void add_f32x2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{ .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n add.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd; }"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ float max3_f32(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Reductions over 32 registers with four independent chains (a single chain of 32 dependent ops is latency-bound).
__device__ __forceinline__ float row_max32(const uint32_t (&r)[32]) {
  float m[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    m[q] = max3_f32(__uint_as_float(r[8 * q]), __uint_as_float(r[8 * q + 1]), __uint_as_float(r[8 * q + 2]));
    m[q] = max3_f32(m[q], __uint_as_float(r[8 * q + 3]), __uint_as_float(r[8 * q + 4]));
    m[q] = max3_f32(m[q], __uint_as_float(r[8 * q + 5]), __uint_as_float(r[8 * q + 6]));
    m[q] = fmaxf(m[q], __uint_as_float(r[8 * q + 7]));
  }
  return fmaxf(max3_f32(m[0], m[1], m[2]), m[3]);
}
__device__ __forceinline__ float row_sum32(const float (&p)[32]) {
  float s0 = p[0], s1 = p[1], s2 = p[2], s3 = p[3];   // two two-lane chains
#pragma unroll
  for (int i = 4; i < 32; i += 4) {
    add_f32x2(s0, s1, s0, s1, p[i], p[i + 1]);
    add_f32x2(s2, s3, s2, s3, p[i + 2], p[i + 3]);
  }
  return (s0 + s1) + (s2 + s3);
}

// Rotate one row of a Q or K tile in place in swizzled shared memory.
template <int D, bool kBf16>
__device__ __forceinline__ void rope_row_inplace(uint8_t* tile, int r, int pos, const AttnArgs& a) {
  constexpr int ELT = kBf16 ? 2 : 4;
  constexpr int EPP = 16 / ELT;        // elements per 16-B piece
  constexpr int PIECES = D / EPP;      // pieces per row
  const float* ct = a.rope_cos + static_cast<long long>(pos) * (D / 2);
  const float* st = a.rope_sin + static_cast<long long>(pos) * (D / 2);
  auto piece_ptr = [&](int pc) -> uint4* {
    const int chunk = pc >> 3, within = pc & 7;
    return reinterpret_cast<uint4*>(tile + chunk * ATTN_CHUNK_BYTES + r * 128 + ((within ^ (r & 7)) << 4));
  };
  auto unpack = [&](const uint4& q, float* f) {
    if constexpr (kBf16) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    } else {
      f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
    }
  };
  auto pack = [&](const float* f) -> uint4 {
    uint4 q;
    if constexpr (kBf16) {
      __nv_bfloat162 h[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      q.x = *reinterpret_cast<uint32_t*>(&h[0]); q.y = *reinterpret_cast<uint32_t*>(&h[1]);
      q.z = *reinterpret_cast<uint32_t*>(&h[2]); q.w = *reinterpret_cast<uint32_t*>(&h[3]);
    } else {
      q.x = __float_as_uint(f[0]); q.y = __float_as_uint(f[1]); q.z = __float_as_uint(f[2]); q.w = __float_as_uint(f[3]);
    }
    return q;
  };
  if (a.rope_style == ROPE_INTERLEAVED) {
#pragma unroll
    for (int pc = 0; pc < PIECES; ++pc) {
      uint4* p = piece_ptr(pc);
      float f[EPP];
      unpack(*p, f);
      // pairs (pc*EPP/2 .. +EPP/2) are consecutive table entries: one vector load each for cos and sin
      float cs[EPP / 2], sn[EPP / 2];
      if constexpr (EPP == 8) {
        const float4 c4 = __ldg(reinterpret_cast<const float4*>(ct) + pc), s4 = __ldg(reinterpret_cast<const float4*>(st) + pc);
        cs[0] = c4.x; cs[1] = c4.y; cs[2] = c4.z; cs[3] = c4.w; sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
      } else {
        const float2 c2 = __ldg(reinterpret_cast<const float2*>(ct) + pc), s2 = __ldg(reinterpret_cast<const float2*>(st) + pc);
        cs[0] = c2.x; cs[1] = c2.y; sn[0] = s2.x; sn[1] = s2.y;
      }
#pragma unroll
      for (int e = 0; e < EPP; e += 2) {
        const float c = cs[e >> 1], s = sn[e >> 1];
        const float x0 = f[e], x1 = f[e + 1];
        f[e] = x0 * c - x1 * s;
        f[e + 1] = x0 * s + x1 * c;
      }
      *p = pack(f);
    }
  } else {
#pragma unroll
    for (int pc = 0; pc < PIECES / 2; ++pc) {
      uint4* p0 = piece_ptr(pc);
      uint4* p1 = piece_ptr(pc + PIECES / 2);
      float f0[EPP], f1[EPP];
      unpack(*p0, f0);
      unpack(*p1, f1);
      float cs[EPP], sn[EPP];  // pairs (i, i + D/2), i = pc*EPP .. +EPP: consecutive table entries
#pragma unroll
      for (int q = 0; q < EPP / 4; ++q) {
        const float4 c4 = __ldg(reinterpret_cast<const float4*>(ct + pc * EPP) + q);
        const float4 s4 = __ldg(reinterpret_cast<const float4*>(st + pc * EPP) + q);
        cs[4 * q] = c4.x; cs[4 * q + 1] = c4.y; cs[4 * q + 2] = c4.z; cs[4 * q + 3] = c4.w;
        sn[4 * q] = s4.x; sn[4 * q + 1] = s4.y; sn[4 * q + 2] = s4.z; sn[4 * q + 3] = s4.w;
      }
#pragma unroll
      for (int e = 0; e < EPP; ++e) {
        const float c = cs[e], s = sn[e];
        const float x0 = f0[e], x1 = f1[e];
        f0[e] = x0 * c - x1 * s;
        f1[e] = x1 * c + x0 * s;
      }
      *p0 = pack(f0);
      *p1 = pack(f1);
    }
  }
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(ATTN_THREADS, AttnCfg<D, kBf16>::MIN_CTAS)
flash_attn_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, const AttnArgs args) {
  using Cfg = AttnCfg<D, kBf16>;
  constexpr int ELT = Cfg::ELT;
  constexpr int NCH = Cfg::NCH;
  constexpr int CHE = 128 / ELT;            // elements per 128-B chunk
  constexpr int UMMA_K = 32 / ELT;
  constexpr uint32_t IDESC_S = make_idesc(kBf16, 128, ATTN_TILE, false, false);  // Q (K-major) x K (K-major)
  constexpr uint32_t IDESC_O = make_idesc(kBf16, 128, D, false, true);           // P (TMEM)    x V (MN-major)

  // causal launches start with the last query tiles: those walk the most key tiles, and the launch should end on short CTAs
  const int qtile = args.causal ? static_cast<int>(gridDim.x - 1 - blockIdx.x) : static_cast<int>(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z;
  int row0, L;
  if (args.cu_seqlens) {
    row0 = args.cu_seqlens[b];
    L = args.cu_seqlens[b + 1] - row0;
  } else {
    row0 = b * args.S;
    L = args.S;
  }
  const int q0 = qtile * ATTN_TILE;
  if (q0 >= L) return;  // uniform for the CTA; nothing allocated yet
  int n_kv = (L + ATTN_TILE - 1) / ATTN_TILE;
  if (args.causal) n_kv = min(n_kv, qtile + 1);
  const int q_rows = min(ATTN_TILE, L - q0);   // valid query rows of this tile

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::Q_BYTES;
  uint8_t* sV = sK + Cfg::Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + Cfg::Q_BYTES);
  uint64_t* bar_q = bars + 0;     // Q tile landed
  uint64_t* bar_k = bars + 1;     // K tile landed
  uint64_t* bar_v = bars + 2;     // V tile landed
  uint64_t* bar_s = bars + 3;     // S = Q K^T complete in TMEM
  uint64_t* bar_p = bars + 4;     // P written to TMEM (and O_j of the previous step fully read): one arrive per warp
  uint64_t* bar_o = bars + 5;     // O_j = P V complete in TMEM
  uint64_t* bar_rq = bars + 6;    // Q rotated (RoPE)
  uint64_t* bar_rk = bars + 7;    // K rotated (RoPE)
  uint64_t* bar_or = bars + 8;    // O_j read out of TMEM (only when it shares columns with the next S): one arrive per warp
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool rope = args.rope_style != ROPE_NONE;
  const bool rope_k = rope && !args.rope_k_done;   // K may have been rotated by a pre-pass (long sequences)

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1);
    mbar_init(bar_s, 1); mbar_init(bar_p, 4); mbar_init(bar_o, 1);
    mbar_init(bar_rq, 4); mbar_init(bar_rk, 4); mbar_init(bar_or, 4);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
  }
  if (warp == 4) {
    tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + Cfg::O_COL;

#define ATTN_FAIL()                                         \
  do {                                                      \
    if (!*abort_flag) atomicCAS(args.err, 0, ERR_WAIT_ATTN); \
    *abort_flag = 1;                                        \
  } while (0)

  if (warp == 4) {
    if (lane == 0) {
      // -------------------------------------------------------- TMA + MMA issuer
      const int colq = h * D;
      mbar_expect_tx(bar_q, Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < NCH; ++c) tma_load_2d(sQ + c * ATTN_CHUNK_BYTES, &tmap_q, bar_q, colq + c * CHE, row0 + q0);
      mbar_expect_tx(bar_k, Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < NCH; ++c) tma_load_2d(sK + c * ATTN_CHUNK_BYTES, &tmap_k, bar_k, colq + c * CHE, row0);
      mbar_expect_tx(bar_v, Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < NCH; ++c) tma_load_2d(sV + c * ATTN_CHUNK_BYTES, &tmap_v, bar_v, colq + c * CHE, row0);

      bool ok = mbar_wait(rope ? bar_rq : bar_q, 0, abort_flag);
      if (!ok) ATTN_FAIL();
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t ph = j & 1;
        const int kv_len = min(ATTN_TILE, L - j * ATTN_TILE);           // valid keys of this step
        const int n_s = (kv_len + 31) & ~31;                             // score columns computed (multiples of 32: N = 16 mod 32 is slow)
        const uint32_t idesc_s = (IDESC_S & ~(0x3Fu << 17)) | (static_cast<uint32_t>(n_s >> 3) << 17);
        if (!mbar_wait(rope_k ? bar_rk : bar_k, ph, abort_flag)) { ATTN_FAIL(); break; }
        if constexpr (Cfg::SHARE_O) {
          // the scores of this step overwrite the columns that hold O of the previous step: wait until it has been read
          if (j > 0 && !mbar_wait(bar_or, (j - 1) & 1, abort_flag)) { ATTN_FAIL(); break; }
        }
        tc_fence_after();
        // S = Q K_j^T : D/UMMA_K k-steps of 32 B, walking the 128-B chunks
#pragma unroll
        for (int ks = 0; ks < D / UMMA_K; ++ks) {
          const int chunk = (ks * 32) / 128, off = (ks * 32) % 128;
          const uint64_t adesc = make_smem_desc_sw128(smem_u32(sQ) + chunk * ATTN_CHUNK_BYTES + off, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(sK) + chunk * ATTN_CHUNK_BYTES + off, 16, 1024);
          umma_ss<kBf16>(tmem_s, adesc, bdesc, idesc_s, ks != 0 ? 1u : 0u);
        }
        umma_commit(bar_s);
        if (!mbar_wait(bar_s, ph, abort_flag)) { ATTN_FAIL(); break; }
        if (j + 1 < n_kv) {  // K buffer is free again: fetch the next key tile
          mbar_expect_tx(bar_k, Cfg::Q_BYTES);
#pragma unroll
          for (int c = 0; c < NCH; ++c)
            tma_load_2d(sK + c * ATTN_CHUNK_BYTES, &tmap_k, bar_k, colq + c * CHE, row0 + (j + 1) * ATTN_TILE);
        }
        if (!mbar_wait(bar_p, ph, abort_flag)) { ATTN_FAIL(); break; }
        if (!mbar_wait(bar_v, ph, abort_flag)) { ATTN_FAIL(); break; }
        tc_fence_after();
        // O_j = P V_j : P from TMEM (8 columns per k-step in either precision), V as loaded (MN-major);
        // only the k-steps that cover valid keys are issued (P is zero-filled up to a multiple of 32 keys)
        const int ksteps = (kv_len + UMMA_K - 1) / UMMA_K;
        for (int ks = 0; ks < ksteps; ++ks) {
          const uint64_t bdesc = make_smem_desc_mn<kBf16>(smem_u32(sV) + ks * (UMMA_K * 128), ATTN_CHUNK_BYTES);
          umma_ts<kBf16>(tmem_o, tmem_s + ks * 8, bdesc, IDESC_O, ks != 0 ? 1u : 0u);
        }
        umma_commit(bar_o);
        if (!mbar_wait(bar_o, ph, abort_flag)) { ATTN_FAIL(); break; }
        if (j + 1 < n_kv) {  // V buffer is free again
          mbar_expect_tx(bar_v, Cfg::Q_BYTES);
#pragma unroll
          for (int c = 0; c < NCH; ++c)
            tma_load_2d(sV + c * ATTN_CHUNK_BYTES, &tmap_v, bar_v, colq + c * CHE, row0 + (j + 1) * ATTN_TILE);
        }
      }
    }
  } else {
    // ---------------------------------------------------------- softmax / output threads
    const int t = threadIdx.x;            // query row inside the tile, also the TMEM lane
    const int qi = q0 + t;                // query position in its sequence
    const bool warp_active = warp * 32 < q_rows;   // warps whose 32 rows are all padding only keep the barriers moving
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const float kLog2e = 1.4426950408889634f;
    float o_acc[D];
#pragma unroll
    for (int d = 0; d < D; ++d) o_acc[d] = 0.f;
    float m_ref = -INFINITY, l_run = 0.f;   // reference point of the exponentials (log2 units, integer-valued) and row sum
    const float* kmask = args.key_mask ? args.key_mask + static_cast<long long>(b) * args.S : nullptr;
    bool ok = true;

    if (rope) {
      if (mbar_wait(bar_q, 0, abort_flag)) {
        rope_row_inplace<D, kBf16>(sQ, t, min(qi, args.S - 1), args);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rq);
      } else { ATTN_FAIL(); ok = false; }
    }

    for (int j = 0; j < n_kv && ok; ++j) {
      const uint32_t ph = j & 1;
      const int k0 = j * ATTN_TILE;
      const int kv_len = min(ATTN_TILE, L - k0);
      const int nchunks = (kv_len + 31) >> 5;      // 32-key chunks that hold at least one valid key
      if (rope_k) {
        if (!mbar_wait(bar_k, ph, abort_flag)) { ATTN_FAIL(); break; }
        rope_row_inplace<D, kBf16>(sK, t, min(k0 + t, args.S - 1), args);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rk);
      }
      if (!mbar_wait(bar_s, ph, abort_flag)) { ATTN_FAIL(); break; }
      tc_fence_after();

      float alpha = 1.f, l_tile = 0.f;
      if (warp_active) {
        // The exponentials of a row refer to a reference point m_ref kept in log2 units (scale folded in) and at an
        // INTEGER value: moving it multiplies everything accumulated so far by an exact power of two.
        // Only tiles that touch the end of the sequence, the causal diagonal or a key mask need per-element mask logic
        // (warp-uniform test) and take two sweeps over the scores (row maximum first). Interior tiles take ONE sweep:
        // a chunk's exponentials use the reference point as it stands, and only if a chunk's maximum has outgrown it by
        // more than 2^8 is it moved up, with the row's earlier P chunks, row sums and accumulator scaled down to match
        // (rare after the first key tiles; P stays at most 2^9, harmless in bf16 / tf32 and in the fp32 sums).
        const bool tile_mask = kmask != nullptr || k0 + ATTN_TILE > L || (args.causal && k0 + ATTN_TILE - 1 > q0) ||
                               !(args.scale > 0.f);
        const float sl2 = args.scale * kLog2e;
        // 2^k for an integer-valued k <= 0 (k = -inf or below the normal range gives 0)
        auto pow2_int = [](float k) { return k < -126.f ? 0.f : __int_as_float((static_cast<int>(k) + 127) << 23); };
        if (tile_mask) {
          // ---- sweep 1: row maximum
          float m_tile = -INFINITY;
          // bit i of validw: key kc + i exists; of the returned word: it also passes the key mask and the causal rule
          // (warp-wide call: the key mask word comes from one load per lane and a ballot)
          auto keep_word = [&](int kc, uint32_t validw) {
            uint32_t w = validw;
            if (args.causal) w &= prefix_bits(qi - kc + 1);
            if (kmask) w &= __ballot_sync(0xffffffffu, kc + lane < L && __ldg(kmask + kc + lane) >= 0.5f);
            return w;
          };
#pragma unroll 1
          for (int c = 0; c < nchunks; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_s + lane_addr + c * 32, r);
            tmem_ld_wait();
            // masked keys score -1e9 (what the reference adds), absent ones -inf
            const int kc = k0 + c * 32;
            const uint32_t validw = prefix_bits(L - kc);
            const uint32_t keepw = keep_word(kc, validw);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float sc = __uint_as_float(r[i]) * args.scale;
              r[i] = __float_as_uint(((keepw >> i) & 1u) ? sc : (((validw >> i) & 1u) ? -1e9f : -INFINITY));
            }
            m_tile = fmaxf(m_tile, row_max32(r));
          }
          const float m_tile_l2 = m_tile * kLog2e;
          const float new_ref = m_tile_l2 > m_ref ? ceilf(m_tile_l2) : m_ref;
          alpha = pow2_int(m_ref - new_ref);          // 0 on the first step (m_ref = -inf)
          m_ref = new_ref;
          const float m_l2 = m_ref;
          const float x_masked = -1e9f * kLog2e - m_l2;
          // ---- sweep 2: p = exp(s - m) in the MMA operand precision, row sum, P written over S in TMEM
#pragma unroll 1
          for (int c = 0; c < nchunks; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_s + lane_addr + c * 32, r);
            tmem_ld_wait();
            float p[32];
            const uint32_t validw = prefix_bits(L - (k0 + c * 32));
            const uint32_t keepw = keep_word(k0 + c * 32, validw);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float x = fmaf(__uint_as_float(r[i]), sl2, -m_l2);
              p[i] = fast_exp2(((keepw >> i) & 1u) ? x : (((validw >> i) & 1u) ? x_masked : -INFINITY));
            }
            if constexpr (kBf16) {
              // two bf16 per 32-bit column (even key in the low half): chunk c -> columns [16c, 16c+16).
              // In-place is safe in increasing c: those columns hold scores of chunk c/2, already consumed.
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(p[2 * i], p[2 * i + 1]);
              l_tile += row_sum32(p);   // the unrounded sum: bf16 rounding of P averages out over the row
              tmem_st_32x16(tmem_s + lane_addr + c * 16, pk);
            } else {
              uint32_t pk[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                p[i] = round_to_tf32(p[i]);
                pk[i] = __float_as_uint(p[i]);
              }
              l_tile += row_sum32(p);
              tmem_st_32x32(tmem_s + lane_addr + c * 32, pk);
            }
          }
        } else {
          // ---- one sweep (all 32-key chunks of an interior tile are full)
#pragma unroll 1
          for (int c = 0; c < nchunks; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_s + lane_addr + c * 32, r);
            tmem_ld_wait();
            const float cmax = row_max32(r) * sl2;              // scale > 0 here: the maximum commutes with it
            const bool move = cmax > m_ref + 8.0f || m_ref == -INFINITY;
            if (__any_sync(0xffffffffu, move)) {
              // this lane's factor (1 for the rows that stay): exact power of two
              float a = 1.f;
              if (move) {
                const float new_ref = ceilf(cmax);
                a = pow2_int(m_ref - new_ref);
                m_ref = new_ref;
              }
              tmem_st_wait();                                    // the P chunks written so far have landed
              for (int cc = 0; cc < c; ++cc) {
                if constexpr (kBf16) {
                  uint32_t q[16];
                  tmem_ld_32x16(tmem_s + lane_addr + cc * 16, q);
                  tmem_ld_wait();
#pragma unroll
                  for (int i = 0; i < 16; ++i)
                    q[i] = pack_bf16x2(__uint_as_float(q[i] << 16) * a, __uint_as_float(q[i] & 0xffff0000u) * a);
                  tmem_st_32x16(tmem_s + lane_addr + cc * 16, q);
                } else {
                  uint32_t q[32];
                  tmem_ld_32x32(tmem_s + lane_addr + cc * 32, q);
                  tmem_ld_wait();
#pragma unroll
                  for (int i = 0; i < 32; ++i) q[i] = __float_as_uint(__uint_as_float(q[i]) * a);
                  tmem_st_32x32(tmem_s + lane_addr + cc * 32, q);
                }
              }
              l_tile *= a;
              l_run *= a;
#pragma unroll
              for (int d = 0; d < D; d += 2) mul_f32x2(o_acc[d], o_acc[d + 1], o_acc[d], o_acc[d + 1], a, a);
            }
            float p[32];
            const float neg_m = -m_ref;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float x0, x1;
              fma_f32x2(x0, x1, __uint_as_float(r[i]), __uint_as_float(r[i + 1]), sl2, sl2, neg_m, neg_m);
              p[i] = fast_exp2(x0);
              p[i + 1] = fast_exp2(x1);
            }
            if constexpr (kBf16) {
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(p[2 * i], p[2 * i + 1]);
              l_tile += row_sum32(p);
              tmem_st_32x16(tmem_s + lane_addr + c * 16, pk);
            } else {
              uint32_t pk[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                p[i] = round_to_tf32(p[i]);
                pk[i] = __float_as_uint(p[i]);
              }
              l_tile += row_sum32(p);
              tmem_st_32x32(tmem_s + lane_addr + c * 32, pk);
            }
          }
          // alpha stays 1: the accumulated sums were scaled where the reference point moved
        }
        tmem_st_wait();
      }
      tc_fence_before();          // this thread's TMEM reads and writes are ordered before the MMA that follows the barrier
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);

      l_run = l_run * alpha + l_tile;
      // the running maximum of a row stops moving after the first key tiles: skip the rescale when no row of the warp needs it
      if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int d = 0; d < D; d += 2) mul_f32x2(o_acc[d], o_acc[d + 1], o_acc[d], o_acc[d + 1], alpha, alpha);
      }

      if (!mbar_wait(bar_o, ph, abort_flag)) { ATTN_FAIL(); break; }
      tc_fence_after();
      if (warp_active) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_o + lane_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            add_f32x2(o_acc[c * 32 + i], o_acc[c * 32 + i + 1], o_acc[c * 32 + i], o_acc[c * 32 + i + 1], __uint_as_float(r[i]),
                      __uint_as_float(r[i + 1]));
        }
      }
      tc_fence_before();
      if constexpr (Cfg::SHARE_O) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_or);
      }
    }

    if (ok && qi < L && !*abort_flag) {
      const float inv = 1.f / l_run;
      const long long orow = static_cast<long long>(row0 + qi) * args.ld_out + h * D;
      if (args.out_bf16) {
        __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(args.out) + orow;
        const bool v8 = (args.ld_out % 8 == 0) && ((reinterpret_cast<uintptr_t>(args.out) & 15) == 0) && (D % 8 == 0);
#pragma unroll
        for (int d = 0; d < D; d += 8) {
          uint4 q;   // eight bf16 per 16-byte store
          q.x = pack_bf16x2(o_acc[d] * inv, o_acc[d + 1] * inv);
          q.y = pack_bf16x2(o_acc[d + 2] * inv, o_acc[d + 3] * inv);
          q.z = pack_bf16x2(o_acc[d + 4] * inv, o_acc[d + 5] * inv);
          q.w = pack_bf16x2(o_acc[d + 6] * inv, o_acc[d + 7] * inv);
          if (v8) *reinterpret_cast<uint4*>(op + d) = q;
          else {
            uint32_t* o32 = reinterpret_cast<uint32_t*>(op + d);
            o32[0] = q.x; o32[1] = q.y; o32[2] = q.z; o32[3] = q.w;
          }
        }
      } else {
        float* op = reinterpret_cast<float*>(args.out) + orow;
        const bool v4 = (args.ld_out % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.out) & 15) == 0);
#pragma unroll
        for (int d = 0; d < D; d += 4) {
          float4 q = make_float4(o_acc[d] * inv, o_acc[d + 1] * inv, o_acc[d + 2] * inv, o_acc[d + 3] * inv);
          if (args.round_tf32) {
            q.x = round_to_tf32(q.x); q.y = round_to_tf32(q.y); q.z = round_to_tf32(q.z); q.w = round_to_tf32(q.w);
          }
          if (v4) *reinterpret_cast<float4*>(op + d) = q;
          else { op[d] = q.x; op[d + 1] = q.y; op[d + 2] = q.z; op[d + 3] = q.w; }
        }
      }
    }
  }
#undef ATTN_FAIL

  if (*abort_flag) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 4) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace gb
