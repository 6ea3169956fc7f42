// Persistent, warp-specialised TMA -> tcgen05 GEMM for sm_100a.
//
//   D[M,N] = epilogue( A[M,K] * B )      A is K-major (row-major [M][K]).
//   B is either K-major  ([N][K] row-major: the `linear` weight layout W(out,in)),
//   or          MN-major ([K][N] row-major: the `gemm_mnk` B operand).
//
// One CTA per SM walks output tiles of 128 x BN. Warp 0 feeds a ring of shared
// memory stages with TMA, warp 1 issues tcgen05.mma into one of two TMEM
// accumulators, warps 2..9 drain the other accumulator (tcgen05.ld), apply the
// fused epilogue and store. Element type is fp32 consumed as tf32
// (kind::tf32) or bf16 (kind::f16); accumulation is always fp32.
#pragma once
#include "ptx.cuh"
#include "args.h"
#include <cuda_bf16.h>

namespace gb {



__device__ __forceinline__ float round_to_tf32(float x) {
  uint32_t u = __float_as_uint(x);
  // round to nearest even on the 13 dropped mantissa bits; inf/nan pass through
  if ((u & 0x7F800000u) != 0x7F800000u) {
    u += 0x00000FFFu + ((u >> 13) & 1u);
    u &= 0xFFFFE000u;
  }
  return __uint_as_float(u);
}

__device__ __forceinline__ float act_gelu_tanh(float x) {
  // 0.5 x (1 + tanh(u)) == x * sigmoid(2u) == x / (1 + 2^(-2u log2 e)),  u = sqrt(2/pi) (x + 0.044715 x^3)
  const float k1 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
  const float k3 = k1 * 0.044715f;
  const float t = x * fmaf(k3, x * x, k1);
  return __fdividef(x, 1.0f + exp2f(t));  // t -> +inf gives x/inf = 0, t -> -inf gives x
}
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ float act_silu(float x) {
  float xc = fminf(fmaxf(x, -88.f), 88.f);
  return __fdividef(x, 1.f + __expf(-xc));
}
__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case ACT_GELU_TANH: return act_gelu_tanh(v);
    case ACT_SILU: return act_silu(v);
    case ACT_RELU: return fmaxf(v, 0.f);
    default: return v;
  }
}

template <int BN>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int A_BYTES = BM * 128;            // 128 rows x 128 B
  static constexpr int B_BYTES = BN * 128;            // BN rows x 128 B (either major)
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int MAX_SMEM = 227 * 1024;
  static constexpr int STAGES_RAW = (MAX_SMEM - 2048) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
  static_assert(2 * BN <= 512, "two accumulators must fit TMEM");
  static_assert(BN % 32 == 0, "epilogue drains 32 columns at a time");
};

constexpr int GEMM_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue

template <int BN, bool kBf16, bool kBMnMajor>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmArgs args) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ELT = kBf16 ? 2 : 4;
  constexpr int BK = 128 / ELT;                 // K elements per stage (128 B per row)
  constexpr int CH = 128 / ELT;                 // M/N elements per 128-B chunk (MN-major B)
  constexpr int UMMA_K = 32 / ELT;              // K elements per instruction (32 B)
  constexpr int KSTEPS = BK / UMMA_K;           // 4
  constexpr uint32_t IDESC = make_idesc(kBf16, 128, BN, false, kBMnMajor);

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
  const int num_tiles = args.num_m_tiles * args.num_n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m_blk = tile / args.num_n_tiles;
        const int n_blk = tile % args.num_n_tiles;
        for (int kb = 0; kb < args.num_k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            if (!*abort_flag) atomicCAS(args.err, 0, ERR_WAIT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m_blk * 128);
          if constexpr (kBMnMajor) {
#pragma unroll
            for (int c = 0; c < BN / CH; ++c)
              tma_load_2d(sb + c * (BK * 128), &tmap_b, &full_bar[stage], n_blk * BN + c * CH, kb * BK);
          } else {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * BK, n_blk * BN);
          }
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
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) {
          if (!*abort_flag) atomicCAS(args.err, 0, ERR_WAIT_TMEM_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < args.num_k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            if (!*abort_flag) atomicCAS(args.err, 0, ERR_WAIT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            const uint64_t adesc = make_smem_desc_sw128(sa + ks * 32, 16, 1024);
            uint64_t bdesc;
            if constexpr (kBMnMajor)
              bdesc = make_smem_desc_mn<kBf16>(sb + ks * (UMMA_K * 128), BK * 128);
            else
              bdesc = make_smem_desc_sw128(sb + ks * 32, 16, 1024);
            umma_ss<kBf16>(d_tmem, adesc, bdesc, IDESC, (kb | ks) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tmem_full[acc]);  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    // Two warps per TMEM lane quadrant; each takes every other 32-column chunk of the accumulator.
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;          // 0 or 1: which chunks of the tile this warp drains
    int it = 0;
    const bool out_al16 = (reinterpret_cast<uintptr_t>(args.out) & 15) == 0;
    const bool vec_ok = !args.out_bf16 && (args.ld_out % 4 == 0) && out_al16;
    const bool vec8_ok = args.out_bf16 && (args.ld_out % 8 == 0) && out_al16;
    const bool res_vec_ok = args.residual && (args.ld_res % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.residual) & 15) == 0);
    const bool bias_vec_ok = args.bias && ((reinterpret_cast<uintptr_t>(args.bias) & 15) == 0);
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int m_blk = tile / args.num_n_tiles;
      const int n_blk = tile % args.num_n_tiles;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag)) {
        if (!*abort_flag) atomicCAS(args.err, 0, ERR_WAIT_TMEM_FULL);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int row = m_blk * 128 + quad * 32 + lane;
      const bool row_ok = row < args.M;
      float mean = 0.f, rstd = 1.f;
      if (args.row_rstd && row_ok) {
        rstd = args.row_rstd[row];
        if (args.row_mean) mean = args.row_mean[row];
      }
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = half; c < BN / 32; c += 2) {
        uint32_t r[32];
        __syncwarp();  // tcgen05.ld is warp-collective: reconverge after the lane-dependent skip below
        tmem_ld_32x32(taddr_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c * 32;
        if (!row_ok || col0 >= args.N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (col0 + 32 <= args.N) {
          // ---------------- fast path: the whole 32-column chunk is inside the matrix
          if (args.row_rstd) {
            if (args.row_mean) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = rstd * (v[j] - mean * __ldg(args.col_sum + col0 + j));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] *= rstd;
            }
          }
          if (bias_vec_ok) {
            const float4* bp = reinterpret_cast<const float4*>(args.bias + col0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 q = __ldg(bp + j);
              v[4 * j] += q.x; v[4 * j + 1] += q.y; v[4 * j + 2] += q.z; v[4 * j + 3] += q.w;
            }
          } else if (args.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += __ldg(args.bias + col0 + j);
          }
          if (args.swiglu_pairs) {
            // (gate, up) pairs -> 16 output columns
            float o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              o[j] = v[2 * j] * act_silu(v[2 * j + 1]);
              if (args.round_tf32) o[j] = round_to_tf32(o[j]);
            }
            const long long idx = static_cast<long long>(row) * args.ld_out + (col0 >> 1);
            if (args.out_bf16) {
              __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(args.out) + idx;
              if (vec8_ok) {
#pragma unroll
                for (int j = 0; j < 16; j += 8) {
                  uint4 pk;
                  pk.x = pack_bf16x2(o[j], o[j + 1]); pk.y = pack_bf16x2(o[j + 2], o[j + 3]);
                  pk.z = pack_bf16x2(o[j + 4], o[j + 5]); pk.w = pack_bf16x2(o[j + 6], o[j + 7]);
                  *reinterpret_cast<uint4*>(op + j) = pk;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) op[j] = __float2bfloat16(o[j]);
              }
            } else {
              float* op = reinterpret_cast<float*>(args.out) + idx;
              if (vec_ok) {
#pragma unroll
                for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(op + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) op[j] = o[j];
              }
            }
            continue;
          }
          if (args.act == ACT_GELU_TANH) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = act_gelu_tanh(v[j]);
          } else if (args.act == ACT_SILU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = act_silu(v[j]);
          } else if (args.act == ACT_RELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
          }
          if (args.residual) {
            const float* rp = args.residual + static_cast<long long>(row) * args.ld_res + col0;
            if (res_vec_ok) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 q = __ldg(reinterpret_cast<const float4*>(rp) + j);
                v[4 * j] += q.x; v[4 * j + 1] += q.y; v[4 * j + 2] += q.z; v[4 * j + 3] += q.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += __ldg(rp + j);
            }
          }
          if (args.round_tf32) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = round_to_tf32(v[j]);
          }
          if (args.out_bf16) {
            __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(args.out) + static_cast<long long>(row) * args.ld_out + col0;
            if (vec8_ok) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 pk;
                pk.x = pack_bf16x2(v[j], v[j + 1]); pk.y = pack_bf16x2(v[j + 2], v[j + 3]);
                pk.z = pack_bf16x2(v[j + 4], v[j + 5]); pk.w = pack_bf16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(op + j) = pk;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) op[j] = __float2bfloat16(v[j]);
            }
          } else {
            float* op = reinterpret_cast<float*>(args.out) + static_cast<long long>(row) * args.ld_out + col0;
            if (vec_ok) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(op + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) op[j] = v[j];
            }
          }
          continue;
        }
        // ---------------- ragged right edge: per-column bounds checks, scalar accesses
        // (fully unrolled with predicates so that v[] stays in registers)
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = col0 + j;
          if (col < args.N) {
            float x = v[j];
            if (args.row_rstd) x = rstd * (x - (args.row_mean ? mean * args.col_sum[col] : 0.f));
            if (args.bias) x += __ldg(args.bias + col);
            v[j] = x;
          }
        }
        if (args.swiglu_pairs) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const int col = col0 + j;
            if (col + 1 < args.N) {
              float o = v[j] * act_silu(v[j + 1]);
              if (args.round_tf32) o = round_to_tf32(o);
              const long long idx = static_cast<long long>(row) * args.ld_out + (col >> 1);
              if (args.out_bf16) reinterpret_cast<__nv_bfloat16*>(args.out)[idx] = __float2bfloat16(o);
              else reinterpret_cast<float*>(args.out)[idx] = o;
            }
          }
          continue;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = col0 + j;
          if (col < args.N) {
            float x = apply_act(v[j], args.act);
            if (args.residual) x += __ldg(args.residual + static_cast<long long>(row) * args.ld_res + col);
            if (args.round_tf32) x = round_to_tf32(x);
            const long long idx = static_cast<long long>(row) * args.ld_out + col;
            if (args.out_bf16) reinterpret_cast<__nv_bfloat16*>(args.out)[idx] = __float2bfloat16(x);
            else reinterpret_cast<float*>(args.out)[idx] = x;
          }
        }
      }
      // this warp has finished reading the accumulator
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    // give copies and MMAs still in flight time to land before the CTA's
    // shared memory and TMEM go away (bounded: about 1 ms)
    for (int i = 0; i < 100; ++i) __nanosleep(10000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace gb
