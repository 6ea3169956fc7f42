// Persistent, warp-specialised TMA -> tcgen05 GEMM for sm_100a.
//
//   D[M,N] = epilogue( A[M,K] * B )      A is K-major (row-major [M][K]).
//   (`linear` normally runs swapped: the weight matrix is the 128-row operand and 256 tokens are the N dimension of
//   the MMA, because one tcgen05.mma takes the same time for N = 64 as for N = 256.)
//   B is either K-major  ([N][K] row-major: the `linear` weight layout W(out,in)),
//   or          MN-major ([K][N] row-major: the `gemm_mnk` B operand).
//
// One CTA per SM walks output tiles of 128 x BN. Warp 0 feeds a ring of shared
// memory stages with TMA, warp 1 issues tcgen05.mma into one of two TMEM
// accumulators, warps 2..17 drain the other accumulator (tcgen05.ld), apply the
// fused epilogue and store. Element type is fp32 consumed as tf32
// (kind::tf32) or bf16 (kind::f16); accumulation is always fp32.
#pragma once
#include "ptx.cuh"
#include "args.h"
#include <cuda_bf16.h>

namespace gb {



__device__ __forceinline__ float round_to_tf32(float x) {
  // nearest tf32 value (10-bit mantissa, ties away from zero, what cvt.rna.tf32.f32 gives), as an fp32 bit pattern
  // with the low 13 bits clear; two integer instructions instead of a conversion-pipe instruction
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}

__device__ __forceinline__ float act_gelu_tanh(float x) {
  // 0.5 x (1 + tanh(u)), u = sqrt(2/pi) (x + 0.044715 x^3); tanh.approx is ONE special-function instruction
  // (absolute error about 5e-4 in tanh, so at most 2.5e-4 |x| in the result)
  const float k1 = 0.7978845608028654f;
  const float k3 = k1 * 0.044715f;
  const float u = x * fmaf(k3, x * x, k1);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  const float h = 0.5f * x;
  return fmaf(h, t, h);
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

// Further destinations of a gemm_mnk result (fp32, same pitch as the first output), e.g. the C matrices of the other
// GPUs of a column-split product. They travel in constant memory, not in GemmArgs: the `linear` kernels are compiled
// at their register limit and a larger argument struct alone made them spill. Set by the launcher in the stream
// before the launch. Only a launch whose GemmArgs::multi_out is non-zero reads the list, so plain GEMMs that run on
// the same GPU at the same time (other streams, other contexts) are not affected by it.
struct GemmExtraOut {
  int n;
  void* p[7];
};
static __constant__ GemmExtraOut g_gemm_extra_out;

// gate * act(up) of the pair epilogue: SiLU (SwiGLU) unless the launch asks for GELU (GeGLU)
__device__ __forceinline__ float glu_pair(float gate, float up, int act) {
  return gate * (act == ACT_GELU_TANH ? act_gelu_tanh(up) : act_silu(up));
}

struct EpiFlags {
  bool vec_ok, vec8_ok, res_vec_ok, bias_vec_ok;
};

// gemm_mnk with several destinations (args.multi_out > 0): the plain fp32 product goes to args.out and to every
// further destination. A warp holds a 32 x 32 block with one row per lane; it is transposed inside the warp (five
// exchange stages) so that every store instruction writes 32 consecutive columns of ONE row, a full 128-byte
// line: stores to a peer GPU then leave as whole lines instead of 16-byte pieces of 32 different rows.
// Called by all 32 lanes of the warp, whatever their row; row0 is the first row of the warp's block.
__device__ __forceinline__ void epilogue_chunk_multi(const GemmArgs& args, const uint32_t (&r)[32], int row0, int col0, int lane) {
  uint32_t v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = r[j];
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) {
    const bool upper = (lane & s) != 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if ((j & s) == 0) {
        const uint32_t send = upper ? v[j] : v[j + s];
        const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, s);
        if (upper) v[j] = recv; else v[j + s] = recv;
      }
    }
  }
  // now v[i] of lane l is element (row0 + i, col0 + l)
  for (int d = 0; d <= args.multi_out; ++d) {
    float* base = reinterpret_cast<float*>(d == 0 ? args.out : g_gemm_extra_out.p[d - 1]) + col0 + lane;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (row0 + i < args.M) base[static_cast<long long>(row0 + i) * args.ld_out] = __uint_as_float(v[i]);
  }
}

// Applies the fused epilogue to 32 consecutive accumulator columns of one row and stores them.
__device__ __forceinline__ void epilogue_chunk(const GemmArgs& args, const EpiFlags& f, const uint32_t (&r)[32], int row,
                                               int col0, float mean, float rstd) {
  const bool vec_ok = f.vec_ok, vec8_ok = f.vec8_ok, res_vec_ok = f.res_vec_ok, bias_vec_ok = f.bias_vec_ok;
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
        o[j] = glu_pair(v[2 * j], v[2 * j + 1], args.act);
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
      return;
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
    if (args.residual && args.residual_bf16) {
      const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(args.residual) + static_cast<long long>(row) * args.ld_res + col0;
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += __bfloat162float(rb[j]);
    } else if (args.residual) {
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
    return;
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
        float o = glu_pair(v[j], v[j + 1], args.act);
        if (args.round_tf32) o = round_to_tf32(o);
        const long long idx = static_cast<long long>(row) * args.ld_out + (col >> 1);
        if (args.out_bf16) reinterpret_cast<__nv_bfloat16*>(args.out)[idx] = __float2bfloat16(o);
        else reinterpret_cast<float*>(args.out)[idx] = o;
      }
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const int col = col0 + j;
    if (col < args.N) {
      float x = apply_act(v[j], args.act);
      if (args.residual) x += args.residual_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(args.residual)[static_cast<long long>(row) * args.ld_res + col]) : __ldg(args.residual + static_cast<long long>(row) * args.ld_res + col);
      if (args.round_tf32) x = round_to_tf32(x);
      const long long idx = static_cast<long long>(row) * args.ld_out + col;
      if (args.out_bf16) reinterpret_cast<__nv_bfloat16*>(args.out)[idx] = __float2bfloat16(x);
      else reinterpret_cast<float*>(args.out)[idx] = x;
    }
  }
}

// Fast path of the swapped epilogue (all 32 tokens in range, fp32 output, fp32 or no residual). Element by element:
// bias, activation, residual, tf32 rounding, then the store straight away, so that the load/store unit drains
// stores while the arithmetic of the following elements issues. With all arithmetic first and all stores last,
// the epilogue warps of an SM compute together and then queue on the store unit together, and the two phases add up.
__device__ __forceinline__ void st_global_f32(float* p, float v) {
  asm volatile("st.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
template <int ACT, bool RES>
__device__ __forceinline__ void epilogue_swapped_fast(const GemmArgs& args, const uint32_t (&r)[32], int f, int t0, float b) {
  float* op = reinterpret_cast<float*>(args.out) + static_cast<long long>(t0) * args.ld_out + f;
  const float* rp = RES ? args.residual + static_cast<long long>(t0) * args.ld_res + f : nullptr;
  const bool rnd = args.round_tf32 != 0;
#pragma unroll
  for (int g = 0; g < 32; g += 8) {
    float res[8];
    if constexpr (RES) {
#pragma unroll
      for (int u = 0; u < 8; ++u) res[u] = __ldg(rp + static_cast<long long>(g + u) * args.ld_res);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      float v = __uint_as_float(r[g + u]) + b;
      if constexpr (ACT == ACT_GELU_TANH) v = act_gelu_tanh(v);
      else if constexpr (ACT == ACT_SILU) v = act_silu(v);
      else if constexpr (ACT == ACT_RELU) v = fmaxf(v, 0.f);
      if constexpr (RES) v += res[u];
      if (rnd) v = round_to_tf32(v);
      st_global_f32(op + static_cast<long long>(g + u) * args.ld_out, v);
    }
  }
}
// bf16 output without a residual: neighbouring lanes hold neighbouring features; they swap one value per pair of tokens,
// so that the even lane has both features of token j and the odd lane both of token j + 1, and every lane stores 4 bytes
// (a bf16 pair) instead of 2. `live` = the lanes of the warp that are here (whole feature pairs: N is even).
template <int ACT>
__device__ __forceinline__ void epilogue_swapped_fast_bf16(const GemmArgs& args, const uint32_t (&r)[32], int f, int t0, float b,
                                                           unsigned live) {
  const int odd = f & 1;
  uint32_t* op = reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(args.out) + static_cast<long long>(t0 + odd) * args.ld_out + (f & ~1));
  const long long pitch = args.ld_out >> 1;
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    float v0 = __uint_as_float(r[j]) + b, v1 = __uint_as_float(r[j + 1]) + b;
    if constexpr (ACT == ACT_GELU_TANH) { v0 = act_gelu_tanh(v0); v1 = act_gelu_tanh(v1); }
    else if constexpr (ACT == ACT_SILU) { v0 = act_silu(v0); v1 = act_silu(v1); }
    else if constexpr (ACT == ACT_RELU) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); }
    const float got = __shfl_xor_sync(live, odd ? v0 : v1, 1);
    op[static_cast<long long>(j) * pitch] = odd ? pack_bf16x2(got, v1) : pack_bf16x2(v0, got);
  }
}

// Swapped orientation (the 128-row operand is the weight matrix, so TMEM lanes are output features and the
// accumulator columns are tokens): r[] holds 32 consecutive tokens t0.. for feature f. For a fixed register the
// 32 lanes of a warp touch 32 consecutive features of one token, i.e. one 128-byte line of the row-major output.
__device__ __forceinline__ void epilogue_chunk_swapped(const GemmArgs& args, const uint32_t (&r)[32], int f, int t0) {
  const bool f_ok = f < args.N;
  const bool full = t0 + 32 <= args.M;
  // taken here, where the whole warp is still together (lanes beyond N leave below, lanes on the fast path right away):
  // the lanes that reach the bf16 pair exchange at the end (whole feature pairs when N is even)
  const unsigned live = __ballot_sync(0xffffffffu, f_ok);
  const bool pairs_ok = !(args.N & 1) && !(args.ld_out & 1) && !(reinterpret_cast<uintptr_t>(args.out) & 3);   // warp-uniform
  if (full && f_ok && args.out_bf16 && pairs_ok && !args.residual && !args.row_rstd && !args.swiglu_pairs) {
    const float b = args.bias ? __ldg(args.bias + f) : 0.f;
    switch (args.act) {
      case ACT_GELU_TANH: return epilogue_swapped_fast_bf16<ACT_GELU_TANH>(args, r, f, t0, b, live);
      case ACT_SILU: return epilogue_swapped_fast_bf16<ACT_SILU>(args, r, f, t0, b, live);
      case ACT_RELU: return epilogue_swapped_fast_bf16<ACT_RELU>(args, r, f, t0, b, live);
      default: return epilogue_swapped_fast_bf16<ACT_NONE>(args, r, f, t0, b, live);
    }
  }
  if (full && f_ok && !args.out_bf16 && !args.row_rstd && !args.swiglu_pairs && !(args.residual && args.residual_bf16)) {
    const float b = args.bias ? __ldg(args.bias + f) : 0.f;
    if (args.residual) {
      switch (args.act) {
        case ACT_GELU_TANH: return epilogue_swapped_fast<ACT_GELU_TANH, true>(args, r, f, t0, b);
        case ACT_SILU: return epilogue_swapped_fast<ACT_SILU, true>(args, r, f, t0, b);
        case ACT_RELU: return epilogue_swapped_fast<ACT_RELU, true>(args, r, f, t0, b);
        default: return epilogue_swapped_fast<ACT_NONE, true>(args, r, f, t0, b);
      }
    }
    switch (args.act) {
      case ACT_GELU_TANH: return epilogue_swapped_fast<ACT_GELU_TANH, false>(args, r, f, t0, b);
      case ACT_SILU: return epilogue_swapped_fast<ACT_SILU, false>(args, r, f, t0, b);
      case ACT_RELU: return epilogue_swapped_fast<ACT_RELU, false>(args, r, f, t0, b);
      default: return epilogue_swapped_fast<ACT_NONE, false>(args, r, f, t0, b);
    }
  }
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  if (args.row_rstd) {
    const float cs = (args.row_mean && f_ok) ? __ldg(args.col_sum + f) : 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (full || t0 + j < args.M) {
        const float rs = __ldg(args.row_rstd + t0 + j);
        const float mu = args.row_mean ? __ldg(args.row_mean + t0 + j) : 0.f;
        v[j] = rs * (v[j] - mu * cs);
      }
    }
  }
  if (args.bias) {
    const float b = f_ok ? __ldg(args.bias + f) : 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] += b;
  }
  if (args.swiglu_pairs) {
    // features come as (gate, up) pairs in neighbouring lanes: even lanes produce out[:, f/2]
    const bool writer = f_ok && (f + 1 < args.N) && !(f & 1);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float up = __shfl_xor_sync(0xffffffffu, v[j], 1);
      if (writer && (full || t0 + j < args.M)) {
        float o = glu_pair(v[j], up, args.act);
        if (args.round_tf32) o = round_to_tf32(o);
        const long long idx = static_cast<long long>(t0 + j) * args.ld_out + (f >> 1);
        if (args.out_bf16) reinterpret_cast<__nv_bfloat16*>(args.out)[idx] = __float2bfloat16(o);
        else reinterpret_cast<float*>(args.out)[idx] = o;
      }
    }
    return;
  }
  if (!f_ok) return;
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
  if (args.residual && args.residual_bf16) {
    const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(args.residual) + static_cast<long long>(t0) * args.ld_res + f;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (full || t0 + j < args.M) v[j] += __bfloat162float(rp[static_cast<long long>(j) * args.ld_res]);
  } else if (args.residual) {
    const float* rp = args.residual + static_cast<long long>(t0) * args.ld_res + f;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] += __ldg(rp + static_cast<long long>(j) * args.ld_res);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (t0 + j < args.M) v[j] += __ldg(rp + static_cast<long long>(j) * args.ld_res);
    }
  }
  if (args.round_tf32) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = round_to_tf32(v[j]);
  }
  if (args.out_bf16) {
    // Neighbouring lanes hold neighbouring features. They swap one value per pair of tokens, so that the even lane
    // has both features of token j and the odd lane both of token j + 1, and every lane stores 4 bytes (a bf16 pair)
    // instead of 2: half the store instructions for the same lines.
    if (pairs_ok) {
      const int odd = f & 1;
      uint32_t* op = reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(args.out) + static_cast<long long>(t0 + odd) * args.ld_out + (f & ~1));
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float got = __shfl_xor_sync(live, odd ? v[j] : v[j + 1], 1);
        const uint32_t pk = odd ? pack_bf16x2(got, v[j + 1]) : pack_bf16x2(v[j], got);
        if (full || t0 + j + odd < args.M) op[static_cast<long long>(j) * (args.ld_out >> 1)] = pk;
      }
    } else {
      __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(args.out) + static_cast<long long>(t0) * args.ld_out + f;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (full || t0 + j < args.M) op[static_cast<long long>(j) * args.ld_out] = __float2bfloat16(v[j]);
    }
  } else {
    float* op = reinterpret_cast<float*>(args.out) + static_cast<long long>(t0) * args.ld_out + f;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; ++j) op[static_cast<long long>(j) * args.ld_out] = v[j];
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (t0 + j < args.M) op[static_cast<long long>(j) * args.ld_out] = v[j];
    }
  }
}

// Tile order of the persistent loops. Tiles that run at the same time should share operand rows, and the set of
// co-running tiles (one per SM) should be roughly square in loaded rows, or a large problem re-reads one operand
// from DRAM once per row of tiles. `fast` blocks are walked in groups of `group`: inside a group the fast index
// varies first, then the slow one; with group >= num_fast this is plain fast-major order.
// Out of line on purpose: inlined, the compiler hoists the division set-up out of the persistent loops and keeps it
// in registers next to the 64 accumulator registers of the epilogue, which then spills.
static __device__ __noinline__ uint32_t tile_coords_packed(int tile, int num_fast, int num_slow, int group) {
  const int per_group = group * num_slow;
  const int g = tile / per_group;
  const int first = g * group;
  const int gsz = min(num_fast - first, group);
  const int r = tile - g * per_group;
  const int slow = r / gsz;
  const int fast = first + (r - slow * gsz);
  return static_cast<uint32_t>(fast) | (static_cast<uint32_t>(slow) << 16);
}
__device__ __forceinline__ void tile_coords(int tile, int num_fast, int num_slow, int group, int& fast, int& slow) {
  if (group >= num_fast) {   // one group: plain fast-major order (every launch of the encoder)
    slow = tile / num_fast;
    fast = tile - slow * num_fast;
    return;
  }
  const uint32_t p = tile_coords_packed(tile, num_fast, num_slow, group);   // both counts are below 65536
  fast = static_cast<int>(p & 0xffffu);
  slow = static_cast<int>(p >> 16);
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

#ifndef GEMM_EPI_WARPS
#define GEMM_EPI_WARPS 16
#endif
static_assert(GEMM_EPI_WARPS % 4 == 0 && GEMM_EPI_WARPS >= 4 && GEMM_EPI_WARPS <= 16, "epilogue warps come in groups of 4");
constexpr int GEMM_THREADS = 64 + 32 * GEMM_EPI_WARPS;  // warp 0 TMA, warp 1 MMA, the rest epilogue

template <int BN, bool kBf16, bool kBMnMajor, bool kSwap>
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
      mbar_init(&tmem_empty[a], GEMM_EPI_WARPS);
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
        // un-swapped: column blocks fastest (neighbouring CTAs share the A rows); swapped: the weight blocks
        // (128-row operand) fastest, so neighbouring CTAs share one block of tokens
        int m_blk, n_blk;
        if constexpr (kSwap) tile_coords(tile, args.num_m_tiles, args.num_n_tiles, args.tile_group, m_blk, n_blk);
        else tile_coords(tile, args.num_n_tiles, args.num_m_tiles, args.tile_group, n_blk, m_blk);
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
      constexpr uint32_t B_KSTEP_BYTES = kBMnMajor ? UMMA_K * 128 : 32;  // advance of B per 32-byte k-step
      const uint32_t smem_base = smem_u32(smem);
      const uint64_t a_desc0 = make_smem_desc_sw128(smem_base, 16, 1024);
      const uint64_t b_desc0 = kBMnMajor ? make_smem_desc_mn<kBf16>(smem_base + Cfg::A_BYTES, BK * 128)
                                         : make_smem_desc_sw128(smem_base + Cfg::A_BYTES, 16, 1024);
      const uint32_t a_desc_lo = static_cast<uint32_t>(a_desc0), a_desc_hi = static_cast<uint32_t>(a_desc0 >> 32);
      const uint32_t b_desc_lo = static_cast<uint32_t>(b_desc0), b_desc_hi = static_cast<uint32_t>(b_desc0 >> 32);
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
          // descriptors differ from the stage-0 / k-step-0 ones only in the 14-bit start-address field
          // (units of 16 bytes), so a 32-bit add on the low word replaces rebuilding them for every MMA
          const uint32_t a_lo = a_desc_lo + stage * (Cfg::STAGE_BYTES >> 4);
          const uint32_t b_lo = b_desc_lo + stage * (Cfg::STAGE_BYTES >> 4);
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            const uint64_t adesc = (static_cast<uint64_t>(a_desc_hi) << 32) | (a_lo + ks * 2);
            const uint64_t bdesc = (static_cast<uint64_t>(b_desc_hi) << 32) | (b_lo + ks * (B_KSTEP_BYTES >> 4));
            umma_ss<kBf16>(d_tmem, adesc, bdesc, IDESC, (kb | ks) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tmem_full[acc]);  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2 .. 2+GEMM_EPI_WARPS-1)
    // GEMM_EPI_WARPS/4 warps per TMEM lane quadrant share the 32-column chunks of the accumulator round-robin.
    // The TMEM load of a warp's next chunk is in flight while it works on the current one.
    constexpr int NCHUNK = BN / 32;
    constexpr int G = GEMM_EPI_WARPS / 4;
    constexpr int MAXIT = (NCHUNK + G - 1) / G;
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    const int group = (warp - 2) >> 2;         // which chunks of the tile this warp drains: group, group+G, ...
    int it = 0;
    EpiFlags f;
    const bool out_al16 = (reinterpret_cast<uintptr_t>(args.out) & 15) == 0;
    f.vec_ok = !args.out_bf16 && (args.ld_out % 4 == 0) && out_al16;
    f.vec8_ok = args.out_bf16 && (args.ld_out % 8 == 0) && out_al16;
    f.res_vec_ok = args.residual && (args.ld_res % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.residual) & 15) == 0);
    f.bias_vec_ok = args.bias && ((reinterpret_cast<uintptr_t>(args.bias) & 15) == 0);
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      int m_blk, n_blk;
      if constexpr (kSwap) tile_coords(tile, args.num_m_tiles, args.num_n_tiles, args.tile_group, m_blk, n_blk);
      else tile_coords(tile, args.num_n_tiles, args.num_m_tiles, args.tile_group, n_blk, m_blk);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag)) {
        if (!*abort_flag) atomicCAS(args.err, 0, ERR_WAIT_TMEM_FULL);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int row = m_blk * 128 + quad * 32 + lane;   // un-swapped: output row; swapped: output feature
      const bool row_ok = kSwap ? true : row < args.M;
      float mean = 0.f, rstd = 1.f;
      if (!kSwap && args.row_rstd && row_ok) {
        rstd = args.row_rstd[row];
        if (args.row_mean) mean = args.row_mean[row];
      }
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      uint32_t ra[32], rb[32];
      __syncwarp();
      if (group < NCHUNK) tmem_ld_32x32(taddr_row + group * 32, ra);
#pragma unroll
      for (int i = 0; i < MAXIT; ++i) {
        const int c = group + i * G;           // warp-uniform
        uint32_t (&cur)[32] = (i & 1) ? rb : ra;
        uint32_t (&nxt)[32] = (i & 1) ? ra : rb;
        __syncwarp();                          // tcgen05.ld / wait are warp-collective: reconverge first
        if (c < NCHUNK) tmem_ld_wait();
        if (c + G < NCHUNK) tmem_ld_32x32(taddr_row + (c + G) * 32, nxt);
        const int col0 = n_blk * BN + c * 32;
        if constexpr (kSwap) {
          if (c < NCHUNK && col0 < args.M) epilogue_chunk_swapped(args, cur, row, col0);
        } else {
          if (args.multi_out > 0) {   // launcher guarantees fp32 output and N a multiple of 32
            if (c < NCHUNK && col0 < args.N) epilogue_chunk_multi(args, cur, row - lane, col0, lane);
          } else if (c < NCHUNK && row_ok && col0 < args.N) {
            epilogue_chunk(args, f, cur, row, col0, mean, rstd);
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
