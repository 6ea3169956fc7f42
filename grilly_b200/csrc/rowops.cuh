// HBM-bound row kernels: LayerNorm / RMSNorm (optionally with a residual add on
// the way in), row statistics, row softmax, element-wise activations, the fused
// embedding gather + position/type add + LayerNorm, masked mean-pool + L2
// normalise, tf32 rounding and fp32<->bf16 casts. One warp owns one row and
// keeps it in registers when it fits, so each tensor is read once and written once.
#pragma once
#include "gemm.cuh"
#include <cuda_bf16.h>

namespace gb {


__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}


// VPL = float4 vectors per lane; the row (F = 128 * VPL floats max) lives in registers.
template <int VPL>
__global__ void __launch_bounds__(256) norm_rows_kernel(const NormArgs a) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = a.F >> 2;
  for (long long it = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); it < a.rows;
       it += static_cast<long long>(gridDim.x) * warps_per_block) {
    const long long row = a.reverse ? a.rows - 1 - it : it;
    const float4* xp = reinterpret_cast<const float4*>(a.x + row * a.F);
    const float4* rp = a.residual ? reinterpret_cast<const float4*>(a.residual + row * a.F) : nullptr;
    float4 v[VPL];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
        v[i] = __ldg(xp + idx);
        if (rp) { float4 r = __ldg(rp + idx); v[i].x += r.x; v[i].y += r.y; v[i].z += r.z; v[i].w += r.w; }
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      } else {
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    float mean = 0.f;
    if (a.mode == NORM_LAYER) mean = warp_sum(s) / static_cast<float>(a.F);
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
        const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
        sq += (dx * dx + dy * dy) + (dz * dz + dw * dw);
      }
    }
    const float var = warp_sum(sq) / static_cast<float>(a.F);
    const float rstd = rsqrtf(var + a.eps);
    // rsqrtf is within 2 ulp; one Newton step brings it to the rounding of 1/sqrt
    const float rstd_n = rstd * (1.5f - 0.5f * (var + a.eps) * rstd * rstd);
    if (lane == 0) {
      if (a.mean_out) a.mean_out[row] = mean;
      if (a.rstd_out) a.rstd_out[row] = rstd_n;
      if (a.ratio_max) atomicMax(a.ratio_max, __float_as_uint(fabsf(mean) * rstd_n));   // non-negative floats order like their bits
    }
    if (!a.y) continue;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
        float4 g = a.gamma ? __ldg(reinterpret_cast<const float4*>(a.gamma) + idx) : make_float4(1.f, 1.f, 1.f, 1.f);
        float4 bt = (a.beta && a.mode == NORM_LAYER) ? __ldg(reinterpret_cast<const float4*>(a.beta) + idx)
                                                     : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 o;
        o.x = (v[i].x - mean) * rstd_n * g.x + bt.x;
        o.y = (v[i].y - mean) * rstd_n * g.y + bt.y;
        o.z = (v[i].z - mean) * rstd_n * g.z + bt.z;
        o.w = (v[i].w - mean) * rstd_n * g.w + bt.w;
        if (a.round_tf32) { o.x = round_to_tf32(o.x); o.y = round_to_tf32(o.y); o.z = round_to_tf32(o.z); o.w = round_to_tf32(o.w); }
        if (a.out_bf16) {
          __nv_bfloat162 p0 = __floats2bfloat162_rn(o.x, o.y), p1 = __floats2bfloat162_rn(o.z, o.w);
          uint2 pk;
          pk.x = *reinterpret_cast<uint32_t*>(&p0);
          pk.y = *reinterpret_cast<uint32_t*>(&p1);
          reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.y) + row * a.F)[idx] = pk;
        } else {
          reinterpret_cast<float4*>(reinterpret_cast<float*>(a.y) + row * a.F)[idx] = o;
        }
      }
    }
  }
}

// Any F (no alignment demands): the row is re-read from memory/L1 for each pass.
__global__ void __launch_bounds__(256) norm_rows_generic_kernel(const NormArgs a) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); row < a.rows;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const float* xp = a.x + row * a.F;
    const float* rp = a.residual ? a.residual + row * a.F : nullptr;
    const __nv_bfloat16* xh = reinterpret_cast<const __nv_bfloat16*>(a.x) + row * a.F;
    const __nv_bfloat16* rh = a.residual ? reinterpret_cast<const __nv_bfloat16*>(a.residual) + row * a.F : nullptr;
    auto in = [&](int i) {
      if (a.x_bf16) return __bfloat162float(xh[i]) + (a.residual ? __bfloat162float(rh[i]) : 0.f);
      return xp[i] + (rp ? rp[i] : 0.f);
    };
    float s = 0.f;
    for (int i = lane; i < a.F; i += 32) s += in(i);
    float mean = 0.f;
    if (a.mode == NORM_LAYER) mean = warp_sum(s) / static_cast<float>(a.F);
    float sq = 0.f;
    for (int i = lane; i < a.F; i += 32) {
      const float d = in(i) - mean;
      sq += d * d;
    }
    const float var = warp_sum(sq) / static_cast<float>(a.F);
    float rstd = rsqrtf(var + a.eps);
    rstd = rstd * (1.5f - 0.5f * (var + a.eps) * rstd * rstd);
    if (lane == 0) {
      if (a.mean_out) a.mean_out[row] = mean;
      if (a.rstd_out) a.rstd_out[row] = rstd;
      if (a.ratio_max) atomicMax(a.ratio_max, __float_as_uint(fabsf(mean) * rstd));
    }
    if (!a.y) continue;
    for (int i = lane; i < a.F; i += 32) {
      float o = (in(i) - mean) * rstd * (a.gamma ? a.gamma[i] : 1.f) +
                ((a.beta && a.mode == NORM_LAYER) ? a.beta[i] : 0.f);
      if (a.round_tf32) o = round_to_tf32(o);
      if (a.out_bf16) reinterpret_cast<__nv_bfloat16*>(a.y)[row * a.F + i] = __float2bfloat16(o);
      else reinterpret_cast<float*>(a.y)[row * a.F + i] = o;
    }
  }
}

// Row softmax over the last dimension: max, exp, sum, divide. One warp per row.
__global__ void __launch_bounds__(256) softmax_rows_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                           long long rows, int cols) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const float* xp = x + row * cols;
    float* yp = y + row * cols;
    float m = -INFINITY;
    for (int i = lane; i < cols; i += 32) m = fmaxf(m, xp[i]);
    m = warp_max(m);
    float s = 0.f;
    for (int i = lane; i < cols; i += 32) s += __expf(xp[i] - m);
    s = warp_sum(s);
    const float inv = 1.f / s;
    for (int i = lane; i < cols; i += 32) yp[i] = __expf(xp[i] - m) * inv;
  }
}

// Element-wise: y = act(a), y = a + b, or SwiGLU on halves of the last dim
// (y[r, c] = a[r, c] * silu(a[r, c + half]), the reference's activation form).
__global__ void __launch_bounds__(256) eltwise_kernel(int op, const float* __restrict__ a, const float* __restrict__ b,
                                                      float* __restrict__ y, long long n, int half) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v;
    switch (op) {
      case ELT_GELU: {
        // exact tanh here: the stand-alone activation is HBM-bound, accuracy is free
        const float x = a[i];
        v = 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
        break;
      }
      case ELT_SILU: { const float x = a[i]; v = x / (1.f + expf(-x)); break; }
      case ELT_RELU: v = fmaxf(a[i], 0.f); break;
      case ELT_ADD: v = a[i] + b[i]; break;
      case ELT_SWIGLU: {
        const long long r = i / half, c = i % half;
        const float x1 = a[r * 2 * half + c], x2 = a[r * 2 * half + half + c];
        v = x1 * (x2 / (1.f + expf(-x2)));
        break;
      }
      default: v = a[i];
    }
    y[i] = v;
  }
}

// Activations with parameters: GCU x cos(x) (backend/fnn.py:385-440, activation-gcu.glsl) and RoSwish
// (x + alpha) sigmoid(beta x) - alpha / 2 (backend/fnn.py:442-497, activation-roswish.glsl).
__global__ void __launch_bounds__(256) act_params_kernel(int op, const float* __restrict__ a, float* __restrict__ y, long long n,
                                                         float p0, float p1) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float x = a[i];
    y[i] = op == ELT_GCU ? x * cosf(x) : (x + p0) / (1.f + expf(-p1 * x)) - 0.5f * p0;
  }
}

__global__ void __launch_bounds__(256) round_tf32_kernel(const float* __restrict__ x, float* __restrict__ y, long long n) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = round_to_tf32(x[i]);
}
__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = __float2bfloat16(x[i]);
}
__global__ void __launch_bounds__(256) bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ y, long long n) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = __bfloat162float(x[i]);
}

// Plain gather (embedding_lookup): out[t] = table[ids[t]], zero row for ids outside [0, vocab).
__global__ void __launch_bounds__(256) gather_rows_kernel(const int* __restrict__ ids, const float* __restrict__ table,
                                                          float* __restrict__ out, long long n_tokens, int vocab, int F) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long t = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); t < n_tokens;
       t += static_cast<long long>(gridDim.x) * warps_per_block) {
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const float* src = table + static_cast<long long>(ok ? id : 0) * F;
    float* dst = out + t * F;
    for (int i = lane; i < F; i += 32) dst[i] = ok ? __ldg(src + i) : 0.f;
  }
}


// Fused: word[id] (+ type0) (+ pos[s]) -> LayerNorm -> out row. One warp per token, F <= 128*VPL.
template <int VPL>
__global__ void __launch_bounds__(256) embed_ln_kernel(const EmbedArgs a) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = a.F >> 2;
  const long long total = static_cast<long long>(a.B) * a.S;
  for (long long tok = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); tok < total;
       tok += static_cast<long long>(gridDim.x) * warps_per_block) {
    const int b = static_cast<int>(tok / a.S), s = static_cast<int>(tok % a.S);
    long long orow;
    if (a.cu_seqlens) {
      const int start = a.cu_seqlens[b], len = a.cu_seqlens[b + 1] - start;
      if (s >= len) continue;
      orow = start + s;
    } else {
      orow = tok;
    }
    const int id = a.ids[tok];
    const bool ok = id >= 0 && id < a.vocab;
    const float4* wp = reinterpret_cast<const float4*>(a.word + static_cast<long long>(ok ? id : 0) * a.F);
    const float4* pp = (a.pos && s < a.max_pos) ? reinterpret_cast<const float4*>(a.pos + static_cast<long long>(s) * a.F) : nullptr;
    const float4* tp = a.type0 ? reinterpret_cast<const float4*>(a.type0) : nullptr;
    float4 v[VPL];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int idx = lane + i * 32;
      v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (idx < nvec) {
        if (ok) v[i] = __ldg(wp + idx);
        if (tp) { float4 q = __ldg(tp + idx); v[i].x += q.x; v[i].y += q.y; v[i].z += q.z; v[i].w += q.w; }
        if (pp) { float4 q = __ldg(pp + idx); v[i].x += q.x; v[i].y += q.y; v[i].z += q.z; v[i].w += q.w; }
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    }
    float mean = 0.f, rstd = 1.f;
    if (a.gamma) {
      mean = warp_sum(sum) / static_cast<float>(a.F);
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int idx = lane + i * 32;
        if (idx < nvec) {
          const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
          sq += (dx * dx + dy * dy) + (dz * dz + dw * dw);
        }
      }
      const float var = warp_sum(sq) / static_cast<float>(a.F);
      rstd = rsqrtf(var + a.eps);
      rstd = rstd * (1.5f - 0.5f * (var + a.eps) * rstd * rstd);
    }
    float4* op = reinterpret_cast<float4*>(a.out + orow * a.F);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
        float4 o = v[i];
        if (a.gamma) {
          const float4 g = __ldg(reinterpret_cast<const float4*>(a.gamma) + idx);
          const float4 bt = a.beta ? __ldg(reinterpret_cast<const float4*>(a.beta) + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
          o.x = (o.x - mean) * rstd * g.x + bt.x;
          o.y = (o.y - mean) * rstd * g.y + bt.y;
          o.z = (o.z - mean) * rstd * g.z + bt.z;
          o.w = (o.w - mean) * rstd * g.w + bt.w;
        }
        if (a.round_tf32) { o.x = round_to_tf32(o.x); o.y = round_to_tf32(o.y); o.z = round_to_tf32(o.z); o.w = round_to_tf32(o.w); }
        if (a.out_bf16) {
          uint2 pk;
          pk.x = pack_bf16x2(o.x, o.y);
          pk.y = pack_bf16x2(o.z, o.w);
          reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.out) + orow * a.F)[idx] = pk;
        } else {
          op[idx] = o;
        }
      }
    }
  }
}


// Masked mean over the tokens of one sequence, then optional L2 normalise. One CTA per sequence.
__global__ void __launch_bounds__(128) pool_normalize_kernel(const PoolArgs a) {
  extern __shared__ float pooled[];  // F floats + 4 partial sums
  const int b = blockIdx.x;
  int row0, len;
  if (a.cu_seqlens) { row0 = a.cu_seqlens[b]; len = a.cu_seqlens[b + 1] - row0; }
  else { row0 = b * a.S; len = a.S; }
  if (a.cls) len = min(len, 1);   // CLS pooling: the first token stands for the sequence (zero vector for an empty one)
  const float* mk = (a.mask && !a.cls) ? a.mask + static_cast<long long>(b) * a.S : nullptr;
  float count = 0.f;
  if (mk) { for (int s = 0; s < len; ++s) count += (mk[s] > 0.5f) ? 1.f : 0.f; }
  else count = static_cast<float>(len);
  float nrm = 0.f;
  for (int f = threadIdx.x; f < a.F; f += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < len; ++s) {
      if (!mk || mk[s] > 0.5f) acc += a.x[static_cast<long long>(row0 + s) * a.F + f];
    }
    const float v = count > 0.f ? acc / count : 0.f;
    pooled[f] = v;
    nrm += v * v;
  }
  float* part = pooled + a.F;
  nrm = warp_sum(nrm);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = nrm;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) tot += part[w];
  const float inv = a.normalize ? 1.f / (sqrtf(tot) + 1e-8f) : 1.f;
  for (int f = threadIdx.x; f < a.F; f += blockDim.x) a.out[static_cast<long long>(b) * a.F + f] = pooled[f] * inv;
}

// The same for feature counts that are a multiple of 4 (up to 128 * VPL) and 16-byte aligned rows: the four warps take
// every fourth token of the sequence, a lane holds VPL 16-byte pieces of the running sum, and several rows' loads are
// in flight per thread (the scalar form above has one 4-byte load per thread and row in flight and reaches a third of
// the copy bandwidth). The four partial sums meet in shared memory and are added in warp order, so a sequence's vector
// does not depend on what else is in the batch.
template <int VPL>
__global__ void __launch_bounds__(128) pool_normalize_vec_kernel(const PoolArgs a) {
  __shared__ float4 part[4][32 * VPL];
  __shared__ float red[4];
  const int b = blockIdx.x, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nv = a.F >> 2;
  int row0, len;
  if (a.cu_seqlens) { row0 = a.cu_seqlens[b]; len = a.cu_seqlens[b + 1] - row0; }
  else { row0 = b * a.S; len = a.S; }
  if (a.cls) len = min(len, 1);
  const float* mk = (a.mask && !a.cls) ? a.mask + static_cast<long long>(b) * a.S : nullptr;
  float count = 0.f;
  if (mk) { for (int s = 0; s < len; ++s) count += (mk[s] > 0.5f) ? 1.f : 0.f; }
  else count = static_cast<float>(len);
  float4 acc[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int s = w; s < len; s += 4) {
    if (mk && !(mk[s] > 0.5f)) continue;
    const float4* rp = reinterpret_cast<const float4*>(a.x + static_cast<long long>(row0 + s) * a.F);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int j = lane + 32 * i;
      if (j < nv) {
        const float4 v = __ldg(rp + j);
        acc[i].x += v.x; acc[i].y += v.y; acc[i].z += v.z; acc[i].w += v.w;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) part[w][lane + 32 * i] = acc[i];
  __syncthreads();
  const float inv_count = count > 0.f ? 1.f / count : 0.f;
  float nrm = 0.f;
  for (int j = threadIdx.x; j < nv; j += 128) {
    float4 v = part[0][j];
#pragma unroll
    for (int ww = 1; ww < 4; ++ww) { const float4 p = part[ww][j]; v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w; }
    v.x *= inv_count; v.y *= inv_count; v.z *= inv_count; v.w *= inv_count;
    part[0][j] = v;                                   // only this thread touches piece j from here on
    nrm += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  nrm = warp_sum(nrm);
  if (lane == 0) red[w] = nrm;
  __syncthreads();
  const float tot = red[0] + red[1] + red[2] + red[3];
  const float inv = a.normalize ? 1.f / (sqrtf(tot) + 1e-8f) : 1.f;
  float4* op = reinterpret_cast<float4*>(a.out + static_cast<long long>(b) * a.F);
  for (int j = threadIdx.x; j < nv; j += 128) {
    float4 v = part[0][j];
    v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
    op[j] = v;
  }
}

// ---- unfused attention (compatibility with callers of attention_scores / attention_mask / attention_output) ----
// These materialise the (B,H,S,S) tensor exactly as the reference's three dispatches do; plain fp32 FMAs.
// scores[b,h,q,k] = scale * sum_d Q[b,q,h,d] K[b,k,h,d]; one warp per (b,h,q), lanes over keys.
__global__ void __launch_bounds__(256) attn_scores_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                          float* __restrict__ scores, int B, int S, int H, int D, float scale) {
  const int lane = threadIdx.x & 31;
  const long long n_rows = static_cast<long long>(B) * H * S;
  const int warps_per_block = blockDim.x >> 5;
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); row < n_rows;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const int qi = static_cast<int>(row % S);
    const int h = static_cast<int>((row / S) % H);
    const int b = static_cast<int>(row / (static_cast<long long>(S) * H));
    const float* qp = q + ((static_cast<long long>(b) * S + qi) * H + h) * D;
    for (int kk = lane; kk < S; kk += 32) {
      const float* kp = k + ((static_cast<long long>(b) * S + kk) * H + h) * D;
      float acc = 0.f;
      for (int d = 0; d < D; ++d) acc = fmaf(__ldg(qp + d), __ldg(kp + d), acc);
      scores[row * S + kk] = acc * scale;
    }
  }
}
// causal: key > query -> mask_value; otherwise key-padding mask (B,S), < 0.5 -> mask_value (attention-mask.glsl:42-53)
__global__ void __launch_bounds__(256) attn_mask_kernel(float* __restrict__ scores, const float* __restrict__ mask, long long n,
                                                        int H, int S, int use_causal, float mask_value) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int kk = static_cast<int>(i % S);
    const int qi = static_cast<int>((i / S) % S);
    const long long b = i / (static_cast<long long>(S) * S * H);
    if (use_causal) { if (kk > qi) scores[i] = mask_value; }
    else if (mask[b * S + kk] < 0.5f) scores[i] = mask_value;
  }
}
// out[b,q,h,:] = sum_k W[b,h,q,k] V[b,k,h,:]; one warp per (b,h,q), lanes over the head dim. W is (B,H,Sq,Sk) and V
// (B,Sk,H,D): Sq == Sk for attention-output.glsl; causal keeps k <= q (attention-output-gpt.glsl); Sq != Sk is the
// decoder-over-encoder form of attention-output-t5.glsl.
__global__ void __launch_bounds__(256) attn_output_kernel(const float* __restrict__ w, const float* __restrict__ v,
                                                          float* __restrict__ out, int B, int Sq, int Sk, int H, int D, int causal) {
  const int lane = threadIdx.x & 31;
  const long long n_rows = static_cast<long long>(B) * H * Sq;
  const int warps_per_block = blockDim.x >> 5;
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); row < n_rows;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const int qi = static_cast<int>(row % Sq);
    const int h = static_cast<int>((row / Sq) % H);
    const int b = static_cast<int>(row / (static_cast<long long>(Sq) * H));
    const float* wp = w + row * Sk;
    const int k_end = causal ? min(qi + 1, Sk) : Sk;
    for (int d = lane; d < D; d += 32) {
      float acc = 0.f;
      for (int kk = 0; kk < k_end; ++kk) acc = fmaf(__ldg(wp + kk), __ldg(v + ((static_cast<long long>(b) * Sk + kk) * H + h) * D + d), acc);
      out[((static_cast<long long>(b) * Sq + qi) * H + h) * D + d] = acc;
    }
  }
}

// cos/sin tables for RoPE: theta(pos, i) = (pos / scaling) * base^(-2 i / D), computed in double.
__global__ void rope_table_kernel(float* __restrict__ cos_t, float* __restrict__ sin_t, int S, int D, float base, float scaling) {
  const int half = D / 2;
  const long long n = static_cast<long long>(S) * half;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int pos = static_cast<int>(idx / half), i = static_cast<int>(idx % half);
    const double inv_freq = pow(static_cast<double>(base), -2.0 * i / D);
    const double th = (static_cast<double>(pos) / scaling) * inv_freq;
    cos_t[idx] = static_cast<float>(cos(th));
    sin_t[idx] = static_cast<float>(sin(th));
  }
}

// RoPE pre-pass for long-sequence attention: rotates every head of a 2-D view [rows][pitch] (head h in columns
// [h*D, (h+1)*D)) into a dense [rows][H*D] copy. A row's position is its index inside its sequence (padded: row % S,
// packed: row - cu_seqlens[b]). One thread per 16-byte piece (interleaved) or per pair of pieces (rotate-half).
template <bool kBf16>
__global__ void __launch_bounds__(256) rope_rows_kernel(const void* __restrict__ src, void* __restrict__ dst, long long rows,
                                                        long long pitch, int H, int D, int S, const int* __restrict__ cu_seqlens,
                                                        int B, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                        int style) {
  constexpr int ELT = kBf16 ? 2 : 4;
  constexpr int EPP = 16 / ELT;
  const int pieces = D / EPP;
  const int work_per_head = style == 1 ? pieces : pieces / 2;
  const long long total = rows * H * work_per_head;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int w = static_cast<int>(idx % work_per_head);
    const long long rh = idx / work_per_head;
    const int h = static_cast<int>(rh % H);
    const long long row = rh / H;
    int pos;
    if (cu_seqlens) {
      int lo = 0, hi = B;  // last b with cu_seqlens[b] <= row
      while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (cu_seqlens[mid] <= row) lo = mid; else hi = mid; }
      pos = static_cast<int>(row - cu_seqlens[lo]);
    } else {
      pos = static_cast<int>(row % S);
    }
    pos = min(pos, S - 1);
    const float* ct = cos_t + static_cast<long long>(pos) * (D / 2);
    const float* st = sin_t + static_cast<long long>(pos) * (D / 2);
    const uint4* sp = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(src) + (row * pitch + h * D) * ELT);
    uint4* dp = reinterpret_cast<uint4*>(reinterpret_cast<char*>(dst) + (row * H + h) * static_cast<long long>(D) * ELT);
    auto unpack = [&](const uint4& q, float* f) {
      if constexpr (kBf16) {
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(hh[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
      } else {
        f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
      }
    };
    auto pack = [&](const float* f) -> uint4 {
      uint4 q;
      if constexpr (kBf16) {
        q.x = pack_bf16x2(f[0], f[1]); q.y = pack_bf16x2(f[2], f[3]); q.z = pack_bf16x2(f[4], f[5]); q.w = pack_bf16x2(f[6], f[7]);
      } else {
        q.x = __float_as_uint(round_to_tf32(f[0])); q.y = __float_as_uint(round_to_tf32(f[1]));
        q.z = __float_as_uint(round_to_tf32(f[2])); q.w = __float_as_uint(round_to_tf32(f[3]));
      }
      return q;
    };
    if (style == 1) {
      float f[EPP];
      unpack(sp[w], f);
#pragma unroll
      for (int e = 0; e < EPP; e += 2) {
        const int i = (w * EPP + e) >> 1;
        const float c = __ldg(ct + i), sn = __ldg(st + i);
        const float x0 = f[e], x1 = f[e + 1];
        f[e] = x0 * c - x1 * sn;
        f[e + 1] = x0 * sn + x1 * c;
      }
      dp[w] = pack(f);
    } else {
      float f0[EPP], f1[EPP];
      unpack(sp[w], f0);
      unpack(sp[w + pieces / 2], f1);
#pragma unroll
      for (int e = 0; e < EPP; ++e) {
        const int i = w * EPP + e;
        const float c = __ldg(ct + i), sn = __ldg(st + i);
        const float x0 = f0[e], x1 = f1[e];
        f0[e] = x0 * c - x1 * sn;
        f1[e] = x1 * c + x0 * sn;
      }
      dp[w] = pack(f0);
      dp[w + pieces / 2] = pack(f1);
    }
  }
}

// Stand-alone RoPE on a [B][S][H][D] tensor (apply_rope): out may alias x.
__global__ void __launch_bounds__(256) rope_apply_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                         const int* __restrict__ position_ids, long long n_pairs, int S,
                                                         int H, int D, int style) {
  const int half = D / 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n_pairs; idx += stride) {
    const int i = static_cast<int>(idx % half);
    const long long tok_head = idx / half;           // (b*S + s)*H + h
    const long long tok = tok_head / H;              // b*S + s
    const int pos = position_ids ? position_ids[tok] : static_cast<int>(tok % S);
    const float c = cos_t[static_cast<long long>(pos) * half + i], s = sin_t[static_cast<long long>(pos) * half + i];
    const long long base = tok_head * D;
    const int i0 = (style == 1) ? 2 * i : i;
    const int i1 = (style == 1) ? 2 * i + 1 : i + half;
    const float x0 = x[base + i0], x1 = x[base + i1];
    y[base + i0] = x0 * c - x1 * s;
    y[base + i1] = x1 * c + x0 * s;
  }
}

}  // namespace gb
