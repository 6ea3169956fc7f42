// y = LayerNorm(x W^T + bias + residual) * gamma + beta in ONE kernel: the post-LN step of a BERT layer
// (utils/vulkan_sentence_transformer.py:1000-1004 and 1018-1026 in the reference: linear, add the residual, LayerNorm)
// without the pre-norm sum ever reaching memory.
//
// The row statistics need a whole output row in one place, so the tile is 128 token rows x ALL N features (N <= 512,
// a multiple of 128): tokens are the 128-row MMA operand (one TMEM lane = one token), the N features are the
// accumulator's columns, written by two tcgen05.mma of N/2 columns per k-step. One thread of the epilogue owns one
// token row, so mean and variance are plain per-thread sums:
//   pass 1 over the accumulator: v = acc + bias + residual, written back to TMEM; sum and sum of squares of (v - v_0)
//   pass 2: (v - mean) * rstd * gamma + beta, optional tf32 rounding, staged in swizzled shared memory and stored
//           with cp.async.bulk.tensor (fp32 output; whole 128-byte lines leave the SM, ragged last rows are clipped
//           by the copy engine) or with 16-byte vector stores (bf16 output).
// The accumulator takes N of the 512 TMEM columns, so there is one buffer: the main loop of the next tile starts when
// the epilogue has read the last column (operand loads for it run ahead through the shared-memory ring).
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer + TMEM allocation, warps 2..5 epilogue (one per TMEM lane quadrant).
// Every wait is bounded (ptx.cuh); a wait that gives up records a status and the CTA drains.
#pragma once
#include "gemm.cuh"

namespace gb {

constexpr int GEMM_LN_THREADS = 192;      // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int GEMM_LN_STAGING = 4 * 4096; // per epilogue warp: 32 rows x 128 B of output in the TMA store's swizzle

template <int NCHUNK>
struct GemmLnCfg {
  static constexpr int N = NCHUNK * 32;
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = N * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int MAX_SMEM = 227 * 1024;
  static constexpr int STAGES_RAW = (MAX_SMEM - 1024 - GEMM_LN_STAGING - 512) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + GEMM_LN_STAGING + 1024 /*align slack*/ + 512 /*barriers*/;
  static constexpr int TMEM_COLS = N <= 32 ? 32 : N <= 64 ? 64 : N <= 128 ? 128 : N <= 256 ? 256 : 512;
  static_assert(N <= 512 && N % 32 == 0, "one accumulator of N columns must fit TMEM");
  static_assert((N / 2) % 16 == 0 && N / 2 <= 256, "each half is one tcgen05.mma");
  static_assert(STAGES >= 2, "the operand ring needs at least two stages");
  static_assert(NCHUNK % 2 == 0, "the epilogue walks the chunks in pairs");
};

// 32 residual values of one row as registers (fp32: 8 x 16 bytes, bf16: 4 x 16 bytes)
template <bool kBf16>
struct ResChunk {
  uint4 q[kBf16 ? 4 : 8];
};
template <bool kBf16>
__device__ __forceinline__ void load_res(ResChunk<kBf16>& r, const void* residual, long long ld_res, int row, int col0, bool ok) {
  constexpr int NQ = kBf16 ? 4 : 8;
  if (ok) {
    const char* p = reinterpret_cast<const char*>(residual) + (static_cast<long long>(row) * ld_res + col0) * (kBf16 ? 2 : 4);
#pragma unroll
    for (int i = 0; i < NQ; ++i) r.q[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
  } else {
#pragma unroll
    for (int i = 0; i < NQ; ++i) r.q[i] = make_uint4(0u, 0u, 0u, 0u);
  }
}
template <bool kBf16>
__device__ __forceinline__ float res_at(const ResChunk<kBf16>& r, int j) {   // j is a compile-time constant after unrolling
  if constexpr (kBf16) {
    const uint4 q = r.q[j >> 3];
    const uint32_t w = ((j >> 1) & 3) == 0 ? q.x : ((j >> 1) & 3) == 1 ? q.y : ((j >> 1) & 3) == 2 ? q.z : q.w;
    return __uint_as_float((j & 1) ? (w & 0xffff0000u) : (w << 16));
  } else {
    const uint4 q = r.q[j >> 2];
    const uint32_t w = (j & 3) == 0 ? q.x : (j & 3) == 1 ? q.y : (j & 3) == 2 ? q.z : q.w;
    return __uint_as_float(w);
  }
}

template <int NCHUNK, bool kBf16>
__global__ void __launch_bounds__(GEMM_LN_THREADS, 1)
gemm_rowln_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ CUtensorMap tmap_out, const GemmLnArgs args) {
  using Cfg = GemmLnCfg<NCHUNK>;
  constexpr int N = Cfg::N;
  constexpr int NH = N / 2;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ELT = kBf16 ? 2 : 4;
  constexpr int BK = 128 / ELT;
  constexpr int KSTEPS = 4;
  constexpr uint32_t IDESC = make_idesc(kBf16, 128, NH, false, false);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * Cfg::STAGE_BYTES;                 // 1024-byte aligned (stage sizes are multiples of 1024)
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + GEMM_LN_STAGING);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, 4);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_out);
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
      for (int tile = blockIdx.x; tile < args.num_tiles && ok; tile += gridDim.x) {
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
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, tile * 128);
          tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * BK, 0);              // weight rows [0, N/2)
          tma_load_2d(sb + NH * 128, &tmap_b, &full_bar[stage], kb * BK, NH);  // weight rows [N/2, N)
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
      for (int tile = blockIdx.x; tile < args.num_tiles && ok; tile += gridDim.x, ++it) {
        // the one accumulator is free again when the epilogue of the previous tile has read it
        if (!mbar_wait(tmem_empty, (static_cast<uint32_t>(it) & 1u) ^ 1u, abort_flag)) {
          if (!*abort_flag) atomicCAS(args.err, 0, ERR_WAIT_TMEM_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < args.num_k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            if (!*abort_flag) atomicCAS(args.err, 0, ERR_WAIT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_desc_lo + stage * (Cfg::STAGE_BYTES >> 4);
          const uint32_t b_lo = b_desc_lo + stage * (Cfg::STAGE_BYTES >> 4);
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            const uint64_t adesc = (static_cast<uint64_t>(a_desc_hi) << 32) | (a_lo + ks * 2);
            const uint64_t bdesc0 = (static_cast<uint64_t>(b_desc_hi) << 32) | (b_lo + ks * 2);
            const uint64_t bdesc1 = (static_cast<uint64_t>(b_desc_hi) << 32) | (b_lo + ((NH * 128) >> 4) + ks * 2);
            const uint32_t acc = (kb | ks) != 0 ? 1u : 0u;
            umma_ss<kBf16>(tmem_base, adesc, bdesc0, IDESC, acc);
            umma_ss<kBf16>(tmem_base + NH, adesc, bdesc1, IDESC, acc);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tmem_full);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue: one thread = one token row
    const int quad = warp & 3;
    uint8_t* my_stage = staging + (warp - 2) * 4096;
    const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const float inv_n = 1.0f / static_cast<float>(N);
    int it = 0;
    for (int tile = blockIdx.x; tile < args.num_tiles; tile += gridDim.x, ++it) {
      const int row0 = tile * 128 + quad * 32;       // first row of this warp's 32
      const int row = row0 + lane;
      const bool row_ok = row < args.M;
      const bool res_ok = row_ok && args.residual != nullptr;
      // the first residual chunk is on its way before the accumulator is complete
      ResChunk<kBf16> res;
      load_res<kBf16>(res, args.residual, args.ld_res, row, 0, res_ok);
      if (!mbar_wait(tmem_full, static_cast<uint32_t>(it) & 1u, abort_flag)) {
        if (!*abort_flag) atomicCAS(args.err, 0, ERR_WAIT_TMEM_FULL);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      uint32_t ra[32], rb[32];
      // ---------------- pass 1: v = acc + bias + residual -> TMEM; shifted sums for the row statistics
      float shift = 0.f, s1 = 0.f, s2 = 0.f;
      __syncwarp();
      tmem_ld_32x32(taddr_row, ra);
      // chunks are walked in pairs (the two register buffers alternate); the pair loop is not unrolled, which keeps
      // the compiler from hoisting a whole tile's parameter loads into registers
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
#pragma unroll
        for (int j = 0; j < 32; ++j) cur[j] = __float_as_uint(__uint_as_float(cur[j]) + res_at<kBf16>(res, j));
        // the residual registers are free: the next chunk's loads fly while this chunk is finished
        if (c + 1 < NCHUNK) load_res<kBf16>(res, args.residual, args.ld_res, row, (c + 1) * 32, res_ok);
        if (args.bias) {
          const float4* bp = reinterpret_cast<const float4*>(args.bias + c * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 q = __ldg(bp + j);
            cur[4 * j] = __float_as_uint(__uint_as_float(cur[4 * j]) + q.x);
            cur[4 * j + 1] = __float_as_uint(__uint_as_float(cur[4 * j + 1]) + q.y);
            cur[4 * j + 2] = __float_as_uint(__uint_as_float(cur[4 * j + 2]) + q.z);
            cur[4 * j + 3] = __float_as_uint(__uint_as_float(cur[4 * j + 3]) + q.w);
          }
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
      const float mean_d = s1 * inv_n;
      const float var = fmaxf(fmaf(-mean_d, mean_d, s2 * inv_n), 0.f);
      const float mean = shift + mean_d;
      float rstd = rsqrtf(var + args.eps);
      rstd = rstd * (1.5f - 0.5f * (var + args.eps) * rstd * rstd);   // one Newton step: the rounding of 1/sqrt
      // ---------------- pass 2: normalise, scale, shift, store
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
        const bool bf16_out = kBf16 && args.out_bf16;
        if (!bf16_out) {
          // the staging tile is free once the previous bulk store has READ it
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
        }
        uint8_t* rowp = my_stage + lane * 128;
        // four columns at a time, finished and put away, so that few values are live at once
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 g4 = args.gamma ? __ldg(reinterpret_cast<const float4*>(args.gamma + c * 32) + q) : make_float4(1.f, 1.f, 1.f, 1.f);
          const float4 b4 = args.beta ? __ldg(reinterpret_cast<const float4*>(args.beta + c * 32) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
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
              *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(args.out) + static_cast<long long>(row) * args.ld_out + c * 32 + 4 * q) = pk;
            }
          } else {
            // 128-byte swizzle of the tensor map: 16-byte chunk q of row r lives at chunk (q ^ (r & 7))
            *reinterpret_cast<float4*>(rowp + ((q ^ (lane & 7)) << 4)) = o;
          }
        }
        if (!bf16_out) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < args.M) {
            tma_store_2d(&tmap_out, my_stage, c * 32, row0);   // rows beyond M are clipped by the copy engine
            tma_store_commit();
          }
        }
      }
      }
      // this warp has finished reading the accumulator
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty);
    }
    if (lane == 0) tma_store_wait_all<0>();   // the staging memory must outlive the last bulk store's read, the data must land
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);   // let copies and MMAs in flight land (about 1 ms)
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace gb
