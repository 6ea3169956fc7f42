// "tf32x3": fp32-accurate products on the tf32 tensor-core path, for callers that derive argmax / top-k indices
// from the result and need them to agree with an fp32 reference (the reference computes linear and gemm in fp32:
// fnn-linear.glsl:43-57, gemm_mnk.glsl:48-87, numba_ops.py:233-238).
//
// A single tf32 product is about 3e-4 off per output, enough to swap near-equal neighbours. Every fp32 value v is
// written as hi + lo with hi = v rounded to tf32 and lo = (v - hi) rounded to tf32 (both exactly representable, so
// the MMA's operand truncation changes nothing), and the product runs over K' = 3K:
//     [hi | lo | hi] . [hi | hi | lo] = hi.hi + lo.hi + hi.lo
// in one fp32 accumulator, i.e. the fp32 dot product up to the dropped lo.lo term (2^-22 relative). Costs three
// times the MMAs plus one pass over each operand; scratch of 3 x the operand bytes comes from the context's pool.
#include "gemm.cuh"  // round_to_tf32, GemmArgs
#include "internal.h"

namespace gb {

// One warp per row: out[row] = [hi | lo | hi] (lo_second) or [hi | hi | lo], each part dim_pad wide (zero padded);
// norm2[row] = sum x^2 in fp32 when norm2 is given.
__global__ void __launch_bounds__(256) split_rows_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                         float* __restrict__ norm2, long long rows, int dim, int dim_pad,
                                                         int lo_second) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* xp = x + row * dim;
  float* op = out + row * 3LL * dim_pad;
  float s = 0.f;
  for (int d = lane; d < dim_pad; d += 32) {
    const float v = d < dim ? __ldg(xp + d) : 0.f;
    const float hi = round_to_tf32(v);
    const float lo = round_to_tf32(v - hi);
    s = fmaf(v, v, s);
    op[d] = hi;
    op[dim_pad + d] = lo_second ? lo : hi;
    op[2 * dim_pad + d] = lo_second ? hi : lo;
  }
  if (norm2) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) norm2[row] = s;
  }
}

// The [K][N] operand of gemm_mnk, split along K: out rows [0,K) = hi, [K,2K) = hi, [2K,3K) = lo.
__global__ void __launch_bounds__(256) split_stack_kernel(const float* __restrict__ b, float* __restrict__ out, long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = __ldg(b + i);
    const float hi = round_to_tf32(v);
    out[i] = hi;
    out[n + i] = hi;
    out[2 * n + i] = round_to_tf32(v - hi);
  }
}

int launch_split_rows(grilly_ctx* ctx, const float* x, float* out, float* norm2, long long rows, int dim, int dim_pad,
                      bool lo_second) {
  if (rows <= 0) return GRILLY_OK;
  if ((rows + 7) / 8 > 2147483647LL) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "split: too many rows");
  split_rows_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, ctx->stream>>>(x, out, norm2, rows, dim, dim_pad, lo_second ? 1 : 0);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  return GRILLY_OK;
}

namespace {
struct PoolScratch {   // stream-ordered scratch that is returned to the pool when the call ends
  grilly_ctx* ctx;
  std::vector<void*> ptrs;
  explicit PoolScratch(grilly_ctx* c) : ctx(c) {}
  float* get(size_t bytes) {
    void* p = nullptr;
    if (cudaMallocAsync(&p, bytes ? bytes : 16, ctx->stream) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    ptrs.push_back(p);
    return static_cast<float*>(p);
  }
  ~PoolScratch() { for (void* p : ptrs) cudaFreeAsync(p, ctx->stream); }
};
}  // namespace

// y = act(x W^T + b) (+ residual) with fp32-accurate products: x [M][K] and W [N][K] are raw (unrounded) fp32.
int linear_tf32x3(grilly_ctx* ctx, const float* x, const float* w, GemmArgs& args) {
  const int K = args.K, Kp = (K + 3) & ~3;
  const long long k3 = 3LL * Kp;
  if (k3 > 2147483647LL) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "linear (tf32x3): K too large");
  PoolScratch s(ctx);
  float* xs = s.get(static_cast<size_t>(args.M) * k3 * sizeof(float));
  float* ws = s.get(static_cast<size_t>(args.N) * k3 * sizeof(float));
  if (!xs || !ws) return set_error(ctx, GRILLY_ERR_OOM, "linear (tf32x3): no memory for the split operands (3 x the operand bytes)");
  int rc;
  if ((rc = launch_split_rows(ctx, x, xs, nullptr, args.M, K, Kp, true))) return rc;
  if ((rc = launch_split_rows(ctx, w, ws, nullptr, args.N, K, Kp, false))) return rc;
  args.K = static_cast<int>(k3);
  return launch_gemm(ctx, false, false, xs, ws, args, 0);
}

// C = A B with fp32-accurate products: A [M][K], B [K][N] raw fp32, N a multiple of 4.
int gemm_mnk_tf32x3(grilly_ctx* ctx, const float* a, const float* b, GemmArgs& args) {
  const int K = args.K, Kp = (K + 3) & ~3;
  const long long k3 = 3LL * Kp;
  if (k3 > 2147483647LL) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "gemm_mnk (tf32x3): K too large");
  if (Kp != K) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "gemm_mnk (tf32x3): K must be a multiple of 4 (pad K)");
  PoolScratch s(ctx);
  float* as = s.get(static_cast<size_t>(args.M) * k3 * sizeof(float));
  float* bs = s.get(static_cast<size_t>(k3) * args.N * sizeof(float));
  if (!as || !bs) return set_error(ctx, GRILLY_ERR_OOM, "gemm_mnk (tf32x3): no memory for the split operands (3 x the operand bytes)");
  int rc;
  if ((rc = launch_split_rows(ctx, a, as, nullptr, args.M, K, Kp, true))) return rc;
  const long long n = static_cast<long long>(K) * args.N;
  const int blocks = static_cast<int>(std::min<long long>((n + 255) / 256, 16LL * ctx->num_sms));
  split_stack_kernel<<<blocks, 256, 0, ctx->stream>>>(b, bs, n);
  ctx->launches++;
  GB_CUDA_CHECK(ctx, cudaGetLastError());
  args.K = static_cast<int>(k3);
  return launch_gemm(ctx, false, true, as, bs, args, 0);
}

}  // namespace gb
