// Vector search on top of the GEMM: pairwise distances (reference backend/faiss.py:25-104, shader
// faiss-distance.glsl:29-83) and top-k selection per query (backend/faiss.py:106-195, shader faiss-topk.glsl).
//
// Distances are one tcgen05 GEMM over split operands plus one elementwise pass that turns dot products into
// distances (kept out of the GEMM's epilogue: that code is shared with the encoder's launches and is
// register-critical). A single tf32 pass is 5e-4 off per dot product, which reorders near neighbours, so every
// vector x is written as hi + lo (hi = x rounded to tf32, lo = (x - hi) rounded to tf32) and the GEMM runs over
// K' = 3 dim with rows [hi | lo | hi] for the queries and [hi | hi | lo] for the database: hi.hi + lo.hi + hi.lo in
// one fp32 accumulator, i.e. the fp32 dot product up to the dropped lo.lo term (2^-22 relative). The squared norms
// the L2 and cosine forms need are taken from the unsplit fp32 values by the kernel that writes the split rows.
//
// Top-k is exact: a radix select over order-preserving 32-bit keys finds the k-th smallest distance of a row (or of
// a segment of a long row, when there are few rows) in four histogram passes, one more pass collects everything
// below it and, in index order, as many ties as are still needed, and a bitonic sort in shared memory puts the k
// results in ascending (distance, index) order.
#include "gemm.cuh"  // round_to_tf32, GemmArgs
#include "internal.h"
#include <algorithm>
#include <mutex>

namespace gb {

// In place: out[q][d] holds q.d on entry; qn2 / dn2 are the squared norms.
__global__ void __launch_bounds__(256) dot_to_distance_kernel(float* __restrict__ out, const float* __restrict__ qn2,
                                                              const float* __restrict__ dn2, int nq, int ndb, int mode) {
  const long long total = static_cast<long long>(nq) * ndb;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int q = static_cast<int>(i / ndb), d = static_cast<int>(i - static_cast<long long>(q) * ndb);
    const float acc = out[i];
    float r;
    if (mode == DIST_L2) r = sqrtf(fmaxf(__ldg(qn2 + q) + __ldg(dn2 + d) - 2.f * acc, 0.f));
    else if (mode == DIST_COSINE) r = 1.f - acc / (sqrtf(__ldg(qn2 + q)) * sqrtf(__ldg(dn2 + d)) + 1e-8f);
    else r = -acc;
    out[i] = r;
  }
}

// float -> uint32 whose unsigned order is the float order (-0 < +0, NaNs at the ends)
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int TOPK_THREADS = 256;
constexpr int TOPK_MAX_K = 1024;

// One CTA per (row, segment): the k smallest of vals[row][seg_begin .. seg_end) in ascending (value, position) order.
// With segs > 1 a row is cut into equal parts and the k winners of each part are written side by side
// (out row = row * segs + seg) for a second launch to merge; src_idx, when given, maps positions of that second
// launch back to column indices of the original row. Every segment must hold at least k elements.
__global__ void __launch_bounds__(TOPK_THREADS) topk_rows_kernel(const float* __restrict__ vals, long long ld, int len, int segs,
                                                                 int k, const uint32_t* __restrict__ src_idx,
                                                                 uint32_t* __restrict__ idx_out, float* __restrict__ val_out,
                                                                 uint32_t idx_base = 0, long long out_ld = 0, long long out_off = 0) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_need, s_count, s_ties;
  __shared__ uint32_t warp_tot[TOPK_THREADS / 32];
  __shared__ uint32_t cand_key[TOPK_MAX_K];
  __shared__ uint32_t cand_idx[TOPK_MAX_K];
  const int row_id = blockIdx.x / segs, seg = blockIdx.x - row_id * segs;
  const int seg_begin = static_cast<int>(static_cast<long long>(len) * seg / segs);
  const int ndb = static_cast<int>(static_cast<long long>(len) * (seg + 1) / segs) - seg_begin;   // elements of this segment
  const float* row = vals + static_cast<long long>(row_id) * ld + seg_begin;
  const uint32_t* src = src_idx ? src_idx + static_cast<long long>(row_id) * ld + seg_begin : nullptr;
  const int t = threadIdx.x;

  // ---- radix select: after the loop s_prefix is the key of the k-th smallest element and s_need (>= 1) says how
  // many elements equal to it belong to the result
  if (t == 0) { s_prefix = 0; s_need = static_cast<uint32_t>(k); }
  __syncthreads();
  for (int shift = 24; shift >= 0; shift -= 8) {
    hist[t] = 0;                                    // TOPK_THREADS == 256 bins
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = t; i < ndb; i += TOPK_THREADS) {
      const uint32_t key = order_key(__ldg(row + i));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (t == 0) {
      uint32_t need = s_need, bin = 0;
      for (; bin < 255u; ++bin) {
        if (hist[bin] >= need) break;
        need -= hist[bin];
      }
      s_prefix = prefix | (bin << shift);
      s_need = need;
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;
  const uint32_t need_ties = s_need;

  // ---- collect: everything below the k-th key in any order, ties in index order until need_ties are taken
  if (t == 0) { s_count = 0; s_ties = 0; }
  __syncthreads();
  const int lane = t & 31, warp = t >> 5;
  for (int base = 0; base < ndb; base += TOPK_THREADS) {
    const int i = base + t;
    const uint32_t key = i < ndb ? order_key(__ldg(row + i)) : 0xffffffffu;
    const bool below = i < ndb && key < kth;
    const bool tie = i < ndb && key == kth;
    if (below) {
      const uint32_t slot = atomicAdd(&s_count, 1u);
      cand_key[slot] = key;
      cand_idx[slot] = static_cast<uint32_t>(i);
    }
    if (__syncthreads_or(tie)) {
      // rank of each tie inside this block of 256 consecutive indices
      const uint32_t bal = __ballot_sync(0xffffffffu, tie);
      if (lane == 0) warp_tot[warp] = __popc(bal);
      __syncthreads();
      uint32_t before = s_ties;
      for (int w = 0; w < warp; ++w) before += warp_tot[w];
      const uint32_t rank = before + __popc(bal & ((1u << lane) - 1u));
      if (tie && rank < need_ties) {
        const uint32_t slot = atomicAdd(&s_count, 1u);
        cand_key[slot] = key;
        cand_idx[slot] = static_cast<uint32_t>(i);
      }
      __syncthreads();
      if (t == 0) {
        uint32_t tot = 0;
        for (int w = 0; w < TOPK_THREADS / 32; ++w) tot += warp_tot[w];
        s_ties += tot;
      }
      __syncthreads();
    }
  }
  __syncthreads();

  // ---- sort the k candidates by (key, index): bitonic network over the next power of two, padded with maxima
  int n2 = 1;
  while (n2 < k) n2 <<= 1;
  for (int i = k + t; i < n2; i += TOPK_THREADS) { cand_key[i] = 0xffffffffu; cand_idx[i] = 0xffffffffu; }
  __syncthreads();
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = t; i < n2; i += TOPK_THREADS) {
        const int j = i ^ stride;
        if (j > i) {
          const bool up = (i & size) == 0;
          const uint32_t ki = cand_key[i], kj = cand_key[j], ii = cand_idx[i], ij = cand_idx[j];
          const bool gt = ki > kj || (ki == kj && ii > ij);
          if (gt == up) { cand_key[i] = kj; cand_key[j] = ki; cand_idx[i] = ij; cand_idx[j] = ii; }
        }
      }
      __syncthreads();
    }
  }
  // default: one packed row of k results per (row, segment); with out_ld the k results go to row_id * out_ld + out_off
  // (the winners of one database chunk inside a wider candidate matrix) and idx_base is added to the positions
  const long long out0 = out_ld > 0 ? static_cast<long long>(row_id) * out_ld + out_off + static_cast<long long>(seg) * k
                                    : static_cast<long long>(blockIdx.x) * k;
  for (int i = t; i < k; i += TOPK_THREADS) {
    const uint32_t id = cand_idx[i];
    idx_out[out0 + i] = src ? __ldg(src + id) : idx_base + static_cast<uint32_t>(seg_begin) + id;
    val_out[out0 + i] = __ldg(row + id);
  }
}

}  // namespace gb

using namespace gb;

extern "C" {

int grilly_faiss_distances(grilly_ctx* ctx, const float* queries, const float* database, float* out, int num_queries,
                           int num_database, int dim, int distance_type) {
  if (!ctx) return GRILLY_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (cudaSetDevice(ctx->device) != cudaSuccess) return set_error(ctx, GRILLY_ERR_CUDA, "cudaSetDevice failed");
  if (!queries || !database || !out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "faiss_distances: null operand");
  if (num_queries <= 0 || num_database <= 0 || dim <= 0)
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "faiss_distances: sizes must be positive");
  if (distance_type < GRILLY_DIST_L2 || distance_type > GRILLY_DIST_DOT)
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "faiss_distances: distance_type must be L2, COSINE or DOT");
  const int dim_pad = (dim + 3) & ~3;                       // 16-byte rows for the TMA descriptors
  const long long kq = 3LL * dim_pad;
  if (kq > 2147483647LL) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "faiss_distances: dim too large");
  float *qs = nullptr, *ds = nullptr, *qn = nullptr, *dn = nullptr;
  const size_t q_bytes = static_cast<size_t>(num_queries) * kq * sizeof(float);
  const size_t d_bytes = static_cast<size_t>(num_database) * kq * sizeof(float);
  cudaError_t e = cudaMallocAsync(&qs, q_bytes, ctx->stream);
  if (e == cudaSuccess) e = cudaMallocAsync(&ds, d_bytes, ctx->stream);
  if (e == cudaSuccess) e = cudaMallocAsync(&qn, static_cast<size_t>(num_queries) * sizeof(float), ctx->stream);
  if (e == cudaSuccess) e = cudaMallocAsync(&dn, static_cast<size_t>(num_database) * sizeof(float), ctx->stream);
  int rc = GRILLY_OK;
  if (e != cudaSuccess) {
    cudaGetLastError();
    rc = set_error(ctx, GRILLY_ERR_OOM, "faiss_distances: no memory for the split operands (3 x the size of queries + database)");
  } else {
    rc = launch_split_rows(ctx, queries, qs, qn, num_queries, dim, dim_pad, true);
    if (!rc) rc = launch_split_rows(ctx, database, ds, dn, num_database, dim, dim_pad, false);
    GemmArgs a{};
    a.M = num_queries; a.N = num_database; a.K = static_cast<int>(kq);
    a.out = out; a.ld_out = num_database;
    if (!rc) rc = launch_gemm(ctx, false, false, qs, ds, a, 0);
    if (!rc) {
      const long long total = static_cast<long long>(num_queries) * num_database;
      const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 8LL * ctx->num_sms));
      dot_to_distance_kernel<<<blocks, 256, 0, ctx->stream>>>(out, qn, dn, num_queries, num_database, distance_type);  // GRILLY_DIST_* == gb::DIST_*
      ctx->launches++;
      if (cudaGetLastError() != cudaSuccess) rc = set_error(ctx, GRILLY_ERR_CUDA, "faiss_distances: launch failed");
    }
  }
  if (qs) cudaFreeAsync(qs, ctx->stream);
  if (ds) cudaFreeAsync(ds, ctx->stream);
  if (qn) cudaFreeAsync(qn, ctx->stream);
  if (dn) cudaFreeAsync(dn, ctx->stream);
  return rc;
}

int grilly_faiss_search(grilly_ctx* ctx, const float* queries, const float* database, int num_queries, int num_database, int dim,
                        int k, int distance_type, unsigned int* indices_out, float* distances_out) {
  if (!ctx) return GRILLY_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (cudaSetDevice(ctx->device) != cudaSuccess) return set_error(ctx, GRILLY_ERR_CUDA, "cudaSetDevice failed");
  if (!queries || !database || !indices_out || !distances_out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "faiss_search: null operand");
  if (num_queries <= 0 || num_database <= 0 || dim <= 0 || k <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "faiss_search: sizes must be positive");
  if (k > num_database) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "faiss_search: k exceeds the number of database vectors");
  if (k > TOPK_MAX_K) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "faiss_search: k is limited to 1024");
  if (distance_type != GRILLY_DIST_L2 && distance_type != GRILLY_DIST_COSINE && distance_type != GRILLY_DIST_DOT)
    return set_error(ctx, GRILLY_ERR_INVALID_ARG, "faiss_search: unknown distance type");
  const int dim_pad = (dim + 3) & ~3;
  const long long kq = 3LL * dim_pad;
  if (kq > 2147483647LL) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "faiss_search: dim too large");
  // Database chunks whose distance block (num_queries x chunk floats) stays in L2: the block is written by the GEMM,
  // turned into distances and reduced to its k best per query while it is still there; the full matrix never exists.
  long long chunk = (16LL << 20) / num_queries;
  chunk = std::max<long long>(2048, std::min<long long>(chunk, 65536)) & ~255LL;
  const int nchunks = static_cast<int>((num_database + chunk - 1) / chunk);
  const long long per = (num_database + nchunks - 1) / nchunks;            // balanced: every chunk holds at least k vectors
  const long long chunk_cols = (per + 3) & ~3LL;                            // row pitch of the distance block (16-byte rows)
  const long long cand = static_cast<long long>(nchunks) * k;
  float *qs = nullptr, *ds = nullptr, *qn = nullptr, *dn = nullptr, *blk = nullptr, *cval = nullptr;
  uint32_t* cidx = nullptr;
  cudaError_t e = cudaMallocAsync(&qs, static_cast<size_t>(num_queries) * kq * sizeof(float), ctx->stream);
  if (e == cudaSuccess) e = cudaMallocAsync(&ds, static_cast<size_t>(chunk_cols) * kq * sizeof(float), ctx->stream);
  if (e == cudaSuccess) e = cudaMallocAsync(&qn, static_cast<size_t>(num_queries) * sizeof(float), ctx->stream);
  if (e == cudaSuccess) e = cudaMallocAsync(&dn, static_cast<size_t>(chunk_cols) * sizeof(float), ctx->stream);
  if (e == cudaSuccess) e = cudaMallocAsync(&blk, static_cast<size_t>(num_queries) * chunk_cols * sizeof(float), ctx->stream);
  if (e == cudaSuccess && nchunks > 1) e = cudaMallocAsync(&cval, static_cast<size_t>(num_queries) * cand * sizeof(float), ctx->stream);
  if (e == cudaSuccess && nchunks > 1) e = cudaMallocAsync(&cidx, static_cast<size_t>(num_queries) * cand * sizeof(uint32_t), ctx->stream);
  int rc = GRILLY_OK;
  if (e != cudaSuccess) {
    cudaGetLastError();
    rc = set_error(ctx, GRILLY_ERR_OOM, "faiss_search: no memory for the scratch (split operands of one chunk, one distance block, candidates)");
  } else {
    rc = launch_split_rows(ctx, queries, qs, qn, num_queries, dim, dim_pad, true);
    for (int c = 0; c < nchunks && !rc; ++c) {
      const long long c0 = c * per;
      const int n = static_cast<int>(std::min<long long>(per, num_database - c0));
      const int n_pad = (n + 3) & ~3;
      rc = launch_split_rows(ctx, database + c0 * dim, ds, dn, n, dim, dim_pad, false);
      if (rc) break;
      GemmArgs a{};
      a.M = num_queries; a.N = n; a.K = static_cast<int>(kq);
      a.out = blk; a.ld_out = n_pad;
      if ((rc = launch_gemm(ctx, false, false, qs, ds, a, 0))) break;
      // distances in place on the block (row pitch n_pad; the padding columns are never read)
      const long long total = static_cast<long long>(num_queries) * n_pad;
      const int blocks = static_cast<int>(std::min<long long>((total + 255) / 256, 8LL * ctx->num_sms));
      dot_to_distance_kernel<<<blocks, 256, 0, ctx->stream>>>(blk, qn, dn, num_queries, n_pad, distance_type);
      if (nchunks == 1) {
        topk_rows_kernel<<<num_queries, TOPK_THREADS, 0, ctx->stream>>>(blk, n_pad, n, 1, k, nullptr, indices_out, distances_out);
      } else {
        topk_rows_kernel<<<num_queries, TOPK_THREADS, 0, ctx->stream>>>(blk, n_pad, n, 1, k, nullptr, cidx, cval,
                                                                        static_cast<uint32_t>(c0), cand, static_cast<long long>(c) * k);
      }
      ctx->launches += 2;
      if (cudaGetLastError() != cudaSuccess) rc = set_error(ctx, GRILLY_ERR_CUDA, "faiss_search: launch failed");
    }
    if (!rc && nchunks > 1) {
      topk_rows_kernel<<<num_queries, TOPK_THREADS, 0, ctx->stream>>>(cval, cand, static_cast<int>(cand), 1, k, cidx, indices_out, distances_out);
      ctx->launches++;
      if (cudaGetLastError() != cudaSuccess) rc = set_error(ctx, GRILLY_ERR_CUDA, "faiss_search: merge launch failed");
    }
  }
  for (void* p : {static_cast<void*>(qs), static_cast<void*>(ds), static_cast<void*>(qn), static_cast<void*>(dn), static_cast<void*>(blk),
                  static_cast<void*>(cval), static_cast<void*>(cidx)})
    if (p) cudaFreeAsync(p, ctx->stream);
  return rc;
}

int grilly_faiss_topk(grilly_ctx* ctx, const float* distances, int num_queries, int num_database, int k,
                      unsigned int* indices_out, float* distances_out) {
  if (!ctx) return GRILLY_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (cudaSetDevice(ctx->device) != cudaSuccess) return set_error(ctx, GRILLY_ERR_CUDA, "cudaSetDevice failed");
  if (!distances || !indices_out || !distances_out) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "faiss_topk: null operand");
  if (num_queries <= 0 || num_database <= 0 || k <= 0) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "faiss_topk: sizes must be positive");
  if (k > num_database) return set_error(ctx, GRILLY_ERR_INVALID_ARG, "faiss_topk: k exceeds the number of database vectors");
  if (k > TOPK_MAX_K) return set_error(ctx, GRILLY_ERR_UNSUPPORTED, "faiss_topk: k is limited to 1024");
  // Few long rows: cut each row into segments so that the whole GPU works on them, then merge the segments' winners.
  int segs = 1;
  if (num_queries < 2 * ctx->num_sms && num_database >= 65536) {
    const int want = (4 * ctx->num_sms + num_queries - 1) / num_queries;
    const int most = num_database / std::max(k, 8192);                     // every segment keeps at least k elements
    segs = std::max(1, std::min(want, most));
  }
  if (segs == 1) {
    topk_rows_kernel<<<num_queries, TOPK_THREADS, 0, ctx->stream>>>(distances, num_database, num_database, 1, k, nullptr,
                                                                    indices_out, distances_out);
    ctx->launches++;
    GB_CUDA_CHECK(ctx, cudaGetLastError());
    return GRILLY_OK;
  }
  const size_t cand = static_cast<size_t>(num_queries) * segs * k;
  uint32_t* cidx = nullptr;
  float* cval = nullptr;
  GB_CUDA_CHECK(ctx, cudaMallocAsync(&cidx, cand * sizeof(uint32_t), ctx->stream));
  cudaError_t e = cudaMallocAsync(&cval, cand * sizeof(float), ctx->stream);
  if (e != cudaSuccess) {
    cudaFreeAsync(cidx, ctx->stream);
    cudaGetLastError();
    return set_error(ctx, GRILLY_ERR_OOM, "faiss_topk: no memory for the per-segment candidates");
  }
  topk_rows_kernel<<<num_queries * segs, TOPK_THREADS, 0, ctx->stream>>>(distances, num_database, num_database, segs, k, nullptr, cidx, cval);
  topk_rows_kernel<<<num_queries, TOPK_THREADS, 0, ctx->stream>>>(cval, static_cast<long long>(segs) * k, segs * k, 1, k, cidx,
                                                                  indices_out, distances_out);
  ctx->launches += 2;
  e = cudaGetLastError();
  cudaFreeAsync(cidx, ctx->stream);
  cudaFreeAsync(cval, ctx->stream);
  if (e != cudaSuccess) return set_error(ctx, GRILLY_ERR_CUDA, std::string("faiss_topk: ") + cudaGetErrorString(e));
  return GRILLY_OK;
}

}  // extern "C"
