// Block-sparse attention indexer (MiniMax-M3 "MSA"): score every 128-token block of the context
// with a small index head, keep the top-k blocks (the first `init` blocks and the `local` blocks
// around the query are always kept), and hand the selection to the paged attention kernel as a
// *virtual block table*: the pages of the selected blocks in ascending order plus the number of
// visible tokens. RoPE is applied when keys are written, so attention over the virtual table with
// the ordinary paged GQA decode kernel equals attention restricted to the selected blocks.
//
//   block_score[t, j] = max over index heads h and tokens s of block j with s <= pos(t) of
//                       scale * iq[t, h, :] . ik[s, :]
//
// The reference scores blocks with one threadgroup per (block, sequence) and selects with a
// single-thread insertion sort (msa_indexer.metal:7-171, launch msa_indexer.cpp:238-256), then
// attends over explicit token positions (msa_paged_attention.metal:34-236); its prefill builds a
// dense mask instead (models/minimax_m3.py:456-565).
#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

constexpr int kMaxIdxHeads = 8;
constexpr int kMaxTopk = 64;

__device__ __forceinline__ int find_seq(const int* cu_q, int B, int t) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// grid (sparse blocks, T); thread = one key token of the block
__global__ void __launch_bounds__(128) msa_block_scores_kernel(const bf16* __restrict__ iq, const bf16* __restrict__ cache,
                                                               const int* __restrict__ block_tables,
                                                               const int* __restrict__ cu_q,
                                                               const int* __restrict__ positions,
                                                               float* __restrict__ scores, int64_t ld, int B, int Hi,
                                                               int Di, int max_blocks, int page, int sparse_block,
                                                               float scale) {
  extern __shared__ float q_s[];  // [Hi][Di]
  __shared__ float red[32];
  const int t = blockIdx.y, j = blockIdx.x;
  const int pos = positions[t];
  if (j * sparse_block > pos) {
    if (threadIdx.x == 0) scores[t * ld + j] = -INFINITY;
    return;
  }
  for (int i = threadIdx.x; i < Hi * Di; i += blockDim.x) q_s[i] = __bfloat162float(iq[static_cast<size_t>(t) * Hi * Di + i]);
  __syncthreads();
  const int seq = cu_q ? find_seq(cu_q, B, t) : t;
  const int* bt = block_tables + static_cast<size_t>(seq) * max_blocks;
  float best = -INFINITY;
  for (int r = threadIdx.x; r < sparse_block; r += blockDim.x) {
    const int kp = j * sparse_block + r;
    if (kp > pos) continue;
    const bf16* krow = cache + (static_cast<size_t>(bt[kp / page]) * page + kp % page) * Di;
    float dot[kMaxIdxHeads];
#pragma unroll
    for (int h = 0; h < kMaxIdxHeads; ++h) dot[h] = 0.f;
    for (int d = 0; d < Di; d += 8) {
      const bf16x8 kv = ld_bf16x8(krow + d);
      float kf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f2 = unpack_bf16x2(kv.u[e]);
        kf[2 * e] = f2.x;
        kf[2 * e + 1] = f2.y;
      }
#pragma unroll
      for (int h = 0; h < kMaxIdxHeads; ++h) {
        if (h < Hi) {
#pragma unroll
          for (int e = 0; e < 8; ++e) dot[h] = fmaf(kf[e], q_s[h * Di + d + e], dot[h]);
        }
      }
    }
#pragma unroll
    for (int h = 0; h < kMaxIdxHeads; ++h)
      if (h < Hi) best = fmaxf(best, dot[h] * scale);
  }
  best = block_reduce_max(best, red);
  if (threadIdx.x == 0) scores[t * ld + j] = best;
}

// one warp per query token: forced blocks, top-k by repeated arg-max, ascending order, page expansion
__global__ void __launch_bounds__(32) msa_select_kernel(const float* __restrict__ scores, int64_t ld,
                                                        const int* __restrict__ positions,
                                                        const int* __restrict__ block_tables,
                                                        const int* __restrict__ cu_q, int B, int max_blocks, int page,
                                                        int sparse_block, int topk, int init_blocks, int local_blocks,
                                                        int* __restrict__ v_tables, int64_t ld_vt,
                                                        int* __restrict__ v_ctx) {
  __shared__ int sel[kMaxTopk];
  const int t = blockIdx.x, lane = threadIdx.x;
  const int pos = positions[t];
  const int cur = pos / sparse_block;
  const int n_blocks = cur + 1;  // causal blocks
  const int k = topk < n_blocks ? topk : n_blocks;
  const int local_start = cur - local_blocks + 1 > 0 ? cur - local_blocks + 1 : 0;
  const float* s = scores + static_cast<size_t>(t) * ld;
  auto value = [&](int j) -> float {
    if (j >= local_start && local_blocks > 0) return 1e29f;
    if (j < init_blocks) return 1e30f;
    const float v = s[j];
    return v == v ? v : -INFINITY;
  };
  // k rounds of arg-max; ties resolve to the lower block index; chosen blocks are excluded by a
  // per-lane bitmap over the lane's strided blocks (up to 32 * 64 blocks = 262144 tokens / 128)
  unsigned long long taken = 0ull;
  for (int r = 0; r < k; ++r) {
    float best = -INFINITY;
    int arg = -1;
    for (int j = lane, c = 0; j < n_blocks; j += 32, ++c) {
      if (c < 64 && ((taken >> c) & 1ull)) continue;
      const float v = value(j);
      if (arg < 0 || v > best) {
        best = v;
        arg = j;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
      if (oa >= 0 && (arg < 0 || ob > best || (ob == best && oa < arg))) {
        best = ob;
        arg = oa;
      }
    }
    if (arg >= 0 && (arg & 31) == lane) taken |= 1ull << (arg >> 5);
    if (lane == 0) sel[r] = arg;
  }
  __syncwarp();
  // ascending order (k <= 64): rank sort by lanes
  __shared__ int sorted[kMaxTopk];
  for (int i = lane; i < k; i += 32) {
    const int v = sel[i];
    int rank = 0;
    for (int m = 0; m < k; ++m) rank += (sel[m] < v) ? 1 : 0;
    sorted[rank] = v;
  }
  __syncwarp();
  const int seq = cu_q ? find_seq(cu_q, B, t) : t;
  const int* bt = block_tables + static_cast<size_t>(seq) * max_blocks;
  const int ppb = sparse_block / page;
  int* vt = v_tables + static_cast<size_t>(t) * ld_vt;
  for (int i = lane; i < k * ppb; i += 32) {
    const int blk = sorted[i / ppb];
    const int pg = blk * ppb + i % ppb;
    vt[i] = pg < max_blocks ? bt[pg] : 0;
  }
  // the query's own block is always selected (local) and is the last one: it is visible up to pos
  if (lane == 0) v_ctx[t] = (k - 1) * sparse_block + (pos - cur * sparse_block) + 1;
}

}  // namespace

PXL_EXPORT int pxl_msa_block_scores(const void* iq, const void* index_cache, const int* block_tables, const int* cu_q,
                                    const int* positions, float* scores, int64_t ld, int T, int B, int Hi, int Di,
                                    int max_blocks, int page, int sparse_block, int max_ctx, float scale,
                                    cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (Hi <= 0 || Hi > kMaxIdxHeads || Di % 8 || sparse_block % page || max_ctx <= 0) return PXL_ERR_INVALID_ARG;
  const int nb = pxl::ceil_div(max_ctx, sparse_block);
  if (nb > ld || nb > 2048) return PXL_ERR_INVALID_ARG;  // the selection bitmap covers 32 x 64 blocks
  dim3 grid(nb, T);
  msa_block_scores_kernel<<<grid, 128, Hi * Di * sizeof(float), stream>>>(
      static_cast<const pxl::bf16*>(iq), static_cast<const pxl::bf16*>(index_cache), block_tables, cu_q, positions, scores,
      ld, B, Hi, Di, max_blocks, page, sparse_block, scale);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_msa_select(const float* scores, int64_t ld, const int* positions, const int* block_tables,
                              const int* cu_q, int T, int B, int max_blocks, int page, int sparse_block, int topk,
                              int init_blocks, int local_blocks, int* v_tables, int64_t ld_vt, int* v_ctx,
                              cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (topk <= 0 || topk > kMaxTopk || local_blocks < 1 || sparse_block % page) return PXL_ERR_INVALID_ARG;
  if (ld_vt < static_cast<int64_t>(topk) * (sparse_block / page)) return PXL_ERR_INVALID_ARG;
  msa_select_kernel<<<T, 32, 0, stream>>>(scores, ld, positions, block_tables, cu_q, B, max_blocks, page, sparse_block,
                                          topk, init_blocks, local_blocks, v_tables, ld_vt, v_ctx);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}
