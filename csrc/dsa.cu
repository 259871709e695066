// DeepSeek sparse attention (V3.2 "lightning indexer"): key scoring, top-k selection, key store.
//
//   score[t, j] = sum_h relu(q_idx[t, h, :] . k_idx[j, :]) * w[t, h]      for j <= position(t)
//
// The reference scores one context token per threadgroup (dsa_indexer.metal:34-116, launch in
// dsa_indexer.cpp:153-196) and selects the top-k with a framework argpartition
// (parallax_extensions/ops.py:361-367). Here one CTA scores a tile of 64 keys for all index
// heads with tensor-core MMAs, and a radix select picks the k best positions per query row
// without sorting.
#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

constexpr int kDi = 128;          // index head dim
constexpr int kHiMax = 64;        // index heads handled per CTA (one pass)
constexpr int kKeyTile = 64;
constexpr int kPitch = kDi + 8;   // smem row pitch (elements)

__device__ __forceinline__ int find_seq(const int* cu_q, int B, int t) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// grid (key tiles, T), 128 threads: warp w owns index heads [16w, 16w+16)
__global__ void __launch_bounds__(128) dsa_scores_kernel(const bf16* __restrict__ q, const float* __restrict__ w,
                                                         const bf16* __restrict__ cache,
                                                         const int* __restrict__ block_tables,
                                                         const int* __restrict__ cu_q,
                                                         const int* __restrict__ positions,
                                                         float* __restrict__ scores, int64_t ld_scores, int B,
                                                         int Hi, int max_blocks, int page) {
  __shared__ __align__(16) bf16 q_s[kHiMax * kPitch];
  __shared__ __align__(16) bf16 k_s[kKeyTile * kPitch];
  __shared__ float acc[kKeyTile];
  const int t = blockIdx.y;
  const int j0 = blockIdx.x * kKeyTile;
  const int pos = positions[t];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* out = scores + static_cast<size_t>(t) * ld_scores;
  if (j0 > pos) {  // whole tile beyond the causal limit
    if (tid < kKeyTile) out[j0 + tid] = -INFINITY;
    return;
  }
  const int seq = cu_q ? find_seq(cu_q, B, t) : t;
  const int* bt = block_tables + static_cast<size_t>(seq) * max_blocks;
  for (int c = tid; c < kHiMax * (kDi / 8); c += 128) {
    const int r = c / (kDi / 8), ch = c % (kDi / 8);
    cp_async_16(smem_u32(&q_s[r * kPitch + ch * 8]), q + (static_cast<size_t>(t) * Hi + (r < Hi ? r : 0)) * kDi + ch * 8,
                r < Hi);
  }
  for (int c = tid; c < kKeyTile * (kDi / 8); c += 128) {
    const int r = c / (kDi / 8), ch = c % (kDi / 8);
    const int kp = j0 + r;
    const bf16* src = cache;
    if (kp <= pos) src = cache + (static_cast<size_t>(bt[kp / page]) * page + kp % page) * kDi + ch * 8;
    cp_async_16(smem_u32(&k_s[r * kPitch + ch * 8]), src, kp <= pos);
  }
  cp_async_commit();
  if (tid < kKeyTile) acc[tid] = 0.f;
  cp_async_wait<0>();
  __syncthreads();

  const int g = lane >> 2, qd = lane & 3, mi = lane >> 3;
  float s[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n)
#pragma unroll
    for (int k = 0; k < 4; ++k) s[n][k] = 0.f;
  const uint32_t q_base = smem_u32(&q_s[(warp * 16 + (lane & 15)) * kPitch + (lane >> 4) * 8]);
#pragma unroll
  for (int ks = 0; ks < kDi / 16; ++ks) {
    uint32_t qa[4];
    ldmatrix_x4(qa, q_base + ks * 32);
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t kb[4];
      ldmatrix_x4(kb, smem_u32(&k_s[(np * 16 + (mi >> 1) * 8 + (lane & 7)) * kPitch + ks * 16 + (mi & 1) * 8]));
      const uint32_t b0[2] = {kb[0], kb[1]};
      const uint32_t b1[2] = {kb[2], kb[3]};
      mma_m16n8k16_bf16(s[2 * np], qa, b0);
      mma_m16n8k16_bf16(s[2 * np + 1], qa, b1);
    }
  }
  const int h_lo = warp * 16 + g, h_hi = h_lo + 8;
  const float w_lo = h_lo < Hi ? w[static_cast<size_t>(t) * Hi + h_lo] : 0.f;
  const float w_hi = h_hi < Hi ? w[static_cast<size_t>(t) * Hi + h_hi] : 0.f;
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    float c0 = fmaxf(s[n][0], 0.f) * w_lo + fmaxf(s[n][2], 0.f) * w_hi;
    float c1 = fmaxf(s[n][1], 0.f) * w_lo + fmaxf(s[n][3], 0.f) * w_hi;
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {  // sum over the 8 row groups of the warp
      c0 += __shfl_xor_sync(0xffffffffu, c0, off);
      c1 += __shfl_xor_sync(0xffffffffu, c1, off);
    }
    if (g == 0) {
      atomicAdd(&acc[n * 8 + qd * 2], c0);
      atomicAdd(&acc[n * 8 + qd * 2 + 1], c1);
    }
  }
  __syncthreads();
  if (tid < kKeyTile) out[j0 + tid] = (j0 + tid <= pos) ? acc[tid] : -INFINITY;
}

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// one CTA per query row: radix select of the k largest scores among positions [0, pos]
__global__ void __launch_bounds__(512) topk_select_kernel(const float* __restrict__ scores, int64_t ld,
                                                          const int* __restrict__ positions, int k,
                                                          int* __restrict__ out, int64_t ld_out) {
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix, s_mask;
  __shared__ int s_remaining, s_gt, s_eq;
  const int t = blockIdx.x;
  const int n = positions[t] + 1;
  const float* s = scores + static_cast<size_t>(t) * ld;
  int* o = out + static_cast<size_t>(t) * ld_out;
  if (n <= k) {  // nothing to select: the attention kernel reads "row starts with -1" as dense
    for (int i = threadIdx.x; i < k; i += blockDim.x) o[i] = -1;
    return;
  }
  if (threadIdx.x == 0) {
    s_prefix = 0;
    s_mask = 0;
    s_remaining = k;
    s_gt = 0;
    s_eq = 0;
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = s_mask;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t u = order_key(s[i]);
      if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int remaining = s_remaining, cum = 0, b = 255;
      for (; b > 0; --b) {
        if (cum + hist[b] >= remaining) break;
        cum += hist[b];
      }
      s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      s_mask = mask | (0xffu << shift);
      s_remaining = remaining - cum;
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;
  const int take_eq = s_remaining;  // how many keys equal to the threshold still fit
  const int n_gt = k - take_eq;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const uint32_t u = order_key(s[i]);
    if (u > thr) {
      const int idx = atomicAdd(&s_gt, 1);
      if (idx < n_gt) o[idx] = i;
    } else if (u == thr) {
      const int j = atomicAdd(&s_eq, 1);
      if (j < take_eq) o[n_gt + j] = i;
    }
  }
}

__global__ void store_rows_kernel(const bf16* __restrict__ src, int64_t ld, const int64_t* __restrict__ slots,
                                  bf16* __restrict__ cache, int D, int64_t num_slots, int* status) {
  const int t = blockIdx.x;
  const int64_t slot = slots[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, PXL_DEV_BAD_INDEX);
    return;
  }
  for (int i = threadIdx.x; i < D / 8; i += blockDim.x)
    st_bf16x8(cache + slot * D + i * 8, ld_bf16x8(src + t * ld + i * 8));
}

// Indexer pre-processing of one step, one block (128 threads) per token:
//   q_idx[t, h, :R]  <- interleaved RoPE at position(t), in place (every index head)
//   cache[slot(t)]   <- RoPE(LayerNorm(kv[t, k_off : k_off + Di]) * w + b) on the first R dims
//   w_out[t, h]      <- kv[t, w_off + h] * w_scale                              (fp32)
// The model code did this with five framework calls per layer (layer norm, two rotations, two concatenations)
// and a separate store; semantics follow the reference's indexer (deepseek_v32.py:84-238).
__global__ void __launch_bounds__(128)
dsa_index_prep_kernel(bf16* __restrict__ q_idx, int64_t ldq, const bf16* __restrict__ kv, int64_t ldkv, int k_off,
                      int w_off, const bf16* __restrict__ ln_w, const bf16* __restrict__ ln_b, float ln_eps,
                      const float* __restrict__ cos_sin, const int* __restrict__ positions, int max_pos,
                      const int64_t* __restrict__ slots, bf16* __restrict__ cache, int64_t num_slots,
                      float* __restrict__ w_out, float w_scale, int Hi, int R, int* status) {
  __shared__ float red[32];
  __shared__ float y_s[kDi];
  const int t = blockIdx.x, d = threadIdx.x;
  const int pos = positions[t];
  const bool pos_ok = pos >= 0 && (max_pos <= 0 || pos < max_pos);
  if (!pos_ok && d == 0 && status) atomicCAS(status, 0, PXL_DEV_BAD_POSITION);
  const float* cs = cos_sin + static_cast<size_t>(pos_ok ? pos : 0) * R;
  const int half = R >> 1;
  // ---- head weights
  if (d < Hi) w_out[static_cast<size_t>(t) * Hi + d] = __bfloat162float(kv[t * ldkv + w_off + d]) * w_scale;
  // ---- queries: one thread per (head, pair)
  if (pos_ok) {
    for (int idx = d; idx < Hi * half; idx += blockDim.x) {
      const int h = idx / half, i = idx % half;
      bf16* p = q_idx + t * ldq + static_cast<int64_t>(h) * kDi + 2 * i;
      const float x0 = __bfloat162float(p[0]), x1 = __bfloat162float(p[1]);
      const float c = cs[i], sn = cs[half + i];
      p[0] = __float2bfloat16(x0 * c - x1 * sn);
      p[1] = __float2bfloat16(x0 * sn + x1 * c);
    }
  }
  // ---- key: layer norm over the Di dims (two passes in fp32), rotation, store
  const float x = __bfloat162float(kv[t * ldkv + k_off + d]);
  const float mean = block_reduce_sum(x, red) * (1.f / kDi);
  const float dx = x - mean;
  const float var = block_reduce_sum(dx * dx, red) * (1.f / kDi);
  const float y = dx * rsqrtf(var + ln_eps) * __bfloat162float(ln_w[d]) + (ln_b ? __bfloat162float(ln_b[d]) : 0.f);
  y_s[d] = y;
  __syncthreads();
  float out = y;
  if (pos_ok && d < R) {
    const int i = d >> 1;
    const float c = cs[i], sn = cs[half + i];
    out = (d & 1) ? y_s[d - 1] * sn + y * c : y * c - y_s[d + 1] * sn;
  }
  const int64_t slot = slots[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (d == 0 && status) atomicCAS(status, 0, PXL_DEV_BAD_INDEX);
    return;
  }
  cache[slot * kDi + d] = __float2bfloat16(out);
}

}  // namespace

PXL_EXPORT int pxl_dsa_index_prep(void* q_idx, int64_t ldq, const void* kv, int64_t ldkv, int k_off, int w_off,
                                  const void* ln_w, const void* ln_b, float ln_eps, const float* cos_sin,
                                  const int* positions, int max_pos, const int64_t* slots, void* cache,
                                  int64_t num_slots, float* w_out, float w_scale, int T, int Hi, int Di, int R,
                                  int* status, cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (Di != kDi || Hi <= 0 || Hi > 128 || R <= 0 || R > Di || (R & 1)) return PXL_ERR_INVALID_ARG;
  dsa_index_prep_kernel<<<T, 128, 0, stream>>>(static_cast<pxl::bf16*>(q_idx), ldq, static_cast<const pxl::bf16*>(kv),
                                               ldkv, k_off, w_off, static_cast<const pxl::bf16*>(ln_w),
                                               static_cast<const pxl::bf16*>(ln_b), ln_eps, cos_sin, positions,
                                               max_pos, slots, static_cast<pxl::bf16*>(cache), num_slots, w_out,
                                               w_scale, Hi, R, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_dsa_index_scores(const void* q, const float* w, const void* index_cache,
                                    const int* block_tables, const int* cu_q, const int* positions,
                                    float* scores, int64_t ld_scores, int T, int B, int Hi, int Di,
                                    int max_blocks, int page, int max_ctx, cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (Di != kDi || Hi <= 0 || Hi > kHiMax || max_ctx <= 0) return PXL_ERR_INVALID_ARG;
  const int tiles = pxl::ceil_div(max_ctx, kKeyTile);
  if (static_cast<int64_t>(tiles) * kKeyTile > ld_scores) return PXL_ERR_INVALID_ARG;
  dim3 grid(tiles, T);
  dsa_scores_kernel<<<grid, 128, 0, stream>>>(static_cast<const pxl::bf16*>(q), w,
                                              static_cast<const pxl::bf16*>(index_cache), block_tables, cu_q,
                                              positions, scores, ld_scores, B, Hi, max_blocks, page);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_topk_select(const float* scores, int64_t ld, const int* positions, int T, int k, int* out,
                               int64_t ld_out, cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (k <= 0 || ld_out < k) return PXL_ERR_INVALID_ARG;
  topk_select_kernel<<<T, 512, 0, stream>>>(scores, ld, positions, k, out, ld_out);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_store_rows(const void* src, int64_t ld, const int64_t* slots, void* cache, int T, int D,
                              int64_t num_slots, int* status, cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (D % 8 || ld % 8) return PXL_ERR_INVALID_ARG;
  store_rows_kernel<<<T, 64, 0, stream>>>(static_cast<const pxl::bf16*>(src), ld, slots,
                                          static_cast<pxl::bf16*>(cache), D, num_slots, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}
