// Multi-head latent attention (DeepSeek-V3 / V3.2, Kimi-K2, GLM-DSA) on the compressed cache.
//
// The cache holds one row per token: [kv_lora_rank latent | rope_dim positional key], bf16,
// paged as [blocks, 1, page, 576]. Attention runs in "absorbed" form for decode AND prefill:
// the query is projected into latent space first (q_lat = q_nope * W_UK), scores are
// q_lat . latent + q_pe . k_pe, and the output is the probability-weighted sum of latents
// (projected back by W_UV afterwards). One kernel therefore serves
//   * dense decode            (reference Metal kernel mla_paged_attention.metal:8-104),
//   * dense causal prefill    (reference expands K/V instead: models/deepseek_v3.py:74-83),
//   * sparse decode / prefill over top-k positions chosen by the lightning indexer
//     (reference dsa_paged_attention.metal:34-240 and the dense-mask prefill of
//     models/deepseek_v32.py:432-446).
//
// Work decomposition: one CTA per (query token, block of 64 heads), 8 warps. Key/value rows are
// streamed in tiles of 32 tokens through a cp.async double buffer and shared by all 64 heads.
// QK^T: warp (mt, nh) computes the 16-head x 16-token block; softmax runs on the 64x32 score
// tile in shared memory; PV: warp w owns output columns [64w, 64w+64) of the 512-wide latent
// for all 64 heads, so the fp32 accumulator is 128 registers per thread.
#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

constexpr int kL = 512;            // latent width
constexpr int kR = 64;             // rope width
constexpr int kRow = kL + kR;      // cache row, elements
constexpr int kRowPad = kRow + 8;  // shared-memory row pitch (elements): 1168 B, breaks bank alignment
constexpr int kHB = 64;            // heads per CTA
constexpr int kTile = 32;          // key tokens per tile
constexpr int kPPitch = 40;        // P row pitch (bf16 elements)
constexpr int kSPitch = 33;        // S row pitch (floats)
constexpr int kMlaThreads = 256;

struct MlaSmem {
  bf16 q[kHB * kRowPad];
  bf16 kv[2][kTile * kRowPad];
  float s[kHB * kSPitch];
  bf16 p[2][kHB * kPPitch];
  float m[kHB], l[kHB], alpha[2][kHB];
};

struct MlaArgs {
  const bf16* q_lat;        // [H, Tpad, 512] head-major
  const bf16* q_pe;         // [T, H, 64]
  const bf16* cache;        // [blocks, page, 576]
  const int* block_tables;  // [B, max_blocks]
  const int* cu_q;          // [B+1] or null (token i belongs to sequence i)
  const int* positions;     // [T] absolute position of each query token
  const int* topk;          // [T, topk_stride] key positions (-1 = none) or null
  bf16* out;                // [H, Tpad, 512] head-major
  int tok_begin, Tpad, H, B, max_blocks, page, topk_k, topk_stride;
  float scale_log2;
};

__device__ __forceinline__ int find_seq(const int* cu_q, int B, int t) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(kMlaThreads, 1) mla_attn_kernel(const MlaArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  MlaSmem& sm = *reinterpret_cast<MlaSmem*>(smem_raw);
  const int t = a.tok_begin + blockIdx.x;  // token index in the batch-wide activation matrices
  const int h0 = blockIdx.y * kHB;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq = a.cu_q ? find_seq(a.cu_q, a.B, t) : static_cast<int>(blockIdx.x);
  const int pos = a.positions[t];
  const int* bt = a.block_tables + static_cast<size_t>(seq) * a.max_blocks;
  const int* tk = a.topk ? a.topk + static_cast<size_t>(t) * a.topk_stride : nullptr;
  const bool sparse = tk != nullptr && tk[0] >= 0;
  const int n_keys = sparse ? a.topk_k : pos + 1;
  const int n_tiles = ceil_div(n_keys, kTile);

  auto key_pos = [&](int j) -> int {
    if (j >= n_keys) return -1;
    const int kp = sparse ? tk[j] : j;
    return (kp >= 0 && kp <= pos) ? kp : -1;
  };
  auto load_tile = [&](int ti, int buf) {
    constexpr int CH = kRow / 8;  // 16-byte chunks per row
    for (int c = tid; c < kTile * CH; c += kMlaThreads) {
      const int r = c / CH, ch = c % CH;
      const int kp = key_pos(ti * kTile + r);
      const bf16* src = a.cache;
      if (kp >= 0) {
        const int blk = bt[kp / a.page];
        src = a.cache + (static_cast<size_t>(blk) * a.page + kp % a.page) * kRow + ch * 8;
      }
      cp_async_16(smem_u32(&sm.kv[buf][r * kRowPad + ch * 8]), src, kp >= 0);
    }
  };

  // ---- prologue: Q tile (latent part head-major, rope part token-major) and the first KV tile
  for (int c = tid; c < kHB * (kRow / 8); c += kMlaThreads) {
    const int r = c / (kRow / 8), ch = c % (kRow / 8);
    const int h = h0 + r;
    const bf16* src = a.q_lat;
    if (h < a.H) {
      src = ch < kL / 8 ? a.q_lat + (static_cast<size_t>(h) * a.Tpad + t) * kL + ch * 8
                        : a.q_pe + (static_cast<size_t>(t) * a.H + h) * kR + (ch - kL / 8) * 8;
    }
    cp_async_16(smem_u32(&sm.q[r * kRowPad + ch * 8]), src, h < a.H);
  }
  if (tid < kHB) {
    sm.m[tid] = -INFINITY;
    sm.l[tid] = 0.f;
  }
  if (n_tiles > 0) load_tile(0, 0);
  cp_async_commit();

  float o[4][8][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) o[i][j][k] = 0.f;

  const int mt = warp & 3, nh = warp >> 2;
  const int g = lane >> 2, qd = lane & 3;
  const int mi = lane >> 3;

  for (int ti = 0; ti < n_tiles; ++ti) {
    const int buf = ti & 1;
    cp_async_wait<0>();
    __syncthreads();  // tile ti landed; every warp is done with tile ti-1
    if (ti + 1 < n_tiles) load_tile(ti + 1, buf ^ 1);
    cp_async_commit();

    // ---- S block (16 heads x 16 tokens) = Q . K^T over the 576-wide rows
    {
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t q_base = smem_u32(&sm.q[(mt * 16 + (lane & 15)) * kRowPad + (lane >> 4) * 8]);
      const uint32_t k_base =
          smem_u32(&sm.kv[buf][(nh * 16 + (mi >> 1) * 8 + (lane & 7)) * kRowPad + (mi & 1) * 8]);
#pragma unroll 4
      for (int ks = 0; ks < kRow / 16; ++ks) {
        uint32_t qa[4], kb[4];
        ldmatrix_x4(qa, q_base + ks * 32);
        ldmatrix_x4(kb, k_base + ks * 32);
        const uint32_t b0[2] = {kb[0], kb[1]};
        const uint32_t b1[2] = {kb[2], kb[3]};
        mma_m16n8k16_bf16(s0, qa, b0);
        mma_m16n8k16_bf16(s1, qa, b1);
      }
      float* srow0 = &sm.s[(mt * 16 + g) * kSPitch + nh * 16 + qd * 2];
      float* srow1 = srow0 + 8 * kSPitch;
      srow0[0] = s0[0]; srow0[1] = s0[1]; srow1[0] = s0[2]; srow1[1] = s0[3];
      srow0[8] = s1[0]; srow0[9] = s1[1]; srow1[8] = s1[2]; srow1[9] = s1[3];
    }
    __syncthreads();

    // ---- online softmax on the 64 x 32 tile: 4 threads per row, 8 columns each
    {
      const int row = tid >> 2, c0 = (tid & 3) * 8;
      float v[8];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool valid = key_pos(ti * kTile + c0 + j) >= 0;
        v[j] = valid ? sm.s[row * kSPitch + c0 + j] * a.scale_log2 : -INFINITY;
        mx = fmaxf(mx, v[j]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_old = sm.m[row];
      const float m_new = fmaxf(m_old, mx);
      const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_old - m_new);
      float sum = 0.f;
      bf16x8 pk;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p0 = (m_new == -INFINITY) ? 0.f : exp2f(v[2 * j] - m_new);
        const float p1 = (m_new == -INFINITY) ? 0.f : exp2f(v[2 * j + 1] - m_new);
        sum += p0 + p1;
        pk.u[j] = pack_bf16x2(p0, p1);
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      *reinterpret_cast<uint4*>(&sm.p[buf][row * kPPitch + c0]) = *reinterpret_cast<uint4*>(&pk);
      __syncwarp();
      if ((tid & 3) == 0) {
        sm.m[row] = m_new;
        sm.l[row] = sm.l[row] * alpha + sum;
        sm.alpha[buf][row] = alpha;
      }
    }
    __syncthreads();

    // ---- O[:, 64w .. 64w+64) = alpha * O + P . V   (V = latent part of the tile)
    {
#pragma unroll
      for (int m4 = 0; m4 < 4; ++m4) {
        const float a0 = sm.alpha[buf][m4 * 16 + g], a1 = sm.alpha[buf][m4 * 16 + g + 8];
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          o[m4][n][0] *= a0; o[m4][n][1] *= a0;
          o[m4][n][2] *= a1; o[m4][n][3] *= a1;
        }
      }
#pragma unroll
      for (int ks = 0; ks < kTile / 16; ++ks) {
        uint32_t pa[4][4];
#pragma unroll
        for (int m4 = 0; m4 < 4; ++m4)
          ldmatrix_x4(pa[m4], smem_u32(&sm.p[buf][(m4 * 16 + (lane & 15)) * kPPitch + ks * 16 + (lane >> 4) * 8]));
        const uint32_t v_base =
            smem_u32(&sm.kv[buf][(ks * 16 + (mi & 1) * 8 + (lane & 7)) * kRowPad + warp * 64 + (mi >> 1) * 8]);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, v_base + np * 32);
          const uint32_t b0[2] = {vb[0], vb[1]};
          const uint32_t b1[2] = {vb[2], vb[3]};
#pragma unroll
          for (int m4 = 0; m4 < 4; ++m4) {
            mma_m16n8k16_bf16(o[m4][2 * np], pa[m4], b0);
            mma_m16n8k16_bf16(o[m4][2 * np + 1], pa[m4], b1);
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- normalise and store (head-major)
#pragma unroll
  for (int m4 = 0; m4 < 4; ++m4) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = m4 * 16 + g + half * 8;
      const int h = h0 + r;
      if (h >= a.H) continue;
      const float l = sm.l[r];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = a.out + (static_cast<size_t>(h) * a.Tpad + t) * kL + warp * 64 + qd * 2;
#pragma unroll
      for (int n = 0; n < 8; ++n)
        *reinterpret_cast<uint32_t*>(dst + n * 8) =
            pack_bf16x2(o[m4][n][half * 2] * inv, o[m4][n][half * 2 + 1] * inv);
    }
  }
}

// ---- cache write: RMSNorm over the latent, interleaved RoPE on the positional key ----------
__global__ void __launch_bounds__(128) mla_kv_prep_kernel(const bf16* __restrict__ ckv, int64_t ld,
                                                          const bf16* __restrict__ norm_w,
                                                          const float* __restrict__ cos_sin,
                                                          const int* __restrict__ positions,
                                                          const int64_t* __restrict__ slots,
                                                          bf16* __restrict__ cache, int64_t num_slots,
                                                          float eps, int* status) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int64_t slot = slots[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, PXL_DEV_BAD_INDEX);
    return;
  }
  const bf16* src = ckv + t * ld;
  bf16* dst = cache + slot * kRow;
  // 128 threads x 4 elements cover the 512-wide latent
  float x[4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    x[j] = __bfloat162float(src[threadIdx.x * 4 + j]);
    ss += x[j] * x[j];
  }
  ss = block_reduce_sum(ss, red);
  const float inv = rsqrtf(ss / kL + eps);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    dst[threadIdx.x * 4 + j] = __float2bfloat16(x[j] * inv * __bfloat162float(norm_w[threadIdx.x * 4 + j]));
  if (threadIdx.x < kR / 2) {
    const int i = threadIdx.x;
    const float* cs = cos_sin + static_cast<size_t>(positions[t]) * kR;
    const float c = cs[i], s = cs[kR / 2 + i];
    const float x0 = __bfloat162float(src[kL + 2 * i]), x1 = __bfloat162float(src[kL + 2 * i + 1]);
    dst[kL + 2 * i] = __float2bfloat16(x0 * c - x1 * s);
    dst[kL + 2 * i + 1] = __float2bfloat16(x0 * s + x1 * c);
  }
}

// ---- query split: no-position part head-major for the absorb GEMM, rope part rotated ---------
__global__ void __launch_bounds__(128) mla_q_prep_kernel(const bf16* __restrict__ q, int64_t ld,
                                                         const float* __restrict__ cos_sin,
                                                         const int* __restrict__ positions,
                                                         bf16* __restrict__ q_nope_hm,
                                                         bf16* __restrict__ q_pe, int T, int Tpad, int H,
                                                         int nope) {
  const int t = blockIdx.x;
  const bf16* src = q + t * ld;
  const float* cs = cos_sin + static_cast<size_t>(positions[t]) * kR;
  const int qd = nope + kR;
  for (int i = threadIdx.x; i < H * nope / 2; i += blockDim.x) {
    const int h = (2 * i) / nope, d = (2 * i) % nope;
    *reinterpret_cast<uint32_t*>(q_nope_hm + (static_cast<size_t>(h) * Tpad + t) * nope + d) =
        *reinterpret_cast<const uint32_t*>(src + h * qd + d);
  }
  for (int i = threadIdx.x; i < H * kR / 2; i += blockDim.x) {
    const int h = i / (kR / 2), j = i % (kR / 2);
    const float c = cs[j], s = cs[kR / 2 + j];
    const float x0 = __bfloat162float(src[h * qd + nope + 2 * j]);
    const float x1 = __bfloat162float(src[h * qd + nope + 2 * j + 1]);
    *reinterpret_cast<uint32_t*>(q_pe + (static_cast<size_t>(t) * H + h) * kR + 2 * j) =
        pack_bf16x2(x0 * c - x1 * s, x0 * s + x1 * c);
  }
}

}  // namespace

PXL_EXPORT int pxl_mla_attn(const void* q_lat, const void* q_pe, const void* cache, const int* block_tables,
                            const int* cu_q, const int* positions, const int* topk, void* out,
                            int tok_begin, int n_tok, int Tpad, int H, int B, int max_blocks, int page,
                            int latent, int rope, int topk_k, int topk_stride, float scale,
                            cudaStream_t stream) {
  if (n_tok <= 0) return PXL_OK;
  if (latent != kL || rope != kR || H <= 0 || tok_begin < 0 || Tpad < tok_begin + n_tok || page <= 0)
    return PXL_ERR_INVALID_ARG;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(mla_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(sizeof(MlaSmem))) != cudaSuccess)
      return PXL_ERR_CUDA;
    configured[dev] = true;
  }
  MlaArgs a;
  a.q_lat = static_cast<const pxl::bf16*>(q_lat);
  a.q_pe = static_cast<const pxl::bf16*>(q_pe);
  a.cache = static_cast<const pxl::bf16*>(cache);
  a.block_tables = block_tables;
  a.cu_q = cu_q;
  a.positions = positions;
  a.topk = topk;
  a.out = static_cast<pxl::bf16*>(out);
  a.tok_begin = tok_begin; a.Tpad = Tpad; a.H = H; a.B = B; a.max_blocks = max_blocks; a.page = page;
  a.topk_k = topk_k; a.topk_stride = topk_stride;
  a.scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(n_tok, pxl::ceil_div(H, kHB));
  mla_attn_kernel<<<grid, kMlaThreads, sizeof(MlaSmem), stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_mla_kv_prep(const void* ckv, int64_t ld, const void* norm_w, const float* cos_sin,
                               const int* positions, const int64_t* slots, void* cache, int T, int latent,
                               int rope, int64_t num_slots, float eps, int* status, cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (latent != kL || rope != kR) return PXL_ERR_INVALID_ARG;
  mla_kv_prep_kernel<<<T, 128, 0, stream>>>(static_cast<const pxl::bf16*>(ckv), ld,
                                            static_cast<const pxl::bf16*>(norm_w), cos_sin, positions, slots,
                                            static_cast<pxl::bf16*>(cache), num_slots, eps, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_mla_q_prep(const void* q, int64_t ld, const float* cos_sin, const int* positions,
                              void* q_nope_hm, void* q_pe, int T, int Tpad, int H, int nope, int rope,
                              cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (rope != kR || (nope % 2)) return PXL_ERR_INVALID_ARG;
  mla_q_prep_kernel<<<T, 128, 0, stream>>>(static_cast<const pxl::bf16*>(q), ld, cos_sin, positions,
                                           static_cast<pxl::bf16*>(q_nope_hm), static_cast<pxl::bf16*>(q_pe), T,
                                           Tpad, H, nope);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}
