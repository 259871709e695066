// Paged GQA attention for decode (single query, split-KV) and ragged causal prefill
// with a cached KV prefix. Cache layout: K, V = [num_blocks, Hkv, page_size, D] bf16.
//
// Both kernels stream 64-token K/V tiles of one KV head into swizzled shared memory
// with cp.async (double buffered; the per-token block-table lookup makes any page size
// work) and run QK^T / PV on the warp-level tensor path with fp32 online softmax.
// All q heads of a KV-head group share the tile: in decode they are the rows of one
// 16-row MMA tile and the four warps split the tile's tokens; in prefill the CTA's 64
// rows are (token, group-head) pairs.
//
// Behavioural counterparts in the reference: the single-query kernel with sliding
// window and attention sinks and its split-KV variant
// (src/parallax_extensions/kernels/paged_attention/paged_attention.metal:794-1347),
// and the prefix-aware prefill (src/parallax/utils/prefix_cache_utils.py:11-144).
#include <cuda_fp8.h>

#include <atomic>

#include "common.cuh"
#include "pxl_api.h"
#include "pxl_noalloc.h"

namespace {
using namespace pxl;

constexpr int TILE = 64;  // KV tokens per shared-memory tile
constexpr float kLog2e = 1.4426950408889634f;

struct KVTileArgs {
  const void* k_cache;   // bf16 elements, or e4m3 bytes for the FP8 kernels
  const void* v_cache;
  const int* block_table;  // row of this sequence
  int max_blocks;
  int64_t num_blocks;
  int Hkv;
  int kvh;
  int page_size;
};

// byte offset of 16-byte chunk `chunk` of row `row` inside a [TILE][D] bf16 tile
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return static_cast<uint32_t>(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}
// Same for a tile that TMA wrote with the 128-byte swizzle: two halves of [TILE][64] elements
// (128-byte rows); inside a half the 16-byte chunk c of row r sits at position c ^ (r % 8).
__device__ __forceinline__ uint32_t tile_off_sw128(int row, int chunk) {
  return static_cast<uint32_t>((chunk >> 3) * (64 * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// Eight e4m3 bytes -> eight bf16 (exact: every e4m3 value is a bf16 value), as one 16-byte vector.
__device__ __forceinline__ uint4 e4m3x8_to_bf16x8(uint2 raw) {
  uint4 out;
  uint32_t* o = &out.x;
  const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_fp8x2_storage_t pair = static_cast<__nv_fp8x2_storage_t>((w[i >> 1] >> ((i & 1) * 16)) & 0xffffu);
    const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
    o[i] = pack_bf16x2(f.x, f.y);
  }
  return out;
}

// Issue the loads of K and V rows for tokens [tok0, tok0+TILE) ∩ [0, hi): cp.async for a bf16 cache;
// for an e4m3 cache (FP8) each thread reads 8 bytes, widens them to bf16 and stores the 16-byte
// chunk itself, so that the MMA code behind it is the same. The scales of an e4m3 cache are applied
// by the caller (K: folded into the score scale, V: into the output normalisation).
template <int D, bool FP8 = false>
__device__ __forceinline__ void load_kv_tile(const KVTileArgs& a, int tok0, int hi, uint32_t k_smem,
                                             uint32_t v_smem, int* status) {
  constexpr int CPR = D / 8;  // 8-element chunks per row
  constexpr int ITERS = TILE * CPR / 128;
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const int c = i * 128 + threadIdx.x;
    const int row = c / CPR;
    const int chunk = c % CPR;
    const int tok = tok0 + row;
    bool pred = tok < hi;
    int64_t base = 0;
    if (pred) {
      const int bi = tok / a.page_size;
      const int blk = (bi < a.max_blocks) ? a.block_table[bi] : -1;
      if (blk < 0 || blk >= a.num_blocks) {
        pred = false;
        if (status) atomicCAS(status, 0, PXL_DEV_BAD_BLOCK_PREFILL);
      } else {
        base = ((static_cast<int64_t>(blk) * a.Hkv + a.kvh) * a.page_size + (tok % a.page_size)) *
                   D +
               chunk * 8;
      }
    }
    const uint32_t off = tile_off<D>(row, chunk);
    if constexpr (FP8) {
      uint2 kr = make_uint2(0u, 0u), vr = make_uint2(0u, 0u);
      if (pred) {
        kr = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(a.k_cache) + base));
        vr = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(a.v_cache) + base));
      }
      const uint4 kb = e4m3x8_to_bf16x8(kr), vb = e4m3x8_to_bf16x8(vr);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(k_smem + off), "r"(kb.x), "r"(kb.y),
                   "r"(kb.z), "r"(kb.w) : "memory");
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(v_smem + off), "r"(vb.x), "r"(vb.y),
                   "r"(vb.z), "r"(vb.w) : "memory");
    } else {
      cp_async_16(k_smem + off, static_cast<const bf16*>(a.k_cache) + base, pred);
      cp_async_16(v_smem + off, static_cast<const bf16*>(a.v_cache) + base, pred);
    }
  }
}

// S[16 x 16] += Q[16 x D] * K[tokens r0..r0+15]^T ; s[j] is the n-tile of tokens r0+8j..
template <int D, bool SW128 = false>
__device__ __forceinline__ void qk_16x16(const uint32_t (&qf)[D / 16][4], uint32_t k_smem, int r0,
                                         float (&s0)[4], float (&s1)[4]) {
  const int lane = threadIdx.x & 31;
  const int mi = lane >> 3;
  const int row = r0 + (mi >> 1) * 8 + (lane & 7);
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t r[4];
    ldmatrix_x4(r, k_smem + (SW128 ? tile_off_sw128(row, ks * 2 + (mi & 1)) : tile_off<D>(row, ks * 2 + (mi & 1))));
    const uint32_t b0[2] = {r[0], r[1]};
    const uint32_t b1[2] = {r[2], r[3]};
    mma_m16n8k16_bf16(s0, qf[ks], b0);
    mma_m16n8k16_bf16(s1, qf[ks], b1);
  }
}

// O[16 x D] += P[16 x 16] * V[tokens r0..r0+15]
template <int D, bool SW128 = false>
__device__ __forceinline__ void pv_16x16(const uint32_t (&pf)[4], uint32_t v_smem, int r0,
                                         float (&o)[D / 8][4]) {
  const int lane = threadIdx.x & 31;
  const int mi = lane >> 3;
  const int row = r0 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
  for (int np = 0; np < D / 16; ++np) {
    uint32_t r[4];
    ldmatrix_x4_trans(r, v_smem + (SW128 ? tile_off_sw128(row, np * 2 + (mi >> 1)) : tile_off<D>(row, np * 2 + (mi >> 1))));
    const uint32_t b0[2] = {r[0], r[1]};
    const uint32_t b1[2] = {r[2], r[3]};
    mma_m16n8k16_bf16(o[2 * np], pf, b0);
    mma_m16n8k16_bf16(o[2 * np + 1], pf, b1);
  }
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  return v;
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

// =============================================================================== decode
template <int D, bool FP8 = false>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const bf16* __restrict__ q, int64_t q_stride, const void* __restrict__ k_cache,
                   const void* __restrict__ v_cache, const int* __restrict__ block_tables,
                   const int* __restrict__ ctx_lens, bf16* __restrict__ out,
                   float* __restrict__ workspace, const float* __restrict__ sinks, int Hq, int Hkv,
                   int page_size, int max_blocks, int64_t num_blocks, float scale_log2, int window,
                   int num_splits, float v_scale, int* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int TILE_BYTES = TILE * D * 2;
  const uint32_t k_smem0 = smem_u32(smem);
  const uint32_t v_smem0 = k_smem0 + 2 * TILE_BYTES;

  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctx = ctx_lens[b];
  const int hi = ctx;
  const int lo = (window > 0 && ctx > window) ? ctx - window : 0;
  const int tile_lo = lo / TILE;
  const int tiles_total = hi > lo ? ceil_div(hi, TILE) - tile_lo : 0;
  const int per_split = ceil_div(tiles_total, num_splits);
  const int t_begin = tile_lo + split * per_split;
  const int t_end = min(tile_lo + tiles_total, t_begin + per_split);

  KVTileArgs ka{k_cache, v_cache, block_tables + static_cast<size_t>(b) * max_blocks, max_blocks,
                num_blocks, Hkv, kvh, page_size};

  // Q fragments: row r of the MMA tile is q head kvh*G + r (rows >= G are zero)
  uint32_t qf[D / 16][4];
  {
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    const bf16* q_lo = q + static_cast<size_t>(b) * q_stride + (kvh * G + r_lo) * D;
    const bf16* q_hi = q + static_cast<size_t>(b) * q_stride + (kvh * G + r_hi) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int c = ks * 16 + 2 * (lane & 3);
      qf[ks][0] = r_lo < G ? *reinterpret_cast<const uint32_t*>(q_lo + c) : 0u;
      qf[ks][1] = r_hi < G ? *reinterpret_cast<const uint32_t*>(q_hi + c) : 0u;
      qf[ks][2] = r_lo < G ? *reinterpret_cast<const uint32_t*>(q_lo + c + 8) : 0u;
      qf[ks][3] = r_hi < G ? *reinterpret_cast<const uint32_t*>(q_hi + c + 8) : 0u;
    }
  }

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  int buf = 0;
  if (t_begin < t_end) load_kv_tile<D, FP8>(ka, t_begin * TILE, hi, k_smem0, v_smem0, status);
  cp_async_commit();
  for (int t = t_begin; t < t_end; ++t) {
    cp_async_wait<0>();
    __syncthreads();
    if (t + 1 < t_end)
      load_kv_tile<D, FP8>(ka, (t + 1) * TILE, hi, k_smem0 + (buf ^ 1) * TILE_BYTES,
                      v_smem0 + (buf ^ 1) * TILE_BYTES, status);
    cp_async_commit();

    const int r0 = warp * 16;
    const int tok_base = t * TILE + r0;
    if (tok_base < hi && tok_base + 16 > lo) {  // warp-uniform
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      qk_16x16<D>(qf, k_smem0 + buf * TILE_BYTES, r0, s[0], s[1]);
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = tok_base + j * 8 + 2 * (lane & 3) + (e & 1);
          const bool valid = tok < hi && tok >= lo;
          s[j][e] = valid ? s[j][e] * scale_log2 : -INFINITY;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
        }
      }
      float corr[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = quad_max(mx[h]);
        const float m_new = fmaxf(m_run[h], mx[h]);
        m_use[h] = (m_new == -INFINITY) ? 0.f : m_new;
        corr[h] = exp2f(m_run[h] - m_use[h]);
        m_run[h] = m_new;
      }
      float ps[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[j][e] = exp2f(s[j][e] - m_use[e >> 1]);
          ps[e >> 1] += s[j][e];
        }
      l_run[0] = l_run[0] * corr[0] + ps[0];
      l_run[1] = l_run[1] * corr[1] + ps[1];
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
      uint32_t pf[4];
      pf[0] = pack_bf16x2(s[0][0], s[0][1]);
      pf[1] = pack_bf16x2(s[0][2], s[0][3]);
      pf[2] = pack_bf16x2(s[1][0], s[1][1]);
      pf[3] = pack_bf16x2(s[1][2], s[1][3]);
      pv_16x16<D>(pf, v_smem0 + buf * TILE_BYTES, r0, o);
    }
    buf ^= 1;
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the four warps' partial softmax states through shared memory
  float* o_sm = reinterpret_cast<float*>(smem);          // [4][16][D]
  float* m_sm = o_sm + 4 * 16 * D;                       // [4][16]
  float* l_sm = m_sm + 4 * 16;                           // [4][16]
  l_run[0] = quad_sum(l_run[0]);
  l_run[1] = quad_sum(l_run[1]);
  {
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    float* ow = o_sm + warp * 16 * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int c = i * 8 + 2 * (lane & 3);
      ow[r_lo * D + c] = o[i][0];
      ow[r_lo * D + c + 1] = o[i][1];
      ow[r_hi * D + c] = o[i][2];
      ow[r_hi * D + c + 1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      m_sm[warp * 16 + r_lo] = m_run[0];
      m_sm[warp * 16 + r_hi] = m_run[1];
      l_sm[warp * 16 + r_lo] = l_run[0];
      l_sm[warp * 16 + r_hi] = l_run[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += 128) {
    const int r = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, m_sm[w * 16 + r]);
    const int head = kvh * G + r;
    const float sink = (sinks && num_splits == 1) ? sinks[head] * kLog2e : -INFINITY;
    const float Mx = fmaxf(M, sink);
    const float Mu = (Mx == -INFINITY) ? 0.f : Mx;
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(m_sm[w * 16 + r] - Mu);
      L += l_sm[w * 16 + r] * f;
      acc += o_sm[(w * 16 + r) * D + d] * f;
    }
    if (num_splits == 1) {
      const float denom = L + exp2f(sink - Mu);
      out[(static_cast<size_t>(b) * Hq + head) * D + d] =
          __float2bfloat16(denom > 0.f ? acc / denom * v_scale : 0.f);
    } else {
      // partial: normalised output + log2-sum-exp
      float* po = workspace;
      float* plse = workspace + static_cast<size_t>(gridDim.y) * Hq * num_splits * D;
      const size_t row = (static_cast<size_t>(b) * Hq + head) * num_splits + split;
      po[row * D + d] = L > 0.f ? acc / L * v_scale : 0.f;
      if (d == 0) plse[row] = L > 0.f ? Mu + log2f(L) : -INFINITY;
    }
  }
}

// ---- decode, TMA-fed variant (D = 128; page_size 16, 32 or 64) ------------------------------------
// A (block, kv head) page of the cache is one contiguous [page, 128] matrix, so a KV tile of 64
// tokens is 64 / page box loads per operand half: one thread issues them through the TMA engine
// (128-byte swizzle, completion on an mbarrier) up to three tiles ahead of the four consumer warps.
// This removes the per-thread address arithmetic and the 2048 cp.async instructions per tile of the
// kernel above, which was issue-bound at half of the DRAM bandwidth. The issuing lane sits in a warp
// of its own (warp 4) and the stages are handed back through "empty" mbarriers (one arrival per
// consumer warp), so the consumer warps never meet at a CTA-wide barrier inside the loop: with the
// producer inside warp 0 and a __syncthreads per tile the top stall was that barrier.
constexpr int kDecStages = 3;
constexpr int kDecThreads = 160;  // 4 consumer warps + 1 producer warp

__global__ void __launch_bounds__(kDecThreads, 2)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const bf16* __restrict__ q, int64_t q_stride, const int* __restrict__ block_tables,
                       const int* __restrict__ ctx_lens, bf16* __restrict__ out, float* __restrict__ workspace,
                       const float* __restrict__ sinks, int Hq, int Hkv, int page_size, int max_blocks,
                       int64_t num_blocks, float scale_log2, int window, int num_splits, int* status) {
  constexpr int D = 128;
  constexpr int TILE_BYTES = TILE * D * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t stage0 = smem_u32(smem);  // stage s: K tile at s * 2 * TILE_BYTES, V tile behind it
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kDecStages * 2 * TILE_BYTES);  // full[S], empty[S]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kDecStages);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + kDecStages);
  pdl_wait();
  pdl_launch_dependents();

  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctx = ctx_lens[b];
  const int hi = ctx;
  const int lo = (window > 0 && ctx > window) ? ctx - window : 0;
  const int tile_lo = lo / TILE;
  const int tiles_total = hi > lo ? ceil_div(hi, TILE) - tile_lo : 0;
  const int per_split = ceil_div(tiles_total, num_splits);
  const int t_begin = tile_lo + split * per_split;
  const int t_end = min(tile_lo + tiles_total, t_begin + per_split);
  const int n_tiles = t_end > t_begin ? t_end - t_begin : 0;
  const int* bt = block_tables + static_cast<size_t>(b) * max_blocks;
  const int ppt = TILE / page_size;  // pages per tile

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kDecStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 4);  // one arrival per consumer warp
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  __syncthreads();

  int failed = 0;
  if (warp == 4) {
    // ---- producer warp, up to kDecStages tiles ahead of the consumers. Lane p looks up the block of
    // page p of the tile and issues that page's four box loads: the block-table reads of a tile are in
    // flight together and are issued before the wait for the stage.
    for (int it = 0; it < n_tiles; ++it) {
      const int stage = it % kDecStages;
      int blk = 0;
      if (lane < ppt) {
        int bi = (t_begin + it) * ppt + lane;
        if (bi * page_size >= hi) bi = (hi - 1) / page_size;  // beyond the context: re-read the last page (masked)
        blk = bi < max_blocks ? bt[bi] : -1;
        if (blk < 0 || blk >= num_blocks) {
          if (status) atomicCAS(status, 0, PXL_DEV_BAD_BLOCK_DECODE);
          blk = 0;
        }
      }
      int okf = 1;
      if (it >= kDecStages && lane == 0)
        okf = mbar_wait_bounded(empty0 + 8 * stage, ((it / kDecStages) - 1) & 1, abort_flag, status,
                                PXL_DEV_TIMEOUT_EMPTY) ? 1 : 0;
      okf = __shfl_sync(0xffffffffu, okf, 0);
      if (!okf) {
        failed = 1;
        break;
      }
      const uint32_t bar = full0 + 8 * stage;
      const uint32_t k_dst = stage0 + stage * 2 * TILE_BYTES, v_dst = k_dst + TILE_BYTES;
      if (lane == 0) mbar_arrive_expect_tx(bar, 2 * TILE_BYTES);
      __syncwarp();
      if (lane < ppt) {
        const int row0 = (blk * Hkv + kvh) * page_size;
        const uint32_t off = lane * page_size * 128;
        tma_load_2d(k_dst + off, &tm_k, bar, 0, row0);
        tma_load_2d(k_dst + TILE * 128 + off, &tm_k, bar, 64, row0);
        tma_load_2d(v_dst + off, &tm_v, bar, 0, row0);
        tma_load_2d(v_dst + TILE * 128 + off, &tm_v, bar, 64, row0);
      }
    }
  }

  uint32_t qf[D / 16][4];
  {
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    const bf16* q_lo = q + static_cast<size_t>(b) * q_stride + (kvh * G + r_lo) * D;
    const bf16* q_hi = q + static_cast<size_t>(b) * q_stride + (kvh * G + r_hi) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int c = ks * 16 + 2 * (lane & 3);
      qf[ks][0] = r_lo < G ? *reinterpret_cast<const uint32_t*>(q_lo + c) : 0u;
      qf[ks][1] = r_hi < G ? *reinterpret_cast<const uint32_t*>(q_hi + c) : 0u;
      qf[ks][2] = r_lo < G ? *reinterpret_cast<const uint32_t*>(q_lo + c + 8) : 0u;
      qf[ks][3] = r_hi < G ? *reinterpret_cast<const uint32_t*>(q_hi + c + 8) : 0u;
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  for (int it = 0; warp < 4 && it < n_tiles; ++it) {
    const int stage = it % kDecStages;
    if (!mbar_wait_bounded(full0 + 8 * stage, (it / kDecStages) & 1, abort_flag, status, PXL_DEV_TIMEOUT_FULL)) {
      failed = 1;
      break;  // reported to the whole CTA at the barrier behind the loop
    }
    const int t = t_begin + it;
    const uint32_t k_smem = stage0 + stage * 2 * TILE_BYTES, v_smem = k_smem + TILE_BYTES;
    const int r0 = warp * 16;
    const int tok_base = t * TILE + r0;
    if (tok_base < hi && tok_base + 16 > lo) {  // warp-uniform
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      qk_16x16<D, true>(qf, k_smem, r0, s[0], s[1]);
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = tok_base + j * 8 + 2 * (lane & 3) + (e & 1);
          const bool valid = tok < hi && tok >= lo;
          s[j][e] = valid ? s[j][e] * scale_log2 : -INFINITY;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
        }
      }
      float corr[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = quad_max(mx[h]);
        const float m_new = fmaxf(m_run[h], mx[h]);
        m_use[h] = (m_new == -INFINITY) ? 0.f : m_new;
        corr[h] = exp2f(m_run[h] - m_use[h]);
        m_run[h] = m_new;
      }
      float ps[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[j][e] = exp2f(s[j][e] - m_use[e >> 1]);
          ps[e >> 1] += s[j][e];
        }
      l_run[0] = l_run[0] * corr[0] + ps[0];
      l_run[1] = l_run[1] * corr[1] + ps[1];
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
      uint32_t pf[4];
      pf[0] = pack_bf16x2(s[0][0], s[0][1]);
      pf[1] = pack_bf16x2(s[0][2], s[0][3]);
      pf[2] = pack_bf16x2(s[1][0], s[1][1]);
      pf[3] = pack_bf16x2(s[1][2], s[1][3]);
      pv_16x16<D, true>(pf, v_smem, r0, o);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * stage);  // this warp is done with the stage
  }
  if (__syncthreads_or(failed)) {
    // loads that are still in flight must land before the CTA's shared memory is released
    __nanosleep(200000);
    return;
  }

  // ---- merge the four warps' partial softmax states through shared memory
  float* o_sm = reinterpret_cast<float*>(smem);          // [4][16][D]
  float* m_sm = o_sm + 4 * 16 * D;                       // [4][16]
  float* l_sm = m_sm + 4 * 16;                           // [4][16]
  l_run[0] = quad_sum(l_run[0]);
  l_run[1] = quad_sum(l_run[1]);
  if (warp < 4) {
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    float* ow = o_sm + warp * 16 * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int c = i * 8 + 2 * (lane & 3);
      ow[r_lo * D + c] = o[i][0];
      ow[r_lo * D + c + 1] = o[i][1];
      ow[r_hi * D + c] = o[i][2];
      ow[r_hi * D + c + 1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      m_sm[warp * 16 + r_lo] = m_run[0];
      m_sm[warp * 16 + r_hi] = m_run[1];
      l_sm[warp * 16 + r_lo] = l_run[0];
      l_sm[warp * 16 + r_hi] = l_run[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; warp < 4 && idx < G * D; idx += 128) {
    const int r = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, m_sm[w * 16 + r]);
    const int head = kvh * G + r;
    const float sink = (sinks && num_splits == 1) ? sinks[head] * kLog2e : -INFINITY;
    const float Mx = fmaxf(M, sink);
    const float Mu = (Mx == -INFINITY) ? 0.f : Mx;
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(m_sm[w * 16 + r] - Mu);
      L += l_sm[w * 16 + r] * f;
      acc += o_sm[(w * 16 + r) * D + d] * f;
    }
    if (num_splits == 1) {
      const float denom = L + exp2f(sink - Mu);
      out[(static_cast<size_t>(b) * Hq + head) * D + d] = __float2bfloat16(denom > 0.f ? acc / denom : 0.f);
    } else {
      float* po = workspace;
      float* plse = workspace + static_cast<size_t>(gridDim.y) * Hq * num_splits * D;
      const size_t row = (static_cast<size_t>(b) * Hq + head) * num_splits + split;
      po[row * D + d] = L > 0.f ? acc / L : 0.f;
      if (d == 0) plse[row] = L > 0.f ? Mu + log2f(L) : -INFINITY;
    }
  }
}

template <int D>
__global__ void __launch_bounds__(D)
attn_decode_reduce_kernel(const float* __restrict__ workspace, const float* __restrict__ sinks,
                          bf16* __restrict__ out, int Hq, int num_splits) {
  pdl_wait();
  pdl_launch_dependents();
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const float* po = workspace;
  const float* plse = workspace + static_cast<size_t>(gridDim.y) * Hq * num_splits * D;
  const size_t row0 = (static_cast<size_t>(b) * Hq + head) * num_splits;
  const float sink = sinks ? sinks[head] * kLog2e : -INFINITY;
  float M = sink;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, plse[row0 + s]);
  const float Mu = (M == -INFINITY) ? 0.f : M;
  float denom = exp2f(sink - Mu), acc = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float w = exp2f(plse[row0 + s] - Mu);
    denom += w;
    acc += w * po[(row0 + s) * D + d];
  }
  out[(static_cast<size_t>(b) * Hq + head) * D + d] =
      __float2bfloat16(denom > 0.f ? acc / denom : 0.f);
}

// ============================================================================== prefill
template <int D, bool FP8 = false>
__global__ void __launch_bounds__(128)
attn_prefill_kernel(const bf16* __restrict__ q, int64_t q_stride, const void* __restrict__ k_cache,
                    const void* __restrict__ v_cache, const int* __restrict__ block_tables,
                    const int* __restrict__ cu_q, const int* __restrict__ ctx_lens,
                    bf16* __restrict__ out, int64_t out_stride, const float* __restrict__ sinks,
                    int Hq, int Hkv, int page_size, int max_blocks, int64_t num_blocks,
                    float scale_log2, int window, float v_scale, int* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int TILE_BYTES = TILE * D * 2;
  const uint32_t k_smem0 = smem_u32(smem);
  const uint32_t v_smem0 = k_smem0 + 2 * TILE_BYTES;

  const int qt = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = Hq / Hkv;
  const int TQ = 64 / G;  // query tokens per CTA (rows = TQ * G <= 64)
  const int q0 = cu_q[b];
  const int q_len = cu_q[b + 1] - q0;
  if (qt * TQ >= q_len) return;
  const int ctx = ctx_lens[b];
  const int prefix = ctx - q_len;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // rows owned by this thread: r_lo = warp*16 + lane/4, r_hi = r_lo + 8
  int rtok[2], rhead[2];
  bool rvalid[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + (lane >> 2) + h * 8;
    const int tq = qt * TQ + r / G;
    rvalid[h] = (r < TQ * G) && (tq < q_len);
    rtok[h] = tq;
    rhead[h] = kvh * G + r % G;
  }
  uint32_t qf[D / 16][4];
  {
    const bf16* q_lo = q + static_cast<size_t>(q0 + rtok[0]) * q_stride + rhead[0] * D;
    const bf16* q_hi = q + static_cast<size_t>(q0 + rtok[1]) * q_stride + rhead[1] * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int c = ks * 16 + 2 * (lane & 3);
      qf[ks][0] = rvalid[0] ? *reinterpret_cast<const uint32_t*>(q_lo + c) : 0u;
      qf[ks][1] = rvalid[1] ? *reinterpret_cast<const uint32_t*>(q_hi + c) : 0u;
      qf[ks][2] = rvalid[0] ? *reinterpret_cast<const uint32_t*>(q_lo + c + 8) : 0u;
      qf[ks][3] = rvalid[1] ? *reinterpret_cast<const uint32_t*>(q_hi + c + 8) : 0u;
    }
  }
  // visible key range per row: [rlo, rpos]
  int rpos[2], rlo[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    rpos[h] = rvalid[h] ? prefix + rtok[h] : -1;
    rlo[h] = (window > 0 && rpos[h] >= window) ? rpos[h] - window + 1 : 0;
  }
  // warp-level bounds (rows of one warp span consecutive tokens)
  const int w_tok_first = qt * TQ + (warp * 16) / G;
  const int w_tok_last = min(q_len - 1, qt * TQ + (warp * 16 + 15) / G);
  const bool warp_active = (warp * 16 < TQ * G) && (w_tok_first < q_len);
  const int w_hi = prefix + w_tok_last;  // last visible key for this warp
  const int w_lo = (window > 0 && prefix + w_tok_first >= window) ? prefix + w_tok_first - window + 1 : 0;

  // CTA-level key range
  const int c_tok_last = min(q_len - 1, qt * TQ + TQ - 1);
  const int c_hi = prefix + c_tok_last + 1;  // exclusive
  const int c_lo = (window > 0 && prefix + qt * TQ >= window) ? prefix + qt * TQ - window + 1 : 0;
  const int t_begin = c_lo / TILE;
  const int t_end = ceil_div(c_hi, TILE);

  KVTileArgs ka{k_cache, v_cache, block_tables + static_cast<size_t>(b) * max_blocks, max_blocks,
                num_blocks, Hkv, kvh, page_size};

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  int buf = 0;
  load_kv_tile<D, FP8>(ka, t_begin * TILE, c_hi, k_smem0, v_smem0, status);
  cp_async_commit();
  for (int t = t_begin; t < t_end; ++t) {
    cp_async_wait<0>();
    __syncthreads();
    if (t + 1 < t_end)
      load_kv_tile<D, FP8>(ka, (t + 1) * TILE, c_hi, k_smem0 + (buf ^ 1) * TILE_BYTES,
                      v_smem0 + (buf ^ 1) * TILE_BYTES, status);
    cp_async_commit();

    const int tok0 = t * TILE;
    if (warp_active && tok0 <= w_hi && tok0 + TILE > w_lo) {
      const uint32_t ks_addr = k_smem0 + buf * TILE_BYTES;
      const uint32_t vs_addr = v_smem0 + buf * TILE_BYTES;
      float s[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int g = 0; g < 4; ++g) qk_16x16<D>(qf, ks_addr, g * 16, s[2 * g], s[2 * g + 1]);

      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          const int tok = tok0 + j * 8 + 2 * (lane & 3) + (e & 1);
          const bool valid = tok <= rpos[h] && tok >= rlo[h];
          s[j][e] = valid ? s[j][e] * scale_log2 : -INFINITY;
          mx[h] = fmaxf(mx[h], s[j][e]);
        }
      float corr[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = quad_max(mx[h]);
        const float m_new = fmaxf(m_run[h], mx[h]);
        m_use[h] = (m_new == -INFINITY) ? 0.f : m_new;
        corr[h] = exp2f(m_run[h] - m_use[h]);
        m_run[h] = m_new;
      }
      float ps[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[j][e] = exp2f(s[j][e] - m_use[e >> 1]);
          ps[e >> 1] += s[j][e];
        }
      l_run[0] = l_run[0] * corr[0] + ps[0];
      l_run[1] = l_run[1] * corr[1] + ps[1];
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint32_t pf[4];
        pf[0] = pack_bf16x2(s[2 * g][0], s[2 * g][1]);
        pf[1] = pack_bf16x2(s[2 * g][2], s[2 * g][3]);
        pf[2] = pack_bf16x2(s[2 * g + 1][0], s[2 * g + 1][1]);
        pf[3] = pack_bf16x2(s[2 * g + 1][2], s[2 * g + 1][3]);
        pv_16x16<D>(pf, vs_addr, g * 16, o);
      }
    }
    buf ^= 1;
  }
  cp_async_wait<0>();

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!rvalid[h]) continue;
    float L = quad_sum(l_run[h]);
    float M = m_run[h];
    const float sink = sinks ? sinks[rhead[h]] * kLog2e : -INFINITY;
    const float Mx = fmaxf(M, sink);
    const float Mu = (Mx == -INFINITY) ? 0.f : Mx;
    const float f = exp2f(M - Mu);
    const float denom = L * f + exp2f(sink - Mu);
    const float inv = denom > 0.f ? f / denom * v_scale : 0.f;
    bf16* dst = out + static_cast<size_t>(q0 + rtok[h]) * out_stride + rhead[h] * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int c = i * 8 + 2 * (lane & 3);
      *reinterpret_cast<uint32_t*>(dst + c) =
          pack_bf16x2(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
    }
  }
}

inline int check_launch() { return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA; }

template <typename K>
int set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) ==
                 cudaSuccess
             ? PXL_OK
             : PXL_ERR_CUDA;
}

}  // namespace

PXL_EXPORT int pxl_attn_decode_splits(int B, int Hkv, int max_ctx) {
  const int blocks = B * Hkv;
  const int target = 2 * pxl_host::num_sms();
  int s = blocks >= target ? 1 : pxl::ceil_div(target, blocks);
  const int max_by_ctx = pxl::ceil_div(max_ctx > 0 ? max_ctx : 1, 256);
  if (s > max_by_ctx) s = max_by_ctx;
  if (s > 64) s = 64;
  if (s < 1) s = 1;
  return s;
}

namespace {
int attn_decode_impl(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                     const int* block_tables, const int* ctx_lens, void* out, float* workspace,
                     const float* sinks, int B, int Hq, int Hkv, int D, int page_size, int max_blocks,
                     int64_t num_blocks, float scale, int window, int num_splits, int max_ctx,
                     bool cache_fp8, float k_scale, float v_scale, int* status, pxl_stream_t stream) {
  if (B <= 0) return PXL_OK;
  if (Hkv <= 0 || Hq % Hkv || Hq / Hkv > 16 || page_size <= 0) return PXL_ERR_INVALID_ARG;
  if (num_splits <= 0) num_splits = pxl_attn_decode_splits(B, Hkv, max_ctx);
  if (num_splits > 1 && workspace == nullptr) return PXL_ERR_INVALID_ARG;
  const float scale_log2 = scale * kLog2e;
  dim3 grid(Hkv, B, num_splits);
  if (!cache_fp8 && D == 128 && (page_size == 16 || page_size == 32 || page_size == 64) &&
      num_blocks * Hkv * page_size < (1ll << 31)) {
    // TMA-fed kernel: the cache is a 2-D matrix [blocks * Hkv * page, 128], one box = one page half
    CUtensorMap tk, tv;
    const uint64_t rows = static_cast<uint64_t>(num_blocks) * Hkv * page_size;
    if (!pxl_host::make_tmap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k_cache, rows, 128, 128, page_size, 64) ||
        !pxl_host::make_tmap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v_cache, rows, 128, 128, page_size, 64))
      return PXL_ERR_TENSORMAP;
    constexpr int SMEM = 1024 + kDecStages * 2 * TILE * 128 * 2 + 128;
    static bool done[64] = {false};      // function attributes are per device
    const int dev = pxl_host::current_device_slot();
    if (!done[dev]) {
      if (set_smem(attn_decode_tma_kernel, SMEM)) return PXL_ERR_CUDA;
      done[dev] = true;
    }
    pxl_host::launch(attn_decode_tma_kernel, grid, kDecThreads, SMEM, stream,
        tk, tv, static_cast<const bf16*>(q), q_stride, block_tables, ctx_lens, static_cast<bf16*>(out), workspace,
        sinks, Hq, Hkv, page_size, max_blocks, num_blocks, scale_log2, window, num_splits, status);
    if (num_splits > 1)
      pxl_host::launch(attn_decode_reduce_kernel<128>, dim3(Hq, B), 128, 0, stream, workspace, sinks,
                       static_cast<bf16*>(out), Hq, num_splits);
    return check_launch();
  }
#define PXL_DEC(DD, F8)                                                                          \
  {                                                                                              \
    constexpr int SMEM = 4 * TILE * DD * 2 > (4 * 16 * DD + 128) * 4 ? 4 * TILE * DD * 2         \
                                                                     : (4 * 16 * DD + 128) * 4;  \
    static bool done[64] = {false};                                                              \
    const int dev = pxl_host::current_device_slot();                                                       \
    if (!done[dev]) {                                                                            \
      if (set_smem(attn_decode_kernel<DD, F8>, SMEM)) return PXL_ERR_CUDA;                       \
      done[dev] = true;                                                                          \
    }                                                                                            \
    attn_decode_kernel<DD, F8><<<grid, 128, SMEM, stream>>>(                                     \
        static_cast<const bf16*>(q), q_stride, k_cache, v_cache, block_tables, ctx_lens,         \
        static_cast<bf16*>(out), workspace, sinks, Hq, Hkv, page_size, max_blocks, num_blocks,   \
        scale_log2 * k_scale, window, num_splits, v_scale, status);                              \
    if (num_splits > 1)                                                                          \
      attn_decode_reduce_kernel<DD><<<dim3(Hq, B), DD, 0, stream>>>(                             \
          workspace, sinks, static_cast<bf16*>(out), Hq, num_splits);                            \
  }
  if (cache_fp8) {
    if (D == 128) PXL_DEC(128, true)
    else if (D == 64) PXL_DEC(64, true)
    else return PXL_ERR_INVALID_ARG;
  } else {
    if (D == 128) PXL_DEC(128, false)
    else if (D == 64) PXL_DEC(64, false)
    else return PXL_ERR_INVALID_ARG;
  }
#undef PXL_DEC
  return check_launch();
}
}  // namespace

PXL_EXPORT int pxl_attn_decode(const void* q, int64_t q_stride, const void* k_cache,
                               const void* v_cache,
                               const int* block_tables, const int* ctx_lens, void* out,
                               float* workspace, const float* sinks, int B, int Hq, int Hkv, int D,
                               int page_size, int max_blocks, int64_t num_blocks, float scale,
                               int window, int num_splits, int max_ctx, int* status,
                               pxl_stream_t stream) {
  return attn_decode_impl(q, q_stride, k_cache, v_cache, block_tables, ctx_lens, out, workspace, sinks,
                          B, Hq, Hkv, D, page_size, max_blocks, num_blocks, scale, window, num_splits,
                          max_ctx, false, 1.f, 1.f, status, stream);
}

// Decode attention over e4m3 caches written by pxl_qk_norm_rope_cache_fp8 / pxl_reshape_and_cache_fp8
// with the same scales. The cache bytes are widened to bf16 on their way into shared memory, the K
// scale is folded into the score scale and the V scale into the output normalisation.
PXL_EXPORT int pxl_attn_decode_fp8(const void* q, int64_t q_stride, const void* k_cache,
                                   const void* v_cache, const int* block_tables,
                                   const int* ctx_lens, void* out, float* workspace,
                                   const float* sinks, int B, int Hq, int Hkv, int D, int page_size,
                                   int max_blocks, int64_t num_blocks, float scale, int window,
                                   int num_splits, int max_ctx, float k_scale, float v_scale,
                                   int* status, pxl_stream_t stream) {
  if (!(k_scale > 0.f) || !(v_scale > 0.f)) return PXL_ERR_INVALID_ARG;
  return attn_decode_impl(q, q_stride, k_cache, v_cache, block_tables, ctx_lens, out, workspace, sinks,
                          B, Hq, Hkv, D, page_size, max_blocks, num_blocks, scale, window, num_splits,
                          max_ctx, true, k_scale, v_scale, status, stream);
}

namespace {
int attn_prefill_impl(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                      const int* block_tables, const int* cu_q, const int* ctx_lens, void* out,
                      int64_t out_stride, const float* sinks, int B, int max_q_len, int Hq, int Hkv,
                      int D, int page_size, int max_blocks, int64_t num_blocks, float scale,
                      int window, bool cache_fp8, float k_scale, float v_scale, int* status,
                      pxl_stream_t stream) {
  if (B <= 0 || max_q_len <= 0) return PXL_OK;
  if (Hkv <= 0 || Hq % Hkv || Hq / Hkv > 64 || page_size <= 0) return PXL_ERR_INVALID_ARG;
  const int G = Hq / Hkv;
  const int TQ = 64 / G;
  const float scale_log2 = scale * kLog2e;
  dim3 grid(pxl::ceil_div(max_q_len, TQ), Hkv, B);
#define PXL_PRE(DD, F8)                                                                          \
  {                                                                                              \
    constexpr int SMEM = 4 * TILE * DD * 2;                                                      \
    static bool done[64] = {false};                                                              \
    const int dev = pxl_host::current_device_slot();                                             \
    if (!done[dev]) {                                                                            \
      if (set_smem(attn_prefill_kernel<DD, F8>, SMEM)) return PXL_ERR_CUDA;                      \
      done[dev] = true;                                                                          \
    }                                                                                            \
    attn_prefill_kernel<DD, F8><<<grid, 128, SMEM, stream>>>(                                    \
        static_cast<const bf16*>(q), q_stride, k_cache, v_cache, block_tables, cu_q, ctx_lens,   \
        static_cast<bf16*>(out), out_stride, sinks, Hq, Hkv, page_size, max_blocks, num_blocks,  \
        scale_log2 * k_scale, window, v_scale, status);                                          \
  }
  if (cache_fp8) {
    if (D == 128) PXL_PRE(128, true)
    else if (D == 64) PXL_PRE(64, true)
    else return PXL_ERR_INVALID_ARG;
  } else {
    if (D == 128) PXL_PRE(128, false)
    else if (D == 64) PXL_PRE(64, false)
    else return PXL_ERR_INVALID_ARG;
  }
#undef PXL_PRE
  return check_launch();
}
}  // namespace

PXL_EXPORT int pxl_attn_prefill(const void* q, int64_t q_stride, const void* k_cache,
                                const void* v_cache, const int* block_tables, const int* cu_q,
                                const int* ctx_lens, void* out, int64_t out_stride,
                                const float* sinks, int B, int max_q_len, int Hq, int Hkv, int D,
                                int page_size, int max_blocks, int64_t num_blocks, float scale,
                                int window, int* status, pxl_stream_t stream) {
  return attn_prefill_impl(q, q_stride, k_cache, v_cache, block_tables, cu_q, ctx_lens, out, out_stride,
                           sinks, B, max_q_len, Hq, Hkv, D, page_size, max_blocks, num_blocks, scale,
                           window, false, 1.f, 1.f, status, stream);
}

// Prefix-aware prefill over e4m3 caches (see pxl_attn_decode_fp8).
PXL_EXPORT int pxl_attn_prefill_fp8(const void* q, int64_t q_stride, const void* k_cache,
                                    const void* v_cache, const int* block_tables, const int* cu_q,
                                    const int* ctx_lens, void* out, int64_t out_stride,
                                    const float* sinks, int B, int max_q_len, int Hq, int Hkv, int D,
                                    int page_size, int max_blocks, int64_t num_blocks, float scale,
                                    int window, float k_scale, float v_scale, int* status,
                                    pxl_stream_t stream) {
  if (!(k_scale > 0.f) || !(v_scale > 0.f)) return PXL_ERR_INVALID_ARG;
  return attn_prefill_impl(q, q_stride, k_cache, v_cache, block_tables, cu_q, ctx_lens, out, out_stride,
                           sinks, B, max_q_len, Hq, Hkv, D, page_size, max_blocks, num_blocks, scale,
                           window, true, k_scale, v_scale, status, stream);
}

// ----------------------------------------------------------------------------------------
// Allocation-free decode attention (see pxl_noalloc.h). The scratch for the split-KV partial
// results is this file-scope device array. In host code `g_decode_static_scratch` is only a
// stand-in for the symbol, not a device address, so the launcher asks the runtime for the
// real address once per device and hands that pointer to the kernels.
static __device__ __align__(256) float g_decode_static_scratch[PXL_DECODE_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
// Written by whichever host thread asks first; two threads racing on the first call store the
// same value, and the atomic makes that store and the later loads well defined.
std::atomic<float*> g_static_scratch_addr[kMaxDevices];

// Device address of the scratch array on the current device, or nullptr on error.
float* static_scratch_ptr() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  float* known = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (known == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_decode_static_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();  // leave no sticky error behind for the caller
      return nullptr;
    }
    known = static_cast<float*>(p);
    g_static_scratch_addr[dev].store(known, std::memory_order_release);
  }
  return known;
}
}  // namespace

PXL_EXPORT int pxl_attn_decode_static_scratch(const void* q, int64_t q_stride, const void* k_cache,
                                              const void* v_cache, const int* block_tables,
                                              const int* ctx_lens, void* out, const float* sinks,
                                              int B, int Hq, int Hkv, int D, int page_size,
                                              int max_blocks, int64_t num_blocks, float scale,
                                              int window, int num_splits, int* status,
                                              pxl_stream_t stream) {
  if (B <= 0) return PXL_OK;
  if (num_splits < 1 || Hq <= 0 || D <= 0) return PXL_ERR_INVALID_ARG;
  float* scratch = nullptr;
  if (num_splits > 1) {
    const int64_t need = static_cast<int64_t>(B) * Hq * num_splits * (D + 2);
    if (need > static_cast<int64_t>(PXL_DECODE_STATIC_SCRATCH_FLOATS)) return PXL_ERR_TOO_LARGE;
    scratch = static_scratch_ptr();
    if (scratch == nullptr) return PXL_ERR_CUDA;
  }
  // Every (sequence, head, split) partial that the reduction reads is written by the main
  // kernel of this same call, so the array needs no clearing between calls.
  return pxl_attn_decode(q, q_stride, k_cache, v_cache, block_tables, ctx_lens, out, scratch, sinks,
                         B, Hq, Hkv, D, page_size, max_blocks, num_blocks, scale, window, num_splits,
                         0, status, stream);
}
