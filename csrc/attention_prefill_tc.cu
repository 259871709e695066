// Ragged causal prefill attention over the paged KV cache on the 5th-generation tensor cores
// (head dim 128, page 16 / 32 / 64).
//
// One CTA = 128 query tokens of one (sequence, query head); it walks the keys it may see in tiles
// of 128:
//   warp 8   : TMA producer. Q tile once, then K and V tiles (page boxes of the cache, 128-byte
//              swizzle) through a two-stage ring guarded by full / empty mbarriers.
//   warp 9   : MMA issuer. S = Q K^T (tcgen05.mma 128x128x16, both operands K-major) into one of
//              two TMEM score buffers, so the scores of tile i+1 are computed while the softmax
//              warps work on tile i; then O += P V with V taken MN-major straight from the
//              [token, dim] layout of the cache (two 64-wide halves of the head dim).
//   warps 0-7: softmax. A query row is one TMEM lane; warps w and w + 4 share a lane quarter and
//              split the columns: each thread reads 64 scores of its row with tcgen05.ld, masks
//              (causal, context end, sliding window), the two halves exchange their row maximum
//              through shared memory, each writes its half of P as bf16 into the swizzled
//              A-operand tile. The output accumulates in TMEM over all tiles (the second MMA
//              adds to it) relative to a reference maximum that only moves, with a rescale of the
//              TMEM rows by tcgen05.ld / st, when a row maximum grew by more than 2^8; so the
//              softmax of tile i+1 does not wait for the P V product of tile i.
// Every wait is bounded; on expiry the kernel records a status code, all roles unwind, TMEM is freed.
//
// Reference counterpart: the MLX SDPA call with a gathered KV prefix
// (src/parallax/server/cache/prefix_cache_utils.py:11-91, src/parallax/models/qwen3.py:84-120).
#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

constexpr int kQ = 128;         // query rows per CTA
constexpr int kT = 128;         // keys per tile
constexpr int kD = 128;         // head dim
constexpr int kHalf = kQ * 128; // bytes of one 64-column half of a 128-row operand tile
constexpr int kTileBytes = 2 * kHalf;
constexpr int kStages = 2;
constexpr int kSoftmaxWarps = 8;   // two per TMEM lane quarter: each takes one half of the columns
constexpr int kProducerWarp = 8, kMmaWarp = 9;
constexpr int kThreads = 320;
constexpr float kLog2eF = 1.4426950408889634f;

// shared memory map (after 1024-byte alignment)
constexpr int kOffQ = 0;
constexpr int kOffP = kTileBytes;
constexpr int kOffKV = 2 * kTileBytes;                       // stage s: K at +s*2*tile, V behind it
constexpr int kOffBars = kOffKV + kStages * 2 * kTileBytes;  // 196608
constexpr int kOffXchg = kOffBars + 256;                     // row max [2 tiles][2 halves][128], row sum [2][128]
constexpr int kSmemBytes = 1024 + kOffXchg + 3 * 2 * 128 * 4;

// B operand stored [key rows, 64 dims] (MN-major: the dim index is contiguous), 128-byte swizzle:
// rows of 128 B, groups of 8 key rows 1024 B apart. Only one 64-wide chunk of the MN extent is
// addressed per instruction (N = 64), so the leading-dimension offset is not used.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ float fast_exp2(float x) {  // 2^x, -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr uint32_t kIdescS = umma_idesc(kQ, kT, 1, 1);
constexpr uint32_t kIdescPV = umma_idesc(kQ, 64, 1, 1) | (1u << 16);  // B (V) is MN-major

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const int* __restrict__ block_tables,
                       const int* __restrict__ cu_q, const int* __restrict__ ctx_lens, bf16* __restrict__ out,
                       int64_t out_stride, const float* __restrict__ sinks, int Hq, int Hkv, int page_size,
                       int max_blocks, int64_t num_blocks, float scale_log2, int window, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sm0 = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  // 0 q_full | 1,2 kv_full | 3,4 kv_empty | 5,6 s_full | 7 p_ready | 8 o_full
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t q_full = bar0, kv_full = bar0 + 8, kv_empty = bar0 + 24, s_full = bar0 + 40, p_ready = bar0 + 56,
                 o_full = bar0 + 64;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  pdl_wait();
  pdl_launch_dependents();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, head = blockIdx.y;
  const int kvh = head / (Hq / Hkv);
  const int q_begin = cu_q[b], L = cu_q[b + 1] - q_begin;
  const int ctx = ctx_lens[b];
  // heavy blocks (late queries see the most keys) are scheduled first
  const int qb = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int q0 = qb * kQ;
  if (q0 >= L) return;  // uniform for the CTA, before any barrier or allocation
  const int pos0 = ctx - L + q0;                        // position of query row 0
  const int rows = L - q0 < kQ ? L - q0 : kQ;           // valid query rows
  const int hi = pos0 + rows;                           // keys [lo, hi) are visible to some row
  const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int t_begin = lo / kT;
  const int n_tiles = ceil_div(hi, kT) - t_begin;
  const int* bt = block_tables + static_cast<size_t>(b) * max_blocks;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(kv_full + 8 * s, 1);
      mbar_init(kv_empty + 8 * s, 1);
      mbar_init(s_full + 8 * s, 1);
    }
    mbar_init(p_ready, kSoftmaxWarps);  // one arrival per softmax warp
    mbar_init(o_full, 1);
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), 512);  // S0 | S1 | O (384 columns, allocated as a power of two)
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_o = tmem_base + 2 * kT;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp works: lane p looks up the block of page p of the tile and issues that page's
    // four box loads, so the block-table reads of a tile are in flight together (one lane doing them
    // one after the other cost more than the tile's math) and are issued before the wait for the stage.
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, kTileBytes);
      tma_load_2d(sm0 + kOffQ, &tm_q, q_full, head * kD, q_begin + q0);
      tma_load_2d(sm0 + kOffQ + kHalf, &tm_q, q_full, head * kD + 64, q_begin + q0);
    }
    const int ppt = kT / page_size;
    for (int it = 0; it < n_tiles; ++it) {
      const int stage = it % kStages;
      int blk = 0;
      if (lane < ppt) {
        int bi = (t_begin + it) * ppt + lane;
        if (bi * page_size >= ctx) bi = (ctx - 1) / page_size;  // beyond the context: re-read the last page (masked)
        blk = bi < max_blocks ? bt[bi] : -1;
        if (blk < 0 || blk >= num_blocks) {
          if (status) atomicCAS(status, 0, PXL_DEV_BAD_BLOCK_PREFILL);
          blk = 0;
        }
      }
      int okf = 1;
      if (it >= kStages && lane == 0)
        okf = mbar_wait_bounded(kv_empty + 8 * stage, ((it / kStages) - 1) & 1, abort_flag, status,
                                PXL_DEV_TIMEOUT_EMPTY) ? 1 : 0;
      okf = __shfl_sync(0xffffffffu, okf, 0);
      if (!okf) break;
      const uint32_t bar = kv_full + 8 * stage;
      const uint32_t k_dst = sm0 + kOffKV + stage * 2 * kTileBytes, v_dst = k_dst + kTileBytes;
      if (lane == 0) mbar_arrive_expect_tx(bar, 2 * kTileBytes);
      __syncwarp();
      if (lane < ppt) {
        const int row0 = (blk * Hkv + kvh) * page_size;
        const uint32_t off = lane * page_size * 128;
        tma_load_2d(k_dst + off, &tm_k, bar, 0, row0);
        tma_load_2d(k_dst + kHalf + off, &tm_k, bar, 64, row0);
        tma_load_2d(v_dst + off, &tm_v, bar, 0, row0);
        tma_load_2d(v_dst + kHalf + off, &tm_v, bar, 64, row0);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      auto issue_s = [&](int it) {  // S[it % 2] = Q K(it)^T
        const int stage = it % kStages;
        const uint32_t k_addr = sm0 + kOffKV + stage * 2 * kTileBytes;
        const uint32_t d_tmem = tmem_base + (it & 1) * kT;
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks) {
          const uint32_t off = (ks >> 2) * kHalf + (ks & 3) * 32;
          tc_mma_f16(d_tmem, umma_desc_k_sw128(sm0 + kOffQ + off), umma_desc_k_sw128(k_addr + off), kIdescS,
                     ks > 0 ? 1u : 0u);
        }
        tc_commit(s_full + 8 * (it & 1));
      };
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag, status, PXL_DEV_TIMEOUT_FULL);
      ok = ok && mbar_wait_bounded(kv_full, 0, abort_flag, status, PXL_DEV_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0);
      }
      for (int it = 0; ok && it < n_tiles; ++it) {
        const int stage = it % kStages;
        if (it + 1 < n_tiles) {
          // scores of the next tile while the softmax warps work on this one
          ok = mbar_wait_bounded(kv_full + 8 * ((it + 1) % kStages), ((it + 1) / kStages) & 1, abort_flag, status,
                                 PXL_DEV_TIMEOUT_FULL);
          if (!ok) break;
          tc_fence_after_sync();
          issue_s(it + 1);
        }
        ok = mbar_wait_bounded(p_ready, it & 1, abort_flag, status, PXL_DEV_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t v_addr = sm0 + kOffKV + stage * 2 * kTileBytes + kTileBytes;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int ks = 0; ks < kT / 16; ++ks) {
            const uint64_t da = umma_desc_k_sw128(sm0 + kOffP + (ks >> 2) * kHalf + (ks & 3) * 32);
            const uint64_t db = umma_desc_mn_sw128(v_addr + h * kHalf + ks * 2048);
            tc_mma_f16(tm_o + h * 64, da, db, kIdescPV, (it > 0 || ks > 0) ? 1u : 0u);  // O stays in TMEM
          }
        }
        tc_commit(o_full);
        tc_commit(kv_empty + 8 * stage);  // K and V of this stage are no longer read
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps
    const int q4 = warp & 3, hc = warp >> 2;  // TMEM lane quarter, column half
    const int r = q4 * 32 + lane;             // query row = TMEM lane
    const int q_pos = pos0 + r;
    const bool row_valid = r < rows;
    const int key_lo = (window > 0 && q_pos - window + 1 > 0) ? q_pos - window + 1 : 0;
    const uint32_t lane_sel = static_cast<uint32_t>(q4 * 32) << 16;
    const uint32_t p_row = sm0 + kOffP + hc * kHalf + r * 128;  // this thread's 64 keys = one swizzled 128-byte row
    float* mx_sm = reinterpret_cast<float*>(smem + kOffXchg);    // [tile parity][half][row]
    float* l_sm = mx_sm + 2 * 2 * 128;                           // [half][row]
    float m_run = -INFINITY, l_run = 0.f;
    // 1 after a wait ran out; agreed among the 256 softmax threads at the barrier of every tile, so
    // that they all leave the loop at the same place
    int failed = 0;
    auto agree = [&](int f) {
      int r_out;
      asm volatile(
          "{\n\t"
          ".reg .pred pin, pout;\n\t"
          "setp.ne.b32 pin, %1, 0;\n\t"
          "bar.red.or.pred pout, 1, 256, pin;\n\t"
          "selp.b32 %0, 1, 0, pout;\n\t"
          "}\n"
          : "=r"(r_out)
          : "r"(f)
          : "memory");
      return r_out;
    };
    for (int it = 0; it < n_tiles; ++it) {
      if (!failed)
        failed = mbar_wait_bounded(s_full + 8 * (it & 1), (it >> 1) & 1, abort_flag, status, PXL_DEV_TIMEOUT_TMEM_FULL) ? 0 : 1;
      failed = __any_sync(0xffffffffu, failed);  // warp-uniform: the TMEM loads below are warp-wide
      const uint32_t t_s = tmem_base + (it & 1) * kT + hc * 64 + lane_sel;
      const int tile_key0 = (t_begin + it) * kT;
      // interior tile: every key is visible to every row of the block, no masking needed
      const bool interior = tile_key0 + kT - 1 <= pos0 && (window <= 0 || tile_key0 >= pos0 + kQ - window);
      // this thread's 64 scores stay in registers between the maximum and the exponentials
      uint32_t sc[64];
      float mx = -INFINITY;
      if (!failed) {
        tc_fence_after_sync();
        tmem_ld_32x32b_x32(t_s, *reinterpret_cast<uint32_t(*)[32]>(&sc[0]));
        tmem_ld_32x32b_x32(t_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&sc[32]));
        tmem_ld_wait();
        if (!interior) {
          // keys this thread's row may see among its 64 columns: [a, e)
          const int key0 = tile_key0 + hc * 64;
          const int a = key_lo - key0, e = (row_valid ? q_pos + 1 : 0) - key0;
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (j < a || j >= e) sc[j] = 0xff800000u;  // -inf
        }
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 64; j += 4) {
#pragma unroll
          for (int k = 0; k < 4; ++k) m4[k] = fmaxf(m4[k], __uint_as_float(sc[j + k]));
        }
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      }
      mx_sm[((it & 1) * 2 + hc) * 128 + r] = mx;
      failed = agree(failed);
      if (failed) break;
      mx = fmaxf(mx, mx_sm[((it & 1) * 2 + (hc ^ 1)) * 128 + r]) * scale_log2;  // scale > 0
      const float m_new = fmaxf(m_run, mx);
      // The output accumulates in TMEM across tiles, relative to the reference maximum m_run. The
      // reference only moves (and O is rescaled) when some row of this lane quarter grew by more
      // than 2^8: until then the stale reference keeps every probability below 256, which bf16 and
      // the fp32 sums hold without trouble. Both warps of a lane quarter see the same 32 rows and
      // the same maxima, so they take the same decision.
      const bool grow = __any_sync(0xffffffffu, m_new > m_run + 8.f);
      // P of the previous tile must have been consumed (and O be complete) before either is touched
      if (it > 0) failed = mbar_wait_bounded(o_full, (it - 1) & 1, abort_flag, status, PXL_DEV_TIMEOUT_TMEM_FULL) ? 0 : 1;
      failed = __any_sync(0xffffffffu, failed);
      if (it == 0) {
        m_run = m_new;
      } else if (grow && !failed) {
        const float corr = fast_exp2(m_run - (m_new == -INFINITY ? 0.f : m_new));
        m_run = m_new;
        l_run *= corr;
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < 64; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tm_o + lane_sel + hc * 64 + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
          tmem_st_32x32b_x32(tm_o + lane_sel + hc * 64 + c, v);
        }
        tmem_st_wait();
      }
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      // probabilities -> bf16 A-operand tile (K-major, 128-byte swizzle), partial row sum
      float sum2[2] = {0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 64; c += 8) {
        uint32_t pk[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(sc[c + j]), scale_log2, -m_use));
          const float p1 = fast_exp2(fmaf(__uint_as_float(sc[c + j + 1]), scale_log2, -m_use));
          sum2[0] += p0;
          sum2[1] += p1;
          pk[j >> 1] = pack_bf16x2(p0, p1);
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + (((c >> 3) ^ (r & 7)) << 4)), "r"(pk[0]),
                     "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                     : "memory");
      }
      l_run += sum2[0] + sum2[1];
      tc_fence_before_sync();
      fence_proxy_async_smem();  // P was written through the generic proxy, the MMA reads it through the async one
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    // the last P V
    if (!failed && n_tiles > 0)
      failed = mbar_wait_bounded(o_full, (n_tiles - 1) & 1, abort_flag, status, PXL_DEV_TIMEOUT_TMEM_FULL) ? 0 : 1;
    failed = __any_sync(0xffffffffu, failed);
    // the two halves of a row saw the same maxima, so their partial sums just add up
    l_sm[hc * 128 + r] = l_run;
    failed = agree(failed);
    if (!failed) {  // the same for all softmax threads: the TMEM loads below are warp-wide
      float denom = l_run + l_sm[(hc ^ 1) * 128 + r];
      float f = 1.f;
      if (sinks) {
        const float sink = sinks[head] * kLog2eF;
        const float M = fmaxf(m_run, sink);
        f = exp2f(m_run - M);
        denom = denom * f + exp2f(sink - M);
      }
      const float inv = denom > 0.f ? f / denom : 0.f;
      bf16* dst = out + static_cast<size_t>(q_begin + q0 + r) * out_stride + head * kD + hc * 64;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tm_o + lane_sel + hc * 64 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int c8 = 0; c8 < 32; c8 += 8) {
          bf16x8 ov;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            ov.u[j] = pack_bf16x2(__uint_as_float(v[c8 + 2 * j]) * inv, __uint_as_float(v[c8 + 2 * j + 1]) * inv);
          if (row_valid) st_bf16x8(dst + c + c8, ov);
        }
      }
      tc_fence_before_sync();
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_flag) __nanosleep(200000);  // loads that are still in flight must land before smem is released
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, 512);
}

}  // namespace

// Same contract as pxl_attn_prefill plus total_q = rows of q / out (sum of the new lengths): the
// query tile is fetched with TMA boxes of 128 rows and rows past total_q must read as zeros.
PXL_EXPORT int pxl_attn_prefill_tc(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                   const int* block_tables, const int* cu_q, const int* ctx_lens, void* out,
                                   int64_t out_stride, const float* sinks, int B, int max_q_len, int total_q, int Hq,
                                   int Hkv, int D, int page_size, int max_blocks, int64_t num_blocks, float scale,
                                   int window, int* status, cudaStream_t stream) {
  if (B <= 0 || max_q_len <= 0 || total_q <= 0) return PXL_OK;
  if (D != kD || Hkv <= 0 || Hq % Hkv) return PXL_ERR_INVALID_ARG;
  if (page_size != 16 && page_size != 32 && page_size != 64) return PXL_ERR_INVALID_ARG;
  if ((q_stride % 8) || (out_stride % 8) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return PXL_ERR_INVALID_ARG;
  if (num_blocks * Hkv * page_size >= (1ll << 31) || scale <= 0.f) return PXL_ERR_INVALID_ARG;
  CUtensorMap tq, tk, tv;
  const uint64_t rows = static_cast<uint64_t>(num_blocks) * Hkv * page_size;
  if (!pxl_host::make_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, total_q, static_cast<uint64_t>(Hq) * kD,
                              q_stride, kQ, 64) ||
      !pxl_host::make_tmap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k_cache, rows, 128, 128, page_size, 64) ||
      !pxl_host::make_tmap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v_cache, rows, 128, 128, page_size, 64))
    return PXL_ERR_TENSORMAP;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
        cudaSuccess)
      return PXL_ERR_CUDA;
    configured[dev] = true;
  }
  dim3 grid(pxl::ceil_div(max_q_len, kQ), Hq, B);
  pxl_host::launch(attn_prefill_tc_kernel, grid, kThreads, kSmemBytes, stream,
      tq, tk, tv, block_tables, cu_q, ctx_lens, static_cast<pxl::bf16*>(out), out_stride, sinks, Hq, Hkv, page_size,
      max_blocks, num_blocks, scale * kLog2eF, window, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}
