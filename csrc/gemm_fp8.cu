// Block-scaled fp8 (e4m3) GEMM on the 5th-generation tensor cores:
//
//   C[m, n] = sum_kb  a_s[m, kb] * w_s[n / 64, kb] * sum_{k in block kb} A[m, k] * W[n, k]
//
// A: activations quantised in 1 x 128 groups (a_s [M, K/128] fp32), W: weights quantised in
// 128 x 128 blocks; the weight scales are passed at 64-row granularity (w_s [N/64, K/128]) so
// that gate/up matrices interleaved in groups of 64 rows keep their own scales. This is the
// DeepSeek-V3 checkpoint format, which the reference hands to its GPU backends as
// `quantization="fp8"` (src/parallax/sglang/model_runner.py:358-366).
//
// One CTA per 128 x 128 output tile, two CTAs per SM. Per 128-wide K block the MMA warp issues
// four tcgen05.mma (kind::f8f6f4, K = 32) into one of two TMEM partial accumulators; the four
// epilogue warps drain each finished partial with tcgen05.ld and add it, multiplied by the
// block's scales, to fp32 accumulators held in registers. Draining partial kb overlaps the
// MMAs of block kb + 1. Dense and grouped (per-expert m-tile lists) modes; epilogues: plain,
// +residual, SiLU-mul. Every wait is time-bounded.
#include <cuda_fp8.h>

#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

constexpr int FM = 128, FN = 128, FK = 128;  // tile; FK bytes = one 128-byte swizzle row of fp8
constexpr int F_STAGES = 3;
constexpr int F_STAGE_BYTES = (FM + FN) * FK;  // 32 KB
constexpr int F_SMEM = 1024 + F_STAGES * F_STAGE_BYTES + 256;
constexpr int F_THREADS = 192;

struct Fp8Args {
  const float* a_s;   // [M, kb_total]
  const float* w_s;   // [w_rows / 64, kb_total]
  bf16* C;
  const bf16* residual;
  int ldc, M, N, K, epi;
  // grouped mode
  const int* mt_expert;
  const int* mt_row0;
  const int* mt_row_end;
  const int* num_mt;
  int w_rows_per_expert;
};

__global__ void __launch_bounds__(F_THREADS, 2)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const Fp8Args g, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + F_STAGES * F_STAGE_BYTES);
  // bars: [0,S) full, [S,2S) empty, [2S,2S+2) part_full, [2S+2,2S+4) part_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * F_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + F_STAGES);
  const uint32_t pfull0 = smem_u32(bars + 2 * F_STAGES), pempty0 = smem_u32(bars + 2 * F_STAGES + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- tile coordinates
  const int num_n = ceil_div(g.N, FN);
  int a_row, b_row, row_end, n_blk;
  {
    const int tile = blockIdx.x;
    if (g.num_mt != nullptr) {
      const int mt = tile / num_n;
      if (mt >= *g.num_mt) return;
      n_blk = tile % num_n;
      a_row = g.mt_row0[mt];
      row_end = g.mt_row_end[mt];
      b_row = g.mt_expert[mt] * g.w_rows_per_expert + n_blk * FN;
    } else {
      const int num_m = ceil_div(g.M, FM);
      n_blk = tile / num_m;
      a_row = (tile % num_m) * FM;
      row_end = g.M;
      b_row = n_blk * FN;
    }
  }
  const int num_kb = g.K / FK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < F_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(pfull0 + 8 * a, 1);
      mbar_init(pempty0 + 8 * a, 4);
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 2 * FN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1, abort_flag, status, PXL_DEV_TIMEOUT_EMPTY)) break;
        const uint32_t fb = full0 + 8 * stage;
        mbar_arrive_expect_tx(fb, F_STAGE_BYTES);
        tma_load_2d(smem_u32(smem + stage * F_STAGE_BYTES), &tmap_a, fb, kb * FK, a_row);
        tma_load_2d(smem_u32(smem + stage * F_STAGE_BYTES + FM * FK), &tmap_b, fb, kb * FK, b_row);
        if (++stage == F_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(FM, FN, 0, 0);  // e4m3 x e4m3 -> fp32
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int part = kb & 1;
        const uint32_t pphase = (kb >> 1) & 1;
        if (!mbar_wait_bounded(pempty0 + 8 * part, pphase ^ 1, abort_flag, status, PXL_DEV_TIMEOUT_TMEM_EMPTY)) break;
        if (!mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag, status, PXL_DEV_TIMEOUT_FULL)) break;
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(smem + stage * F_STAGE_BYTES);
        const uint32_t b_addr = a_addr + FM * FK;
#pragma unroll
        for (int k = 0; k < FK / 32; ++k)
          tc_mma_f8(tmem_base + part * FN, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32),
                    idesc, k > 0 ? 1u : 0u);
        tc_commit(empty0 + 8 * stage);
        tc_commit(pfull0 + 8 * part);
        if (++stage == F_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ---- epilogue warps: thread = one accumulator row
    const int q = warp & 3;
    const int row = a_row + q * 32 + lane;
    const bool row_ok = row < row_end;
    const int kb_total = g.K / FK;
    const float* as_row = g.a_s + static_cast<size_t>(row_ok ? row : a_row) * kb_total;
    const float* ws0 = g.w_s + static_cast<size_t>(b_row / 64) * kb_total;
    const float* ws1 = ws0 + kb_total;
    float acc[FN];
#pragma unroll
    for (int i = 0; i < FN; ++i) acc[i] = 0.f;
    bool ok = true;
    for (int kb = 0; kb < num_kb; ++kb) {
      const int part = kb & 1;
      const uint32_t pphase = (kb >> 1) & 1;
      ok = mbar_wait_bounded(pfull0 + 8 * part, pphase, abort_flag, status, PXL_DEV_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const float sa = as_row[kb];
      const float s0 = sa * ws0[kb], s1 = sa * ws1[kb];
      const uint32_t t_row = tmem_base + part * FN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
      for (int c = 0; c < FN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c, r);
        tmem_ld_wait();
        const float sc = c < 64 ? s0 : s1;
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(__uint_as_float(r[j]), sc, acc[c + j]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(pempty0 + 8 * part);
    }
    if (ok && row_ok) {
      if (g.epi == PXL_EPI_SILU_MUL) {
        // columns [0,64) gate, [64,128) up of the same 64 outputs
        bf16* dst = g.C + static_cast<size_t>(row) * g.ldc + n_blk * (FN / 2);
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          bf16x8 o;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float g0 = acc[v * 8 + 2 * j], g1 = acc[v * 8 + 2 * j + 1];
            g0 = g0 / (1.f + __expf(-g0));
            g1 = g1 / (1.f + __expf(-g1));
            o.u[j] = pack_bf16x2(g0 * acc[64 + v * 8 + 2 * j], g1 * acc[64 + v * 8 + 2 * j + 1]);
          }
          if (n_blk * (FN / 2) + v * 8 < g.N / 2) st_bf16x8(dst + v * 8, o);
        }
      } else {
        const size_t off = static_cast<size_t>(row) * g.ldc + n_blk * FN;
#pragma unroll
        for (int v = 0; v < 16; ++v) {
          if (n_blk * FN + v * 8 >= g.N) continue;
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = acc[v * 8 + j];
          if (g.epi == PXL_EPI_RESIDUAL) {
            const bf16x8 rr = ld_bf16x8(g.residual + off + v * 8);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 t2 = unpack_bf16x2(rr.u[j]);
              f[2 * j] += t2.x;
              f[2 * j + 1] += t2.y;
            }
          }
          bf16x8 o;
#pragma unroll
          for (int j = 0; j < 4; ++j) o.u[j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
          st_bf16x8(g.C + off + v * 8, o);
        }
      }
    }
  }

  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * FN);
}

// one warp per row: amax over 128-column groups -> e4m3 + scale
__global__ void __launch_bounds__(128) quant_fp8_rows_kernel(const bf16* __restrict__ x, int64_t ld,
                                                             uint8_t* __restrict__ q, float* __restrict__ s, int T,
                                                             int K) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  const int groups = K / 128;
  for (int gidx = 0; gidx < groups; ++gidx) {
    const bf16* src = x + row * ld + gidx * 128 + lane * 4;
    float v[4];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] = __bfloat162float(src[j]);
      amax = fmaxf(amax, fabsf(v[j]));
    }
    amax = warp_reduce_max(amax);
    const float scale = fmaxf(amax, 1e-12f) / 448.f;
    const float inv = 1.f / scale;
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, __NV_E4M3);
      packed |= static_cast<uint32_t>(b) << (8 * j);
    }
    *reinterpret_cast<uint32_t*>(q + static_cast<size_t>(row) * K + gidx * 128 + lane * 4) = packed;
    if (lane == 0) s[static_cast<size_t>(row) * groups + gidx] = scale;
  }
}

int launch_fp8(const void* A, const void* W, const Fp8Args& g, uint64_t a_rows, uint64_t w_rows, int lda, int ldw,
               int tiles, int* status, cudaStream_t stream) {
  CUtensorMap ta, tb;
  if (!pxl_host::make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, a_rows, g.K, lda, FM, FK)) return PXL_ERR_TENSORMAP;
  if (!pxl_host::make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, w_rows, g.K, ldw, FN, FK)) return PXL_ERR_TENSORMAP;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM) != cudaSuccess)
      return PXL_ERR_CUDA;
    configured[dev] = true;
  }
  gemm_fp8_kernel<<<tiles, F_THREADS, F_SMEM, stream>>>(ta, tb, g, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

}  // namespace

PXL_EXPORT int pxl_gemm_fp8_block(const void* A, const float* a_s, const void* W, const float* w_s, void* C,
                                  const void* residual, int M, int N, int K, int lda, int ldw, int ldc, int epi,
                                  int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return PXL_ERR_INVALID_ARG;
  if ((K % FK) || (N % FN) || (lda % 16) || (ldw % 16) || (ldc % 8)) return PXL_ERR_INVALID_ARG;
  if (epi != PXL_EPI_NONE && epi != PXL_EPI_RESIDUAL && epi != PXL_EPI_SILU_MUL) return PXL_ERR_INVALID_ARG;
  if (epi == PXL_EPI_RESIDUAL && residual == nullptr) return PXL_ERR_INVALID_ARG;
  if (epi == PXL_EPI_SILU_MUL && (N % FN)) return PXL_ERR_INVALID_ARG;
  Fp8Args g{};
  g.a_s = a_s; g.w_s = w_s; g.C = static_cast<pxl::bf16*>(C); g.residual = static_cast<const pxl::bf16*>(residual);
  g.ldc = ldc; g.M = M; g.N = N; g.K = K; g.epi = epi;
  const int tiles = pxl::ceil_div(M, FM) * pxl::ceil_div(N, FN);
  return launch_fp8(A, W, g, M, N, lda, ldw, tiles, status, stream);
}

PXL_EXPORT int pxl_gemm_fp8_block_grouped(const void* A, const float* a_s, const void* W, const float* w_s, void* C,
                                          int P, int E, int N, int K, int lda, int ldw, int ldc,
                                          const int* mt_expert, const int* mt_row0, const int* mt_row_end,
                                          const int* num_mt, int max_m_tiles, int epi, int* status,
                                          cudaStream_t stream) {
  if (P <= 0 || E <= 0 || N <= 0 || K <= 0 || max_m_tiles <= 0) return PXL_ERR_INVALID_ARG;
  if ((K % FK) || (N % FN) || (lda % 16) || (ldw % 16) || (ldc % 8)) return PXL_ERR_INVALID_ARG;
  if (epi != PXL_EPI_NONE && epi != PXL_EPI_SILU_MUL) return PXL_ERR_INVALID_ARG;
  Fp8Args g{};
  g.a_s = a_s; g.w_s = w_s; g.C = static_cast<pxl::bf16*>(C);
  g.ldc = ldc; g.M = P; g.N = N; g.K = K; g.epi = epi;
  g.mt_expert = mt_expert; g.mt_row0 = mt_row0; g.mt_row_end = mt_row_end; g.num_mt = num_mt;
  g.w_rows_per_expert = N;
  const int tiles = max_m_tiles * (N / FN);
  return launch_fp8(A, W, g, P, static_cast<uint64_t>(E) * N, lda, ldw, tiles, status, stream);
}

PXL_EXPORT int pxl_quant_fp8_rows(const void* x, int64_t ld, void* q, float* scales, int T, int K,
                                  cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (K % 128) return PXL_ERR_INVALID_ARG;
  quant_fp8_rows_kernel<<<pxl::ceil_div(T, 4), 128, 0, stream>>>(static_cast<const pxl::bf16*>(x), ld,
                                                                static_cast<uint8_t*>(q), scales, T, K);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}
