// bf16 GEMM on the 5th-generation tensor cores:  C[M,N] = A[M,K] * W[N,K]^T (+ epilogue)
//
// Design (one persistent CTA per SM, 6 warps):
//   warp 0   : TMA producer. One elected lane streams 128xBK A tiles and BNxBK W
//              tiles (both K-major, 128-byte swizzle) through a ring of shared-memory
//              stages guarded by full/empty mbarriers.
//   warp 1   : MMA issuer. One elected lane issues tcgen05.mma (M=128, N=BN, K=16)
//              straight from shared memory into a TMEM accumulator; tcgen05.commit
//              releases the smem stage / publishes the finished accumulator.
//   warps 2-5: epilogue. Each warp owns one 32-lane quarter of TMEM, reads the fp32
//              accumulator with tcgen05.ld, applies the fused epilogue and stores bf16.
// Two accumulators (2*BN TMEM columns) let the epilogue of tile i overlap the MMAs of
// tile i+1. Every mbarrier wait is time-bounded: on expiry the kernel records an error
// code in the status word, unwinds all roles, frees its TMEM and returns.
//
// Covers the dense projections reached through the reference's GPU backend
// (src/parallax/sglang/model_runner.py:358-366; the reference itself ships no GPU GEMM).
#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;
constexpr int A_STAGE_BYTES = BM * BK * 2;

template <int BN>
struct GemmCfg {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGES = (192 * 1024) / (A_STAGE_BYTES + B_STAGE_BYTES);
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = 1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 256;
};

struct GemmEpilogueArgs {
  bf16* C;
  const bf16* residual;  // EPI_RESIDUAL: same shape/stride as C
  const bf16* bias;      // optional, length N (pre-activation columns)
  float* C_f32;          // EPI_F32 output
  int ldc;
};

// Grouped (per-expert) mode: the m-tiles are listed on the device, one entry per 128-row
// tile of an expert's segment of the permuted activation matrix. num_mt == nullptr selects
// the plain dense mode.
struct GemmGroupArgs {
  const int* mt_expert;    // expert id of m-tile i
  const int* mt_row0;      // first row of m-tile i in A / C
  const int* mt_row_end;   // end (exclusive) of the expert's segment: rows beyond are not stored
  const int* num_mt;       // number of m-tiles (device scalar)
  int w_rows_per_expert;   // rows of W per expert (N of one expert's matrix)
};

struct TileCoord {
  int a_row, b_row, row_end, n_blk;
};

template <int BN>
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n, int M,
                                                const GemmGroupArgs& g) {
  TileCoord c;
  if (g.num_mt != nullptr) {
    const int mt = tile / num_n;
    c.n_blk = tile % num_n;
    c.a_row = g.mt_row0[mt];
    c.row_end = g.mt_row_end[mt];
    c.b_row = g.mt_expert[mt] * g.w_rows_per_expert + c.n_blk * BN;
  } else {
    const int m_blk = tile % num_m;
    c.n_blk = tile / num_m;
    c.a_row = m_blk * BM;
    c.row_end = M;
    c.b_row = c.n_blk * BN;
  }
  return c;
}

template <int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b, GemmEpilogueArgs ep,
                         GemmGroupArgs grp, int M, int N, int K, int* status) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_b + STAGES * Cfg::B_STAGE_BYTES);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + STAGES);
  const uint32_t tfull0 = smem_u32(bars + 2 * STAGES);
  const uint32_t tempty0 = smem_u32(bars + 2 * STAGES + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = grp.num_mt != nullptr ? *grp.num_mt : ceil_div(M, BM);
  const int num_n = ceil_div(N, BN);
  const int num_tiles = num_m * num_n;
  const int num_kb = ceil_div(K, BK);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 4);  // one arrival per epilogue warp
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord tc = tile_coord<BN>(tile, num_m, num_n, M, grp);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1, abort_flag, status,
                                 PXL_DEV_TIMEOUT_EMPTY);
          if (!ok) break;
          const uint32_t fb = full0 + 8 * stage;
          mbar_arrive_expect_tx(fb, A_STAGE_BYTES + Cfg::B_STAGE_BYTES);
          tma_load_2d(smem_u32(smem_a + stage * A_STAGE_BYTES), &tmap_a, fb, kb * BK, tc.a_row);
          tma_load_2d(smem_u32(smem_b + stage * Cfg::B_STAGE_BYTES), &tmap_b, fb, kb * BK,
                      tc.b_row);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        ok = mbar_wait_bounded(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag, status,
                               PXL_DEV_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag, status,
                                 PXL_DEV_TIMEOUT_FULL);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + stage * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(smem_b + stage * Cfg::B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = umma_desc_k_sw128(a_addr + k * UMMA_K * 2);
            const uint64_t db = umma_desc_k_sw128(b_addr + k * UMMA_K * 2);
            tc_mma_f16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(empty0 + 8 * stage);  // stage reusable once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit(tfull0 + 8 * acc);  // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const TileCoord tc = tile_coord<BN>(tile, num_m, num_n, M, grp);
      const int n_blk = tc.n_blk;
      const int M_end = tc.row_end;
      ok = mbar_wait_bounded(tfull0 + 8 * acc, acc_phase, abort_flag, status,
                             PXL_DEV_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tc.a_row + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      if constexpr (EPI == PXL_EPI_SILU_MUL) {
        // W rows come in groups of 128: 64 gate rows then the 64 up rows of the same outputs
        const int n_out = N / 2;
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          const int grp = c / 64, cin = c % 64;
          const int out_col = n_blk * (BN / 2) + c;
          uint32_t g[32], u[32];
          tmem_ld_32x32b_x32(t_row + grp * 128 + cin, g);
          tmem_ld_32x32b_x32(t_row + grp * 128 + 64 + cin, u);
          tmem_ld_wait();
          if (row < M_end) {
            bf16* dst = ep.C + static_cast<size_t>(row) * ep.ldc + out_col;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (out_col + v * 8 < n_out) {
                bf16x8 o;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float g0 = __uint_as_float(g[v * 8 + 2 * j]);
                  float g1 = __uint_as_float(g[v * 8 + 2 * j + 1]);
                  const float u0 = __uint_as_float(u[v * 8 + 2 * j]);
                  const float u1 = __uint_as_float(u[v * 8 + 2 * j + 1]);
                  g0 = g0 / (1.f + __expf(-g0));
                  g1 = g1 / (1.f + __expf(-g1));
                  o.u[j] = pack_bf16x2(g0 * u0, g1 * u1);
                }
                st_bf16x8(dst + v * 8, o);
              }
            }
          }
        }
      } else {
        const int col0 = n_blk * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + c0, r);
          tmem_ld_wait();
          if (row < M_end) {
            const size_t off = static_cast<size_t>(row) * ep.ldc + col0 + c0;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = col0 + c0 + v * 8;
              if (col < N) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
                if (ep.bias) {
                  const bf16x8 b = ld_bf16x8(ep.bias + col);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 bb = unpack_bf16x2(b.u[j]);
                    f[2 * j] += bb.x;
                    f[2 * j + 1] += bb.y;
                  }
                }
                if constexpr (EPI == PXL_EPI_RESIDUAL) {
                  const bf16x8 rr = ld_bf16x8(ep.residual + off + v * 8);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 bb = unpack_bf16x2(rr.u[j]);
                    f[2 * j] += bb.x;
                    f[2 * j + 1] += bb.y;
                  }
                }
                if constexpr (EPI == PXL_EPI_F32) {
                  float4* d4 = reinterpret_cast<float4*>(ep.C_f32 + off + v * 8);
                  d4[0] = make_float4(f[0], f[1], f[2], f[3]);
                  d4[1] = make_float4(f[4], f[5], f[6], f[7]);
                } else {
                  bf16x8 o;
#pragma unroll
                  for (int j = 0; j < 4; ++j) o.u[j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
                  st_bf16x8(ep.C + off + v * 8, o);
                }
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_flag) {
    // give loads that are still in flight time to land before the smem is released
    __nanosleep(200000);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

template <int BN, int EPI>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmEpilogueArgs& ep,
                const GemmGroupArgs& grp, int max_tiles, int M, int N, int K, int* status,
                cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, EPI>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) !=
        cudaSuccess)
      return PXL_ERR_CUDA;
    configured[dev] = true;
  }
  const int tiles = max_tiles > 0 ? max_tiles : pxl::ceil_div(M, BM) * pxl::ceil_div(N, BN);
  const int grid = tiles < pxl_host::num_sms() ? tiles : pxl_host::num_sms();
  kern<<<grid, kGemmThreads, Cfg::SMEM_BYTES, stream>>>(ta, tb, ep, grp, M, N, K, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

template <int BN>
int dispatch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const GemmEpilogueArgs& ep,
                 const GemmGroupArgs& grp, int max_tiles, int M, int N, int K, int* status,
                 cudaStream_t stream) {
#define PXL_GEMM_CASE(E) \
  case E: return launch_gemm<BN, E>(ta, tb, ep, grp, max_tiles, M, N, K, status, stream)
  switch (epi) {
    PXL_GEMM_CASE(PXL_EPI_NONE);
    PXL_GEMM_CASE(PXL_EPI_RESIDUAL);
    PXL_GEMM_CASE(PXL_EPI_SILU_MUL);
    PXL_GEMM_CASE(PXL_EPI_F32);
    default: return PXL_ERR_INVALID_ARG;
  }
#undef PXL_GEMM_CASE
}

}  // namespace

// Tile width heuristic: the widest tile that still yields at least one tile per SM;
// below that the narrowest, so that small-M (decode) problems spread their weight
// traffic over as many SMs as possible.
PXL_EXPORT int pxl_gemm_bf16_pick_bn(int M, int N, int epi) {
  const int sms = pxl_host::num_sms();
  const int num_m = pxl::ceil_div(M, BM);
  const int cands[3] = {256, 128, 64};
  for (int i = 0; i < 3; ++i) {
    const int bn = cands[i];
    if (epi == PXL_EPI_SILU_MUL && ((N % bn) != 0 || bn < 128)) continue;
    if (num_m * pxl::ceil_div(N, bn) >= sms) return bn;
  }
  return epi == PXL_EPI_SILU_MUL ? 128 : 64;
}

PXL_EXPORT int pxl_gemm_bf16(const void* A, const void* W, void* C, const void* residual,
                             const void* bias, int M, int N, int K, int lda, int ldw, int ldc,
                             int epi, int bn, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return PXL_ERR_INVALID_ARG;
  if ((K % 8) || (lda % 8) || (ldw % 8) || (ldc % 8) || (N % 8)) return PXL_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) |
       reinterpret_cast<uintptr_t>(C)) & 15)
    return PXL_ERR_INVALID_ARG;
  if (epi == PXL_EPI_RESIDUAL && residual == nullptr) return PXL_ERR_INVALID_ARG;
  if (bn == 0) bn = pxl_gemm_bf16_pick_bn(M, N, epi);
  if (epi == PXL_EPI_SILU_MUL && ((N % bn) != 0 || bn < 128)) return PXL_ERR_INVALID_ARG;

  CUtensorMap ta, tb;
  if (!pxl_host::make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, M, K, lda, BM, BK))
    return PXL_ERR_TENSORMAP;
  if (!pxl_host::make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, N, K, ldw, bn, BK))
    return PXL_ERR_TENSORMAP;
  GemmEpilogueArgs ep;
  ep.C = static_cast<pxl::bf16*>(C);
  ep.C_f32 = static_cast<float*>(C);
  ep.residual = static_cast<const pxl::bf16*>(residual);
  ep.bias = static_cast<const pxl::bf16*>(bias);
  ep.ldc = ldc;
  GemmGroupArgs grp{nullptr, nullptr, nullptr, nullptr, 0};
  switch (bn) {
    case 256: return dispatch_epi<256>(epi, ta, tb, ep, grp, 0, M, N, K, status, stream);
    case 128: return dispatch_epi<128>(epi, ta, tb, ep, grp, 0, M, N, K, status, stream);
    case 64: return dispatch_epi<64>(epi, ta, tb, ep, grp, 0, M, N, K, status, stream);
    default: return PXL_ERR_INVALID_ARG;
  }
}

// Grouped GEMM over experts: for every m-tile i listed on the device,
//   C[rows of tile i, :] = A[rows of tile i, :] * W[expert_i]^T
// A: [P, K] activations permuted so that each expert's tokens are contiguous; W: [E*N, K]
// (expert matrices stacked); C: [P, N] (N/2 columns with PXL_EPI_SILU_MUL).
// max_m_tiles bounds the device-side count and sizes the grid.
PXL_EXPORT int pxl_gemm_bf16_grouped(const void* A, const void* W, void* C, int P, int E, int N,
                                     int K, int lda, int ldw, int ldc, const int* mt_expert,
                                     const int* mt_row0, const int* mt_row_end, const int* num_mt,
                                     int max_m_tiles, int epi, int bn, int* status,
                                     cudaStream_t stream) {
  if (P <= 0 || E <= 0 || N <= 0 || K <= 0 || max_m_tiles <= 0) return PXL_ERR_INVALID_ARG;
  if ((K % 8) || (lda % 8) || (ldw % 8) || (ldc % 8) || (N % 8)) return PXL_ERR_INVALID_ARG;
  if (epi == PXL_EPI_RESIDUAL) return PXL_ERR_INVALID_ARG;
  if (bn == 0) bn = (N % 256 == 0 && N >= 1024) ? 256 : 128;
  if (N % bn) return PXL_ERR_INVALID_ARG;  // a tile must not straddle two experts' rows of W
  CUtensorMap ta, tb;
  if (!pxl_host::make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, P, K, lda, BM, BK))
    return PXL_ERR_TENSORMAP;
  if (!pxl_host::make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W,
                              static_cast<uint64_t>(E) * N, K, ldw, bn, BK))
    return PXL_ERR_TENSORMAP;
  GemmEpilogueArgs ep;
  ep.C = static_cast<pxl::bf16*>(C);
  ep.C_f32 = static_cast<float*>(C);
  ep.residual = nullptr;
  ep.bias = nullptr;
  ep.ldc = ldc;
  GemmGroupArgs grp{mt_expert, mt_row0, mt_row_end, num_mt, N};
  const int max_tiles = max_m_tiles * pxl::ceil_div(N, bn);
  switch (bn) {
    case 256: return dispatch_epi<256>(epi, ta, tb, ep, grp, max_tiles, P, N, K, status, stream);
    case 128: return dispatch_epi<128>(epi, ta, tb, ep, grp, max_tiles, P, N, K, status, stream);
    case 64: return dispatch_epi<64>(epi, ta, tb, ep, grp, max_tiles, P, N, K, status, stream);
    default: return PXL_ERR_INVALID_ARG;
  }
}
