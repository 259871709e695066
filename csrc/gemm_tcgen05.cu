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
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int kAgChunkRows = 8;                     // rows per all-gather copy chunk
constexpr int kAgChunksPerTile = BM / kAgChunkRows;  // flags per 128-row tile

template <int BN>
struct GemmCfg {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGES = (192 * 1024) / (A_STAGE_BYTES + B_STAGE_BYTES);
  // two accumulators; tensor memory is allocated in powers of two (384 columns round up to 512)
  static constexpr int TMEM_COLS = 2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512);
  static constexpr int SMEM_BYTES = 1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 256;
};

// Reduce-scatter epilogue staging: one 128-byte line (64 bf16) per accumulator row, padded to
// 144 bytes so that the 16-byte vector stores of a quarter-warp fall into distinct banks.
constexpr int kRsLinePitch = 144;
constexpr int kRsStageBytes = BM * kRsLinePitch;
template <int BN, int EPI>
constexpr int gemm_smem_bytes() {
  return GemmCfg<BN>::SMEM_BYTES + ((EPI == PXL_EPI_RS || EPI == PXL_EPI_SCATTER) ? kRsStageBytes : 0);
}

struct GemmEpilogueArgs {
  bf16* C;
  const bf16* residual;  // EPI_RESIDUAL: same shape/stride as C
  const bf16* bias;      // optional, length N (pre-activation columns)
  float* C_f32;          // EPI_F32 output
  int ldc;
  bf16* const* row_ptrs; // EPI_SCATTER: destination of every output row (null = drop), N elements each
  uint32_t* done_counter;  // EPI_SCATTER: local counter for the "last CTA publishes the flags" step
  // EPI_SPLITK_T (operands swapped: accumulator row = output column, accumulator column = token)
  float* ws;                 // [splitk][tokens][ldws] fp32 partial sums, one slab per K range
  uint32_t* tile_counters;   // one per 128 output columns, zero between launches
  int splitk, ldws;
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

// Fused collectives (tensor parallelism inside a pipeline stage). All pointers in the arrays
// are peer-mapped symmetric-memory addresses, index = rank.
//  * reduce-scatter epilogue (EPI == PXL_EPI_RS): the tile of partial sums is stored straight
//    into the staging slot [this rank] of the rank that owns the tile's rows, then a flag is
//    published; after its own tiles every CTA reduces owned tiles whose tp partials arrived.
//  * all-gather prologue (ag_ncopy > 0): the last ag_ncopy CTAs pull the other ranks' row
//    shards of A into this GPU's copy of the full matrix and publish one flag per 128-row
//    tile; the TMA producer waits for a tile's flag before loading it.
struct GemmCommArgs {
  bf16* stage[8];            // RS: [tp][rows_per_rank][ldc] staging buffer of rank i
  uint32_t* flags[8];        // RS: [tp][tiles_per_shard] arrival flags of rank i
  const bf16* ag_src[8];     // AG: rank i's copy of the full A matrix [tp*rows_per_rank][lda]
  uint32_t* ag_ready[8];     // AG: [tp] "shard of rank j is complete" flags of rank i
  uint32_t* ag_tile_flags;   // AG: local [num_m_tiles] flags, set when a tile has landed
  bf16* ag_dst;              // AG: this rank's copy of the full A matrix (written by copy CTAs)
  bf16* out;                 // RS: local result [rows_per_rank][ldo]
  const bf16* residual;      // RS: optional local residual shard [rows_per_rank][ldo]
  int rank, tp, rows_per_rank, ldo, lda, ag_ncopy, first_shard;
  uint32_t epoch;
};

struct TileCoord {
  int a_row, b_row, row_end, n_blk;
};

template <int BN>
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n, int M,
                                                const GemmGroupArgs& g, const GemmCommArgs& comm) {
  TileCoord c;
  if (g.num_mt != nullptr) {
    const int mt = tile / num_n;
    c.n_blk = tile % num_n;
    c.a_row = g.mt_row0[mt];
    c.row_end = g.mt_row_end[mt];
    c.b_row = g.mt_expert[mt] * g.w_rows_per_expert + c.n_blk * BN;
  } else {
    int m_blk;
    if (comm.tp > 1) {
      // fused-collective order: one row shard after the other, starting at comm.first_shard,
      // so that every rank computes (and ships / needs) a different shard at any moment
      const int mps = comm.rows_per_rank / BM;
      const int per_shard = mps * num_n;
      const int within = tile % per_shard;
      const int shard = (comm.first_shard + tile / per_shard) % comm.tp;
      m_blk = shard * mps + within % mps;
      c.n_blk = within / mps;
    } else {
      m_blk = tile % num_m;
      c.n_blk = tile / num_m;
    }
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
                         GemmGroupArgs grp, const __grid_constant__ GemmCommArgs comm, int M, int N,
                         int K, int* status) {
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
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);  // split-K: this CTA finishes the tile
  // reduce-scatter epilogue staging lines (allocated only for that epilogue)
  uint8_t* rs_stage = smem_b + STAGES * Cfg::B_STAGE_BYTES + 256;

  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + STAGES);
  const uint32_t tfull0 = smem_u32(bars + 2 * STAGES);
  const uint32_t tempty0 = smem_u32(bars + 2 * STAGES + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int gemm_ctas = gridDim.x - comm.ag_ncopy;
  if (comm.ag_ncopy > 0 && static_cast<int>(blockIdx.x) >= gemm_ctas) {
    // ---------------------------------------------------------- all-gather copy CTA
    // One warp per copy CTA drives the TMA engine: chunks of kAgChunkRows rows are pulled from
    // the peer's shard into this CTA's shared memory with untiled bulk copies (a whole chunk
    // in flight per buffer, up to three buffers) and written to the local full matrix with
    // bulk stores. Chunks of a shard are dealt round-robin to the copy CTAs so that all of
    // them work on the first tiles first; one flag per chunk tells the producer what landed.
    __shared__ uint64_t cbar[3];
    __shared__ int c_abort;
    pdl_wait();
    pdl_launch_dependents();
    if (warp != 0) return;
    const int c = blockIdx.x - gemm_ctas;
    if (lane == 0) {
      c_abort = 0;
      for (int i = 0; i < 3; ++i) mbar_init(smem_u32(&cbar[i]), 1);
      mbar_fence_init();
      fence_proxy_async_smem();
    }
    __syncwarp();
    if (c == 0 && lane < comm.tp) {
      // this rank's shard is complete (the launch is ordered after its producer): tell everyone
      __threadfence_system();
      st_release_sys_u32(comm.ag_ready[lane] + comm.rank, comm.epoch);
    }
    const uint32_t row_bytes = static_cast<uint32_t>(K) * 2u;
    const uint32_t chunk_bytes = kAgChunkRows * row_bytes;
    int nbuf = static_cast<int>((192u * 1024u) / chunk_bytes);
    nbuf = nbuf > 3 ? 3 : nbuf;  // the host rejects K for which not even one chunk fits
    const int chunks_per_shard = comm.rows_per_rank / kAgChunkRows;
    const uint32_t smem0 = smem_u32(smem);
    int n_issue = 0, n_done = 0;  // sequence numbers: buffer = n % nbuf, parity = (n / nbuf) & 1
    bool ok = true;
    for (int step = 1; ok && step < comm.tp; ++step) {
      const int src = (comm.rank + step) % comm.tp;
      int okf = 1;
      if (lane == 0)
        okf = flag_wait_bounded<true>(comm.ag_ready[comm.rank] + src, comm.epoch, nullptr, status) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, okf, 0) != 0;
      if (!ok) break;
      const bf16* sbase = comm.ag_src[src] + static_cast<size_t>(src) * comm.rows_per_rank * comm.lda;
      bf16* dbase = comm.ag_dst + static_cast<size_t>(src) * comm.rows_per_rank * comm.lda;
      auto issue_load = [&](int chunk) {
        const int buf = n_issue % nbuf;
        const uint32_t bar = smem_u32(&cbar[buf]);
        if (lane == 0) mbar_arrive_expect_tx(bar, chunk_bytes);
        __syncwarp();
        if (lane < kAgChunkRows)
          bulk_load_g2s(smem0 + buf * chunk_bytes + lane * row_bytes,
                        sbase + static_cast<size_t>(chunk * kAgChunkRows + lane) * comm.lda, row_bytes, bar);
        ++n_issue;
      };
      int next = c, cur = c;
      while (n_issue - n_done < nbuf && next < chunks_per_shard) {
        issue_load(next);
        next += comm.ag_ncopy;
      }
      while (cur < chunks_per_shard) {
        const int buf = n_done % nbuf;
        if (lane == 0)
          okf = mbar_wait_bounded(smem_u32(&cbar[buf]), (n_done / nbuf) & 1, &c_abort, status,
                                  PXL_DEV_TIMEOUT_FULL) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, okf, 0) != 0;
        if (!ok) break;
        if (lane < kAgChunkRows) {
          bulk_store_s2g(dbase + static_cast<size_t>(cur * kAgChunkRows + lane) * comm.lda,
                         smem0 + buf * chunk_bytes + lane * row_bytes, row_bytes);
          bulk_commit();
          bulk_wait_read_all();
        }
        __syncwarp();
        ++n_done;
        if (next < chunks_per_shard) {  // refill the buffer that was just drained
          issue_load(next);
          next += comm.ag_ncopy;
        }
        if (lane < kAgChunkRows) bulk_wait_all();
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          const int row0 = src * comm.rows_per_rank + cur * kAgChunkRows;
          st_release_gpu_u32(comm.ag_tile_flags + (row0 / BM) * kAgChunksPerTile + (row0 % BM) / kAgChunkRows,
                             comm.epoch);
        }
        cur += comm.ag_ncopy;
      }
    }
    if (!ok) {
      // loads that are still in flight must land before this CTA's shared memory is released
      for (int i = 0; i < 64; ++i) __nanosleep(20000);
    }
    return;
  }

  const int num_m = grp.num_mt != nullptr ? *grp.num_mt : ceil_div(M, BM);
  const int num_n = ceil_div(N, BN);
  const int num_tiles = num_m * num_n;
  const int num_kb = ceil_div(K, BK);
  // split-K (small-M path only): work item = (tile, K range); every range holds at least one k-block
  constexpr bool kCluster = EPI == PXL_EPI_SPLITK_C || EPI == PXL_EPI_SPLITK_CN;
  constexpr bool kSplit = EPI == PXL_EPI_SPLITK_T || kCluster;
  const int splitk = kSplit ? ep.splitk : 1;
  const int kb_per = ceil_div(num_kb, splitk);
  const int num_items = num_tiles * splitk;
  // item -> (tile, K range). Cluster variant: the CTAs of a cluster (consecutive block ids) share a
  // tile, the cluster rank is the K range, and the grid holds exactly one CTA per item.
  auto item_tile = [&](int item) { return kCluster ? item / splitk : item % num_tiles; };
  auto item_ks = [&](int item) { return kCluster ? item % splitk : item / num_tiles; };
  bool acc_ready = false;  // cluster variant: this CTA's accumulator is complete

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
  // everything above touched only this CTA's shared and tensor memory: with a programmatic dependent
  // launch it overlaps the tail of the previous kernel, whose results are needed from here on
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gemm_ctas) {
        const int tile = item_tile(item);
        const int kb0 = item_ks(item) * kb_per;
        const int kb1 = kb0 + kb_per < num_kb ? kb0 + kb_per : num_kb;
        const TileCoord tc = tile_coord<BN>(tile, num_m, num_n, M, grp, comm);
        if (comm.ag_ncopy > 0 && tc.a_row / comm.rows_per_rank != comm.rank) {
          // rows of another rank: wait until the copy CTAs have landed this tile locally
          const uint32_t* tf = comm.ag_tile_flags + (tc.a_row / BM) * kAgChunksPerTile;
          for (int ch = 0; ok && ch < kAgChunksPerTile; ++ch)
            ok = flag_wait_bounded<false>(tf + ch, comm.epoch, abort_flag, status);
          if (!ok) break;
          fence_proxy_async_all();
        }
        for (int kb = kb0; kb < kb1; ++kb) {
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
      for (int item = blockIdx.x; ok && item < num_items; item += gemm_ctas) {
        const int kb0 = item_ks(item) * kb_per;
        const int kb1 = kb0 + kb_per < num_kb ? kb0 + kb_per : num_kb;
        ok = mbar_wait_bounded(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag, status,
                               PXL_DEV_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
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
            tc_mma_f16(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
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
    for (int item = blockIdx.x; ok && item < num_items; item += gemm_ctas) {
      const int tile = item_tile(item);
      const TileCoord tc = tile_coord<BN>(tile, num_m, num_n, M, grp, comm);
      const int n_blk = tc.n_blk;
      const int M_end = tc.row_end;
      ok = mbar_wait_bounded(tfull0 + 8 * acc, acc_phase, abort_flag, status,
                             PXL_DEV_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      if constexpr (kCluster) {
        acc_ready = true;  // drained after the cluster barrier below
        break;
      }
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
      } else if constexpr (EPI == PXL_EPI_RS || EPI == PXL_EPI_SCATTER) {
        // RS: partial sums go to the staging slot [this rank] of the rank that owns the rows.
        // SCATTER: every row has its own destination (a row of a peer's combine buffer).
        // Each lane packs 64 columns of its row into its private 128-byte line of shared memory and
        // ships the line with one bulk store: NVLink sees 128-byte writes instead of 16-byte ones.
        const int col0 = n_blk * BN;
        bf16* dst_row;
        if constexpr (EPI == PXL_EPI_RS) {
          const int owner = row / comm.rows_per_rank;
          const int lrow = row - owner * comm.rows_per_rank;
          dst_row = comm.stage[owner] +
                    (static_cast<size_t>(comm.rank) * comm.rows_per_rank + lrow) * ep.ldc + col0;
        } else {
          dst_row = row < M_end ? ep.row_ptrs[row] : nullptr;
          if (dst_row != nullptr) dst_row += col0;
        }
        const uint32_t line = smem_u32(rs_stage) + (q * 32 + lane) * kRsLinePitch;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(t_row + c0, r0);
          tmem_ld_32x32b_x32(t_row + c0 + 32, r1);
          bulk_wait_read_all();  // the previous bulk store has read this lane's line
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(line + v * 16),
                         "r"(pack_bf16x2(__uint_as_float(r0[v * 8 + 0]), __uint_as_float(r0[v * 8 + 1]))),
                         "r"(pack_bf16x2(__uint_as_float(r0[v * 8 + 2]), __uint_as_float(r0[v * 8 + 3]))),
                         "r"(pack_bf16x2(__uint_as_float(r0[v * 8 + 4]), __uint_as_float(r0[v * 8 + 5]))),
                         "r"(pack_bf16x2(__uint_as_float(r0[v * 8 + 6]), __uint_as_float(r0[v * 8 + 7])))
                         : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(line + 64 + v * 16),
                         "r"(pack_bf16x2(__uint_as_float(r1[v * 8 + 0]), __uint_as_float(r1[v * 8 + 1]))),
                         "r"(pack_bf16x2(__uint_as_float(r1[v * 8 + 2]), __uint_as_float(r1[v * 8 + 3]))),
                         "r"(pack_bf16x2(__uint_as_float(r1[v * 8 + 4]), __uint_as_float(r1[v * 8 + 5]))),
                         "r"(pack_bf16x2(__uint_as_float(r1[v * 8 + 6]), __uint_as_float(r1[v * 8 + 7])))
                         : "memory");
          }
          fence_proxy_async_smem();
          if (row < M_end && col0 + c0 < N && dst_row != nullptr) bulk_store_s2g(dst_row + c0, line, 128);
          bulk_commit();
        }
      } else if constexpr (EPI == PXL_EPI_SPLITK_T) {
        // operands swapped: this thread's accumulator row is output column `row`, accumulator
        // column j is token j (N = number of tokens). Every K range has its own slab of the
        // scratch, so the sums are formed in a fixed order; a warp stores 32 neighbouring floats.
        float* slab = ep.ws + static_cast<size_t>(item_ks(item)) * N * ep.ldws;
#pragma unroll 1
        for (int c0 = 0; c0 < BN && c0 < N; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + c0, r);
          tmem_ld_wait();
          if (row < M_end) {
            float* w = slab + static_cast<size_t>(c0) * ep.ldws + row;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < N) __stcg(w + static_cast<size_t>(j) * ep.ldws, __uint_as_float(r[j]));
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
            size_t off = static_cast<size_t>(row) * ep.ldc + col0 + c0;
            bf16* c_base = ep.C;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = col0 + c0 + v * 8;
              if (col < N) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
                if (ep.bias) {
                  // indexed by the row of W: with grouped experts every expert has its own bias
                  const bf16x8 b = ld_bf16x8(ep.bias + tc.b_row + c0 + v * 8);
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
                  st_bf16x8(c_base + off + v * 8, o);
                }
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
      if constexpr (EPI == PXL_EPI_SPLITK_T) {
        // the CTA whose partial sums arrive last adds the slabs of the tile in K order (+ bias,
        // + residual), writes bf16 and resets the tile's counter for the next launch
        __threadfence();
        named_bar_sync(1, 128);
        if (threadIdx.x == 64) {
          const uint32_t old = atomicAdd(ep.tile_counters + tile, 1u);
          const int last = old == static_cast<uint32_t>(splitk - 1) ? 1 : 0;
          if (last) ep.tile_counters[tile] = 0;
          *last_flag = last;
        }
        named_bar_sync(1, 128);
        if (*last_flag) {
          __threadfence();
          // four outputs (of four floats) per thread and up to four K ranges per round: sixteen
          // independent loads are in flight before the first add, always summed in K order
          const size_t slab_stride = static_cast<size_t>(N) * ep.ldws;
          const int n_items = N * 32;
          constexpr int U = 4;
          for (int i0 = threadIdx.x - 64; i0 < n_items; i0 += 128 * U) {
            const float* wp[U];
            size_t c_off[U];
            int col[U];
            bool valid[U];
            float4 acc[U];
            uint2 res[U], bia[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int i = i0 + u * 128;
              const int t = i >> 5;
              col[u] = tc.a_row + (i & 31) * 4;
              valid[u] = i < n_items && col[u] < M_end;
              wp[u] = ep.ws + static_cast<size_t>(t) * ep.ldws + col[u];
              c_off[u] = static_cast<size_t>(t) * ep.ldc + col[u];
              acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
              res[u] = make_uint2(0u, 0u);
              bia[u] = make_uint2(0u, 0u);
              if (valid[u] && ep.residual) res[u] = *reinterpret_cast<const uint2*>(ep.residual + c_off[u]);
              if (valid[u] && ep.bias) bia[u] = *reinterpret_cast<const uint2*>(ep.bias + col[u]);
            }
            for (int ks = 0; ks < splitk; ks += 4) {
              float4 v[U][4];
#pragma unroll
              for (int u = 0; u < U; ++u) {
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                  v[u][k4] = (valid[u] && ks + k4 < splitk)
                                 ? __ldcg(reinterpret_cast<const float4*>(wp[u] + (ks + k4) * slab_stride))
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
                }
              }
#pragma unroll
              for (int u = 0; u < U; ++u) {
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                  acc[u].x += v[u][k4].x, acc[u].y += v[u][k4].y, acc[u].z += v[u][k4].z, acc[u].w += v[u][k4].w;
                }
              }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
              if (!valid[u]) continue;
              float4 a = acc[u];
              const float2 b0 = unpack_bf16x2(bia[u].x), b1 = unpack_bf16x2(bia[u].y);
              const float2 r0 = unpack_bf16x2(res[u].x), r1 = unpack_bf16x2(res[u].y);
              a.x += b0.x + r0.x, a.y += b0.y + r0.y, a.z += b1.x + r1.x, a.w += b1.y + r1.y;
              if (ep.C_f32 != nullptr) {
                *reinterpret_cast<float4*>(ep.C_f32 + c_off[u]) = a;
              } else {
                uint2 o;
                o.x = pack_bf16x2(a.x, a.y);
                o.y = pack_bf16x2(a.z, a.w);
                *reinterpret_cast<uint2*>(ep.C + c_off[u]) = o;
              }
            }
          }
        }
      }
      if constexpr (EPI == PXL_EPI_RS) {
        // all 128 epilogue threads have stored their rows of the tile: publish it to the owner
        bulk_wait_all();
        __threadfence_system();
        named_bar_sync(1, 128);
        if (threadIdx.x == 64) {
          const int owner = tc.a_row / comm.rows_per_rank;
          const int t_in_shard = ((tc.a_row - owner * comm.rows_per_rank) / BM) * num_n + n_blk;
          st_release_sys_u32(comm.flags[owner] + comm.rank * (comm.rows_per_rank / BM) * num_n + t_in_shard,
                             comm.epoch);
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if constexpr (EPI == PXL_EPI_SCATTER) {
      // every row of this CTA is on its way: the CTA that finishes last tells all peers
      bulk_wait_all();
      __threadfence_system();
      named_bar_sync(1, 128);
      if (threadIdx.x == 64) {
        const uint32_t old = atomicAdd(ep.done_counter, 1u);
        if (old == gridDim.x - 1) {
          *ep.done_counter = 0;
          __threadfence_system();
          for (int r = 0; r < comm.tp; ++r) st_release_sys_u32(comm.flags[r] + comm.rank, comm.epoch);
        }
      }
    }
  }

  if constexpr (EPI == PXL_EPI_SPLITK_C) {
    // ------------------------------------- split-K reduction inside the cluster (DSMEM)
    // Every thread of every CTA passes both cluster barriers, also after a failed wait (all other
    // waits are bounded). Barrier 1: all accumulators of the cluster are complete, so nobody's
    // pipeline stages are in use any more and can receive partial sums: CTA r collects, from every
    // CTA of the cluster, the tokens [r*S, (r+1)*S) as [source][S][128 columns] floats. Barrier 2:
    // the partial sums have landed; each CTA adds its tokens in K order and writes the result.
    __syncwarp();
    cluster_sync_all();
    const uint32_t my_rank = cluster_cta_rank();
    const int n_tok = N;
    const int S = ceil_div(n_tok, splitk);
    const uint32_t recv0 = smem_u32(smem);
    if (warp >= 2 && acc_ready) {
      const int q = warp & 3;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      const uint32_t col_off = (my_rank * S * 128 + q * 32 + lane) * 4;
      int owner = 0, tl = 0;
      uint32_t dst = cluster_map_shared(recv0, 0) + col_off;
#pragma unroll 1
      for (int c0 = 0; c0 < BN && c0 < n_tok; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (c0 + j < n_tok) {
            st_shared_cluster_f32(dst + tl * 512, __uint_as_float(r[j]));
            if (++tl == S) {
              tl = 0;
              ++owner;
              if (owner < splitk) dst = cluster_map_shared(recv0, owner) + col_off;
            }
          }
        }
      }
    }
    tc_fence_before_sync();
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2 && acc_ready) {
      const int tile = blockIdx.x / splitk;
      const int n0 = tile * BM;  // first output column of the tile (num_n == 1)
      const int t0 = my_rank * S;
      const int s_valid = n_tok - t0 < S ? n_tok - t0 : S;
      for (int i = threadIdx.x - 64; i < s_valid * 32; i += 128) {
        const int tl = i >> 5, c4 = (i & 31) * 4;
        const int n = n0 + c4;
        if (n < M) {
          const uint32_t src = recv0 + (tl * 128 + c4) * 4;
          float4 a = ld_shared_f32x4(src);
          for (int r = 1; r < splitk; ++r) {
            const float4 b = ld_shared_f32x4(src + r * S * 512);
            a.x += b.x, a.y += b.y, a.z += b.z, a.w += b.w;
          }
          const size_t c_off = static_cast<size_t>(t0 + tl) * ep.ldc + n;
          if (ep.bias) {
            const uint2 b = *reinterpret_cast<const uint2*>(ep.bias + n);
            const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y);
            a.x += b0.x, a.y += b0.y, a.z += b1.x, a.w += b1.y;
          }
          if (ep.residual) {
            const uint2 b = *reinterpret_cast<const uint2*>(ep.residual + c_off);
            const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y);
            a.x += b0.x, a.y += b0.y, a.z += b1.x, a.w += b1.y;
          }
          if (ep.C_f32 != nullptr) {
            *reinterpret_cast<float4*>(ep.C_f32 + c_off) = a;
          } else {
            uint2 o;
            o.x = pack_bf16x2(a.x, a.y);
            o.y = pack_bf16x2(a.z, a.w);
            *reinterpret_cast<uint2*>(ep.C + c_off) = o;
          }
        }
      }
    }
  }

  if constexpr (EPI == PXL_EPI_SPLITK_CN) {
    // ------------------------- split-K reduction inside the cluster, operands NOT swapped
    // (129 to about a thousand tokens: too few 128-row tiles to fill the SMs, too many rows for the
    // swapped path). Accumulator row = token, column = output column. Reducer r of the cluster owns
    // the columns [r*cs, (r+1)*cs) of the tile; every OTHER CTA sends it those columns of its partial
    // sums as [source][column / 4][128 tokens][4 columns] floats: one 16-byte remote store per thread
    // and four columns, a warp writes 512 contiguous bytes (scalar remote stores cost about as much per
    // instruction and made the exchange the longest phase of the kernel). The reducer's own partial
    // sums never leave its tensor memory. Same barrier protocol as the swapped variant above.
    __syncwarp();
    cluster_sync_all();
    const uint32_t my_rank = cluster_cta_rank();
    const int cs = ceil_div(BN / 8, splitk) * 8;
    const uint32_t recv0 = smem_u32(smem);
    const int q = warp & 3;
    const int trow = q * 32 + lane;  // token row of the tile = this thread's TMEM lane
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    if (warp >= 2 && acc_ready) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        // skip the chunk if it lies entirely in this CTA's own slice
        const int o_first = c0 / cs, o_last = (c0 + 31) / cs;
        if (o_first == static_cast<int>(my_rank) && o_last == static_cast<int>(my_rank)) continue;
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const int col = c0 + 4 * g;
          const int owner = col / cs;
          if (owner != static_cast<int>(my_rank) && owner < splitk) {
            const int cl = col - owner * cs;
            const uint32_t dst = cluster_map_shared(recv0, owner) +
                                 ((my_rank * (cs / 4) + cl / 4) * 128 + trow) * 16;
            st_shared_cluster_f32x4(dst, __uint_as_float(r[4 * g]), __uint_as_float(r[4 * g + 1]),
                                    __uint_as_float(r[4 * g + 2]), __uint_as_float(r[4 * g + 3]));
          }
        }
      }
    }
    tc_fence_before_sync();
    __syncwarp();
    cluster_sync_all();
    tc_fence_after_sync();
    if (warp >= 2 && acc_ready) {
      const int tile = blockIdx.x / splitk;
      const TileCoord tc = tile_coord<BN>(tile, num_m, num_n, M, grp, comm);
      const int row = tc.a_row + trow;
      const int c_begin = my_rank * cs;
      const int c_end = c_begin + cs < BN ? c_begin + cs : BN;
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 8) {
        const int col = tc.n_blk * BN + c;
        uint32_t own[8];
        tmem_ld_32x32b_x8(t_row + c, own);   // warp-collective: every lane takes part
        tmem_ld_wait();
        if (col < N && row < tc.row_end) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(own[j]);
        const int cg = (c - c_begin) / 4;
        for (int r = 0; r < splitk; ++r) {
          if (r == static_cast<int>(my_rank)) continue;
          const uint32_t src = recv0 + ((r * (cs / 4) + cg) * 128 + trow) * 16;
          const float4 a = ld_shared_f32x4(src);
          const float4 b = ld_shared_f32x4(src + 128 * 16);
          f[0] += a.x, f[1] += a.y, f[2] += a.z, f[3] += a.w;
          f[4] += b.x, f[5] += b.y, f[6] += b.z, f[7] += b.w;
        }
        const size_t c_off = static_cast<size_t>(row) * ep.ldc + col;
        if (ep.bias) {
          const bf16x8 bb8 = ld_bf16x8(ep.bias + col);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 bb = unpack_bf16x2(bb8.u[j]);
            f[2 * j] += bb.x;
            f[2 * j + 1] += bb.y;
          }
        }
        if (ep.residual) {
          const bf16x8 bb8 = ld_bf16x8(ep.residual + c_off);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 bb = unpack_bf16x2(bb8.u[j]);
            f[2 * j] += bb.x;
            f[2 * j + 1] += bb.y;
          }
        }
        if (ep.C_f32 != nullptr) {
          float4* d4 = reinterpret_cast<float4*>(ep.C_f32 + c_off);
          d4[0] = make_float4(f[0], f[1], f[2], f[3]);
          d4[1] = make_float4(f[4], f[5], f[6], f[7]);
        } else {
          bf16x8 o;
#pragma unroll
          for (int j = 0; j < 4; ++j) o.u[j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
          st_bf16x8(ep.C + c_off, o);
        }
        }  // valid row and column
      }
    }
  }

  if constexpr (EPI == PXL_EPI_RS) {
    if (warp >= 2) {
      // ---------------------------------------------- reduce the rows this rank owns
      // Work item = one 32-row quarter of an owned tile, dealt round-robin over all CTAs; each of
      // the four warps sums 8 rows, every row's loads (residual + tp partials) issued up front.
      const int q = warp & 3;
      const int tiles_per_shard = (comm.rows_per_rank / BM) * num_n;
      const bf16* my_stage = comm.stage[comm.rank];
      const uint32_t* my_flags = comm.flags[comm.rank];
      constexpr int LPR = BN / 8;        // lanes per row (16 bytes each)
      constexpr int RPP = 32 / LPR;      // rows per pass of the warp
      constexpr int PASSES = 8 / RPP;
      bool ok = !*abort_flag;
      for (int item = blockIdx.x; ok && item < tiles_per_shard * 4; item += gemm_ctas) {
        const int ot = item >> 2, quarter = item & 3;
        int okf = 1;
        if (lane == 0) {
          for (int src = 0; src < comm.tp && okf; ++src)
            okf = flag_wait_bounded<true>(my_flags + src * tiles_per_shard + ot, comm.epoch, abort_flag, status) ? 1 : 0;
        }
        ok = __shfl_sync(0xffffffffu, okf, 0) != 0;
        if (!ok) break;
        const int col = (ot % num_n) * BN + (lane % LPR) * 8;
        const int row_base = (ot / num_n) * BM + quarter * 32 + q * 8 + lane / LPR;
        if (col < N) {
          float f[PASSES][8];
#pragma unroll
          for (int p = 0; p < PASSES; ++p) {
            if (comm.residual) {
              const bf16x8 r8 = ld_bf16x8(comm.residual + static_cast<size_t>(row_base + p * RPP) * comm.ldo + col);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 t2 = unpack_bf16x2(r8.u[j]);
                f[p][2 * j] = t2.x;
                f[p][2 * j + 1] = t2.y;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) f[p][j] = 0.f;
            }
          }
#pragma unroll 1
          for (int src = 0; src < comm.tp; ++src) {
            bf16x8 part[PASSES];
#pragma unroll
            for (int p = 0; p < PASSES; ++p)
              part[p] = ld_bf16x8(my_stage + (static_cast<size_t>(src) * comm.rows_per_rank + row_base + p * RPP) * ep.ldc + col);
#pragma unroll
            for (int p = 0; p < PASSES; ++p) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 t2 = unpack_bf16x2(part[p].u[j]);
                f[p][2 * j] += t2.x;
                f[p][2 * j + 1] += t2.y;
              }
            }
          }
#pragma unroll
          for (int p = 0; p < PASSES; ++p) {
            bf16x8 o;
#pragma unroll
            for (int j = 0; j < 4; ++j) o.u[j] = pack_bf16x2(f[p][2 * j], f[p][2 * j + 1]);
            st_bf16x8(comm.out + static_cast<size_t>(row_base + p * RPP) * comm.ldo + col, o);
          }
        }
      }
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
                const GemmGroupArgs& grp, const GemmCommArgs& comm, int max_tiles, int M, int N,
                int K, int* status, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, EPI>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm_smem_bytes<BN, EPI>()) !=
        cudaSuccess)
      return PXL_ERR_CUDA;
    configured[dev] = true;
  }
  const int tiles = max_tiles > 0 ? max_tiles : pxl::ceil_div(M, BM) * pxl::ceil_div(N, BN);
  int grid = tiles < pxl_host::num_sms() ? tiles : pxl_host::num_sms();
  if (comm.ag_ncopy > 0) {
    // copy CTAs ride along: keep the whole grid co-resident (one CTA per SM)
    grid = grid + comm.ag_ncopy <= pxl_host::num_sms() ? grid + comm.ag_ncopy : pxl_host::num_sms();
    if (grid <= comm.ag_ncopy) return PXL_ERR_INVALID_ARG;
  }
  pxl_host::launch(kern, grid, kGemmThreads, gemm_smem_bytes<BN, EPI>(), stream, ta, tb, ep, grp, comm, M, N, K, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

// Cluster variant of the small-M path: one CTA per (tile, K range), the K ranges of a tile in one
// cluster. max_clusters (optional) receives how many such clusters the device runs at once.
template <int BN, int EPI = PXL_EPI_SPLITK_C>
int launch_gemm_cluster(const CUtensorMap& ta, const CUtensorMap& tb, const GemmEpilogueArgs& ep, int items,
                        int cluster, int M, int N, int K, int* status, cudaStream_t stream, int* max_clusters) {
  auto kern = gemm_bf16_tcgen05_kernel<BN, EPI>;
  constexpr int smem = gemm_smem_bytes<BN, EPI>();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return PXL_ERR_CUDA;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(items), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pxl_host::pdl_flag() && max_clusters == nullptr) ? 2 : 1;
  if (max_clusters != nullptr) {
    cfg.gridDim = dim3(static_cast<unsigned>(cluster) * 64u, 1, 1);  // the query only needs a legal grid
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    *max_clusters = n;
    return PXL_OK;
  }
  GemmGroupArgs grp{nullptr, nullptr, nullptr, nullptr, 0};
  GemmCommArgs comm{};
  if (cudaLaunchKernelEx(&cfg, kern, ta, tb, ep, grp, comm, M, N, K, status) != cudaSuccess) {
    cudaGetLastError();
    return PXL_ERR_CUDA;
  }
  return PXL_OK;
}

template <int BN>
int dispatch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const GemmEpilogueArgs& ep,
                 const GemmGroupArgs& grp, const GemmCommArgs& comm, int max_tiles, int M, int N,
                 int K, int* status, cudaStream_t stream) {
#define PXL_GEMM_CASE(E) \
  case E: return launch_gemm<BN, E>(ta, tb, ep, grp, comm, max_tiles, M, N, K, status, stream)
  switch (epi) {
    PXL_GEMM_CASE(PXL_EPI_NONE);
    PXL_GEMM_CASE(PXL_EPI_RESIDUAL);
    PXL_GEMM_CASE(PXL_EPI_SILU_MUL);
    PXL_GEMM_CASE(PXL_EPI_F32);
    PXL_GEMM_CASE(PXL_EPI_RS);
    PXL_GEMM_CASE(PXL_EPI_SCATTER);
    default: return PXL_ERR_INVALID_ARG;
  }
#undef PXL_GEMM_CASE
}

}  // namespace

// Tile width heuristic: estimated time = waves over the SMs x tile width / relative throughput of
// that width (measured on compute-bound shapes: a 256-wide tile keeps the tensor pipe busiest, a
// 64-wide one reaches about a third of it). Large problems take the width that wastes the least of
// the last wave; problems with few tiles end up with narrow ones, which put more SMs to work.
PXL_EXPORT int pxl_gemm_bf16_pick_bn(int M, int N, int epi) {
  const int sms = pxl_host::num_sms();
  const int num_m = pxl::ceil_div(M, BM);
  const int cands[4] = {256, 192, 128, 64};
  const double eff[4] = {1.0, 0.87, 0.68, 0.37};
  const bool plain = epi == PXL_EPI_NONE || epi == PXL_EPI_RESIDUAL || epi == PXL_EPI_F32;
  int best = 0;
  double best_cost = 1e300;
  for (int i = 0; i < 4; ++i) {
    const int bn = cands[i];
    if (epi == PXL_EPI_SILU_MUL && ((N % bn) != 0 || bn < 128 || bn == 192)) continue;
    if (bn == 192 && !plain) continue;
    const int tiles = num_m * pxl::ceil_div(N, bn);
    const double cost = static_cast<double>(pxl::ceil_div(tiles, sms)) * bn / eff[i];
    if (cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best ? best : 128;
}

namespace {
// fp32 scratch of the small-M path: one per (device, stream) so that GEMMs on different streams
// never share partial sums. Allocated on first use; the arrival counters behind it are zeroed once
// and every launch leaves them zeroed.
constexpr int kSmallMaxM = 128;
constexpr int kSmallMaxN = 32768;
constexpr size_t kSmallScratchFloats = static_cast<size_t>(kSmallMaxM) * kSmallMaxN;  // 16 MB
struct SmallMScratch {
  int dev;
  cudaStream_t stream;
  float* ws;
  uint32_t* counters;
};
constexpr int kSmallMaxScratch = 64;
SmallMScratch g_small[kSmallMaxScratch];
int g_small_n = 0;
std::mutex g_small_mu;

bool small_m_scratch(cudaStream_t stream, float** ws, uint32_t** counters) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(g_small_mu);
  for (int i = 0; i < g_small_n; ++i) {
    if (g_small[i].dev == dev && g_small[i].stream == stream) {
      *ws = g_small[i].ws;
      *counters = g_small[i].counters;
      return true;
    }
  }
  if (g_small_n == kSmallMaxScratch) return false;
  const size_t ws_bytes = kSmallScratchFloats * sizeof(float);
  const size_t cnt_bytes = (kSmallMaxN / BM) * sizeof(uint32_t);
  void* p = nullptr;
  if (cudaMalloc(&p, ws_bytes + cnt_bytes) != cudaSuccess) return false;
  if (cudaMemset(p, 0, ws_bytes + cnt_bytes) != cudaSuccess) {
    cudaFree(p);
    return false;
  }
  SmallMScratch& e = g_small[g_small_n++];
  e.dev = dev;
  e.stream = stream;
  e.ws = static_cast<float*>(p);
  e.counters = reinterpret_cast<uint32_t*>(static_cast<char*>(p) + ws_bytes);
  *ws = e.ws;
  *counters = e.counters;
  return true;
}

bool small_m_disabled() {
  static const bool off = getenv("PXL_NO_SMALL_M_GEMM") != nullptr;
  return off;
}

// K ranges per 128 output columns: as many as fill the SMs once, at least four k-blocks each.
int small_m_splitk(int N, int K) {
  const int tiles = pxl::ceil_div(N, BM);
  const int num_kb = pxl::ceil_div(K, BK);
  int s = pxl_host::num_sms() / tiles;
  if (s > num_kb / 4) s = num_kb / 4;
  if (s > 32) s = 32;
  if (s < 1) s = 1;
  return s;
}
}  // namespace

PXL_EXPORT int pxl_gemm_bf16_uses_small_m(int M, int N, int K, int epi) {
  if (small_m_disabled()) return 0;
  if (M <= 0 || M > kSmallMaxM || N > kSmallMaxN || (N % 8) || K <= 0) return 0;
  if (epi != PXL_EPI_NONE && epi != PXL_EPI_RESIDUAL && epi != PXL_EPI_F32) return 0;
  // with at least one 128-column tile per SM the plain kernel already streams from every SM
  return pxl::ceil_div(N, BM) <= pxl_host::num_sms() ? 1 : 0;
}

namespace {
// How many clusters of `cluster` CTAs of the small-M kernel the device keeps resident at once
// (cached per device, token-slot width and cluster size; 0 = unknown or not launchable).
int small_m_max_clusters(int bn_tok, int cluster) {
  static int cache[64][3][9];
  static bool known[64][3][9] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || cluster < 1 || cluster > 8) return 0;
  const int bi = bn_tok == 32 ? 0 : (bn_tok == 64 ? 1 : 2);
  std::lock_guard<std::mutex> lock(mu);
  if (!known[dev][bi][cluster]) {
    int n = 0;
    CUtensorMap dummy{};
    GemmEpilogueArgs ep{};
    switch (bn_tok) {
      case 32: launch_gemm_cluster<32>(dummy, dummy, ep, 0, cluster, 0, 0, 0, nullptr, nullptr, &n); break;
      case 64: launch_gemm_cluster<64>(dummy, dummy, ep, 0, cluster, 0, 0, 0, nullptr, nullptr, &n); break;
      default: launch_gemm_cluster<128>(dummy, dummy, ep, 0, cluster, 0, 0, 0, nullptr, nullptr, &n); break;
    }
    cache[dev][bi][cluster] = n;
    known[dev][bi][cluster] = true;
  }
  return cache[dev][bi][cluster];
}

// mode 0 = automatic, 1 = scratch slabs + last-CTA finish, 2 = cluster reduction over DSMEM
int gemm_small_m(const void* A, const void* W, void* C, bool f32_out, const void* residual, const void* bias, int M,
                 int N, int K, int lda, int ldw, int ldc, int splitk, int mode, int* status, cudaStream_t stream) {
  if (M <= 0 || M > kSmallMaxM || N <= 0 || N > kSmallMaxN || K <= 0) return PXL_ERR_INVALID_ARG;
  if ((K % 8) || (lda % 8) || (ldw % 8) || (ldc % 8) || (N % 8)) return PXL_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(bias)) & 15)
    return PXL_ERR_INVALID_ARG;
  if (mode < 0 || mode > 2) return PXL_ERR_INVALID_ARG;
  const int num_kb = pxl::ceil_div(K, BK);
  const int tiles = pxl::ceil_div(N, BM);
  const int bn_tok = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  const bool auto_split = splitk <= 0;
  if (auto_split) splitk = small_m_splitk(N, K);
  if (splitk > num_kb) splitk = num_kb;
  if (mode != 1) {
    // the widest cluster (at most 8 CTAs, at most the K ranges asked for) of which all tiles' clusters
    // are resident at once; an explicit splitk is only narrowed by the hardware limit of 8
    int c = splitk < 8 ? splitk : 8;
    if (auto_split) {
      while (c > 1 && small_m_max_clusters(bn_tok, c) < tiles) --c;
    }
    const bool launchable = small_m_max_clusters(bn_tok, c) > 0;
    // few tiles and a long K: more K ranges than a cluster holds put more SMs to work
    const bool prefer_scratch = auto_split && splitk > c && tiles * c * 2 < pxl_host::num_sms();
    if (launchable && (mode == 2 || !prefer_scratch)) {
      splitk = c;
      mode = 2;
    } else if (mode == 2) {
      return PXL_ERR_CUDA;
    } else {
      mode = 1;
    }
  }
  // no empty K range: an accumulator that no MMA wrote would be added as is
  if (mode == 1) {
    while (splitk > 1 && static_cast<size_t>(splitk) * M * N > kSmallScratchFloats) --splitk;
  }
  splitk = pxl::ceil_div(num_kb, pxl::ceil_div(num_kb, splitk));
  // swapped operand slots: the weights take the 128-row slot, the tokens the narrow one
  CUtensorMap ta, tb;
  if (!pxl_host::make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, N, K, ldw, BM, BK))
    return PXL_ERR_TENSORMAP;
  if (!pxl_host::make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, M, K, lda, bn_tok, BK))
    return PXL_ERR_TENSORMAP;
  GemmEpilogueArgs ep{};
  ep.C = static_cast<pxl::bf16*>(C);
  ep.C_f32 = f32_out ? static_cast<float*>(C) : nullptr;
  ep.residual = static_cast<const pxl::bf16*>(residual);
  ep.bias = static_cast<const pxl::bf16*>(bias);
  ep.ldc = ldc;
  ep.ldws = N;
  ep.splitk = splitk;
  const int items = tiles * splitk;
  // kernel view: M' = output columns, N' = tokens
  if (mode == 2) {
    switch (bn_tok) {
      case 32: return launch_gemm_cluster<32>(ta, tb, ep, items, splitk, N, M, K, status, stream, nullptr);
      case 64: return launch_gemm_cluster<64>(ta, tb, ep, items, splitk, N, M, K, status, stream, nullptr);
      default: return launch_gemm_cluster<128>(ta, tb, ep, items, splitk, N, M, K, status, stream, nullptr);
    }
  }
  if (!small_m_scratch(stream, &ep.ws, &ep.tile_counters)) return PXL_ERR_CUDA;
  GemmGroupArgs grp{nullptr, nullptr, nullptr, nullptr, 0};
  switch (bn_tok) {
    case 32:
      return launch_gemm<32, PXL_EPI_SPLITK_T>(ta, tb, ep, grp, GemmCommArgs{}, items, N, M, K, status, stream);
    case 64:
      return launch_gemm<64, PXL_EPI_SPLITK_T>(ta, tb, ep, grp, GemmCommArgs{}, items, N, M, K, status, stream);
    default:
      return launch_gemm<128, PXL_EPI_SPLITK_T>(ta, tb, ep, grp, GemmCommArgs{}, items, N, M, K, status, stream);
  }
}
}  // namespace

namespace {
// ---- mid-M path: 129 .. kMidMaxM tokens, operands in their usual slots, K split inside a cluster ----
constexpr int kMidMaxM = 1024;

int mid_m_max_clusters(int bn, int cluster) {
  static int cache[64][2][9];
  static bool known[64][2][9] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || cluster < 1 || cluster > 8) return 0;
  const int bi = bn == 128 ? 0 : 1;
  std::lock_guard<std::mutex> lock(mu);
  if (!known[dev][bi][cluster]) {
    int n = 0;
    CUtensorMap dummy{};
    GemmEpilogueArgs ep{};
    if (bn == 128)
      launch_gemm_cluster<128, PXL_EPI_SPLITK_CN>(dummy, dummy, ep, 0, cluster, 0, 0, 0, nullptr, nullptr, &n);
    else
      launch_gemm_cluster<256, PXL_EPI_SPLITK_CN>(dummy, dummy, ep, 0, cluster, 0, 0, 0, nullptr, nullptr, &n);
    cache[dev][bi][cluster] = n;
    known[dev][bi][cluster] = true;
  }
  return cache[dev][bi][cluster];
}

// Cost model (microseconds) of one launch, fitted to CUDA-event timings of the four Qwen3-8B projection
// shapes at 192 / 320 / 512 rows (weights streamed from HBM):
//   plain persistent kernel   rounds x (k-blocks x t_kb) + 7
//   cluster split-K           k-blocks per CTA x t_kb + 8 + splitk x bn / 128   (exchange of partial sums)
// t_kb = time of one 64-deep k-block per CTA, set by what the SM can pull from L2 (48 KB per k-block for a
// 128 x 256 tile, 32 KB for 128 x 128). Split variants are only considered when all clusters are resident at
// once (a second round pays the fixed cost again and was always slower) and for 2 or 4 K ranges (clusters of
// 3 pack the GPCs badly: 144 CTAs in clusters of 3 ran as slowly as two rounds).
struct MidPlan {
  int bn, splitk;
  double cost;
};

MidPlan mid_m_plan(int M, int N, int K) {
  const int num_kb = pxl::ceil_div(K, BK);
  const int num_m = pxl::ceil_div(M, BM);
  const int sms = pxl_host::num_sms();
  MidPlan best{0, 1, 1e300};
  const int bns[3] = {256, 128, 192};
  const double t_kb[3] = {0.43, 0.29, 0.36};
  for (int i = 0; i < 3; ++i) {
    const int tiles = num_m * pxl::ceil_div(N, bns[i]);
    const double plain = pxl::ceil_div(tiles, sms) * (num_kb * t_kb[i]) + 7.0;
    if (plain < best.cost) best = MidPlan{bns[i], 1, plain};
    if (bns[i] == 192) continue;  // the cluster variant exists for 128- and 256-wide tiles
    for (int sk = 2; sk <= 4; sk += 2) {
      if (num_kb / sk < 4) break;
      const int kb_per = pxl::ceil_div(num_kb, sk);
      if (pxl::ceil_div(num_kb, kb_per) != sk) continue;  // no empty K range
      if (tiles > mid_m_max_clusters(bns[i], sk)) continue;
      const double cost = kb_per * t_kb[i] + 8.0 + sk * (bns[i] / 128);
      if (cost < best.cost) best = MidPlan{bns[i], sk, cost};
    }
  }
  return best;
}

bool mid_m_disabled() {
  static const bool off = getenv("PXL_NO_MID_M_GEMM") != nullptr;
  return off;
}

int gemm_mid_m(const void* A, const void* W, void* C, bool f32_out, const void* residual, const void* bias, int M,
               int N, int K, int lda, int ldw, int ldc, int bn, int splitk, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || splitk < 2 || splitk > 8) return PXL_ERR_INVALID_ARG;
  if (bn != 128 && bn != 256) return PXL_ERR_INVALID_ARG;
  if ((K % 8) || (lda % 8) || (ldw % 8) || (ldc % 8) || (N % 8)) return PXL_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(bias)) & 15)
    return PXL_ERR_INVALID_ARG;
  const int num_kb = pxl::ceil_div(K, BK);
  if (splitk > num_kb) return PXL_ERR_INVALID_ARG;
  splitk = pxl::ceil_div(num_kb, pxl::ceil_div(num_kb, splitk));  // no empty K range
  if (splitk < 2) return PXL_ERR_INVALID_ARG;
  CUtensorMap ta, tb;
  if (!pxl_host::make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, M, K, lda, BM, BK))
    return PXL_ERR_TENSORMAP;
  if (!pxl_host::make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, N, K, ldw, bn, BK))
    return PXL_ERR_TENSORMAP;
  GemmEpilogueArgs ep{};
  ep.C = static_cast<pxl::bf16*>(C);
  ep.C_f32 = f32_out ? static_cast<float*>(C) : nullptr;
  ep.residual = static_cast<const pxl::bf16*>(residual);
  ep.bias = static_cast<const pxl::bf16*>(bias);
  ep.ldc = ldc;
  ep.splitk = splitk;
  const int items = pxl::ceil_div(M, BM) * pxl::ceil_div(N, bn) * splitk;
  if (bn == 128)
    return launch_gemm_cluster<128, PXL_EPI_SPLITK_CN>(ta, tb, ep, items, splitk, M, N, K, status, stream, nullptr);
  return launch_gemm_cluster<256, PXL_EPI_SPLITK_CN>(ta, tb, ep, items, splitk, M, N, K, status, stream, nullptr);
}
}  // namespace

// Which (tile width, K ranges) pxl_gemm_bf16 picks for a shape with 128 < M <= 1024: returns
// bn * 16 + splitk, splitk == 1 meaning the plain persistent kernel.
PXL_EXPORT int pxl_gemm_bf16_mid_m_plan(int M, int N, int K, int epi) {
  if (mid_m_disabled() || M <= BM || M > kMidMaxM) return 0;
  if (epi != PXL_EPI_NONE && epi != PXL_EPI_RESIDUAL && epi != PXL_EPI_F32) return 0;
  const MidPlan p = mid_m_plan(M, N, K);
  return p.bn * 16 + p.splitk;
}

// Explicit entry to the mid-M cluster split-K kernel (tests and benchmarks; pxl_gemm_bf16 picks it by itself).
PXL_EXPORT int pxl_gemm_bf16_mid_m(const void* A, const void* W, void* C, const void* residual, const void* bias,
                                   int M, int N, int K, int lda, int ldw, int ldc, int bn, int splitk, int f32_out,
                                   int* status, cudaStream_t stream) {
  return gemm_mid_m(A, W, C, f32_out != 0, residual, bias, M, N, K, lda, ldw, ldc, bn, splitk, status, stream);
}

PXL_EXPORT int pxl_gemm_bf16_small_m(const void* A, const void* W, void* C, const void* residual,
                                     const void* bias, int M, int N, int K, int lda, int ldw, int ldc,
                                     int splitk, int mode, int* status, cudaStream_t stream) {
  return gemm_small_m(A, W, C, false, residual, bias, M, N, K, lda, ldw, ldc, splitk, mode, status, stream);
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
  if (bn == 0 && pxl_gemm_bf16_uses_small_m(M, N, K, epi) &&
      !((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(bias)) & 15))
    return gemm_small_m(A, W, C, epi == PXL_EPI_F32, epi == PXL_EPI_RESIDUAL ? residual : nullptr, bias, M, N, K,
                        lda, ldw, ldc, 0, 0, status, stream);
  if (bn == 0 && !((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(bias)) & 15)) {
    const int plan = pxl_gemm_bf16_mid_m_plan(M, N, K, epi);
    if (plan > 0 && (plan & 15) > 1)
      return gemm_mid_m(A, W, C, epi == PXL_EPI_F32, epi == PXL_EPI_RESIDUAL ? residual : nullptr, bias, M, N, K, lda,
                        ldw, ldc, plan >> 4, plan & 15, status, stream);
  }
  if (bn == 0) bn = pxl_gemm_bf16_pick_bn(M, N, epi);
  if (epi == PXL_EPI_SILU_MUL && ((N % bn) != 0 || bn < 128)) return PXL_ERR_INVALID_ARG;

  CUtensorMap ta, tb;
  if (!pxl_host::make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, M, K, lda, BM, BK))
    return PXL_ERR_TENSORMAP;
  if (!pxl_host::make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, N, K, ldw, bn, BK))
    return PXL_ERR_TENSORMAP;
  GemmEpilogueArgs ep{};
  ep.C = static_cast<pxl::bf16*>(C);
  ep.C_f32 = static_cast<float*>(C);
  ep.residual = static_cast<const pxl::bf16*>(residual);
  ep.bias = static_cast<const pxl::bf16*>(bias);
  ep.ldc = ldc;
  GemmGroupArgs grp{nullptr, nullptr, nullptr, nullptr, 0};
  switch (bn) {
    case 256: return dispatch_epi<256>(epi, ta, tb, ep, grp, GemmCommArgs{}, 0, M, N, K, status, stream);
    case 192:  // plain epilogues only: fills the last wave better when N / 256 leaves SMs idle
      switch (epi) {
        case PXL_EPI_NONE:
          return launch_gemm<192, PXL_EPI_NONE>(ta, tb, ep, grp, GemmCommArgs{}, 0, M, N, K, status, stream);
        case PXL_EPI_RESIDUAL:
          return launch_gemm<192, PXL_EPI_RESIDUAL>(ta, tb, ep, grp, GemmCommArgs{}, 0, M, N, K, status, stream);
        case PXL_EPI_F32:
          return launch_gemm<192, PXL_EPI_F32>(ta, tb, ep, grp, GemmCommArgs{}, 0, M, N, K, status, stream);
        default: return PXL_ERR_INVALID_ARG;
      }
    case 128: return dispatch_epi<128>(epi, ta, tb, ep, grp, GemmCommArgs{}, 0, M, N, K, status, stream);
    case 64: return dispatch_epi<64>(epi, ta, tb, ep, grp, GemmCommArgs{}, 0, M, N, K, status, stream);
    default: return PXL_ERR_INVALID_ARG;
  }
}

// Grouped GEMM over experts: for every m-tile i listed on the device,
//   C[rows of tile i, :] = A[rows of tile i, :] * W[expert_i]^T
// A: [P, K] activations permuted so that each expert's tokens are contiguous; W: [E*N, K]
// (expert matrices stacked); C: [P, N] (N/2 columns with PXL_EPI_SILU_MUL); bias: optional [E*N].
// max_m_tiles bounds the device-side count and sizes the grid.
PXL_EXPORT int pxl_gemm_bf16_grouped(const void* A, const void* W, void* C, const void* bias, int P, int E,
                                     int N, int K, int lda, int ldw, int ldc, const int* mt_expert,
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
  GemmEpilogueArgs ep{};
  ep.C = static_cast<pxl::bf16*>(C);
  ep.C_f32 = static_cast<float*>(C);
  ep.residual = nullptr;
  ep.bias = static_cast<const pxl::bf16*>(bias);  // optional [E * N], applied with PXL_EPI_NONE / F32
  ep.ldc = ldc;
  GemmGroupArgs grp{mt_expert, mt_row0, mt_row_end, num_mt, N};
  const int max_tiles = max_m_tiles * pxl::ceil_div(N, bn);
  switch (bn) {
    case 256: return dispatch_epi<256>(epi, ta, tb, ep, grp, GemmCommArgs{}, max_tiles, P, N, K, status, stream);
    case 128: return dispatch_epi<128>(epi, ta, tb, ep, grp, GemmCommArgs{}, max_tiles, P, N, K, status, stream);
    case 64: return dispatch_epi<64>(epi, ta, tb, ep, grp, GemmCommArgs{}, max_tiles, P, N, K, status, stream);
    default: return PXL_ERR_INVALID_ARG;
  }
}


// Grouped GEMM whose output rows leave through per-row pointers (expert-parallel combine fused
// into the down projection): row i of the expert-sorted result is stored to row_ptrs[i] (N bf16,
// 16-byte aligned, may be peer memory; null = drop). When the whole grid is done, flag_ptrs[r][rank]
// of every rank r is set to `epoch` (release, system scope).
PXL_EXPORT int pxl_gemm_bf16_grouped_scatter(const void* A, const void* W, void* const* row_ptrs, int P, int E,
                                             int N, int K, int lda, int ldw, const int* mt_expert,
                                             const int* mt_row0, const int* mt_row_end, const int* num_mt,
                                             int max_m_tiles, void* const* flag_ptrs, uint32_t* done_counter,
                                             int rank, int ep_size, uint32_t epoch, int* status,
                                             cudaStream_t stream) {
  if (P <= 0 || E <= 0 || N <= 0 || K <= 0 || max_m_tiles <= 0) return PXL_ERR_INVALID_ARG;
  if ((K % 8) || (lda % 8) || (ldw % 8) || (N % 128)) return PXL_ERR_INVALID_ARG;
  if (ep_size < 1 || ep_size > 8 || rank < 0 || rank >= ep_size) return PXL_ERR_INVALID_ARG;
  const int bn = 128;
  CUtensorMap ta, tb;
  if (!pxl_host::make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, P, K, lda, BM, BK))
    return PXL_ERR_TENSORMAP;
  if (!pxl_host::make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, static_cast<uint64_t>(E) * N, K, ldw, bn, BK))
    return PXL_ERR_TENSORMAP;
  GemmEpilogueArgs ep{};
  ep.ldc = N;
  ep.row_ptrs = reinterpret_cast<pxl::bf16* const*>(row_ptrs);
  ep.done_counter = done_counter;
  GemmCommArgs comm{};
  for (int i = 0; i < ep_size; ++i) comm.flags[i] = static_cast<uint32_t*>(flag_ptrs[i]);
  comm.rank = rank;
  comm.tp = ep_size;
  comm.epoch = epoch;
  GemmGroupArgs grp{mt_expert, mt_row0, mt_row_end, num_mt, N};
  return dispatch_epi<128>(PXL_EPI_SCATTER, ta, tb, ep, grp, comm, max_m_tiles * (N / bn), P, N, K, status, stream);
}

namespace {
int check_comm_common(int tp, int rank, int rows_per_rank, int K, int N) {
  if (tp < 2 || tp > 8 || rank < 0 || rank >= tp) return PXL_ERR_INVALID_ARG;
  if (rows_per_rank <= 0 || rows_per_rank % BM) return PXL_ERR_INVALID_ARG;
  if ((K % 8) || (N % 8)) return PXL_ERR_INVALID_ARG;
  return PXL_OK;
}
}  // namespace

// Fused GEMM -> reduce-scatter over tensor-parallel ranks.
//   A [tp*rows_per_rank, K] (this rank's K-slice of the activations), W [N, K];
//   out[rows_per_rank, N] = sum over ranks of (A_r W_r^T)[rows owned by this rank] (+ residual).
// stage_ptrs[i] / flag_ptrs[i]: rank i's staging buffer [tp][rows_per_rank][N] bf16 and flag
// array [tp][tiles] uint32 in peer-mapped symmetric memory (flags zero-initialised once;
// `epoch` must grow by one on every call that uses the same buffers).
PXL_EXPORT int pxl_gemm_bf16_rs(const void* A, const void* W, void* out, const void* residual,
                                void* const* stage_ptrs, void* const* flag_ptrs, int rank, int tp,
                                int rows_per_rank, int N, int K, int lda, int ldw, int ldo,
                                uint32_t epoch, int bn, int* status, cudaStream_t stream) {
  int rc = check_comm_common(tp, rank, rows_per_rank, K, N);
  if (rc) return rc;
  if ((lda % 8) || (ldw % 8) || (ldo % 8)) return PXL_ERR_INVALID_ARG;
  const int M = tp * rows_per_rank;
  // wide tiles only when they still give every SM a tile
  if (bn == 0) bn = (N % 256 == 0 && (M / BM) * (N / 256) >= pxl_host::num_sms()) ? 256 : 128;
  if (N % bn) return PXL_ERR_INVALID_ARG;
  CUtensorMap ta, tb;
  if (!pxl_host::make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, M, K, lda, BM, BK))
    return PXL_ERR_TENSORMAP;
  if (!pxl_host::make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, N, K, ldw, bn, BK))
    return PXL_ERR_TENSORMAP;
  GemmEpilogueArgs ep{};
  ep.ldc = N;
  GemmCommArgs comm{};
  for (int i = 0; i < tp; ++i) {
    comm.stage[i] = static_cast<pxl::bf16*>(stage_ptrs[i]);
    comm.flags[i] = static_cast<uint32_t*>(flag_ptrs[i]);
  }
  comm.out = static_cast<pxl::bf16*>(out);
  comm.residual = static_cast<const pxl::bf16*>(residual);
  comm.rank = rank;
  comm.tp = tp;
  comm.rows_per_rank = rows_per_rank;
  comm.ldo = ldo;
  comm.first_shard = (rank + 1) % tp;  // own rows last: the partials of the peers arrive meanwhile
  comm.epoch = epoch;
  GemmGroupArgs grp{nullptr, nullptr, nullptr, nullptr, 0};
  switch (bn) {
    case 256: return dispatch_epi<256>(PXL_EPI_RS, ta, tb, ep, grp, comm, 0, M, N, K, status, stream);
    case 128: return dispatch_epi<128>(PXL_EPI_RS, ta, tb, ep, grp, comm, 0, M, N, K, status, stream);
    default: return PXL_ERR_INVALID_ARG;
  }
}

// Fused all-gather -> GEMM. Every rank holds the full-size matrix X [tp*rows_per_rank, K] in
// symmetric memory but only its own row shard is valid on entry; copy CTAs pull the other
// shards over NVLink while the tensor cores already work on the local shard.
//   C[tp*rows_per_rank, N] = X_full W^T  with the usual epilogues (bias / SiLU-mul).
// x_ptrs[i]: rank i's X; ready_ptrs[i]: rank i's [tp] shard-ready flags (symmetric memory);
// tile_flags: local [tp*rows_per_rank/128][16] flags (one per 8-row chunk). Flags zero-initialised
// once; epoch grows.
PXL_EXPORT int pxl_gemm_bf16_ag(void* const* x_ptrs, void* const* ready_ptrs, void* tile_flags,
                                const void* W, void* C, const void* bias, int rank, int tp,
                                int rows_per_rank, int N, int K, int lda, int ldw, int ldc, int epi,
                                uint32_t epoch, int ncopy, int bn, int* status, cudaStream_t stream) {
  int rc = check_comm_common(tp, rank, rows_per_rank, K, N);
  if (rc) return rc;
  if (epi != PXL_EPI_NONE && epi != PXL_EPI_SILU_MUL && epi != PXL_EPI_F32) return PXL_ERR_INVALID_ARG;
  if ((lda % 8) || (ldw % 8) || (ldc % 8)) return PXL_ERR_INVALID_ARG;
  const int M = tp * rows_per_rank;
  if (ncopy <= 0) {
    // copy CTAs take SMs from the GEMM: many when the GEMM is short (latency matters), few
    // when it runs for several waves anyway and the copy hides behind the local shard's tiles
    const int tiles = (M / BM) * pxl::ceil_div(N, 256);
    ncopy = tiles >= 2 * pxl_host::num_sms() ? 8 : (tiles >= pxl_host::num_sms() ? 16 : 32);
  }
  if (ncopy >= pxl_host::num_sms()) return PXL_ERR_INVALID_ARG;
  // a chunk of kAgChunkRows rows must fit into the copy CTA's shared memory
  if (static_cast<long long>(kAgChunkRows) * K * 2 > 192 * 1024 || (lda % 8)) return PXL_ERR_INVALID_ARG;
  if (bn == 0)
    bn = (N % 256 == 0 && (M / BM) * (N / 256) >= pxl_host::num_sms() - ncopy) ? 256 : 128;
  if (epi == PXL_EPI_SILU_MUL && ((N % bn) != 0 || bn < 128)) return PXL_ERR_INVALID_ARG;
  CUtensorMap ta, tb;
  if (!pxl_host::make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x_ptrs[rank], M, K, lda, BM, BK))
    return PXL_ERR_TENSORMAP;
  if (!pxl_host::make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, N, K, ldw, bn, BK))
    return PXL_ERR_TENSORMAP;
  GemmEpilogueArgs ep{};
  ep.C = static_cast<pxl::bf16*>(C);
  ep.C_f32 = static_cast<float*>(C);
  ep.bias = static_cast<const pxl::bf16*>(bias);
  ep.ldc = ldc;
  GemmCommArgs comm{};
  for (int i = 0; i < tp; ++i) {
    comm.ag_src[i] = static_cast<const pxl::bf16*>(x_ptrs[i]);
    comm.ag_ready[i] = static_cast<uint32_t*>(ready_ptrs[i]);
  }
  comm.ag_dst = static_cast<pxl::bf16*>(x_ptrs[rank]);
  comm.ag_tile_flags = static_cast<uint32_t*>(tile_flags);
  comm.rank = rank;
  comm.tp = tp;
  comm.rows_per_rank = rows_per_rank;
  comm.lda = lda;
  comm.ag_ncopy = ncopy;
  comm.first_shard = rank;  // local rows first
  comm.epoch = epoch;
  GemmGroupArgs grp{nullptr, nullptr, nullptr, nullptr, 0};
  switch (bn) {
    case 256: return dispatch_epi<256>(epi, ta, tb, ep, grp, comm, 0, M, N, K, status, stream);
    case 128: return dispatch_epi<128>(epi, ta, tb, ep, grp, comm, 0, M, N, K, status, stream);
    case 64: return dispatch_epi<64>(epi, ta, tb, ep, grp, comm, 0, M, N, K, status, stream);
    default: return PXL_ERR_INVALID_ARG;
  }
}
