// Expert-parallel MoE over NVLink peer memory: dispatch and combine without a collective library.
//
// Every rank owns E / ep consecutive experts and a slice of the batch's token rows. Per MoE layer:
//   1. ep_dispatch   (source side)  each (row, slot) pair is pushed into the receive region
//                                    [source rank] of the rank that owns its expert: the token row
//                                    (coalesced 16-byte peer stores) plus a meta word; the CTA that
//                                    finishes last publishes the per-destination counts and flags.
//   2. ep_recv_ids   (owner side)   waits (bounded) for every source's flag and lists the local
//                                    expert id of every received row (-1 for unused slots), which is
//                                    what the expert alignment / grouped GEMM take as input.
//   3. ep_row_ptrs   (owner side)   destination pointer of every expert-sorted row inside the
//                                    source rank's combine buffer; the down-projection GEMM stores
//                                    its rows straight through them (PXL_EPI_SCATTER) and raises
//                                    the return flags when its grid is done.
//   4. ep_combine    (source side)  waits for every owner's return flag, then
//                                    out[row] = base[row] + sum_j w[row, j] * returned[row, j].
// The reference has no expert parallelism (moe_ep_size = 1 is hard-coded in
// src/parallax/sglang/model_runner.py:394-395; the MLX path shards every expert's FFN dimension,
// src/parallax/models/minimax_m3.py:871-892).
#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

struct EpPeers {
  bf16* recv_x[8];        // rank d: [ep][cap][H]
  int* recv_meta[8];      // rank d: [ep][cap][2]  (local expert, row * k + slot)
  int* recv_cnt[8];       // rank d: [ep]
  uint32_t* disp_flag[8]; // rank d: [ep]
};

// grid-stride over (row, slot) pairs, one warp per pair
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const bf16* __restrict__ x, int64_t ldx,
                                                          const int* __restrict__ ids, int n_rows, int k, int H,
                                                          int experts_per_rank, int cap, int rank, int ep,
                                                          const EpPeers peers, int* __restrict__ cursor,
                                                          uint32_t* __restrict__ done_counter, uint32_t epoch,
                                                          int* status) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int pair = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; pair < n_rows * k; pair += warps) {
    const int e = ids[pair];
    const int d = e / experts_per_rank;
    if (e < 0 || d >= ep) {
      if (lane == 0 && status) atomicCAS(status, 0, PXL_DEV_BAD_INDEX);
      continue;
    }
    int pos = 0;
    if (lane == 0) pos = atomicAdd(&cursor[d], 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (pos >= cap) {
      if (lane == 0 && status) atomicCAS(status, 0, PXL_DEV_BAD_INDEX);
      continue;
    }
    const size_t slot = static_cast<size_t>(rank) * cap + pos;
    if (lane == 0) {
      int2 m = make_int2(e - d * experts_per_rank, pair);
      *reinterpret_cast<int2*>(peers.recv_meta[d] + slot * 2) = m;
    }
    const bf16* src = x + (pair / k) * ldx;
    bf16* dst = peers.recv_x[d] + slot * H;
    for (int c = lane; c < H / 8; c += 32) st_bf16x8(dst + c * 8, ld_bf16x8(src + c * 8));
  }
  // last CTA: counts + flags to every destination
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(done_counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (threadIdx.x < ep) {
    const int d = threadIdx.x;
    const int n = min(cursor[d], cap);
    peers.recv_cnt[d][rank] = n;
    cursor[d] = 0;
    __threadfence_system();
    st_release_sys_u32(peers.disp_flag[d] + rank, epoch);
  }
  if (threadIdx.x == 0) *done_counter = 0;
}

__global__ void __launch_bounds__(256) ep_recv_ids_kernel(const int* __restrict__ recv_meta,
                                                          const int* __restrict__ recv_cnt,
                                                          const uint32_t* __restrict__ disp_flag, int ep, int cap,
                                                          uint32_t epoch, int* __restrict__ ids_out, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int s = 0; s < ep && ok; ++s) ok = flag_wait_bounded<true>(disp_flag + s, epoch, nullptr, status);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < ep * cap; i += gridDim.x * blockDim.x) {
    const int s = i / cap, pos = i - s * cap;
    ids_out[i] = (ok && pos < recv_cnt[s]) ? recv_meta[static_cast<size_t>(i) * 2] : -1;
  }
}

struct EpCombPtrs {
  bf16* comb[8];  // rank s: [rows][k][H]
};

struct EpRetFlags {
  uint32_t* ret[8];  // rank r: [ep] return flags
};

__global__ void __launch_bounds__(256) ep_row_ptrs_kernel(const int* __restrict__ src_slot, const int* __restrict__ n_rows,
                                                          const int* __restrict__ recv_meta, int cap, int H,
                                                          const EpCombPtrs comb, bf16** __restrict__ row_ptrs,
                                                          int max_rows) {
  const int n = *n_rows;
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < max_rows; p += gridDim.x * blockDim.x) {
    bf16* ptr = nullptr;
    if (p < n) {
      const int slot = src_slot[p];  // index into the [ep][cap] receive region
      const int s = slot / cap;
      const int pair = recv_meta[static_cast<size_t>(slot) * 2 + 1];
      ptr = comb.comb[s] + static_cast<size_t>(pair) * H;
    }
    row_ptrs[p] = ptr;
  }
}

// one CTA per token row
__global__ void __launch_bounds__(256) ep_combine_kernel(const bf16* __restrict__ comb, const float* __restrict__ w,
                                                         const bf16* __restrict__ base, int64_t ld_base,
                                                         bf16* __restrict__ out, int64_t ld_out,
                                                         const uint32_t* __restrict__ ret_flag, int ep, uint32_t epoch,
                                                         int n_rows, int k, int H, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int s = 0; s < ep && ok; ++s) ok = flag_wait_bounded<true>(ret_flag + s, epoch, nullptr, status);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const int row = blockIdx.x;
  if (row >= n_rows) return;  // a rank without rows still has to wait for the return flags
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    float f[8];
    if (base) {
      const bf16x8 b = ld_bf16x8(base + row * ld_base + c * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t2 = unpack_bf16x2(b.u[j]);
        f[2 * j] = t2.x;
        f[2 * j + 1] = t2.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
    }
    for (int s = 0; s < k; ++s) {
      const float ws = w[row * k + s];
      const bf16x8 y = ld_bf16x8(comb + (static_cast<size_t>(row) * k + s) * H + c * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t2 = unpack_bf16x2(y.u[j]);
        f[2 * j] = fmaf(ws, t2.x, f[2 * j]);
        f[2 * j + 1] = fmaf(ws, t2.y, f[2 * j + 1]);
      }
    }
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) o.u[j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
    st_bf16x8(out + row * ld_out + c * 8, o);
  }
}

// Return trip as a kernel of its own (used when the down projection cannot store through row pointers,
// e.g. the block-scaled fp8 grouped GEMM): row p of the expert-sorted result goes to row_ptrs[p]; the CTA
// that finishes last raises the return flag of every peer.
__global__ void __launch_bounds__(256) ep_return_rows_kernel(const bf16* __restrict__ y, int64_t ldy,
                                                             bf16* const* __restrict__ row_ptrs,
                                                             const int* __restrict__ n_rows, int max_rows, int H,
                                                             EpRetFlags flags, uint32_t* __restrict__ done_counter,
                                                             int rank, int ep, uint32_t epoch) {
  const int n = min(*n_rows, max_rows);
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < n; p += warps) {
    bf16* dst = row_ptrs[p];
    if (dst == nullptr) continue;
    const bf16* src = y + static_cast<size_t>(p) * ldy;
    for (int c = lane; c < H / 8; c += 32) st_bf16x8(dst + c * 8, ld_bf16x8(src + c * 8));
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t old = atomicAdd(done_counter, 1u);
    if (old == gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < ep; ++r) st_release_sys_u32(flags.ret[r] + rank, epoch);
    }
  }
}

}  // namespace

// y [>= *n_rows, H] expert-sorted rows (row stride ldy); row_ptrs as written by pxl_ep_row_ptrs; flag_ptrs[r]:
// rank r's return-flag array; done_counter: local scratch, zero on entry (left zero).
PXL_EXPORT int pxl_ep_return_rows(const void* y, int64_t ldy, void* const* row_ptrs, const int* n_rows, int max_rows,
                                  int H, void* const* flag_ptrs, uint32_t* done_counter, int rank, int ep,
                                  uint32_t epoch, cudaStream_t stream) {
  if (ep < 1 || ep > 8 || rank < 0 || rank >= ep || H % 8 || ldy % 8 || max_rows <= 0) return PXL_ERR_INVALID_ARG;
  EpRetFlags f{};
  for (int i = 0; i < ep; ++i) f.ret[i] = static_cast<uint32_t*>(flag_ptrs[i]);
  int grid = pxl::ceil_div(max_rows, 8);
  const int max_grid = 2 * pxl_host::num_sms();
  if (grid > max_grid) grid = max_grid;
  ep_return_rows_kernel<<<grid, 256, 0, stream>>>(static_cast<const pxl::bf16*>(y), ldy,
                                                  reinterpret_cast<pxl::bf16* const*>(row_ptrs), n_rows, max_rows, H, f,
                                                  done_counter, rank, ep, epoch);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

// x [n_rows, H] (row stride ldx), ids [n_rows, k] global expert ids. recv_x_ptrs / recv_meta_ptrs /
// recv_cnt_ptrs / flag_ptrs: per-rank peer-mapped addresses of the receive regions. cursor [ep] and
// done_counter: local scratch, zero on entry (the kernel leaves them zero).
PXL_EXPORT int pxl_ep_dispatch(const void* x, int64_t ldx, const int* ids, int n_rows, int k, int H,
                               int experts_per_rank, int cap, int rank, int ep, void* const* recv_x_ptrs,
                               void* const* recv_meta_ptrs, void* const* recv_cnt_ptrs, void* const* flag_ptrs,
                               int* cursor, uint32_t* done_counter, uint32_t epoch, int* status,
                               cudaStream_t stream) {
  if (ep < 1 || ep > 8 || rank < 0 || rank >= ep || H % 8 || ldx % 8 || k <= 0 || cap <= 0) return PXL_ERR_INVALID_ARG;
  EpPeers peers{};
  for (int i = 0; i < ep; ++i) {
    peers.recv_x[i] = static_cast<pxl::bf16*>(recv_x_ptrs[i]);
    peers.recv_meta[i] = static_cast<int*>(recv_meta_ptrs[i]);
    peers.recv_cnt[i] = static_cast<int*>(recv_cnt_ptrs[i]);
    peers.disp_flag[i] = static_cast<uint32_t*>(flag_ptrs[i]);
  }
  const int pairs = n_rows > 0 ? n_rows * k : 0;
  int grid = pxl::ceil_div(pairs > 0 ? pairs : 1, 8);
  const int max_grid = 2 * pxl_host::num_sms();
  if (grid > max_grid) grid = max_grid;
  ep_dispatch_kernel<<<grid, 256, 0, stream>>>(static_cast<const pxl::bf16*>(x), ldx, ids, n_rows > 0 ? n_rows : 0, k, H,
                                               experts_per_rank, cap, rank, ep, peers, cursor, done_counter, epoch,
                                               status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_ep_recv_ids(const int* recv_meta, const int* recv_cnt, const void* disp_flag, int ep, int cap,
                               uint32_t epoch, int* ids_out, int* status, cudaStream_t stream) {
  if (ep < 1 || ep > 8 || cap <= 0) return PXL_ERR_INVALID_ARG;
  int grid = pxl::ceil_div(ep * cap, 256);
  if (grid > pxl_host::num_sms()) grid = pxl_host::num_sms();
  ep_recv_ids_kernel<<<grid, 256, 0, stream>>>(recv_meta, recv_cnt, static_cast<const uint32_t*>(disp_flag), ep, cap,
                                               epoch, ids_out, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_ep_row_ptrs(const int* src_slot, const int* n_rows, const int* recv_meta, int cap, int H, int ep,
                               void* const* comb_ptrs, void** row_ptrs, int max_rows, cudaStream_t stream) {
  if (ep < 1 || ep > 8 || max_rows <= 0) return PXL_ERR_INVALID_ARG;
  EpCombPtrs c{};
  for (int i = 0; i < ep; ++i) c.comb[i] = static_cast<pxl::bf16*>(comb_ptrs[i]);
  int grid = pxl::ceil_div(max_rows, 256);
  if (grid > pxl_host::num_sms()) grid = pxl_host::num_sms();
  ep_row_ptrs_kernel<<<grid, 256, 0, stream>>>(src_slot, n_rows, recv_meta, cap, H, c,
                                               reinterpret_cast<pxl::bf16**>(row_ptrs), max_rows);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_ep_combine(const void* comb, const float* w, const void* base, int64_t ld_base, void* out,
                              int64_t ld_out, const void* ret_flag, int ep, uint32_t epoch, int n_rows, int k, int H,
                              int* status, cudaStream_t stream) {
  if (ep < 1 || ep > 8 || H % 8) return PXL_ERR_INVALID_ARG;
  ep_combine_kernel<<<n_rows > 0 ? n_rows : 1, 256, 0, stream>>>(static_cast<const pxl::bf16*>(comb), w,
                                                static_cast<const pxl::bf16*>(base), ld_base,
                                                static_cast<pxl::bf16*>(out), ld_out,
                                                static_cast<const uint32_t*>(ret_flag), ep, epoch, n_rows > 0 ? n_rows : 0, k, H, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}
