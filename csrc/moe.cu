// Mixture-of-experts support kernels: top-k routing, token permutation (alignment to
// 128-row expert tiles), gather, and weighted combine. The expert FFNs themselves run on the
// grouped tcgen05 GEMM (gemm_tcgen05.cu).
//
// Routing semantics:
//   mode 0  softmax over all experts, top-k, optional renormalisation (Qwen3-MoE, GPT-OSS
//           style; the reference gets it from mlx-lm's switch layers, src/parallax/models/
//           qwen3_moe.py)
//   mode 1  sigmoid scores, selection on score + per-expert correction bias with optional
//           group-limited routing, weights = unbiased scores renormalised and scaled
//           (DeepSeek-V3 "noaux_tc"; MiniMax-M3 uses the ungrouped form,
//           src/parallax/models/minimax_m3.py:155-173)
#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

constexpr int kMaxEPL = 16;  // experts per lane: supports up to 512 experts

template <bool BF16>
__device__ __forceinline__ float load_score(const void* p, size_t i) {
  if constexpr (BF16) return __bfloat162float(static_cast<const bf16*>(p)[i]);
  else return static_cast<const float*>(p)[i];
}

// One warp per token.
template <bool BF16>
__global__ void __launch_bounds__(128)
moe_route_kernel(const void* __restrict__ logits, const float* __restrict__ e_bias, int T, int E,
                 int k, int mode, int renorm, int n_group, int topk_group, float routed_scale,
                 int* __restrict__ out_ids, float* __restrict__ out_w) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= T) return;
  const int epl = (E + 31) / 32;
  float s[kMaxEPL];    // unbiased score (softmax prob or sigmoid)
  float sel[kMaxEPL];  // selection score
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxEPL; ++j) {
    const int e = j * 32 + lane;
    s[j] = (j < epl && e < E) ? load_score<BF16>(logits, static_cast<size_t>(t) * E + e) : -INFINITY;
    mx = fmaxf(mx, s[j]);
  }
  if (mode == 0) {
    mx = warp_reduce_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxEPL; ++j) {
      s[j] = (s[j] == -INFINITY) ? 0.f : __expf(s[j] - mx);
      sum += s[j];
    }
    sum = warp_reduce_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < kMaxEPL; ++j) {
      const int e = j * 32 + lane;
      s[j] *= inv;
      sel[j] = (j < epl && e < E) ? s[j] : -INFINITY;
    }
  } else {
#pragma unroll
    for (int j = 0; j < kMaxEPL; ++j) {
      const int e = j * 32 + lane;
      const bool ok = j < epl && e < E;
      s[j] = ok ? 1.f / (1.f + __expf(-s[j])) : 0.f;
      sel[j] = ok ? s[j] + (e_bias ? e_bias[e] : 0.f) : -INFINITY;
    }
    if (n_group > 1 && topk_group < n_group) {
      // group score = sum of the two best selection scores inside the group
      const int gsize = E / n_group;
      float gscore_mine = -INFINITY;  // lane g (< n_group) holds the score of group g
      for (int g = 0; g < n_group; ++g) {
        float b1 = -INFINITY, b2 = -INFINITY;
#pragma unroll
        for (int j = 0; j < kMaxEPL; ++j) {
          const int e = j * 32 + lane;
          if (j < epl && e < E && e / gsize == g) {
            if (sel[j] > b1) { b2 = b1; b1 = sel[j]; }
            else if (sel[j] > b2) b2 = sel[j];
          }
        }
        // merge (b1, b2) pairs across lanes
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float o1 = __shfl_xor_sync(0xffffffffu, b1, o);
          const float o2 = __shfl_xor_sync(0xffffffffu, b2, o);
          const float n1 = fmaxf(b1, o1);
          const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
          b1 = n1; b2 = n2;
        }
        if (lane == g) gscore_mine = b1 + (b2 == -INFINITY ? 0.f : b2);
      }
      // pick topk_group groups; keep a bitmask of allowed groups (n_group <= 32)
      unsigned allowed = 0;
      float gs = lane < n_group ? gscore_mine : -INFINITY;
      for (int it = 0; it < topk_group; ++it) {
        float best = gs;
        int arg = lane;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
          if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        allowed |= 1u << arg;
        if (lane == arg) gs = -INFINITY;
      }
#pragma unroll
      for (int j = 0; j < kMaxEPL; ++j) {
        const int e = j * 32 + lane;
        if (j < epl && e < E && !((allowed >> (e / gsize)) & 1u)) sel[j] = -INFINITY;
      }
    }
  }
  // iterative top-k over the warp
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int it = 0; it < k; ++it) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    float best_s = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxEPL; ++j) {
      const int e = j * 32 + lane;
      if (j < epl && e < E && (sel[j] > best || (sel[j] == best && e < arg))) {
        best = sel[j]; arg = e; best_s = s[j];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; best_s = os; }
    }
    if (arg != 0x7fffffff && (arg & 31) == lane) {
#pragma unroll
      for (int j = 0; j < kMaxEPL; ++j)
        if (j == (arg >> 5)) sel[j] = -INFINITY;  // static indices keep sel[] in registers
    }
    wsum += best_s;
    if (lane == it) { my_w = best_s; my_id = arg == 0x7fffffff ? 0 : arg; }
  }
  if (lane < k) {
    float w = my_w;
    if (renorm) w = w / fmaxf(wsum, 1e-20f);
    out_ids[static_cast<size_t>(t) * k + lane] = my_id;
    out_w[static_cast<size_t>(t) * k + lane] = w * routed_scale;
  }
}

// ------------------------------------------------------------------ alignment
// counts[e] = number of (token, slot) pairs routed to expert e (ids < 0 or >= E are skipped)
__global__ void moe_count_kernel(const int* __restrict__ ids, int n, int E, int e_lo, int e_hi,
                                 int* __restrict__ counts) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = ids[i];
  if (e >= e_lo && e < e_hi && e < E) atomicAdd(&counts[e - e_lo], 1);
}

// Single block: exclusive scan of counts into 128-aligned... no padding is inserted: segments are
// contiguous; m-tiles are listed per expert. Writes offsets[E+1], the m-tile list and num_mt,
// and resets cursor[e] = offsets[e].
__global__ void __launch_bounds__(1024)
moe_scan_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                int* __restrict__ cursor, int* __restrict__ mt_expert, int* __restrict__ mt_row0,
                int* __restrict__ mt_row_end, int* __restrict__ num_mt, int max_mt) {
  __shared__ int s_off[1025];
  __shared__ int s_mt[1025];
  const int tid = threadIdx.x;
  // serial scan by thread 0 is fine for E <= 1024 (a few microseconds)
  if (tid == 0) {
    int o = 0, m = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = o;
      s_mt[e] = m;
      o += counts[e];
      m += (counts[e] + 127) / 128;
    }
    s_off[E] = o;
    s_mt[E] = m;
    *num_mt = m < max_mt ? m : max_mt;
  }
  __syncthreads();
  for (int e = tid; e <= E; e += blockDim.x) offsets[e] = s_off[e];
  for (int e = tid; e < E; e += blockDim.x) {
    cursor[e] = s_off[e];
    const int n_t = s_mt[e + 1] - s_mt[e];
    for (int i = 0; i < n_t; ++i) {
      const int mt = s_mt[e] + i;
      if (mt < max_mt) {
        mt_expert[mt] = e;
        mt_row0[mt] = s_off[e] + i * 128;
        mt_row_end[mt] = s_off[e + 1];
      }
    }
  }
}

// pos_of[i] = row of pair i in the permuted matrix (or -1), src_tok[row] = token of that row
__global__ void moe_place_kernel(const int* __restrict__ ids, int n, int k, int E, int e_lo,
                                 int e_hi, int* __restrict__ cursor, int* __restrict__ pos_of,
                                 int* __restrict__ src_tok) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = ids[i];
  if (e >= e_lo && e < e_hi && e < E) {
    const int p = atomicAdd(&cursor[e - e_lo], 1);
    pos_of[i] = p;
    src_tok[p] = i / k;
  } else {
    pos_of[i] = -1;
  }
}

// x_perm[p, :] = x[src_tok[p], :]   for p < *n_rows
__global__ void __launch_bounds__(128)
moe_gather_kernel(const bf16* __restrict__ x, const int* __restrict__ src_tok,
                  const int* __restrict__ n_rows, bf16* __restrict__ x_perm, int H) {
  const int p = blockIdx.x;
  if (p >= *n_rows) return;
  const bf16* src = x + static_cast<size_t>(src_tok[p]) * H;
  bf16* dst = x_perm + static_cast<size_t>(p) * H;
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x)
    st_bf16x8(dst + v * 8, ld_bf16x8(src + v * 8));
}

// out[t, :] = (base ? base[t, :] : 0) + sum_j w[t, j] * y_perm[pos_of[t*k + j], :]
__global__ void __launch_bounds__(256)
moe_combine_kernel(const bf16* __restrict__ y_perm, const int* __restrict__ pos_of,
                   const float* __restrict__ w, const bf16* __restrict__ base,
                   bf16* __restrict__ out, int k, int H) {
  const size_t t = blockIdx.x;
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) {
    float acc[8];
    if (base) {
      const bf16x8 b = ld_bf16x8(base + t * H + v * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(b.u[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    for (int s = 0; s < k; ++s) {
      const int p = pos_of[t * k + s];
      if (p < 0) continue;
      const float ws = w[t * k + s];
      const bf16x8 y = ld_bf16x8(y_perm + static_cast<size_t>(p) * H + v * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(y.u[j]);
        acc[2 * j] += ws * f.x;
        acc[2 * j + 1] += ws * f.y;
      }
    }
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) o.u[j] = pack_bf16x2(acc[2 * j], acc[2 * j + 1]);
    st_bf16x8(out + t * H + v * 8, o);
  }
}

inline int check_launch() { return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA; }

}  // namespace

PXL_EXPORT int pxl_moe_route(const void* logits, int logits_bf16, const float* e_bias, int T, int E,
                             int k, int mode, int renorm, int n_group, int topk_group,
                             float routed_scale, int* out_ids, float* out_w, pxl_stream_t stream) {
  if (T <= 0) return PXL_OK;
  if (E <= 0 || E > 32 * kMaxEPL || k <= 0 || k > 32 || k > E) return PXL_ERR_INVALID_ARG;
  if (n_group > 32 || (n_group > 1 && E % n_group)) return PXL_ERR_INVALID_ARG;
  const unsigned grid = (T + 3) / 4;
  if (logits_bf16)
    moe_route_kernel<true><<<grid, 128, 0, stream>>>(logits, e_bias, T, E, k, mode, renorm, n_group,
                                                     topk_group, routed_scale, out_ids, out_w);
  else
    moe_route_kernel<false><<<grid, 128, 0, stream>>>(logits, e_bias, T, E, k, mode, renorm,
                                                      n_group, topk_group, routed_scale, out_ids,
                                                      out_w);
  return check_launch();
}

// Build the expert-sorted layout for experts [e_lo, e_hi) (all experts: 0, E).
// ids [T*k]; counts/cursor [n_local]; offsets [n_local+1]; m-tile arrays [max_mt]; pos_of [T*k];
// src_tok [T*k]. `counts` must be zero on entry.
PXL_EXPORT int pxl_moe_align(const int* ids, int T, int k, int E, int e_lo, int e_hi, int* counts,
                             int* offsets, int* cursor, int* mt_expert, int* mt_row0,
                             int* mt_row_end, int* num_mt, int max_mt, int* pos_of, int* src_tok,
                             pxl_stream_t stream) {
  const int n = T * k;
  const int n_local = e_hi - e_lo;
  if (n <= 0 || n_local <= 0 || n_local > 1024) return PXL_ERR_INVALID_ARG;
  const unsigned grid = (n + 255) / 256;
  moe_count_kernel<<<grid, 256, 0, stream>>>(ids, n, E, e_lo, e_hi, counts);
  moe_scan_kernel<<<1, 1024, 0, stream>>>(counts, n_local, offsets, cursor, mt_expert, mt_row0,
                                          mt_row_end, num_mt, max_mt);
  moe_place_kernel<<<grid, 256, 0, stream>>>(ids, n, k, E, e_lo, e_hi, cursor, pos_of, src_tok);
  return check_launch();
}

PXL_EXPORT int pxl_moe_gather(const void* x, const int* src_tok, const int* n_rows, void* x_perm,
                              int max_rows, int H, pxl_stream_t stream) {
  if (max_rows <= 0) return PXL_OK;
  if (H % 8) return PXL_ERR_INVALID_ARG;
  moe_gather_kernel<<<max_rows, 128, 0, stream>>>(static_cast<const bf16*>(x), src_tok, n_rows,
                                                  static_cast<bf16*>(x_perm), H);
  return check_launch();
}

PXL_EXPORT int pxl_moe_combine(const void* y_perm, const int* pos_of, const float* w,
                               const void* base, void* out, int T, int k, int H,
                               pxl_stream_t stream) {
  if (T <= 0) return PXL_OK;
  if (H % 8) return PXL_ERR_INVALID_ARG;
  moe_combine_kernel<<<T, 256, 0, stream>>>(static_cast<const bf16*>(y_perm), pos_of, w,
                                            static_cast<const bf16*>(base),
                                            static_cast<bf16*>(out), k, H);
  return check_launch();
}
