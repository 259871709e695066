// Token sampling on the last pipeline stage: greedy arg-max and temperature /
// top-k / top-p / min-p sampling without a sort.
//
// Semantics follow the reference sampler, which sorts the softmax probabilities in
// descending order and keeps rank r iff r < top_k (top_k <= 0: no limit), the mass
// strictly before r is <= top_p, and p_r >= p_0 * min_p, then draws from the
// survivors (src/parallax/server/sampling/sampler.py:65-120). All three filters are
// monotone in rank, so the kept set is {p >= tau}; tau is found by bisection on the
// scaled logit, each probe being one block-wide count/mass reduction over the row.
#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

template <bool BF16>
__device__ __forceinline__ float load_logit(const void* row, int i) {
  if constexpr (BF16)
    return __bfloat162float(static_cast<const bf16*>(row)[i]);
  else
    return static_cast<const float*>(row)[i];
}

struct MaxIdx {
  float v;
  int i;
};
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

template <bool BF16>
__device__ MaxIdx block_argmax(const void* row, int V, MaxIdx* sm) {
  MaxIdx best{-INFINITY, 0x7fffffff};
  if constexpr (BF16) {
    const bf16* r = static_cast<const bf16*>(row);
    const bool aligned = (reinterpret_cast<uintptr_t>(r) & 15) == 0;
    const int nvec = aligned ? (V >> 3) : 0;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const bf16x8 a = ld_bf16x8(r + v * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(a.u[j]);
        best = better(best, MaxIdx{f.x, v * 8 + 2 * j});
        best = better(best, MaxIdx{f.y, v * 8 + 2 * j + 1});
      }
    }
    for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x)
      best = better(best, MaxIdx{__bfloat162float(r[i]), i});
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      best = better(best, MaxIdx{static_cast<const float*>(row)[i], i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sm[warp] = best;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  MaxIdx r = lane < nw ? sm[lane] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other{__shfl_xor_sync(0xffffffffu, r.v, o), __shfl_xor_sync(0xffffffffu, r.i, o)};
    r = better(r, other);
  }
  __syncthreads();
  return r;
}

template <bool BF16>
__device__ float block_sumexp(const void* row, int V, float mx, float inv_t, float* red) {
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x)
    s += __expf((load_logit<BF16>(row, i) - mx) * inv_t);
  return block_reduce_sum(s, red);
}

template <bool BF16>
__global__ void __launch_bounds__(1024)
argmax_kernel(const void* logits, int64_t ld, int V, int* out_ids, float* out_logprob, int* status) {
  __shared__ MaxIdx sm[32];
  __shared__ float red[32];
  const char* base = static_cast<const char*>(logits);
  const void* row = base + static_cast<size_t>(blockIdx.x) * ld * (BF16 ? 2 : 4);
  const MaxIdx r = block_argmax<BF16>(row, V, sm);
  if (r.i < 0 || r.i >= V) {
    // no logit of the row compared greater than -inf: the row is all NaN (or -inf). Report it and
    // hand out a valid id, so that nothing downstream indexes a table with the sentinel.
    if (threadIdx.x == 0) {
      if (status) atomicCAS(status, 0, PXL_DEV_NONFINITE_LOGITS);
      out_ids[blockIdx.x] = 0;
      if (out_logprob) out_logprob[blockIdx.x] = 0.f;
    }
    return;
  }
  if (threadIdx.x == 0) out_ids[blockIdx.x] = r.i;
  if (out_logprob) {
    const float z = block_sumexp<BF16>(row, V, r.v, 1.f, red);
    if (threadIdx.x == 0) out_logprob[blockIdx.x] = -logf(z);
  }
}

template <bool BF16>
__global__ void __launch_bounds__(1024)
sample_kernel(const void* logits, int64_t ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const float* __restrict__ uniform, int* out_ids,
              float* out_prob, int* status) {
  __shared__ MaxIdx sm[32];
  __shared__ float red[32];
  __shared__ float scan[1024];
  __shared__ int chosen;
  const int b = blockIdx.x;
  const char* base = static_cast<const char*>(logits);
  const void* row = base + static_cast<size_t>(b) * ld * (BF16 ? 2 : 4);
  const float temp = temperature ? temperature[b] : 1.f;
  const int k = top_k ? top_k[b] : 0;
  const float tp = top_p ? top_p[b] : 1.f;
  const float mp = min_p ? min_p[b] : 0.f;

  const MaxIdx best = block_argmax<BF16>(row, V, sm);
  if (best.i < 0 || best.i >= V) {  // all-NaN row: see argmax_kernel
    if (threadIdx.x == 0) {
      if (status) atomicCAS(status, 0, PXL_DEV_NONFINITE_LOGITS);
      out_ids[b] = 0;
      if (out_prob) out_prob[b] = 0.f;
    }
    return;
  }
  if (temp <= 0.f || k == 1) {
    if (threadIdx.x == 0) out_ids[b] = best.i;
    if (out_prob) {
      const float z = block_sumexp<BF16>(row, V, best.v, temp > 0.f ? 1.f / temp : 1.f, red);
      if (threadIdx.x == 0) out_prob[b] = 1.f / z;
    }
    return;
  }
  const float inv_t = 1.f / temp;
  const float Z = block_sumexp<BF16>(row, V, best.v, inv_t, red);

  // bisection on the scaled logit z = (l - max)/T in [-88, 0]
  float lo = -88.f, hi = 0.f;
  const float z_minp = mp > 0.f ? logf(mp) : -INFINITY;  // z >= log(min_p) <=> p >= pmax*min_p
  const bool need_search = (k > 0 && k < V) || tp < 1.f || mp > 0.f;
  if (need_search) {
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f, mass = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float z = (load_logit<BF16>(row, i) - best.v) * inv_t;
        if (z > mid) {
          cnt += 1.f;
          mass += __expf(z);
        }
      }
      cnt = block_reduce_sum(cnt, red);
      mass = block_reduce_sum(mass, red);
      const bool keep = (k <= 0 || cnt < static_cast<float>(k)) && (mass <= tp * Z) &&
                        (mid >= z_minp);
      if (keep) hi = mid; else lo = mid;
    }
  } else {
    lo = -INFINITY;
  }
  // The filters keep token i exactly when the condition above holds at mid = z_i (the tokens
  // strictly above it are fewer than k and weigh at most top_p). The condition flips at the
  // scaled logit of the last kept token: `hi` closes in on it from above and would leave that
  // token out, `lo` ends at most 88 / 2^26 below it, so the draw takes everything above `lo`.
  const float tau = lo;

  // draw: contiguous chunk per thread, block scan of chunk masses
  const int chunk = ceil_div(V, static_cast<int>(blockDim.x));
  const int i0 = threadIdx.x * chunk, i1 = min(V, i0 + chunk);
  float local = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float z = (load_logit<BF16>(row, i) - best.v) * inv_t;
    if (z >= tau) local += __expf(z);
  }
  scan[threadIdx.x] = local;
  if (threadIdx.x == 0) chosen = best.i;  // fallback (rounding at the tail)
  __syncthreads();
  // Hillis-Steele inclusive scan over 1024 entries
  for (int off = 1; off < blockDim.x; off <<= 1) {
    const float add = threadIdx.x >= off ? scan[threadIdx.x - off] : 0.f;
    __syncthreads();
    scan[threadIdx.x] += add;
    __syncthreads();
  }
  const float total = scan[blockDim.x - 1];
  const float target = uniform[b] * total;
  const float before = threadIdx.x ? scan[threadIdx.x - 1] : 0.f;
  const float after = scan[threadIdx.x];
  if (local > 0.f && target >= before && target < after) {
    float acc = before;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      const float z = (load_logit<BF16>(row, i) - best.v) * inv_t;
      if (z >= tau) {
        acc += __expf(z);
        pick = i;
        if (acc > target) break;
      }
    }
    if (pick >= 0) chosen = pick;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    out_ids[b] = chosen;
    if (out_prob)
      out_prob[b] = __expf((load_logit<BF16>(row, chosen) - best.v) * inv_t) / Z;
  }
}

// Repetition / presence / frequency penalties, in place on the logits of the rows that are about to be
// sampled. The host lists, per row, the distinct tokens the request has seen (CSR: row_off [B + 1], tok_ids,
// out_cnt = how often the token was GENERATED, 0 for tokens that only occur in the prompt):
//   repetition (prompt and output tokens):  l > 0 ? l / rep : l * rep
//   frequency, presence (output tokens):    l -= freq * count + pres
// Every (row, token) pair is listed once, so no two threads touch the same logit.
template <bool BF16>
__global__ void __launch_bounds__(256)
penalties_kernel(void* logits, int64_t ld, int V, const int* __restrict__ row_off, const int* __restrict__ tok_ids,
                 const int* __restrict__ out_cnt, const float* __restrict__ rep, const float* __restrict__ pres,
                 const float* __restrict__ freq, int* status) {
  const int b = blockIdx.x;
  const float r = rep[b], p = pres[b], f = freq[b];
  for (int j = row_off[b] + threadIdx.x; j < row_off[b + 1]; j += blockDim.x) {
    const int t = tok_ids[j];
    if (t < 0 || t >= V) {
      if (status) atomicCAS(status, 0, PXL_DEV_BAD_ROW_ID);
      continue;
    }
    const size_t at = static_cast<size_t>(b) * ld + t;
    float l = BF16 ? __bfloat162float(static_cast<bf16*>(logits)[at]) : static_cast<float*>(logits)[at];
    if (r != 1.f) l = l > 0.f ? l / r : l * r;
    const int c = out_cnt[j];
    if (c > 0) l -= f * static_cast<float>(c) + p;
    if (BF16) static_cast<bf16*>(logits)[at] = __float2bfloat16(l);
    else static_cast<float*>(logits)[at] = l;
  }
}

}  // namespace

PXL_EXPORT int pxl_apply_penalties(void* logits, int logits_bf16, int64_t ld, int B, int V, const int* row_off,
                                   const int* tok_ids, const int* out_cnt, const float* rep, const float* pres,
                                   const float* freq, int* status, pxl_stream_t stream) {
  if (B <= 0) return PXL_OK;
  if (!row_off || !tok_ids || !out_cnt || !rep || !pres || !freq) return PXL_ERR_INVALID_ARG;
  if (logits_bf16)
    penalties_kernel<true><<<B, 256, 0, stream>>>(logits, ld, V, row_off, tok_ids, out_cnt, rep, pres, freq, status);
  else
    penalties_kernel<false><<<B, 256, 0, stream>>>(logits, ld, V, row_off, tok_ids, out_cnt, rep, pres, freq, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_argmax(const void* logits, int logits_bf16, int64_t ld, int B, int V,
                          int* out_ids, float* out_logprob, int* status, pxl_stream_t stream) {
  if (B <= 0) return PXL_OK;
  if (logits_bf16)
    argmax_kernel<true><<<B, 1024, 0, stream>>>(logits, ld, V, out_ids, out_logprob, status);
  else
    argmax_kernel<false><<<B, 1024, 0, stream>>>(logits, ld, V, out_ids, out_logprob, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_sample(const void* logits, int logits_bf16, int64_t ld, int B, int V,
                          const float* temperature, const int* top_k, const float* top_p,
                          const float* min_p, const float* uniform, int* out_ids, float* out_prob,
                          int* status, pxl_stream_t stream) {
  if (B <= 0) return PXL_OK;
  if (!uniform) return PXL_ERR_INVALID_ARG;
  if (logits_bf16)
    sample_kernel<true><<<B, 1024, 0, stream>>>(logits, ld, V, temperature, top_k, top_p, min_p,
                                                uniform, out_ids, out_prob, status);
  else
    sample_kernel<false><<<B, 1024, 0, stream>>>(logits, ld, V, temperature, top_k, top_p, min_p,
                                                 uniform, out_ids, out_prob, status);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}
