// Gated DeltaNet linear-attention layers (Qwen3-Next / Qwen3.5 hybrids): short causal convolution
// with a carried window, and the gated delta-rule recurrence with a per-request state matrix.
//
//   conv:   y[t, c] = silu( sum_j w[c, j] * u[t - (K-1) + j, c] ),  u = [carried window | x]
//   delta:  S <- S * exp(g_t);  d = (v_t - S k_t) * beta_t;  S <- S + d k_t^T;  o_t = S q_t
//           g_t = -exp(A_log) * softplus(a_t + dt_bias),  beta_t = sigmoid(b_t)
//           q, k are l2-normalised (eps 1e-6 on the sum of squares); q is scaled by Dk^-1/2;
//           out = rmsnorm(o_t) * norm_w * silu(z_t)
// State lives in per-request slots (not pages): conv window [slots, C, K-1] bf16, recurrent
// state [slots, Hv, Dv, Dk] fp32. A sequence whose first token of this step sits at position 0
// starts from a zero state. The reference runs these layers through mlx-lm's
// gated_delta_update (src/parallax/models/qwen3_next.py:149-230) and keeps the states in a
// LinearCache (src/parallax/server/cache/linear_cache.py).
#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

constexpr int kMaxConvK = 8;

// grid (channel blocks, sequences); thread = one channel, walks the sequence's tokens in order
__global__ void __launch_bounds__(128) conv1d_silu_kernel(const bf16* __restrict__ x, int64_t ldx,
                                                          const bf16* __restrict__ w, const bf16* __restrict__ bias,
                                                          bf16* __restrict__ conv_state, const int* __restrict__ seq_cu,
                                                          const int* __restrict__ seq_slots,
                                                          const int* __restrict__ positions, bf16* __restrict__ out,
                                                          int64_t ldo, int C, int K) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C) return;
  const int t0 = seq_cu[b], t1 = seq_cu[b + 1];
  if (t1 <= t0) return;
  const int slot = seq_slots[b];
  const bool fresh = positions[t0] == 0;
  float win[kMaxConvK];  // win[0..K-2] = previous inputs, oldest first
  float wk[kMaxConvK];
  bf16* st = conv_state + (static_cast<size_t>(slot) * C + c) * (K - 1);
  for (int j = 0; j < K - 1; ++j) win[j] = fresh ? 0.f : __bfloat162float(st[j]);
  for (int j = 0; j < K; ++j) wk[j] = __bfloat162float(w[c * K + j]);
  const float bs = bias ? __bfloat162float(bias[c]) : 0.f;
  for (int t = t0; t < t1; ++t) {
    const float xin = __bfloat162float(x[t * ldx + c]);
    float acc = bs + wk[K - 1] * xin;
    for (int j = 0; j < K - 1; ++j) acc += wk[j] * win[j];
    for (int j = 0; j + 1 < K - 1; ++j) win[j] = win[j + 1];
    win[K - 2] = xin;
    out[t * ldo + c] = __float2bfloat16(acc / (1.f + __expf(-acc)));
  }
  for (int j = 0; j < K - 1; ++j) st[j] = __float2bfloat16(win[j]);
}

// grid (value heads, sequences), Dv threads; thread i owns row i of the state matrix [Dv, Dk]
template <int DK>
__global__ void __launch_bounds__(128) gated_delta_kernel(const bf16* __restrict__ qkv, int64_t ld_qkv,
                                                          const bf16* __restrict__ a_in, const bf16* __restrict__ b_in,
                                                          int64_t ld_ab, const float* __restrict__ A_log,
                                                          const float* __restrict__ dt_bias, const bf16* __restrict__ z,
                                                          int64_t ld_z, const bf16* __restrict__ norm_w,
                                                          float* __restrict__ rec_state, const int* __restrict__ seq_cu,
                                                          const int* __restrict__ seq_slots,
                                                          const int* __restrict__ positions, bf16* __restrict__ out,
                                                          int64_t ld_out, int Hk, int Hv, int Dv, float eps) {
  __shared__ float qs[DK], ks[DK];
  __shared__ float red[32];
  const int hv = blockIdx.x, b = blockIdx.y;
  const int i = threadIdx.x;  // row of S / element of v, z, out
  const int t0 = seq_cu[b], t1 = seq_cu[b + 1];
  if (t1 <= t0) return;
  const int hk = hv / (Hv / Hk);
  const int slot = seq_slots[b];
  const bool fresh = positions[t0] == 0;
  float* Sg = rec_state + ((static_cast<size_t>(slot) * Hv + hv) * Dv + i) * DK;
  float S[DK];
  if (i < Dv) {
#pragma unroll
    for (int j = 0; j < DK; j += 4) {
      const float4 v4 = fresh ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(Sg + j);
      S[j] = v4.x; S[j + 1] = v4.y; S[j + 2] = v4.z; S[j + 3] = v4.w;
    }
  }
  const float neg_a = -__expf(A_log[hv]);
  const float dtb = dt_bias[hv];
  const float nw = i < Dv ? __bfloat162float(norm_w[i]) : 0.f;
  const int q_off = hk * DK, k_off = Hk * DK + hk * DK, v_off = 2 * Hk * DK + hv * Dv;
  const float inv_scale = rsqrtf(static_cast<float>(DK));
  for (int t = t0; t < t1; ++t) {
    const bf16* row = qkv + t * ld_qkv;
    // q, k of this key head: l2-normalise and scale
    float qv = 0.f, kv = 0.f;
    if (i < DK) {
      qv = __bfloat162float(row[q_off + i]);
      kv = __bfloat162float(row[k_off + i]);
    }
    const float q2 = block_reduce_sum(qv * qv, red);
    const float k2 = block_reduce_sum(kv * kv, red);
    if (i < DK) {
      qs[i] = qv * rsqrtf(q2 + 1e-6f) * inv_scale;  // l2-normalised, then scaled by Dk^-1/2
      ks[i] = kv * rsqrtf(k2 + 1e-6f);
    }
    __syncthreads();
    const float av = __bfloat162float(a_in[t * ld_ab + hv]) + dtb;
    const float sp = av > 20.f ? av : log1pf(__expf(av));
    const float decay = __expf(neg_a * sp);
    const float beta = 1.f / (1.f + __expf(-__bfloat162float(b_in[t * ld_ab + hv])));
    float o = 0.f;
    if (i < Dv) {
      float mem = 0.f;
#pragma unroll
      for (int j = 0; j < DK; ++j) {
        S[j] *= decay;
        mem = fmaf(S[j], ks[j], mem);
      }
      const float d = (__bfloat162float(row[v_off + i]) - mem) * beta;
#pragma unroll
      for (int j = 0; j < DK; ++j) {
        S[j] = fmaf(d, ks[j], S[j]);
        o = fmaf(S[j], qs[j], o);
      }
    }
    // gated RMSNorm over the head's Dv outputs
    const float o2 = block_reduce_sum(i < Dv ? o * o : 0.f, red);
    if (i < Dv) {
      const float zz = __bfloat162float(z[t * ld_z + hv * Dv + i]);
      const float y = o * rsqrtf(o2 / Dv + eps) * nw * (zz / (1.f + __expf(-zz)));
      out[t * ld_out + hv * Dv + i] = __float2bfloat16(y);
    }
    __syncthreads();
  }
  if (i < Dv) {
#pragma unroll
    for (int j = 0; j < DK; j += 4) *reinterpret_cast<float4*>(Sg + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
  }
}

__global__ void sigmoid_gate_mul_kernel(const bf16* __restrict__ x, int64_t ldx, const bf16* __restrict__ gate,
                                        int64_t ldg, bf16* __restrict__ out, int64_t ldo, int n8) {
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < n8; v += blockDim.x) {
    const bf16x8 a = ld_bf16x8(x + t * ldx + v * 8), g = ld_bf16x8(gate + t * ldg + v * 8);
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 av = unpack_bf16x2(a.u[j]), gv = unpack_bf16x2(g.u[j]);
      o.u[j] = pack_bf16x2(av.x / (1.f + __expf(-gv.x)), av.y / (1.f + __expf(-gv.y)));
    }
    st_bf16x8(out + t * ldo + v * 8, o);
  }
}

// out = (res +) x * sigmoid(gate[:, col / group]): one gate value per `group` consecutive columns (a head of the
// attention output, or a whole row for the shared expert's scalar gate); group is a multiple of 8
__global__ void gate_mul_grouped_kernel(const bf16* __restrict__ x, int64_t ldx, const bf16* __restrict__ gate,
                                        int64_t ldg, const bf16* __restrict__ res, int64_t ldr,
                                        bf16* __restrict__ out, int64_t ldo, int n8, int group8) {
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < n8; v += blockDim.x) {
    const float g = __bfloat162float(gate[t * ldg + v / group8]);
    const float s = 1.f / (1.f + __expf(-g));
    const bf16x8 a = ld_bf16x8(x + t * ldx + v * 8);
    bf16x8 r;
    if (res != nullptr) r = ld_bf16x8(res + t * ldr + v * 8);
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 av = unpack_bf16x2(a.u[j]);
      float2 ov = make_float2(av.x * s, av.y * s);
      if (res != nullptr) {
        const float2 rv = unpack_bf16x2(r.u[j]);
        ov.x += rv.x;
        ov.y += rv.y;
      }
      o.u[j] = pack_bf16x2(ov.x, ov.y);
    }
    st_bf16x8(out + t * ldo + v * 8, o);
  }
}

// out[t] = x[t, :] . w  (one warp per row; the one-column projection of a scalar gate is too thin for a GEMM tile)
__global__ void row_dot_kernel(const bf16* __restrict__ x, int64_t ldx, const bf16* __restrict__ w,
                               bf16* __restrict__ out, int T, int k8) {
  const int t = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (t >= T) return;
  const int lane = threadIdx.x % 32;
  float acc = 0.f;
  for (int v = lane; v < k8; v += 32) {
    const bf16x8 a = ld_bf16x8(x + t * ldx + v * 8), b = ld_bf16x8(w + v * 8);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 av = unpack_bf16x2(a.u[j]), bv = unpack_bf16x2(b.u[j]);
      acc += av.x * bv.x + av.y * bv.y;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[t] = __float2bfloat16(acc);
}

}  // namespace

PXL_EXPORT int pxl_causal_conv1d_silu(const void* x, int64_t ldx, const void* w, const void* bias, void* conv_state,
                                      const int* seq_cu, const int* seq_slots, const int* positions, void* out,
                                      int64_t ldo, int B, int C, int K, cudaStream_t stream) {
  if (B <= 0) return PXL_OK;
  if (K < 2 || K > kMaxConvK) return PXL_ERR_INVALID_ARG;
  dim3 grid(pxl::ceil_div(C, 128), B);
  conv1d_silu_kernel<<<grid, 128, 0, stream>>>(static_cast<const pxl::bf16*>(x), ldx, static_cast<const pxl::bf16*>(w),
                                               static_cast<const pxl::bf16*>(bias), static_cast<pxl::bf16*>(conv_state),
                                               seq_cu, seq_slots, positions, static_cast<pxl::bf16*>(out), ldo, C, K);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_gated_delta_rule(const void* qkv, int64_t ld_qkv, const void* a, const void* b, int64_t ld_ab,
                                    const float* A_log, const float* dt_bias, const void* z, int64_t ld_z,
                                    const void* norm_w, float* rec_state, const int* seq_cu, const int* seq_slots,
                                    const int* positions, void* out, int64_t ld_out, int B, int Hk, int Hv, int Dk,
                                    int Dv, float eps, cudaStream_t stream) {
  if (B <= 0) return PXL_OK;
  if (Dk != 128 || Dv > 128 || Dv <= 0 || Hk <= 0 || Hv % Hk) return PXL_ERR_INVALID_ARG;
  dim3 grid(Hv, B);
  gated_delta_kernel<128><<<grid, 128, 0, stream>>>(
      static_cast<const pxl::bf16*>(qkv), ld_qkv, static_cast<const pxl::bf16*>(a), static_cast<const pxl::bf16*>(b),
      ld_ab, A_log, dt_bias, static_cast<const pxl::bf16*>(z), ld_z, static_cast<const pxl::bf16*>(norm_w), rec_state,
      seq_cu, seq_slots, positions, static_cast<pxl::bf16*>(out), ld_out, Hk, Hv, Dv, eps);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_sigmoid_gate_mul(const void* x, int64_t ldx, const void* gate, int64_t ldg, void* out,
                                    int64_t ldo, int T, int N, cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (N % 8) return PXL_ERR_INVALID_ARG;
  sigmoid_gate_mul_kernel<<<T, 128, 0, stream>>>(static_cast<const pxl::bf16*>(x), ldx,
                                                 static_cast<const pxl::bf16*>(gate), ldg,
                                                 static_cast<pxl::bf16*>(out), ldo, N / 8);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_gate_mul_grouped(const void* x, int64_t ldx, const void* gate, int64_t ldg, const void* res,
                                    int64_t ldr, void* out, int64_t ldo, int T, int N, int group,
                                    cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (N % 8 || group <= 0 || group % 8 || N % group) return PXL_ERR_INVALID_ARG;
  gate_mul_grouped_kernel<<<T, 128, 0, stream>>>(static_cast<const pxl::bf16*>(x), ldx,
                                                 static_cast<const pxl::bf16*>(gate), ldg,
                                                 static_cast<const pxl::bf16*>(res), ldr,
                                                 static_cast<pxl::bf16*>(out), ldo, N / 8, group / 8);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}

PXL_EXPORT int pxl_row_dot(const void* x, int64_t ldx, const void* w, void* out, int T, int K, cudaStream_t stream) {
  if (T <= 0) return PXL_OK;
  if (K % 8) return PXL_ERR_INVALID_ARG;
  row_dot_kernel<<<pxl::ceil_div(T, 4), 128, 0, stream>>>(static_cast<const pxl::bf16*>(x), ldx,
                                                          static_cast<const pxl::bf16*>(w),
                                                          static_cast<pxl::bf16*>(out), T, K / 8);
  return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA;
}
