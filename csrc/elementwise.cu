// Memory-bound elementwise / normalisation kernels: RMSNorm(+residual), fused per-head
// q/k-norm + RoPE + paged-cache scatter, activation-and-multiply, row gather.
//
// These replace what the reference reaches through third-party GPU layers
// (RMSNorm / RoPE / SiLU-mul, src/parallax/server/executor/sglang_executor.py:419-452)
// and its own Metal cache-scatter kernel
// (src/parallax_extensions/kernels/reshape_and_cache/reshape_and_cache.metal:32-96).
#include <cuda_fp8.h>

#include <type_traits>

#include "common.cuh"
#include "pxl_api.h"

namespace {
using namespace pxl;

// ----------------------------------------------------------------------------- RMSNorm
template <bool HAS_RES>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ out,
               bf16* __restrict__ residual, int H, float eps, float w_offset) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const size_t row = blockIdx.x;
  const bf16* xr = x + row * H;
  bf16* rr = HAS_RES ? residual + row * H : nullptr;
  bf16* outr = out + row * H;
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    bf16x8 a = ld_bf16x8(xr + v * 8);
    if constexpr (HAS_RES) {
      const bf16x8 b = ld_bf16x8(rr + v * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = unpack_bf16x2(a.u[j]);
        const float2 fb = unpack_bf16x2(b.u[j]);
        a.u[j] = pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
      }
      st_bf16x8(rr + v * 8, a);  // the sum (rounded to bf16) is the new residual stream
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(a.u[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = block_reduce_sum(ss, red);
  const float inv = rsqrtf(ss / static_cast<float>(H) + eps);
  const bf16* src = HAS_RES ? rr : xr;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const bf16x8 a = ld_bf16x8(src + v * 8);
    const bf16x8 ww = ld_bf16x8(w + v * 8);
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(a.u[j]);
      const float2 g = unpack_bf16x2(ww.u[j]);
      o.u[j] = pack_bf16x2(f.x * inv * (g.x + w_offset), f.y * inv * (g.y + w_offset));
    }
    st_bf16x8(outr + v * 8, o);
  }
}

// One warp per row, the row held in registers between the sum of squares and the scaling: one read
// and one write of every element, no block-wide barrier. NV = 16-byte vectors per lane (H <= NV * 256).
template <bool HAS_RES, int NV>
__global__ void __launch_bounds__(256)
rmsnorm_warp_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ out,
                    bf16* __restrict__ residual, int T, int H, float eps, float w_offset) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= T) return;
  const bf16* xr = x + static_cast<size_t>(row) * H;
  bf16* rr = HAS_RES ? residual + static_cast<size_t>(row) * H : nullptr;
  bf16* outr = out + static_cast<size_t>(row) * H;
  const int nvec = H >> 3;
  bf16x8 a[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) a[i] = ld_bf16x8(xr + v * 8);
  }
  if constexpr (HAS_RES) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        const bf16x8 b = ld_bf16x8(rr + v * 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = unpack_bf16x2(a[i].u[j]);
          const float2 fb = unpack_bf16x2(b.u[j]);
          a[i].u[j] = pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
        }
        st_bf16x8(rr + v * 8, a[i]);  // the sum (rounded to bf16) is the new residual stream
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + 32 * i < nvec) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(a[i].u[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = rsqrtf(ss / static_cast<float>(H) + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      const bf16x8 ww = ld_bf16x8(w + v * 8);
      bf16x8 o;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(a[i].u[j]);
        const float2 g = unpack_bf16x2(ww.u[j]);
        o.u[j] = pack_bf16x2(f.x * inv * (g.x + w_offset), f.y * inv * (g.y + w_offset));
      }
      st_bf16x8(outr + v * 8, o);
    }
  }
}

// Row-strided variant (rows of a column slice of a wider matrix; in place when out == x).
__global__ void __launch_bounds__(256)
rmsnorm_strided_kernel(const bf16* __restrict__ x, int64_t ldx, const bf16* __restrict__ w, bf16* __restrict__ out,
                       int64_t ldo, int H, float eps, float w_offset) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const bf16* xr = x + row * ldx;
  bf16* outr = out + row * ldo;
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const bf16x8 a = ld_bf16x8(xr + v * 8);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(a.u[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = block_reduce_sum(ss, red);
  const float inv = rsqrtf(ss / static_cast<float>(H) + eps);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const bf16x8 a = ld_bf16x8(xr + v * 8);
    const bf16x8 ww = ld_bf16x8(w + v * 8);
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(a.u[j]);
      const float2 g = unpack_bf16x2(ww.u[j]);
      o.u[j] = pack_bf16x2(f.x * inv * (g.x + w_offset), f.y * inv * (g.y + w_offset));
    }
    st_bf16x8(outr + v * 8, o);
  }
}

// ------------------------------------------------- q/k norm + RoPE + cache scatter
// One warp per (token, head slot). Head slots: [0,Hq) q heads, [Hq,Hq+Hkv) k heads,
// [Hq+Hkv, Hq+2Hkv) v heads. D <= 256, D % 32 == 0... each lane owns D/32 contiguous dims.
// FP8: the caches hold e4m3 bytes; a value is stored as value * inv_scale (saturating), the
// attention kernels multiply by the scale again when they read it (the reference's optional
// fp8 cache: src/parallax_extensions/kernels/reshape_and_cache/reshape_and_cache.metal:32-96).
__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

template <int D, bool FP8 = false>
__global__ void __launch_bounds__(256)
qk_norm_rope_cache_kernel(bf16* __restrict__ qkv, const bf16* __restrict__ q_norm_w,
                          const bf16* __restrict__ k_norm_w, const float* __restrict__ cos_sin,
                          const int* __restrict__ positions,
                          const int64_t* __restrict__ slot_mapping, void* __restrict__ k_cache,
                          void* __restrict__ v_cache, int T, int Hq, int Hkv, int rot_dim,
                          int page_size, int64_t num_slots, float eps, float w_offset,
                          float k_inv_scale, float v_inv_scale, int max_pos, int* status) {
  constexpr int EPL = D / 32;  // elements per lane
  __shared__ float sh[8][D];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = Hq + 2 * Hkv;
  const int64_t gw = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  if (gw >= static_cast<int64_t>(T) * heads) return;
  const int t = static_cast<int>(gw / heads);
  const int hs = static_cast<int>(gw % heads);
  bf16* src = qkv + static_cast<size_t>(t) * heads * D + static_cast<size_t>(hs) * D;

  const bool is_q = hs < Hq;
  const bool is_k = !is_q && hs < Hq + Hkv;
  const int64_t slot = slot_mapping ? slot_mapping[t] : -1;

  float v[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) v[j] = __bfloat162float(src[lane * EPL + j]);

  if (is_q || is_k) {
    const bf16* nw = is_q ? q_norm_w : k_norm_w;
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) ss += v[j] * v[j];
      ss = warp_reduce_sum(ss);
      const float inv = rsqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        // match a bf16 module: normalised value is rounded before RoPE
        v[j] = __bfloat162float(
            __float2bfloat16(v[j] * inv * (__bfloat162float(nw[lane * EPL + j]) + w_offset)));
      }
    }
    const int p = rot_dim > 0 ? positions[t] : 0;
    const bool p_ok = p >= 0 && (max_pos <= 0 || p < max_pos);
    if (rot_dim > 0 && !p_ok && status && lane == 0) atomicCAS(status, 0, PXL_DEV_BAD_POSITION);
    if (rot_dim > 0 && p_ok) {   // a position outside the table is reported, its row is left unrotated
#pragma unroll
      for (int j = 0; j < EPL; ++j) sh[warp][lane * EPL + j] = v[j];
      __syncwarp();
      const int half = rot_dim >> 1;
      const float* cs = cos_sin + static_cast<size_t>(p) * rot_dim;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const int e = lane * EPL + j;
        if (e < rot_dim) {
          const int i = e < half ? e : e - half;
          const float c = cs[i], s = cs[half + i];
          const float partner = e < half ? -sh[warp][e + half] : sh[warp][e - half];
          v[j] = v[j] * c + partner * s;
        }
      }
    }
  }

  if (is_q) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) src[lane * EPL + j] = __float2bfloat16(v[j]);
    return;
  }
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (status && lane == 0) atomicCAS(status, 0, PXL_DEV_BAD_SLOT);
    return;
  }
  const int kvh = is_k ? hs - Hq : hs - Hq - Hkv;
  const int64_t blk = slot / page_size;
  const int off = static_cast<int>(slot % page_size);
  const int64_t at = ((blk * Hkv + kvh) * page_size + off) * static_cast<int64_t>(D);
  if constexpr (FP8) {
    uint8_t* dst = static_cast<uint8_t*>(is_k ? k_cache : v_cache) + at;
    const float inv = is_k ? k_inv_scale : v_inv_scale;
#pragma unroll
    for (int j = 0; j < EPL; ++j) dst[lane * EPL + j] = to_e4m3(v[j] * inv);
  } else {
    bf16* dst = static_cast<bf16*>(is_k ? k_cache : v_cache) + at;
#pragma unroll
    for (int j = 0; j < EPL; ++j) dst[lane * EPL + j] = __float2bfloat16(v[j]);
  }
}

// ------------------------------------------------------------ plain cache scatter
template <bool FP8>
__global__ void __launch_bounds__(256)
reshape_and_cache_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v, int64_t k_stride,
                         int64_t v_stride, const int64_t* __restrict__ slot_mapping,
                         void* __restrict__ k_cache_v, void* __restrict__ v_cache_v, int Hkv, int Dk,
                         int Dv, int page_size, int64_t num_slots, float k_inv_scale,
                         float v_inv_scale, int* status) {
  using CT = typename std::conditional<FP8, uint8_t, bf16>::type;
  CT* k_cache = static_cast<CT*>(k_cache_v);
  CT* v_cache = static_cast<CT*>(v_cache_v);
  auto conv = [](bf16 x, float inv) -> CT {
    if constexpr (FP8) return to_e4m3(__bfloat162float(x) * inv);
    else return x;
  };
  const int t = blockIdx.x;
  const int64_t slot = slot_mapping[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (status && threadIdx.x == 0) atomicCAS(status, 0, PXL_DEV_BAD_SLOT);
    return;
  }
  const int64_t blk = slot / page_size;
  const int off = static_cast<int>(slot % page_size);
  if (k_cache) {
    for (int i = threadIdx.x; i < Hkv * Dk; i += blockDim.x) {
      const int h = i / Dk, d = i % Dk;
      k_cache[((blk * Hkv + h) * page_size + off) * static_cast<int64_t>(Dk) + d] =
          conv(k[t * k_stride + i], k_inv_scale);
    }
  }
  if (v_cache) {
    for (int i = threadIdx.x; i < Hkv * Dv; i += blockDim.x) {
      const int h = i / Dv, d = i % Dv;
      v_cache[((blk * Hkv + h) * page_size + off) * static_cast<int64_t>(Dv) + d] =
          conv(v[t * v_stride + i], v_inv_scale);
    }
  }
}

// --------------------------------------------------------------- act(gate) * up
__device__ __forceinline__ float act_mul(float g, float u, int mode, float limit) {
  if (mode == 0) return g / (1.f + __expf(-g)) * u;
  if (mode == 1) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + __expf(-1.702f * g)) * (u + 1.f);
  }
  const float c = 0.7978845608028654f;
  const float t = tanhf(c * (g + 0.044715f * g * g * g));
  return 0.5f * g * (1.f + t) * u;
}

__global__ void __launch_bounds__(256)
act_mul_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, int I, int mode, float limit) {
  const size_t row = blockIdx.x;
  const bf16* g = x + row * 2 * I;
  const bf16* u = g + I;
  bf16* o = out + row * I;
  for (int v = threadIdx.x; v < (I >> 3); v += blockDim.x) {
    const bf16x8 a = ld_bf16x8(g + v * 8);
    const bf16x8 b = ld_bf16x8(u + v * 8);
    bf16x8 r;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = unpack_bf16x2(a.u[j]);
      const float2 fb = unpack_bf16x2(b.u[j]);
      r.u[j] = pack_bf16x2(act_mul(fa.x, fb.x, mode, limit), act_mul(fa.y, fb.y, mode, limit));
    }
    st_bf16x8(o + v * 8, r);
  }
}

// --------------------------------------------------------------------- row gather
template <typename IdT>
__global__ void __launch_bounds__(128)
gather_rows_kernel(const bf16* __restrict__ table, const IdT* __restrict__ ids,
                   bf16* __restrict__ out, int H, int64_t num_rows, int* status) {
  const size_t t = blockIdx.x;
  int64_t id = static_cast<int64_t>(ids[t]);
  if (id < 0 || id >= num_rows) {
    if (status && threadIdx.x == 0) atomicCAS(status, 0, PXL_DEV_BAD_ROW_ID);
    id = 0;
  }
  const bf16* src = table + id * H;
  bf16* dst = out + t * H;
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x)
    st_bf16x8(dst + v * 8, ld_bf16x8(src + v * 8));
}

__global__ void __launch_bounds__(256) add_inplace_kernel(bf16* y, const bf16* x, int64_t nvec) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  bf16x8 a = ld_bf16x8(y + i * 8);
  const bf16x8 b = ld_bf16x8(x + i * 8);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 fa = unpack_bf16x2(a.u[j]);
    const float2 fb = unpack_bf16x2(b.u[j]);
    a.u[j] = pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
  }
  st_bf16x8(y + i * 8, a);
}

inline int check_launch() { return cudaGetLastError() == cudaSuccess ? PXL_OK : PXL_ERR_CUDA; }

}  // namespace

PXL_EXPORT int pxl_rmsnorm(const void* x, const void* weight, void* out, void* residual, int T,
                           int H, float eps, float w_offset, pxl_stream_t stream) {
  if (T <= 0) return PXL_OK;
  if (H % 8) return PXL_ERR_INVALID_ARG;
  const bf16* xp = static_cast<const bf16*>(x);
  const bf16* wp = static_cast<const bf16*>(weight);
  bf16* op = static_cast<bf16*>(out);
  bf16* rp = static_cast<bf16*>(residual);
  if (H <= 8192 && T >= 64) {
    // many rows: one warp per row with the row in registers
    const unsigned grid = static_cast<unsigned>((T + 7) / 8);
#define PXL_RMS_WARP(NV)                                                                          \
  do {                                                                                            \
    if (residual)                                                                                 \
      pxl_host::launch(rmsnorm_warp_kernel<true, NV>, grid, 256, 0, stream, xp, wp, op, rp, T, H, eps, w_offset); \
    else                                                                                          \
      pxl_host::launch(rmsnorm_warp_kernel<false, NV>, grid, 256, 0, stream, xp, wp, op, rp, T, H, eps, w_offset); \
  } while (0)
    if (H <= 2048) PXL_RMS_WARP(8);
    else if (H <= 4096) PXL_RMS_WARP(16);
    else PXL_RMS_WARP(32);
#undef PXL_RMS_WARP
    return check_launch();
  }
  if (residual)
    pxl_host::launch(rmsnorm_kernel<true>, T, 256, 0, stream, xp, wp, op, rp, H, eps, w_offset);
  else
    pxl_host::launch(rmsnorm_kernel<false>, T, 256, 0, stream, xp, wp, op, static_cast<bf16*>(nullptr), H, eps, w_offset);
  return check_launch();
}

PXL_EXPORT int pxl_rmsnorm_strided(const void* x, int64_t ldx, const void* weight, void* out, int64_t ldo, int T,
                                   int H, float eps, float w_offset, pxl_stream_t stream) {
  if (T <= 0) return PXL_OK;
  if ((H % 8) || (ldx % 8) || (ldo % 8)) return PXL_ERR_INVALID_ARG;
  rmsnorm_strided_kernel<<<T, 256, 0, stream>>>(static_cast<const bf16*>(x), ldx, static_cast<const bf16*>(weight),
                                                static_cast<bf16*>(out), ldo, H, eps, w_offset);
  return check_launch();
}

namespace {
int qk_norm_rope_cache_impl(void* qkv, const void* q_norm_w, const void* k_norm_w,
                            const float* cos_sin, const int* positions,
                            const int64_t* slot_mapping, void* k_cache, void* v_cache, int T, int Hq,
                            int Hkv, int D, int rot_dim, int page_size, int64_t num_slots, float eps,
                            float norm_w_offset, bool cache_fp8, float k_inv_scale,
                            float v_inv_scale, int max_pos, int* status, pxl_stream_t stream) {
  if (T <= 0) return PXL_OK;
  if (rot_dim > D || (rot_dim & 1)) return PXL_ERR_INVALID_ARG;
  const int64_t warps = static_cast<int64_t>(T) * (Hq + 2 * Hkv);
  const unsigned grid = static_cast<unsigned>((warps + 7) / 8);
#define PXL_QKROPE(DD)                                                                        \
  if (cache_fp8)                                                                              \
    pxl_host::launch(qk_norm_rope_cache_kernel<DD, true>, grid, 256, 0, stream,                \
        static_cast<bf16*>(qkv), static_cast<const bf16*>(q_norm_w),                          \
        static_cast<const bf16*>(k_norm_w), cos_sin, positions, slot_mapping, k_cache,        \
        v_cache, T, Hq, Hkv, rot_dim, page_size, num_slots, eps, norm_w_offset, k_inv_scale,  \
        v_inv_scale, max_pos, status);                                                        \
  else                                                                                        \
    pxl_host::launch(qk_norm_rope_cache_kernel<DD, false>, grid, 256, 0, stream,               \
        static_cast<bf16*>(qkv), static_cast<const bf16*>(q_norm_w),                          \
        static_cast<const bf16*>(k_norm_w), cos_sin, positions, slot_mapping, k_cache,        \
        v_cache, T, Hq, Hkv, rot_dim, page_size, num_slots, eps, norm_w_offset, 1.f, 1.f,     \
        max_pos, status)
  switch (D) {
    case 64: PXL_QKROPE(64); break;
    case 96: PXL_QKROPE(96); break;
    case 128: PXL_QKROPE(128); break;
    case 256: PXL_QKROPE(256); break;
    default: return PXL_ERR_INVALID_ARG;
  }
#undef PXL_QKROPE
  return check_launch();
}
}  // namespace

PXL_EXPORT int pxl_qk_norm_rope_cache(void* qkv, const void* q_norm_w, const void* k_norm_w,
                                      const float* cos_sin, const int* positions,
                                      const int64_t* slot_mapping, void* k_cache, void* v_cache,
                                      int T, int Hq, int Hkv, int D, int rot_dim, int page_size,
                                      int64_t num_slots, float eps, float norm_w_offset,
                                      int max_pos, int* status, pxl_stream_t stream) {
  return qk_norm_rope_cache_impl(qkv, q_norm_w, k_norm_w, cos_sin, positions, slot_mapping, k_cache,
                                 v_cache, T, Hq, Hkv, D, rot_dim, page_size, num_slots, eps,
                                 norm_w_offset, false, 1.f, 1.f, max_pos, status, stream);
}

// Same with e4m3 caches: K is stored as k / k_scale, V as v / v_scale (scales > 0).
PXL_EXPORT int pxl_qk_norm_rope_cache_fp8(void* qkv, const void* q_norm_w, const void* k_norm_w,
                                          const float* cos_sin, const int* positions,
                                          const int64_t* slot_mapping, void* k_cache, void* v_cache,
                                          int T, int Hq, int Hkv, int D, int rot_dim, int page_size,
                                          int64_t num_slots, float eps, float norm_w_offset,
                                          float k_scale, float v_scale, int max_pos, int* status,
                                          pxl_stream_t stream) {
  if (!(k_scale > 0.f) || !(v_scale > 0.f)) return PXL_ERR_INVALID_ARG;
  return qk_norm_rope_cache_impl(qkv, q_norm_w, k_norm_w, cos_sin, positions, slot_mapping, k_cache,
                                 v_cache, T, Hq, Hkv, D, rot_dim, page_size, num_slots, eps,
                                 norm_w_offset, true, 1.f / k_scale, 1.f / v_scale, max_pos, status, stream);
}

// dst[dst_idx[i]] = src[src_idx[i]]: the decode rows of a step take their input ids from the token
// tensor that the previous step sampled on the device (the host has not read those tokens yet).
__global__ void patch_i32_kernel(int* __restrict__ dst, const int* __restrict__ dst_idx, const int* __restrict__ src,
                                 const int* __restrict__ src_idx, int n, int dst_len, int src_len, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int d = dst_idx[i], s = src_idx[i];
  if (d < 0 || d >= dst_len || s < 0 || s >= src_len) {
    if (status) atomicCAS(status, 0, PXL_DEV_BAD_ROW_ID);
    return;
  }
  dst[d] = src[s];
}

// Self-test of the bounded peer wait: one thread waits for `flag` to reach `epoch` the way the fused
// kernels wait for a peer. With a flag that nothing sets the wait runs out after its limit (about 1.5 s),
// the kernel records PXL_DEV_TIMEOUT_PEER in *status and returns; *result is 1 if the flag arrived, 0 if
// the wait gave up. The context stays usable either way.
__global__ void bounded_wait_selftest_kernel(const uint32_t* flag, uint32_t epoch, int* result, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *result = flag_wait_bounded<false>(flag, epoch, nullptr, status) ? 1 : 0;
}

PXL_EXPORT int pxl_selftest_bounded_wait(const uint32_t* flag, uint32_t epoch, int* result, int* status,
                                         pxl_stream_t stream) {
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(flag, epoch, result, status);
  return check_launch();
}

PXL_EXPORT int pxl_patch_i32(int* dst, const int* dst_idx, const int* src, const int* src_idx, int n, int dst_len,
                             int src_len, int* status, pxl_stream_t stream) {
  if (n <= 0) return PXL_OK;
  patch_i32_kernel<<<(n + 255) / 256, 256, 0, stream>>>(dst, dst_idx, src, src_idx, n, dst_len, src_len, status);
  return check_launch();
}

PXL_EXPORT int pxl_reshape_and_cache(const void* k, const void* v, int64_t k_stride,
                                     int64_t v_stride, const int64_t* slot_mapping, void* k_cache,
                                     void* v_cache, int T, int Hkv, int Dk, int Dv, int page_size,
                                     int64_t num_slots, int* status, pxl_stream_t stream) {
  if (T <= 0) return PXL_OK;
  reshape_and_cache_kernel<false><<<T, 256, 0, stream>>>(
      static_cast<const bf16*>(k), static_cast<const bf16*>(v), k_stride, v_stride, slot_mapping,
      k_cache, v_cache, Hkv, Dk, Dv, page_size, num_slots, 1.f, 1.f, status);
  return check_launch();
}

PXL_EXPORT int pxl_reshape_and_cache_fp8(const void* k, const void* v, int64_t k_stride,
                                         int64_t v_stride, const int64_t* slot_mapping,
                                         void* k_cache, void* v_cache, int T, int Hkv, int Dk, int Dv,
                                         int page_size, int64_t num_slots, float k_scale,
                                         float v_scale, int* status, pxl_stream_t stream) {
  if (T <= 0) return PXL_OK;
  if (!(k_scale > 0.f) || !(v_scale > 0.f)) return PXL_ERR_INVALID_ARG;
  reshape_and_cache_kernel<true><<<T, 256, 0, stream>>>(
      static_cast<const bf16*>(k), static_cast<const bf16*>(v), k_stride, v_stride, slot_mapping,
      k_cache, v_cache, Hkv, Dk, Dv, page_size, num_slots, 1.f / k_scale, 1.f / v_scale, status);
  return check_launch();
}

PXL_EXPORT int pxl_act_mul(const void* x, void* out, int T, int I, int mode, float limit,
                           pxl_stream_t stream) {
  if (T <= 0) return PXL_OK;
  if (I % 8) return PXL_ERR_INVALID_ARG;
  act_mul_kernel<<<T, 256, 0, stream>>>(static_cast<const bf16*>(x), static_cast<bf16*>(out), I,
                                        mode, limit);
  return check_launch();
}

PXL_EXPORT int pxl_gather_rows(const void* table, const void* ids, void* out, int T, int H,
                               int64_t num_rows, int ids_are_i64, int* status,
                               pxl_stream_t stream) {
  if (T <= 0) return PXL_OK;
  if (H % 8) return PXL_ERR_INVALID_ARG;
  if (ids_are_i64)
    gather_rows_kernel<int64_t><<<T, 128, 0, stream>>>(static_cast<const bf16*>(table),
                                                       static_cast<const int64_t*>(ids),
                                                       static_cast<bf16*>(out), H, num_rows,
                                                       status);
  else
    gather_rows_kernel<int><<<T, 128, 0, stream>>>(static_cast<const bf16*>(table),
                                                   static_cast<const int*>(ids),
                                                   static_cast<bf16*>(out), H, num_rows, status);
  return check_launch();
}

PXL_EXPORT int pxl_add_inplace(void* y, const void* x, int64_t n, pxl_stream_t stream) {
  if (n <= 0) return PXL_OK;
  if (n % 8) return PXL_ERR_INVALID_ARG;
  const int64_t nvec = n / 8;
  add_inplace_kernel<<<static_cast<unsigned>((nvec + 255) / 256), 256, 0, stream>>>(
      static_cast<bf16*>(y), static_cast<const bf16*>(x), nvec);
  return check_launch();
}
