// Native stage executor: runs every layer of a dense GQA pipeline stage for one step with ONE call
// from the host runtime. The per-kernel launches (RMSNorm, tcgen05 GEMMs with fused epilogues, the
// fused q/k-norm + RoPE + cache write, paged prefill and decode attention) are issued from C++ in
// sequence on the caller's stream, so a step costs one foreign-function call per stage instead of
// roughly ten per layer. Activations live in a caller-provided workspace; nothing is allocated.
//
// Counterpart in the reference: the per-layer Python loop of ShardedModel.__call__
// (src/parallax/server/model.py:75-180), which dispatches framework ops layer by layer.
#include <cstdlib>

#include "common.cuh"
#include "pxl_api.h"

extern "C" {

// One decoder layer; all pointers are device pointers (optional ones may be null).
struct PxlDenseLayer {
  const void* ln1;
  const void* ln2;
  const void* w_qkv;   // [(Hq + 2 Hkv) D, H]
  const void* b_qkv;   // optional
  const void* q_norm;  // optional [D]
  const void* k_norm;  // optional [D]
  const void* w_o;     // [H, Hq D]
  const void* b_o;     // optional [H]
  const void* w_gu;    // [2 I, H], gate/up interleaved in groups of 64
  const void* w_down;  // [H, I]
  void* k_cache;       // [blocks, Hkv, page, D]
  void* v_cache;
  const float* sinks;  // optional [Hq]
  int window;
  int pad_;
};

struct PxlStageDesc {
  int H, Hq, Hkv, D, I, rot_dim, page, n_layers;
  int64_t num_blocks;
  float eps, norm_offset, scale;
  int max_pos;             // rows of cos_sin
  const float* cos_sin;
  const PxlDenseLayer* layers;  // host array of n_layers entries
};

struct PxlStepDesc {
  int T, Tp, Bp, Bd, p_max_q, d_max_ctx, p_max_blocks, d_max_blocks;
  const int* positions;
  const int64_t* slots;
  const int* p_cu_q;
  const int* p_ctx;
  const int* p_bt;
  const int* d_ctx;
  const int* d_bt;
};

struct PxlStageWorkspace {
  void* xn;        // [T, H]
  void* qkv;       // [T, (Hq + 2 Hkv) D]
  void* attn;      // [T, Hq D]
  void* act;       // [T, I]
  void* h_a;       // [T, H] ping
  void* h_b;       // [T, H] pong
  float* decode;   // split-KV partials: Bd * Hq * splits * (D + 2) floats
  int64_t decode_floats;
};

}  // extern "C"

// With PXL_STAGE_DEBUG set in the environment every launch is followed by a synchronising read of
// the status word; the call then returns 1000 + 16 * layer + op so that the failing kernel is named.
static bool stage_debug() {
  static const bool on = getenv("PXL_STAGE_DEBUG") != nullptr;
  return on;
}
static int stage_probe(int* status, cudaStream_t stream, int layer, int op) {
  if (!stage_debug() || status == nullptr) return PXL_OK;
  int code = 0;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return PXL_ERR_CUDA;
  if (cudaMemcpy(&code, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return PXL_ERR_CUDA;
  return code ? 1000 + 16 * layer + op : PXL_OK;
}

#define PXL_TRY(expr)                                  \
  do {                                                 \
    const int rc_ = (expr);                            \
    if (rc_ != PXL_OK) return rc_;                     \
    const int pr_ = stage_probe(status, stream, li, ++op_); \
    if (pr_ != PXL_OK) return pr_;                     \
  } while (0)

// h_in [T, H] -> returns the pointer that holds the stage's output hidden states in *h_out (one of
// the workspace's ping/pong buffers). *launches receives the number of kernels launched.
PXL_EXPORT int pxl_stage_forward_dense(const PxlStageDesc* st, const PxlStepDesc* sp, const PxlStageWorkspace* ws,
                                       const void* h_in, void** h_out, int* launches, int* status,
                                       cudaStream_t stream) {
  if (!st || !sp || !ws || !h_in || !h_out) return PXL_ERR_INVALID_ARG;
  const int T = sp->T, H = st->H, Hq = st->Hq, Hkv = st->Hkv, D = st->D, I = st->I;
  if (T <= 0) return PXL_ERR_INVALID_ARG;
  const int qkv_n = (Hq + 2 * Hkv) * D;
  const int64_t num_slots = st->num_blocks * st->page;
  const void* h = h_in;
  int n = 0;
  pxl::bf16* qkv = static_cast<pxl::bf16*>(ws->qkv);
  pxl::bf16* attn = static_cast<pxl::bf16*>(ws->attn);
  // tcgen05 prefill attention where its layout rules hold, else the mma.sync kernel
  static const bool prefill_legacy = getenv("PXL_PREFILL_LEGACY") != nullptr;
  const bool prefill_tc = !prefill_legacy && D == 128 && (st->page == 16 || st->page == 32 || st->page == 64) &&
                          (qkv_n % 8) == 0 && (reinterpret_cast<uintptr_t>(ws->qkv) & 15) == 0 &&
                          st->num_blocks * Hkv * st->page < (1ll << 31);
  int splits = 0;
  if (sp->Bd > 0) {
    splits = pxl_attn_decode_splits(sp->Bd, Hkv, sp->d_max_ctx);
    if (splits > 1 && static_cast<int64_t>(sp->Bd) * Hq * splits * (D + 2) > ws->decode_floats) return PXL_ERR_TOO_LARGE;
  }
  // every kernel of the sequence waits (griddepcontrol.wait) before it touches global memory, so each
  // launch may overlap its prologue with the tail of the kernel before it
  static const bool no_pdl = getenv("PXL_NO_PDL") != nullptr;
  struct PdlScope {
    bool prev;
    explicit PdlScope(bool on) : prev(pxl_host::pdl_flag()) { pxl_host::pdl_flag() = on; }
    ~PdlScope() { pxl_host::pdl_flag() = prev; }
  } pdl_scope(!no_pdl && !stage_debug());
  for (int li = 0; li < st->n_layers; ++li) {
    const PxlDenseLayer& L = st->layers[li];
    int op_ = 0;  // 1 norm, 2 qkv, 3 rope+cache, 4 prefill, 5 decode (4 if no prefill), then o_proj, norm, gate_up, down
    void* h_mid = (h == ws->h_a) ? ws->h_b : ws->h_a;
    PXL_TRY(pxl_rmsnorm(h, L.ln1, ws->xn, nullptr, T, H, st->eps, st->norm_offset, stream));
    PXL_TRY(pxl_gemm_bf16(ws->xn, L.w_qkv, qkv, nullptr, L.b_qkv, T, qkv_n, H, H, H, qkv_n, PXL_EPI_NONE, 0, status,
                          stream));
    PXL_TRY(pxl_qk_norm_rope_cache(qkv, L.q_norm, L.k_norm, st->cos_sin, sp->positions, sp->slots, L.k_cache,
                                   L.v_cache, T, Hq, Hkv, D, st->rot_dim, st->page, num_slots, st->eps,
                                   st->norm_offset, st->max_pos, status, stream));
    n += 3;
    if (sp->Tp > 0) {
      if (prefill_tc) {
        PXL_TRY(pxl_attn_prefill_tc(qkv, qkv_n, L.k_cache, L.v_cache, sp->p_bt, sp->p_cu_q, sp->p_ctx, attn,
                                    static_cast<int64_t>(Hq) * D, L.sinks, sp->Bp, sp->p_max_q, sp->Tp, Hq, Hkv, D,
                                    st->page, sp->p_max_blocks, st->num_blocks, st->scale, L.window, status, stream));
      } else {
        PXL_TRY(pxl_attn_prefill(qkv, qkv_n, L.k_cache, L.v_cache, sp->p_bt, sp->p_cu_q, sp->p_ctx, attn,
                                 static_cast<int64_t>(Hq) * D, L.sinks, sp->Bp, sp->p_max_q, Hq, Hkv, D, st->page,
                                 sp->p_max_blocks, st->num_blocks, st->scale, L.window, status, stream));
      }
      ++n;
    }
    if (sp->Bd > 0) {
      PXL_TRY(pxl_attn_decode(qkv + static_cast<size_t>(sp->Tp) * qkv_n, qkv_n, L.k_cache, L.v_cache, sp->d_bt,
                              sp->d_ctx, attn + static_cast<size_t>(sp->Tp) * Hq * D, ws->decode, L.sinks, sp->Bd, Hq,
                              Hkv, D, st->page, sp->d_max_blocks, st->num_blocks, st->scale, L.window, splits,
                              sp->d_max_ctx, status, stream));
      n += splits > 1 ? 2 : 1;
    }
    PXL_TRY(pxl_gemm_bf16(attn, L.w_o, h_mid, h, L.b_o, T, H, Hq * D, Hq * D, Hq * D, H, PXL_EPI_RESIDUAL, 0, status,
                          stream));
    PXL_TRY(pxl_rmsnorm(h_mid, L.ln2, ws->xn, nullptr, T, H, st->eps, st->norm_offset, stream));
    PXL_TRY(pxl_gemm_bf16(ws->xn, L.w_gu, ws->act, nullptr, nullptr, T, 2 * I, H, H, H, I, PXL_EPI_SILU_MUL, 0, status,
                          stream));
    void* h_next = (h_mid == ws->h_a) ? ws->h_b : ws->h_a;
    PXL_TRY(pxl_gemm_bf16(ws->act, L.w_down, h_next, h_mid, nullptr, T, H, I, I, I, H, PXL_EPI_RESIDUAL, 0, status,
                          stream));
    n += 4;
    h = h_next;
  }
  *h_out = const_cast<void*>(h);
  if (launches) *launches = n;
  return PXL_OK;
}
