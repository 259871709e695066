// C ABI of libpxl_kernels.so — the sm_100a kernel library of parallax_b200.
//
// Conventions
//   * every pointer is a device pointer unless its name ends in `_host`;
//   * bf16 tensors are passed as `void*`; shapes are row-major, innermost last;
//   * `stream` is a cudaStream_t passed as an opaque pointer;
//   * launchers return 0 (PXL_OK) or a PxlStatus error code; they never
//     synchronise and never allocate device memory unless stated otherwise;
//   * `status` is an optional device int. Kernels with bounded waits or index
//     checks write a non-zero PxlStatus code there instead of trapping.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* pxl_stream_t;

// GEMM epilogues
#define PXL_EPI_NONE 0      // C = A W^T (+bias)                      bf16 out
#define PXL_EPI_RESIDUAL 1  // C = A W^T (+bias) + residual           bf16 out
#define PXL_EPI_SILU_MUL 2  // C[:, j] = silu(gate_j) * up_j          bf16 out, N/2 columns
#define PXL_EPI_F32 3       // C = A W^T (+bias)                      fp32 out
#define PXL_EPI_RS 4        // partial sums scattered to the owning rank + reduce (pxl_gemm_bf16_rs)
#define PXL_EPI_SCATTER 5   // every output row stored through its own pointer, possibly on a peer GPU
#define PXL_EPI_SPLITK_T 6  // internal: small-M path (operands swapped, split along K, fp32 slabs + last-CTA finish)
#define PXL_EPI_SPLITK_C 7  // internal: small-M path, the K ranges of a tile form a cluster and reduce over DSMEM
#define PXL_EPI_SPLITK_CN 8 // internal: mid-M path (operands not swapped), K ranges of a tile reduce inside a cluster

// ---- gemm_tcgen05.cu -------------------------------------------------------
// C[M,N] = A[M,K] * W[N,K]^T. lda/ldw/ldc in elements. `bn` = tile width (64/128/256)
// or 0 to pick automatically. For PXL_EPI_SILU_MUL the rows of W must be arranged in
// groups of 128: 64 gate rows followed by the 64 up rows of the same outputs (bn >= 128).
int pxl_gemm_bf16(const void* A, const void* W, void* C, const void* residual, const void* bias,
                  int M, int N, int K, int lda, int ldw, int ldc, int epi, int bn, int* status,
                  pxl_stream_t stream);
int pxl_gemm_bf16_pick_bn(int M, int N, int epi);
// Small-M (decode) GEMM, M <= 128: the weight matrix takes the 128-row operand slot of the tensor
// core, the few activation rows the narrow one, and K is split over `splitk` CTAs per 128 output
// columns (0 = automatic) so that every SM streams weights. mode 2: the CTAs of one tile form a
// thread-block cluster (splitk <= 8), exchange their fp32 partial sums through distributed shared
// memory and each finishes a slice of the tokens (+ bias, + residual, bf16 out). mode 1: partial
// sums meet in an fp32 scratch owned by the library (one per stream) and the CTA that arrives last
// finishes the tile. mode 0 picks. Sums are formed in K order either way (bitwise repeatable).
// pxl_gemm_bf16 takes this path by itself when bn == 0 and the shape qualifies.
int pxl_gemm_bf16_small_m(const void* A, const void* W, void* C, const void* residual, const void* bias,
                          int M, int N, int K, int lda, int ldw, int ldc, int splitk, int mode, int* status,
                          pxl_stream_t stream);
// 1 when pxl_gemm_bf16(bn = 0) would use the small-M path for this shape and epilogue.
int pxl_gemm_bf16_uses_small_m(int M, int N, int K, int epi);

// ---- elementwise.cu ----------------------------------------------------------
// out = x * rsqrt(mean(x^2) + eps) * (w + w_offset). If residual != NULL:
// residual += x first (in place) and the norm is taken of the sum.
int pxl_rmsnorm(const void* x, const void* weight, void* out, void* residual, int T, int H,
                float eps, float w_offset, pxl_stream_t stream);
// Same without residual for rows with their own strides (a column slice of a wider matrix; out may be x).
int pxl_rmsnorm_strided(const void* x, int64_t ldx, const void* weight, void* out, int64_t ldo, int T, int H,
                        float eps, float w_offset, pxl_stream_t stream);
// Per-head q/k RMSNorm (optional) + rotary embedding (neox pairing, first `rot_dim`
// dims) on a packed qkv activation [T, (Hq + 2*Hkv) * D], writing q in place and
// scattering k, v into the paged cache [blocks, Hkv, page, D] at slot_mapping[t]
// (slot < 0: skip). cos_sin: fp32 [max_pos, rot_dim] = cos | sin halves. A position outside [0, max_pos)
// sets PXL_DEV_BAD_POSITION and leaves its row unrotated (max_pos <= 0: not checked).
int pxl_qk_norm_rope_cache(void* qkv, const void* q_norm_w, const void* k_norm_w,
                           const float* cos_sin, const int* positions, const int64_t* slot_mapping,
                           void* k_cache, void* v_cache, int T, int Hq, int Hkv, int D, int rot_dim,
                           int page_size, int64_t num_slots, float eps, float norm_w_offset,
                           int max_pos, int* status, pxl_stream_t stream);
// Plain scatter of k, v [T, Hkv, D] (row strides in elements) into the paged cache.
int pxl_reshape_and_cache(const void* k, const void* v, int64_t k_stride, int64_t v_stride,
                          const int64_t* slot_mapping, void* k_cache, void* v_cache, int T,
                          int Hkv, int Dk, int Dv, int page_size, int64_t num_slots, int* status,
                          pxl_stream_t stream);
// e4m3 KV cache ("fp8 KV"): the caches hold one byte per element; K is stored as k / k_scale and V as
// v / v_scale (saturating, scales > 0) and the *_fp8 attention entry points undo the scaling. Same
// arguments as the bf16 functions plus the two scales.
int pxl_qk_norm_rope_cache_fp8(void* qkv, const void* q_norm_w, const void* k_norm_w,
                               const float* cos_sin, const int* positions,
                               const int64_t* slot_mapping, void* k_cache, void* v_cache, int T,
                               int Hq, int Hkv, int D, int rot_dim, int page_size, int64_t num_slots,
                               float eps, float norm_w_offset, float k_scale, float v_scale,
                               int max_pos, int* status, pxl_stream_t stream);
int pxl_reshape_and_cache_fp8(const void* k, const void* v, int64_t k_stride, int64_t v_stride,
                              const int64_t* slot_mapping, void* k_cache, void* v_cache, int T,
                              int Hkv, int Dk, int Dv, int page_size, int64_t num_slots,
                              float k_scale, float v_scale, int* status, pxl_stream_t stream);
int pxl_attn_decode_fp8(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                        const int* block_tables, const int* ctx_lens, void* out, float* workspace,
                        const float* sinks, int B, int Hq, int Hkv, int D, int page_size,
                        int max_blocks, int64_t num_blocks, float scale, int window, int num_splits,
                        int max_ctx, float k_scale, float v_scale, int* status, pxl_stream_t stream);
int pxl_attn_prefill_fp8(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                         const int* block_tables, const int* cu_q, const int* ctx_lens, void* out,
                         int64_t out_stride, const float* sinks, int B, int max_q_len, int Hq,
                         int Hkv, int D, int page_size, int max_blocks, int64_t num_blocks,
                         float scale, int window, float k_scale, float v_scale, int* status,
                         pxl_stream_t stream);
// out[T, I] = act(x[:, :I]) * x[:, I:]; mode 0 = silu, 1 = clipped swiglu-oai
// (alpha 1.702, limit), 2 = gelu-tanh.
int pxl_act_mul(const void* x, void* out, int T, int I, int mode, float limit, pxl_stream_t stream);
// out[t, :] = table[ids[t], :]  (ids int32 or int64 per `ids_are_i64`)
int pxl_gather_rows(const void* table, const void* ids, void* out, int T, int H, int64_t num_rows,
                    int ids_are_i64, int* status, pxl_stream_t stream);
// Bounded-wait self-test (see elementwise.cu): waits for *flag >= epoch like a fused kernel waits for a peer;
// *result = 1 when it arrived, 0 when the wait ran out (then *status = PXL_DEV_TIMEOUT_PEER).
int pxl_selftest_bounded_wait(const uint32_t* flag, uint32_t epoch, int* result, int* status, pxl_stream_t stream);
// dst[dst_idx[i]] = src[src_idx[i]] for i < n (int32 words; indices checked against dst_len / src_len)
int pxl_patch_i32(int* dst, const int* dst_idx, const int* src, const int* src_idx, int n, int dst_len, int src_len,
                  int* status, pxl_stream_t stream);
// y += x (bf16), n elements (multiple of 8)
int pxl_add_inplace(void* y, const void* x, int64_t n, pxl_stream_t stream);

// ---- attention_decode.cu -----------------------------------------------------
// Single-query GQA attention over the paged cache [blocks, Hkv, page, D] (D = 64 or 128).
// q [B, Hq, D] with row stride q_stride elements; out [B, Hq, D]; block_tables [B, max_blocks]; ctx_lens [B].
// window <= 0: full attention. sinks: optional fp32 [Hq] logits added to the
// softmax denominator. workspace: fp32, >= B*Hq*num_splits*(D+2) floats when
// num_splits > 1. num_splits = 0 picks automatically (see pxl_attn_decode_splits).
int pxl_attn_decode(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                    const int* block_tables, const int* ctx_lens, void* out, float* workspace,
                    const float* sinks, int B, int Hq, int Hkv, int D, int page_size,
                    int max_blocks, int64_t num_blocks, float scale, int window, int num_splits,
                    int max_ctx, int* status, pxl_stream_t stream);
int pxl_attn_decode_splits(int B, int Hkv, int max_ctx);

// ---- attention_prefill.cu ----------------------------------------------------
// Ragged causal attention of new query tokens against the paged cache, which must
// already hold K/V of the new tokens and of any cached prefix. q/out [T, Hq, D]
// with row stride q_stride/out_stride elements; cu_q [B+1] token offsets;
// ctx_lens[b] = prefix + new length of sequence b.
int pxl_attn_prefill(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                     const int* block_tables, const int* cu_q, const int* ctx_lens, void* out,
                     int64_t out_stride, const float* sinks, int B, int max_q_len, int Hq, int Hkv,
                     int D, int page_size, int max_blocks, int64_t num_blocks, float scale,
                     int window, int* status, pxl_stream_t stream);

// ---- attention_prefill_tc.cu ------------------------------------------------------
// Same contract on the tcgen05 tensor cores (D = 128, page 16 / 32 / 64). total_q = rows of q / out.
int pxl_attn_prefill_tc(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                        const int* block_tables, const int* cu_q, const int* ctx_lens, void* out,
                        int64_t out_stride, const float* sinks, int B, int max_q_len, int total_q, int Hq,
                        int Hkv, int D, int page_size, int max_blocks, int64_t num_blocks, float scale,
                        int window, int* status, pxl_stream_t stream);

// ---- sampler.cu ----------------------------------------------------------------
// Greedy arg-max over logits [B, V] (bf16 if logits_bf16 else fp32, row stride ld).
// A row without a finite maximum (all NaN) yields token 0 and sets PXL_DEV_NONFINITE_LOGITS in *status
// (status may be null).
int pxl_argmax(const void* logits, int logits_bf16, int64_t ld, int B, int V, int* out_ids,
               float* out_logprob, int* status, pxl_stream_t stream);
// Temperature / top-k / top-p / min-p sampling, one uniform random number per row.
// temperature <= 0 or top_k == 1 selects arg-max for that row.
int pxl_sample(const void* logits, int logits_bf16, int64_t ld, int B, int V,
               const float* temperature, const int* top_k, const float* top_p, const float* min_p,
               const float* uniform, int* out_ids, float* out_prob, int* status, pxl_stream_t stream);

// ---- moe.cu ------------------------------------------------------------------
// Router: scores [T, E] fp32/bf16 logits -> top-k expert ids and weights.
// mode 0: softmax then top-k (optionally renormalised); mode 1: sigmoid + per-expert
// correction bias for selection, grouped top-k (n_group/topk_group, 1/1 = none),
// weights = sigmoid scores renormalised and scaled by routed_scale.
int pxl_moe_route(const void* logits, int logits_bf16, const float* e_bias, int T, int E, int k,
                  int mode, int renorm, int n_group, int topk_group, float routed_scale,
                  int* out_ids, float* out_w, pxl_stream_t stream);

int pxl_moe_align(const int* ids, int T, int k, int E, int e_lo, int e_hi, int* counts,
                  int* offsets, int* cursor, int* mt_expert, int* mt_row0, int* mt_row_end,
                  int* num_mt, int max_mt, int* pos_of, int* src_tok, pxl_stream_t stream);
int pxl_moe_gather(const void* x, const int* src_tok, const int* n_rows, void* x_perm,
                   int max_rows, int H, pxl_stream_t stream);
int pxl_moe_combine(const void* y_perm, const int* pos_of, const float* w, const void* base,
                    void* out, int T, int k, int H, pxl_stream_t stream);
// Grouped GEMM over experts (see gemm_tcgen05.cu).
int pxl_gemm_bf16_grouped(const void* A, const void* W, void* C, const void* bias, int P, int E, int N, int K,
                          int lda, int ldw, int ldc, const int* mt_expert, const int* mt_row0,
                          const int* mt_row_end, const int* num_mt, int max_m_tiles, int epi,
                          int bn, int* status, pxl_stream_t stream);

// Fused tensor-parallel collectives (see gemm_tcgen05.cu for the buffer contracts).
int pxl_gemm_bf16_rs(const void* A, const void* W, void* out, const void* residual,
                     void* const* stage_ptrs, void* const* flag_ptrs, int rank, int tp,
                     int rows_per_rank, int N, int K, int lda, int ldw, int ldo, uint32_t epoch,
                     int bn, int* status, pxl_stream_t stream);
int pxl_gemm_bf16_ag(void* const* x_ptrs, void* const* ready_ptrs, void* tile_flags, const void* W,
                     void* C, const void* bias, int rank, int tp, int rows_per_rank, int N, int K,
                     int lda, int ldw, int ldc, int epi, uint32_t epoch, int ncopy, int bn,
                     int* status, pxl_stream_t stream);

// ---- mla.cu: multi-head latent attention on the compressed cache [blocks, page, 512 + 64] ----
// RMSNorm(latent) + interleaved RoPE(k_pe) of ckv [T, 576] (row stride ld) written to the cache.
int pxl_mla_kv_prep(const void* ckv, int64_t ld, const void* norm_w, const float* cos_sin,
                    const int* positions, const int64_t* slots, void* cache, int T, int latent,
                    int rope, int64_t num_slots, float eps, int* status, pxl_stream_t stream);
// q [T, H, nope + 64] -> q_nope_hm [H, Tpad, nope] (head-major, input of the absorb GEMM) and
// q_pe [T, H, 64] with interleaved RoPE applied.
int pxl_mla_q_prep(const void* q, int64_t ld, const float* cos_sin, const int* positions,
                   void* q_nope_hm, void* q_pe, int T, int Tpad, int H, int nope, int rope,
                   pxl_stream_t stream);
// Absorbed attention for tokens [tok_begin, tok_begin + n_tok): q_lat [H, Tpad, 512], q_pe
// [T, H, 64] -> out [H, Tpad, 512]. Query token t sits at positions[t] of sequence
// cu_q-lookup(t) (cu_q NULL: sequence t - tok_begin) and attends keys 0..positions[t], or, when
// topk != NULL and topk[t][0] >= 0, the listed positions only (topk rows indexed by t).
int pxl_mla_attn(const void* q_lat, const void* q_pe, const void* cache, const int* block_tables,
                 const int* cu_q, const int* positions, const int* topk, void* out, int tok_begin,
                 int n_tok, int Tpad, int H, int B, int max_blocks, int page, int latent, int rope,
                 int topk_k, int topk_stride, float scale, pxl_stream_t stream);

// ---- dsa.cu: lightning indexer -------------------------------------------------------------
// scores[t, j] = sum_h relu(q[t,h,:] . k_j) * w[t,h] for j <= positions[t], -inf beyond;
// ld_scores >= ceil(max_ctx / 64) * 64.
int pxl_dsa_index_scores(const void* q, const float* w, const void* index_cache,
                         const int* block_tables, const int* cu_q, const int* positions,
                         float* scores, int64_t ld_scores, int T, int B, int Hi, int Di,
                         int max_blocks, int page, int max_ctx, pxl_stream_t stream);
// Positions of the k largest scores among [0, positions[t]] per row (unordered); rows with at
// most k candidates are filled with -1 ("attend densely").
int pxl_topk_select(const float* scores, int64_t ld, const int* positions, int T, int k, int* out,
                    int64_t ld_out, pxl_stream_t stream);
// Indexer pre-processing of a step (Di == 128): q_idx [T, Hi*Di] gets the interleaved rotation on the first R
// dims of every head in place; the index key kv[t, k_off : k_off+Di] is layer-normed (w, optional b), rotated
// on its first R dims and stored at cache[slots[t]]; w_out[t, h] = kv[t, w_off+h] * w_scale (fp32).
int pxl_dsa_index_prep(void* q_idx, int64_t ldq, const void* kv, int64_t ldkv, int k_off, int w_off,
                       const void* ln_w, const void* ln_b, float ln_eps, const float* cos_sin,
                       const int* positions, int max_pos, const int64_t* slots, void* cache, int64_t num_slots,
                       float* w_out, float w_scale, int T, int Hi, int Di, int R, int* status,
                       pxl_stream_t stream);
// cache[slots[t], :] = src[t, :] (slot < 0: skip)
int pxl_store_rows(const void* src, int64_t ld, const int64_t* slots, void* cache, int T, int D,
                   int64_t num_slots, int* status, pxl_stream_t stream);

// ---- gemm_fp8.cu: block-scaled e4m3 GEMM (1x128 activation groups, weight scales per 64 rows x 128 cols)
// C[M,N] bf16 = sum over 128-wide K blocks of a_s[m,kb] * w_s[n/64,kb] * (A_kb W_kb^T). K % 128 == 0,
// N % 128 == 0. epi: PXL_EPI_NONE / PXL_EPI_RESIDUAL / PXL_EPI_SILU_MUL (W rows interleaved as for bf16).
int pxl_gemm_fp8_block(const void* A, const float* a_s, const void* W, const float* w_s, void* C,
                       const void* residual, int M, int N, int K, int lda, int ldw, int ldc, int epi,
                       int* status, pxl_stream_t stream);
int pxl_gemm_fp8_block_grouped(const void* A, const float* a_s, const void* W, const float* w_s, void* C,
                               int P, int E, int N, int K, int lda, int ldw, int ldc, const int* mt_expert,
                               const int* mt_row0, const int* mt_row_end, const int* num_mt, int max_m_tiles,
                               int epi, int* status, pxl_stream_t stream);
// x [T,K] bf16 (row stride ld) -> q [T,K] e4m3 + scales [T, K/128]: x ~= q * scale per group
int pxl_quant_fp8_rows(const void* x, int64_t ld, void* q, float* scales, int T, int K, pxl_stream_t stream);

// ---- moe_ep.cu + the scatter epilogue of gemm_tcgen05.cu: expert parallelism over peer memory ----
int pxl_ep_dispatch(const void* x, int64_t ldx, const int* ids, int n_rows, int k, int H,
                    int experts_per_rank, int cap, int rank, int ep, void* const* recv_x_ptrs,
                    void* const* recv_meta_ptrs, void* const* recv_cnt_ptrs, void* const* flag_ptrs,
                    int* cursor, uint32_t* done_counter, uint32_t epoch, int* status, pxl_stream_t stream);
int pxl_ep_recv_ids(const int* recv_meta, const int* recv_cnt, const void* disp_flag, int ep, int cap,
                    uint32_t epoch, int* ids_out, int* status, pxl_stream_t stream);
int pxl_ep_row_ptrs(const int* src_slot, const int* n_rows, const int* recv_meta, int cap, int H, int ep,
                    void* const* comb_ptrs, void** row_ptrs, int max_rows, pxl_stream_t stream);
int pxl_gemm_bf16_grouped_scatter(const void* A, const void* W, void* const* row_ptrs, int P, int E, int N,
                                  int K, int lda, int ldw, const int* mt_expert, const int* mt_row0,
                                  const int* mt_row_end, const int* num_mt, int max_m_tiles,
                                  void* const* flag_ptrs, uint32_t* done_counter, int rank, int ep_size,
                                  uint32_t epoch, int* status, pxl_stream_t stream);
int pxl_ep_combine(const void* comb, const float* w, const void* base, int64_t ld_base, void* out,
                   int64_t ld_out, const void* ret_flag, int ep, uint32_t epoch, int n_rows, int k, int H,
                   int* status, pxl_stream_t stream);

// ---- linear_attn.cu: gated delta-net layers (per-request state slots) ---------------------------
// y = silu(causal_conv(x)) per channel with the last K-1 inputs carried in conv_state [slots, C, K-1];
// sequence b covers tokens [seq_cu[b], seq_cu[b+1]) and uses slot seq_slots[b]; a sequence whose
// first token has position 0 starts from zeros.
int pxl_causal_conv1d_silu(const void* x, int64_t ldx, const void* w, const void* bias, void* conv_state,
                           const int* seq_cu, const int* seq_slots, const int* positions, void* out,
                           int64_t ldo, int B, int C, int K, pxl_stream_t stream);
// Gated delta rule over qkv [T, 2*Hk*Dk + Hv*Dv] (q | k | v), gates a, b [T, Hv] (shared row stride),
// output gate z [T, Hv*Dv]; rec_state [slots, Hv, Dv, Dk] fp32; out [T, Hv*Dv] after the gated RMSNorm.
int pxl_gated_delta_rule(const void* qkv, int64_t ld_qkv, const void* a, const void* b, int64_t ld_ab,
                         const float* A_log, const float* dt_bias, const void* z, int64_t ld_z,
                         const void* norm_w, float* rec_state, const int* seq_cu, const int* seq_slots,
                         const int* positions, void* out, int64_t ld_out, int B, int Hk, int Hv, int Dk,
                         int Dv, float eps, pxl_stream_t stream);
// out = x * sigmoid(gate), rows of N elements with their own strides
int pxl_sigmoid_gate_mul(const void* x, int64_t ldx, const void* gate, int64_t ldg, void* out, int64_t ldo,
                         int T, int N, pxl_stream_t stream);

// out = (res +) x * sigmoid(gate[:, col / group]); gate [T, N / group]; res may be null; group % 8 == 0
int pxl_gate_mul_grouped(const void* x, int64_t ldx, const void* gate, int64_t ldg, const void* res, int64_t ldr,
                         void* out, int64_t ldo, int T, int N, int group, pxl_stream_t stream);
// out[t] = x[t, :K] . w[:K] (bf16 out)
int pxl_row_dot(const void* x, int64_t ldx, const void* w, void* out, int T, int K, pxl_stream_t stream);

// ---- msa.cu: block-sparse attention indexer --------------------------------------------------
// scores[t, j] = max over index heads and visible tokens of 128-token block j of scale * iq . ik
int pxl_msa_block_scores(const void* iq, const void* index_cache, const int* block_tables, const int* cu_q,
                         const int* positions, float* scores, int64_t ld, int T, int B, int Hi, int Di,
                         int max_blocks, int page, int sparse_block, int max_ctx, float scale,
                         pxl_stream_t stream);
// top-k blocks per query (first init_blocks and the last local_blocks always kept) expanded into a
// virtual block table v_tables [T, topk * sparse_block / page] and visible-token count v_ctx [T]
int pxl_msa_select(const float* scores, int64_t ld, const int* positions, const int* block_tables,
                   const int* cu_q, int T, int B, int max_blocks, int page, int sparse_block, int topk,
                   int init_blocks, int local_blocks, int* v_tables, int64_t ld_vt, int* v_ctx,
                   pxl_stream_t stream);

// ---- stage_exec.cu: all layers of a dense GQA stage for one step behind one call --------------
// The descriptor structs are defined in stage_exec.cu (mirrored by parallax_b200/engine/native_stage.py).
struct PxlStageDesc;
struct PxlStepDesc;
struct PxlStageWorkspace;
int pxl_stage_forward_dense(const struct PxlStageDesc* stage, const struct PxlStepDesc* step,
                            const struct PxlStageWorkspace* ws, const void* h_in, void** h_out, int* launches,
                            int* status, pxl_stream_t stream);

#ifdef __cplusplus
}
#endif
