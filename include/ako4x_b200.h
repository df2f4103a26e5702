/*
 * ako4x_b200 — C ABI of the B200 (sm_100a) operator library.
 *
 * One entry point per operator of the AKO4X / FlashInfer-Bench operator set. Every function
 *   - takes raw DEVICE pointers, sizes and scalars only (no framework types),
 *   - launches on the CUDA stream it is given (a cudaStream_t passed as void*) and never
 *     synchronises the host, reads device memory from the host, allocates or frees,
 *   - keeps no state between calls that changes a result (no pointer-keyed caches, no cached
 *     outputs; the only words that outlive a call are the sticky diagnostic status words below),
 *   - initialises whatever part of `workspace` it later reads, so the workspace may hold garbage,
 *   - returns AKO4X_OK or a negative status; nothing throws across this boundary.
 * The matching `*_workspace_bytes` function gives the scratch size a call with the same
 * dimensions needs; the caller owns that buffer (256-byte aligned) for the duration of the call.
 *
 * Each declaration cites the reference plug-in (`kernel.py::run`, a Python function called by the
 * FlashInfer-Bench engine) whose arithmetic the entry point replaces. Paths are relative to the
 * reference project root.
 */
#ifndef AKO4X_B200_H_
#define AKO4X_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AKO4X_OK 0
#define AKO4X_EINVAL (-1)            /* null pointer, negative size, misaligned pointer */
#define AKO4X_EUNSUPPORTED_SHAPE (-2) /* a compile-time dimension (heads, head_dim, ...) differs */
#define AKO4X_ELAUNCH (-3)           /* the CUDA runtime refused a launch */
#define AKO4X_EWORKSPACE (-4)        /* workspace_bytes smaller than *_workspace_bytes() */
#define AKO4X_ETOOLARGE (-5)         /* a fixed internal limit (built-in scratch) is exceeded */

/* Version of this ABI; bumped when a signature changes. */
int ako4x_abi_version(void);

/* ---- a1. RMSNorm, hidden = 128 -------------------------------------------------------------
 * Replaces run(hidden_states, weight):
 *   reference/rmsnorm-h128/variants/triton_tiered_rows/kernel.py:261-278 (kernel :205-239).
 * y = bf16( f32(x) * rsqrt(mean(f32(x)^2) + 1e-6) * f32(w) ); x, y bf16 [rows,128]; w bf16 [128].
 */
int ako4x_rmsnorm_h128(const void* x, const void* weight, void* y, int64_t rows, void* stream);

/* ---- a2. Paged GQA decode, 32 query heads, 8 KV heads, head_dim 128 -----------------------
 * Replaces run(q, k_cache, v_cache, kv_indptr, kv_indices, sm_scale):
 *   reference/gqa-paged-decode-h32-kv8-d128-ps1/variants/triton_pdl_grid_dispatch/kernel.py:420-532.
 * q bf16 [batch,32,128]; k_cache, v_cache bf16 [pages,page_size,8,128]; kv_indptr int32
 * [batch+1]; kv_indices int32 [kv_indptr[batch]] (page ids); o bf16 [batch,32,128];
 * lse fp32 [batch,32] = log2(sum exp(logit)); empty sequence gives o = 0, lse = -inf.
 * `num_kv_indices` (the length of kv_indices) sizes the split heuristic and the workspace; it is
 * a shape, not device data, and it must bound the device-side list: kv_indptr[batch] <=
 * num_kv_indices. A longer device-side list is cut to what the workspace holds and status code 20
 * is recorded (ako4x_gqa_paged_decode_device_status).
 */
size_t ako4x_gqa_paged_decode_workspace_bytes(int64_t batch, int64_t num_kv_indices,
                                              int64_t page_size);
int ako4x_gqa_paged_decode(const void* q, const void* k_cache, const void* v_cache,
                           const int32_t* kv_indptr, const int32_t* kv_indices, float sm_scale,
                           void* o, float* lse, int64_t batch, int64_t num_kv_indices,
                           int64_t page_size, void* workspace, size_t workspace_bytes,
                           void* stream);

/* The gather pipeline waits on mbarriers with a cycle limit. A wait that gives up makes its CTA
 * stop consuming and stores a non-zero code in a device status word; this call returns that word
 * (0 = no wait has given up since the library was loaded). A non-zero word means that the outputs
 * of the call that set it are invalid; later calls are not affected by it (every launch starts its
 * waits afresh). It synchronises the device: for tests and post-mortems only. */
int ako4x_gqa_paged_decode_device_status(void);

/* The same operator for callers that have no scratch memory to pass and cannot allocate any (a
 * plug-in host that supplies only input and output tensors; a serving process whose HBM is fully
 * committed to its KV-cache pool). It has no counterpart in the reference. The split-KV partials
 * live in a 16 MiB array inside the library image (held by every GPU that loads the library);
 * ako4x_gqa_paged_decode_noalloc_max_scratch_bytes() returns that limit. A call that would need
 * more (compare ako4x_gqa_paged_decode_workspace_bytes) returns AKO4X_ETOOLARGE and launches
 * nothing. Calls on one device share the array: calls that can overlap on the GPU race, so keep
 * them on one stream. The first call on a device looks up the array's address; make it at
 * start-up, before any stream capture. Nothing is allocated or freed by this call. */
size_t ako4x_gqa_paged_decode_noalloc_max_scratch_bytes(void);
int ako4x_gqa_paged_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                   const int32_t* kv_indptr, const int32_t* kv_indices,
                                   float sm_scale, void* o, float* lse, int64_t batch,
                                   int64_t num_kv_indices, int64_t page_size, void* stream);

/* ---- a3. Paged MLA decode, 16 heads, ckv 512, kpe 64 ---------------------------------------
 * Replaces run(q_nope, q_pe, ckv_cache, kpe_cache, kv_indptr, kv_indices, sm_scale):
 *   reference/mla-paged-decode-h16-ckv512-kpe64-ps1/variants/triton_split_kv_2d_reduce_pdl_rw2/kernel.py:369-435.
 * logit = (q_nope.ckv + q_pe.kpe) * sm_scale; o = softmax(logit) . ckv; lse base 2.
 * q_nope bf16 [batch,16,512]; q_pe bf16 [batch,16,64]; ckv_cache bf16 [pages,page_size,512];
 * kpe_cache bf16 [pages,page_size,64]; o bf16 [batch,16,512]; lse fp32 [batch,16].
 */
size_t ako4x_mla_paged_decode_workspace_bytes(int64_t batch, int64_t num_kv_indices,
                                              int64_t page_size);
int ako4x_mla_paged_decode(const void* q_nope, const void* q_pe, const void* ckv_cache,
                           const void* kpe_cache, const int32_t* kv_indptr,
                           const int32_t* kv_indices, float sm_scale, void* o, float* lse,
                           int64_t batch, int64_t num_kv_indices, int64_t page_size,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Device status word shared by the MLA decode / prefill / DSA sparse attention kernels (same
 * meaning as ako4x_gqa_paged_decode_device_status; synchronises the device). */
int ako4x_mla_attention_device_status(void);

/* ---- a4. Paged causal MLA prefill ----------------------------------------------------------
 * Replaces run(q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, sm_scale):
 *   reference/mla-paged-prefill-causal-h16-ckv512-kpe64-ps1/variants/
 *   iter6-triton-split-K-grid-pid0-kvsplit/submission_no_cache.py:537-692.
 * Ragged batch; query i of a sequence sees keys j <= (kv_len - q_len) + i; a query that sees no
 * key gets o = 0, lse = -inf. q_nope bf16 [total_q,16,512]; q_pe bf16 [total_q,16,64].
 * From 48 query tokens on, the call needs a workspace (256-byte aligned) of 2176 bytes per key
 * (a contiguous copy of the keys and a transposed copy of the values for the tensor cores);
 * smaller calls need none.
 */
size_t ako4x_mla_paged_prefill_workspace_bytes(int64_t total_q, int64_t batch,
                                               int64_t num_kv_indices, int64_t page_size);
int ako4x_mla_paged_prefill(const void* q_nope, const void* q_pe, const void* ckv_cache,
                            const void* kpe_cache, const int32_t* qo_indptr,
                            const int32_t* kv_indptr, const int32_t* kv_indices, float sm_scale,
                            void* o, float* lse, int64_t total_q, int64_t batch,
                            int64_t num_kv_indices, int64_t page_size, void* workspace,
                            size_t workspace_bytes, void* stream);

/* ---- a5. DSA FP8 top-k indexer, 64 index heads, dim 128, page 64, top-2048 -----------------
 * Replaces run(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table):
 *   reference/dsa-topk-indexer/variants/v8_radix_bt256/kernel.py:569-655
 *   (score :506-546, select :298-451).
 * score[r,t] = (sum_h w[r,h] * relu(q[r,h,:] . k[t,:])) * kscale[t] for t < seq_lens[r]; token t
 * of row r lives in page block_table[r, t/64], slot t%64. Each cache page is 8448 bytes: 64x128
 * e4m3 values, then 64 fp32 scales. Output int32 [rows,2048]: the global slots page*64+slot of
 * the 2048 highest fp32 scores (ties: lower token position wins), listed in ascending token
 * position, then -1 padding; a row with seq_len <= 2048 lists all its tokens.
 */
size_t ako4x_dsa_topk_indexer_workspace_bytes(int64_t rows, int64_t max_pages);
int ako4x_dsa_topk_indexer(const void* q_index_fp8, const void* k_index_cache, const float* weights,
                           const int32_t* seq_lens, const int32_t* block_table,
                           int32_t* topk_indices, int64_t rows, int64_t max_pages,
                           int64_t num_cache_pages, void* workspace, size_t workspace_bytes,
                           void* stream);
/* The two halves of the indexer, exported so that selection can be checked on given scores.
 * scores fp32 [rows, max_pages*64] (entries at t >= seq_len are ignored). */
int ako4x_dsa_index_scores(const void* q_index_fp8, const void* k_index_cache, const float* weights,
                           const int32_t* seq_lens, const int32_t* block_table, float* scores,
                           int64_t rows, int64_t max_pages, int64_t num_cache_pages, void* stream);
int ako4x_dsa_topk_select(const float* scores, const int32_t* seq_lens, const int32_t* block_table,
                          int32_t* topk_indices, int64_t rows, int64_t max_pages, void* stream);

/* Device status word of the tensor-core score kernel (same meaning as
 * ako4x_gqa_paged_decode_device_status; synchronises the device). */
int ako4x_dsa_indexer_device_status(void);

/* ---- a6. DSA sparse MLA attention ----------------------------------------------------------
 * Replaces run(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale):
 *   reference/dsa-sparse-attention/variants/hybrid_pdl_v2/kernel.py:557-626
 *   (arithmetic: variants/pure_triton/kernel.py:24-155).
 * Keys of token t are rows sparse_indices[t,:] (int32 [tokens,topk], -1 ignored) of the caches
 * flattened to [pages*page_size, 512] and [.., 64]. An all -1 row gives o = 0, lse = -inf.
 */
size_t ako4x_dsa_sparse_attention_workspace_bytes(int64_t tokens, int64_t topk);
int ako4x_dsa_sparse_attention(const void* q_nope, const void* q_pe, const void* ckv_cache,
                               const void* kpe_cache, const int32_t* sparse_indices,
                               float sm_scale, void* o, float* lse, int64_t tokens, int64_t topk,
                               int64_t num_cache_rows, void* workspace, size_t workspace_bytes,
                               void* stream);

/* ---- a7. FP8 block-scale MoE, DeepSeek-V3 routing ------------------------------------------
 * Replaces run(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
 *              gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
 *              routed_scaling_factor):
 *   reference/moe-fp8-block-scale/variants/fused_routing_v2/kernel.py:509-667.
 * 256 global experts in 8 groups, top-4 groups by top-2 sum, top-8 experts; hidden 7168,
 * intermediate 2048, `num_local_experts` local experts starting at `local_expert_offset`.
 * routing_logits fp32 [tokens,256]; routing_bias fp32 or bf16 [256] (bias_is_bf16);
 * hidden_states e4m3 [tokens,7168]; hidden_states_scale fp32 [56,tokens];
 * gemm1_weights e4m3 [E,4096,7168], scale fp32 [E,32,56]; gemm2_weights e4m3 [E,7168,2048],
 * scale fp32 [E,56,16]; out bf16 [tokens,7168].
 */
size_t ako4x_moe_fp8_block_scale_workspace_bytes(int64_t tokens, int64_t num_local_experts);
int ako4x_moe_fp8_block_scale(const float* routing_logits, const void* routing_bias,
                              int bias_is_bf16, const void* hidden_states,
                              const float* hidden_states_scale, const void* gemm1_weights,
                              const float* gemm1_weights_scale, const void* gemm2_weights,
                              const float* gemm2_weights_scale, int32_t local_expert_offset,
                              float routed_scaling_factor, void* out, int64_t tokens,
                              int64_t num_local_experts, void* workspace, size_t workspace_bytes,
                              void* stream);
/* Byte offset, inside a workspace for `tokens`, of a 32-bit status word that the call leaves at
 * 0 on success. The tensor-core GEMM kernels bound every wait on an mbarrier; a wait that runs out
 * of its cycle limit stores a non-zero code there (1 producer, 2/3 MMA issuer, 4 epilogue) and the
 * kernel unwinds instead of hanging. A caller may read the word after synchronising the stream. */
size_t ako4x_moe_fp8_block_scale_status_offset(int64_t tokens);
/* The same call with measurement hooks: `stage_events` is NULL or an array of 5 cudaEvent_t
 * (as void*, entries may be NULL) recorded on `stream` before routing [0], before GEMM1 [1],
 * between GEMM1 and GEMM2 [2], after GEMM2 [3] and after the combine [4]. */
int ako4x_moe_fp8_block_scale_staged(const float* routing_logits, const void* routing_bias,
                                     int bias_is_bf16, const void* hidden_states,
                                     const float* hidden_states_scale, const void* gemm1_weights,
                                     const float* gemm1_weights_scale, const void* gemm2_weights,
                                     const float* gemm2_weights_scale, int32_t local_expert_offset,
                                     float routed_scaling_factor, void* out, int64_t tokens,
                                     int64_t num_local_experts, void* workspace,
                                     size_t workspace_bytes, void* stream, void* const* stage_events);
/* Routing alone (same arithmetic as the first stage of the call above): the 8 selected global
 * expert ids per token in ascending id order and their weights. topk_ids int32 [tokens,8];
 * topk_weights fp32 [tokens,8]. Reference: fused_routing_v2/kernel.py:350-391. */
int ako4x_moe_ds_routing(const float* routing_logits, const void* routing_bias, int bias_is_bf16,
                         float routed_scaling_factor, int32_t* topk_ids, float* topk_weights,
                         int64_t tokens, void* stream);

/* Expert-parallel combine (no counterpart in the reference, which is single-GPU): out[t] =
 * bf16(sum over ranks g in ascending order of rows[pos[t,g]]) with fp32 accumulation; entries
 * pos < 0 are skipped. rows bf16 [n, cols]; pos int32 [tokens, world]; out bf16 [tokens, cols];
 * cols a multiple of 8. */
int ako4x_moe_ep_combine(const void* rows, const int32_t* pos, void* out, int64_t tokens,
                         int64_t world, int64_t cols, void* stream);

/* ---- The producers in front of the operator set (same layer, one step earlier) ---------------
 * FP8 activation quantiser: x bf16 [rows, cols] (cols a multiple of 128) -> q e4m3 [rows, cols] and
 * scale fp32 [cols/128, rows] (block-major, the layout a7 takes as hidden_states_scale). Per 128
 * consecutive values: scale = amax / 448 (1.0 when amax <= 1e-10), q = e4m3(x / scale), the rule
 * of reference/moe-fp8-block-scale/variants/fused_routing_v2/kernel.py:495-503. */
int ako4x_fp8_quantize_1x128(const void* x, void* q, float* scale, int64_t rows, int64_t cols,
                             void* stream);
/* Index-K cache writer: k bf16 [tokens, 128] -> the paged cache a5 reads (8448 bytes per page: 64 x
 * 128 e4m3 values, then 64 fp32 scales; reference/dsa-topk-indexer/variants/v8_radix_bt256/
 * kernel.py:562, 621-625). slot_mapping int32 [tokens] = page * 64 + slot of every token, -1 to skip
 * it. Per token: scale = amax / 448 (1.0 when amax <= 1e-10), values e4m3(k / scale). */
int ako4x_dsa_index_k_cache_write(const void* k, const int32_t* slot_mapping, void* k_index_cache,
                                  int64_t tokens, int64_t num_cache_pages, void* stream);
/* a5 followed by a6 on one stream, the top-k list staying on the device: the arguments of both
 * operators, `topk_indices` int32 [rows, 2048] as the hand-over buffer (an output as well), one
 * workspace of ako4x_dsa_indexer_attention_workspace_bytes bytes. The attention kernels are
 * launched with programmatic dependent launch so that their prologue overlaps the selection's
 * tail. References as for a5 and a6. */
size_t ako4x_dsa_indexer_attention_workspace_bytes(int64_t rows, int64_t max_pages);
int ako4x_dsa_indexer_attention(const void* q_index_fp8, const void* k_index_cache, const float* weights,
                                const int32_t* seq_lens, const int32_t* block_table,
                                const void* q_nope, const void* q_pe, const void* ckv_cache,
                                const void* kpe_cache, float sm_scale, int32_t* topk_indices, void* o,
                                float* lse, int64_t rows, int64_t max_pages, int64_t num_cache_pages,
                                void* workspace, size_t workspace_bytes, void* stream);

/* ---- Expert-parallel form of a7 over NVLink peer memory (no counterpart in the reference, which is
 * single-GPU) ---------------------------------------------------------------------------------
 * One process per GPU; rank r owns experts [32r, 32r+32) (routing group r). Every rank allocates
 * one buffer of ako4x_moe_ep_buffer_bytes(world, cap_rows) bytes that all ranks can address (CUDA
 * peer / IPC / fabric mapping; the Python side uses torch symmetric memory), zero-fills its first
 * 4096 bytes once, and passes the `world` mapped addresses, in rank order, as `peer_buffers` (a HOST
 * array). `cap_rows` bounds the tokens any rank contributes to a step; `pair_capacity` bounds the
 * (token, expert) pairs this rank computes (about world * cap_rows for uniform routing; pairs beyond
 * it are dropped and status 9 is recorded in the workspace status word); `step` is 1, 2, 3, ... and
 * must be the same on every rank for the same step. The call routes this rank's `tokens` tokens,
 * stores one copy of each token row into the receive area of every rank that owns one of its eight
 * experts, runs the operator on the rows it received, stores each row's bf16 partial back into the
 * sender's return area and sums, in rank order and in fp32, the partial rows of its own tokens into
 * `out` (bf16 [tokens, 7168]). Everything runs on `stream`; there is no host synchronisation and no
 * collective library call. Waits on peers are bounded (about two seconds): a rank that never
 * arrives leaves a code in the buffer's status word (ako4x_moe_ep_status) instead of a hang.
 * Experts that no participating rank owns (world < 8) are dropped, as the single-GPU operator
 * drops non-local experts. */
size_t ako4x_moe_ep_buffer_bytes(int64_t world, int64_t cap_rows);
size_t ako4x_moe_ep_workspace_bytes(int64_t tokens, int64_t world, int64_t cap_rows,
                                    int64_t pair_capacity);
int ako4x_moe_fp8_block_scale_ep(const float* routing_logits, const void* routing_bias,
                                 int bias_is_bf16, const void* hidden_states,
                                 const float* hidden_states_scale, const void* gemm1_weights,
                                 const float* gemm1_weights_scale, const void* gemm2_weights,
                                 const float* gemm2_weights_scale, float routed_scaling_factor,
                                 void* out, int64_t tokens, int64_t world, int64_t rank,
                                 int64_t cap_rows, int64_t pair_capacity, int32_t step,
                                 void* const* peer_buffers, void* workspace, size_t workspace_bytes,
                                 void* stream);
/* 0, or the code of a bounded wait on a peer that gave up (50 + source rank: its rows never arrived;
 * 60 + expert rank: its results never arrived). Synchronises the device. */
int ako4x_moe_ep_status(const void* my_buffer);

/* ---- Gated Delta Net decode (definition gdn_decode_qk4_v8_d128_k_last) -------------------------
 * Replaces run(q, k, v, state, A_log, a, dt_bias, b, scale) of
 * reference/gdn-decode/variants/cuda_bv32_register_resident/kernel.py:456-523.
 * q, k bf16 [batch, 1, 4, 128]; v bf16 [batch, 1, 8, 128]; state fp32 [batch, 8, 128 (v), 128 (k)] or
 * NULL (zeros); A_log, dt_bias fp32 [8]; a, b bf16 [batch, 1, 8]; out bf16 [batch, 1, 8, 128];
 * new_state fp32 like state (may not alias state). v head h reads q/k head h / 2.
 *   g = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b), delta = beta (v - g S k),
 *   new_state = g S + delta k^T, out = scale q . new_state.
 * scale is used as given (the Python wrapper maps None / 0 to 1/sqrt(128)). q, k, state and
 * new_state must be 16-byte aligned. One launch, no workspace. */
int ako4x_gdn_decode(const void* q, const void* k, const void* v, const float* state,
                     const float* A_log, const void* a, const float* dt_bias, const void* b,
                     float scale, void* out, float* new_state, int64_t batch, void* stream);

/* ---- Dense GEMM (definition gemm_n2048_k4096) --------------------------------------------------
 * C[m, n] = A[m, k] * B[n, k]^T with fp32 accumulation; A, B, C fp16 (is_bf16 = 0) or bf16 (1),
 * row-major and contiguous, 16-byte aligned. Replaces the reference family's best implementation,
 * torch.matmul(A, B.T) (reference/gemm-n2048-k4096/README.md: N = 2048, K = 4096, M = 1 ... 16 294).
 * n must be a multiple of 256 and k of 64 (AKO4X_EUNSUPPORTED_SHAPE otherwise); any m >= 0. One
 * launch, no workspace. */
int ako4x_gemm_f16_nt(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                      int is_bf16, void* stream);
/* The same GEMM with a caller-owned workspace, which lets small and medium M split the K dimension
 * over CTAs (partial products in fp32 in the workspace, summed in split order by a second kernel:
 * deterministic). ako4x_gemm_workspace_bytes gives the size for a shape (0 when no split is used);
 * a NULL workspace runs the unsplit kernel; a workspace that is too small is AKO4X_EWORKSPACE. */
size_t ako4x_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k);
int ako4x_gemm_f16_nt_ws(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                         int is_bf16, void* workspace, size_t workspace_bytes, void* stream);
/* 0, or the code of a bounded wait of the GEMM kernels that gave up (71-74). Synchronises. */
int ako4x_gemm_device_status(void);

/* ---- Gated Delta Net prefill (definition gdn_prefill_qk4_v8_d128_k_last) ------------------------
 * Replaces run(q, k, v, state, A_log, a, dt_bias, b, cu_seqlens, scale) of
 * reference/gdn-prefill/variants/cuda_graph_v5/kernel.py:1333. q, k bf16 [tokens, 4, 128]; v bf16
 * [tokens, 8, 128]; state fp32 [num_seqs, 8, 128 (v), 128 (k)] or NULL (zeros); A_log, dt_bias fp32
 * [8]; a, b bf16 [tokens, 8]; cu_seqlens int64 [num_seqs + 1] (device memory, ascending; sequence s
 * owns tokens cu_seqlens[s] .. cu_seqlens[s+1]); out bf16 [tokens, 8, 128]; new_state like state.
 * The decode recurrence (ako4x_gdn_decode) applied to every token of a sequence in order, the
 * output taken after each update. An empty sequence gets a zero new_state (as the definition
 * does); tokens that belong to no sequence are not written.
 * With a workspace of ako4x_gdn_prefill_workspace_bytes(total_tokens, num_seqs) bytes (16-byte
 * aligned) calls with one or two sequences run the recurrence in chunks of 16 tokens (a kernel
 * that tabulates k_i.k_j and q_i.k_j per chunk, then the state kernel: only a 16-step substitution
 * is serial per chunk); with a NULL workspace, and from three sequences on, it runs token by token
 * in one launch. Same results up to fp32 rounding order. */
size_t ako4x_gdn_prefill_workspace_bytes(int64_t total_tokens, int64_t num_seqs);
int ako4x_gdn_prefill(const void* q, const void* k, const void* v, const float* state,
                      const float* A_log, const void* a, const float* dt_bias, const void* b,
                      const int64_t* cu_seqlens, float scale, void* out, float* new_state,
                      int64_t total_tokens, int64_t num_seqs, void* workspace,
                      size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AKO4X_B200_H_ */
