/* C ABI of libhk_attn: bf16 grouped-query flash-attention forward and paged-KV decode for NVIDIA B200.
 *
 * Plain pointers and sizes only. All pointers are DEVICE pointers on `device` unless a comment says
 * otherwise. Every function returns 0 on success or a negative HK_E* code; none aborts or throws.
 * Kernels are launched asynchronously on `cuda_stream` (NULL = the legacy default stream), exactly as
 * the reference launcher does (kernels/attn/gqa/kernel.cpp:576-581).
 * `device` is the CUDA device index the pointers live on (< 0 = the calling thread's current device). An entry
 * point makes that device current while it runs and puts the caller's current device back before it returns.
 * The first call on a device sets the kernels' attributes and allocates one 4-byte status word there (the only
 * allocation the library makes; hk_attn_paged_decode_static does not need it); if that set-up fails the call
 * returns the error and the next call tries again.
 */
#ifndef HK_ATTN_H_
#define HK_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HK_OK 0
#define HK_EINVAL (-1)       /* bad shape, null or misaligned pointer */
#define HK_EUNSUPPORTED (-2) /* head dim / page size / device not supported */
#define HK_ECUDA (-3)        /* a CUDA runtime or driver call failed; see hk_last_cuda_error() */
#define HK_ETIMEOUT (-4)     /* a bounded device-side wait expired; results are invalid */
#define HK_EWORKSPACE (-5)   /* workspace missing or too small */
#define HK_EBADPAGE (-6)     /* a block-table entry outside [0, num_pages) was met; it was not dereferenced */
#define HK_EBADLEN (-7)      /* a context length beyond max_pages_per_seq * page_size was met; it was clamped */

/* Attention forward.
 * Replaces dispatch_micro<D>(attn_globals<D>) (kernels/attn/gqa/kernel.cpp:93-100,576-581, causal twin
 * kernels/attn/gqa_causal/kernel.cpp) and dispatch_fwd<D> (training/llama/csrc/attn_fwd_causal.cpp:624-630).
 *   q, o   : bf16 [B, N, H, D] contiguous          k, v : bf16 [B, N, H_KV, D] contiguous
 *   lse    : fp32 [B, H, 1, N] contiguous, natural-log logsumexp of the scaled logits
 *   D in {64, 128}; any N >= 1 (the reference needs a multiple of 256: kernels/attn/gqa/kernel.cpp:26,29,97);
 *   H a multiple of H_KV; pointers 16-byte aligned.
 *   causal != 0 applies the lower-triangular mask; softmax_scale <= 0 selects 1/sqrt(D).
 * Shapes, causality and scale are compile-time constants in the reference; here they are arguments. */
int hk_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                int B, int N, int H, int H_KV, int D, int causal, float softmax_scale,
                int device, void* cuda_stream);

/* Same forward for q, k, v that are strided views: q_strides / k_strides / v_strides are HOST arrays of three element
 * strides (batch, sequence, head); the D dimension must be contiguous and every stride a multiple of 8 elements.
 * This reads q, k, v straight out of a packed projection output ([B,N,3,H,D] or [B,N,2,H_KV,D]) without the
 * `.contiguous()` copies the reference's call site makes (training/llama/llama/models/attentions/hipkittens.py:37-39,
 * after mha.py:213-243 split the projection). o and lse are contiguous as in hk_attn_fwd. */
int hk_attn_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse,
                        int B, int N, int H, int H_KV, int D,
                        const long long* q_strides, const long long* k_strides, const long long* v_strides,
                        int causal, float softmax_scale, int device, void* cuda_stream);

/* Same forward with key padding: kv_lens is a DEVICE array int32 [B] (or NULL); batch element b attends to keys
 * [0, kv_lens[b]) only, as the reference's PyTorch path does with key_padding_mask
 * (training/llama/llama/models/attentions/base.py:97-103, used by training/bert through attention_mask). Lengths are
 * clamped to [1, N]; all N query rows are still computed. KV tiles beyond a batch element's length are neither loaded
 * nor multiplied. Strides as in hk_attn_fwd_strided. With causal != 0 the mask is aligned to the kept keys as in
 * hk_attn_fwd_cross below (Nk = N). */
int hk_attn_fwd_varlen(const void* q, const void* k, const void* v, void* o, float* lse,
                       int B, int N, int H, int H_KV, int D,
                       const long long* q_strides, const long long* k_strides, const long long* v_strides,
                       const int32_t* kv_lens, int causal, float softmax_scale, int device, void* cuda_stream);

/* The general forward: Nq query rows against Nk keys per batch element (Nq != Nk allowed). This is what the
 * reference's math path computes for CrossAttention(q, kv) (base.py:78-120) and what inference with a cache calls
 * (training/llama/llama/models/mha.py:164-168: inner_cross_attn(q, kv) with kv longer than q).
 *   q, o : bf16 [B, Nq, H, D]    k, v : bf16 [B, Nk, H_KV, D]    lse : fp32 [B, H, 1, Nq]
 *   kv_lens : DEVICE int32 [B] or NULL; kept keys per batch element, clamped to [1, Nk] (NULL = Nk)
 *   causal != 0: query row r sees key c iff c <= r + (kv_len_b - Nq) (and c < kv_len_b), the reference's alignment of
 *   the mask to the last query and the last kept key (base.py:104-116). A row that sees no key at all (possible
 *   when kv_len_b < Nq) gets O = 0 and L = -inf; the reference's -10000 fill would instead spread such a row
 *   uniformly over masked keys, an artefact that is not reproduced.
 * Strides as in hk_attn_fwd_strided (q_strides for [B, Nq, H], k/v_strides for [B, Nk, H_KV]). */
int hk_attn_fwd_cross(const void* q, const void* k, const void* v, void* o, float* lse,
                      int B, int Nq, int Nk, int H, int H_KV, int D,
                      const long long* q_strides, const long long* k_strides, const long long* v_strides,
                      const int32_t* kv_lens, int causal, float softmax_scale, int device, void* cuda_stream);

/* Chunked prefill against the paged KV cache: T query rows per sequence against that sequence's cached context,
 * K and V read page by page through the block table (the multi-token sibling of hk_attn_paged_decode; the reference
 * has neither - its cache is contiguous, training/llama/llama/models/mha.py:16-42,164-168).
 *   q, o : bf16 [S, T, H, D]     lse : fp32 [S, H, 1, T]
 *   k_pages, v_pages, block_table as in hk_attn_paged_decode; ctx_lens[s] = keys of sequence s, clamped to
 *   [1, max_pages_per_seq * 16]. The chunk's own keys are expected to be in the cache already (append first).
 *   causal != 0: query row r of the chunk sees keys up to r + (ctx_lens[s] - T), i.e. the chunk is the last T
 *   tokens of the context (the alignment of hk_attn_fwd_cross); a row that sees no key gets O = 0, L = -inf.
 *   D in {64, 128}, page_size = 16. A block-table entry outside [0, num_pages) is not dereferenced and is reported
 *   as HK_EBADPAGE by hk_last_device_status. Same kernel as hk_attn_fwd: results are bit-identical to
 *   hk_attn_fwd_cross on the gathered K and V. Cache rows the context does not cover must hold finite values. */
int hk_attn_fwd_paged(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_table,
                      const int32_t* ctx_lens, void* o, float* lse, int S, int T, int H, int H_KV, int D,
                      int page_size, int max_pages_per_seq, int num_pages, int causal, float softmax_scale,
                      int device, void* cuda_stream);

/* Paged-KV decode: one query token per sequence attends to its whole context. No counterpart exists in
 * the reference (its nearest relative is the contiguous cache update training/llama/llama/models/mha.py:16-42).
 *   q, o        : bf16 [S, 1, H, D]                 lse : fp32 [S, H, 1, 1]
 *   k_pages, v_pages : bf16 [num_pages, page_size, H_KV, D]
 *   block_table : int32 [S, max_pages_per_seq]; token j of sequence s is row j % page_size of page
 *                 block_table[s, j / page_size]; entries must lie in [0, num_pages)
 *   ctx_lens    : int32 [S], 1 <= ctx_lens[s] <= max_pages_per_seq * page_size. A larger value is clamped to
 *                 that capacity on the device (nothing beyond the block-table row is read) and reported as
 *                 HK_EBADLEN by hk_last_device_status; a value <= 0 gives O = 0 and L = -inf.
 *   D = 128, page_size = 16, H / H_KV from 1 to 8; S and H_KV at most 65535, max_pages_per_seq at most 8192
 *   (HK_EUNSUPPORTED beyond, and hk_attn_paged_decode_workspace_bytes then returns 0).
 *   workspace   : device scratch of at least hk_attn_paged_decode_workspace_bytes(...) bytes, 256-byte
 *                 aligned; holds the per-split partial results between the two kernels. */
size_t hk_attn_paged_decode_workspace_bytes(int S, int H, int D, int max_pages_per_seq, int page_size);
int hk_attn_paged_decode(const void* q, const void* k_pages, const void* v_pages,
                         const int32_t* block_table, const int32_t* ctx_lens, void* o, float* lse,
                         int S, int H, int H_KV, int D, int page_size, int max_pages_per_seq, int num_pages,
                         float softmax_scale, void* workspace, size_t workspace_bytes,
                         int device, void* cuda_stream);

/* ---- attention backward ------------------------------------------------------------------------------
 * The reference runs three kernels per backward pass (training/llama/llama/models/attentions/hipkittens.py:
 * 110-112): tk_kernel_bkwd_prep.dispatch_prep(O, dO, delta), tk_kernel_bkwd.dispatch_bwd_combined(q, k, v,
 * dO, dQ_in, dK, dV, L, delta) and tk_kernel_bkwd_prep.dispatch_dq_shuffle(dQ_in, dQ). The three entry
 * points below replace them one for one. All are asynchronous on `cuda_stream`. */

/* delta[b,h,0,n] = sum_d O[b,n,h,d] * dO[b,n,h,d] in fp32.
 * Replaces dispatch_prep (kernels/attn/gqa_backwards/attn_bkwd_prep.cpp:164-195,230-234).
 *   o, d_o : bf16 [B,N,H,D] contiguous      delta : fp32 [B,H,1,N]      D in {64, 128} */
int hk_attn_bwd_prep(const void* o, const void* d_o, float* delta, int B, int N, int H, int D, int device,
                     void* cuda_stream);

/* Layout in which hk_attn_bwd writes dQ. */
#define HK_DQ_BNHD 0 /* [B,N,H,D], the layout of q: no shuffle pass needed afterwards */
#define HK_DQ_BHND 1 /* [B,H,N,D], the reference's pre-shuffle scratch layout (dQ_in) */

/* dQ, dK, dV of O = softmax(scale * Q K^T) V given dO, the forward pass's L and delta from hk_attn_bwd_prep.
 * Replaces dispatch_bwd_combined (kernels/attn/gqa_backwards/attn_bkwd_non_causal.cpp:37-49,3164-3185;
 * causal twin kernels/attn/gqa_causal_backwards/attn_bkwd_causal.cpp). The reference accumulates dQ with
 * atomic adds into a zero-filled [B,H,N,D] scratch and needs dispatch_dq_shuffle afterwards; here dQ is
 * written once, in the layout `dq_layout` names, and does not need to be zero-filled.
 *   q, d_o, dq : bf16 [B,N,H,D] (dq as dq_layout says)    k, v, dk, dv : bf16 [B,N,H_KV,D]
 *   lse, delta : fp32 [B,H,1,N]
 *   D in {64, 128}; any N >= 1 (the reference needs a multiple of 256); tensor pointers 16-byte aligned, lse and
 *   delta 4-byte aligned; softmax_scale <= 0 selects 1/sqrt(D).
 * Results are bit-identical from run to run (no atomics). */
int hk_attn_bwd(const void* q, const void* k, const void* v, const void* d_o, const float* lse, const float* delta,
                void* dq, void* dk, void* dv, int B, int N, int H, int H_KV, int D, int causal, float softmax_scale,
                int dq_layout, int device, void* cuda_stream);

/* hk_attn_bwd for right-padded batches: batch element b attends to its first kv_lens[b] keys only, the backward of
 * hk_attn_fwd_varlen (the reference's key_padding_mask, training/llama/llama/models/attentions/base.py:97-103; its
 * kernels have no counterpart). kv_lens: device int32 [B], values clamped to [1, N]; null = no padding. dK and dV
 * rows of padded keys come back as zeros. With causal != 0 the mask is aligned to the kept keys as in
 * hk_attn_bwd_cross below (Nk = N). */
int hk_attn_bwd_varlen(const void* q, const void* k, const void* v, const void* d_o, const float* lse,
                       const float* delta, void* dq, void* dk, void* dv, int B, int N, int H, int H_KV, int D,
                       const int32_t* kv_lens, int causal, float softmax_scale, int dq_layout, int device,
                       void* cuda_stream);

/* The general backward, of hk_attn_fwd_cross: Nq query rows against Nk keys (the reference's math path for
 * CrossAttention(q, kv), base.py:78-120, differentiated; its kernels need Nq = Nk).
 *   q, d_o, dq : bf16 [B,Nq,H,D] (dq as dq_layout says)    k, v, dk, dv : bf16 [B,Nk,H_KV,D]
 *   lse, delta : fp32 [B,H,1,Nq], lse as hk_attn_fwd_cross wrote it (-inf for a row that sees no key)
 *   kv_lens and causal as in hk_attn_fwd_cross. Keys nobody sees get dK = dV = 0, rows that see no key dQ = 0. */
int hk_attn_bwd_cross(const void* q, const void* k, const void* v, const void* d_o, const float* lse,
                      const float* delta, void* dq, void* dk, void* dv, int B, int Nq, int Nk, int H, int H_KV, int D,
                      const int32_t* kv_lens, int causal, float softmax_scale, int dq_layout, int device,
                      void* cuda_stream);

/* dq_bnhd[b,n,h,:] = dq_bhnd[b,h,n,:]. Replaces dispatch_dq_shuffle (attn_bkwd_prep.cpp:199-223,236-239); only
 * needed after hk_attn_bwd with HK_DQ_BHND. D a multiple of 8; the two buffers must not alias. */
int hk_attn_dq_shuffle(const void* dq_bhnd, void* dq_bnhd, int B, int N, int H, int D, int device,
                       void* cuda_stream);

/* Rotary position embedding of q or k, the step before attention (training/llama/llama/models/mha.py:217-220).
 * Replaces tk_kernel.dispatch_rotary(x, o, sin, cos) (kernels/rotary/kernel.cpp:44-98):
 *   x, o : bf16 [B, H, N, D] contiguous        sin, cos : bf16 [N, rotary_dim / 2]
 *   o[.., i] = x[.., i] cos[n,i] - x[.., i+R/2] sin[n,i],  o[.., i+R/2] = x[.., i+R/2] cos[n,i] + x[.., i] sin[n,i]
 *   for i < R/2 (R = rotary_dim; <= 0 selects D), o[.., R:] = x[.., R:]. Products and sums are rounded to bf16 one
 *   by one, as in the reference kernel, so results are bit-identical to the harness's bf16 PyTorch expression.
 *   D a multiple of 8, rotary_dim a multiple of 16 and <= D (the reference is built for D = rotary_dim = 128);
 *   x and o may be the same buffer. Asynchronous on `cuda_stream`. */
int hk_rotary(const void* x, void* o, const void* sin, const void* cos, int B, int H, int N, int D, int rotary_dim,
              int device, void* cuda_stream);

/* hk_rotary for x, o in the layout the attention entries read, bf16 [B, N, H, D], so that q and k are rotated where
 * they lie (the reference's kernel wants [B, H, N, D], kernels/rotary/kernel.cpp:44-98, and its call site rotates
 * before attention, training/llama/llama/models/mha.py:217-220). Row n of the sequence takes row n + pos_offset of
 * sin / cos [>= N + pos_offset, rotary_dim / 2]: a chunk that continues a cached prefix passes the prefix length.
 * Same arithmetic as hk_rotary (bit-identical results); x and o may be the same buffer. */
int hk_rotary_bnhd(const void* x, void* o, const void* sin, const void* cos, int B, int N, int H, int D,
                   int rotary_dim, int pos_offset, int device, void* cuda_stream);

/* Appends T new tokens per sequence to the paged KV cache read by hk_attn_paged_decode.
 * Paged counterpart of the reference's contiguous cache update, kv_cache[b, offset : offset + T] = kv
 * (training/llama/llama/models/mha.py:16-42, _update_kv_cache).
 *   k_new, v_new : bf16 [S, T, H_KV, D]          k_pages, v_pages : bf16 [num_pages, page_size, H_KV, D]
 *   start_pos    : int32 [S]; token t of sequence s is written at position start_pos[s] + t, i.e. row
 *                  (pos % page_size) of page block_table[s, pos / page_size]
 *   page_size = 16; H_KV * D a multiple of 8; pointers 16-byte aligned.
 * A position beyond max_pages_per_seq pages or a page id outside [0, num_pages) is skipped and reported as
 * HK_EBADPAGE by hk_last_device_status. Asynchronous on `cuda_stream`. */
int hk_paged_kv_append(const void* k_new, const void* v_new, void* k_pages, void* v_pages,
                       const int32_t* block_table, const int32_t* start_pos,
                       int S, int T, int H_KV, int D, int page_size, int max_pages_per_seq, int num_pages,
                       int device, void* cuda_stream);

/* hk_paged_kv_append with the rotary embedding of K fused in: k_new is rotated on its way into the pages (V is
 * copied), token t of sequence s with row start_pos[s] + t of sin / cos [cos_rows, rotary_dim / 2]. The reference
 * rotates k with its rotary kernel and then updates the cache (mha.py:217-220, then 16-42); the pages end up
 * bit-identical to hk_rotary_bnhd followed by hk_paged_kv_append, with one read and one write of K instead of two.
 * rotary_dim <= 0 selects D; D a multiple of 8, rotary_dim a multiple of 16. A position at or beyond cos_rows is
 * skipped and reported like a position beyond the block table (HK_EBADPAGE). */
int hk_paged_kv_append_rotary(const void* k_new, const void* v_new, void* k_pages, void* v_pages,
                              const int32_t* block_table, const int32_t* start_pos, const void* sin, const void* cos,
                              int S, int T, int H_KV, int D, int rotary_dim, int cos_rows, int page_size,
                              int max_pages_per_seq, int num_pages, int device, void* cuda_stream);

/* Paged-KV decode for callers that cannot allocate device memory. No counterpart in the reference.
 *
 * Who needs it: a serving engine that hands all of HBM to its own block allocator at start-up leaves nothing
 * for a plug-in to cudaMalloc, and a latency-critical decode loop cannot afford cudaMalloc's device-wide
 * synchronisation. hk_attn_paged_decode() makes such callers bring a workspace (and its first call on a device
 * allocates a status word); this variant brings its own: the per-chunk partial results live in a fixed
 * HK_DECODE_STATIC_SCRATCH_BYTES array that is part of the library image, so every GPU that loads the library
 * holds that much memory until the process exits. (With CUDA's default lazy module loading the array takes its
 * place in device memory when the library's kernels are first used on that device - by any entry point, this
 * one included - not when the shared object is loaded; an engine that is about to claim all remaining HBM
 * should therefore make one call on each device first.) It calls no cudaMalloc / cudaFree and no allocating
 * library routine.
 *
 * Same arguments and results as hk_attn_paged_decode() minus the workspace, plus `status_out`:
 *   status_out  HOST pointer or NULL. When given, the call waits for its own kernels on `cuda_stream` and stores
 *               HK_OK, HK_EBADPAGE or HK_EBADLEN there; with NULL the call is asynchronous and the status is
 *               dropped. Pass NULL while `cuda_stream` is being captured: the wait is a stream synchronisation,
 *               which a capturing stream refuses (HK_ECUDA).
 * Limit: hk_attn_paged_decode_workspace_bytes(S, H, D, max_pages_per_seq, page_size) must not exceed
 * HK_DECODE_STATIC_SCRATCH_BYTES (e.g. S=16, H=64 at up to 7680 tokens per sequence); larger problems are
 * refused with HK_EWORKSPACE before anything is launched - use hk_attn_paged_decode() for them.
 * The first call on each device looks up the device address of the array (one-time set-up, under a lock; a
 * failed set-up is retried by the next call); make that first call before any stream capture begins.
 * All calls on a device share the one array: it still holds the previous call's partials (every value a call
 * reads it has written first, and the status word is cleared on the stream at the start of each call), and two
 * calls whose kernels overlap on the GPU - different streams, or different host threads - race on it. Serialise them. */
#define HK_DECODE_STATIC_SCRATCH_BYTES (8u << 20)
int hk_attn_paged_decode_static(const void* q, const void* k_pages, const void* v_pages,
                                const int32_t* block_table, const int32_t* ctx_lens, void* o, float* lse,
                                int S, int H, int H_KV, int D, int page_size, int max_pages_per_seq, int num_pages,
                                float softmax_scale, int device, void* cuda_stream, int* status_out);

/* Synchronises `device` and reports the device-side status word of the kernels above: HK_OK,
 * HK_ETIMEOUT when a bounded wait inside a kernel expired, HK_EBADPAGE or HK_EBADLEN. The word is cleared on read.
 * The reference launchers check nothing after launch (include/pyutils/util.cuh:6-16). */
int hk_last_device_status(int device);

/* Self-test of the bounded-wait path: launches a one-warp kernel that waits on a barrier nobody ever
 * signals, with a time limit of `limit_us` microseconds, then synchronises. Returns HK_ETIMEOUT when the
 * wait gave up as designed (the expected result) and leaves the context usable. Has no counterpart in the
 * reference, whose kernels have no bounded waits. */
int hk_selftest_bounded_wait(int device, unsigned limit_us);

/* Host-only self-test (no GPU needed): the multiply-and-shift division by launch constants with which the kernels
 * turn a work-item index into (batch, kv head, head, tile) is checked against integer division over divisors
 * 1..4096, divisors around every power of two and dividends at the edges of [0, 2^31). Returns HK_OK. The reference
 * decodes its block index with plain divisions (kernels/attn/gqa/kernel.cpp:104-118). */
int hk_selftest_fastdiv(void);

/* Number of kernels this library has launched in the calling process (all devices). */
unsigned long long hk_kernel_launch_count(void);

/* Text for an HK_* code, and the text of the last CUDA error seen by the calling thread. */
const char* hk_strerror(int code);
const char* hk_last_cuda_error(void);

#ifdef HK_TRACE
/* Tuning builds only (the library compiled with -DHK_TRACE; the shipped build has neither symbol): the prefill
 * kernels' first CTA appends (event, SM clock) pairs per role to `buf`, a device array of 3 x 4096 int64, or
 * stamps nothing when buf is NULL. For the backward, `which` selects the kernel that stamps (0 dK/dV, 1 dQ). */
void hk_debug_set_trace(long long* buf);
void hk_debug_set_trace_bwd_kernel(int which);
#endif

#ifdef __cplusplus
}
#endif
#endif /* HK_ATTN_H_ */
