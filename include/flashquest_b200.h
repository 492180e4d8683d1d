/*
 * flashquest_b200 — C ABI of the B200 (sm_100a) sparse-decode kernels.
 *
 * The reference (flashquest) is pure Python: its "operator interface" is a set of
 * Python call signatures.  Every entry point below replaces one of those functions (the
 * reference file:line is cited beside each) and is what a ctypes/cffi binding on the
 * reference side would call.  Conventions:
 *   - all pointers are DEVICE pointers unless stated; nothing here allocates or frees
 *     device memory, and nothing synchronises the stream;
 *   - tensors are described by pointer + element strides of the outer dimensions; the
 *     innermost dimension is always contiguous;
 *   - dtype codes: FQ_F32 / FQ_F16 / FQ_BF16;
 *   - `stream` is a cudaStream_t passed as void*;
 *   - return value: 0 on success, a negative FQ_ERR_* otherwise; the message of the last
 *     failure on the calling thread is returned by fq_last_error_string().  Invalid
 *     arguments are rejected on the host; no kernel traps or asserts on the device.
 */
#ifndef FLASHQUEST_B200_H
#define FLASHQUEST_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FQ_F32 0
#define FQ_F16 1
#define FQ_BF16 2

#define FQ_OK 0
#define FQ_ERR_ARG (-1)         /* bad shape / size / null pointer */
#define FQ_ERR_DTYPE (-2)       /* unsupported dtype code */
#define FQ_ERR_ALIGN (-3)       /* pointer or stride alignment not met */
#define FQ_ERR_UNSUPPORTED (-4) /* head_dim / page_size outside the built set */
#define FQ_ERR_CUDA (-5)        /* CUDA runtime error at launch */
#define FQ_ERR_WORKSPACE (-6)   /* workspace too small */
#define FQ_ERR_TIMEOUT (-7)     /* a bounded device-side wait gave up (see fq_device_status) */

const char* fq_last_error_string(void);
const char* fq_version(void);

/* Reads and clears the device-side status word of the current device (synchronises the
 * device).  0 = no kernel reported a problem; FQ_ERR_TIMEOUT = a bounded wait on an
 * asynchronous copy ran out and the kernel returned early. */
int fq_device_status(void);

/* ------------------------------------------------------------------------------------
 * INT4 KV quantisation ("pack on append").
 * Replaces quantize_k_int4 (kernel/kv_quant.py:152-171), quantize_v_int4 (:189-205) and
 * the page-flush part of PersistentInt4KVCache.update_quantized
 * (cache/persistent_int4.py:94-130), bit-exactly.
 *
 * The token stream of every (b,h) is  head[0:n_head] ++ new[0:n_new]  (the staged partial
 * page followed by the new tokens; n_head = 0 for a plain quantize call).  Its first
 * n_quant tokens are quantised: K per page and channel (scale,min in the INPUT dtype, codes
 * from fp32 division, round-half-even), V per token in fp32; two codes per byte, low nibble =
 * even channel.  A ragged last page (n_quant % page != 0) takes min/max over its valid
 * tokens only.  Outputs are written at token 0 / page 0 of the given pointers — pass
 * pointers already offset into the cache.  Stream token t >= n_quant is left in staging row
 * t - n_quant of stage_K/stage_V (unless those pointers are NULL); the head may BE the
 * staging buffer: with n_quant == 0 its tokens stay where they are and the new ones follow.
 * K or V (and their outputs) may be NULL to quantise only the other one; K_packed alone may
 * be NULL to get only the per-page K metadata (what quantize_k_turbo keeps for scoring,
 * kernel/kv_quant.py:355).
 *
 *   K_head,V_head : (B,H,n_head,D) dtype, strides hd_sb,hd_sh,hd_ss (elements)
 *   K_new, V_new  : (B,H,n_new,D)  dtype, strides nw_sb,nw_sh,nw_ss
 *   K_packed,V_packed : (B,H,n_quant,D/2) u8, strides pk_sb,pk_sh,pk_ss (bytes)
 *   K_scale,K_mn  : (B,H,ceil(n_quant/page),D) bf16, strides km_sb,km_sh,km_sp
 *   V_scale,V_mn  : (B,H,n_quant) bf16, strides vm_sb,vm_sh,vm_ss
 *   stage_K,stage_V : (B,H,page,D) dtype, strides st_sb,st_sh,st_ss
 * D must be 8,16,...,256 with D/8 a power of two; rows 16-byte aligned.
 */
int fq_quantize_kv_int4(
    const void* K_head, const void* V_head, int64_t hd_sb, int64_t hd_sh, int64_t hd_ss, int n_head,
    const void* K_new, const void* V_new, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    int dtype, int B, int H, int D, int page, int n_quant,
    uint8_t* K_packed, uint8_t* V_packed, int64_t pk_sb, int64_t pk_sh, int64_t pk_ss,
    void* K_scale, void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    void* V_scale, void* V_mn, int64_t vm_sb, int64_t vm_sh, int64_t vm_ss,
    void* stage_K, void* stage_V, int64_t st_sb, int64_t st_sh, int64_t st_ss,
    void* stream);

/* dequantize_k_int4 / dequantize_v_int4 (kernel/kv_quant.py:174-186, :208-215):
 * out = bf16(code*scale + mn), used by the prefill branch
 * (eager/llama_persistent_patch.py:196-201).  per_page != 0: metadata (B,H,P,D) (K);
 * else (B,H,S) (V).  out (B,H,S,D) bf16 with strides o_sb,o_sh,o_ss. */
int fq_dequantize_int4(
    const uint8_t* packed, int64_t pk_sb, int64_t pk_sh, int64_t pk_ss,
    const void* scale, const void* mn, int64_t m_sb, int64_t m_sh, int64_t m_s2,
    int per_page, int B, int H, int S, int D, int page,
    void* out, int64_t o_sb, int64_t o_sh, int64_t o_ss, void* stream);

/* ------------------------------------------------------------------------------------
 * Page scores from INT4 metadata.
 * Replaces page_scores_int4_fast (eager/criticality.py:128-163) for S_q == 1:
 *   score[b,hq,p] = sum_d q*K_mn[p,d] + 15 * sum_d relu(q)*K_scale[p,d]   (fp32)
 * One pass over the metadata serves all query heads of a KV group.  Summation order is
 * fixed, so results are reproducible bit for bit: channels are cut into chunks of 8; lane l
 * (0..7) owns chunks l, l+8, ... and accumulates them in ascending order with fused
 * multiply-adds from zero; the eight lane sums combine as ((p0+p4)+(p2+p6))+((p1+p5)+(p3+p7));
 * the product by 15 and the final add are separate roundings.
 *   Q (B,Hq,D) dtype q_dtype strides q_sb,q_sh; K_scale,K_mn (B,Hkv,P,D) bf16 strides
 *   km_sb,km_sh,km_sp; scores (B,Hq,P) fp32 strides sc_sb,sc_sh.  D in {32,64,128,256}.
 */
int fq_page_scores_int4(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P, int D,
    float* scores, int64_t sc_sb, int64_t sc_sh, void* stream);

/* ------------------------------------------------------------------------------------
 * Top-k page selection with static k_max, sinks and window; optional compact index.
 * Replaces select_pages_vectorized (eager/selection.py:65-126) and
 * build_compact_selection (:129-164).
 *   k_h = clamp(ceil(fp32(r_h) * P), 0, P) with r_h = retention_per_head[h] (device fp32,
 *   length H) or the scalar `retention` when that pointer is NULL; the k_max largest
 *   scores are found and the first min(k_h,k_max) kept; pages [0,min(sinks,P)) and
 *   [P-min(window,P),P) are forced on.  Ties between equal scores: the lower page index
 *   wins (torch.topk leaves this unspecified).
 * Outputs (each optional, NULL to skip):
 *   mask    (B,H,P) u8 0/1, strides mk_sb,mk_sh
 *   compact (B,H,bucket) int32: selected ids in DESCENDING order, truncated to bucket,
 *           padded with -1 (exactly build_compact_selection's output), strides cp_sb,cp_sh
 *   count   (B,H) int32: number of selected pages (contiguous)
 */
int fq_select_pages(
    const float* scores, int64_t sc_sb, int64_t sc_sh, int B, int H, int P,
    const float* retention_per_head, float retention, int k_max, int sinks, int window,
    uint8_t* mask, int64_t mk_sb, int64_t mk_sh,
    int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    int32_t* count, void* stream);

/* build_compact_selection (eager/selection.py:129-164) on an existing mask.
 * mask (rows,P) u8 with row stride mk_sr; compact (rows,bucket) int32 with stride cp_sr. */
int fq_build_compact(const uint8_t* mask, int64_t mk_sr, int64_t rows, int P,
                     int32_t* compact, int64_t cp_sr, int bucket, void* stream);
/* The same, and count (rows) int32 receives min(selected pages, bucket) per row: the number of real entries at
 * the front of the row's list (or NULL).  Hand it to fq_sparse_decode_int4_counted so that the padding of a list as
 * wide as the page count -- what a mask-driven call produces -- is not walked. */
int fq_build_compact_counted(const uint8_t* mask, int64_t mk_sr, int64_t rows, int P,
                             int32_t* compact, int64_t cp_sr, int bucket, int32_t* count, void* stream);

/* Page scores, top-k and compact index in ONE launch: fq_page_scores_int4 (levels 15) or
 * fq_page_scores_int8 (levels 255) followed by fq_select_pages with a compact list and no mask, i.e.
 * page_scores_int4_fast / page_scores_int8_fast -> select_pages_vectorized -> build_compact_selection
 * (eager/criticality.py:77-163, eager/selection.py:65-164) as the decode branch chains them
 * (eager/llama_persistent_patch.py:214-228).  Same arguments and the same bits in `scores` and
 * `compact` as the two separate calls.  A thread-block cluster of 8 CTAs per (batch, KV head) scores
 * the pages once for the whole GQA group and hands each head's keys through distributed shared memory
 * to the CTA that selects for it.  Shapes: at most 4 query heads per KV head, P <= 16384, head_dim in
 * {32,64,128,256} (fq_score_select_supported tells; other shapes take the two separate calls).
 * first_fresh_page: the caller's word that the metadata rows of pages below it were written BEFORE the
 * launch that precedes this call in the stream (a decode step that appended one token passes the index
 * of the page that token went to); their copies are then requested ahead of the dependency wait and
 * overlap the previous kernel.  0 = no such promise. */
int fq_score_select_supported(int Hq, int Hkv, int P, int D);
int fq_score_select(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P, int D, int levels, float* scores, int64_t sc_sb, int64_t sc_sh,
    const float* retention_per_head, float retention, int k_max, int sinks, int window,
    int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket, int32_t* count, int first_fresh_page, void* stream);

/* ------------------------------------------------------------------------------------
 * INT8 KV variant (cache.kv_bits == 8): KIVI-style asymmetric uint8, one code per byte.
 * fq_quantize_kv_int8 replaces quantize_k / quantize_v (kernel/kv_quant.py:45-62, :81-93):
 *   K per page and channel, scale = (mx - mn) / 255 and mn in the INPUT dtype, eps clamp 1e-6,
 *   codes = clamp(rint((K_f32 - mn) / scale), 0, 255); V per token in fp32; metadata stored bf16.
 *   K, V (B,H,S,D) dtype with strides in_sb,in_sh,in_ss (either may be NULL); codes (B,H,S,D) u8
 *   strides c_sb,c_sh,c_ss; K_scale,K_mn (B,H,P,D) bf16; V_scale,V_mn (B,H,S) bf16.
 * fq_dequantize_int8 replaces dequantize_k / dequantize_v (:65-78, :96-103): bf16(code*scale + mn).
 * fq_page_scores_int8 replaces page_scores_int8_fast (eager/criticality.py:77-125): the INT4 score
 *   with 255 levels, same fixed summation order.
 * fq_sparse_decode_int8 replaces flash_attn_sparse_fwd (kernel/sparse_fwd.py:140-228) over a compact
 *   page list (as fq_sparse_decode_int4; a bool mask goes through fq_build_compact first), with the
 *   optional staged tail in the same softmax.  O (B,Hq,D) q_dtype dense, lse (B,Hq) fp32 or NULL.
 *   workspace: fq_sparse_decode_int8_workspace_bytes(B,Hq,D,n_split) bytes, always needed, no
 *   initial contents required.
 */
int fq_quantize_kv_int8(
    const void* K, const void* V, int64_t in_sb, int64_t in_sh, int64_t in_ss, int dtype, int B, int H, int S, int D, int page,
    uint8_t* K_uint8, uint8_t* V_uint8, int64_t c_sb, int64_t c_sh, int64_t c_ss,
    void* K_scale, void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    void* V_scale, void* V_mn, int64_t vm_sb, int64_t vm_sh, void* stream);
int fq_dequantize_int8(
    const uint8_t* codes, int64_t c_sb, int64_t c_sh, int64_t c_ss,
    const void* scale, const void* mn, int64_t m_sb, int64_t m_sh, int64_t m_s2,
    int per_page, int B, int H, int S, int D, int page, void* out, int64_t o_sb, int64_t o_sh, int64_t o_ss, void* stream);
int fq_page_scores_int8(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P, int D,
    float* scores, int64_t sc_sb, int64_t sc_sh, void* stream);
size_t fq_sparse_decode_int8_workspace_bytes(int B, int Hq, int D, int n_split);
int fq_sparse_decode_int8(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_uint8, const uint8_t* V_uint8, int64_t kv_sb, int64_t kv_sh, int64_t kv_ss,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss, int tail_len,
    int B, int Hq, int Hkv, int S_kv, int P, int D, int page, float sm_scale,
    void* O, float* lse, void* workspace, size_t workspace_bytes, int n_split, void* stream);
/* The same for a list whose real entries sit at the front (what fq_build_compact_counted makes from a mask):
 * list_count (B*Hq) int32 bounds the entries walked per row; NULL = all of them. */
int fq_sparse_decode_int8_counted(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_uint8, const uint8_t* V_uint8, int64_t kv_sb, int64_t kv_sh, int64_t kv_ss,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket, const int32_t* list_count,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss, int tail_len,
    int B, int Hq, int Hkv, int S_kv, int P, int D, int page, float sm_scale,
    void* O, float* lse, void* workspace, size_t workspace_bytes, int n_split, void* stream);

/* ------------------------------------------------------------------------------------
 * Dense causal attention of the prefill branch (S_q > 1).
 * Replaces the torch.nn.functional.scaled_dot_product_attention(q, K_full, V_full,
 * is_causal=True, enable_gqa=True) call of the patched forward
 * (eager/llama_persistent_patch.py:196-201), where K_full / V_full are the dequantised
 * completed pages followed by the staged tail.  The causal mask is aligned at the top left,
 * as torch aligns it when S_q != S_kv: query i attends keys 0..i.  Tensor-core kernels, fp32
 * accumulation and softmax: tcgen05 (S and P.V in tensor memory, TMA-staged operands) for head_dim 128
 * with at least 128 queries, mma.sync otherwise.
 *   Q (B,Hq,Sq,D), K,V (B,Hkv,Skv,D), O (B,Hq,Sq,D): all `dtype` (F16|BF16), element strides
 *   *_sb,*_sh,*_ss (head_dim contiguous; pass O's strides to write a (B,Sq,Hq*D) buffer).
 * D in {64,128}; Q/K/V rows 16-byte aligned.
 */
int fq_prefill_attention(
    const void* Q, int64_t q_sb, int64_t q_sh, int64_t q_ss,
    const void* K, int64_t k_sb, int64_t k_sh, int64_t k_ss,
    const void* V, int64_t v_sb, int64_t v_sh, int64_t v_ss,
    int dtype, int B, int Hq, int Hkv, int Sq, int Skv, int D, float sm_scale,
    void* O, int64_t o_sb, int64_t o_sh, int64_t o_ss, void* stream);

/* ------------------------------------------------------------------------------------
 * Sparse decode attention over selected packed INT4 pages (GQA, split-K, LSE merge).
 * Replaces flash_attn_sparse_int4_fwd_compact (kernel/sparse_int4_fwd_compact.py:153-244)
 * and, with a compact list built from the mask, flash_attn_sparse_int4_fwd
 * (kernel/sparse_int4_fwd.py:160-248); with a tail it also covers
 * _bf16_dense_attn_with_lse + _merge_two_attentions
 * (eager/llama_persistent_patch.py:30-61) in the same softmax.
 *
 *   Q (B,Hq,D) q_dtype (F16|BF16), strides q_sb,q_sh;  O same dtype, strides o_sb,o_sh
 *   K_packed,V_packed (B,Hkv,S_kv,D/2) u8, strides in bytes; token stride must be D/2
 *   K_scale,K_mn (B,Hkv,P,D) bf16;  V_scale,V_mn (B,Hkv,S_kv) bf16 (token stride 1)
 *   compact (B,Hq,bucket) int32 page ids; ids < 0 or >= P are skipped (order irrelevant)
 *   K_tail,V_tail (B,Hkv,tail_len,D) tail_dtype (F16|BF16) or NULL with tail_len = 0
 *   lse (B,Hq) fp32 in nats or NULL.  Nothing attended => O = 0, lse = -inf.
 *   n_split: CTAs per (b,hq) row (1..1024); with n_split > 1 `workspace` must hold
 *   fq_sparse_decode_workspace_bytes(...) bytes whose first B*Hq*4 bytes were zeroed once
 *   (the kernel leaves them zero again); concurrent calls must not share a workspace.
 * D in {64,128}; page in {8,16,32,64,128}.  Page rows must be 16-byte aligned.
 */
size_t fq_sparse_decode_workspace_bytes(int B, int Hq, int D, int n_split);
int fq_sparse_decode_default_splits(int B, int Hq, int bucket, int page);
int fq_sparse_decode_int4(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_packed, int64_t kp_sb, int64_t kp_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const uint8_t* V_packed, int64_t vp_sb, int64_t vp_sh,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss,
    int tail_len,
    int B, int Hq, int Hkv, int S_kv, int P, int D, int page, float sm_scale,
    void* O, int64_t o_sb, int64_t o_sh, float* lse,
    void* workspace, size_t workspace_bytes, int n_split, void* stream);
/* fq_sparse_decode_int4 for a list whose real entries sit at the front: list_count (B*Hq) int32, contiguous, gives per
 * (b,hq) row how many leading entries to walk (clamped to [0, bucket]); NULL = all of them.  This is how
 * flash_attn_sparse_int4_fwd (kernel/sparse_int4_fwd.py:160-248, the bool-mask form) runs: fq_build_compact_counted,
 * then this call. */
int fq_sparse_decode_int4_counted(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_packed, int64_t kp_sb, int64_t kp_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const uint8_t* V_packed, int64_t vp_sb, int64_t vp_sh,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket, const int32_t* list_count,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss,
    int tail_len,
    int B, int Hq, int Hkv, int S_kv, int P, int D, int page, float sm_scale,
    void* O, int64_t o_sb, int64_t o_sh, float* lse,
    void* workspace, size_t workspace_bytes, int n_split, void* stream);

/* Sparse decode attention with built-in scratch: same computation and arguments as
 * fq_sparse_decode_int4, minus the workspace.  It has no counterpart in the reference; it
 * exists for hosts that cannot supply device memory when they call in (a language binding
 * without a CUDA allocator, a loop that must stay clear of cudaMalloc/cudaFree because they
 * stall the device, a plugin that only receives its inputs and outputs).  The split-K scratch
 * is a fixed array of FQ_SPARSE_DECODE_STATIC_SCRATCH_BYTES inside the library, resident on
 * every GPU that loads it until the process ends.  The call allocates and frees nothing.
 *   - Limit: fq_sparse_decode_workspace_bytes(B,Hq,D,n_split) must not exceed the array
 *     (4 MiB: e.g. B*Hq*n_split <= 8000 at D = 128); larger requests return
 *     FQ_ERR_WORKSPACE and touch nothing.  n_split <= 0 picks the default split count.
 *   - The first call on a device looks up the array's device address; make that call
 *     outside any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents; the entry
 *     point clears the ticket words it needs at zero on `stream` before launching.  Two calls
 *     whose work overlaps on the GPU (different streams) corrupt each other: serialise them.
 */
#define FQ_SPARSE_DECODE_STATIC_SCRATCH_BYTES (4u << 20)
int fq_sparse_decode_int4_static(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_packed, int64_t kp_sb, int64_t kp_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const uint8_t* V_packed, int64_t vp_sb, int64_t vp_sh,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss,
    int tail_len,
    int B, int Hq, int Hkv, int S_kv, int P, int D, int page, float sm_scale,
    void* O, int64_t o_sb, int64_t o_sh, float* lse, int n_split, void* stream);

/* ------------------------------------------------------------------------------------
 * TurboQuant K3-V3: Walsh-Hadamard rotation, 3-bit Lloyd-Max codes in bit planes.
 *
 * fq_wht — wht_along_head_dim (kernel/wht.py:17-41): normalised WHT along the last axis of
 * n_rows dense rows of D values (D a power of two <= 1024), every butterfly stage and the
 * final division by sqrt(D) rounded to `dtype` as the reference's eager ops do (bit-exact).
 */
int fq_wht(const void* x, void* out, int dtype, int64_t n_rows, int D, void* stream);

/* quantize_k_turbo / quantize_v_turbo without the raw page metadata
 * (kernel/kv_quant.py:327-405).  Token stream head[0:n_head] ++ new[0:n_new] as in
 * fq_quantize_kv_int4; its first n_quant tokens are rotated (WHT in the input dtype), scaled
 * by their RMS (fp32: each of 32 lanes sums the squares of its D/32 consecutive values in
 * ascending order with fused multiply-adds, the lane sums combine by an xor butterfly
 * 16,8,4,2,1; then /D, sqrt, clamp at 1e-6), coded to the nearest of the 8 codebook values
 * (first index on ties) and split into planes: bit i of msb byte k = (idx[8k+i] >> 2) & 1,
 * bits 2i..2i+1 of lsb byte k = idx[4k+i] & 3.  Bit-exact against the reference except where
 * the summation order of the RMS moves a value across a code boundary.
 *   msb (B,H,n_quant,D/8) u8, lsb (B,H,n_quant,D/4) u8, scale (B,H,n_quant) bf16.
 * The per-page K metadata that quantize_k_turbo also returns (kv_quant.py:355) and the
 * staging of left-over tokens come from fq_quantize_kv_int4 with K_packed = V_packed = NULL. */
int fq_quantize_turbo(
    const void* head, int64_t hd_sb, int64_t hd_sh, int64_t hd_ss, int n_head,
    const void* nw, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    int dtype, int B, int H, int D, int n_quant,
    uint8_t* msb, int64_t ms_sb, int64_t ms_sh, int64_t ms_ss,
    uint8_t* lsb, int64_t ls_sb, int64_t ls_sh, int64_t ls_ss,
    void* scale, int64_t sc_sb, int64_t sc_sh, int64_t sc_ss, void* stream);

/* dequantize_k_turbo / dequantize_v_turbo (kernel/kv_quant.py:366-378, :408-420):
 * codebook[idx]*scale in fp32, WHT in fp32, result bf16 (B,H,S,D) in the raw basis. */
int fq_dequantize_turbo(
    const uint8_t* msb, int64_t ms_sb, int64_t ms_sh, int64_t ms_ss,
    const uint8_t* lsb, int64_t ls_sb, int64_t ls_sh, int64_t ls_ss,
    const void* scale, int64_t sc_sb, int64_t sc_sh, int64_t sc_ss,
    int B, int H, int S, int D, void* out, int64_t o_sb, int64_t o_sh, int64_t o_ss, void* stream);

/* Sparse decode attention over K3-V3 planes in the ROTATED basis: the kernel part of
 * flash_attn_sparse_turbo_fwd (kernel/sparse_turbo_fwd.py:110-346).  The caller rotates Q
 * with fq_wht before and O after, as the reference wrapper does (:305, :343-344).
 * Q_rot, O_rot (B,Hq,D) fp16|bf16; planes and scales as produced by fq_quantize_turbo
 * (scale token stride 1); compact, lse, workspace, n_split as for fq_sparse_decode_int4.
 * D in {64,128}; page a multiple of 16. */
int fq_sparse_decode_turbo(
    const void* Q_rot, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_msb, int64_t km_sb, int64_t km_sh, int64_t km_ss,
    const uint8_t* K_lsb, int64_t kl_sb, int64_t kl_sh, int64_t kl_ss,
    const void* K_scale, int64_t ks_sb, int64_t ks_sh,
    const uint8_t* V_msb, int64_t vm_sb, int64_t vm_sh, int64_t vm_ss,
    const uint8_t* V_lsb, int64_t vl_sb, int64_t vl_sh, int64_t vl_ss,
    const void* V_scale, int64_t vs_sb, int64_t vs_sh,
    const int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    int B, int Hq, int Hkv, int S_kv, int P, int D, int page, float sm_scale,
    void* O_rot, int64_t o_sb, int64_t o_sh, float* lse,
    void* workspace, size_t workspace_bytes, int n_split, void* stream);

/* _merge_two_attentions (eager/llama_persistent_patch.py:50-61) for n partial results that
 * share Q: O_parts (n,rows,D) dtype, lse_parts (n,rows) fp32 nats -> O (rows,D) dtype,
 * lse (rows) fp32 or NULL.  Rows whose parts are all empty (lse = -inf) give O = 0. */
int fq_lse_merge(const void* O_parts, const float* lse_parts, int dtype, int n, int64_t rows, int D,
                 void* O, float* lse, void* stream);

/* fq_lse_merge with strided parts: part i of row r starts at O_parts + i*o_part_stride + r*D
 * (elements of dtype) and lse_parts + i*lse_part_stride + r (floats), e.g. messages gathered
 * from several GPUs that each hold (O, lse) back to back. */
int fq_lse_merge_strided(const void* O_parts, int64_t o_part_stride, const float* lse_parts, int64_t lse_part_stride,
                         int dtype, int n, int64_t rows, int D, void* O, float* lse, void* stream);

/* ------------------------------------------------------------------------------------
 * Context split: ONE long sequence whose pages are split over G GPUs by contiguous range (rank r
 * owns pages [lo, hi) with their packed codes and metadata; Q is replicated).  Not in the
 * reference, which is single-GPU; the result equals the single-GPU result of
 * select_pages_vectorized (eager/selection.py:65-126) + flash_attn_sparse_int4_fwd_compact
 * (kernel/sparse_int4_fwd_compact.py:153-244) + tail + merge over the whole sequence.  Per decode
 * step and layer the host runs, on every rank,
 *   fq_ctx_local_candidates -> all-gather of msg -> fq_ctx_select_attend -> all-gather of
 *   (O, lse) -> fq_lse_merge_strided,
 * with both all-gathers delivering into this rank's own memory (e.g. ncclAllGather); none of the
 * kernels reads another GPU's memory.  All three calls only enqueue work on `stream` and can be
 * captured in a CUDA graph together with the collectives.
 *   k_global = the single-GPU k (clamp(ceil(fp32(retention)*P_global), 0, P_global), capped by
 *   the static k_max); k_c = min(k_global, largest page count of any rank) candidate slots per
 *   rank and head; bucket_local = min(P_local, k_global + sinks + window).
 *   msg (B,Hq,2,k_c) fp32: scores and (bit-cast) global page ids of this rank's candidates;
 *   gathered (G,B,Hq,2,k_c): all ranks' messages in rank order.
 *   O_msg (B,Hq,D) q_dtype and lse_msg (B,Hq) fp32: this rank's partial result, to be gathered.
 *   scratch: fq_ctx_scratch_bytes(B,Hq,G,k_c,P_local,bucket_local) bytes, the same buffer for
 *   both calls; workspace / n_split as for fq_sparse_decode_int4.
 * Scalar retention only.  K_tail / V_tail: the staged tokens, on the last rank only. */
size_t fq_ctx_scratch_bytes(int B, int Hq, int G, int k_c, int P_local, int bucket_local);
int fq_ctx_local_candidates(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P_local, int D, int lo, int k_c, int G, int bucket_local,
    void* scratch, size_t scratch_bytes, float* msg, void* stream);
int fq_ctx_select_attend(
    const float* gathered, int G, int k_c, int k_global, int sinks, int window, int lo, int hi, int P_global,
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_packed, int64_t kp_sb, int64_t kp_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const uint8_t* V_packed, int64_t vp_sb, int64_t vp_sh,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss, int tail_len,
    int B, int Hq, int Hkv, int D, int page, float sm_scale, int bucket_local,
    void* scratch, size_t scratch_bytes, void* O_msg, float* lse_msg,
    void* workspace, size_t workspace_bytes, int n_split, void* stream);

/* ------------------------------------------------------------------------------------
 * AWQ W4A16 GEMV, several projections of the same input fused in one launch.
 * Replaces fused_qkv_proj / fused_gate_up_proj (kernel/fused_proj.py:18-53), which in the
 * reference call AutoAWQ 0.2.9 modules one after the other (third party, not part of the
 * reference tree: parity is against a restatement of AutoAWQ's published GEMM format, not
 * against reference outputs).  Layout per quant/awq_layout.py:18-44: qweight (K, N/8) int32,
 * scales (K/G, N) fp16, qzeros (K/G, N/8) int32; w = (code - zero) * scale; `interleaved` != 0:
 * nibble i of an int32 holds column 8c + {0,2,4,6,1,3,5,7}[i] (AutoAWQ GEMM order), else 8c + i.
 *   x (M,K) fp16 dense, 1 <= M <= 8; arrays of n_proj (<= 4) HOST arrays holding device
 *   pointers / sizes; bias NULL, or n_proj entries each NULL or (N[i]) fp16, added in fp32
 *   before the rounding to fp16; y[i] (M,N[i]) fp16 dense.  fp32 accumulation.
 *   k_split (1, 2, 4 or 8; ask fq_awq_gemv_default_splits): the CTAs that share one tile of
 *   256 outputs split K between them as one thread-block cluster and merge their partial sums
 *   through distributed shared memory in rank order — no workspace, no atomics.
 *
 * fq_awq_gemv_fused is the same launch with the element-wise operator in front of the linear and
 * the rotary embedding behind it folded in, for the decode step of a Llama-shaped layer (the
 * Hugging Face modules around the patched attention, eager/llama_persistent_patch.py:164-190,
 * 246-251: input_layernorm -> q/k/v_proj -> apply_rotary_pos_emb; post_attention_layernorm ->
 * gate/up_proj; act_fn(gate) * up -> down_proj), with the same roundings to fp16 as the separate
 * operators (fq_add_rmsnorm, fq_swiglu, fq_rope):
 *   pro (NULL = none): FQ_GEMV_ADD_RMSNORM: input = weight * fp16((x + b) * rsqrt(mean((x+b)^2) + eps)),
 *     b NULL or (M,K); x + b is also written to `out` (M,K) when given (the new residual stream; it
 *     must not alias x or b).  FQ_GEMV_SWIGLU: input = fp16(silu(x)) * b with x = gate, b = up (M,K);
 *     written to `out` when given.
 *   rope (NULL = none): outputs of projection i with bit i of proj_mask set are rotated in place of
 *     the plain store, rotate_half convention, position *pos_dev when pos_dev is given, else pos;
 *     the same position for all M rows.  head_dim must divide 256, N[i] be a multiple of it. */
enum { FQ_GEMV_PLAIN = 0, FQ_GEMV_ADD_RMSNORM = 1, FQ_GEMV_SWIGLU = 2 };
typedef struct fq_gemv_prologue {
    int kind;
    const void* b;
    const void* weight;
    float eps;
    void* out;
} fq_gemv_prologue;
typedef struct fq_gemv_rope {
    unsigned proj_mask;
    const int* pos_dev;
    int pos;
    float theta;
    int head_dim;
} fq_gemv_rope;
int fq_awq_gemv_default_splits(int K, int N_total, int group);
int fq_awq_gemv(
    const void* x, int M, int K, int group, int n_proj,
    const int32_t* const* qweight, const void* const* scales, const int32_t* const* qzeros, const void* const* bias,
    const int* N, void* const* y, int interleaved, int k_split, void* stream);
int fq_awq_gemv_fused(
    const void* x, int M, int K, int group, int n_proj,
    const int32_t* const* qweight, const void* const* scales, const int32_t* const* qzeros, const void* const* bias,
    const int* N, void* const* y, int interleaved, const fq_gemv_prologue* pro, const fq_gemv_rope* rope, int k_split, void* stream);

/* AWQ W4A16 dequant-GEMM for prefill / batched shapes (any M >= 1): the same computation as
 * fq_awq_gemv — the linears kernel/fused_proj.py:36-39,51-53 and the patched forward
 * (eager/llama_persistent_patch.py:176-178,251) run through AutoAWQ's GEMM modules — on the tensor
 * cores (tcgen05.mma, fp32 accumulation in tensor memory, operands staged by TMA).  The codes are
 * dequantised to fp16, (code - zero) * scale rounded once, as AutoAWQ's GEMM kernels do.  Parity
 * unpinned, as for fq_awq_gemv.
 *   x (M,K) fp16 dense; up to 4 projections that share x (fused QKV, gate/up): arrays of n_proj
 *   HOST arrays of device pointers / sizes; N[i] a multiple of 128, K a multiple of the group
 *   size (64, 128 or 256); y[i] (M,N[i]) fp16 dense; bias NULL or per projection NULL / (N[i]) fp16.
 * Needs no workspace.  The call builds TMA descriptors on the host (no allocation, no sync). */
int fq_awq_gemm(
    const void* x, int M, int K, int group, int n_proj,
    const int32_t* const* qweight, const void* const* scales, const int32_t* const* qzeros, const void* const* bias,
    const int* N, void* const* y, int interleaved, void* stream);

/* ------------------------------------------------------------------------------------
 * One decode step of one layer on a persistent INT4 cache: append + score + select + attend.
 * Replaces, in one host call and four launches, what the reference's patched forward does
 * per layer and step around the projections (eager/llama_persistent_patch.py:193-245):
 * cache.update_quantized (cache/persistent_int4.py:69-132), page_scores_int4_fast,
 * select_pages_vectorized + build_compact_selection, the sparse kernel, the partial-page
 * tail attention and the LSE merge.
 *
 * fq_int4_cache describes the storage of PersistentInt4KVCache (cache/persistent_int4.py:46-61):
 * base pointers of layer 0 and element strides of the (layer, batch, head, row) axes; the
 * innermost axis is dense.  `seen` is the number of tokens in the layer BEFORE this call
 * (the reference keeps it in _seen_tokens); the call appends n_new tokens and attends over
 * seen + n_new tokens with S_q = 1.
 */
typedef struct fq_int4_cache {
    uint8_t* K_packed; uint8_t* V_packed;          /* (L,B,H,S,D/2) u8 */
    int64_t pk_sl, pk_sb, pk_sh, pk_ss;            /* bytes */
    void* K_scale; void* K_mn;                     /* (L,B,H,P,D) bf16 */
    int64_t km_sl, km_sb, km_sh, km_sp;
    void* V_scale; void* V_mn;                     /* (L,B,H,S) bf16, token stride 1 */
    int64_t vm_sl, vm_sb, vm_sh;
    void* K_partial; void* V_partial;              /* (L,B,H,page,D) kv_dtype */
    int64_t pt_sl, pt_sb, pt_sh, pt_ss;
    int kv_dtype;                                  /* FQ_F16 | FQ_BF16 */
    int L, B, Hkv, D, page, max_seq_len;
} fq_int4_cache;

typedef struct fq_decode_params {
    int Hq;
    const float* retention_per_head;               /* device, length Hq, or NULL */
    float retention;
    int k_max_static, sinks, window, bucket;       /* bucket = k_max_static + sinks + window */
    float sm_scale;
    int n_split;                                   /* 0: fq_sparse_decode_default_splits */
} fq_decode_params;

/* K_new,V_new (B,Hkv,n_new,D) kv_dtype with strides nw_sb,nw_sh,nw_ss; Q (B,Hq,D) q_dtype;
 * scores (B,Hq,P_max) fp32 and compact (B,Hq,bucket) int32 are caller-provided scratch, dense;
 * O (B,Hq,D) q_dtype dense, lse (B,Hq) fp32 or NULL; workspace as for fq_sparse_decode_int4.
 * Fails with FQ_ERR_ARG if seen + n_new exceeds max_seq_len or layer is out of range. */
int fq_decode_layer_int4(
    const fq_int4_cache* cache, int layer, int seen,
    const void* K_new, const void* V_new, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const fq_decode_params* params,
    float* scores, int32_t* compact, void* O, float* lse,
    void* workspace, size_t workspace_bytes, void* stream);

/* One decode step of one layer on a persistent TurboQuant K3-V3 cache, in one host call: what the
 * reference's patched forward does for cache.kv_bits == 3 (eager/llama_persistent_patch.py:93-115,
 * 193-245): PersistentTurboKVCache.update_quantized (cache/persistent_turbo.py:83-147),
 * page_scores_int4_fast on K_scale_raw / K_mn_raw, select_pages_vectorized +
 * build_compact_selection, flash_attn_sparse_turbo_fwd (with the rotation of Q before and of O
 * after the kernel, kernel/sparse_turbo_fwd.py:305,343-344), _bf16_dense_attn_with_lse over the
 * staged tokens and _merge_two_attentions.
 * fq_turbo_cache describes the storage of PersistentTurboKVCache (cache/persistent_turbo.py:46-66)
 * like fq_int4_cache does for the INT4 cache; both msb planes share one set of strides, both lsb
 * planes another, both token scales a third.  Q and O are dense (B,Hq,D) in the RAW basis;
 * scores (B,Hq,P) and compact (B,Hq,bucket) are scratch; `scratch` holds
 * fq_decode_layer_turbo_scratch_bytes(B,Hq,D) bytes (rotated Q and O, the two partial results);
 * workspace / n_split as for fq_sparse_decode_turbo.  page must be a multiple of 16. */
typedef struct fq_turbo_cache {
    uint8_t* K_msb; uint8_t* K_lsb; uint8_t* V_msb; uint8_t* V_lsb;   /* (L,B,H,S,D/8) and (L,B,H,S,D/4) u8 */
    int64_t ms_sl, ms_sb, ms_sh, ms_ss;            /* msb planes, bytes */
    int64_t ls_sl, ls_sb, ls_sh, ls_ss;            /* lsb planes, bytes */
    void* K_scale_turbo; void* V_scale_turbo;      /* (L,B,H,S) bf16, token stride 1 */
    int64_t st_sl, st_sb, st_sh;
    void* K_scale_raw; void* K_mn_raw;             /* (L,B,H,P,D) bf16 */
    int64_t km_sl, km_sb, km_sh, km_sp;
    void* K_partial; void* V_partial;              /* (L,B,H,page,D) kv_dtype */
    int64_t pt_sl, pt_sb, pt_sh, pt_ss;
    int kv_dtype;                                  /* FQ_F16 | FQ_BF16 */
    int L, B, Hkv, D, page, max_seq_len;
} fq_turbo_cache;
size_t fq_decode_layer_turbo_scratch_bytes(int B, int Hq, int D);
int fq_decode_layer_turbo(
    const fq_turbo_cache* cache, int layer, int seen,
    const void* K_new, const void* V_new, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const fq_decode_params* params,
    float* scores, int32_t* compact, void* scratch, size_t scratch_bytes, void* O, float* lse,
    void* workspace, size_t workspace_bytes, void* stream);

/* fq_decode_layer_int4 for layers [0, n_layers) in one foreign call — the layer loop of the
 * caller (the decoder-layer loop around eager/llama_persistent_patch.py:164-305, or
 * BASELINE-style stacked independent layers) without one host round trip per layer.  Every
 * per-layer array is addressed as base + layer * stride: K_new/V_new stride nw_sl, Q stride q_sl
 * (elements), scores stride sc_sl, compact stride cp_sl, O stride o_sl, lse stride lse_sl
 * (elements), workspace stride ws_sl (bytes; each layer needs its own split-K workspace).
 * seen[layer] (host array) is the number of tokens already in that layer; params is one
 * struct for all layers (params_stride 0) or an array of structs params_stride bytes apart.
 * Stops at the first failing layer and returns its error. */
int fq_decode_step_int4(
    const fq_int4_cache* cache, int n_layers, const int* seen,
    const void* K_new, const void* V_new, int64_t nw_sl, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    const void* Q, int q_dtype, int64_t q_sl, int64_t q_sb, int64_t q_sh,
    const fq_decode_params* params, size_t params_stride,
    float* scores, int64_t sc_sl, int32_t* compact, int64_t cp_sl, void* O, int64_t o_sl, float* lse, int64_t lse_sl,
    void* workspace, size_t ws_sl, size_t workspace_bytes, void* stream);

/* fq_decode_step_int4 whose launches do not depend on the sequence length, so that the step can be
 * captured once in a CUDA graph and replayed for every new token: pos (DEVICE array, one int per
 * layer) holds the tokens already cached; every kernel reads it on the device, and the last
 * launch adds n_new to each entry.  1 <= n_new < page.  scores must be (B,Hq,P_max) per layer with
 * P_max = max_seq_len / page.  The caller keeps its own count and must not run past max_seq_len
 * (on the device a full layer silently appends nothing). */
int fq_decode_step_int4_dev(
    const fq_int4_cache* cache, int n_layers, int* pos,
    const void* K_new, const void* V_new, int64_t nw_sl, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    const void* Q, int q_dtype, int64_t q_sl, int64_t q_sb, int64_t q_sh,
    const fq_decode_params* params, size_t params_stride,
    float* scores, int64_t sc_sl, int32_t* compact, int64_t cp_sl, void* O, int64_t o_sl, float* lse, int64_t lse_sl,
    void* workspace, size_t ws_sl, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------
 * The operators around the sparse-decode path in a Llama-shaped decode step.  The reference
 * inherits them from the Hugging Face modules its patched forward wraps
 * (eager/llama_persistent_patch.py:164-305: q/k/v_proj, apply_rotary_pos_emb, o_proj; the
 * decoder layer adds the norms, residuals and the SwiGLU MLP); same fp16 roundings here.
 * All tensors fp16, dense.
 *   fq_add_rmsnorm: h = a (+ b if not NULL); sum_out = h (if not NULL); y = weight * fp16(h * rsqrt(mean(h^2)+eps)),
 *                   rows x H.
 *   fq_rope:        rotate-half rotary embedding in place on q (B,Hq,D) and k (B,Hkv,D) (element strides sb, sh)
 *                   at position pos, base theta.
 *   fq_swiglu:      out = fp16(silu(gate)) * up over n elements (n even).
 *   fq_gemv_f16:    y (M,N) = x (M,K) @ W(N,K)^T, fp32 accumulation, 1 <= M <= 8 (the lm_head at decode).
 *   fq_argmax_f16:  index of the first maximum of each row of x (rows,N). */
int fq_add_rmsnorm(const void* a, const void* b, const void* weight, float eps, int64_t rows, int H,
                   void* sum_out, void* y, void* stream);
int fq_rope(void* q, int64_t q_sb, int64_t q_sh, int Hq, void* k, int64_t k_sb, int64_t k_sh, int Hkv,
            int B, int D, int pos, float theta, void* stream);
/* The same rotation for n_tokens consecutive tokens of ONE sequence (prefill): row t of q / k
 * (token strides q_st / k_st, head strides q_sh / k_sh, elements) is rotated for position pos0 + t. */
int fq_rope_tokens(void* q, int64_t q_st, int64_t q_sh, int Hq, void* k, int64_t k_st, int64_t k_sh, int Hkv,
                   int n_tokens, int D, int pos0, float theta, void* stream);
int fq_swiglu(const void* gate, const void* up, int64_t n, void* out, void* stream);
int fq_gemv_f16(const void* x, const void* W, int M, int K, int N, void* y, void* stream);
int fq_argmax_f16(const void* x, int64_t rows, int N, int32_t* out, void* stream);

/* ------------------------------------------------------------------------------------
 * One greedy decode step of a Llama-shaped model in ONE foreign call: the decoder-layer loop
 * around eager/llama_persistent_patch.py:164-305 (Hugging Face's LlamaDecoderLayer / LlamaMLP /
 * LlamaRMSNorm semantics) issued from native code, 8 launches per layer and no host work
 * between them.  Per layer: fq_awq_gemv_fused (add+RMSNorm -> q/k/v -> RoPE), fq_decode_layer_int4
 * (append + score + select + attend), AWQ o GEMV, fq_awq_gemv_fused (add+RMSNorm -> gate/up),
 * fq_awq_gemv_fused (SwiGLU -> down); then add+RMSNorm, fp16 lm_head GEMV, argmax.  fp16 model,
 * B <= 8 sequences.
 * All pointers inside the structs are device pointers except `layers` (host array). */
typedef struct fq_awq_linear {
    const int32_t* qweight; const void* scales; const int32_t* qzeros; const void* bias;   /* bias may be NULL */
    int K, N;
} fq_awq_linear;

typedef struct fq_llama_layer {
    const void* input_norm; fq_awq_linear q, k, v, o;
    const void* post_norm; fq_awq_linear gate, up, down;
} fq_llama_layer;

typedef struct fq_llama_model {
    int hidden, n_layers, q_heads, kv_heads, head_dim, ffn, vocab, group, interleaved;
    float rope_theta, rms_eps;
    const fq_llama_layer* layers;                  /* host array of n_layers entries */
    const void* final_norm; const void* lm_head;   /* (hidden), (vocab, hidden) fp16 */
} fq_llama_model;

typedef struct fq_llama_scratch {
    void *resid0, *resid1, *normed;                /* (B, hidden) fp16 */
    void *q, *k, *v;                               /* (B, q_heads*D), (B, kv_heads*D) x2 fp16 */
    void *attn_out, *down;                         /* (B, hidden) fp16 */
    void *gate, *up;                               /* (B, ffn) fp16 */
    void* logits; int32_t* next_ids;               /* (B, vocab) fp16, (B) */
    float* scores; int64_t sc_sl;                  /* per layer (B,Hq,P_max) fp32, layer stride in elements */
    int32_t* compact; int64_t cp_sl;               /* per layer (B,Hq,bucket) */
    void* O; int64_t o_sl;                         /* per layer (B,Hq,D) fp16 */
    void* attn_ws; size_t attn_ws_sl, attn_ws_bytes;   /* per layer split-K scratch of the attention, tickets zero */
} fq_llama_scratch;

/* x (B, hidden) fp16: the embedding rows of this step's tokens; seen[layer] tokens already cached
 * (all sequences of the batch are at the same position).  Writes scratch->logits and next_ids. */
int fq_llama_decode_step(const fq_llama_model* model, const fq_int4_cache* cache, const fq_decode_params* params,
                         const int* seen, const void* x, int B, const fq_llama_scratch* scratch, void* stream);
/* The same step with the positions in a DEVICE array (one int per layer, advanced by the last
 * launch): no launch depends on the sequence length, so the step can be captured in a CUDA graph
 * once and replayed per token (see fq_decode_step_int4_dev). */
int fq_llama_decode_step_dev(const fq_llama_model* model, const fq_int4_cache* cache, const fq_decode_params* params,
                             int* pos, const void* x, int B, const fq_llama_scratch* scratch, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHQUEST_B200_H */
