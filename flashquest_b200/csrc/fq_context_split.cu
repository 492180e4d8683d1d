// One very long sequence split over several GPUs by page range: the device side of the two
// exchange steps.  (Not in the reference, which is single-GPU; the result is the single-GPU
// result: same page set, same softmax.)
//
// Rank r owns pages [lo, hi) of the sequence.  One decode step of one layer:
//   phase 1 (fq_ctx_local_candidates): local page scores, local top-min(k, P_local) pages, and a
//           message of (score, global page id) pairs for them;
//   all-gather of the messages (issued by the host between the phases, into this rank's memory);
//   phase 2 (fq_ctx_select_attend): the gathered candidates are packed in ascending global page id
//           (padding slots dropped, so that ties resolve exactly as on one GPU: lower page index
//           first), the same top-k kernel picks the global winners, the winners in [lo, hi) plus
//           this rank's share of the forced sink / window pages become the local compact list, and
//           the sparse attention kernel runs over it, writing (O, lse) straight into the message
//           buffer of the second exchange;
//   all-gather of (O_r, lse_r);
//   phase 3 (fq_ctx_merge): n-way LSE merge of the gathered partial results.
// Everything remote is in local memory before a kernel reads it: no peer loads, no multicast.
#include "fq_common.cuh"

namespace fq {

// msg (B,H,2,k_c): plane 0 = score of the j-th local candidate, plane 1 = its global page id
// (int bits); the candidates are the local top-k list as the selection kernel emits it
// (descending page id, -1 padded).
__global__ void ctx_emit_candidates_kernel(const float* __restrict__ scores, int64_t sc_row, const int32_t* __restrict__ compact,
                                           int k_c, int lo, float* __restrict__ msg, int64_t rows) {
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * k_c) return;
    const int64_t row = i / k_c;
    const int j = (int)(i - row * k_c);
    const int id = compact[row * k_c + j];
    msg[(row * 2 + 0) * k_c + j] = id >= 0 ? scores[row * sc_row + id] : -INFINITY;
    msg[(row * 2 + 1) * k_c + j] = __int_as_float(id >= 0 ? id + lo : -1);
}

// gathered (G,rows,2,k_c) -> cand_scores / cand_ids (rows, G*k_c): valid candidates in ascending global
// page id (rank-major, each rank's descending list walked backwards), then -inf / -1 padding.
__global__ void __launch_bounds__(256) ctx_pack_candidates_kernel(const float* __restrict__ gathered, int G, int64_t rows, int k_c,
                                                                  float* __restrict__ cand_scores, int32_t* __restrict__ cand_ids) {
    __shared__ unsigned s_warp[8];
    __shared__ unsigned s_base;
    const int64_t row = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = G * k_c;
    if (tid == 0) s_base = 0u;
    __syncthreads();
    for (int c0 = 0; c0 < n; c0 += 256) {
        const int m = c0 + tid;
        bool valid = false;
        float sc = 0.f;
        int id = -1;
        if (m < n) {
            const int r = m / k_c, j = k_c - 1 - (m - r * k_c);
            const float* src = gathered + (((int64_t)r * rows + row) * 2) * k_c;
            id = __float_as_int(src[k_c + j]);
            sc = src[j];
            valid = id >= 0;
        }
        const unsigned ballot = __ballot_sync(0xffffffffu, valid);
        if (lane == 0) s_warp[warp] = __popc(ballot);
        __syncthreads();
        unsigned before = s_base;
        for (int w = 0; w < warp; ++w) before += s_warp[w];
        if (valid) {
            const unsigned at = before + __popc(ballot & ((1u << lane) - 1u));
            cand_scores[row * n + at] = sc;
            cand_ids[row * n + at] = id;
        }
        __syncthreads();
        if (tid == 0) {
            unsigned tot = 0;
            for (int w = 0; w < 8; ++w) tot += s_warp[w];
            s_base += tot;
        }
        __syncthreads();
    }
    for (int m = s_base + tid; m < n; m += 256) {
        cand_scores[row * n + m] = -INFINITY;
        cand_ids[row * n + m] = -1;
    }
}

// win (rows, n) u8 over the packed candidates -> local mask (rows, P_local) u8: winners whose page lies in
// [lo, hi), plus the forced pages [0, sinks) and [P_global - window, P_global) that fall in the range.
__global__ void __launch_bounds__(256) ctx_scatter_winners_kernel(const uint8_t* __restrict__ win, const int32_t* __restrict__ cand_ids, int n,
                                                                  int lo, int hi, int P_global, int sinks, int window,
                                                                  uint8_t* __restrict__ mask) {
    const int64_t row = blockIdx.x;
    const int P_local = hi - lo;
    uint8_t* mrow = mask + row * P_local;
    for (int i = threadIdx.x; i < P_local; i += blockDim.x) {
        const int pg = lo + i;
        mrow[i] = (pg < min(sinks, P_global) || pg >= P_global - min(window, P_global)) ? 1 : 0;
    }
    __syncthreads();
    for (int m = threadIdx.x; m < n; m += blockDim.x) {
        const int id = cand_ids[row * n + m];
        if (win[row * n + m] && id >= lo && id < hi) mrow[id - lo] = 1;
    }
}

// n-way merge with strided parts: O_parts part i of row r at O_parts + i*o_part + r*D, lse at lse_parts + i*l_part + r.
template <typename T>
__global__ void __launch_bounds__(128) lse_merge_strided_kernel(const T* __restrict__ O_parts, int64_t o_part, const float* __restrict__ lse_parts,
                                                                int64_t l_part, int n, int64_t rows, int D, T* __restrict__ O, float* __restrict__ lse) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= rows) return;
    float m = -INFINITY;
    for (int i = 0; i < n; ++i) m = fmaxf(m, lse_parts[i * l_part + r]);
    if (m == -INFINITY) {
        for (int d = lane; d < D; d += 32) O[r * D + d] = from_f32<T>(0.f);
        if (lane == 0 && lse) lse[r] = -INFINITY;
        return;
    }
    float wsum = 0.f;
    for (int i = 0; i < n; ++i) wsum += expf(lse_parts[i * l_part + r] - m);
    for (int d = lane; d < D; d += 32) {
        float a = 0.f;
        for (int i = 0; i < n; ++i) a = fmaf(expf(lse_parts[i * l_part + r] - m), Dt<T>::to_f32(O_parts[i * o_part + r * D + d]), a);
        O[r * D + d] = from_f32<T>(a / wsum);
    }
    if (lane == 0 && lse) lse[r] = m + logf(wsum);
}

}  // namespace fq

extern "C" size_t fq_ctx_scratch_bytes(int B, int Hq, int G, int k_c, int P_local, int bucket_local) {
    if (B <= 0 || Hq <= 0 || G <= 0 || k_c < 0 || P_local < 0 || bucket_local < 0) return 0;
    const size_t rows = (size_t)B * Hq, n = (size_t)G * k_c;
    auto pad = [](size_t x) { return (x + 255) & ~(size_t)255; };
    // local scores | local candidate list | packed candidate scores | packed ids | winner mask | local mask | local compact list
    return pad(rows * (size_t)(P_local > 0 ? P_local : 1) * 4) + pad(rows * (size_t)k_c * 4) + pad(rows * n * 4) + pad(rows * n * 4) +
           pad(rows * n) + pad(rows * (size_t)(P_local > 0 ? P_local : 1)) + pad(rows * (size_t)(bucket_local > 0 ? bucket_local : 1) * 4);
}

namespace {
struct CtxScratch {
    float* scores; int32_t* cand_local; float* cand_scores; int32_t* cand_ids; uint8_t* win; uint8_t* mask; int32_t* compact;
};
CtxScratch ctx_carve(void* scratch, int B, int Hq, int G, int k_c, int P_local, int bucket_local) {
    const size_t rows = (size_t)B * Hq, n = (size_t)G * k_c;
    auto pad = [](size_t x) { return (x + 255) & ~(size_t)255; };
    char* p = static_cast<char*>(scratch);
    CtxScratch s;
    s.scores = reinterpret_cast<float*>(p); p += pad(rows * (size_t)(P_local > 0 ? P_local : 1) * 4);
    s.cand_local = reinterpret_cast<int32_t*>(p); p += pad(rows * (size_t)k_c * 4);
    s.cand_scores = reinterpret_cast<float*>(p); p += pad(rows * n * 4);
    s.cand_ids = reinterpret_cast<int32_t*>(p); p += pad(rows * n * 4);
    s.win = reinterpret_cast<uint8_t*>(p); p += pad(rows * n);
    s.mask = reinterpret_cast<uint8_t*>(p); p += pad(rows * (size_t)(P_local > 0 ? P_local : 1));
    s.compact = reinterpret_cast<int32_t*>(p);
    return s;
}
}  // namespace

extern "C" int fq_ctx_local_candidates(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P_local, int D, int lo, int k_c, int G, int bucket_local,
    void* scratch, size_t scratch_bytes, float* msg, void* stream) {
    using namespace fq;
    const char* fn = "fq_ctx_local_candidates";
    FQ_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && P_local >= 0 && k_c >= 1 && G >= 1 && lo >= 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(scratch && msg && scratch_bytes >= fq_ctx_scratch_bytes(B, Hq, G, k_c, P_local, bucket_local), FQ_ERR_WORKSPACE,
                 "%s: scratch of %zu B needed, %zu given", fn, fq_ctx_scratch_bytes(B, Hq, G, k_c, P_local, bucket_local), scratch_bytes);
    const CtxScratch s = ctx_carve(scratch, B, Hq, G, k_c, P_local, bucket_local);
    const int64_t rows = (int64_t)B * Hq;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc;
    if (P_local > 0) {
        rc = fq_page_scores_int4(Q, q_dtype, q_sb, q_sh, K_scale, K_mn, km_sb, km_sh, km_sp, B, Hq, Hkv, P_local, D, s.scores, (int64_t)Hq * P_local, P_local, stream);
        if (rc != FQ_OK) return rc;
        // the local top-min(k_c, P_local) pages, ties to the lower page index as on one GPU
        rc = fq_select_pages(s.scores, (int64_t)Hq * P_local, P_local, B, Hq, P_local, nullptr, 1.0f, k_c < P_local ? k_c : P_local, 0, 0,
                             nullptr, 0, 0, s.cand_local, (int64_t)Hq * k_c, k_c, k_c, nullptr, stream);
        if (rc != FQ_OK) return rc;
    } else {
        cudaError_t e = cudaMemsetAsync(s.cand_local, 0xff, (size_t)rows * k_c * 4, st);     // all -1: nothing to offer
        if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: %s", fn, cudaGetErrorString(e));
    }
    const int64_t total = rows * k_c;
    launch_k(PDL_GEMV, ctx_emit_candidates_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st,
             static_cast<const float*>(s.scores), (int64_t)P_local, static_cast<const int32_t*>(s.cand_local), k_c, lo, msg, rows);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" int fq_ctx_select_attend(
    const float* gathered, int G, int k_c, int k_global, int sinks, int window, int lo, int hi, int P_global,
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_packed, int64_t kp_sb, int64_t kp_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const uint8_t* V_packed, int64_t vp_sb, int64_t vp_sh,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss, int tail_len,
    int B, int Hq, int Hkv, int D, int page, float sm_scale, int bucket_local,
    void* scratch, size_t scratch_bytes, void* O_msg, float* lse_msg,
    void* workspace, size_t workspace_bytes, int n_split, void* stream) {
    using namespace fq;
    const char* fn = "fq_ctx_select_attend";
    const int P_local = hi - lo;
    FQ_CHECK_ARG(gathered && G >= 1 && k_c >= 1 && k_global >= 0 && P_local >= 0 && lo >= 0 && hi <= P_global, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(scratch && scratch_bytes >= fq_ctx_scratch_bytes(B, Hq, G, k_c, P_local, bucket_local), FQ_ERR_WORKSPACE,
                 "%s: scratch of %zu B needed, %zu given", fn, fq_ctx_scratch_bytes(B, Hq, G, k_c, P_local, bucket_local), scratch_bytes);
    const CtxScratch s = ctx_carve(scratch, B, Hq, G, k_c, P_local, bucket_local);
    const int64_t rows = (int64_t)B * Hq;
    const int n = G * k_c;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    FQ_CHECK_ARG(rows <= 0x7fffffff, FQ_ERR_ARG, "%s: too many rows", fn);
    ctx_pack_candidates_kernel<<<(unsigned)rows, 256, 0, st>>>(gathered, G, rows, k_c, s.cand_scores, s.cand_ids);
    FQ_CHECK_LAUNCH(fn);
    // global top-k over the candidates (every page that can be among the global top k is among them)
    int rc = fq_select_pages(s.cand_scores, (int64_t)Hq * n, n, B, Hq, n, nullptr, 1.0f, k_global < n ? k_global : n, 0, 0,
                             s.win, (int64_t)Hq * n, n, nullptr, 0, 0, 0, nullptr, stream);
    if (rc != FQ_OK) return rc;
    if (P_local > 0) {
        ctx_scatter_winners_kernel<<<(unsigned)rows, 256, 0, st>>>(s.win, s.cand_ids, n, lo, hi, P_global, sinks, window, s.mask);
        FQ_CHECK_LAUNCH(fn);
        rc = fq_build_compact(s.mask, P_local, rows, P_local, s.compact, bucket_local, bucket_local, stream);
        if (rc != FQ_OK) return rc;
    }
    return fq_sparse_decode_int4(Q, q_dtype, q_sb, q_sh, K_packed, kp_sb, kp_sh, K_scale, K_mn, km_sb, km_sh, km_sp,
                                 V_packed, vp_sb, vp_sh, V_scale, V_mn, vm_sb, vm_sh,
                                 s.compact, (int64_t)Hq * bucket_local, bucket_local, P_local > 0 ? bucket_local : 0,
                                 K_tail, V_tail, tail_dtype, tl_sb, tl_sh, tl_ss, tail_len,
                                 B, Hq, Hkv, P_local * page, P_local, D, page, sm_scale,
                                 O_msg, (int64_t)Hq * D, D, lse_msg, workspace, workspace_bytes, n_split, stream);
}

extern "C" int fq_lse_merge_strided(const void* O_parts, int64_t o_part_stride, const float* lse_parts, int64_t lse_part_stride,
                                    int dtype, int n, int64_t rows, int D, void* O, float* lse, void* stream) {
    using namespace fq;
    const char* fn = "fq_lse_merge_strided";
    FQ_CHECK_ARG(n >= 1 && rows >= 0 && D >= 1, FQ_ERR_ARG, "%s: bad sizes", fn);
    if (rows == 0) return FQ_OK;
    FQ_CHECK_ARG(O_parts && lse_parts && O, FQ_ERR_ARG, "%s: null pointer", fn);
    const unsigned blocks = (unsigned)((rows + 3) / 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == FQ_F32) launch_k(PDL_GEMV, lse_merge_strided_kernel<float>, dim3(blocks), dim3(128), 0, st, static_cast<const float*>(O_parts), o_part_stride, lse_parts, lse_part_stride, n, rows, D, static_cast<float*>(O), lse);
    else if (dtype == FQ_F16) launch_k(PDL_GEMV, lse_merge_strided_kernel<__half>, dim3(blocks), dim3(128), 0, st, static_cast<const __half*>(O_parts), o_part_stride, lse_parts, lse_part_stride, n, rows, D, static_cast<__half*>(O), lse);
    else if (dtype == FQ_BF16) launch_k(PDL_GEMV, lse_merge_strided_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, st, static_cast<const __nv_bfloat16*>(O_parts), o_part_stride, lse_parts, lse_part_stride, n, rows, D, static_cast<__nv_bfloat16*>(O), lse);
    else return fail(FQ_ERR_DTYPE, "%s: dtype code %d", fn, dtype);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}
