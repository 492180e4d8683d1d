// Page scores read straight from the INT4 K metadata.
//
// score[b,hq,p] = sum_d q[d]*K_mn[p,d] + 15 * sum_d relu(q[d])*K_scale[p,d]
//
// HBM-bound: the only real traffic is the metadata, 2*D*2 bytes per (kv head, page), read
// exactly once and shared by all query heads of the GQA group.  Eight lanes (a quarter
// warp) own one page: each lane issues 16-byte loads of 8 channels, the eight lanes of a
// page read 128 contiguous bytes per instruction and the four quarter-warps read four
// consecutive pages, so every warp load is one contiguous 512-byte run.  Each lane keeps
// its slice of q for all NR query heads in registers; the per-page reduction is a 3-step
// xor shuffle inside the quarter warp.
#include "fq_score_lane.cuh"

namespace fq {

constexpr int SCORE_THREADS = 128;            // 16 pages per CTA iteration
constexpr int SCORE_PAGES_PER_CTA = 32;       // 2 iterations per CTA

// NR = query heads handled per pass (<= 4), CH = 8-channel chunks per lane (D = 64*CH, or
// D = 32 with CH = 1 where lanes 4..7 hold no chunk).
template <typename QT, int NR, int CH>
__global__ void __launch_bounds__(SCORE_THREADS) page_scores_kernel(
    const QT* __restrict__ Q, int64_t q_sb, int64_t q_sh,
    const uint16_t* __restrict__ K_scale, const uint16_t* __restrict__ K_mn,
    int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int Hq, int Hkv, int P, int D, int head_off,
    float* __restrict__ scores, int64_t sc_sb, int64_t sc_sh, const int* __restrict__ pos, int pos_new, int pos_page, int pos_early, float levels) {
    const int b = blockIdx.z, hkv = blockIdx.y;
    const int n_rep = Hq / Hkv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane & 7, qw = lane >> 3;
    const int n_chunks = D >> 3;
    const int nr = min(NR, n_rep - head_off);   // heads actually present in this pass
    int pos_v = 0;
    if (pos && pos_early) pos_v = __ldcg(pos);             // in flight during the wait (see DynPos::early)
    pdl_wait();        // Q and the newest metadata row come from the kernels before this one
    pdl_trigger();
    if (pos) {
        if (!pos_early) pos_v = *pos;
        P = min(P, (pos_v + pos_new) / pos_page);          // completed pages after this step's append
    }

    // Metadata loads of every page this quarter warp will score are issued first, the q loads
    // after them, so the two global-memory latencies overlap instead of adding up.
    constexpr int ITERS = SCORE_PAGES_PER_CTA / 16;
    const int p_base = blockIdx.x * SCORE_PAGES_PER_CTA;
    const uint16_t* sc_base = K_scale + b * km_sb + hkv * km_sh;
    const uint16_t* mn_base = K_mn + b * km_sb + hkv * km_sh;
    uint4 m4[ITERS][CH], s4[ITERS][CH];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int p = p_base + it * 16 + warp * 4 + qw;
        score_load_meta<CH>(sc_base, mn_base, km_sp, p, p < P, l, n_chunks, m4[it], s4[it]);
    }
    float q[NR][CH][8];
    score_load_q<QT, NR, CH>(Q + b * q_sb, q_sh, hkv * n_rep + head_off, nr, l, n_chunks, q);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int p = p_base + it * 16 + warp * 4 + qw;
        const float v = score_page<NR, CH>(q, m4[it], s4[it], l, levels);
        if (p < P && l < nr) scores[b * sc_sb + (hkv * n_rep + head_off + l) * sc_sh + p] = v;
    }
}

// page_scores_kernel for the decode step, where the position may be read before the dependency wait
// (DynPos::early): the rows of the pages completed before this step -- nothing in flight writes them -- are
// requested before the wait as well, so the CTA spends the end of the previous kernel fetching instead of waiting.
template <typename QT, int NR, int CH>
__global__ void __launch_bounds__(SCORE_THREADS) page_scores_early_kernel(
    const QT* __restrict__ Q, int64_t q_sb, int64_t q_sh,
    const uint16_t* __restrict__ K_scale, const uint16_t* __restrict__ K_mn,
    int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int Hq, int Hkv, int P, int D, int head_off,
    float* __restrict__ scores, int64_t sc_sb, int64_t sc_sh, const int* __restrict__ pos, int pos_new, int pos_page, float levels) {
    const int b = blockIdx.z, hkv = blockIdx.y;
    const int n_rep = Hq / Hkv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane & 7, qw = lane >> 3;
    const int n_chunks = D >> 3;
    const int nr = min(NR, n_rep - head_off);   // heads actually present in this pass
    constexpr int ITERS = SCORE_PAGES_PER_CTA / 16;
    const int p_base = blockIdx.x * SCORE_PAGES_PER_CTA;
    const uint16_t* sc_base = K_scale + b * km_sb + hkv * km_sh;
    const uint16_t* mn_base = K_mn + b * km_sb + hkv * km_sh;
    uint4 m4[ITERS][CH], s4[ITERS][CH];
    const int pos_v = __ldcg(pos);
    const int P_old = min(P, pos_v / pos_page);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int p = p_base + it * 16 + warp * 4 + qw;
        if (p < P_old) score_load_meta<CH>(sc_base, mn_base, km_sp, p, true, l, n_chunks, m4[it], s4[it]);
    }
    pdl_wait();        // Q and the newest metadata row come from the kernels before this one
    pdl_trigger();
    P = min(P, (pos_v + pos_new) / pos_page);              // completed pages after this step's append
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int p = p_base + it * 16 + warp * 4 + qw;
        if (p >= P_old) score_load_meta<CH>(sc_base, mn_base, km_sp, p, p < P, l, n_chunks, m4[it], s4[it]);
    }
    float q[NR][CH][8];
    score_load_q<QT, NR, CH>(Q + b * q_sb, q_sh, hkv * n_rep + head_off, nr, l, n_chunks, q);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int p = p_base + it * 16 + warp * 4 + qw;
        const float v = score_page<NR, CH>(q, m4[it], s4[it], l, levels);
        if (p < P && l < nr) scores[b * sc_sb + (hkv * n_rep + head_off + l) * sc_sh + p] = v;
    }
}

template <typename QT, int NR>
static void launch_scores(int CH, dim3 grid, cudaStream_t st, const void* Q, int64_t q_sb, int64_t q_sh,
                          const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
                          int Hq, int Hkv, int P, int D, int head_off, float* scores, int64_t sc_sb, int64_t sc_sh, const DynPos& dp, float levels) {
#define FQ_LAUNCH_SC(CHV)                                                                              \
    do {                                                                                               \
        if (dp.pos != nullptr && dp.early)                                                             \
            launch_k(PDL_SCORES, page_scores_early_kernel<QT, NR, CHV>, grid, dim3(SCORE_THREADS), 0, st,              \
                     static_cast<const QT*>(Q), q_sb, q_sh, static_cast<const uint16_t*>(K_scale),     \
                     static_cast<const uint16_t*>(K_mn), km_sb, km_sh, km_sp, Hq, Hkv, P, D, head_off, scores, sc_sb, sc_sh, \
                     dp.pos, dp.n_new, dp.page, levels);                                               \
        else                                                                                           \
            launch_k(PDL_SCORES, page_scores_kernel<QT, NR, CHV>, grid, dim3(SCORE_THREADS), 0, st,    \
                     static_cast<const QT*>(Q), q_sb, q_sh, static_cast<const uint16_t*>(K_scale),     \
                     static_cast<const uint16_t*>(K_mn), km_sb, km_sh, km_sp, Hq, Hkv, P, D, head_off, scores, sc_sb, sc_sh, \
                     dp.pos, dp.n_new, dp.page, 0, levels);                                            \
    } while (0)
    if (CH == 1) FQ_LAUNCH_SC(1);
    else if (CH == 2) FQ_LAUNCH_SC(2);
    else FQ_LAUNCH_SC(4);
#undef FQ_LAUNCH_SC
}

template <typename QT>
static void launch_scores_nr(int nr, int CH, dim3 grid, cudaStream_t st, const void* Q, int64_t q_sb, int64_t q_sh,
                             const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
                             int Hq, int Hkv, int P, int D, int head_off, float* scores, int64_t sc_sb, int64_t sc_sh, const DynPos& dp, float levels) {
#define FQ_ARGS CH, grid, st, Q, q_sb, q_sh, K_scale, K_mn, km_sb, km_sh, km_sp, Hq, Hkv, P, D, head_off, scores, sc_sb, sc_sh, dp, levels
    if (nr == 1) launch_scores<QT, 1>(FQ_ARGS);
    else if (nr == 2) launch_scores<QT, 2>(FQ_ARGS);
    else if (nr == 3) launch_scores<QT, 3>(FQ_ARGS);
    else launch_scores<QT, 4>(FQ_ARGS);
#undef FQ_ARGS
}

int page_scores_int4_launch(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P, int D,
    float* scores, int64_t sc_sb, int64_t sc_sh, void* stream, const DynPos& dp, float levels) {
    const char* fn = levels == 255.0f ? "fq_page_scores_int8" : "fq_page_scores_int4";
    FQ_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && P >= 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(Hq % Hkv == 0, FQ_ERR_ARG, "%s: H_q=%d must be divisible by H_kv=%d", fn, Hq, Hkv);
    FQ_CHECK_ARG(D == 32 || D == 64 || D == 128 || D == 256, FQ_ERR_UNSUPPORTED, "%s: head_dim %d not in {32,64,128,256}", fn, D);
    FQ_CHECK_ARG(q_dtype == FQ_F32 || q_dtype == FQ_F16 || q_dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: dtype code %d", fn, q_dtype);
    if (P == 0) return FQ_OK;
    FQ_CHECK_ARG(Q && K_scale && K_mn && scores, FQ_ERR_ARG, "%s: null pointer", fn);
    const int64_t qa = q_dtype == FQ_F32 ? 4 : 8;
    FQ_CHECK_ARG(q_sb % qa == 0 && q_sh % qa == 0 && aligned(Q, 16), FQ_ERR_ALIGN, "%s: Q rows must be 16-byte aligned", fn);
    FQ_CHECK_ARG(km_sb % 8 == 0 && km_sh % 8 == 0 && km_sp % 8 == 0 && aligned(K_scale, 16) && aligned(K_mn, 16),
                 FQ_ERR_ALIGN, "%s: K metadata rows must be 16-byte aligned", fn);
    const int n_rep = Hq / Hkv;
    const int CH = D <= 64 ? 1 : D / 64;
    dim3 grid((unsigned)((P + SCORE_PAGES_PER_CTA - 1) / SCORE_PAGES_PER_CTA), (unsigned)Hkv, (unsigned)B);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // query heads of a group are served four at a time (one pass over the metadata per four)
    for (int off = 0; off < n_rep; off += 4) {
        const int nr = n_rep - off < 4 ? n_rep - off : 4;
#define FQ_ARGS nr, CH, grid, st, Q, q_sb, q_sh, K_scale, K_mn, km_sb, km_sh, km_sp, Hq, Hkv, P, D, off, scores, sc_sb, sc_sh, dp, levels
        if (q_dtype == FQ_F32) launch_scores_nr<float>(FQ_ARGS);
        else if (q_dtype == FQ_F16) launch_scores_nr<__half>(FQ_ARGS);
        else launch_scores_nr<__nv_bfloat16>(FQ_ARGS);
#undef FQ_ARGS
        FQ_CHECK_LAUNCH(fn);
    }
    return FQ_OK;
}

}  // namespace fq

extern "C" int fq_page_scores_int4(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P, int D,
    float* scores, int64_t sc_sb, int64_t sc_sh, void* stream) {
    return fq::page_scores_int4_launch(Q, q_dtype, q_sb, q_sh, K_scale, K_mn, km_sb, km_sh, km_sp, B, Hq, Hkv, P, D,
                                       scores, sc_sb, sc_sh, stream, fq::DynPos{}, 15.0f);
}

extern "C" int fq_page_scores_int8(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P, int D,
    float* scores, int64_t sc_sb, int64_t sc_sh, void* stream) {
    return fq::page_scores_int4_launch(Q, q_dtype, q_sb, q_sh, K_scale, K_mn, km_sb, km_sh, km_sp, B, Hq, Hkv, P, D,
                                       scores, sc_sb, sc_sh, stream, fq::DynPos{}, 255.0f);
}
