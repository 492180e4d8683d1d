// The arithmetic of one page score, shared by the scoring kernel and the fused score + select
// kernel so that both produce the same bits:
//   score[hq, p] = sum_d q[d]*K_mn[p,d] + levels * sum_d relu(q[d])*K_scale[p,d]
// Eight lanes (a quarter warp) own one page; lane l holds the 8-channel chunks l, l+8, ... of
// the metadata rows and of q for NR query heads.  Summation order: chunk by chunk, channel by
// channel inside the lane (fma), then a 3-step xor shuffle over the quarter warp.
#pragma once
#include "fq_common.cuh"

namespace fq {

// q slices of this lane for NR heads of the group that starts at head hq0 (nr heads present)
template <typename QT, int NR, int CH>
__device__ __forceinline__ void score_load_q(const QT* __restrict__ Qb, int64_t q_sh, int hq0, int nr, int l, int n_chunks,
                                             float (&q)[NR][CH][8]) {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int hq = hq0 + min(r, nr - 1);
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int chunk = l + 8 * c;
            if (chunk < n_chunks) {
                load8<QT>(Qb + hq * q_sh + 8 * chunk, q[r][c]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) q[r][c][e] = 0.f;
            }
        }
    }
}

// metadata chunks of page p for this lane (zeros past the row or the head dimension)
template <int CH>
__device__ __forceinline__ void score_load_meta(const uint16_t* __restrict__ sc_base, const uint16_t* __restrict__ mn_base,
                                                int64_t km_sp, int p, bool live, int l, int n_chunks, uint4 (&m4)[CH], uint4 (&s4)[CH]) {
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int chunk = l + 8 * c;
        if (live && chunk < n_chunks) {
            m4[c] = ldg16(mn_base + (int64_t)p * km_sp + 8 * chunk);
            s4[c] = ldg16(sc_base + (int64_t)p * km_sp + 8 * chunk);
        } else {
            m4[c] = make_uint4(0, 0, 0, 0);
            s4[c] = make_uint4(0, 0, 0, 0);
        }
    }
}

// the score of head (lane & 7) of the group, valid on lanes l < NR; all 32 lanes must call
template <int NR, int CH>
__device__ __forceinline__ float score_page(const float (&q)[NR][CH][8], const uint4 (&m4)[CH], const uint4 (&s4)[CH], int l, float levels) {
    float t1[NR], t2[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) { t1[r] = 0.f; t2[r] = 0.f; }
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const uint32_t mw[4] = {m4[c].x, m4[c].y, m4[c].z, m4[c].w};
        const uint32_t sw[4] = {s4[c].x, s4[c].y, s4[c].z, s4[c].w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float mn = (e & 1) ? bf16_hi(mw[e >> 1]) : bf16_lo(mw[e >> 1]);
            const float sc = (e & 1) ? bf16_hi(sw[e >> 1]) : bf16_lo(sw[e >> 1]);
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const float qv = q[r][c][e];
                t1[r] = __fmaf_rn(qv, mn, t1[r]);
                t2[r] = __fmaf_rn(fmaxf(qv, 0.f), sc, t2[r]);
            }
        }
    }
#pragma unroll
    for (int off = 4; off >= 1; off >>= 1) {
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            t1[r] = __fadd_rn(t1[r], __shfl_xor_sync(0xffffffffu, t1[r], off));
            t2[r] = __fadd_rn(t2[r], __shfl_xor_sync(0xffffffffu, t2[r], off));
        }
    }
    float v1 = t1[0], v2 = t2[0];
#pragma unroll
    for (int r = 1; r < NR; ++r) {
        if (l == r) { v1 = t1[r]; v2 = t2[r]; }
    }
    return __fadd_rn(v1, __fmul_rn(v2, levels));
}

// larger float -> larger key; -0 folds onto +0; every NaN (either sign) takes the largest key,
// which is how torch.topk orders NaNs.
__device__ __forceinline__ uint32_t score_key(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

}  // namespace fq
