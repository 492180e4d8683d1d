// Static-kmax top-k page selection, sinks/window union, bool mask and compact index.
//
// One CTA per (batch, head) row of P fp32 scores.  The row is read from global memory ONCE
// (all loads in flight together) and kept in shared memory as order-preserving 32-bit keys;
// every later pass runs out of shared memory.  The k-th largest key is found with a 4-pass,
// 8-bit-digit radix select (one private 256-bin histogram per warp in shared memory, plain
// shared atomics, a warp whose 32 digits are all equal adds once); the selected set is
// { key > T } plus the
// lowest-indexed pages with key == T until k are taken.  Output positions come from warp
// ballots and a block-level scan, so the compact list is produced directly (descending page
// id, -1 padded) without a sort.  Latency-bound, not bandwidth-bound: P*4 bytes in,
// P + 4*bucket bytes out.  Rows too long for shared memory (P > 40960) re-read global memory.
#include "fq_common.cuh"

namespace fq {

constexpr int SEL_MAX_WARPS = 32;

// larger float -> larger key; -0 folds onto +0; NaN with a clear sign bit sorts above +inf.
__device__ __forceinline__ uint32_t score_key(float f) {
    uint32_t u = __float_as_uint(f);
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct SelShared {
    unsigned hist[256];
    unsigned warp_tot[SEL_MAX_WARPS];
    unsigned prefix;      // key bits fixed so far
    unsigned remaining;   // rank still to find inside the current prefix bucket
    unsigned misc[4];
};

// Exclusive scan of one value per warp (value valid on every lane of the warp).
// Returns this warp's exclusive prefix; *total receives the block total.  Uses sh.warp_tot.
__device__ __forceinline__ unsigned block_warp_scan(unsigned warp_val, SelShared& sh, unsigned* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) sh.warp_tot[warp] = warp_val;
    __syncthreads();
    unsigned v = lane < nwarps ? sh.warp_tot[lane] : 0u;
    unsigned incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        unsigned n = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += n;
    }
    *total = __shfl_sync(0xffffffffu, incl, 31);
    return __shfl_sync(0xffffffffu, incl - v, warp);
}

template <bool SMEM_KEYS>
__global__ void select_pages_kernel(
    const float* __restrict__ scores, int64_t sc_sb, int64_t sc_sh, int H, int P,
    const float* __restrict__ retention_per_head, float retention, int k_max, int sinks, int window,
    uint8_t* __restrict__ mask, int64_t mk_sb, int64_t mk_sh,
    int32_t* __restrict__ compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    int32_t* __restrict__ count) {
    __shared__ SelShared sh;
    extern __shared__ unsigned s_dyn[];
    unsigned* s_hist = s_dyn;                                   // [nwarps][256] private histograms
    unsigned* s_keys = s_dyn + (blockDim.x >> 5) * 256;         // [P] keys (SMEM_KEYS only)
    const int b = blockIdx.y, h = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const float* row = scores + b * sc_sb + h * sc_sh;
    if (SMEM_KEYS) {
#pragma unroll 4
        for (int i = tid; i < P; i += blockDim.x) s_keys[i] = score_key(__ldg(row + i));
        __syncthreads();
    }
    auto key_at = [&](int i) -> unsigned { return SMEM_KEYS ? s_keys[i] : score_key(row[i]); };

    // k_h = clamp(ceil(fp32(r) * fp32(P)), 0, P), then capped by the static k_max
    const float r = retention_per_head ? retention_per_head[h] : retention;
    float kf = ceilf(__fmul_rn(r, (float)P));
    int k = kf > 0.f ? (kf < (float)P ? (int)kf : P) : 0;
    k = min(k, min(k_max, P));
    const int ns = min(sinks, P), nw = min(window, P);

    // ---- radix select of the k-th largest key (only when 0 < k < P) ----
    unsigned T = 0u;           // threshold key
    unsigned need_eq = 0u;     // how many pages with key == T are kept
    if (k > 0 && k < P) {
        if (tid == 0) { sh.prefix = 0u; sh.remaining = (unsigned)k; }
        for (int shift = 24; shift >= 0; shift -= 8) {
            unsigned* my_hist = s_hist + warp * 256;
            for (int i = tid; i < nwarps * 256; i += blockDim.x) s_hist[i] = 0u;
            __syncthreads();
            const unsigned prefix = sh.prefix;
            const unsigned hi_mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            const int P_round = (P + 31) & ~31;   // whole warps stay converged for the vote
            for (int i = tid; i < P_round; i += blockDim.x) {
                const bool in = i < P;
                const unsigned key = in ? key_at(i) : 0u;
                const bool cand = in && ((key & hi_mask) == prefix);
                const unsigned digit = cand ? ((key >> shift) & 255u) : 256u;
                int same = 0;
                __match_all_sync(0xffffffffu, digit, &same);
                if (same) {
                    if (cand && lane == 0) atomicAdd(&my_hist[digit], 32u);
                } else if (cand) {
                    atomicAdd(&my_hist[digit], 1u);
                }
            }
            __syncthreads();
            for (int i = tid; i < 256; i += blockDim.x) {
                unsigned c = 0u;
                for (int w = 0; w < nwarps; ++w) c += s_hist[w * 256 + i];
                sh.hist[i] = c;
            }
            __syncthreads();
            if (warp == 0) {
                // scan bins from the top: find the bin where the cumulative count reaches `remaining`
                const unsigned rem = sh.remaining;
                unsigned c[8], s = 0u;
#pragma unroll
                for (int j = 0; j < 8; ++j) { c[j] = sh.hist[255 - (lane * 8 + j)]; s += c[j]; }
                unsigned incl = s;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    unsigned n = __shfl_up_sync(0xffffffffu, incl, off);
                    if (lane >= off) incl += n;
                }
                unsigned run = incl - s;   // pages in bins above this lane's bins
                if (run < rem && incl >= rem) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (run < rem && run + c[j] >= rem) {
                            sh.prefix = prefix | ((unsigned)(255 - (lane * 8 + j)) << shift);
                            sh.remaining = rem - run;
                        }
                        run += c[j];
                    }
                }
            }
            __syncthreads();
        }
        T = sh.prefix;
        need_eq = sh.remaining;   // 1 <= need_eq <= #(key == T)
    }
    const bool take_all = k >= P;
    const bool take_none = k <= 0;

    // ---- ordered passes: each warp owns a contiguous run of pages ----
    const int per_warp = (((P + nwarps - 1) / nwarps) + 31) & ~31;
    const int w_begin = warp * per_warp;
    const int w_end = min(P, w_begin + per_warp);

    // pass A: pages with key == T in this warp's run
    unsigned eq_before = 0u, eq_total = 0u;
    if (!take_all && !take_none) {
        unsigned cnt = 0u;
        for (int i0 = w_begin; i0 < w_end; i0 += 32) {
            const int i = i0 + lane;
            const bool eq = i < w_end && key_at(i) == T;
            cnt += __popc(__ballot_sync(0xffffffffu, eq));
        }
        eq_before = block_warp_scan(cnt, sh, &eq_total);
    }

    // pass B: selected pages in this warp's run
    auto selected = [&](int i, unsigned& eq_run, bool valid) -> bool {
        bool sel = false;
        bool eq = false;
        if (valid) {
            if (take_all) sel = true;
            else if (!take_none) {
                const unsigned key = key_at(i);
                sel = key > T;
                eq = key == T;
            }
        }
        const unsigned eq_ballot = __ballot_sync(0xffffffffu, eq);
        if (eq) {
            const unsigned rank = eq_run + __popc(eq_ballot & ((1u << lane) - 1u));
            sel = rank < need_eq;
        }
        eq_run += __popc(eq_ballot);
        if (valid && (i < ns || i >= P - nw)) sel = true;
        return sel;
    };

    unsigned sel_cnt = 0u;
    {
        unsigned eq_run = eq_before;
        for (int i0 = w_begin; i0 < w_end; i0 += 32) {
            const int i = i0 + lane;
            const bool s = selected(i, eq_run, i < w_end);
            sel_cnt += __popc(__ballot_sync(0xffffffffu, s));
        }
    }
    unsigned total = 0u;
    const unsigned sel_before = block_warp_scan(sel_cnt, sh, &total);

    // pass C: write mask and compact list (descending page id: position = total-1-ascending rank)
    {
        unsigned eq_run = eq_before, run = sel_before;
        uint8_t* mrow = mask ? mask + b * mk_sb + h * mk_sh : nullptr;
        int32_t* crow = compact ? compact + b * cp_sb + h * cp_sh : nullptr;
        for (int i0 = w_begin; i0 < w_end; i0 += 32) {
            const int i = i0 + lane;
            const bool valid = i < w_end;
            const bool s = selected(i, eq_run, valid);
            const unsigned ballot = __ballot_sync(0xffffffffu, s);
            if (valid && mrow) mrow[i] = s ? 1 : 0;
            if (s && crow) {
                const unsigned asc = run + __popc(ballot & ((1u << lane) - 1u));
                const unsigned pos = total - 1u - asc;
                if (pos < (unsigned)bucket) crow[pos] = i;
            }
            run += __popc(ballot);
        }
        if (crow) {
            for (int i = (int)total + tid; i < bucket; i += blockDim.x) crow[i] = -1;
        }
    }
    if (count && tid == 0) count[b * H + h] = (int32_t)total;
}

// mask (rows,P) u8 -> compact (rows,bucket) int32, descending ids, -1 padded.
__global__ void build_compact_kernel(const uint8_t* __restrict__ mask, int64_t mk_sr, int P,
                                     int32_t* __restrict__ compact, int64_t cp_sr, int bucket) {
    __shared__ SelShared sh;
    const int64_t r = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const uint8_t* mrow = mask + r * mk_sr;
    int32_t* crow = compact + r * cp_sr;
    const int per_warp = (((P + nwarps - 1) / nwarps) + 31) & ~31;
    const int w_begin = warp * per_warp;
    const int w_end = min(P, w_begin + per_warp);
    unsigned cnt = 0u;
    for (int i0 = w_begin; i0 < w_end; i0 += 32) {
        const int i = i0 + lane;
        cnt += __popc(__ballot_sync(0xffffffffu, i < w_end && mrow[i] != 0));
    }
    unsigned total = 0u;
    unsigned run = block_warp_scan(cnt, sh, &total);
    for (int i0 = w_begin; i0 < w_end; i0 += 32) {
        const int i = i0 + lane;
        const bool s = i < w_end && mrow[i] != 0;
        const unsigned ballot = __ballot_sync(0xffffffffu, s);
        if (s) {
            const unsigned pos = total - 1u - (run + __popc(ballot & ((1u << lane) - 1u)));
            if (pos < (unsigned)bucket) crow[pos] = i;
        }
        run += __popc(ballot);
    }
    for (int i = (int)total + tid; i < bucket; i += blockDim.x) crow[i] = -1;
}

static int select_threads(int P) { return P <= 512 ? 128 : (P <= 1024 ? 256 : (P <= 4096 ? 512 : 1024)); }
constexpr int SEL_SMEM_MAX_P = 40960;   // 160 KB of keys + 32 KB of histograms

}  // namespace fq

extern "C" int fq_select_pages(
    const float* scores, int64_t sc_sb, int64_t sc_sh, int B, int H, int P,
    const float* retention_per_head, float retention, int k_max, int sinks, int window,
    uint8_t* mask, int64_t mk_sb, int64_t mk_sh,
    int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    int32_t* count, void* stream) {
    using namespace fq;
    const char* fn = "fq_select_pages";
    FQ_CHECK_ARG(B > 0 && H > 0 && P >= 0, FQ_ERR_ARG, "%s: bad sizes B=%d H=%d P=%d", fn, B, H, P);
    FQ_CHECK_ARG(retention_per_head || (retention >= 0.f && retention <= 1.f), FQ_ERR_ARG,
                 "%s: scalar retention must be in [0, 1]; got %g", fn, (double)retention);
    FQ_CHECK_ARG(k_max >= 0 && sinks >= 0 && window >= 0, FQ_ERR_ARG, "%s: k_max/sinks/window must be >= 0", fn);
    FQ_CHECK_ARG(!compact || bucket >= 1, FQ_ERR_ARG, "%s: BUCKET_MAX must be >= 1, got %d", fn, bucket);
    FQ_CHECK_ARG(P == 0 || scores, FQ_ERR_ARG, "%s: null scores", fn);
    FQ_CHECK_ARG(B <= 65535, FQ_ERR_ARG, "%s: batch %d too large", fn, B);
    dim3 grid((unsigned)H, (unsigned)B);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (P <= SEL_SMEM_MAX_P) {
        const size_t smem = (size_t)P * 4 + (size_t)(select_threads(P) / 32) * 1024;
        if (smem > 40 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(select_pages_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: cannot reserve %zu B of shared memory: %s", fn, smem, cudaGetErrorString(e));
        }
        select_pages_kernel<true><<<grid, select_threads(P), smem, st>>>(
            scores, sc_sb, sc_sh, H, P, retention_per_head, retention, k_max, sinks, window,
            mask, mk_sb, mk_sh, compact, cp_sb, cp_sh, bucket, count);
    } else {
        select_pages_kernel<false><<<grid, select_threads(P), (select_threads(P) / 32) * 1024, st>>>(
            scores, sc_sb, sc_sh, H, P, retention_per_head, retention, k_max, sinks, window,
            mask, mk_sb, mk_sh, compact, cp_sb, cp_sh, bucket, count);
    }
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" int fq_build_compact(const uint8_t* mask, int64_t mk_sr, int64_t rows, int P,
                                int32_t* compact, int64_t cp_sr, int bucket, void* stream) {
    using namespace fq;
    const char* fn = "fq_build_compact";
    FQ_CHECK_ARG(bucket >= 1, FQ_ERR_ARG, "%s: BUCKET_MAX must be >= 1, got %d", fn, bucket);
    FQ_CHECK_ARG(rows >= 0 && P >= 0 && compact && (mask || P == 0 || rows == 0), FQ_ERR_ARG, "%s: bad arguments", fn);
    if (rows == 0) return FQ_OK;
    FQ_CHECK_ARG(rows <= 0x7fffffffLL, FQ_ERR_ARG, "%s: too many rows", fn);
    build_compact_kernel<<<(unsigned)rows, select_threads(P), 0, static_cast<cudaStream_t>(stream)>>>(
        mask, mk_sr, P, compact, cp_sr, bucket);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}
