// Static-kmax top-k page selection, sinks/window union, bool mask and compact index.
//
// One CTA per (batch, head) row of P fp32 scores.  The row is read from global memory ONCE
// (all loads in flight together) and kept in shared memory as order-preserving 32-bit keys;
// every later pass runs out of shared memory.  The k-th largest key T is found by
// distribution select: the keys still in play span [lo, hi]; they are counted into 2048
// equal-width bins of that span (plain shared-memory atomics), a block scan from the top
// finds the bin holding rank k, and the span shrinks to that bin.  Two rounds usually leave a
// handful of candidates, which are ranked directly; a span of width 1 ends the search too, so
// at most three rounds are needed for any input (ties, infinities, NaNs included).
// The selected set is { key > T } plus the lowest-indexed pages with key == T until k are
// taken.  Output positions come from warp ballots and a block-level scan, so the compact
// list is produced directly (descending page id, -1 padded) without a sort.
// Latency-bound, not bandwidth-bound: P*4 bytes in, P + 4*bucket bytes out.  Rows too long
// for shared memory (P > 49152) re-read global memory in every pass.
#include "fq_common.cuh"

namespace fq {

constexpr int SEL_MAX_WARPS = 32;
constexpr int SEL_BINS = 2048;
constexpr int SEL_CAND_MAX = 128;

// larger float -> larger key; -0 folds onto +0; every NaN (either sign) takes the largest key,
// which is how torch.topk orders NaNs.
__device__ __forceinline__ uint32_t score_key(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct SelShared {
    unsigned hist[SEL_BINS];
    unsigned cand[SEL_CAND_MAX];
    unsigned warp_tot[SEL_MAX_WARPS];
    unsigned warp_min[SEL_MAX_WARPS];
    unsigned warp_max[SEL_MAX_WARPS];
    unsigned sel_bin, above, cnt;     // result of one histogram round
    unsigned ncand;
    unsigned T, need_eq, eq_total;    // result of the search
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
    int32_t* __restrict__ count, const int* __restrict__ pos, int pos_new, int pos_page) {
    __shared__ SelShared sh;
    extern __shared__ unsigned s_keys[];                        // [P] keys (SMEM_KEYS only)
    const int b = blockIdx.y, h = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int T_ = blockDim.x;
    const float* row = scores + b * sc_sb + h * sc_sh;
    auto key_at = [&](int i) -> unsigned { return SMEM_KEYS ? s_keys[i] : score_key(row[i]); };
    pdl_wait();        // the scores come from the previous kernel
    pdl_trigger();
    if (pos) {         // row length read on the device: completed pages after this step's append
        P = min(P, (*pos + pos_new) / pos_page);
        k_max = min(k_max, P);
    }

    // ---- load the row once; block min / max of the keys ----
    unsigned kmin = 0xffffffffu, kmax = 0u;
#pragma unroll 4
    for (int i = tid; i < P; i += T_) {
        const unsigned key = score_key(__ldg(row + i));
        if (SMEM_KEYS) s_keys[i] = key;
        kmin = min(kmin, key);
        kmax = max(kmax, key);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, off));
        kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, off));
    }
    if (lane == 0) { sh.warp_min[warp] = kmin; sh.warp_max[warp] = kmax; }
    __syncthreads();
    unsigned lo = sh.warp_min[0], hi = sh.warp_max[0];
    for (int w = 1; w < nwarps; ++w) { lo = min(lo, sh.warp_min[w]); hi = max(hi, sh.warp_max[w]); }

    // k_h = clamp(ceil(fp32(r) * fp32(P)), 0, P), then capped by the static k_max
    const float r = retention_per_head ? retention_per_head[h] : retention;
    float kf = ceilf(__fmul_rn(r, (float)P));
    int k = kf > 0.f ? (kf < (float)P ? (int)kf : P) : 0;
    k = min(k, min(k_max, P));
    const int ns = min(sinks, P), nw = min(window, P);

    // ---- distribution select of the k-th largest key (only when 0 < k < P) ----
    unsigned T = 0u;           // threshold key
    unsigned need_eq = 0u;     // how many pages with key == T are kept
    unsigned eq_total = 0u;    // how many pages have key == T
    if (k > 0 && k < P) {
        unsigned remaining = (unsigned)k;   // rank (1 = largest) still to find inside [lo, hi]
        unsigned in_range = (unsigned)P;    // number of keys inside [lo, hi]
        const int bpt = SEL_BINS / T_;      // bins per thread in the scan (T_ is 128..1024)
        for (int round = 0; round < 4; ++round) {
            const unsigned width = hi - lo;
            if (width == 0u) { T = lo; need_eq = remaining; eq_total = in_range; break; }
            if (in_range <= (unsigned)SEL_CAND_MAX) {
                // ---- few candidates left: rank them directly ----
                if (tid == 0) sh.ncand = 0u;
                __syncthreads();
                for (int i = tid; i < P; i += T_) {
                    const unsigned key = key_at(i);
                    if (key >= lo && key <= hi) sh.cand[atomicAdd(&sh.ncand, 1u)] = key;
                }
                __syncthreads();
                const unsigned c = sh.ncand;
                for (unsigned i = tid; i < c; i += T_) {
                    const unsigned v = sh.cand[i];
                    unsigned g = 0u, ge = 0u;
                    for (unsigned j = 0; j < c; ++j) {
                        const unsigned o = sh.cand[j];
                        g += o > v;
                        ge += o >= v;
                    }
                    if (g < remaining && remaining <= ge) { sh.T = v; sh.need_eq = remaining - g; sh.eq_total = ge - g; }
                }
                __syncthreads();
                T = sh.T; need_eq = sh.need_eq; eq_total = sh.eq_total;
                break;
            }
            const int nb = 32 - __clz(width);
            const int shift = nb > 11 ? nb - 11 : 0;           // (width >> shift) <= 2047
            for (int i = tid; i < SEL_BINS; i += T_) sh.hist[i] = 0u;
            __syncthreads();
            for (int i = tid; i < P; i += T_) {
                const unsigned key = key_at(i);
                if (key >= lo && key <= hi) atomicAdd(&sh.hist[(key - lo) >> shift], 1u);
            }
            __syncthreads();
            // scan from the top bin down: thread t owns bins 2047 - (t*bpt + j)
            unsigned own = 0u;
            for (int j = 0; j < bpt; ++j) own += sh.hist[SEL_BINS - 1 - (tid * bpt + j)];
            unsigned incl = own;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                unsigned n = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += n;
            }
            unsigned tot_unused;
            const unsigned wprefix = block_warp_scan(__shfl_sync(0xffffffffu, incl, 31), sh, &tot_unused);
            unsigned run = wprefix + incl - own;               // keys in bins above this thread's bins
            if (run < remaining && remaining <= run + own) {
                for (int j = 0; j < bpt; ++j) {
                    const int bin = SEL_BINS - 1 - (tid * bpt + j);
                    const unsigned c = sh.hist[bin];
                    if (run < remaining && remaining <= run + c) { sh.sel_bin = (unsigned)bin; sh.above = run; sh.cnt = c; }
                    run += c;
                }
            }
            __syncthreads();
            const unsigned bin = sh.sel_bin;
            remaining -= sh.above;
            in_range = sh.cnt;
            const unsigned new_lo = lo + (bin << shift);
            const unsigned new_hi = (bin == (width >> shift)) ? hi : new_lo + ((1u << shift) - 1u);
            lo = new_lo;
            hi = new_hi;
            if (shift == 0) { T = lo; need_eq = remaining; eq_total = in_range; break; }
        }
    }
    const bool take_all = k >= P;
    const bool take_none = k <= 0;

    // ---- ordered passes: each warp owns a contiguous run of pages ----
    const int per_warp = (((P + nwarps - 1) / nwarps) + 31) & ~31;
    const int w_begin = warp * per_warp;
    const int w_end = min(P, w_begin + per_warp);

    // pass A: pages with key == T in this warp's run
    // (skipped when every page with key == T is kept: then "selected" is simply key >= T)
    unsigned eq_before = 0u;
    const bool rank_ties = !take_all && !take_none && need_eq < eq_total;
    if (rank_ties) {
        unsigned cnt = 0u;
        for (int i0 = w_begin; i0 < w_end; i0 += 32) {
            const int i = i0 + lane;
            const bool eq = i < w_end && key_at(i) == T;
            cnt += __popc(__ballot_sync(0xffffffffu, eq));
        }
        unsigned eq_tot_unused;
        eq_before = block_warp_scan(cnt, sh, &eq_tot_unused);
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
            sel = rank_ties ? (rank < need_eq) : true;
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
constexpr int SEL_SMEM_MAX_P = 49152;   // 192 KB of keys

int select_pages_launch(
    const float* scores, int64_t sc_sb, int64_t sc_sh, int B, int H, int P,
    const float* retention_per_head, float retention, int k_max, int sinks, int window,
    uint8_t* mask, int64_t mk_sb, int64_t mk_sh,
    int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    int32_t* count, void* stream, const DynPos& dp) {
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
        const size_t smem = (size_t)P * 4;
        if (smem > 36 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(select_pages_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: cannot reserve %zu B of shared memory: %s", fn, smem, cudaGetErrorString(e));
        }
        launch_k(PDL_SELECT, select_pages_kernel<true>, grid, dim3(select_threads(P)), smem, st,
            scores, sc_sb, sc_sh, H, P, retention_per_head, retention, k_max, sinks, window,
            mask, mk_sb, mk_sh, compact, cp_sb, cp_sh, bucket, count, dp.pos, dp.n_new, dp.page);
    } else {
        launch_k(PDL_SELECT, select_pages_kernel<false>, grid, dim3(select_threads(P)), 0, st,
            scores, sc_sb, sc_sh, H, P, retention_per_head, retention, k_max, sinks, window,
            mask, mk_sb, mk_sh, compact, cp_sb, cp_sh, bucket, count, dp.pos, dp.n_new, dp.page);
    }
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

}  // namespace fq

extern "C" int fq_select_pages(
    const float* scores, int64_t sc_sb, int64_t sc_sh, int B, int H, int P,
    const float* retention_per_head, float retention, int k_max, int sinks, int window,
    uint8_t* mask, int64_t mk_sb, int64_t mk_sh,
    int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    int32_t* count, void* stream) {
    return fq::select_pages_launch(scores, sc_sb, sc_sh, B, H, P, retention_per_head, retention, k_max, sinks, window,
                                   mask, mk_sb, mk_sh, compact, cp_sb, cp_sh, bucket, count, stream, fq::DynPos{});
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
