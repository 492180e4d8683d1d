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
#include "fq_score_lane.cuh"

#include <cooperative_groups.h>

namespace fq {

constexpr int SEL_MAX_WARPS = 32;
constexpr int SEL_BINS = 2048;
constexpr int SEL_CAND_MAX = 128;

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
// lead_sync = false where a barrier already separates this call from the last reader of sh.warp_tot.
__device__ __forceinline__ unsigned block_warp_scan(unsigned warp_val, SelShared& sh, unsigned* total, bool lead_sync = true) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (lead_sync) __syncthreads();
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

// The selection of one row by the whole CTA.  KEYS_READY: s_keys already holds the row's keys (the
// fused kernel); otherwise they are derived from `row` (and kept in s_keys when SMEM_KEYS).
template <bool SMEM_KEYS, bool KEYS_READY>
__device__ __forceinline__ void select_row(
    SelShared& sh, unsigned* s_keys, const float* __restrict__ row, int b, int h, int H, int P,
    const float* __restrict__ retention_per_head, float retention, int k_max, int sinks, int window,
    uint8_t* __restrict__ mask, int64_t mk_sb, int64_t mk_sh,
    int32_t* __restrict__ compact, int64_t cp_sb, int64_t cp_sh, int bucket, int32_t* __restrict__ count) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int T_ = blockDim.x;
    auto key_at = [&](int i) -> unsigned { return SMEM_KEYS ? s_keys[i] : score_key(row[i]); };

    // ---- load the row once; block min / max of the keys ----
    // (the histogram of the first round and the candidate counter are cleared while the loads are in flight; the
    // barrier behind the min / max exchange covers them)
    for (int i = tid; i < SEL_BINS; i += T_) sh.hist[i] = 0u;
    if (tid == 0) sh.ncand = 0u;
    unsigned kmin = 0xffffffffu, kmax = 0u;
#pragma unroll 4
    for (int i = tid; i < P; i += T_) {
        const unsigned key = KEYS_READY ? s_keys[i] : score_key(__ldg(row + i));
        if (SMEM_KEYS && !KEYS_READY) s_keys[i] = key;
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
            if (round > 0) {
                for (int i = tid; i < SEL_BINS; i += T_) sh.hist[i] = 0u;
                __syncthreads();
            }
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
            const unsigned wprefix = block_warp_scan(__shfl_sync(0xffffffffu, incl, 31), sh, &tot_unused, false);   // the barrier above
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
    const unsigned sel_before = block_warp_scan(sel_cnt, sh, &total, rank_ties);      // every earlier use of the scan is behind a barrier, except the tie count's

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

template <bool SMEM_KEYS>
__global__ void select_pages_kernel(
    const float* __restrict__ scores, int64_t sc_sb, int64_t sc_sh, int H, int P,
    const float* __restrict__ retention_per_head, float retention, int k_max, int sinks, int window,
    uint8_t* __restrict__ mask, int64_t mk_sb, int64_t mk_sh,
    int32_t* __restrict__ compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    int32_t* __restrict__ count, const int* __restrict__ pos, int pos_new, int pos_page, int pos_early) {
    __shared__ SelShared sh;
    extern __shared__ unsigned s_keys[];                        // [P] keys (SMEM_KEYS only)
    const int b = blockIdx.y, h = blockIdx.x;
    int pos_v = 0;
    if (pos && pos_early) pos_v = __ldcg(pos);                  // in flight during the wait (see DynPos::early)
    pdl_wait();        // the scores come from the previous kernel
    pdl_trigger();
    if (pos) {         // row length read on the device: completed pages after this step's append
        if (!pos_early) pos_v = *pos;
        P = min(P, (pos_v + pos_new) / pos_page);
        k_max = min(k_max, P);
    }
    select_row<SMEM_KEYS, false>(sh, s_keys, scores + b * sc_sb + h * sc_sh, b, h, H, P, retention_per_head, retention, k_max,
                                 sinks, window, mask, mk_sb, mk_sh, compact, cp_sb, cp_sh, bucket, count);
}

// ---- page scores and selection in ONE launch ----
// A thread-block cluster of FUSED_CLUSTER CTAs per (batch, kv head): every CTA scores a contiguous
// slice of the pages for all query heads of the group (the metadata is read once), writes the scores
// to global memory and their keys into the shared memory of the CTA that will select for that head
// (rank r of the cluster takes head r of the group); after one cluster barrier those CTAs run the
// selection out of their own shared memory.  Same arithmetic as the two separate kernels.
constexpr int FUSED_THREADS = 512;
constexpr int FUSED_CLUSTER = 8;
constexpr int FUSED_MAX_P = 16384;
constexpr int FUSED_QW = FUSED_THREADS / 8; // quarter warps per CTA = pages scored per pass

struct ScoreSelectParams {
    const void* Q; int64_t q_sb, q_sh;
    const uint16_t *K_scale, *K_mn; int64_t km_sb, km_sh, km_sp;
    int Hq, Hkv, P, D; float levels;
    float* scores; int64_t sc_sb, sc_sh;
    const float* retention_per_head; float retention; int k_max, sinks, window;
    int32_t* compact; int64_t cp_sb, cp_sh; int bucket; int32_t* count;
    const int* pos; int pos_new, pos_page;
    int round;         // pages per ring buffer: 128 (head_dim <= 128) or 64
    int first_fresh;   // pages below it were written before the launch that precedes this one (0: unknown; <0 with pos: derive)
};

__device__ __forceinline__ void ss_cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void ss_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void ss_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Shared memory (dynamic): keys [P] u32 | metadata ring [2][round pages][K_mn row, K_scale row] bf16.
// The metadata of the CTA's slice is copied with cp.async, two rounds in flight; rows below
// `first_fresh` cannot have been written by the launch right before this one, so their copies are
// issued BEFORE the dependency wait and overlap the previous kernel.  The few fresher rows are read
// with plain loads after the wait.
template <typename QT, int NR, int CH>
__global__ void __launch_bounds__(FUSED_THREADS) score_select_kernel(ScoreSelectParams p) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ SelShared sh;
    extern __shared__ __align__(16) unsigned s_keys[];          // [P] keys of the head this CTA selects for
    const int rank = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
    const int n_rep = p.Hq / p.Hkv;                             // == NR heads per group
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int l = lane & 7, qw = lane >> 3;
    const int D = p.D, n_chunks = D >> 3;
    const int key_words = (p.P + 3) & ~3;
    unsigned char* ring = reinterpret_cast<unsigned char*>(s_keys + key_words);
    const int page_bytes = 4 * D;                               // K_mn row then K_scale row
    const int ROUND = p.round;
    cluster.barrier_arrive();          // matched by the wait in front of the first store to another CTA's shared memory

    const uint16_t* sc_base = p.K_scale + b * p.km_sb + hkv * p.km_sh;
    const uint16_t* mn_base = p.K_mn + b * p.km_sb + hkv * p.km_sh;
    const int pieces = D >> 2;                                  // 16-byte pieces per page (both rows)
    int p_lo = 0, p_hi = 0, fresh = 0, n_rounds = 0;
    auto issue = [&](int r) {
        unsigned char* buf = ring + (size_t)(r & 1) * ROUND * page_bytes;
        const int base = p_lo + r * ROUND;
        const int n_pg = min(ROUND, min(p_hi, fresh) - base);     // rows settled before the previous launch
        for (int j = tid; j < n_pg * pieces; j += FUSED_THREADS) {
            const int pg = j / pieces, w = j - pg * pieces;
            const uint16_t* src = (w < n_chunks ? mn_base : sc_base) + (int64_t)(base + pg) * p.km_sp + 8 * (w < n_chunks ? w : w - n_chunks);
            ss_cp_async16(buf + (size_t)pg * page_bytes + w * 16, src);
        }
    };
    auto slice = [&](int P) {
        const int per = ((P + FUSED_CLUSTER - 1) / FUSED_CLUSTER + ROUND - 1) / ROUND * ROUND;
        p_lo = min(P, rank * per); p_hi = min(P, p_lo + per);
        n_rounds = (p_hi - p_lo + ROUND - 1) / ROUND;
    };
    int P = p.P, k_max = p.k_max;
    // first_fresh != 0 is the caller's word that rows below it (below the pages completed before this
    // step's append when it is negative and the length lives on the device) were written before the
    // launch that precedes this one; so was the device-side length
    const bool early = p.first_fresh != 0;
    auto prepare = [&]() {
        if (p.pos) {
            P = min(P, (*p.pos + p.pos_new) / p.pos_page);
            k_max = min(k_max, P);
        }
        slice(P);
        if (!early) fresh = P;
        else if (p.first_fresh > 0) fresh = min(P, p.first_fresh);
        else fresh = p.pos ? min(P, *p.pos / p.pos_page) : 0;
#pragma unroll
        for (int r = 0; r < 2; ++r) { if (r < n_rounds) issue(r); ss_cp_async_commit(); }
    };
    if (early) prepare();
    pdl_wait();                        // Q and the fresh metadata rows come from the kernels before this one
    pdl_trigger();
    if (!early) prepare();
    float q[NR][CH][8];
    score_load_q<QT, NR, CH>(static_cast<const QT*>(p.Q) + b * p.q_sb, p.q_sh, hkv * n_rep, n_rep, l, n_chunks, q);
    cluster.barrier_wait();            // every CTA of the cluster runs: its shared memory may be addressed
    unsigned* keys_of = l < n_rep ? cluster.map_shared_rank(s_keys, l) : nullptr;    // lane l reports head l of the group
    float* srow = p.scores + b * p.sc_sb + (hkv * n_rep + min(l, n_rep - 1)) * p.sc_sh;
    for (int r = 0; r < n_rounds; ++r) {
        ss_cp_async_wait<1>();         // round r has landed (round r+1 may still be in flight)
        __syncthreads();
        const unsigned char* buf = ring + (size_t)(r & 1) * ROUND * page_bytes;
        for (int it = 0; it < ROUND / FUSED_QW; ++it) {
            const int slot = it * FUSED_QW + warp * 4 + qw;
            const int pg = p_lo + r * ROUND + slot;
            const bool live = pg < p_hi;
            uint4 m4[CH], s4[CH];
            if (live && pg >= fresh) {
                score_load_meta<CH>(sc_base, mn_base, p.km_sp, pg, true, l, n_chunks, m4, s4);
            } else {
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    const int chunk = l + 8 * c;
                    if (live && chunk < n_chunks) {
                        m4[c] = *reinterpret_cast<const uint4*>(buf + (size_t)slot * page_bytes + chunk * 16);
                        s4[c] = *reinterpret_cast<const uint4*>(buf + (size_t)slot * page_bytes + (n_chunks + chunk) * 16);
                    } else {
                        m4[c] = make_uint4(0, 0, 0, 0);
                        s4[c] = make_uint4(0, 0, 0, 0);
                    }
                }
            }
            const float v = score_page<NR, CH>(q, m4, s4, l, p.levels);
            if (live && l < n_rep) {
                srow[pg] = v;
                keys_of[pg] = score_key(v);
            }
        }
        __syncthreads();               // the buffer is free again
        if (r + 2 < n_rounds) issue(r + 2);
        ss_cp_async_commit();
    }
    ss_cp_async_wait<0>();
    cluster.sync();                    // all keys of all heads have arrived
    if (rank >= n_rep) return;
    const int h = hkv * n_rep + rank;
    select_row<true, true>(sh, s_keys, nullptr, b, h, p.Hq, P, p.retention_per_head, p.retention, k_max, p.sinks, p.window,
                           nullptr, 0, 0, p.compact, p.cp_sb, p.cp_sh, p.bucket, p.count);
}

// mask (rows,P) u8 -> compact (rows,bucket) int32, descending ids, -1 padded.
__global__ void build_compact_kernel(const uint8_t* __restrict__ mask, int64_t mk_sr, int P,
                                     int32_t* __restrict__ compact, int64_t cp_sr, int bucket, int32_t* __restrict__ count) {
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
    if (count && tid == 0) count[r] = (int32_t)min(total, (unsigned)bucket);      // entries at the front of the list
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
            mask, mk_sb, mk_sh, compact, cp_sb, cp_sh, bucket, count, dp.pos, dp.n_new, dp.page, dp.early ? 1 : 0);
    } else {
        launch_k(PDL_SELECT, select_pages_kernel<false>, grid, dim3(select_threads(P)), 0, st,
            scores, sc_sb, sc_sh, H, P, retention_per_head, retention, k_max, sinks, window,
            mask, mk_sb, mk_sh, compact, cp_sb, cp_sh, bucket, count, dp.pos, dp.n_new, dp.page, dp.early ? 1 : 0);
    }
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

template <typename QT, int NR>
static cudaError_t launch_score_select(int CH, const ScoreSelectParams& p, dim3 grid, size_t smem, cudaStream_t st) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = dim3(FUSED_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[2]{};
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = FUSED_CLUSTER; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 2;
#define FQ_SS(CHV)                                                                                                   \
    do {                                                                                                             \
        if (smem > 36 * 1024) {                                                                                      \
            cudaError_t e = cudaFuncSetAttribute(score_select_kernel<QT, NR, CHV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return e;                                                                          \
        }                                                                                                            \
        return cudaLaunchKernelEx(&cfg, score_select_kernel<QT, NR, CHV>, p);                                        \
    } while (0)
    if (CH == 1) FQ_SS(1);
    else if (CH == 2) FQ_SS(2);
    else FQ_SS(4);
#undef FQ_SS
}

template <typename QT>
static cudaError_t launch_score_select_nr(int n_rep, int CH, const ScoreSelectParams& p, dim3 grid, size_t smem, cudaStream_t st) {
    if (n_rep == 1) return launch_score_select<QT, 1>(CH, p, grid, smem, st);
    if (n_rep == 2) return launch_score_select<QT, 2>(CH, p, grid, smem, st);
    if (n_rep == 3) return launch_score_select<QT, 3>(CH, p, grid, smem, st);
    return launch_score_select<QT, 4>(CH, p, grid, smem, st);
}

bool score_select_fusable(int Hq, int Hkv, int P, int D) {
    return Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 4 && P <= FUSED_MAX_P && (D == 32 || D == 64 || D == 128 || D == 256);
}

int score_select_launch(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P, int D, float levels, float* scores, int64_t sc_sb, int64_t sc_sh,
    const float* retention_per_head, float retention, int k_max, int sinks, int window,
    int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket, int32_t* count, void* stream, const DynPos& dp, int first_fresh) {
    const char* fn = "fq_score_select";
    FQ_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && P >= 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(Hq % Hkv == 0, FQ_ERR_ARG, "%s: H_q=%d must be divisible by H_kv=%d", fn, Hq, Hkv);
    FQ_CHECK_ARG(score_select_fusable(Hq, Hkv, P, D), FQ_ERR_UNSUPPORTED,
                 "%s: the fused launch takes up to 4 query heads per KV head, up to %d pages and head_dim in {32,64,128,256}", fn, FUSED_MAX_P);
    FQ_CHECK_ARG(q_dtype == FQ_F32 || q_dtype == FQ_F16 || q_dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: dtype code %d", fn, q_dtype);
    FQ_CHECK_ARG(retention_per_head || (retention >= 0.f && retention <= 1.f), FQ_ERR_ARG,
                 "%s: scalar retention must be in [0, 1]; got %g", fn, (double)retention);
    FQ_CHECK_ARG(k_max >= 0 && sinks >= 0 && window >= 0, FQ_ERR_ARG, "%s: k_max/sinks/window must be >= 0", fn);
    FQ_CHECK_ARG(compact && bucket >= 1, FQ_ERR_ARG, "%s: BUCKET_MAX must be >= 1, got %d", fn, bucket);
    FQ_CHECK_ARG(Q && scores && (P == 0 || (K_scale && K_mn)), FQ_ERR_ARG, "%s: null pointer", fn);
    FQ_CHECK_ARG(B <= 65535 && Hkv <= 65535, FQ_ERR_ARG, "%s: batch or head count too large", fn);
    const int64_t qa = q_dtype == FQ_F32 ? 4 : 8;
    FQ_CHECK_ARG(q_sb % qa == 0 && q_sh % qa == 0 && aligned(Q, 16), FQ_ERR_ALIGN, "%s: Q rows must be 16-byte aligned", fn);
    FQ_CHECK_ARG(P == 0 || (km_sb % 8 == 0 && km_sh % 8 == 0 && km_sp % 8 == 0 && aligned(K_scale, 16) && aligned(K_mn, 16)),
                 FQ_ERR_ALIGN, "%s: K metadata rows must be 16-byte aligned", fn);
    ScoreSelectParams p;
    p.Q = Q; p.q_sb = q_sb; p.q_sh = q_sh;
    p.K_scale = static_cast<const uint16_t*>(K_scale); p.K_mn = static_cast<const uint16_t*>(K_mn);
    p.km_sb = km_sb; p.km_sh = km_sh; p.km_sp = km_sp;
    p.Hq = Hq; p.Hkv = Hkv; p.P = P; p.D = D; p.levels = levels;
    p.scores = scores; p.sc_sb = sc_sb; p.sc_sh = sc_sh;
    p.retention_per_head = retention_per_head; p.retention = retention; p.k_max = k_max; p.sinks = sinks; p.window = window;
    p.compact = compact; p.cp_sb = cp_sb; p.cp_sh = cp_sh; p.bucket = bucket; p.count = count;
    p.pos = dp.pos; p.pos_new = dp.n_new; p.pos_page = dp.page;
    p.first_fresh = first_fresh;
    p.round = D <= 128 ? 2 * FUSED_QW : FUSED_QW;
    const int CH = D <= 64 ? 1 : D / 64;
    const size_t smem = (size_t)((P + 3) & ~3) * 4 + 2 * (size_t)p.round * 4 * D;
    dim3 grid(FUSED_CLUSTER, (unsigned)Hkv, (unsigned)B);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int n_rep = Hq / Hkv;
    cudaError_t e;
    if (q_dtype == FQ_F32) e = launch_score_select_nr<float>(n_rep, CH, p, grid, smem, st);
    else if (q_dtype == FQ_F16) e = launch_score_select_nr<__half>(n_rep, CH, p, grid, smem, st);
    else e = launch_score_select_nr<__nv_bfloat16>(n_rep, CH, p, grid, smem, st);
    if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: launch failed: %s", fn, cudaGetErrorString(e));
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

extern "C" int fq_build_compact_counted(const uint8_t* mask, int64_t mk_sr, int64_t rows, int P,
                                        int32_t* compact, int64_t cp_sr, int bucket, int32_t* count, void* stream) {
    using namespace fq;
    const char* fn = "fq_build_compact";
    FQ_CHECK_ARG(bucket >= 1, FQ_ERR_ARG, "%s: BUCKET_MAX must be >= 1, got %d", fn, bucket);
    FQ_CHECK_ARG(rows >= 0 && P >= 0 && compact && (mask || P == 0 || rows == 0), FQ_ERR_ARG, "%s: bad arguments", fn);
    if (rows == 0) return FQ_OK;
    FQ_CHECK_ARG(rows <= 0x7fffffffLL, FQ_ERR_ARG, "%s: too many rows", fn);
    build_compact_kernel<<<(unsigned)rows, select_threads(P), 0, static_cast<cudaStream_t>(stream)>>>(
        mask, mk_sr, P, compact, cp_sr, bucket, count);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" int fq_build_compact(const uint8_t* mask, int64_t mk_sr, int64_t rows, int P,
                                int32_t* compact, int64_t cp_sr, int bucket, void* stream) {
    return fq_build_compact_counted(mask, mk_sr, rows, P, compact, cp_sr, bucket, nullptr, stream);
}

extern "C" int fq_score_select(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P, int D, int levels, float* scores, int64_t sc_sb, int64_t sc_sh,
    const float* retention_per_head, float retention, int k_max, int sinks, int window,
    int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket, int32_t* count, int first_fresh_page, void* stream) {
    if (levels != 15 && levels != 255)
        return fq::fail(FQ_ERR_ARG, "fq_score_select: levels must be 15 (INT4 metadata) or 255 (INT8 metadata), got %d", levels);
    return fq::score_select_launch(Q, q_dtype, q_sb, q_sh, K_scale, K_mn, km_sb, km_sh, km_sp, B, Hq, Hkv, P, D, (float)levels,
                                   scores, sc_sb, sc_sh, retention_per_head, retention, k_max, sinks, window,
                                   compact, cp_sb, cp_sh, bucket, count, stream, fq::DynPos{}, first_fresh_page < 0 ? 0 : first_fresh_page);
}

extern "C" int fq_score_select_supported(int Hq, int Hkv, int P, int D) { return fq::score_select_fusable(Hq, Hkv, P, D) ? 1 : 0; }
