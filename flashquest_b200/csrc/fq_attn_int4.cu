// Sparse decode attention over selected packed INT4 pages: GQA, split-K, LSE merge.
//
// Work unit = one chunk of TOK tokens of one selected page (TOK = 16, or 8 for page 8):
//   K payload TOK*D/2 B, V payload TOK*D/2 B, K scale + K min rows 2*D*2 B, V scale + V min
//   2*TOK*2 B  (2624 B at D = 128, TOK = 16).  The two payloads (1 KB each) are staged in
//   shared memory by bulk copies; the small metadata pieces go straight to registers with
//   ordinary 16-byte / 4-byte loads issued at the same moment (a bulk copy per 32-byte piece
//   costs the copy engine as much as a 1 KB one).
// Grid = (n_split, H_q, B); a CTA walks a contiguous slice of the row's compact page list.
// A CTA has ATT_WARPS consumer warps and one producer warp.  Every QUARTER WARP (8 lanes) of
// a consumer warp owns one unit at a time, so a CTA works on 4*ATT_WARPS units per iteration.
// The producer warp stages the payloads into shared memory with bulk asynchronous copies
// (cp.async.bulk + mbarrier complete_tx), ATT_STAGES iterations deep: the copy engine back-
// pressures the issuing thread for as long as the transfer lasts, so the issue must not sit
// in the warps that do the arithmetic.  Per (consumer warp, stage) there is a "full" barrier
// (the producer's expect_tx arrivals + the copies' bytes) and an "empty" barrier (the
// consumer warp's release).  The launch is sized so that all CTAs are resident at once; every
// byte of the selection is then requested in the first microsecond and streams in at HBM
// speed while the consumers work through the units in arrival order.
//
// Arithmetic (CUDA cores, fp32 accumulation, no tensor cores: M is 1):
//   q.k = sum_d (q_d*sc_d)*code_d + sum_d q_d*mn_d      (scale folded into q once per page)
//   o_d = sum_t (p_t*vs_t)*code_td + sum_t p_t*vm_t     (min folded into one scalar)
// A 4-bit code is turned into an fp32 operand with ONE integer instruction: the nibble is
// masked in place and the word reinterpreted as an fp32 (sub)normal, whose value is
// code * 2^(4k-149) for nibble k = 0..5 (bits 0..23 of an fp32 read as an integer times
// 2^-149, across the subnormal/normal boundary).  The power of two is folded into the
// multiplier (pre-scaled by 2^100 to stay in range).  The top byte gives (c6 + 16*c7) and c7
// with one shift each; the multiplier of c7 is corrected by -16*m6.
// A lane owns D/8 channels of every token: K dot products are reduced across the 8 lanes
// with a transposing shuffle (14 shuffles for 16 tokens); the V accumulation needs no
// reduction at all.  Softmax runs in base 2 with sm_scale*log2(e) folded into q.
//
// Split-K: each CTA writes (m, l, acc[D]) to the workspace and takes a ticket; the CTA that
// draws the last ticket of its row merges the partials in split order and writes O / LSE.
// No CTA ever waits for another one.
#include "fq_common.cuh"

namespace fq {

constexpr int ATT_WARPS = 4;                        // consumer warps per CTA (one more warp issues the copies)
constexpr int ATT_THREADS = (ATT_WARPS + 1) * 32;   // consumers + the producer warp
constexpr int ATT_STAGES = 2;
constexpr int ATT_CTAS_PER_SM = 3;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr unsigned WAIT_SPIN_LIMIT = 1u << 24;   // bounded wait on a stage; then give up

struct AttnParams {
    const void* Q; int64_t q_sb, q_sh;
    const uint8_t* K_packed; int64_t kp_sb, kp_sh;
    const uint16_t *K_scale, *K_mn; int64_t km_sb, km_sh, km_sp;
    const uint8_t* V_packed; int64_t vp_sb, vp_sh;
    const uint16_t *V_scale, *V_mn; int64_t vm_sb, vm_sh;
    const int32_t* compact; int64_t cp_sb, cp_sh; int bucket;
    const int32_t* list_count;        // non-null: per (b,hq) row, only the first list_count[row] list entries can be valid
    const void *K_tail, *V_tail; int tail_dtype; int64_t tl_sb, tl_sh, tl_ss; int tail_len;
    int B, Hq, Hkv, S_kv, P, page, cpp_log2;
    float sm_scale;
    void* O; int64_t o_sb, o_sh;
    float* lse;
    int* tickets; float* partials; int n_split;
    const int* pos; int pos_new;      // non-null: S_kv, P and tail_len are derived from *pos on the device (see DynPos)
    int pos_early;                    // *pos may be read before the dependency wait (DynPos::early)
    int* status;
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// global -> shared bulk copy; completion is counted in bytes on the mbarrier.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}


// ---------------------------------------------------------------- unit layout in shared memory
template <int D, int TOK>
struct UnitLayout {
    static constexpr int ROW = D / 2;               // packed bytes per token
    static constexpr int K_OFF = 0;
    static constexpr int V_OFF = TOK * ROW;
    static constexpr int BYTES = 2 * TOK * ROW;
    // stride = 64 mod 128 bytes, so the four quarter warps of a warp hit disjoint bank halves
    // pairwise (two wavefronts for a 256-byte warp read, the minimum)
    static constexpr int STRIDE = (BYTES % 128 == 0) ? BYTES + 64 : ((BYTES + 15) & ~15);
};

// Multiplier pre-scale for channel j (j mod 8 = nibble index) so that
// (code as masked fp32 bits) * mult = code * value * 2^-49.
__device__ __forceinline__ float pow2i(int n) { return __int_as_float((127 + n) << 23); }
__device__ __forceinline__ float nib_scale(int k) {
    // nibble k <= 5 is read as code*2^(4k-149); nibbles 6,7 (after a shift) as *2^-149
    return k <= 5 ? pow2i(100 - 4 * k) : pow2i(100);
}
__device__ __forceinline__ float nib_descale(int k) { return k <= 5 ? pow2i(4 * k - 100) : pow2i(-100); }   // 1 / nib_scale
__device__ __forceinline__ float nib_unscale(int k) { return k <= 5 ? pow2i(49 - 4 * k) : pow2i(49); }

// eight codes of one 32-bit word as fp32 operands (see the header comment)
__device__ __forceinline__ void nib8(uint32_t w, float (&f)[8]) {
    f[0] = __uint_as_float(w & 0x0000000fu);
    f[1] = __uint_as_float(w & 0x000000f0u);
    f[2] = __uint_as_float(w & 0x00000f00u);
    f[3] = __uint_as_float(w & 0x0000f000u);
    f[4] = __uint_as_float(w & 0x000f0000u);
    f[5] = __uint_as_float(w & 0x00f00000u);
    f[6] = __uint_as_float(w >> 24);   // c6 + 16*c7
    f[7] = __uint_as_float(w >> 28);   // c7
}

// N consecutive 32-bit words from shared memory with the widest load (N = 1, 2, 4)
template <int N>
__device__ __forceinline__ void ld_words(const unsigned char* p, uint32_t (&w)[N]) {
    static_assert(N == 1 || N == 2 || N == 4, "words per lane");
    if constexpr (N == 1) { w[0] = *reinterpret_cast<const uint32_t*>(p); }
    else if constexpr (N == 2) { const uint2 v = *reinterpret_cast<const uint2*>(p); w[0] = v.x; w[1] = v.y; }
    else { const uint4 v = *reinterpret_cast<const uint4*>(p); w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
}

// Transposing reduction over the 8 lanes of a quarter warp: in: N partial sums per lane,
// out: lane l holds the full sums of tokens (N/8)*l .. (N/8)*l + N/8-1 in s[0..N/8).
template <int N>
__device__ __forceinline__ void qw_transpose_reduce(float (&s)[N], int l, unsigned qmask) {
    static_assert(N == 8 || N == 16, "N");
    {
        const bool up = l & 4;
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            const float send = up ? s[i] : s[i + N / 2];
            const float keep = up ? s[i + N / 2] : s[i];
            s[i] = keep + __shfl_xor_sync(qmask, send, 4);
        }
    }
    {
        const bool up = l & 2;
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            const float send = up ? s[i] : s[i + N / 4];
            const float keep = up ? s[i + N / 4] : s[i];
            s[i] = keep + __shfl_xor_sync(qmask, send, 2);
        }
    }
    {
        const bool up = l & 1;
#pragma unroll
        for (int i = 0; i < N / 8; ++i) {
            const float send = up ? s[i] : s[i + N / 8];
            const float keep = up ? s[i + N / 8] : s[i];
            s[i] = keep + __shfl_xor_sync(qmask, send, 1);
        }
    }
}

__device__ __forceinline__ float qw_sum(float v, unsigned qmask) {
    v += __shfl_xor_sync(qmask, v, 4);
    v += __shfl_xor_sync(qmask, v, 2);
    v += __shfl_xor_sync(qmask, v, 1);
    return v;
}
__device__ __forceinline__ float qw_max(float v, unsigned qmask) {
    v = fmaxf(v, __shfl_xor_sync(qmask, v, 4));
    v = fmaxf(v, __shfl_xor_sync(qmask, v, 2));
    v = fmaxf(v, __shfl_xor_sync(qmask, v, 1));
    return v;
}

template <typename T>
__device__ __forceinline__ float ld_as_f32(const void* p, int64_t i) { return Dt<T>::to_f32(static_cast<const T*>(p)[i]); }

// ---------------------------------------------------------------- the kernel
// What a quarter warp knows about a unit besides its payload.
template <int DPL, int TPL>
struct UnitCtx {
    int page_id, tok0, n_tok;             // page_id < 0: nothing to do in this slot
    uint4 ks[DPL / 8], km[DPL / 8];       // this lane's DPL channels of the K scale / min rows (bf16)
    uint32_t vs_raw, vm_raw;              // V scale / min of this lane's TPL tokens, bf16 bits (token i in half i)
};

// DYN: the sequence length is read from *p.pos on the device (graph-capturable step); a separate
// instantiation so that the ordinary launches keep their register budget.
template <typename QT, int D, int TOK, bool DYN>
__global__ void __launch_bounds__(ATT_THREADS, ATT_CTAS_PER_SM) sparse_decode_int4_kernel(AttnParams p) {
    using L = UnitLayout<D, TOK>;
    constexpr int DPL = D / 8;        // channels per lane
    constexpr int WPL = DPL / 8;      // 32-bit words per lane per token
    constexpr int TPL = TOK / 8;      // tokens per lane after the reduction
    constexpr int NSTATE = ATT_WARPS * 4 + ATT_WARPS;   // quarter-warp states + per-warp tail states
    constexpr int NBARS = 2 * ATT_WARPS * ATT_STAGES;

    extern __shared__ __align__(128) unsigned char smem[];
    // [stages][warps][4 units] staging | mbarriers | pv broadcast | states; the merge area
    // aliases the staging area once the main loop is over
    unsigned char* stage_base = smem;
    constexpr int STAGING_BYTES = ATT_STAGES * ATT_WARPS * 4 * L::STRIDE;
    uint64_t* full_bars = reinterpret_cast<uint64_t*>(smem + STAGING_BYTES);       // [warps][stages]
    uint64_t* empty_bars = full_bars + ATT_WARPS * ATT_STAGES;                     // [warps][stages]
    float* pv_bcast = reinterpret_cast<float*>(smem + STAGING_BYTES + NBARS * 8);  // [warps*4][TOK]
    float* st_m = pv_bcast + ATT_WARPS * 4 * TOK;   // [NSTATE] running max, then merge weight
    float* st_l = st_m + NSTATE;                    // [NSTATE]
    float* st_acc = reinterpret_cast<float*>(smem);  // [NSTATE][D]

    const int split = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
    const int n_rep = p.Hq / p.Hkv, hkv = hq / n_rep;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, qw = lane >> 3, l = lane & 7;
    const unsigned qmask = 0xffu << (8 * qw);
    const bool is_producer = warp == ATT_WARPS;

    // ---- units of the compact list owned by this CTA ----
    // Units are dealt round-robin to the splits (unit g belongs to split g % n_split), so a
    // list with its valid entries at the front and -1 padding behind them stays balanced.
    const int cpp_log2 = p.cpp_log2;                    // log2(chunks (units) per page)
    constexpr int units_per_iter = ATT_WARPS * 4;
    const int32_t* list = p.compact + b * p.cp_sb + hq * p.cp_sh;

    if (tid == 0) {
        for (int i = 0; i < ATT_WARPS * ATT_STAGES; ++i) {
            mbar_init(&full_bars[i], 4);    // one arrival per unit of the warp
            mbar_init(&empty_bars[i], 1);   // the consumer warp's release
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    int pos_v = 0;
    if constexpr (DYN) {
        if (p.pos_early) pos_v = __ldcg(p.pos);        // in flight during the barrier and the wait
    }
    __syncthreads();
    pdl_wait();        // the page list (and, in the fused step, the freshly packed page) come from the previous kernels
    pdl_trigger();
    if constexpr (DYN) {
        if (!p.pos_early) pos_v = *p.pos;
    }
    // A list made from a selection mask is as wide as the page count; its builder says how many entries at the
    // front are real, and the padding behind them is not walked at all.
    int n_list = p.bucket;
    if (p.list_count) n_list = max(0, min(n_list, __ldg(p.list_count + b * p.Hq + hq)));
    const int total_units = n_list << cpp_log2;
    const int n_units = split < total_units ? (total_units - split + p.n_split - 1) / p.n_split : 0;
    const int n_iter = (n_units + units_per_iter - 1) / units_per_iter;
    // tokens in completed pages; read on the device when the launch must not depend on the sequence length
    int dyn_S = p.S_kv;
    if constexpr (DYN) {
        const int now = pos_v + p.pos_new;
        dyn_S = now - now % p.page;
    }

    const uint8_t* Kp = p.K_packed + b * p.kp_sb + hkv * p.kp_sh;
    const uint8_t* Vp = p.V_packed + b * p.vp_sb + hkv * p.vp_sh;
    const uint16_t* Ks = p.K_scale + b * p.km_sb + hkv * p.km_sh;
    const uint16_t* Km = p.K_mn + b * p.km_sb + hkv * p.km_sh;
    const uint16_t* Vs = p.V_scale + b * p.vm_sb + hkv * p.vm_sh;
    const uint16_t* Vm = p.V_mn + b * p.vm_sb + hkv * p.vm_sh;

    // unit uu (0..units_per_iter) of iteration it -> page id (or -1), first token, valid tokens
    auto locate = [&](int it, int uu, int& page_id, int& tok0, int& n_tok) {
        const int u = it * units_per_iter + uu;
        page_id = -1; tok0 = 0; n_tok = 0;
        if (u < n_units) {
            const int g = u * p.n_split + split;
            const int pg = __ldg(list + (g >> cpp_log2));
            if (pg >= 0 && pg < p.P && pg * p.page < dyn_S) {
                tok0 = pg * p.page + (g & ((1 << cpp_log2) - 1)) * TOK;
                n_tok = min(TOK, dyn_S - tok0);
                if (n_tok > 0) page_id = pg; else n_tok = 0;
            }
        }
    };

    // per quarter-warp online-softmax state (all in base 2); the producer warp keeps the
    // neutral element
    float m_run = -INFINITY;          // running max
    float l_part = 0.f;               // this lane's share of the denominator
    float mn_part = 0.f;              // this lane's share of sum_t p_t * vm_t
    float2 acc[DPL / 2];
#pragma unroll
    for (int j = 0; j < DPL / 2; ++j) acc[j] = make_float2(0.f, 0.f);
    bool timed_out = false;

    if (is_producer) {
        // =========================== producer warp ===========================
        // Lane j handles unit j of the iteration: it waits for the consumer's release of the
        // stage, announces the bytes and issues both payload copies.  One lane per unit: a lane
        // that only issued the second copy could fall two barrier phases behind when a unit is
        // empty (no bytes are awaited then), and a parity wait cannot see that.
        for (int it = 0; it < n_iter && !timed_out; ++it) {
            const int s_ = it % ATT_STAGES;
#pragma unroll
            for (int u0 = 0; u0 < units_per_iter; u0 += 32) {
                const int uu = u0 + lane;
                if (uu < units_per_iter) {
                    const int w = uu >> 2, q = uu & 3;
                    uint64_t* full = &full_bars[w * ATT_STAGES + s_];
                    if (it >= ATT_STAGES) {     // wait until the consumer warp has released the stage
                        const unsigned par = (unsigned)(it / ATT_STAGES - 1) & 1u;
                        unsigned spins = 0;
                        while (!mbar_try_wait(&empty_bars[w * ATT_STAGES + s_], par)) {
                            if (++spins > WAIT_SPIN_LIMIT) { timed_out = true; break; }
                        }
                    }
                    if (!timed_out) {
                        int page_id, tok0, n_tok;
                        locate(it, uu, page_id, tok0, n_tok);
                        if (page_id >= 0) {
                            unsigned char* dst = stage_base + ((s_ * ATT_WARPS + w) * 4 + q) * L::STRIDE;
                            const unsigned payload = (unsigned)n_tok * L::ROW;
                            mbar_arrive_expect_tx(full, 2u * payload);
                            bulk_g2s(dst + L::K_OFF, Kp + (int64_t)tok0 * L::ROW, payload, full);
                            bulk_g2s(dst + L::V_OFF, Vp + (int64_t)tok0 * L::ROW, payload, full);
                        } else {
                            mbar_arrive(full);
                        }
                    }
                }
            }
            timed_out = __any_sync(0xffffffffu, timed_out);
        }
        if (timed_out && lane == 0) atomicExch(p.status, FQ_ERR_TIMEOUT);
    } else {
        // =========================== consumer warps ===========================
        UnitCtx<DPL, TPL> ctx_cur, ctx_nxt;     // metadata of the unit in hand and of the next one
        auto load_ctx = [&](UnitCtx<DPL, TPL>& c, int it) {
            locate(it, warp * 4 + qw, c.page_id, c.tok0, c.n_tok);
            c.vs_raw = 0u; c.vm_raw = 0u;
            if (c.page_id < 0) return;
            const uint16_t* ksr = Ks + (int64_t)c.page_id * p.km_sp + DPL * l;
            const uint16_t* kmr = Km + (int64_t)c.page_id * p.km_sp + DPL * l;
#pragma unroll
            for (int j = 0; j < DPL / 8; ++j) {
                c.ks[j] = ldg16(ksr + 8 * j);
                c.km[j] = ldg16(kmr + 8 * j);
            }
            if (c.n_tok == TOK && TPL == 2) {
                c.vs_raw = __ldg(reinterpret_cast<const uint32_t*>(Vs + c.tok0 + 2 * l));
                c.vm_raw = __ldg(reinterpret_cast<const uint32_t*>(Vm + c.tok0 + 2 * l));
            } else {   // ragged last chunk (or one token per lane): per-token loads
#pragma unroll
                for (int i = 0; i < TPL; ++i) {
                    const int t = TPL * l + i;
                    if (t < c.n_tok) {
                        c.vs_raw |= (uint32_t)__ldg(Vs + c.tok0 + t) << (16 * i);
                        c.vm_raw |= (uint32_t)__ldg(Vm + c.tok0 + t) << (16 * i);
                    }
                }
            }
        };
        ctx_cur.page_id = -1; ctx_nxt.page_id = -1;
        if (n_iter > 0) load_ctx(ctx_cur, 0);

        // ---- q slice of this lane, pre-multiplied by sm_scale*log2(e) and the nibble scale ----
        float qn[DPL];    // q*sm_scale*log2e times the nibble pre-scale (a power of two)
        {
            const QT* qp = static_cast<const QT*>(p.Q) + b * p.q_sb + hq * p.q_sh + DPL * l;
            const float c = p.sm_scale * LOG2E;
#pragma unroll
            for (int j = 0; j < DPL; j += 8) {
                float v[8];
                load8<QT>(qp + j, v);
#pragma unroll
                for (int e = 0; e < 8; ++e) qn[j + e] = v[e] * c * nib_scale(e);
            }
        }
        float* pvb = pv_bcast + (warp * 4 + qw) * TOK;

        // One unit: K dot products, softmax update, V accumulation (see the header comment).
        auto compute_unit = [&](const unsigned char* u, const UnitCtx<DPL, TPL>& c, auto&& prefetch) {
            // ---------------- K: fold the page scale into q; q.mn ----------------
            float qs[DPL];
            float qmn = 0.f;
#pragma unroll
            for (int j = 0; j < DPL; j += 8) {
                const uint4 s4 = c.ks[j / 8];
                const uint4 m4 = c.km[j / 8];
                const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w}, mw[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    qs[j + 2 * e] = qn[j + 2 * e] * bf16_lo(sw[e]);
                    qs[j + 2 * e + 1] = qn[j + 2 * e + 1] * bf16_hi(sw[e]);
                    // q.mn with the pre-scaled q: the power of two moves to mn, the product is the same
                    qmn = fmaf(qn[j + 2 * e], bf16_lo(mw[e]) * nib_descale(2 * e), qmn);
                    qmn = fmaf(qn[j + 2 * e + 1], bf16_hi(mw[e]) * nib_descale(2 * e + 1), qmn);
                }
                qs[j + 7] = fmaf(-16.f, qs[j + 6], qs[j + 7]);   // c7 rides on (c6 + 16 c7)
            }
            qmn = qw_sum(qmn, qmask);
            prefetch();

            float sdot[TOK];
            // one token at a time (interleaving several tokens by hand measured slower: register pressure)
#pragma unroll
            for (int t = 0; t < TOK; ++t) {
                uint32_t w[WPL];
                ld_words<WPL>(u + L::K_OFF + t * L::ROW + 4 * WPL * l, w);
                float2 a = make_float2(0.f, 0.f);
#pragma unroll
                for (int wd = 0; wd < WPL; ++wd) {
                    float f[8];
                    nib8(w[wd], f);
#pragma unroll
                    for (int e = 0; e < 8; e += 2)
                        a = __ffma2_rn(make_float2(f[e], f[e + 1]), make_float2(qs[8 * wd + e], qs[8 * wd + e + 1]), a);
                }
                sdot[t] = a.x + a.y;
            }
            qw_transpose_reduce<TOK>(sdot, l, qmask);

            // ---------------- softmax for this lane's TPL tokens ----------------
            const float UNS = 5.62949953421312e14f;   // 2^49
            float x[TPL];
            float pmax = -INFINITY;
#pragma unroll
            for (int i = 0; i < TPL; ++i) {
                const bool valid = TPL * l + i < c.n_tok;
                x[i] = valid ? fmaf(sdot[i], UNS, qmn) : -INFINITY;
                pmax = fmaxf(pmax, x[i]);
            }
            pmax = qw_max(pmax, qmask);
            const float m_new = fmaxf(m_run, pmax);     // finite: the unit has at least one valid token
            const float alpha = ex2(m_run - m_new);     // ex2(-inf) = 0 on the first unit
            m_run = m_new;
            l_part *= alpha;
            mn_part *= alpha;
#pragma unroll
            for (int i = 0; i < TPL; ++i) {
                const float pr = ex2(x[i] - m_new);
                const float vsi = i == 0 ? bf16_lo(c.vs_raw) : bf16_hi(c.vs_raw);
                const float vmi = i == 0 ? bf16_lo(c.vm_raw) : bf16_hi(c.vm_raw);
                l_part += pr;
                mn_part = fmaf(pr, vmi, mn_part);
                pvb[TPL * l + i] = pr * vsi * 1.2676506002282294e30f;   // * 2^100
            }
            __syncwarp(qmask);

            // ---------------- V ----------------
            const float2 alpha2 = make_float2(alpha, alpha);
#pragma unroll
            for (int j = 0; j < DPL / 2; ++j) acc[j] = __fmul2_rn(acc[j], alpha2);
#pragma unroll
            for (int t4 = 0; t4 < TOK; t4 += 4) {
                const float4 pv4 = *reinterpret_cast<const float4*>(pvb + t4);
                const float pv[4] = {pv4.x, pv4.y, pv4.z, pv4.w};
#pragma unroll
                for (int tt = 0; tt < 4; ++tt) {
                    const int t = t4 + tt;
                    const float2 pp = make_float2(pv[tt], pv[tt]);
                    uint32_t wv[WPL];
                    ld_words<WPL>(u + L::V_OFF + t * L::ROW + 4 * WPL * l, wv);
#pragma unroll
                    for (int wd = 0; wd < WPL; ++wd) {
                        float f[8];
                        nib8(wv[wd], f);
#pragma unroll
                        for (int e = 0; e < 8; e += 2)
                            acc[4 * wd + e / 2] = __ffma2_rn(make_float2(f[e], f[e + 1]), pp, acc[4 * wd + e / 2]);
                    }
                }
            }
            __syncwarp(qmask);   // pv_bcast is rewritten by the next unit
        };


        // ---- main loop: wait for the stage, consume it, release it to the producer ----
        for (int it = 0; it < n_iter && !timed_out; ++it) {
            const int s_ = it % ATT_STAGES;
            const unsigned parity = (unsigned)(it / ATT_STAGES) & 1u;
            unsigned spins = 0;
            bool gave_up = false;
            while (!mbar_try_wait(&full_bars[warp * ATT_STAGES + s_], parity)) {
                if (++spins > WAIT_SPIN_LIMIT) { gave_up = true; break; }
            }
            if (__any_sync(0xffffffffu, gave_up)) { timed_out = true; break; }
            // the next unit's metadata is requested while this unit is being worked on
            auto prefetch = [&]() {
                if (it + 1 < n_iter) load_ctx(ctx_nxt, it + 1);
            };
            if (ctx_cur.page_id >= 0)                  // uniform inside the quarter warp
                compute_unit(stage_base + ((s_ * ATT_WARPS + warp) * 4 + qw) * L::STRIDE, ctx_cur, prefetch);
            else
                prefetch();
            __syncwarp();                              // every lane is done reading this stage
            fence_proxy_async();
            if (lane == 0) mbar_arrive(&empty_bars[warp * ATT_STAGES + s_]);
            ctx_cur = ctx_nxt;
        }
        if (timed_out && lane == 0) atomicExch(p.status, FQ_ERR_TIMEOUT);
    }
    // A CTA that gave up may still have copies in flight into its shared memory; the producer
    // only ever runs ATT_STAGES iterations ahead of the consumers, and the grid-level timeout
    // is reported through the status word.  Wait (bounded) for the full barriers of the last
    // iterations before the staging area is reused.
    timed_out = __syncthreads_or(timed_out);
    if (timed_out && !is_producer) {
        for (int it2 = max(0, n_iter - ATT_STAGES); it2 < n_iter; ++it2) {
            unsigned spins = 0;
            while (!mbar_try_wait(&full_bars[warp * ATT_STAGES + it2 % ATT_STAGES], (unsigned)(it2 / ATT_STAGES) & 1u)) {
                if (++spins > (WAIT_SPIN_LIMIT >> 4)) break;
            }
        }
    }

    // ---------------- un-scale the V accumulators of this quarter warp ----------------
    float o[DPL];
    {
        const float l_q = qw_sum(l_part, qmask);
        const float mn_q = qw_sum(mn_part, qmask);
#pragma unroll
        for (int wd = 0; wd < WPL; ++wd) {
            float a[8];
#pragma unroll
            for (int e = 0; e < 8; e += 2) { a[e] = acc[4 * wd + e / 2].x; a[e + 1] = acc[4 * wd + e / 2].y; }
            a[6] = fmaf(-16.f, a[7], a[6]);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[8 * wd + e] = fmaf(a[e], nib_unscale(e), mn_q);
        }
        l_part = l_q;
    }

    // ---------------- tail: dense attention over the staged (unquantised) tokens ----------------
    // Done by the CTA of split 0; warp w takes tail tokens w, w+WARPS, ...; lane owns D/32 channels.
    constexpr int TD = D / 32;
    float tm = -INFINITY, tl = 0.f, tacc[TD];
#pragma unroll
    for (int j = 0; j < TD; ++j) tacc[j] = 0.f;
    const int dyn_tail = DYN ? (pos_v + p.pos_new) % p.page : p.tail_len;
    if (split == 0 && dyn_tail > 0 && !is_producer) {
        float qt[TD];
        const QT* qp = static_cast<const QT*>(p.Q) + b * p.q_sb + hq * p.q_sh + TD * lane;
#pragma unroll
        for (int j = 0; j < TD; ++j) qt[j] = Dt<QT>::to_f32(qp[j]) * (p.sm_scale * LOG2E);
        for (int t = warp; t < dyn_tail; t += ATT_WARPS) {
            const int64_t ro = b * p.tl_sb + hkv * p.tl_sh + (int64_t)t * p.tl_ss + TD * lane;
            float kv[TD], vv[TD];
#pragma unroll
            for (int j = 0; j < TD; ++j) {
                if (p.tail_dtype == FQ_BF16) {
                    kv[j] = ld_as_f32<__nv_bfloat16>(p.K_tail, ro + j);
                    vv[j] = ld_as_f32<__nv_bfloat16>(p.V_tail, ro + j);
                } else {
                    kv[j] = ld_as_f32<__half>(p.K_tail, ro + j);
                    vv[j] = ld_as_f32<__half>(p.V_tail, ro + j);
                }
            }
            float sdt = 0.f;
#pragma unroll
            for (int j = 0; j < TD; ++j) sdt = fmaf(qt[j], kv[j], sdt);
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) sdt += __shfl_xor_sync(0xffffffffu, sdt, off);
            const float mnew = fmaxf(tm, sdt);
            const float al = ex2(tm - mnew);
            const float pr = ex2(sdt - mnew);
            tl = tl * al + pr;
#pragma unroll
            for (int j = 0; j < TD; ++j) tacc[j] = fmaf(pr, vv[j], tacc[j] * al);
            tm = mnew;
        }
    }

    // ---------------- CTA merge of all states through shared memory ----------------
    __syncthreads();   // every warp is done with the staging area (st_acc aliases it)
    if (!is_producer) {
        const int sid = warp * 4 + qw;
        if (l == 0) { st_m[sid] = m_run; st_l[sid] = l_part; }
#pragma unroll
        for (int j = 0; j < DPL; ++j) st_acc[sid * D + DPL * l + j] = o[j];
        const int tsid = ATT_WARPS * 4 + warp;
        if (lane == 0) { st_m[tsid] = tm; st_l[tsid] = tl; }
#pragma unroll
        for (int j = 0; j < TD; ++j) st_acc[tsid * D + TD * lane + j] = tacc[j];
    }
    __syncthreads();
    // warp 0 turns the per-state maxima into merge weights once; then thread d sums channel d
    static_assert(NSTATE <= 32, "one lane per state");
    __shared__ float s_mcta, s_lcta;
    if (warp == 0) {
        const float mi = lane < NSTATE ? st_m[lane] : -INFINITY;
        float mx = mi;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        const float wgt = (mx == -INFINITY) ? 0.f : ex2(mi - mx);   // 0 for empty states
        float lsum = lane < NSTATE ? st_l[lane] * wgt : 0.f;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
        if (lane < NSTATE) st_m[lane] = wgt;
        if (lane == 0) { s_mcta = mx; s_lcta = lsum; }
    }
    __syncthreads();
    const float m_cta = s_mcta, l_cta = s_lcta;
    float acc_d = 0.f;           // thread d < D owns output channel d
    if (tid < D) {
#pragma unroll
        for (int i = 0; i < NSTATE; ++i) acc_d = fmaf(st_acc[i * D + tid], st_m[i], acc_d);
    }

    QT* Op = static_cast<QT*>(p.O) + b * p.o_sb + hq * p.o_sh;
    const int row = b * p.Hq + hq;
    if (p.n_split == 1) {
        if (tid < D) Op[tid] = from_f32<QT>(l_cta > 0.f ? acc_d / l_cta : 0.f);
        if (tid == 0 && p.lse) p.lse[row] = l_cta > 0.f ? (m_cta + log2f(l_cta)) * LN2 : -INFINITY;
        return;
    }

    // ---------------- split-K: publish the partial, last ticket merges ----------------
    float* part = p.partials + ((int64_t)row * p.n_split + split) * (D + 2);
    if (tid < D) part[2 + tid] = acc_d;
    if (tid == 0) { part[0] = m_cta; part[1] = l_cta; }
    __syncthreads();           // the CTA's stores are ordered before thread 0's fence below
    __shared__ int s_ticket;
    if (tid == 0) {
        // one device-scope release + acquire per CTA, carried by the ticket itself (cumulative over the barrier above;
        // the barrier below hands what the last CTA acquired to its other threads)
        int t;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(t) : "l"(p.tickets + row) : "memory");
        s_ticket = t;
    }
    __syncthreads();
    if (s_ticket != p.n_split - 1) return;
    // The partials of this row are merged in split order with every load independent of the
    // others (a dependent chain of L2 round trips here would cost more than the attention).
    const float* parts = p.partials + (int64_t)row * p.n_split * (D + 2);
    float* mw = reinterpret_cast<float*>(smem);            // [n_split] max, then weight
    float* lw = mw + p.n_split;                             // [n_split] denominators
    __shared__ float s_red[ATT_WARPS + 1];
    constexpr int PRE = 20;    // partial accumulators requested up front, with the maxima
    float pre[PRE];
    if (tid < D) {
#pragma unroll
        for (int i = 0; i < PRE; ++i) pre[i] = i < p.n_split ? __ldcg(parts + (int64_t)i * (D + 2) + 2 + tid) : 0.f;
    }
    float m_loc = -INFINITY;
    for (int i = tid; i < p.n_split; i += ATT_THREADS) {
        const float mi = __ldcg(parts + (int64_t)i * (D + 2));
        mw[i] = mi;
        lw[i] = __ldcg(parts + (int64_t)i * (D + 2) + 1);
        m_loc = fmaxf(m_loc, mi);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) m_loc = fmaxf(m_loc, __shfl_xor_sync(0xffffffffu, m_loc, off));
    if (lane == 0) s_red[warp] = m_loc;
    __syncthreads();
    float m_all = s_red[0];
#pragma unroll
    for (int w = 1; w < ATT_WARPS + 1; ++w) m_all = fmaxf(m_all, s_red[w]);
    float l_all = 0.f, o_all = 0.f;
    if (m_all != -INFINITY) {
        for (int i = tid; i < p.n_split; i += ATT_THREADS) mw[i] = ex2(mw[i] - m_all);
        __syncthreads();
        for (int i = 0; i < p.n_split; ++i) l_all = fmaf(lw[i], mw[i], l_all);
        if (tid < D) {
            const float* col = parts + 2 + tid;
#pragma unroll
            for (int i = 0; i < PRE; ++i) o_all = fmaf(pre[i], i < p.n_split ? mw[i] : 0.f, o_all);
            int i = PRE;
            for (; i + 8 <= p.n_split; i += 8) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = __ldcg(col + (int64_t)(i + j) * (D + 2));
#pragma unroll
                for (int j = 0; j < 8; ++j) o_all = fmaf(v[j], mw[i + j], o_all);
            }
            for (; i < p.n_split; ++i) o_all = fmaf(__ldcg(col + (int64_t)i * (D + 2)), mw[i], o_all);
        }
    }
    if (tid < D) Op[tid] = from_f32<QT>(l_all > 0.f ? o_all / l_all : 0.f);
    if (tid == 0) {
        if (p.lse) p.lse[row] = l_all > 0.f ? (m_all + log2f(l_all)) * LN2 : -INFINITY;
        p.tickets[row] = 0;   // leave the workspace ready for the next call
    }
}

template <int D, int TOK>
static constexpr size_t attn_smem_bytes() {
    using L = UnitLayout<D, TOK>;
    constexpr int NSTATE = ATT_WARPS * 4 + ATT_WARPS;
    size_t staging = (size_t)ATT_STAGES * ATT_WARPS * 4 * L::STRIDE;
    size_t merge = (size_t)NSTATE * D * 4;
    size_t front = staging > merge ? staging : merge;
    return front + 2 * ATT_WARPS * ATT_STAGES * 8 + (size_t)ATT_WARPS * 4 * TOK * 4 + 2 * NSTATE * 4;
}

template <typename QT, int D, int TOK, bool DYN>
static int launch_attn_impl(const AttnParams& p, cudaStream_t st) {
    constexpr size_t smem = attn_smem_bytes<D, TOK>();
    static_assert((size_t)ATT_STAGES * ATT_WARPS * 4 * UnitLayout<D, TOK>::STRIDE >=
                  (size_t)(ATT_WARPS * 5) * D * 4, "merge area must fit in the staging area");
    auto kern = sparse_decode_int4_kernel<QT, D, TOK, DYN>;
    constexpr int MAX_DEV = 64;
    static std::atomic<bool> prepared[MAX_DEV];     // relaxed: concurrent host threads may repeat the idempotent set-up
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return fail(FQ_ERR_CUDA, "fq_sparse_decode_int4: cannot identify the current device");
    if (!prepared[dev].load(std::memory_order_relaxed)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "fq_sparse_decode_int4: cannot reserve %zu B of shared memory: %s", smem, cudaGetErrorString(e));
        prepared[dev].store(true, std::memory_order_relaxed);
    }
    dim3 grid((unsigned)p.n_split, (unsigned)p.Hq, (unsigned)p.B);
    cudaError_t e = launch_k(PDL_ATTN, kern, grid, dim3(ATT_THREADS), smem, st, p);
    if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "fq_sparse_decode_int4: launch failed: %s", cudaGetErrorString(e));
    return FQ_OK;
}

template <typename QT, int D, int TOK>
static int launch_attn(const AttnParams& p, cudaStream_t st) {
    return p.pos ? launch_attn_impl<QT, D, TOK, true>(p, st) : launch_attn_impl<QT, D, TOK, false>(p, st);
}

}  // namespace fq


extern "C" size_t fq_sparse_decode_workspace_bytes(int B, int Hq, int D, int n_split) {
    if (B <= 0 || Hq <= 0 || D <= 0 || n_split <= 1) return 0;
    size_t tickets = ((size_t)B * Hq * 4 + 255) & ~(size_t)255;
    return tickets + (size_t)B * Hq * n_split * (D + 2) * 4;
}

extern "C" int fq_sparse_decode_default_splits(int B, int Hq, int bucket, int page) {
    if (B <= 0 || Hq <= 0 || bucket <= 0 || page <= 0) return 1;
    const int tok = page >= 16 ? 16 : 8;
    const long cpp = page / tok;
    const long units = (long)bucket * cpp;
    const long rows = (long)B * Hq;
    const long per_iter = fq::ATT_WARPS * 4;
    const long total_iters = (units + per_iter - 1) / per_iter;    // per row
    // All CTAs resident at once (148 SMs x ATT_CTAS_PER_SM): the producers then request the
    // first STAGES iterations of every CTA immediately and the memory latency is paid once.
    const long slots = 148L * fq::ATT_CTAS_PER_SM;
    long n_split = slots / rows;
    if (n_split < 1) n_split = 1;
    // One wave that leaves more than 7 % of the slots empty (e.g. 384 rows on 444 slots) finishes when the fullest
    // SMs do while the others idle.  Three times as many, shorter CTAs are handed out as slots free up and keep every
    // SM busy to the end -- worth it while a CTA still has 8 iterations to amortise its start and its merge over
    // (measured at 16 x 24 rows: 113 against 121 us; at 24 rows the single full wave stays).
    if (rows * n_split * 100 < slots * 93 && total_iters >= 3 * n_split * 8) n_split *= 3;
    if (n_split > total_iters) n_split = total_iters;
    if (n_split > bucket) n_split = bucket;
    if (n_split < 1) n_split = 1;
    if (n_split > 1024) n_split = 1024;
    return (int)n_split;
}

namespace fq {
int sparse_decode_int4_launch(
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
    void* workspace, size_t workspace_bytes, int n_split, void* stream, const DynPos& dp, const int32_t* list_count) {
    const char* fn = "fq_sparse_decode_int4";
    FQ_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && S_kv >= 0 && P >= 0 && bucket >= 0 && tail_len >= 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(B <= 65535 && Hq <= 65535, FQ_ERR_ARG, "%s: B and H_q must be <= 65535", fn);
    FQ_CHECK_ARG(Hq % Hkv == 0, FQ_ERR_ARG, "%s: H_q=%d must be divisible by H_kv=%d", fn, Hq, Hkv);
    FQ_CHECK_ARG(D == 64 || D == 128, FQ_ERR_UNSUPPORTED, "%s: head_dim=%d not in (64, 128)", fn, D);
    FQ_CHECK_ARG(page == 8 || page == 16 || page == 32 || page == 64 || page == 128, FQ_ERR_UNSUPPORTED,
                 "%s: page_size=%d not in (8, 16, 32, 64, 128)", fn, page);
    FQ_CHECK_ARG(q_dtype == FQ_F16 || q_dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: Q must be fp16 or bf16 (code %d)", fn, q_dtype);
    FQ_CHECK_ARG(Q && O, FQ_ERR_ARG, "%s: null Q or O", fn);
    FQ_CHECK_ARG(n_split >= 1 && n_split <= 1024, FQ_ERR_ARG, "%s: n_split=%d must be in [1, 1024]", fn, n_split);
    const bool have_pages = bucket > 0 && P > 0 && S_kv > 0;
    if (have_pages) {
        FQ_CHECK_ARG(K_packed && V_packed && K_scale && K_mn && V_scale && V_mn && compact, FQ_ERR_ARG, "%s: null cache pointer", fn);
        FQ_CHECK_ARG((int64_t)P * page >= S_kv, FQ_ERR_ARG, "%s: %d pages of %d tokens do not cover S_kv=%d", fn, P, page, S_kv);
        FQ_CHECK_ARG(aligned(K_packed, 16) && aligned(V_packed, 16) && kp_sb % 16 == 0 && kp_sh % 16 == 0 && vp_sb % 16 == 0 && vp_sh % 16 == 0,
                     FQ_ERR_ALIGN, "%s: packed K/V (b,h) slabs must be 16-byte aligned", fn);
        FQ_CHECK_ARG(aligned(K_scale, 16) && aligned(K_mn, 16) && km_sb % 8 == 0 && km_sh % 8 == 0 && km_sp % 8 == 0,
                     FQ_ERR_ALIGN, "%s: K metadata rows must be 16-byte aligned", fn);
        FQ_CHECK_ARG(aligned(V_scale, 16) && aligned(V_mn, 16) && vm_sb % 8 == 0 && vm_sh % 8 == 0,
                     FQ_ERR_ALIGN, "%s: V metadata (b,h) rows must be 16-byte aligned", fn);
    }
    if (tail_len > 0) {
        FQ_CHECK_ARG(K_tail && V_tail, FQ_ERR_ARG, "%s: null tail pointer", fn);
        FQ_CHECK_ARG(tail_dtype == FQ_F16 || tail_dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: tail must be fp16 or bf16", fn);
    }
    const int64_t qa = 8;
    FQ_CHECK_ARG(aligned(Q, 16) && q_sb % qa == 0 && q_sh % qa == 0, FQ_ERR_ALIGN, "%s: Q rows must be 16-byte aligned", fn);

    AttnParams p;
    p.Q = Q; p.q_sb = q_sb; p.q_sh = q_sh;
    p.K_packed = K_packed; p.kp_sb = kp_sb; p.kp_sh = kp_sh;
    p.K_scale = static_cast<const uint16_t*>(K_scale); p.K_mn = static_cast<const uint16_t*>(K_mn);
    p.km_sb = km_sb; p.km_sh = km_sh; p.km_sp = km_sp;
    p.V_packed = V_packed; p.vp_sb = vp_sb; p.vp_sh = vp_sh;
    p.V_scale = static_cast<const uint16_t*>(V_scale); p.V_mn = static_cast<const uint16_t*>(V_mn);
    p.vm_sb = vm_sb; p.vm_sh = vm_sh;
    p.compact = compact; p.cp_sb = cp_sb; p.cp_sh = cp_sh; p.bucket = have_pages ? bucket : 0;
    p.list_count = list_count;
    p.K_tail = K_tail; p.V_tail = V_tail; p.tail_dtype = tail_dtype; p.tl_sb = tl_sb; p.tl_sh = tl_sh; p.tl_ss = tl_ss;
    p.tail_len = tail_len;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.S_kv = S_kv; p.P = P; p.page = page;
    {
        const int cpp = page >= 16 ? page / 16 : 1;
        p.cpp_log2 = 0;
        while ((1 << p.cpp_log2) < cpp) ++p.cpp_log2;
    }
    p.sm_scale = sm_scale;
    p.O = O; p.o_sb = o_sb; p.o_sh = o_sh; p.lse = lse;
    if (n_split > p.bucket) n_split = p.bucket > 0 ? p.bucket : 1;
    p.n_split = n_split;
    p.tickets = nullptr; p.partials = nullptr;
    p.pos = dp.pos; p.pos_new = dp.n_new; p.pos_early = dp.early ? 1 : 0;
    p.status = device_status_ptr();
    if (p.status == nullptr) return FQ_ERR_CUDA;
    if (n_split > 1) {
        const size_t need = fq_sparse_decode_workspace_bytes(B, Hq, D, n_split);
        FQ_CHECK_ARG(workspace && workspace_bytes >= need, FQ_ERR_WORKSPACE, "%s: workspace of %zu B needed, %zu given", fn, need, workspace_bytes);
        FQ_CHECK_ARG(aligned(workspace, 16), FQ_ERR_ALIGN, "%s: workspace must be 16-byte aligned", fn);
        p.tickets = static_cast<int*>(workspace);
        p.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + (((size_t)B * Hq * 4 + 255) & ~(size_t)255));
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc;
    const bool tok8 = page == 8;
#define FQ_ATT(QT)                                                              \
    (D == 128 ? (tok8 ? launch_attn<QT, 128, 8>(p, st) : launch_attn<QT, 128, 16>(p, st)) \
              : (tok8 ? launch_attn<QT, 64, 8>(p, st) : launch_attn<QT, 64, 16>(p, st)))
    if (q_dtype == FQ_F16) rc = FQ_ATT(__half);
    else rc = FQ_ATT(__nv_bfloat16);
#undef FQ_ATT
    if (rc != FQ_OK) return rc;
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}
}  // namespace fq

extern "C" int fq_sparse_decode_int4(
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
    void* workspace, size_t workspace_bytes, int n_split, void* stream) {
    return fq::sparse_decode_int4_launch(
        Q, q_dtype, q_sb, q_sh, K_packed, kp_sb, kp_sh, K_scale, K_mn, km_sb, km_sh, km_sp,
        V_packed, vp_sb, vp_sh, V_scale, V_mn, vm_sb, vm_sh, compact, cp_sb, cp_sh, bucket,
        K_tail, V_tail, tail_dtype, tl_sb, tl_sh, tl_ss, tail_len,
        B, Hq, Hkv, S_kv, P, D, page, sm_scale, O, o_sb, o_sh, lse,
        workspace, workspace_bytes, n_split, stream, fq::DynPos{});
}

extern "C" int fq_sparse_decode_int4_counted(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_packed, int64_t kp_sb, int64_t kp_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const uint8_t* V_packed, int64_t vp_sb, int64_t vp_sh,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket, const int32_t* list_count,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss, int tail_len,
    int B, int Hq, int Hkv, int S_kv, int P, int D, int page, float sm_scale,
    void* O, int64_t o_sb, int64_t o_sh, float* lse,
    void* workspace, size_t workspace_bytes, int n_split, void* stream) {
    return fq::sparse_decode_int4_launch(
        Q, q_dtype, q_sb, q_sh, K_packed, kp_sb, kp_sh, K_scale, K_mn, km_sb, km_sh, km_sp,
        V_packed, vp_sb, vp_sh, V_scale, V_mn, vm_sb, vm_sh, compact, cp_sb, cp_sh, bucket,
        K_tail, V_tail, tail_dtype, tl_sb, tl_sh, tl_ss, tail_len,
        B, Hq, Hkv, S_kv, P, D, page, sm_scale, O, o_sb, o_sh, lse,
        workspace, workspace_bytes, n_split, stream, fq::DynPos{}, list_count);
}

namespace fq {

// ---------------------------------------------------------------------------------------
// Split-K attention for callers that cannot hand over a workspace.
//
// Some hosts of this library have no way to obtain device memory at the point where they
// call it: a binding from a runtime that owns no CUDA allocator, a serving loop that must
// not touch cudaMalloc/cudaFree because those calls synchronise the whole device, a plugin
// that is only given its inputs and outputs.  For them the split-K scratch (tickets +
// per-split partial results) lives in this fixed array, which every GPU that loads the
// library carries from load until the process exits.
constexpr size_t FQ_STATIC_SCRATCH_BYTES = FQ_SPARSE_DECODE_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[FQ_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device.  In host code the array's name
// is only a handle for the runtime, not a device pointer, so the address is looked up once
// per device (with that device current) and remembered (relaxed atomics: concurrent host threads
// may race to store the same value).  After a cudaDeviceReset() in the host process the
// remembered address is stale: reload the library in that case.
static void* static_scratch_ptr() {
    constexpr int MAX_DEV = 64;
    static std::atomic<void*> ptrs[MAX_DEV];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEV) {
        set_error("fq_sparse_decode_int4_static: cannot identify the current device");
        return nullptr;
    }
    void* ptr = ptrs[dev].load(std::memory_order_relaxed);
    if (ptr == nullptr) {
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            set_error("fq_sparse_decode_int4_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        ptrs[dev].store(ptr, std::memory_order_relaxed);
    }
    return ptr;
}

}  // namespace fq

extern "C" int fq_sparse_decode_int4_static(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_packed, int64_t kp_sb, int64_t kp_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const uint8_t* V_packed, int64_t vp_sb, int64_t vp_sh,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss,
    int tail_len,
    int B, int Hq, int Hkv, int S_kv, int P, int D, int page, float sm_scale,
    void* O, int64_t o_sb, int64_t o_sh, float* lse, int n_split, void* stream) {
    using namespace fq;
    const char* fn = "fq_sparse_decode_int4_static";
    FQ_CHECK_ARG(B > 0 && Hq > 0 && D > 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    if (n_split <= 0) n_split = fq_sparse_decode_default_splits(B, Hq, bucket, page);
    FQ_CHECK_ARG(n_split <= 1024, FQ_ERR_ARG, "%s: n_split=%d must be at most 1024", fn, n_split);
    const size_t need = fq_sparse_decode_workspace_bytes(B, Hq, D, n_split);
    FQ_CHECK_ARG(need <= FQ_STATIC_SCRATCH_BYTES, FQ_ERR_WORKSPACE,
                 "%s: B=%d x H_q=%d x n_split=%d x head_dim=%d needs %zu B of scratch, the built-in array holds %zu B; "
                 "lower n_split or use fq_sparse_decode_int4 with a workspace of your own",
                 fn, B, Hq, n_split, D, need, (size_t)FQ_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    if (n_split > 1) {
        scratch = static_scratch_ptr();
        if (scratch == nullptr) return FQ_ERR_CUDA;
        // The array keeps whatever the previous call left in it; the per-row ticket words are
        // the only part the kernel needs to find at zero.
        const size_t tickets = ((size_t)B * Hq * 4 + 255) & ~(size_t)255;
        cudaError_t e = cudaMemsetAsync(scratch, 0, tickets, static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: clearing the tickets failed: %s", fn, cudaGetErrorString(e));
    }
    return fq_sparse_decode_int4(
        Q, q_dtype, q_sb, q_sh, K_packed, kp_sb, kp_sh, K_scale, K_mn, km_sb, km_sh, km_sp,
        V_packed, vp_sb, vp_sh, V_scale, V_mn, vm_sb, vm_sh, compact, cp_sb, cp_sh, bucket,
        K_tail, V_tail, tail_dtype, tl_sb, tl_sh, tl_ss, tail_len,
        B, Hq, Hkv, S_kv, P, D, page, sm_scale, O, o_sb, o_sh, lse,
        scratch, n_split > 1 ? (size_t)FQ_STATIC_SCRATCH_BYTES : 0, n_split, stream);
}
