// Sparse decode attention over TurboQuant K3-V3 bit planes, in the rotated basis, and the
// n-way LSE merge of partial attention results.
//
// Per selected 16-token unit the kernel reads 16 x (D/8 + D/4 + 2) bytes for K and the same
// for V (1600 B at D = 128).  One warp owns one unit at a time and stages the next one into
// its own double buffer with cp.async while it works.  A lane owns 8 channels (one byte of
// the msb plane, two of the lsb plane) of every NTP-th token.  Decoding is a table look-up:
// two neighbouring channels form a 6-bit index (2 msb bits, 4 lsb bits) into a table of
// codebook PAIRS, replicated per lane so that a warp's 64-bit loads never collide; one
// fma.rn.f32x2 then covers both channels (K: times the q pair, V: times the softmax weight).
// Per-token dot products meet in a transposing shuffle reduction; softmax in base 2, fp32
// accumulation, split-K partials merged by the CTA that draws the last ticket of its row (no
// CTA waits for another).  Bound by the ALU/LSU work of the index assembly and look-ups
// (about 3 instructions per 3-bit element), not by HBM.
#include <atomic>

#include "fq_common.cuh"

namespace fq {

constexpr int TQ_WARPS = 8;
constexpr int TQ_THREADS = TQ_WARPS * 32;
constexpr int TQ_LIST_MAX = 4096;        // page-list entries a CTA packs in shared memory
constexpr float TQ_LOG2E = 1.4426950408889634f;
constexpr float TQ_LN2 = 0.6931471805599453f;

struct TurboAttnParams {
    const void* Q; int64_t q_sb, q_sh;                     // rotated Q (B,Hq,D)
    const uint8_t *K_msb, *K_lsb, *V_msb, *V_lsb;
    int64_t km_sb, km_sh, km_ss, kl_sb, kl_sh, kl_ss, vm_sb, vm_sh, vm_ss, vl_sb, vl_sh, vl_ss;
    const uint16_t *K_scale, *V_scale; int64_t ks_sb, ks_sh, vs_sb, vs_sh;   // (B,Hkv,S) bf16, token stride 1
    const int32_t* compact; int64_t cp_sb, cp_sh; int bucket;
    int B, Hq, Hkv, S_kv, P, page;
    float sm_scale;
    void* O; int64_t o_sb, o_sh; float* lse;
    int* tickets; float* partials; int n_split;
    int fast;            // planes are token-contiguous and 16-byte aligned: 16-byte async copies
};

__device__ __forceinline__ float tq_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// shared-memory loads through 32-bit shared-window addresses (one integer add per address)
__device__ __forceinline__ float2 tq_lds_f2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t tq_lds_u8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t tq_lds_u16(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void tq_cp16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}

// Transposing reduction of N partial sums per lane over the L lanes (L = 2N) that share a
// token group: afterwards lane c holds the complete sum of value index c >> 1 in s[0].
template <int N, int L>
__device__ __forceinline__ void tq_reduce(float (&s)[N], int c) {
    static_assert(L == 2 * N, "lanes per token");
    if constexpr (N >= 8) {
        const bool up = c & (L / 2);
#pragma unroll
        for (int i = 0; i < 4; ++i) s[i] = (up ? s[i + 4] : s[i]) + __shfl_xor_sync(0xffffffffu, up ? s[i] : s[i + 4], L / 2);
    }
    if constexpr (N >= 4) {
        constexpr int H = N >= 8 ? L / 4 : L / 2;
        const bool up = c & H;
#pragma unroll
        for (int i = 0; i < 2; ++i) s[i] = (up ? s[i + 2] : s[i]) + __shfl_xor_sync(0xffffffffu, up ? s[i] : s[i + 2], H);
    }
    {
        const bool up = c & 2;
        s[0] = (up ? s[1] : s[0]) + __shfl_xor_sync(0xffffffffu, up ? s[0] : s[1], 2);
    }
    s[0] += __shfl_xor_sync(0xffffffffu, s[0], 1);
}

template <typename QT, int D>
__global__ void __launch_bounds__(TQ_THREADS, 3) sparse_decode_turbo_kernel(TurboAttnParams p) {
    constexpr int TOK = 16;
    constexpr int LPT = D / 8;           // lanes per token, 8 channels each
    constexpr int NTP = 32 / LPT;        // tokens a warp works on at once
    constexpr int TPL = TOK / NTP;       // tokens per lane
    constexpr int MROW = D / 8, LROW = D / 4;
    constexpr int KM_OFF = 0, KL_OFF = TOK * MROW, VM_OFF = KL_OFF + TOK * LROW, VL_OFF = VM_OFF + TOK * MROW;
    constexpr int UNIT_BYTES = VL_OFF + TOK * LROW;
    static_assert(TPL * 2 == LPT, "the reduction leaves one token per lane pair");
    __shared__ __align__(16) float2 s_lut[64 * 32];                       // [pair index][lane]
    __shared__ __align__(16) unsigned char s_stage[TQ_WARPS][2][UNIT_BYTES];
    __shared__ float s_m[TQ_WARPS], s_l[TQ_WARPS], s_acc[TQ_WARPS][D];
    __shared__ int s_ticket;
    extern __shared__ int s_pages[];                                       // the row's valid pages: min(bucket, TQ_LIST_MAX) entries, or none
    __shared__ int s_cnt[TQ_WARPS];

    const int split = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
    const int n_rep = p.Hq / p.Hkv, hkv = hq / n_rep;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tp = lane / LPT, c = lane % LPT;
    {
        const float cb[8] = {-2.1519f, -1.3439f, -0.7560f, -0.2451f, 0.2451f, 0.7560f, 1.3439f, 2.1519f};
        // pair index = (msb_b msb_a) << 4 | (lsb_b << 2) | lsb_a for the channels a (even) and b = a + 1
        for (int i = tid; i < 64 * 32; i += TQ_THREADS) {
            const int e = i >> 5;
            const int ia = (((e >> 4) & 1) << 2) | (e & 3), ib = (((e >> 5) & 1) << 2) | ((e >> 2) & 3);
            float va = 0.f, vb = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) { va = ia == k ? cb[k] : va; vb = ib == k ? cb[k] : vb; }
            s_lut[i] = make_float2(va, vb);
        }
    }
    __syncthreads();
    pdl_wait();        // the rotated Q and the page list come from the kernels before this one
    pdl_trigger();
    const uint32_t lut_addr = (uint32_t)__cvta_generic_to_shared(s_lut) + lane * 8;      // this lane's column of the table

    float2 q2[4];      // this lane's 8 channels of q * sm_scale * log2(e)
    {
        const QT* qp = static_cast<const QT*>(p.Q) + b * p.q_sb + hq * p.q_sh + 8 * c;
        const float sc = p.sm_scale * TQ_LOG2E;
#pragma unroll
        for (int j = 0; j < 4; ++j) q2[j] = make_float2(Dt<QT>::to_f32(qp[2 * j]) * sc, Dt<QT>::to_f32(qp[2 * j + 1]) * sc);
    }

    // A list made from a selection mask is as wide as the page count and mostly padding.  Every CTA of a row
    // therefore first packs the row's valid entries, in their order, into shared memory (a warp per contiguous
    // eighth of the list: 16 independent loads per lane, ballots, one exchange of the warps' counts); the walk below
    // then meets real pages only.  Lists wider than TQ_LIST_MAX are walked as they are, padding skipped per unit.
    const int32_t* list = p.compact + b * p.cp_sb + hq * p.cp_sh;
    const bool packed = p.bucket <= TQ_LIST_MAX;
    int n_entries = p.bucket;
    if (packed) {
        constexpr int PER_LANE = TQ_LIST_MAX / TQ_THREADS;
        const int seg = (p.bucket + TQ_WARPS - 1) / TQ_WARPS;
        const int e_begin = warp * seg, e_end = min(p.bucket, e_begin + seg);
        int pg[PER_LANE], pos[PER_LANE];
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int e = e_begin + i * 32 + lane;
            pg[i] = e < e_end ? __ldg(list + e) : -1;
        }
        int cnt = 0;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const bool ok = pg[i] >= 0 && pg[i] < p.P && (int64_t)pg[i] * p.page < p.S_kv;
            const unsigned bal = __ballot_sync(0xffffffffu, ok);
            pos[i] = ok ? cnt + __popc(bal & ((1u << lane) - 1u)) : -1;
            cnt += __popc(bal);
        }
        if (lane == 0) s_cnt[warp] = cnt;
        __syncthreads();
        int off = 0, tot = 0;
#pragma unroll
        for (int w = 0; w < TQ_WARPS; ++w) { const int n = s_cnt[w]; off += w < warp ? n : 0; tot += n; }
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i)
            if (pos[i] >= 0) s_pages[off + pos[i]] = pg[i];
        __syncthreads();
        n_entries = tot;
    }
    // Units are dealt round-robin to the splits (unit g belongs to split g % n_split).
    const int cpp = p.page / TOK;
    const int total_units = n_entries * cpp;
    const int n_units = split < total_units ? (total_units - split + p.n_split - 1) / p.n_split : 0;   // of this CTA

    const uint8_t* Kmsb = p.K_msb + b * p.km_sb + hkv * p.km_sh;
    const uint8_t* Klsb = p.K_lsb + b * p.kl_sb + hkv * p.kl_sh;
    const uint8_t* Vmsb = p.V_msb + b * p.vm_sb + hkv * p.vm_sh;
    const uint8_t* Vlsb = p.V_lsb + b * p.vl_sb + hkv * p.vl_sh;
    const uint16_t* Ksc = p.K_scale + b * p.ks_sb + hkv * p.ks_sh;
    const uint16_t* Vsc = p.V_scale + b * p.vs_sb + hkv * p.vs_sh;

    const int t_mine = NTP * (c >> 1) + tp;      // the token whose logit ends up in this lane

    // unit -> first token and number of valid tokens (0: nothing to do)
    // page id of this warp's unit u (-1 past the end); requested two units ahead of its use
    const int cpp_shift = (cpp & (cpp - 1)) == 0 ? __ffs(cpp) - 1 : -1;      // units per page as a shift, where it is one
    auto page_of = [&](int u) -> int {
        const int g = u * p.n_split + split;
        if (u >= n_units) return -1;
        const int e = cpp_shift >= 0 ? g >> cpp_shift : g / cpp;
        return packed ? s_pages[e] : __ldg(list + e);
    };
    auto locate = [&](int u, int pg, int& tok0, int& n_tok) {
        tok0 = 0; n_tok = 0;
        if (pg < 0 || pg >= p.P) return;
        const int g = u * p.n_split + split;
        tok0 = pg * p.page + (cpp_shift >= 0 ? g & (cpp - 1) : g % cpp) * TOK;
        n_tok = max(0, min(TOK, p.S_kv - tok0));
    };
    // this lane's three 16-byte pieces of a full unit: plane, offset inside the unit, bytes per token
    const uint8_t* piece_src[3];
    int piece_dst[3], piece_row[3];
    {
        constexpr int CM = TOK * MROW / 16, CL = TOK * LROW / 16;
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const int i = lane + 32 * r;
            if (i < CM) { piece_src[r] = Kmsb + 16 * i; piece_dst[r] = KM_OFF + 16 * i; piece_row[r] = MROW; }
            else if (i < CM + CL) { piece_src[r] = Klsb + 16 * (i - CM); piece_dst[r] = KL_OFF + 16 * (i - CM); piece_row[r] = LROW; }
            else if (i < 2 * CM + CL) { piece_src[r] = Vmsb + 16 * (i - CM - CL); piece_dst[r] = VM_OFF + 16 * (i - CM - CL); piece_row[r] = MROW; }
            else if (i < 2 * (CM + CL)) { piece_src[r] = Vlsb + 16 * (i - 2 * CM - CL); piece_dst[r] = VL_OFF + 16 * (i - 2 * CM - CL); piece_row[r] = LROW; }
            else { piece_src[r] = nullptr; piece_dst[r] = 0; piece_row[r] = 0; }
        }
        static_assert(2 * (CM + CL) <= 96, "three pieces per lane cover a unit");
    }
    // bring a unit into a staging buffer; scales of this lane's token come back in registers
    auto stage = [&](unsigned char* buf, int tok0, int n_tok, float& ks, float& vs) {
        ks = 0.f; vs = 0.f;
        if (n_tok <= 0) return;
        if (t_mine < n_tok) { ks = bf16_lo(__ldg(Ksc + tok0 + t_mine)); vs = bf16_lo(__ldg(Vsc + tok0 + t_mine)); }
        if (p.fast && n_tok == TOK) {
#pragma unroll
            for (int r = 0; r < 3; ++r)
                if (piece_src[r]) tq_cp16(buf + piece_dst[r], piece_src[r] + (int64_t)tok0 * piece_row[r]);
        } else {
            // ragged last unit or strided planes: byte copies of the valid tokens only
            for (int i = lane; i < n_tok * MROW; i += 32) {
                const int t = i / MROW, x = i % MROW;
                buf[KM_OFF + i] = Kmsb[(int64_t)(tok0 + t) * p.km_ss + x];
                buf[VM_OFF + i] = Vmsb[(int64_t)(tok0 + t) * p.vm_ss + x];
            }
            for (int i = lane; i < n_tok * LROW; i += 32) {
                const int t = i / LROW, x = i % LROW;
                buf[KL_OFF + i] = Klsb[(int64_t)(tok0 + t) * p.kl_ss + x];
                buf[VL_OFF + i] = Vlsb[(int64_t)(tok0 + t) * p.vl_ss + x];
            }
        }
    };
    // codebook pair of channels (2j, 2j+1) of this lane from the raw plane bytes: mask, then shift-and-add
    auto pair_at = [&](uint32_t M, uint32_t L, int j) -> float2 {
        const uint32_t a = lut_addr + ((M & (3u << (2 * j))) << (12 - 2 * j));
        const uint32_t b = j < 2 ? ((L & (15u << (4 * j))) << (8 - 4 * j)) : j == 2 ? (L & 0x0f00u) : ((L >> 4) & 0x0f00u);
        return tq_lds_f2(a + b);
    };

    float m_run = -INFINITY, l_run = 0.f;
    float2 acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = make_float2(0.f, 0.f);

    int cur_tok0 = 0, cur_n = 0;
    float cur_ks = 0.f, cur_vs = 0.f;
    int pg_nxt = page_of(warp + TQ_WARPS);               // page of the unit after the first one
    if (warp < n_units) {
        locate(warp, page_of(warp), cur_tok0, cur_n);
        stage(s_stage[warp][0], cur_tok0, cur_n, cur_ks, cur_vs);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    int it = 0;
    for (int u = warp; u < n_units; u += TQ_WARPS, ++it) {
        int nxt_tok0 = 0, nxt_n = 0;
        float nxt_ks = 0.f, nxt_vs = 0.f;
        const int pg_nxt2 = page_of(u + 2 * TQ_WARPS);   // in flight while this unit is worked on
        if (u + TQ_WARPS < n_units) {
            locate(u + TQ_WARPS, pg_nxt, nxt_tok0, nxt_n);
            stage(s_stage[warp][(it + 1) & 1], nxt_tok0, nxt_n, nxt_ks, nxt_vs);
        }
        pg_nxt = pg_nxt2;
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncwarp();
        if (cur_n > 0) {                                   // warp-uniform
            const uint32_t buf = (uint32_t)__cvta_generic_to_shared(s_stage[warp][it & 1]);
            // plane bytes of this lane's tokens, K and V, are requested before the first look-up depends on one
            // of them: their latencies overlap each other and the V planes arrive during the softmax
            const uint32_t row_m = buf + tp * MROW + c, row_l = buf + tp * LROW + 2 * c;
            uint32_t Mk[TPL], Lk[TPL], Mv[TPL], Lv[TPL];
#pragma unroll
            for (int k = 0; k < TPL; ++k) {
                Mk[k] = tq_lds_u8(row_m + KM_OFF + NTP * k * MROW);
                Lk[k] = tq_lds_u16(row_l + KL_OFF + NTP * k * LROW);
            }
#pragma unroll
            for (int k = 0; k < TPL; ++k) {
                Mv[k] = tq_lds_u8(row_m + VM_OFF + NTP * k * MROW);
                Lv[k] = tq_lds_u16(row_l + VL_OFF + NTP * k * LROW);
            }
            // ---------------- K ----------------
            float dots[TPL];
#pragma unroll
            for (int k = 0; k < TPL; ++k) {
                float2 a = make_float2(0.f, 0.f);
#pragma unroll
                for (int j = 0; j < 4; ++j) a = __ffma2_rn(pair_at(Mk[k], Lk[k], j), q2[j], a);
                dots[k] = a.x + a.y;
            }
            tq_reduce<TPL, LPT>(dots, c);
            const bool valid = t_mine < cur_n;
            const float x = valid ? dots[0] * cur_ks : -INFINITY;
            float pmax = x;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) pmax = fmaxf(pmax, __shfl_xor_sync(0xffffffffu, pmax, off));
            const float m_new = fmaxf(m_run, pmax);            // finite: the unit has a valid token
            const float alpha = tq_ex2(m_run - m_new);
            const float pr = valid ? tq_ex2(x - m_new) : 0.f;
            float psum = (c & 1) ? 0.f : pr;                   // every token sits in two lanes
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
            l_run = l_run * alpha + psum;
            m_run = m_new;
            const float pv_mine = pr * cur_vs;
            // ---------------- V ----------------
            const float2 al2 = make_float2(alpha, alpha);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = __fmul2_rn(acc[j], al2);
#pragma unroll
            for (int k = 0; k < TPL; ++k) {
                const float pv = __shfl_sync(0xffffffffu, pv_mine, tp * LPT + 2 * k);
                const float2 pv2 = make_float2(pv, pv);
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] = __ffma2_rn(pair_at(Mv[k], Lv[k], j), pv2, acc[j]);
            }
        }
        __syncwarp();                                      // the buffer is refilled in the next iteration
        cur_tok0 = nxt_tok0; cur_n = nxt_n; cur_ks = nxt_ks; cur_vs = nxt_vs;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---------------- CTA merge ----------------
    // the token phases of a warp hold partial sums of the same channels
#pragma unroll
    for (int off = LPT; off < 32; off <<= 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[j].x += __shfl_xor_sync(0xffffffffu, acc[j].x, off);
            acc[j].y += __shfl_xor_sync(0xffffffffu, acc[j].y, off);
        }
    }
    if (lane == 0) { s_m[warp] = m_run; s_l[warp] = l_run; }
    if (tp == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) { s_acc[warp][8 * c + 2 * j] = acc[j].x; s_acc[warp][8 * c + 2 * j + 1] = acc[j].y; }
    }
    __syncthreads();
    constexpr int NSTATE = TQ_WARPS;
    float m_cta = -INFINITY;
#pragma unroll
    for (int i = 0; i < NSTATE; ++i) m_cta = fmaxf(m_cta, s_m[i]);
    float l_cta = 0.f, acc_d = 0.f;
    if (m_cta != -INFINITY) {
#pragma unroll
        for (int i = 0; i < NSTATE; ++i) {
            const float w = tq_ex2(s_m[i] - m_cta);
            l_cta = fmaf(s_l[i], w, l_cta);
            if (tid < D) acc_d = fmaf(s_acc[i][tid], w, acc_d);
        }
    }
    QT* Op = static_cast<QT*>(p.O) + b * p.o_sb + hq * p.o_sh;
    const int row = b * p.Hq + hq;
    if (p.n_split == 1) {
        if (tid < D) Op[tid] = from_f32<QT>(l_cta > 0.f ? acc_d / l_cta : 0.f);
        if (tid == 0 && p.lse) p.lse[row] = l_cta > 0.f ? (m_cta + log2f(l_cta)) * TQ_LN2 : -INFINITY;
        return;
    }
    float* part = p.partials + ((int64_t)row * p.n_split + split) * (D + 2);
    if (tid < D) part[2 + tid] = acc_d;
    if (tid == 0) { part[0] = m_cta; part[1] = l_cta; }
    __syncthreads();
    if (tid == 0) {
        // one device-scope release + acquire per CTA, carried by the ticket itself (cumulative over the barrier above)
        int t;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(t) : "l"(p.tickets + row) : "memory");
        s_ticket = t;
    }
    __syncthreads();
    if (s_ticket != p.n_split - 1) return;
    const float* parts = p.partials + (int64_t)row * p.n_split * (D + 2);
    float m_all = -INFINITY;
    for (int i = 0; i < p.n_split; ++i) m_all = fmaxf(m_all, __ldcg(parts + (int64_t)i * (D + 2)));
    float l_all = 0.f, o_all = 0.f;
    if (m_all != -INFINITY) {
        for (int i = 0; i < p.n_split; ++i) {
            const float w = tq_ex2(__ldcg(parts + (int64_t)i * (D + 2)) - m_all);
            l_all = fmaf(__ldcg(parts + (int64_t)i * (D + 2) + 1), w, l_all);
            if (tid < D) o_all = fmaf(__ldcg(parts + (int64_t)i * (D + 2) + 2 + tid), w, o_all);
        }
    }
    if (tid < D) Op[tid] = from_f32<QT>(l_all > 0.f ? o_all / l_all : 0.f);
    if (tid == 0) {
        if (p.lse) p.lse[row] = l_all > 0.f ? (m_all + log2f(l_all)) * TQ_LN2 : -INFINITY;
        p.tickets[row] = 0;
    }
}

// _merge_two_attentions (eager/llama_persistent_patch.py:50-61) for n parts:
// O = sum_i exp(lse_i - m) O_i / sum_i exp(lse_i - m), lse = m + log(sum).  One warp per row.
template <typename T>
__global__ void __launch_bounds__(128) lse_merge_kernel(const T* __restrict__ O_parts, const float* __restrict__ lse_parts,
                                                        int n, int64_t rows, int D, T* __restrict__ O, float* __restrict__ lse) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= rows) return;
    float m = -INFINITY;
    for (int i = 0; i < n; ++i) m = fmaxf(m, lse_parts[(int64_t)i * rows + r]);
    if (m == -INFINITY) {
        for (int d = lane; d < D; d += 32) O[r * D + d] = from_f32<T>(0.f);
        if (lane == 0 && lse) lse[r] = -INFINITY;
        return;
    }
    float wsum = 0.f;
    for (int i = 0; i < n; ++i) wsum += expf(lse_parts[(int64_t)i * rows + r] - m);
    for (int d = lane; d < D; d += 32) {
        float a = 0.f;
        for (int i = 0; i < n; ++i)
            a = fmaf(expf(lse_parts[(int64_t)i * rows + r] - m), Dt<T>::to_f32(O_parts[((int64_t)i * rows + r) * D + d]), a);
        O[r * D + d] = from_f32<T>(a / wsum);
    }
    if (lane == 0 && lse) lse[r] = m + logf(wsum);
}

}  // namespace fq

extern "C" int fq_sparse_decode_turbo(
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
    void* workspace, size_t workspace_bytes, int n_split, void* stream) {
    using namespace fq;
    const char* fn = "fq_sparse_decode_turbo";
    FQ_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && S_kv >= 0 && P >= 0 && bucket >= 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(B <= 65535 && Hq <= 65535, FQ_ERR_ARG, "%s: B and H_q must be <= 65535", fn);
    FQ_CHECK_ARG(Hq % Hkv == 0, FQ_ERR_ARG, "%s: H_q=%d must be divisible by H_kv=%d", fn, Hq, Hkv);
    FQ_CHECK_ARG(D == 64 || D == 128, FQ_ERR_UNSUPPORTED, "%s: head_dim=%d not in (64, 128)", fn, D);
    FQ_CHECK_ARG(page >= 16 && page % 16 == 0, FQ_ERR_UNSUPPORTED, "%s: page_size=%d must be a multiple of 16", fn, page);
    FQ_CHECK_ARG(q_dtype == FQ_F16 || q_dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: Q must be fp16 or bf16 (code %d)", fn, q_dtype);
    FQ_CHECK_ARG(Q_rot && O_rot, FQ_ERR_ARG, "%s: null Q or O", fn);
    FQ_CHECK_ARG(n_split >= 1 && n_split <= 1024, FQ_ERR_ARG, "%s: n_split=%d must be in [1, 1024]", fn, n_split);
    const bool have_pages = bucket > 0 && P > 0 && S_kv > 0;
    if (have_pages) {
        FQ_CHECK_ARG(K_msb && K_lsb && V_msb && V_lsb && K_scale && V_scale && compact, FQ_ERR_ARG, "%s: null cache pointer", fn);
        FQ_CHECK_ARG((int64_t)P * page >= S_kv, FQ_ERR_ARG, "%s: %d pages of %d tokens do not cover S_kv=%d", fn, P, page, S_kv);
    }
    TurboAttnParams p;
    p.Q = Q_rot; p.q_sb = q_sb; p.q_sh = q_sh;
    p.K_msb = K_msb; p.K_lsb = K_lsb; p.V_msb = V_msb; p.V_lsb = V_lsb;
    p.km_sb = km_sb; p.km_sh = km_sh; p.km_ss = km_ss; p.kl_sb = kl_sb; p.kl_sh = kl_sh; p.kl_ss = kl_ss;
    p.vm_sb = vm_sb; p.vm_sh = vm_sh; p.vm_ss = vm_ss; p.vl_sb = vl_sb; p.vl_sh = vl_sh; p.vl_ss = vl_ss;
    p.K_scale = static_cast<const uint16_t*>(K_scale); p.V_scale = static_cast<const uint16_t*>(V_scale);
    p.ks_sb = ks_sb; p.ks_sh = ks_sh; p.vs_sb = vs_sb; p.vs_sh = vs_sh;
    p.compact = compact; p.cp_sb = cp_sb; p.cp_sh = cp_sh; p.bucket = have_pages ? bucket : 0;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.S_kv = S_kv; p.P = P; p.page = page; p.sm_scale = sm_scale;
    p.O = O_rot; p.o_sb = o_sb; p.o_sh = o_sh; p.lse = lse;
    {
        const int mrow = D / 8, lrow = D / 4;
        auto ok16 = [](const void* q, int64_t a, int64_t b2) { return aligned(q, 16) && a % 16 == 0 && b2 % 16 == 0; };
        p.fast = have_pages && km_ss == mrow && vm_ss == mrow && kl_ss == lrow && vl_ss == lrow &&
                 ok16(K_msb, km_sb, km_sh) && ok16(K_lsb, kl_sb, kl_sh) && ok16(V_msb, vm_sb, vm_sh) && ok16(V_lsb, vl_sb, vl_sh);
    }
    if (n_split > p.bucket) n_split = p.bucket > 0 ? p.bucket : 1;
    p.n_split = n_split; p.tickets = nullptr; p.partials = nullptr;
    if (n_split > 1) {
        const size_t need = fq_sparse_decode_workspace_bytes(B, Hq, D, n_split);
        FQ_CHECK_ARG(workspace && workspace_bytes >= need, FQ_ERR_WORKSPACE, "%s: workspace of %zu B needed, %zu given", fn, need, workspace_bytes);
        p.tickets = static_cast<int*>(workspace);
        p.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + (((size_t)B * Hq * 4 + 255) & ~(size_t)255));
    }
    dim3 grid((unsigned)n_split, (unsigned)Hq, (unsigned)B);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t smem = p.bucket <= TQ_LIST_MAX ? (size_t)p.bucket * sizeof(int) : 0;       // the packed page list
    void (*kern)(TurboAttnParams) =
        q_dtype == FQ_F16 ? (D == 128 ? sparse_decode_turbo_kernel<__half, 128> : sparse_decode_turbo_kernel<__half, 64>)
                          : (D == 128 ? sparse_decode_turbo_kernel<__nv_bfloat16, 128> : sparse_decode_turbo_kernel<__nv_bfloat16, 64>);
    {
        // static + dynamic shared memory pass 48 KB: each of the four kernels opts in once per device
        constexpr int MAX_DEV = 64;
        static std::atomic<bool> prepared[MAX_DEV][4];     // relaxed: concurrent host threads may repeat the idempotent set-up
        const int which = (q_dtype == FQ_F16 ? 0 : 2) + (D == 128 ? 0 : 1);
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return fail(FQ_ERR_CUDA, "%s: cannot identify the current device", fn);
        if (!prepared[dev][which].load(std::memory_order_relaxed)) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TQ_LIST_MAX * (int)sizeof(int));
            if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: cannot reserve shared memory for the page list: %s", fn, cudaGetErrorString(e));
            prepared[dev][which].store(true, std::memory_order_relaxed);
        }
    }
    launch_k(PDL_ATTN, kern, grid, dim3(TQ_THREADS), smem, st, p);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" int fq_lse_merge(const void* O_parts, const float* lse_parts, int dtype, int n, int64_t rows, int D,
                            void* O, float* lse, void* stream) {
    using namespace fq;
    const char* fn = "fq_lse_merge";
    FQ_CHECK_ARG(n >= 1 && rows >= 0 && D >= 1, FQ_ERR_ARG, "%s: bad sizes", fn);
    if (rows == 0) return FQ_OK;
    FQ_CHECK_ARG(O_parts && lse_parts && O, FQ_ERR_ARG, "%s: null pointer", fn);
    const unsigned blocks = (unsigned)((rows + 3) / 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == FQ_F32) lse_merge_kernel<float><<<blocks, 128, 0, st>>>(static_cast<const float*>(O_parts), lse_parts, n, rows, D, static_cast<float*>(O), lse);
    else if (dtype == FQ_F16) lse_merge_kernel<__half><<<blocks, 128, 0, st>>>(static_cast<const __half*>(O_parts), lse_parts, n, rows, D, static_cast<__half*>(O), lse);
    else if (dtype == FQ_BF16) lse_merge_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(O_parts), lse_parts, n, rows, D, static_cast<__nv_bfloat16*>(O), lse);
    else return fail(FQ_ERR_DTYPE, "%s: dtype code %d", fn, dtype);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}
