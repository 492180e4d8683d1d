// Sparse decode attention over TurboQuant K3-V3 bit planes, in the rotated basis, and the
// n-way LSE merge of partial attention results.
//
// Per selected 16-token unit the kernel reads 16 x (D/8 + D/4 + 2) bytes for K and the same
// for V (1600 B at D = 128).  One warp owns one unit at a time.  K phase: lane = (token,
// half of the channels); the 3-bit index of a channel is assembled from the two planes and the
// codebook value is fetched from a lane-private column of a shared-memory table (no bank
// conflicts); the two halves of a token meet by one shuffle.  V phase: lane = D/32 channels of
// every token.  Softmax in base 2, fp32 accumulation, split-K partials merged by the CTA
// that draws the last ticket of its row (no CTA waits for another).
// This first version loads straight from global memory (no staging pipeline) and is bound by
// the shared-memory table look-ups, not by HBM.
#include "fq_common.cuh"

namespace fq {

constexpr int TQ_WARPS = 4;
constexpr int TQ_THREADS = TQ_WARPS * 32;
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
};

__device__ __forceinline__ float tq_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename QT, int D>
__global__ void __launch_bounds__(TQ_THREADS) sparse_decode_turbo_kernel(TurboAttnParams p) {
    constexpr int TOK = 16;
    constexpr int HALF = D / 2;          // channels per lane in the K phase
    constexpr int EV = D / 32;           // channels per lane in the V phase
    constexpr int NSTATE = TQ_WARPS;
    __shared__ float s_cb[8 * 32];       // codebook, one column per lane
    __shared__ float s_q[D + 2];         // q * sm_scale * log2(e); second half shifted by one bank
    __shared__ float s_m[NSTATE], s_l[NSTATE], s_acc[NSTATE][D];
    __shared__ int s_ticket;

    const int split = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
    const int n_rep = p.Hq / p.Hkv, hkv = hq / n_rep;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float cb[8] = {-2.1519f, -1.3439f, -0.7560f, -0.2451f, 0.2451f, 0.7560f, 1.3439f, 2.1519f};
    for (int i = tid; i < 8 * 32; i += TQ_THREADS) s_cb[i] = cb[i >> 5];
    {
        const QT* qp = static_cast<const QT*>(p.Q) + b * p.q_sb + hq * p.q_sh;
        for (int d = tid; d < D; d += TQ_THREADS) s_q[d + (d >= HALF ? 1 : 0)] = Dt<QT>::to_f32(qp[d]) * (p.sm_scale * TQ_LOG2E);
    }
    __syncthreads();
    const float* cbl = s_cb + lane;      // cbl[idx * 32]

    const int cpp = p.page / TOK;
    const int slots_per_split = (p.bucket + p.n_split - 1) / p.n_split;
    const int slot_begin = split * slots_per_split;
    const int slot_end = min(p.bucket, slot_begin + slots_per_split);
    const int n_units = max(0, slot_end - slot_begin) * cpp;
    const int32_t* list = p.compact + b * p.cp_sb + hq * p.cp_sh;

    const uint8_t* Kmsb = p.K_msb + b * p.km_sb + hkv * p.km_sh;
    const uint8_t* Klsb = p.K_lsb + b * p.kl_sb + hkv * p.kl_sh;
    const uint8_t* Vmsb = p.V_msb + b * p.vm_sb + hkv * p.vm_sh;
    const uint8_t* Vlsb = p.V_lsb + b * p.vl_sb + hkv * p.vl_sh;
    const uint16_t* Ksc = p.K_scale + b * p.ks_sb + hkv * p.ks_sh;
    const uint16_t* Vsc = p.V_scale + b * p.vs_sb + hkv * p.vs_sh;

    float m_run = -INFINITY, l_run = 0.f, acc[EV];
#pragma unroll
    for (int j = 0; j < EV; ++j) acc[j] = 0.f;

    const int tk = lane >> 1, hh = lane & 1;            // K phase: token, channel half
    const float* qh = s_q + hh * (HALF + 1);
    for (int u = warp; u < n_units; u += TQ_WARPS) {
        const int pg = __ldg(list + slot_begin + u / cpp);
        if (pg < 0 || pg >= p.P) continue;              // warp-uniform
        const int tok0 = pg * p.page + (u % cpp) * TOK;
        const int n_tok = min(TOK, p.S_kv - tok0);
        if (n_tok <= 0) continue;
        // ---------------- K ----------------
        float x = -INFINITY;
        {
            const bool valid = tk < n_tok;
            float dot = 0.f;
            if (valid) {
                const uint32_t* mw = reinterpret_cast<const uint32_t*>(Kmsb + (int64_t)(tok0 + tk) * p.km_ss + hh * (D / 16));
                const uint32_t* lw = reinterpret_cast<const uint32_t*>(Klsb + (int64_t)(tok0 + tk) * p.kl_ss + hh * (D / 8));
#pragma unroll
                for (int w = 0; w < HALF / 32; ++w) {       // 32 channels per msb word
                    const uint32_t m = __ldg(mw + w);
                    const uint32_t l0 = __ldg(lw + 2 * w), l1 = __ldg(lw + 2 * w + 1);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const uint32_t lo = i < 16 ? (l0 >> (2 * i)) & 3u : (l1 >> (2 * (i - 16))) & 3u;
                        const uint32_t idx = (((m >> i) & 1u) << 2) | lo;
                        dot = fmaf(qh[32 * w + i], cbl[idx * 32], dot);
                    }
                }
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            if (valid) x = dot * bf16_lo(__ldg(Ksc + tok0 + tk));
        }
        float pmax = x;
#pragma unroll
        for (int off = 16; off >= 2; off >>= 1) pmax = fmaxf(pmax, __shfl_xor_sync(0xffffffffu, pmax, off));
        const float m_new = fmaxf(m_run, pmax);
        const float alpha = tq_ex2(m_run - m_new);
        const float pr = tq_ex2(x - m_new);                 // both lanes of a token hold the same value
        float psum = hh == 0 ? pr : 0.f;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
        l_run = l_run * alpha + psum;
        m_run = m_new;
        const float pv_mine = (tk < n_tok) ? pr * bf16_lo(__ldg(Vsc + tok0 + tk)) : 0.f;
        // ---------------- V ----------------
#pragma unroll
        for (int j = 0; j < EV; ++j) acc[j] *= alpha;
        const int d0 = lane * EV;
        for (int t = 0; t < n_tok; ++t) {
            const float pv = __shfl_sync(0xffffffffu, pv_mine, 2 * t);
            const uint32_t mb = __ldg(Vmsb + (int64_t)(tok0 + t) * p.vm_ss + (d0 >> 3));
            const uint32_t lb = __ldg(Vlsb + (int64_t)(tok0 + t) * p.vl_ss + (d0 >> 2));
#pragma unroll
            for (int j = 0; j < EV; ++j) {
                const int d = d0 + j;
                const uint32_t idx = (((mb >> (d & 7)) & 1u) << 2) | ((lb >> (2 * (d & 3))) & 3u);
                acc[j] = fmaf(pv, cbl[idx * 32], acc[j]);
            }
        }
    }

    // ---------------- CTA merge ----------------
    if (lane == 0) { s_m[warp] = m_run; s_l[warp] = l_run; }
#pragma unroll
    for (int j = 0; j < EV; ++j) s_acc[warp][lane * EV + j] = acc[j];
    __syncthreads();
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
        __threadfence();
        s_ticket = atomicAdd(&p.tickets[row], 1);
        __threadfence();
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
        FQ_CHECK_ARG(aligned(K_msb, 4) && aligned(K_lsb, 4) && aligned(V_msb, 4) && aligned(V_lsb, 4) &&
                     km_sb % 4 == 0 && km_sh % 4 == 0 && km_ss % 4 == 0 && kl_sb % 4 == 0 && kl_sh % 4 == 0 && kl_ss % 4 == 0,
                     FQ_ERR_ALIGN, "%s: plane rows must be 4-byte aligned", fn);
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
    if (q_dtype == FQ_F16) {
        if (D == 128) sparse_decode_turbo_kernel<__half, 128><<<grid, TQ_THREADS, 0, st>>>(p);
        else sparse_decode_turbo_kernel<__half, 64><<<grid, TQ_THREADS, 0, st>>>(p);
    } else {
        if (D == 128) sparse_decode_turbo_kernel<__nv_bfloat16, 128><<<grid, TQ_THREADS, 0, st>>>(p);
        else sparse_decode_turbo_kernel<__nv_bfloat16, 64><<<grid, TQ_THREADS, 0, st>>>(p);
    }
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
