// Dense causal attention for the prefill branch (S_q > 1): queries of the new tokens over the
// dequantised completed pages followed by the staged tail, grouped-query heads, online softmax.
//
// This is the step that the reference hands to torch's scaled_dot_product_attention with
// is_causal=True and enable_gqa=True (eager/llama_persistent_patch.py:196-201).  The causal mask
// is aligned at the TOP LEFT, as torch aligns it when S_q != S_kv: query i sees keys 0..i.
//
// A real dense contraction (4*S_q*S_kv*D/2 flops per head), so it runs on the tensor cores:
// mma.sync m16n8k16 with fp32 accumulation, bf16 or fp16 operands as the cache stages them.
// One CTA = 64 queries x one query head; 4 warps x 16 query rows.  K and V tiles of 64 keys are
// staged by 16-byte cp.async into a two-deep ring of padded rows (row stride D+8 elements, so
// ldmatrix reads are bank-conflict free); Q stays in registers as A fragments for the whole
// walk; P = softmax(QK^T) goes from the accumulator layout straight into A fragments for P.V.
#include "fq_common.cuh"

namespace fq {

constexpr int PF_BM = 64, PF_BN = 64, PF_THREADS = 128;

struct PrefillParams {
    const void *Q, *K, *V; void* O;
    int64_t q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh, o_ss;
    int B, Hq, Hkv, Sq, Skv;
    float scale_log2;       // sm_scale * log2(e)
};

__device__ __forceinline__ uint32_t pf_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pf_cp16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;      // src-size 0: the 16 bytes are zero-filled, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(pf_smem(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void pf_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void pf_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T> __device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float pf_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename T, int D>
__global__ void __launch_bounds__(PF_THREADS) prefill_attn_kernel(PrefillParams p) {
    constexpr int LD = D + 8;                  // padded row, elements
    constexpr int CPR = D / 8;                 // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char pf_smem_raw[];
    T* sQ = reinterpret_cast<T*>(pf_smem_raw);            // [64][LD]
    T* sK = sQ + PF_BM * LD;                               // [2][64][LD]
    T* sV = sK + 2 * PF_BN * LD;                           // [2][64][LD]

    // the heaviest query tiles (most keys under the causal mask) are scheduled first
    const int qt = gridDim.x - 1 - blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (p.Hq / p.Hkv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int q0 = qt * PF_BM;
    const T* Qg = static_cast<const T*>(p.Q) + b * p.q_sb + hq * p.q_sh;
    const T* Kg = static_cast<const T*>(p.K) + b * p.k_sb + hkv * p.k_sh;
    const T* Vg = static_cast<const T*>(p.V) + b * p.v_sb + hkv * p.v_sh;

    // keys this tile can see: 0 .. min(S_kv, q0 + 64) - 1
    const int kv_end = min(p.Skv, q0 + PF_BM);
    const int n_tiles = (kv_end + PF_BN - 1) / PF_BN;

    auto load_kv = [&](int tile, int stage) {
        const int n0 = tile * PF_BN;
        for (int c = tid; c < PF_BN * CPR; c += PF_THREADS) {
            const int r = c / CPR, ch = c - r * CPR;
            const bool ok = n0 + r < p.Skv;
            const int64_t row = ok ? n0 + r : 0;
            pf_cp16(sK + (stage * PF_BN + r) * LD + 8 * ch, Kg + row * p.k_ss + 8 * ch, ok);
            pf_cp16(sV + (stage * PF_BN + r) * LD + 8 * ch, Vg + row * p.v_ss + 8 * ch, ok);
        }
    };
    for (int c = tid; c < PF_BM * CPR; c += PF_THREADS) {
        const int r = c / CPR, ch = c - r * CPR;
        const bool ok = q0 + r < p.Sq;
        pf_cp16(sQ + r * LD + 8 * ch, Qg + (int64_t)(ok ? q0 + r : 0) * p.q_ss + 8 * ch, ok);
    }
    load_kv(0, 0);
    pf_commit();
    if (n_tiles > 1) load_kv(1, 1);
    pf_commit();
    pf_wait<1>();
    __syncthreads();

    // Q fragments of this warp's 16 rows, for the whole walk
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kb = 0; kb < D / 16; ++kb)
        ldsm_x4(qf[kb], pf_smem(sQ + (warp * 16 + (lane & 15)) * LD + kb * 16 + (lane >> 4) * 8));

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;     // rows g and g+8 (base-2 logits)
    const int row0 = q0 + warp * 16 + g, row1 = row0 + 8;

    for (int tile = 0; tile < n_tiles; ++tile) {
        const int stage = tile & 1;
        const int n0 = tile * PF_BN;
        const T* tK = sK + stage * PF_BN * LD;
        const T* tV = sV + stage * PF_BN * LD;
        // ---- S = Q K^T (16 x 64 per warp) ----
        float s[PF_BN / 8][4];
#pragma unroll
        for (int i = 0; i < PF_BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int kb = 0; kb < D / 16; ++kb) {
#pragma unroll
            for (int nb = 0; nb < PF_BN / 16; ++nb) {
                uint32_t kf[4];
                ldsm_x4(kf, pf_smem(tK + (nb * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + kb * 16 + ((lane >> 3) & 1) * 8));
                mma16816<T>(s[2 * nb], qf[kb], kf[0], kf[1]);
                mma16816<T>(s[2 * nb + 1], qf[kb], kf[2], kf[3]);
            }
        }
        // ---- scale, mask (causal at the top left; keys past S_kv), online softmax ----
        const bool need_mask = n0 + PF_BN > q0 + warp * 16 || n0 + PF_BN > p.Skv;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < PF_BN / 8; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[i][e] * p.scale_log2;
                if (need_mask) {
                    const int col = n0 + 8 * i + 2 * t + (e & 1);
                    const int row = (e & 2) ? row1 : row0;
                    if (col > row || col >= p.Skv) v = -INFINITY;
                }
                s[i][e] = v;
            }
            mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
            mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // a row that has seen nothing yet keeps a finite reference so that exp2(-inf - ref) = 0
        const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
        const float a0 = pf_ex2(m0 - ref0), a1 = pf_ex2(m1 - ref1);
        m0 = mn0; m1 = mn1;
        float ls0 = 0.f, ls1 = 0.f;
        uint32_t pf[PF_BN / 16][4];
#pragma unroll
        for (int i = 0; i < PF_BN / 8; ++i) {
            const float p0 = pf_ex2(s[i][0] - ref0), p1 = pf_ex2(s[i][1] - ref0);
            const float p2 = pf_ex2(s[i][2] - ref1), p3 = pf_ex2(s[i][3] - ref1);
            ls0 += p0 + p1; ls1 += p2 + p3;
            pf[i >> 1][(i & 1) * 2 + 0] = pack2<T>(p0, p1);
            pf[i >> 1][(i & 1) * 2 + 1] = pack2<T>(p2, p3);
        }
        l0 = l0 * a0 + ls0; l1 = l1 * a1 + ls1;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
        // ---- O += P V ----
#pragma unroll
        for (int kb = 0; kb < PF_BN / 16; ++kb) {
#pragma unroll
            for (int db = 0; db < D / 16; ++db) {
                uint32_t vf[4];
                ldsm_x4_t(vf, pf_smem(tV + (kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + db * 16 + (lane >> 4) * 8));
                mma16816<T>(o[2 * db], pf[kb], vf[0], vf[1]);
                mma16816<T>(o[2 * db + 1], pf[kb], vf[2], vf[3]);
            }
        }
        __syncthreads();                       // every warp is done with this stage
        if (tile + 2 < n_tiles) load_kv(tile + 2, stage);
        pf_commit();
        pf_wait<1>();                          // the next tile has landed
        __syncthreads();
    }
    pf_wait<0>();

    // ---- normalise and store ----
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    T* Og = static_cast<T*>(p.O) + b * p.o_sb + hq * p.o_sh;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        const int col = 8 * i + 2 * t;
        if (row0 < p.Sq) *reinterpret_cast<uint32_t*>(Og + (int64_t)row0 * p.o_ss + col) = pack2<T>(o[i][0] * i0, o[i][1] * i0);
        if (row1 < p.Sq) *reinterpret_cast<uint32_t*>(Og + (int64_t)row1 * p.o_ss + col) = pack2<T>(o[i][2] * i1, o[i][3] * i1);
    }
}

template <typename T, int D>
static int launch_prefill(const PrefillParams& p, cudaStream_t st) {
    constexpr size_t smem = (size_t)(PF_BM + 4 * PF_BN) * (D + 8) * sizeof(T);
    auto kern = prefill_attn_kernel<T, D>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "fq_prefill_attention: cannot reserve %zu B of shared memory: %s", smem, cudaGetErrorString(e));
    dim3 grid((unsigned)((p.Sq + PF_BM - 1) / PF_BM), (unsigned)p.Hq, (unsigned)p.B);
    kern<<<grid, PF_THREADS, smem, st>>>(p);
    return FQ_OK;
}

// tcgen05 kernel for head_dim 128 (fq_prefill_attn_tc.cu); false: shape not served there
bool prefill_attention_tc_launch(const void* Q, int64_t q_sb, int64_t q_sh, int64_t q_ss, const void* K, int64_t k_sb, int64_t k_sh, int64_t k_ss,
                                 const void* V, int64_t v_sb, int64_t v_sh, int64_t v_ss, int bf16, int B, int Hq, int Hkv, int Sq, int Skv,
                                 float sm_scale, void* O, int64_t o_sb, int64_t o_sh, int64_t o_ss, cudaStream_t st, int* rc);

}  // namespace fq

extern "C" int fq_prefill_attention(
    const void* Q, int64_t q_sb, int64_t q_sh, int64_t q_ss,
    const void* K, int64_t k_sb, int64_t k_sh, int64_t k_ss,
    const void* V, int64_t v_sb, int64_t v_sh, int64_t v_ss,
    int dtype, int B, int Hq, int Hkv, int Sq, int Skv, int D, float sm_scale,
    void* O, int64_t o_sb, int64_t o_sh, int64_t o_ss, void* stream) {
    using namespace fq;
    const char* fn = "fq_prefill_attention";
    FQ_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && Sq >= 0 && Skv >= 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(B <= 65535 && Hq <= 65535, FQ_ERR_ARG, "%s: B and H_q must be <= 65535", fn);
    FQ_CHECK_ARG(Hq % Hkv == 0, FQ_ERR_ARG, "%s: H_q=%d must be divisible by H_kv=%d", fn, Hq, Hkv);
    FQ_CHECK_ARG(D == 64 || D == 128, FQ_ERR_UNSUPPORTED, "%s: head_dim=%d not in (64, 128)", fn, D);
    FQ_CHECK_ARG(dtype == FQ_F16 || dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: tensors must be fp16 or bf16 (code %d)", fn, dtype);
    if (Sq == 0) return FQ_OK;
    FQ_CHECK_ARG(Q && O && (Skv == 0 || (K && V)), FQ_ERR_ARG, "%s: null pointer", fn);
    FQ_CHECK_ARG(aligned(Q, 16) && aligned(K, 16) && aligned(V, 16) && aligned(O, 4) &&
                 q_sb % 8 == 0 && q_sh % 8 == 0 && q_ss % 8 == 0 && k_sb % 8 == 0 && k_sh % 8 == 0 && k_ss % 8 == 0 &&
                 v_sb % 8 == 0 && v_sh % 8 == 0 && v_ss % 8 == 0 && o_sb % 2 == 0 && o_sh % 2 == 0 && o_ss % 2 == 0,
                 FQ_ERR_ALIGN, "%s: Q/K/V rows must be 16-byte aligned, O rows 4-byte aligned", fn);
    PrefillParams p;
    p.Q = Q; p.K = K; p.V = V; p.O = O;
    p.q_sb = q_sb; p.q_sh = q_sh; p.q_ss = q_ss; p.k_sb = k_sb; p.k_sh = k_sh; p.k_ss = k_ss;
    p.v_sb = v_sb; p.v_sh = v_sh; p.v_ss = v_ss; p.o_sb = o_sb; p.o_sh = o_sh; p.o_ss = o_ss;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Skv = Skv;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc;
    // head_dim 128 with at least one full query tile: the tcgen05 kernel; everything else: mma.sync
    if (D == 128 && Sq >= 128 && Skv >= 1 &&
        prefill_attention_tc_launch(Q, q_sb, q_sh, q_ss, K, k_sb, k_sh, k_ss, V, v_sb, v_sh, v_ss, dtype == FQ_BF16 ? 1 : 0, B, Hq, Hkv, Sq, Skv,
                                    sm_scale, O, o_sb, o_sh, o_ss, st, &rc)) {
        if (rc != FQ_OK) return rc;
        FQ_CHECK_LAUNCH(fn);
        return FQ_OK;
    }
    if (dtype == FQ_BF16) rc = D == 128 ? launch_prefill<__nv_bfloat16, 128>(p, st) : launch_prefill<__nv_bfloat16, 64>(p, st);
    else rc = D == 128 ? launch_prefill<__half, 128>(p, st) : launch_prefill<__half, 64>(p, st);
    if (rc != FQ_OK) return rc;
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}
