// INT4 KV quantisation on append, and the inverse used by prefill.
//
// One warp owns one page of one (batch, kv head).  A lane owns 8 consecutive channels
// (one 16-byte load per token); D/8 lanes cover a token, so a warp reads 32/(D/8) tokens
// per load instruction, fully coalesced.  K needs the page's per-channel min/max before any
// code can be produced, so the page is read twice (the second read is served by L1/L2);
// V is per token and needs one read.  HBM traffic per page: 2*page*D*sizeof(T) in,
// page*D (codes) + 2*D*2 (K metadata) + page*4 (V metadata) out.
#include "fq_common.cuh"

namespace fq {

struct QuantParams {
    const void *K_head, *V_head, *K_new, *V_new;
    int64_t hd_sb, hd_sh, hd_ss, nw_sb, nw_sh, nw_ss;
    int n_head, n_new;
    int B, H, D, page, n_quant, n_pages;
    uint8_t *K_packed, *V_packed;
    int64_t pk_sb, pk_sh, pk_ss;
    uint16_t *K_scale, *K_mn;
    int64_t km_sb, km_sh, km_sp;
    uint16_t *V_scale, *V_mn;
    int64_t vm_sb, vm_sh, vm_ss;
    void *stage_K, *stage_V;
    int64_t st_sb, st_sh, st_ss;
    const int* pos;      // non-null: tokens already cached, read on the device (see DynPos); outputs then point at token 0
    int n_layers;        // > 1 (only with pos): grid.z = n_layers * B, pos[layer], every tensor offset by its layer stride
    int64_t hd_sl, nw_sl, pk_sl, km_sl, vm_sl, st_sl;
    int max_tokens;      // capacity of the cache rows (device-side guard in that mode)
};

// Code of one element: rint((x - mn) / sc) clamped to 0..15, where the quotient is the IEEE
// fp32 quotient (what the reference computes).  The division is replaced by a multiplication
// with the correctly rounded reciprocal: that product is within 3e-6 of the IEEE quotient for
// quotients below 16, so both round to the same integer unless the product lies within 2e-5
// of a half-integer; only then (about 4 elements in 100 000) is the exact division done.
// Rounding to nearest even through the 1.5 * 2^23 constant.  Returns the code as a float.
__device__ __forceinline__ float code4f(float x, float mn, float sc, float rsc) {
    const float d = __fsub_rn(x, mn);
    const float t = __fmul_rn(d, rsc);
    float r = __fsub_rn(__fadd_rn(t, 12582912.0f), 12582912.0f);
    if (!(fabsf(__fsub_rn(t, r)) < 0.49998f) || !(t < 16.0f))     // near a tie, huge, or NaN
        r = rintf(__fdiv_rn(d, sc));
    return fminf(fmaxf(r, 0.0f), 15.0f);
}
// eight codes -> one 32-bit word, nibble i = code i; two exact fp32 sums of four nibbles each
__device__ __forceinline__ uint32_t pack8(const float (&q)[8]) {
    const float lo = fmaf(q[3], 4096.f, fmaf(q[2], 256.f, fmaf(q[1], 16.f, q[0])));
    const float hi = fmaf(q[7], 4096.f, fmaf(q[6], 256.f, fmaf(q[5], 16.f, q[4])));
    return (uint32_t)lo | ((uint32_t)hi << 16);
}

template <typename T>
__device__ __forceinline__ const T* stream_row(const T* head, const T* nw, const QuantParams& p,
                                               int b, int h, int t) {
    return t < p.n_head ? head + b * p.hd_sb + h * p.hd_sh + (int64_t)t * p.hd_ss
                        : nw + b * p.nw_sb + h * p.nw_sh + (int64_t)(t - p.n_head) * p.nw_ss;
}

template <typename T>
__global__ void __launch_bounds__(128) quant_int4_kernel(QuantParams pin) {
    QuantParams p = pin;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int b = blockIdx.z;
    const int h = blockIdx.y;
    if (p.n_layers > 1) {              // one launch appends to every layer
        const int layer = b / p.B;
        b -= layer * p.B;
        p.pos += layer;
        p.K_head = static_cast<const T*>(p.K_head) + layer * p.hd_sl; p.V_head = static_cast<const T*>(p.V_head) + layer * p.hd_sl;
        p.K_new = static_cast<const T*>(p.K_new) + layer * p.nw_sl;   p.V_new = static_cast<const T*>(p.V_new) + layer * p.nw_sl;
        p.K_packed += layer * p.pk_sl; p.V_packed += layer * p.pk_sl;
        p.K_scale += layer * p.km_sl;  p.K_mn += layer * p.km_sl;
        p.V_scale += layer * p.vm_sl;  p.V_mn += layer * p.vm_sl;
        p.stage_K = static_cast<T*>(p.stage_K) + layer * p.st_sl;     p.stage_V = static_cast<T*>(p.stage_V) + layer * p.st_sl;
    }
    const int page_idx = blockIdx.x * 4 + warp;
    const int LPT = p.D >> 3;          // lanes per token
    const int TPI = 32 / LPT;          // tokens per warp iteration
    const int ti = lane / LPT, c = lane % LPT;
    const T* Kh = static_cast<const T*>(p.K_head);
    const T* Kn = static_cast<const T*>(p.K_new);
    const T* Vh = static_cast<const T*>(p.V_head);
    const T* Vn = static_cast<const T*>(p.V_new);
    pdl_wait();        // inputs and the staging rows may come from the previous kernel
    pdl_trigger();
    if (p.pos) {
        // append of n_new tokens behind *pos cached ones: the staged head is the partial page
        const int seen = *p.pos;
        if (seen < 0 || seen + p.n_new > p.max_tokens) return;      // full: nothing is written (the host checks its own count)
        const int partial = seen % p.page;
        const int tok_start = seen - partial, pg_start = tok_start / p.page;
        p.n_head = partial;
        p.n_quant = ((partial + p.n_new) / p.page) * p.page;
        p.n_pages = p.n_quant / p.page;
        if (p.K_packed) p.K_packed += (int64_t)tok_start * p.pk_ss;
        if (p.V_packed) p.V_packed += (int64_t)tok_start * p.pk_ss;
        if (p.K_scale) { p.K_scale += (int64_t)pg_start * p.km_sp; p.K_mn += (int64_t)pg_start * p.km_sp; }
        if (p.V_scale) { p.V_scale += (int64_t)tok_start * p.vm_ss; p.V_mn += (int64_t)tok_start * p.vm_ss; }
    }

    if (page_idx < p.n_pages) {
        const int t0 = page_idx * p.page;
        const int n_tok = min(p.page, p.n_quant - t0);
        // ---------------- K: per page, per channel ----------------
        if (p.K_scale != nullptr) {      // K_packed may be NULL: metadata only
            float mn[8], mx[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { mn[i] = INFINITY; mx[i] = -INFINITY; }
            for (int tt = ti; tt < n_tok; tt += TPI) {
                float v[8];
                load8<T>(stream_row<T>(Kh, Kn, p, b, h, t0 + tt) + 8 * c, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) { mn[i] = fminf(mn[i], v[i]); mx[i] = fmaxf(mx[i], v[i]); }
            }
            for (int off = LPT; off < 32; off <<= 1) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    mn[i] = fminf(mn[i], __shfl_xor_sync(0xffffffffu, mn[i], off));
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], off));
                }
            }
            float sc[8];
            const float eps = Dt<T>::rn(1e-6f);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float diff = Dt<T>::rn(__fsub_rn(mx[i], mn[i]));
                sc[i] = fmaxf(Dt<T>::rn(__fdiv_rn(diff, 15.0f)), eps);
            }
            float rsc[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) rsc[i] = __frcp_rn(sc[i]);
            if (ti == 0) {
                uint32_t s4[4], m4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s4[i] = f32_to_bf16_bits(sc[2 * i]) | ((uint32_t)f32_to_bf16_bits(sc[2 * i + 1]) << 16);
                    m4[i] = f32_to_bf16_bits(mn[2 * i]) | ((uint32_t)f32_to_bf16_bits(mn[2 * i + 1]) << 16);
                }
                int64_t mo = b * p.km_sb + h * p.km_sh + (int64_t)page_idx * p.km_sp + 8 * c;
                *reinterpret_cast<uint4*>(p.K_scale + mo) = make_uint4(s4[0], s4[1], s4[2], s4[3]);
                *reinterpret_cast<uint4*>(p.K_mn + mo) = make_uint4(m4[0], m4[1], m4[2], m4[3]);
            }
            for (int tt = ti; tt < n_tok && p.K_packed != nullptr; tt += TPI) {
                float v[8];
                load8<T>(stream_row<T>(Kh, Kn, p, b, h, t0 + tt) + 8 * c, v);
                float q[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) q[i] = code4f(v[i], mn[i], sc[i], rsc[i]);
                uint8_t* row = p.K_packed + b * p.pk_sb + h * p.pk_sh + (int64_t)(t0 + tt) * p.pk_ss;
                *reinterpret_cast<uint32_t*>(row + 4 * c) = pack8(q);
            }
        }
        // ---------------- V: per token ----------------
        if (p.V_packed != nullptr) {
            for (int tt = ti; tt < n_tok + ti; tt += TPI) {   // uniform trip count for the shuffles
                const bool live = tt < n_tok;
                float v[8];
                if (live) {
                    load8<T>(stream_row<T>(Vh, Vn, p, b, h, t0 + tt) + 8 * c, v);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = 0.f;
                }
                float lo = v[0], hi = v[0];
#pragma unroll
                for (int i = 1; i < 8; ++i) { lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]); }
                for (int off = 1; off < LPT; off <<= 1) {
                    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
                    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
                }
                if (live) {
                    float sc = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), 15.0f), 1e-6f);
                    const float rsc = __frcp_rn(sc);
                    float q[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) q[i] = code4f(v[i], lo, sc, rsc);
                    uint8_t* row = p.V_packed + b * p.pk_sb + h * p.pk_sh + (int64_t)(t0 + tt) * p.pk_ss;
                    *reinterpret_cast<uint32_t*>(row + 4 * c) = pack8(q);
                    if (c == 0) {
                        int64_t mo = b * p.vm_sb + h * p.vm_sh + (int64_t)(t0 + tt) * p.vm_ss;
                        p.V_scale[mo] = f32_to_bf16_bits(sc);
                        p.V_mn[mo] = f32_to_bf16_bits(lo);
                    }
                }
            }
        }
    }
    // ---------------- staging of the tokens that do not fill a page ----------------
    // Stream token t >= n_quant goes to staging row t - n_quant.  With n_quant == 0 the head
    // tokens are already in place (the head IS the staging buffer) and only the new tokens are
    // copied behind them.  Done by the CTA that owns page 0 (the only page that can read the
    // staged head, which may alias the staging buffer), after all of its reads.
    if (blockIdx.x != 0) return;
    __syncthreads();
    const int total = p.n_head + p.n_new;
    const int rem = total - p.n_quant;
    if (rem <= 0) return;
    const int chunks = p.D >> 3;
    for (int i = threadIdx.x; i < rem * chunks; i += blockDim.x) {
        const int r = i / chunks, cc = i % chunks;
        const int t = p.n_quant + r;
        if (p.n_quant == 0 && t < p.n_head) continue;
        const int64_t so = b * p.st_sb + h * p.st_sh + (int64_t)r * p.st_ss + 8 * cc;
        if (p.stage_K != nullptr) {
            const T* src = stream_row<T>(Kh, Kn, p, b, h, t) + 8 * cc;
            T* dst = static_cast<T*>(p.stage_K) + so;
            if (sizeof(T) == 2) {
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
            } else {
                reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<const uint4*>(src)[0];
                reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<const uint4*>(src)[1];
            }
        }
        if (p.stage_V != nullptr) {
            const T* src = stream_row<T>(Vh, Vn, p, b, h, t) + 8 * cc;
            T* dst = static_cast<T*>(p.stage_V) + so;
            if (sizeof(T) == 2) {
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
            } else {
                reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<const uint4*>(src)[0];
                reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<const uint4*>(src)[1];
            }
        }
    }
}

// out = bf16(code * scale + mn); one thread per 8 output elements.
__global__ void __launch_bounds__(256) dequant_int4_kernel(
    const uint8_t* packed, int64_t pk_sb, int64_t pk_sh, int64_t pk_ss,
    const uint16_t* scale, const uint16_t* mn, int64_t m_sb, int64_t m_sh, int64_t m_s2,
    int per_page, int B, int H, int S, int D, int page,
    uint16_t* out, int64_t o_sb, int64_t o_sh, int64_t o_ss) {
    const int chunks = D >> 3;
    const int64_t total = (int64_t)B * H * S * chunks;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % chunks);
        int64_t r = i / chunks;
        const int t = (int)(r % S);
        r /= S;
        const int h = (int)(r % H), b = (int)(r / H);
        const uint32_t w = *reinterpret_cast<const uint32_t*>(packed + b * pk_sb + h * pk_sh + (int64_t)t * pk_ss + 4 * c);
        float sc[8], m[8];
        if (per_page) {
            const int64_t mo = b * m_sb + h * m_sh + (int64_t)(t / page) * m_s2 + 8 * c;
            const uint4 s4 = *reinterpret_cast<const uint4*>(scale + mo);
            const uint4 m4 = *reinterpret_cast<const uint4*>(mn + mo);
            const uint32_t sa[4] = {s4.x, s4.y, s4.z, s4.w}, ma[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                sc[2 * k] = bf16_lo(sa[k]); sc[2 * k + 1] = bf16_hi(sa[k]);
                m[2 * k] = bf16_lo(ma[k]); m[2 * k + 1] = bf16_hi(ma[k]);
            }
        } else {
            const int64_t mo = b * m_sb + h * m_sh + (int64_t)t * m_s2;
            const float s0 = bf16_lo(scale[mo]), m0 = bf16_lo(mn[mo]);
#pragma unroll
            for (int k = 0; k < 8; ++k) { sc[k] = s0; m[k] = m0; }
        }
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float a = __fadd_rn(__fmul_rn((float)((w >> (8 * k)) & 15u), sc[2 * k]), m[2 * k]);
            float bb = __fadd_rn(__fmul_rn((float)((w >> (8 * k + 4)) & 15u), sc[2 * k + 1]), m[2 * k + 1]);
            o[k] = f32_to_bf16_bits(a) | ((uint32_t)f32_to_bf16_bits(bb) << 16);
        }
        *reinterpret_cast<uint4*>(out + b * o_sb + h * o_sh + (int64_t)t * o_ss + 8 * c) =
            make_uint4(o[0], o[1], o[2], o[3]);
    }
}

}  // namespace fq

namespace fq {
int quantize_kv_int4_launch(
    const void* K_head, const void* V_head, int64_t hd_sb, int64_t hd_sh, int64_t hd_ss, int n_head,
    const void* K_new, const void* V_new, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    int dtype, int B, int H, int D, int page, int n_quant,
    uint8_t* K_packed, uint8_t* V_packed, int64_t pk_sb, int64_t pk_sh, int64_t pk_ss,
    void* K_scale, void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    void* V_scale, void* V_mn, int64_t vm_sb, int64_t vm_sh, int64_t vm_ss,
    void* stage_K, void* stage_V, int64_t st_sb, int64_t st_sh, int64_t st_ss,
    void* stream, const DynPos& dp) {
    using namespace fq;
    const char* fn = "fq_quantize_kv_int4";
    FQ_CHECK_ARG(B > 0 && H > 0 && page > 0 && n_head >= 0 && n_new >= 0 && n_quant >= 0, FQ_ERR_ARG,
                 "%s: bad sizes B=%d H=%d page=%d n_head=%d n_new=%d n_quant=%d", fn, B, H, page, n_head, n_new, n_quant);
    FQ_CHECK_ARG(D % 2 == 0, FQ_ERR_ARG, "%s: requires even head_dim; got %d", fn, D);
    FQ_CHECK_ARG(D >= 8 && D <= 256 && (D & (D - 1)) == 0, FQ_ERR_UNSUPPORTED,
                 "%s: head_dim %d not in {8,16,32,64,128,256}", fn, D);
    FQ_CHECK_ARG(n_quant <= n_head + n_new, FQ_ERR_ARG, "%s: n_quant %d exceeds the stream length %d", fn, n_quant, n_head + n_new);
    FQ_CHECK_ARG(n_head == 0 || n_quant == 0 || n_head < page, FQ_ERR_ARG,
                 "%s: a staged head (%d tokens) must be shorter than a page (%d)", fn, n_head, page);
    FQ_CHECK_ARG(dtype == FQ_F32 || dtype == FQ_F16 || dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: dtype code %d", fn, dtype);
    const bool doK = K_packed != nullptr || K_scale != nullptr, doV = V_packed != nullptr;
    if (n_quant > 0) {
        FQ_CHECK_ARG(doK || doV, FQ_ERR_ARG, "%s: neither K nor V outputs given", fn);
        FQ_CHECK_ARG(!doK || (K_scale && K_mn && (K_new || n_new == 0)), FQ_ERR_ARG, "%s: K outputs/inputs missing", fn);
        FQ_CHECK_ARG(!doV || (V_scale && V_mn && (V_new || n_new == 0)), FQ_ERR_ARG, "%s: V outputs/inputs missing", fn);
    }
    const size_t esz = dtype == FQ_F32 ? 4 : 2;
    const size_t row_align = 16 / esz;  // elements per 16 bytes
    FQ_CHECK_ARG(hd_sb % row_align == 0 && hd_sh % row_align == 0 && hd_ss % row_align == 0 &&
                 nw_sb % row_align == 0 && nw_sh % row_align == 0 && nw_ss % row_align == 0 &&
                 st_sb % row_align == 0 && st_sh % row_align == 0 && st_ss % row_align == 0,
                 FQ_ERR_ALIGN, "%s: input/staging strides must keep rows 16-byte aligned", fn);
    FQ_CHECK_ARG(aligned(K_head, 16) && aligned(V_head, 16) && aligned(K_new, 16) && aligned(V_new, 16) &&
                 aligned(stage_K, 16) && aligned(stage_V, 16), FQ_ERR_ALIGN, "%s: input pointers must be 16-byte aligned", fn);
    FQ_CHECK_ARG(pk_sb % 4 == 0 && pk_sh % 4 == 0 && pk_ss % 4 == 0 && aligned(K_packed, 4) && aligned(V_packed, 4),
                 FQ_ERR_ALIGN, "%s: packed rows must be 4-byte aligned", fn);
    FQ_CHECK_ARG(km_sb % 8 == 0 && km_sh % 8 == 0 && km_sp % 8 == 0 && aligned(K_scale, 16) && aligned(K_mn, 16),
                 FQ_ERR_ALIGN, "%s: K metadata rows must be 16-byte aligned", fn);

    QuantParams p;
    p.K_head = K_head; p.V_head = V_head; p.K_new = K_new; p.V_new = V_new;
    p.hd_sb = hd_sb; p.hd_sh = hd_sh; p.hd_ss = hd_ss; p.nw_sb = nw_sb; p.nw_sh = nw_sh; p.nw_ss = nw_ss;
    p.n_head = n_head; p.n_new = n_new;
    p.B = B; p.H = H; p.D = D; p.page = page; p.n_quant = n_quant;
    p.n_pages = (n_quant + page - 1) / page;
    p.K_packed = K_packed; p.V_packed = V_packed; p.pk_sb = pk_sb; p.pk_sh = pk_sh; p.pk_ss = pk_ss;
    p.K_scale = static_cast<uint16_t*>(K_scale); p.K_mn = static_cast<uint16_t*>(K_mn);
    p.km_sb = km_sb; p.km_sh = km_sh; p.km_sp = km_sp;
    p.V_scale = static_cast<uint16_t*>(V_scale); p.V_mn = static_cast<uint16_t*>(V_mn);
    p.vm_sb = vm_sb; p.vm_sh = vm_sh; p.vm_ss = vm_ss;
    p.stage_K = stage_K; p.stage_V = stage_V; p.st_sb = st_sb; p.st_sh = st_sh; p.st_ss = st_ss;
    p.pos = dp.pos; p.max_tokens = dp.pos ? dp.max_tokens : 0x7fffffff;
    p.n_layers = 1; p.hd_sl = p.nw_sl = p.pk_sl = p.km_sl = p.vm_sl = p.st_sl = 0;
    if (p.pos == nullptr && n_quant == 0 && (n_head + n_new == 0 || (!stage_K && !stage_V))) return FQ_OK;

    dim3 grid((unsigned)max(1, (p.n_pages + 3) / 4), (unsigned)H, (unsigned)B);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == FQ_F32) launch_k(PDL_QUANT, quant_int4_kernel<float>, grid, dim3(128), 0, st, p);
    else if (dtype == FQ_F16) launch_k(PDL_QUANT, quant_int4_kernel<__half>, grid, dim3(128), 0, st, p);
    else launch_k(PDL_QUANT, quant_int4_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, p);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

}  // namespace fq

extern "C" int fq_quantize_kv_int4(
    const void* K_head, const void* V_head, int64_t hd_sb, int64_t hd_sh, int64_t hd_ss, int n_head,
    const void* K_new, const void* V_new, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    int dtype, int B, int H, int D, int page, int n_quant,
    uint8_t* K_packed, uint8_t* V_packed, int64_t pk_sb, int64_t pk_sh, int64_t pk_ss,
    void* K_scale, void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    void* V_scale, void* V_mn, int64_t vm_sb, int64_t vm_sh, int64_t vm_ss,
    void* stage_K, void* stage_V, int64_t st_sb, int64_t st_sh, int64_t st_ss,
    void* stream) {
    return fq::quantize_kv_int4_launch(K_head, V_head, hd_sb, hd_sh, hd_ss, n_head, K_new, V_new, nw_sb, nw_sh, nw_ss, n_new,
                                       dtype, B, H, D, page, n_quant, K_packed, V_packed, pk_sb, pk_sh, pk_ss,
                                       K_scale, K_mn, km_sb, km_sh, km_sp, V_scale, V_mn, vm_sb, vm_sh, vm_ss,
                                       stage_K, stage_V, st_sb, st_sh, st_ss, stream, fq::DynPos{});
}

namespace fq {
// Append n_new tokens (1 <= n_new < page) to layers [0, n_layers) in ONE launch, positions read from pos[layer].
int quant_append_layers_dyn(const fq_int4_cache* c, int n_layers, const int* pos, const void* K_new, const void* V_new,
                            int64_t nw_sl, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new, void* stream) {
    const char* fn = "fq_decode_step_int4_dev";
    FQ_CHECK_ARG(aligned(K_new, 16) && aligned(V_new, 16) && nw_sl % 8 == 0 && nw_sb % 8 == 0 && nw_sh % 8 == 0 && nw_ss % 8 == 0,
                 FQ_ERR_ALIGN, "%s: new K/V rows must be 16-byte aligned", fn);
    QuantParams p;
    p.K_head = c->K_partial; p.V_head = c->V_partial; p.K_new = K_new; p.V_new = V_new;
    p.hd_sb = c->pt_sb; p.hd_sh = c->pt_sh; p.hd_ss = c->pt_ss; p.nw_sb = nw_sb; p.nw_sh = nw_sh; p.nw_ss = nw_ss;
    p.n_head = 0; p.n_new = n_new;
    p.B = c->B; p.H = c->Hkv; p.D = c->D; p.page = c->page; p.n_quant = 0; p.n_pages = 1;
    p.K_packed = c->K_packed; p.V_packed = c->V_packed; p.pk_sb = c->pk_sb; p.pk_sh = c->pk_sh; p.pk_ss = c->pk_ss;
    p.K_scale = static_cast<uint16_t*>(c->K_scale); p.K_mn = static_cast<uint16_t*>(c->K_mn);
    p.km_sb = c->km_sb; p.km_sh = c->km_sh; p.km_sp = c->km_sp;
    p.V_scale = static_cast<uint16_t*>(c->V_scale); p.V_mn = static_cast<uint16_t*>(c->V_mn);
    p.vm_sb = c->vm_sb; p.vm_sh = c->vm_sh; p.vm_ss = 1;
    p.stage_K = c->K_partial; p.stage_V = c->V_partial; p.st_sb = c->pt_sb; p.st_sh = c->pt_sh; p.st_ss = c->pt_ss;
    p.pos = pos; p.max_tokens = c->max_seq_len;
    p.n_layers = n_layers; p.hd_sl = c->pt_sl; p.nw_sl = nw_sl; p.pk_sl = c->pk_sl; p.km_sl = c->km_sl; p.vm_sl = c->vm_sl; p.st_sl = c->pt_sl;
    FQ_CHECK_ARG((int64_t)c->B * n_layers <= 65535, FQ_ERR_ARG, "%s: batch x layers = %lld too large for one launch", fn, (long long)c->B * n_layers);
    dim3 grid(1u, (unsigned)c->Hkv, (unsigned)(c->B * n_layers));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (c->kv_dtype == FQ_F16) launch_k(PDL_QUANT, quant_int4_kernel<__half>, grid, dim3(128), 0, st, p);
    else launch_k(PDL_QUANT, quant_int4_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, p);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}
}  // namespace fq

extern "C" int fq_dequantize_int4(
    const uint8_t* packed, int64_t pk_sb, int64_t pk_sh, int64_t pk_ss,
    const void* scale, const void* mn, int64_t m_sb, int64_t m_sh, int64_t m_s2,
    int per_page, int B, int H, int S, int D, int page,
    void* out, int64_t o_sb, int64_t o_sh, int64_t o_ss, void* stream) {
    using namespace fq;
    const char* fn = "fq_dequantize_int4";
    FQ_CHECK_ARG(B > 0 && H > 0 && S >= 0 && page > 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(D >= 8 && D % 8 == 0, FQ_ERR_UNSUPPORTED, "%s: head_dim %d must be a multiple of 8", fn, D);
    FQ_CHECK_ARG(packed && scale && mn && out, FQ_ERR_ARG, "%s: null pointer", fn);
    FQ_CHECK_ARG(pk_sb % 4 == 0 && pk_sh % 4 == 0 && pk_ss % 4 == 0 && aligned(packed, 4), FQ_ERR_ALIGN, "%s: packed rows must be 4-byte aligned", fn);
    FQ_CHECK_ARG(o_sb % 8 == 0 && o_sh % 8 == 0 && o_ss % 8 == 0 && aligned(out, 16), FQ_ERR_ALIGN, "%s: output rows must be 16-byte aligned", fn);
    if (per_page)
        FQ_CHECK_ARG(m_sb % 8 == 0 && m_sh % 8 == 0 && m_s2 % 8 == 0 && aligned(scale, 16) && aligned(mn, 16), FQ_ERR_ALIGN,
                     "%s: K metadata rows must be 16-byte aligned", fn);
    if (S == 0) return FQ_OK;
    const int64_t total = (int64_t)B * H * S * (D / 8);
    const int64_t want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    dequant_int4_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        packed, pk_sb, pk_sh, pk_ss, static_cast<const uint16_t*>(scale), static_cast<const uint16_t*>(mn),
        m_sb, m_sh, m_s2, per_page, B, H, S, D, page, static_cast<uint16_t*>(out), o_sb, o_sh, o_ss);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}
