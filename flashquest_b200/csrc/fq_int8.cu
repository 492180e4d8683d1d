// INT8 KV variant of the path (KIVI-style asymmetric uint8, 255 levels): quantise / dequantise,
// and sparse decode attention over selected uint8 pages.  Same structure as the INT4 variant with
// one code per byte: K per page and channel (scale and min computed in the input dtype), V per
// token in fp32.  The page scores of this variant are the INT4 scoring kernel with 255 levels.
// This is the kv_bits == 8 route of the dispatcher; the decode loop spends its bytes on codes
// (D bytes per token and head for each of K and V), so the kernels stay simple: a warp owns a
// token row, a lane D/32 channels.
#include "fq_common.cuh"

namespace fq {

constexpr float I8_LOG2E = 1.4426950408889634f;
constexpr float I8_LN2 = 0.6931471805599453f;

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float i8_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// K: one warp per (b, h, page); lane owns channels lane, lane+32, ...
template <typename T>
__global__ void __launch_bounds__(128) quant_k_int8_kernel(const T* __restrict__ K, int64_t k_sb, int64_t k_sh, int64_t k_ss,
                                                           int B, int H, int S, int D, int page,
                                                           uint8_t* __restrict__ codes, int64_t c_sb, int64_t c_sh, int64_t c_ss,
                                                           uint16_t* __restrict__ scale, uint16_t* __restrict__ mn, int64_t m_sb, int64_t m_sh, int64_t m_sp) {
    const int lane = threadIdx.x & 31;
    const int P = (S + page - 1) / page;
    const int64_t w = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (w >= (int64_t)B * H * P) return;
    const int p = (int)(w % P), h = (int)((w / P) % H), b = (int)(w / ((int64_t)P * H));
    const int t0 = p * page, n_tok = min(page, S - t0);
    const T* src = K + b * k_sb + h * k_sh + (int64_t)t0 * k_ss;
    for (int d = lane; d < D; d += 32) {
        float lo = INFINITY, hi = -INFINITY;
        for (int t = 0; t < n_tok; ++t) {
            const float v = Dt<T>::to_f32(src[(int64_t)t * k_ss + d]);
            lo = fminf(lo, v); hi = fmaxf(hi, v);
        }
        // scale arithmetic in the input dtype: (mx - mn) rounded to T, the quotient by 255 rounded to T, clamped at T(1e-6)
        const float diff = Dt<T>::rn(__fsub_rn(hi, lo));
        float sc = Dt<T>::rn(__fdiv_rn(diff, 255.0f));
        sc = fmaxf(sc, Dt<T>::rn(1e-6f));
        const int64_t mo = b * m_sb + h * m_sh + (int64_t)p * m_sp + d;
        scale[mo] = f32_to_bf16_bits(sc);
        mn[mo] = f32_to_bf16_bits(lo);
        for (int t = 0; t < n_tok; ++t) {
            const float v = Dt<T>::to_f32(src[(int64_t)t * k_ss + d]);
            const float c = rintf(__fdiv_rn(__fsub_rn(v, lo), sc));
            codes[b * c_sb + h * c_sh + (int64_t)(t0 + t) * c_ss + d] = (uint8_t)fminf(fmaxf(c, 0.f), 255.f);
        }
    }
}

// V: one warp per token
template <typename T>
__global__ void __launch_bounds__(128) quant_v_int8_kernel(const T* __restrict__ V, int64_t v_sb, int64_t v_sh, int64_t v_ss,
                                                           int B, int H, int S, int D,
                                                           uint8_t* __restrict__ codes, int64_t c_sb, int64_t c_sh, int64_t c_ss,
                                                           uint16_t* __restrict__ scale, uint16_t* __restrict__ mn, int64_t m_sb, int64_t m_sh) {
    const int lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (w >= (int64_t)B * H * S) return;
    const int t = (int)(w % S), h = (int)((w / S) % H), b = (int)(w / ((int64_t)S * H));
    const T* src = V + b * v_sb + h * v_sh + (int64_t)t * v_ss;
    float lo = INFINITY, hi = -INFINITY;
    for (int d = lane; d < D; d += 32) {
        const float v = Dt<T>::to_f32(src[d]);
        lo = fminf(lo, v); hi = fmaxf(hi, v);
    }
    lo = warp_min(lo); hi = warp_max(hi);
    const float sc = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), 255.0f), 1e-6f);
    for (int d = lane; d < D; d += 32) {
        const float c = rintf(__fdiv_rn(__fsub_rn(Dt<T>::to_f32(src[d]), lo), sc));
        codes[b * c_sb + h * c_sh + (int64_t)t * c_ss + d] = (uint8_t)fminf(fmaxf(c, 0.f), 255.f);
    }
    if (lane == 0) {
        scale[b * m_sb + h * m_sh + t] = f32_to_bf16_bits(sc);
        mn[b * m_sb + h * m_sh + t] = f32_to_bf16_bits(lo);
    }
}

__global__ void __launch_bounds__(256) dequant_int8_kernel(const uint8_t* __restrict__ codes, int64_t c_sb, int64_t c_sh, int64_t c_ss,
                                                           const uint16_t* __restrict__ scale, const uint16_t* __restrict__ mn,
                                                           int64_t m_sb, int64_t m_sh, int64_t m_s2, int per_page, int B, int H, int S, int D, int page,
                                                           uint16_t* __restrict__ out, int64_t o_sb, int64_t o_sh, int64_t o_ss) {
    const int64_t total = (int64_t)B * H * S * D;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % D);
        int64_t r = i / D;
        const int t = (int)(r % S);
        r /= S;
        const int h = (int)(r % H), b = (int)(r / H);
        const int64_t mo = per_page ? b * m_sb + h * m_sh + (int64_t)(t / page) * m_s2 + d : b * m_sb + h * m_sh + (int64_t)t * m_s2;
        const float v = __fadd_rn(__fmul_rn((float)codes[b * c_sb + h * c_sh + (int64_t)t * c_ss + d], bf16_lo(scale[mo])), bf16_lo(mn[mo]));
        out[b * o_sb + h * o_sh + (int64_t)t * o_ss + d] = f32_to_bf16_bits(v);
    }
}

struct Int8AttnParams {
    const void* Q; int q_dtype; int64_t q_sb, q_sh;
    const uint8_t *K, *V; int64_t kv_sb, kv_sh, kv_ss;
    const uint16_t *K_scale, *K_mn; int64_t km_sb, km_sh, km_sp;
    const uint16_t *V_scale, *V_mn; int64_t vm_sb, vm_sh;
    const int32_t* compact; int64_t cp_sb, cp_sh; int bucket;
    const int32_t* list_count;      // non-null: only the first list_count[row] list entries can be valid
    int vec4;                       // code rows allow 4-byte loads
    const void *K_tail, *V_tail; int tail_dtype; int64_t tl_sb, tl_sh, tl_ss; int tail_len;
    int B, Hq, Hkv, S_kv, P, page;
    float sm_scale;
    float* part_o; float* part_lse; int n_split;      // (n_split, rows, D) fp32 and (n_split, rows): merged by fq_lse_merge
};

__device__ __forceinline__ float i8_ld(const void* p, int dtype, int64_t i) {
    return dtype == FQ_F16 ? __half2float(static_cast<const __half*>(p)[i]) : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

// Grid (n_split, Hq, B), 4 warps.  A warp takes pages of the row's compact list (entry index = split + n_split * (warp +
// 4 * i)); lane owns CPL = D/32 consecutive channels of every token.  Each CTA writes a normalised partial (O, lse).
template <int D>
__global__ void __launch_bounds__(128) sparse_decode_int8_kernel(Int8AttnParams p) {
    constexpr int CPL = D / 32;
    __shared__ float s_m[4], s_l[4];
    __shared__ float s_acc[4][D];
    const int split = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (p.Hq / p.Hkv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float c = p.sm_scale * I8_LOG2E;
    float q[CPL];
#pragma unroll
    for (int j = 0; j < CPL; ++j) q[j] = i8_ld(p.Q, p.q_dtype, b * p.q_sb + hq * p.q_sh + CPL * lane + j) * c;
    float m = -INFINITY, l = 0.f, acc[CPL];
#pragma unroll
    for (int j = 0; j < CPL; ++j) acc[j] = 0.f;
    const int32_t* list = p.compact + b * p.cp_sb + hq * p.cp_sh;
    const uint8_t* Kb = p.K + b * p.kv_sb + hkv * p.kv_sh;
    const uint8_t* Vb = p.V + b * p.kv_sb + hkv * p.kv_sh;
    int n_list = p.bucket;
    if (p.list_count) n_list = max(0, min(n_list, __ldg(p.list_count + b * p.Hq + hq)));
    // four code bytes of this lane's channels as fp32
    auto codes4 = [&](const uint8_t* row, float (&out)[CPL]) {
        if (p.vec4 && CPL == 4) {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(row);
#pragma unroll
            for (int j = 0; j < CPL; ++j) out[j] = (float)((w >> (8 * j)) & 0xffu);
        } else {
#pragma unroll
            for (int j = 0; j < CPL; ++j) out[j] = (float)row[j];
        }
    };
    constexpr int TCH = 8;       // tokens whose logits are formed side by side: their warp reductions overlap
    for (int e = split + p.n_split * warp; e < n_list; e += p.n_split * 4) {
        const int pg = list[e];
        if (pg < 0 || pg >= p.P || pg * p.page >= p.S_kv) continue;
        const int64_t mo = b * p.km_sb + hkv * p.km_sh + (int64_t)pg * p.km_sp + CPL * lane;
        float qs[CPL], qmn = 0.f;
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
            qs[j] = q[j] * bf16_lo(p.K_scale[mo + j]);
            qmn = fmaf(q[j], bf16_lo(p.K_mn[mo + j]), qmn);
        }
        qmn = warp_sum(qmn);
        const int t_end = min((pg + 1) * p.page, p.S_kv);
        for (int t0 = pg * p.page; t0 < t_end; t0 += TCH) {
            float sc[TCH], vs[TCH], vm[TCH];
#pragma unroll
            for (int u = 0; u < TCH; ++u) {
                const int t = min(t0 + u, t_end - 1);        // past the end: a repeat of the last token, masked below
                float kf[CPL];
                codes4(Kb + (int64_t)t * p.kv_ss + CPL * lane, kf);
                float a = 0.f;
#pragma unroll
                for (int j = 0; j < CPL; ++j) a = fmaf(qs[j], kf[j], a);
                sc[u] = a;
                vs[u] = bf16_lo(p.V_scale[b * p.vm_sb + hkv * p.vm_sh + t]);
                vm[u] = bf16_lo(p.V_mn[b * p.vm_sb + hkv * p.vm_sh + t]);
            }
            float mx = -INFINITY;
#pragma unroll
            for (int u = 0; u < TCH; ++u) {
                sc[u] = t0 + u < t_end ? warp_sum(sc[u]) + qmn : -INFINITY;
                mx = fmaxf(mx, sc[u]);
            }
            const float m_new = fmaxf(m, mx);                  // finite: token t0 is valid
            const float al = i8_ex2(m - m_new);
            l *= al;
#pragma unroll
            for (int j = 0; j < CPL; ++j) acc[j] *= al;
#pragma unroll
            for (int u = 0; u < TCH; ++u) {
                const int t = min(t0 + u, t_end - 1);
                const float pr = i8_ex2(sc[u] - m_new);        // 0 past the end
                float vf[CPL];
                codes4(Vb + (int64_t)t * p.kv_ss + CPL * lane, vf);
                l += pr;
                const float ps = pr * vs[u], pm = pr * vm[u];
#pragma unroll
                for (int j = 0; j < CPL; ++j) acc[j] += fmaf(vf[j], ps, pm);
            }
            m = m_new;
        }
    }
    // the staged (unquantised) tail belongs to split 0
    if (split == 0) {
        for (int t = warp; t < p.tail_len; t += 4) {
            const int64_t ro = b * p.tl_sb + hkv * p.tl_sh + (int64_t)t * p.tl_ss + CPL * lane;
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < CPL; ++j) s = fmaf(q[j], i8_ld(p.K_tail, p.tail_dtype, ro + j), s);
            s = warp_sum(s);
            const float m_new = fmaxf(m, s);
            const float al = i8_ex2(m - m_new), pr = i8_ex2(s - m_new);
            l = l * al + pr;
#pragma unroll
            for (int j = 0; j < CPL; ++j) acc[j] = fmaf(pr, i8_ld(p.V_tail, p.tail_dtype, ro + j), acc[j] * al);
            m = m_new;
        }
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int j = 0; j < CPL; ++j) s_acc[warp][CPL * lane + j] = acc[j];
    __syncthreads();
    float mx = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
    float lsum = 0.f, o = 0.f;
    const int d = threadIdx.x;
    if (mx != -INFINITY) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float wgt = i8_ex2(s_m[w] - mx);
            lsum = fmaf(s_l[w], wgt, lsum);
            if (d < D) o = fmaf(s_acc[w][d], wgt, o);
        }
    }
    const int64_t row = (int64_t)b * p.Hq + hq, rows = (int64_t)p.B * p.Hq;
    if (d < D) p.part_o[((int64_t)split * rows + row) * D + d] = lsum > 0.f ? o / lsum : 0.f;
    if (d == 0) p.part_lse[(int64_t)split * rows + row] = lsum > 0.f ? (mx + log2f(lsum)) * I8_LN2 : -INFINITY;
}

// The same computation for 16-byte aligned code and metadata rows.  Eight lanes (a quarter warp) own one token: lane l
// holds D/8 consecutive channels (one 16-byte load of codes at head_dim 128), so a page of 16 tokens is four tokens per
// quarter warp, their loads in flight together, a 3-step shuffle reduction per logit and ONE online-softmax update per
// 16 tokens.  acc holds sum (p * v_scale) * code, the sum of p * v_mn is kept apart and added once at the end; the four
// quarter warps accumulate different tokens of the same channels and are added up before the CTA merge.
template <int D>
__global__ void __launch_bounds__(128) sparse_decode_int8_q_kernel(Int8AttnParams p) {
    constexpr int DPL = D / 8;          // channels per lane
    constexpr int NW = DPL / 4;         // 32-bit words of codes per lane and token
    __shared__ float s_m[4], s_l[4];
    __shared__ float s_acc[4][D];
    const int split = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (p.Hq / p.Hkv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane & 7, qw = lane >> 3;
    const float c = p.sm_scale * I8_LOG2E;
    float q[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) q[j] = i8_ld(p.Q, p.q_dtype, b * p.q_sb + hq * p.q_sh + DPL * l + j) * c;
    float m = -INFINITY, lsum = 0.f, mnacc = 0.f, acc[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[j] = 0.f;
    auto quarter_sum = [](float v) {
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        return v;
    };
    auto warp_max4 = [](float v) {       // over the four quarter warps (lanes of a quarter hold equal values)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
        return v;
    };
    // byte k of w as fp32: the byte becomes the low mantissa byte of 2^23 (one byte permute), which is then subtracted
    auto code_f32 = [](uint32_t w, int k) -> float {
        return __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7540u | (unsigned)k)) - 8388608.0f;
    };
    auto load_codes = [&](const uint8_t* row, uint32_t (&w)[NW]) {
        if constexpr (NW == 4) { const uint4 u = *reinterpret_cast<const uint4*>(row); w[0] = u.x; w[1] = u.y; w[2] = u.z; w[3] = u.w; }
        else { const uint2 u = *reinterpret_cast<const uint2*>(row); w[0] = u.x; w[1] = u.y; }
    };
    const int32_t* list = p.compact + b * p.cp_sb + hq * p.cp_sh;
    const uint8_t* Kb = p.K + b * p.kv_sb + hkv * p.kv_sh + DPL * l;
    const uint8_t* Vb = p.V + b * p.kv_sb + hkv * p.kv_sh + DPL * l;
    const uint16_t* Vsc = p.V_scale + b * p.vm_sb + hkv * p.vm_sh;
    const uint16_t* Vmn = p.V_mn + b * p.vm_sb + hkv * p.vm_sh;
    int n_list = p.bucket;
    if (p.list_count) n_list = max(0, min(n_list, __ldg(p.list_count + b * p.Hq + hq)));
    for (int e = split + p.n_split * warp; e < n_list; e += p.n_split * 4) {
        const int pg = list[e];
        if (pg < 0 || pg >= p.P || pg * p.page >= p.S_kv) continue;
        const int64_t mo = b * p.km_sb + hkv * p.km_sh + (int64_t)pg * p.km_sp + DPL * l;
        float qs[DPL], qmn = 0.f;
#pragma unroll
        for (int c8 = 0; c8 < DPL / 8; ++c8) {
            float sc8[8], mn8[8];
            load8<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(p.K_scale + mo) + 8 * c8, sc8);
            load8<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(p.K_mn + mo) + 8 * c8, mn8);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                qs[8 * c8 + j] = q[8 * c8 + j] * sc8[j];
                qmn = fmaf(q[8 * c8 + j], mn8[j], qmn);
            }
        }
        qmn = quarter_sum(qmn);
        const int t_end = min((pg + 1) * p.page, p.S_kv);
        for (int t0 = pg * p.page; t0 < t_end; t0 += 16) {
            uint32_t kw[4][NW], vw[4][NW];
            float vs[4], vm[4], sc[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int t = min(t0 + qw + 4 * u, t_end - 1);      // past the end: a repeat of the last token, masked below
                load_codes(Kb + (int64_t)t * p.kv_ss, kw[u]);
                load_codes(Vb + (int64_t)t * p.kv_ss, vw[u]);
                vs[u] = bf16_lo(Vsc[t]);
                vm[u] = bf16_lo(Vmn[t]);
            }
            float mx = -INFINITY;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float a = 0.f;
#pragma unroll
                for (int w = 0; w < NW; ++w)
#pragma unroll
                    for (int k = 0; k < 4; ++k) a = fmaf(qs[4 * w + k], code_f32(kw[u][w], k), a);
                a = quarter_sum(a);
                sc[u] = t0 + qw + 4 * u < t_end ? a + qmn : -INFINITY;
                mx = fmaxf(mx, sc[u]);
            }
            mx = warp_max4(mx);
            const float m_new = fmaxf(m, mx);                  // finite: token t0 is valid
            const float al = i8_ex2(m - m_new);
            lsum *= al; mnacc *= al;
#pragma unroll
            for (int j = 0; j < DPL; ++j) acc[j] *= al;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float pr = i8_ex2(sc[u] - m_new);        // 0 past the end
                const float ps = pr * vs[u];
                lsum += pr;
                mnacc = fmaf(pr, vm[u], mnacc);
#pragma unroll
                for (int w = 0; w < NW; ++w)
#pragma unroll
                    for (int k = 0; k < 4; ++k) acc[4 * w + k] = fmaf(ps, code_f32(vw[u][w], k), acc[4 * w + k]);
            }
            m = m_new;
        }
    }
    // the staged (unquantised) tail belongs to split 0: a quarter warp per token
    if (split == 0) {
        for (int t0 = 4 * warp; t0 < p.tail_len; t0 += 16) {       // warp-uniform trip count
            const int t = t0 + qw;
            const bool live = t < p.tail_len;
            const int64_t ro = b * p.tl_sb + hkv * p.tl_sh + (int64_t)(live ? t : 0) * p.tl_ss + DPL * l;
            float a = 0.f;
#pragma unroll
            for (int j = 0; j < DPL; ++j) a = fmaf(q[j], i8_ld(p.K_tail, p.tail_dtype, ro + j), a);
            a = quarter_sum(a);
            const float s = live ? a : -INFINITY;
            const float m_new = fmaxf(m, warp_max4(s));        // finite: token t0 is live
            const float al = i8_ex2(m - m_new), pr = i8_ex2(s - m_new);
            lsum = lsum * al + pr;
            mnacc *= al;
#pragma unroll
            for (int j = 0; j < DPL; ++j) acc[j] = fmaf(pr, live ? i8_ld(p.V_tail, p.tail_dtype, ro + j) : 0.f, acc[j] * al);
            m = m_new;
        }
    }
    // the four quarter warps hold partial sums over different tokens of the same channels
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {
        lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
        mnacc += __shfl_xor_sync(0xffffffffu, mnacc, off);
#pragma unroll
        for (int j = 0; j < DPL; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = lsum; }
    if (qw == 0) {
#pragma unroll
        for (int j = 0; j < DPL; ++j) s_acc[warp][DPL * l + j] = acc[j] + mnacc;
    }
    __syncthreads();
    float mx = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
    float ltot = 0.f, o = 0.f;
    const int d = threadIdx.x;
    if (mx != -INFINITY) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float wgt = i8_ex2(s_m[w] - mx);
            ltot = fmaf(s_l[w], wgt, ltot);
            if (d < D) o = fmaf(s_acc[w][d], wgt, o);
        }
    }
    const int64_t row = (int64_t)b * p.Hq + hq, rows = (int64_t)p.B * p.Hq;
    if (d < D) p.part_o[((int64_t)split * rows + row) * D + d] = ltot > 0.f ? o / ltot : 0.f;
    if (d == 0) p.part_lse[(int64_t)split * rows + row] = ltot > 0.f ? (mx + log2f(ltot)) * I8_LN2 : -INFINITY;
}

// merge of the splits' normalised partial results (fp32) into O (q dtype) and lse; one warp per row
__global__ void __launch_bounds__(128) int8_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, int n_split,
                                                         int64_t rows, int D, void* __restrict__ O, int q_dtype, float* __restrict__ lse) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= rows) return;
    float m = -INFINITY;
    for (int i = 0; i < n_split; ++i) m = fmaxf(m, part_lse[i * rows + r]);
    float wsum = 0.f;
    if (m != -INFINITY)
        for (int i = 0; i < n_split; ++i) wsum += expf(part_lse[i * rows + r] - m);
    for (int d = lane; d < D; d += 32) {
        float a = 0.f;
        if (m != -INFINITY)
            for (int i = 0; i < n_split; ++i) a = fmaf(expf(part_lse[i * rows + r] - m), part_o[(i * rows + r) * D + d], a);
        const float v = m != -INFINITY ? a / wsum : 0.f;
        if (q_dtype == FQ_F16) static_cast<__half*>(O)[r * D + d] = __float2half_rn(v);
        else static_cast<__nv_bfloat16*>(O)[r * D + d] = __float2bfloat16_rn(v);
    }
    if (lane == 0 && lse) lse[r] = m != -INFINITY ? m + logf(wsum) : -INFINITY;
}

template <typename T>
static void launch_quant_int8(const void* K, const void* V, int64_t in_sb, int64_t in_sh, int64_t in_ss, int B, int H, int S, int D, int page,
                              uint8_t* Kc, uint8_t* Vc, int64_t c_sb, int64_t c_sh, int64_t c_ss,
                              uint16_t* Ks, uint16_t* Km, int64_t km_sb, int64_t km_sh, int64_t km_sp,
                              uint16_t* Vs, uint16_t* Vm, int64_t vm_sb, int64_t vm_sh, cudaStream_t st) {
    if (K) {
        const int64_t warps = (int64_t)B * H * ((S + page - 1) / page);
        quant_k_int8_kernel<T><<<(unsigned)((warps + 3) / 4), 128, 0, st>>>(static_cast<const T*>(K), in_sb, in_sh, in_ss, B, H, S, D, page,
                                                                          Kc, c_sb, c_sh, c_ss, Ks, Km, km_sb, km_sh, km_sp);
    }
    if (V) {
        const int64_t warps = (int64_t)B * H * S;
        quant_v_int8_kernel<T><<<(unsigned)((warps + 3) / 4), 128, 0, st>>>(static_cast<const T*>(V), in_sb, in_sh, in_ss, B, H, S, D,
                                                                          Vc, c_sb, c_sh, c_ss, Vs, Vm, vm_sb, vm_sh);
    }
}

}  // namespace fq

extern "C" int fq_quantize_kv_int8(
    const void* K, const void* V, int64_t in_sb, int64_t in_sh, int64_t in_ss, int dtype, int B, int H, int S, int D, int page,
    uint8_t* K_uint8, uint8_t* V_uint8, int64_t c_sb, int64_t c_sh, int64_t c_ss,
    void* K_scale, void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    void* V_scale, void* V_mn, int64_t vm_sb, int64_t vm_sh, void* stream) {
    using namespace fq;
    const char* fn = "fq_quantize_kv_int8";
    FQ_CHECK_ARG(B > 0 && H > 0 && S >= 0 && D > 0 && page > 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(dtype == FQ_F32 || dtype == FQ_F16 || dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: dtype code %d", fn, dtype);
    FQ_CHECK_ARG(!K || (K_uint8 && K_scale && K_mn), FQ_ERR_ARG, "%s: K given without its outputs", fn);
    FQ_CHECK_ARG(!V || (V_uint8 && V_scale && V_mn), FQ_ERR_ARG, "%s: V given without its outputs", fn);
    FQ_CHECK_ARG((int64_t)B * H * S <= 0x7fffffffLL * 4, FQ_ERR_ARG, "%s: too many tokens for one launch", fn);
    if (S == 0) return FQ_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint16_t *ks = static_cast<uint16_t*>(K_scale), *km = static_cast<uint16_t*>(K_mn), *vs = static_cast<uint16_t*>(V_scale), *vm = static_cast<uint16_t*>(V_mn);
    if (dtype == FQ_F32) launch_quant_int8<float>(K, V, in_sb, in_sh, in_ss, B, H, S, D, page, K_uint8, V_uint8, c_sb, c_sh, c_ss, ks, km, km_sb, km_sh, km_sp, vs, vm, vm_sb, vm_sh, st);
    else if (dtype == FQ_F16) launch_quant_int8<__half>(K, V, in_sb, in_sh, in_ss, B, H, S, D, page, K_uint8, V_uint8, c_sb, c_sh, c_ss, ks, km, km_sb, km_sh, km_sp, vs, vm, vm_sb, vm_sh, st);
    else launch_quant_int8<__nv_bfloat16>(K, V, in_sb, in_sh, in_ss, B, H, S, D, page, K_uint8, V_uint8, c_sb, c_sh, c_ss, ks, km, km_sb, km_sh, km_sp, vs, vm, vm_sb, vm_sh, st);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" int fq_dequantize_int8(
    const uint8_t* codes, int64_t c_sb, int64_t c_sh, int64_t c_ss,
    const void* scale, const void* mn, int64_t m_sb, int64_t m_sh, int64_t m_s2,
    int per_page, int B, int H, int S, int D, int page, void* out, int64_t o_sb, int64_t o_sh, int64_t o_ss, void* stream) {
    using namespace fq;
    const char* fn = "fq_dequantize_int8";
    FQ_CHECK_ARG(B > 0 && H > 0 && S >= 0 && D > 0 && page > 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    if (S == 0) return FQ_OK;
    FQ_CHECK_ARG(codes && scale && mn && out, FQ_ERR_ARG, "%s: null pointer", fn);
    const int64_t total = (int64_t)B * H * S * D;
    const int64_t want = (total + 255) / 256;
    dequant_int8_kernel<<<(unsigned)(want < 148 * 16 ? want : 148 * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        codes, c_sb, c_sh, c_ss, static_cast<const uint16_t*>(scale), static_cast<const uint16_t*>(mn), m_sb, m_sh, m_s2, per_page,
        B, H, S, D, page, static_cast<uint16_t*>(out), o_sb, o_sh, o_ss);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" size_t fq_sparse_decode_int8_workspace_bytes(int B, int Hq, int D, int n_split) {
    if (B <= 0 || Hq <= 0 || D <= 0 || n_split < 1) return 0;
    return (size_t)n_split * B * Hq * (D + 1) * 4;
}

extern "C" int fq_sparse_decode_int8_counted(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_uint8, const uint8_t* V_uint8, int64_t kv_sb, int64_t kv_sh, int64_t kv_ss,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket, const int32_t* list_count,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss, int tail_len,
    int B, int Hq, int Hkv, int S_kv, int P, int D, int page, float sm_scale,
    void* O, float* lse, void* workspace, size_t workspace_bytes, int n_split, void* stream) {
    using namespace fq;
    const char* fn = "fq_sparse_decode_int8";
    FQ_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && S_kv >= 0 && P >= 0 && bucket >= 0 && tail_len >= 0 && page > 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(B <= 65535 && Hq <= 65535, FQ_ERR_ARG, "%s: B and H_q must be <= 65535", fn);
    FQ_CHECK_ARG(Hq % Hkv == 0, FQ_ERR_ARG, "%s: H_q=%d must be divisible by H_kv=%d", fn, Hq, Hkv);
    FQ_CHECK_ARG(D == 64 || D == 128, FQ_ERR_UNSUPPORTED, "%s: head_dim=%d not in (64, 128)", fn, D);
    FQ_CHECK_ARG(q_dtype == FQ_F16 || q_dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: Q must be fp16 or bf16 (code %d)", fn, q_dtype);
    FQ_CHECK_ARG(Q && O, FQ_ERR_ARG, "%s: null Q or O", fn);
    FQ_CHECK_ARG(n_split >= 1 && n_split <= 1024, FQ_ERR_ARG, "%s: n_split=%d must be in [1, 1024]", fn, n_split);
    const bool have_pages = bucket > 0 && P > 0 && S_kv > 0;
    if (have_pages) FQ_CHECK_ARG(K_uint8 && V_uint8 && K_scale && K_mn && V_scale && V_mn && compact, FQ_ERR_ARG, "%s: null cache pointer", fn);
    if (tail_len > 0) {
        FQ_CHECK_ARG(K_tail && V_tail, FQ_ERR_ARG, "%s: null tail pointer", fn);
        FQ_CHECK_ARG(tail_dtype == FQ_F16 || tail_dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: tail must be fp16 or bf16", fn);
    }
    const size_t need = fq_sparse_decode_int8_workspace_bytes(B, Hq, D, n_split);
    FQ_CHECK_ARG(workspace && workspace_bytes >= need, FQ_ERR_WORKSPACE, "%s: workspace of %zu B needed, %zu given", fn, need, workspace_bytes);
    Int8AttnParams p;
    p.Q = Q; p.q_dtype = q_dtype; p.q_sb = q_sb; p.q_sh = q_sh;
    p.K = K_uint8; p.V = V_uint8; p.kv_sb = kv_sb; p.kv_sh = kv_sh; p.kv_ss = kv_ss;
    p.K_scale = static_cast<const uint16_t*>(K_scale); p.K_mn = static_cast<const uint16_t*>(K_mn); p.km_sb = km_sb; p.km_sh = km_sh; p.km_sp = km_sp;
    p.V_scale = static_cast<const uint16_t*>(V_scale); p.V_mn = static_cast<const uint16_t*>(V_mn); p.vm_sb = vm_sb; p.vm_sh = vm_sh;
    p.compact = compact; p.cp_sb = cp_sb; p.cp_sh = cp_sh; p.bucket = have_pages ? bucket : 0;
    p.list_count = list_count;
    p.vec4 = (have_pages && aligned(K_uint8, 4) && aligned(V_uint8, 4) && kv_sb % 4 == 0 && kv_sh % 4 == 0 && kv_ss % 4 == 0) ? 1 : 0;
    p.K_tail = K_tail; p.V_tail = V_tail; p.tail_dtype = tail_dtype; p.tl_sb = tl_sb; p.tl_sh = tl_sh; p.tl_ss = tl_ss; p.tail_len = tail_len;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.S_kv = S_kv; p.P = P; p.page = page; p.sm_scale = sm_scale;
    p.n_split = n_split;
    p.part_o = static_cast<float*>(workspace);
    p.part_lse = p.part_o + (size_t)n_split * B * Hq * D;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid((unsigned)n_split, (unsigned)Hq, (unsigned)B);
    // 16-byte aligned code and metadata rows: the quarter-warp-per-token kernel
    const bool vec16 = have_pages && aligned(K_uint8, 16) && aligned(V_uint8, 16) && kv_sb % 16 == 0 && kv_sh % 16 == 0 && kv_ss % 16 == 0 &&
                       aligned(K_scale, 16) && aligned(K_mn, 16) && km_sb % 8 == 0 && km_sh % 8 == 0 && km_sp % 8 == 0;
    if (vec16) {
        if (D == 128) sparse_decode_int8_q_kernel<128><<<grid, 128, 0, st>>>(p);
        else sparse_decode_int8_q_kernel<64><<<grid, 128, 0, st>>>(p);
    } else {
        if (D == 128) sparse_decode_int8_kernel<128><<<grid, 128, 0, st>>>(p);
        else sparse_decode_int8_kernel<64><<<grid, 128, 0, st>>>(p);
    }
    FQ_CHECK_LAUNCH(fn);
    const int64_t rows = (int64_t)B * Hq;
    int8_merge_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(p.part_o, p.part_lse, n_split, rows, D, O, q_dtype, lse);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" int fq_sparse_decode_int8(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_uint8, const uint8_t* V_uint8, int64_t kv_sb, int64_t kv_sh, int64_t kv_ss,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss, int tail_len,
    int B, int Hq, int Hkv, int S_kv, int P, int D, int page, float sm_scale,
    void* O, float* lse, void* workspace, size_t workspace_bytes, int n_split, void* stream) {
    return fq_sparse_decode_int8_counted(Q, q_dtype, q_sb, q_sh, K_uint8, V_uint8, kv_sb, kv_sh, kv_ss, K_scale, K_mn, km_sb, km_sh, km_sp,
                                         V_scale, V_mn, vm_sb, vm_sh, compact, cp_sb, cp_sh, bucket, nullptr,
                                         K_tail, V_tail, tail_dtype, tl_sb, tl_sh, tl_ss, tail_len, B, Hq, Hkv, S_kv, P, D, page, sm_scale,
                                         O, lse, workspace, workspace_bytes, n_split, stream);
}
