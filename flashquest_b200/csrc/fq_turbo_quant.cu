// Walsh-Hadamard rotation and TurboQuant K3-V3 packing (3-bit Lloyd-Max codes in a 1-bit and
// a 2-bit plane, per-token RMS scale).
//
// One warp owns one token row of D values; lane l holds the D/32 consecutive values starting
// at l*D/32.  The butterfly stages with a stride inside a lane are register-only, the others
// exchange with lane ^ (stride / values-per-lane) by shuffle.  Every stage is rounded to the
// tensor's dtype exactly as the reference's eager ops do (kernel/wht.py:26-41), so results are
// bit-identical.  HBM-bound: D*sizeof(T) in, 3*D/8 + 2 bytes out per token.
#include "fq_common.cuh"

namespace fq {

// kernel/kv_quant.py:225-229
__device__ __constant__ float c_turbo_codebook[8] = {-2.1519f, -1.3439f, -0.7560f, -0.2451f,
                                                     0.2451f, 0.7560f, 1.3439f, 2.1519f};

// Packed 16-bit arithmetic for the butterflies.  The reference adds two values of dtype T in
// T: that is the correctly rounded sum, and so is rn_T(fp32 sum) because rounding first to 24
// and then to 11 (or 8) bits is innocuous when 24 >= 2*11 + 2; the packed add is the same
// correctly rounded sum, two values per instruction and no conversions.
template <typename T> struct Pk2;
template <> struct Pk2<__half> {
    using type = __half2;
    __device__ static type make(float a, float b) { return __floats2half2_rn(a, b); }
    __device__ static float2 unpack(type x) { return __half22float2(x); }
};
template <> struct Pk2<__nv_bfloat16> {
    using type = __nv_bfloat162;
    __device__ static type make(float a, float b) { return __floats2bfloat162_rn(a, b); }
    __device__ static float2 unpack(type x) { return __bfloat1622float2(x); }
};
template <typename P2> __device__ __forceinline__ uint32_t p2_bits(P2 x) { return *reinterpret_cast<uint32_t*>(&x); }
template <typename P2> __device__ __forceinline__ P2 p2_from(uint32_t u) { return *reinterpret_cast<P2*>(&u); }

// In-place WHT of the row spread over the warp: v[j] is element lane*EPL + j.
template <typename T, int EPL>
__device__ __forceinline__ void wht_lanes(float (&v)[EPL], int lane, int D) {
    if constexpr (sizeof(T) == 2 && EPL >= 2) {
        using P2 = typename Pk2<T>::type;
        constexpr int NP = EPL / 2;
        P2 x[NP];
#pragma unroll
        for (int i = 0; i < NP; ++i) x[i] = Pk2<T>::make(v[2 * i], v[2 * i + 1]);      // exact: the values are T already
        // stride 1: (a, b) -> (a + b, a - b)
#pragma unroll
        for (int i = 0; i < NP; ++i) {
            const uint32_t u = p2_bits(x[i]);
            const P2 aa = p2_from<P2>(__byte_perm(u, u, 0x1010));                         // (a, a)
            const P2 bm = p2_from<P2>(__byte_perm(u, u, 0x3232) ^ 0x80000000u);           // (b, -b)
            x[i] = __hadd2(aa, bm);
        }
        // strides 2 .. EPL/2: whole registers
#pragma unroll
        for (int h = 1; h < NP; h <<= 1) {
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                if ((i & h) == 0) {
                    const P2 a = x[i], b = x[i + h];
                    x[i] = __hadd2(a, b);
                    x[i + h] = __hsub2(a, b);
                }
            }
        }
        // strides >= EPL: partner lane; the upper lane of a pair computes other - mine
        for (int h = EPL; h < D; h <<= 1) {
            const int lo = h / EPL;
            const uint32_t flip = (lane & lo) ? 0x80008000u : 0u;
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                const uint32_t mine = p2_bits(x[i]);
                const uint32_t other = __shfl_xor_sync(0xffffffffu, mine, lo);
                x[i] = __hadd2(p2_from<P2>(other), p2_from<P2>(mine ^ flip));
            }
        }
        const float cd = (float)sqrt((double)D);
#pragma unroll
        for (int i = 0; i < NP; ++i) {
            const float2 f = Pk2<T>::unpack(x[i]);
            v[2 * i] = Dt<T>::rn(__fdiv_rn(f.x, cd));
            v[2 * i + 1] = Dt<T>::rn(__fdiv_rn(f.y, cd));
        }
    } else {
#pragma unroll
    for (int h = 1; h < EPL; h <<= 1) {
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            if ((j & h) == 0) {
                const float a = v[j], b = v[j + h];
                v[j] = Dt<T>::rn(__fadd_rn(a, b));
                v[j + h] = Dt<T>::rn(__fsub_rn(a, b));
            }
        }
    }
    for (int h = EPL; h < D; h <<= 1) {
        const int lo = h / EPL;                 // partner lane distance
        const bool upper = (lane & lo) != 0;    // this lane holds the "b" half of the pair
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], lo);
            v[j] = upper ? Dt<T>::rn(__fsub_rn(other, v[j])) : Dt<T>::rn(__fadd_rn(v[j], other));
        }
    }
    const float cd = (float)sqrt((double)D);    // the divisor the reference uses: fp32(math.sqrt(D))
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = Dt<T>::rn(__fdiv_rn(v[j], cd));
    }
}

template <typename T, int EPL>
__device__ __forceinline__ void load_row(const T* row, int lane, int D, float (&v)[EPL]) {
    if constexpr (EPL == 4 && sizeof(T) == 2) {
        // four 16-bit values of a lane in one 8-byte load when the row allows it
        if ((reinterpret_cast<uintptr_t>(row) & 7) == 0 && D == 128) {
            const uint2 u = *reinterpret_cast<const uint2*>(row + 4 * lane);
            const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = Dt<T>::to_f32(e[j]);
            return;
        }
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const int i = lane * EPL + j;
        v[j] = i < D ? Dt<T>::to_f32(row[i]) : 0.f;
    }
}

// wht_along_head_dim (kernel/wht.py:17): rows of D values, dtype preserved.
template <typename T, int EPL>
__global__ void __launch_bounds__(128) wht_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n_rows, int D) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    float v[EPL];
    load_row<T, EPL>(x + row * D, lane, D, v);
    wht_lanes<T, EPL>(v, lane, D);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const int i = lane * EPL + j;
        if (i < D) out[row * D + i] = from_f32<T>(v[j]);
    }
}

struct TurboParams {
    const void *head, *nw;                       // token stream: head[0:n_head] ++ new
    int64_t hd_sb, hd_sh, hd_ss, nw_sb, nw_sh, nw_ss;
    int n_head, n_quant, D;
    uint8_t *msb, *lsb;                          // (B,H,n,D/8), (B,H,n,D/4)
    int64_t ms_sb, ms_sh, ms_ss, ls_sb, ls_sh, ls_ss;
    uint16_t* scale;                             // (B,H,n) bf16
    int64_t sc_sb, sc_sh, sc_ss;
};

// quantize_k_turbo / quantize_v_turbo without the raw page metadata
// (kernel/kv_quant.py:327-405): rot = WHT(x) in x's dtype; s = max(sqrt(mean(rot^2)), 1e-6) in
// fp32 (lane partial sums in ascending order, then an xor butterfly 16,8,4,2,1);
// idx = first index of min |rot/s - c_j|; planes per kv_quant.py:253-279.
template <typename T, int EPL>
__global__ void __launch_bounds__(128) turbo_quant_kernel(TurboParams p) {
    __shared__ uint8_t s_idx[4][1024];
    __shared__ float s_cb[9];          // the codebook where lanes may index it independently, +inf behind it
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = blockIdx.z, h = blockIdx.y;
    const int t = blockIdx.x * 4 + warp;
    if (threadIdx.x < 9) s_cb[threadIdx.x] = threadIdx.x < 8 ? c_turbo_codebook[threadIdx.x] : INFINITY;
    __syncthreads();
    if (t >= p.n_quant) return;
    const int D = p.D;
    const T* row = t < p.n_head
        ? static_cast<const T*>(p.head) + b * p.hd_sb + h * p.hd_sh + (int64_t)t * p.hd_ss
        : static_cast<const T*>(p.nw) + b * p.nw_sb + h * p.nw_sh + (int64_t)(t - p.n_head) * p.nw_ss;
    float v[EPL];
    load_row<T, EPL>(row, lane, D, v);
    wht_lanes<T, EPL>(v, lane, D);
    float a = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) a = __fmaf_rn(v[j], v[j], a);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, off));
    const float s = fmaxf(__fsqrt_rn(__fdiv_rn(a, (float)D)), 1e-6f);
    // Nearest codebook entry, first index on ties (torch.argmin): the codebook is sorted, so
    // the winner is one of the two entries around y; which one is decided by the same fp32
    // distances the reference compares.
    auto nearest = [&](float y, float& d0, float& d1) -> int {
        int k = y >= 0.2451f ? 4 : 0;                          // c_4
        k += y >= (k ? 1.3439f : -0.7560f) ? 2 : 0;           // c_6 or c_2
        k += y >= s_cb[k + 1] ? 1 : 0;
        k = min(k, 6);                                        // c_k <= y < c_{k+1}, clamped at both ends
        d0 = fabsf(__fsub_rn(y, s_cb[k]));
        d1 = fabsf(__fsub_rn(y, s_cb[k + 1]));
        return k;
    };
    unsigned idx[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        float d0, d1;
        const int k = nearest(__fdiv_rn(v[j], s), d0, d1);
        idx[j] = (unsigned)(k + (d1 < d0 ? 1 : 0));
    }
    uint8_t* msb = p.msb + b * p.ms_sb + h * p.ms_sh + (int64_t)t * p.ms_ss;
    uint8_t* lsb = p.lsb + b * p.ls_sb + h * p.ls_sh + (int64_t)t * p.ls_ss;
    if constexpr (EPL == 4) {
        // lane = channels 4l..4l+3: exactly one byte of the 2-bit plane, half a byte of the 1-bit plane
        unsigned l8 = 0, m4 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) { l8 |= (idx[j] & 3u) << (2 * j); m4 |= ((idx[j] >> 2) & 1u) << j; }
        const unsigned hi = __shfl_down_sync(0xffffffffu, m4, 1);
        if (4 * lane < D) lsb[lane] = (uint8_t)l8;
        if ((lane & 1) == 0 && 4 * lane < D) msb[lane >> 1] = (uint8_t)(m4 | (hi << 4));
    } else {
        uint8_t* si = s_idx[warp];
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const int i = lane * EPL + j;
            if (i < D) si[i] = (uint8_t)idx[j];
        }
        __syncwarp();
        for (int k = lane; k < D / 8; k += 32) {
            unsigned m = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) m |= (unsigned)((si[8 * k + i] >> 2) & 1) << i;
            msb[k] = (uint8_t)m;
        }
        for (int k = lane; k < D / 4; k += 32) {
            unsigned m = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) m |= (unsigned)(si[4 * k + i] & 3) << (2 * i);
            lsb[k] = (uint8_t)m;
        }
    }
    if (lane == 0) p.scale[b * p.sc_sb + h * p.sc_sh + (int64_t)t * p.sc_ss] = f32_to_bf16_bits(s);
}

// The same coding for the shape that matters (head_dim 128, 16-bit values, 8-byte aligned rows) with about half the
// instructions; results are bit-identical to turbo_quant_kernel (the tests compare both with the reference's planes).
//  * the row stays packed (two values per register) from the load to the end of the butterflies; a butterfly with a
//    partner lane is one shuffle and one packed fma(mine, +-1, other), which rounds once like the add it replaces;
//  * x / fp32(sqrt(128)) rounded to the dtype: for every one of the 65 536 bit patterns the quotient, once rounded to
//    the dtype, equals the rounding of q1 = fma(fma(-q0, cd, x), 1/cd, q0), q0 = x * (1/cd) (fp16), resp. of q0
//    itself (bf16) -- checked exhaustively on the host; only the sign of a zero can differ, which no later step sees;
//  * the nearest codebook entry of y = v / s is found without the division: |v| against the three midpoints times s.
//    A value within 3e-5 (relative) of a midpoint, or that close to zero, takes the exact path (division, the
//    reference's fp32 distances, first index on ties) -- the reference's decision can differ from the midpoint
//    comparison only within a few fp32 roundings (1e-7 relative) of a midpoint;
//  * a warp codes four consecutive tokens in a loop that is NOT unrolled (a short body keeps instruction fetch off
//    the stall list), the next row requested while the current one is coded.
// The reference's own decision (kernel/kv_quant.py:253-279): fp32 quotient, fp32 distances, first index on ties.
// Out of line: it runs for a few values in 10^4 and should not lengthen the loop body.
__device__ __noinline__ unsigned turbo_idx_exact(float v, float s) {
    const float y = __fdiv_rn(v, s);
    int k = y >= 0.2451f ? 4 : 0;
    k += y >= (k ? 1.3439f : -0.7560f) ? 2 : 0;
    k += y >= c_turbo_codebook[k + 1] ? 1 : 0;
    k = min(k, 6);
    const float d0 = fabsf(__fsub_rn(y, c_turbo_codebook[k])), d1 = fabsf(__fsub_rn(y, c_turbo_codebook[k + 1]));
    return (unsigned)(k + (d1 < d0 ? 1 : 0));
}

template <typename T>
__global__ void __launch_bounds__(128) turbo_quant128_kernel(TurboParams p) {
    using P2 = typename Pk2<T>::type;
    constexpr int TPW = 4, D = 128;
    constexpr bool IS_HALF = sizeof(T) == 2 && Dt<T>::code == FQ_F16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = blockIdx.z, h = blockIdx.y;
    const int t0 = (blockIdx.x * 4 + warp) * TPW;
    if (t0 >= p.n_quant) return;
    const int nt = min(TPW, p.n_quant - t0);
    const T* head = static_cast<const T*>(p.head) + b * p.hd_sb + h * p.hd_sh;
    const T* nw = static_cast<const T*>(p.nw) + b * p.nw_sb + h * p.nw_sh;
    uint8_t* msb = p.msb + b * p.ms_sb + h * p.ms_sh;
    uint8_t* lsb = p.lsb + b * p.ls_sb + h * p.ls_sh;
    uint16_t* scale = p.scale + b * p.sc_sb + h * p.sc_sh;

    auto load_row8 = [&](int t) -> uint2 {
        const T* row = t < p.n_head ? head + (int64_t)t * p.hd_ss : nw + (int64_t)(t - p.n_head) * p.nw_ss;
        return *reinterpret_cast<const uint2*>(row + 4 * lane);
    };
    uint2 raw_next = load_row8(t0);
    const uint32_t one = IS_HALF ? 0x3c003c00u : 0x3f803f80u, neg = one | 0x80008000u;
    const P2 pm = p2_from<P2>(IS_HALF ? 0xbc003c00u : 0xbf803f80u);              // (+1, -1)
    P2 sgn[5];                                                                   // (+-1, +-1): -1 in the upper lane of a pair
#pragma unroll
    for (int st = 0; st < 5; ++st) sgn[st] = p2_from<P2>((lane >> st) & 1 ? neg : one);
    constexpr float cd = 11.313708498984761f;                                    // fp32(sqrt(128)), the reference's divisor
    constexpr float rcd = 1.0f / cd;
    // midpoints between neighbouring codebook magnitudes
    constexpr float M0 = 0.50055f, M1 = 1.04995f, M2 = 1.7479f, GUARD = 3e-5f;

#pragma unroll 1
    for (int i = 0; i < nt; ++i) {
        const int t = t0 + i;
        const uint2 raw = raw_next;
        if (i + 1 < nt) raw_next = load_row8(t + 1);       // in flight while this token is coded
        P2 x[2] = {p2_from<P2>(raw.x), p2_from<P2>(raw.y)};
        // stride 1: (a, b) -> (a + b, a - b)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t u = p2_bits(x[r]);
            x[r] = __hfma2(p2_from<P2>(__byte_perm(u, u, 0x3232)), pm, p2_from<P2>(__byte_perm(u, u, 0x1010)));
        }
        // stride 2: the lane's two registers
        {
            const P2 a = x[0], c = x[1];
            x[0] = __hadd2(a, c);
            x[1] = __hsub2(a, c);
        }
        // strides 4 .. 64: partner lane
#pragma unroll
        for (int st = 0; st < 5; ++st) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const P2 other = p2_from<P2>(__shfl_xor_sync(0xffffffffu, p2_bits(x[r]), 1 << st));
                x[r] = __hfma2(x[r], sgn[st], other);
            }
        }
        // divide by sqrt(128), round to the dtype
        float v[4];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float2 f = Pk2<T>::unpack(x[r]);
            float qx = __fmul_rn(f.x, rcd), qy = __fmul_rn(f.y, rcd);
            if constexpr (IS_HALF) {
                qx = __fmaf_rn(__fmaf_rn(-qx, cd, f.x), rcd, qx);
                qy = __fmaf_rn(__fmaf_rn(-qy, cd, f.y), rcd, qy);
            }
            const float2 g = Pk2<T>::unpack(Pk2<T>::make(qx, qy));
            v[2 * r] = g.x; v[2 * r + 1] = g.y;
        }
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) a = __fmaf_rn(v[j], v[j], a);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, off));
        const float s = fmaxf(__fsqrt_rn(__fmul_rn(a, 1.0f / D)), 1e-6f);           // a / 128 is exact either way
        const float th0 = M0 * s, th1 = M1 * s, th2 = M2 * s;
        const float g0 = GUARD * th0, g1 = GUARD * th1, g2 = GUARD * th2, gz = GUARD * s;
        unsigned idx[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float av = fabsf(v[j]);
            const int m = (av > th0 ? 1 : 0) + (av > th1 ? 1 : 0) + (av > th2 ? 1 : 0);
            idx[j] = (unsigned)(v[j] < 0.f ? 3 - m : 4 + m);
            const bool risky = fabsf(av - th0) < g0 || fabsf(av - th1) < g1 || fabsf(av - th2) < g2 || av < gz;
            if (risky) idx[j] = turbo_idx_exact(v[j], s);
        }
        unsigned l8 = 0, m4 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) { l8 |= (idx[j] & 3u) << (2 * j); m4 |= ((idx[j] >> 2) & 1u) << j; }
        const unsigned hi = __shfl_down_sync(0xffffffffu, m4, 1);
        lsb[(int64_t)t * p.ls_ss + lane] = (uint8_t)l8;
        if ((lane & 1) == 0) msb[(int64_t)t * p.ms_ss + (lane >> 1)] = (uint8_t)(m4 | (hi << 4));
        if (lane == 0) scale[(int64_t)t * p.sc_ss] = f32_to_bf16_bits(s);
    }
}

// dequantize_k_turbo / dequantize_v_turbo (kernel/kv_quant.py:366-378, :408-420):
// codebook[idx] * scale in fp32, WHT in fp32, cast to bf16.
template <int EPL>
__global__ void __launch_bounds__(128) turbo_dequant_kernel(
    const uint8_t* __restrict__ msb, int64_t ms_sb, int64_t ms_sh, int64_t ms_ss,
    const uint8_t* __restrict__ lsb, int64_t ls_sb, int64_t ls_sh, int64_t ls_ss,
    const uint16_t* __restrict__ scale, int64_t sc_sb, int64_t sc_sh, int64_t sc_ss,
    int S, int D, uint16_t* __restrict__ out, int64_t o_sb, int64_t o_sh, int64_t o_ss) {
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= S) return;
    const uint8_t* mrow = msb + b * ms_sb + h * ms_sh + (int64_t)t * ms_ss;
    const uint8_t* lrow = lsb + b * ls_sb + h * ls_sh + (int64_t)t * ls_ss;
    const float s = bf16_lo(scale[b * sc_sb + h * sc_sh + (int64_t)t * sc_ss]);
    float v[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const int i = lane * EPL + j;
        v[j] = 0.f;
        if (i < D) {
            const unsigned m = (mrow[i >> 3] >> (i & 7)) & 1u;
            const unsigned l2 = (lrow[i >> 2] >> (2 * (i & 3))) & 3u;
            v[j] = __fmul_rn(c_turbo_codebook[(m << 2) | l2], s);
        }
    }
    wht_lanes<float, EPL>(v, lane, D);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const int i = lane * EPL + j;
        if (i < D) out[b * o_sb + h * o_sh + (int64_t)t * o_ss + i] = f32_to_bf16_bits(v[j]);
    }
}

template <typename T>
static int launch_wht(const void* x, void* out, int64_t n_rows, int D, cudaStream_t st) {
    const int epl = D >= 32 ? D / 32 : 1;
    const unsigned blocks = (unsigned)((n_rows + 3) / 4);
#define FQ_W(E) wht_kernel<T, E><<<blocks, 128, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(out), n_rows, D)
    switch (epl) {
        case 1: FQ_W(1); break;
        case 2: FQ_W(2); break;
        case 4: FQ_W(4); break;
        case 8: FQ_W(8); break;
        case 16: FQ_W(16); break;
        default: FQ_W(32); break;
    }
#undef FQ_W
    return FQ_OK;
}

template <typename T>
static void launch_turbo(const TurboParams& p, dim3 grid, cudaStream_t st) {
    const int epl = p.D >= 32 ? p.D / 32 : 1;
#define FQ_T(E) turbo_quant_kernel<T, E><<<grid, 128, 0, st>>>(p)
    switch (epl) {
        case 1: FQ_T(1); break;
        case 2: FQ_T(2); break;
        case 4: FQ_T(4); break;
        case 8: FQ_T(8); break;
        case 16: FQ_T(16); break;
        default: FQ_T(32); break;
    }
#undef FQ_T
}

}  // namespace fq

extern "C" int fq_wht(const void* x, void* out, int dtype, int64_t n_rows, int D, void* stream) {
    using namespace fq;
    const char* fn = "fq_wht";
    FQ_CHECK_ARG(D > 0 && (D & (D - 1)) == 0, FQ_ERR_ARG, "%s: head_dim must be a positive power of 2, got %d", fn, D);
    FQ_CHECK_ARG(D <= 1024, FQ_ERR_UNSUPPORTED, "%s: head_dim %d above 1024", fn, D);
    FQ_CHECK_ARG(n_rows >= 0 && (n_rows == 0 || (x && out)), FQ_ERR_ARG, "%s: bad arguments", fn);
    if (n_rows == 0) return FQ_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == FQ_F32) launch_wht<float>(x, out, n_rows, D, st);
    else if (dtype == FQ_F16) launch_wht<__half>(x, out, n_rows, D, st);
    else if (dtype == FQ_BF16) launch_wht<__nv_bfloat16>(x, out, n_rows, D, st);
    else return fail(FQ_ERR_DTYPE, "%s: dtype code %d", fn, dtype);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" int fq_quantize_turbo(
    const void* head, int64_t hd_sb, int64_t hd_sh, int64_t hd_ss, int n_head,
    const void* nw, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    int dtype, int B, int H, int D, int n_quant,
    uint8_t* msb, int64_t ms_sb, int64_t ms_sh, int64_t ms_ss,
    uint8_t* lsb, int64_t ls_sb, int64_t ls_sh, int64_t ls_ss,
    void* scale, int64_t sc_sb, int64_t sc_sh, int64_t sc_ss, void* stream) {
    using namespace fq;
    const char* fn = "fq_quantize_turbo";
    FQ_CHECK_ARG(B > 0 && H > 0 && n_head >= 0 && n_new >= 0 && n_quant >= 0 && n_quant <= n_head + n_new, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(D % 8 == 0, FQ_ERR_ARG, "%s: requires head_dim multiple of 8; got %d", fn, D);
    FQ_CHECK_ARG(D > 0 && (D & (D - 1)) == 0, FQ_ERR_ARG, "%s: head_dim must be a positive power of 2, got %d", fn, D);
    FQ_CHECK_ARG(D <= 1024, FQ_ERR_UNSUPPORTED, "%s: head_dim %d above 1024", fn, D);
    FQ_CHECK_ARG(dtype == FQ_F32 || dtype == FQ_F16 || dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: dtype code %d", fn, dtype);
    if (n_quant == 0) return FQ_OK;
    FQ_CHECK_ARG(msb && lsb && scale && (nw || n_new == 0) && (head || n_head == 0), FQ_ERR_ARG, "%s: null pointer", fn);
    FQ_CHECK_ARG(B <= 65535 && H <= 65535, FQ_ERR_ARG, "%s: B and H must be <= 65535", fn);
    TurboParams p;
    p.head = head; p.nw = nw; p.hd_sb = hd_sb; p.hd_sh = hd_sh; p.hd_ss = hd_ss;
    p.nw_sb = nw_sb; p.nw_sh = nw_sh; p.nw_ss = nw_ss; p.n_head = n_head; p.n_quant = n_quant; p.D = D;
    p.msb = msb; p.lsb = lsb; p.ms_sb = ms_sb; p.ms_sh = ms_sh; p.ms_ss = ms_ss; p.ls_sb = ls_sb; p.ls_sh = ls_sh; p.ls_ss = ls_ss;
    p.scale = static_cast<uint16_t*>(scale); p.sc_sb = sc_sb; p.sc_sh = sc_sh; p.sc_ss = sc_ss;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    {
        // head_dim 128, 16-bit values, every row 8-byte aligned: the short kernel (four tokens per warp)
        auto rows8 = [](const void* q, int64_t a, int64_t b2, int64_t c) { return q == nullptr || (aligned(q, 8) && a % 4 == 0 && b2 % 4 == 0 && c % 4 == 0); };
        if (D == 128 && dtype != FQ_F32 && rows8(head, hd_sb, hd_sh, hd_ss) && rows8(nw, nw_sb, nw_sh, nw_ss)) {
            dim3 grid16((unsigned)((n_quant + 15) / 16), (unsigned)H, (unsigned)B);
            if (dtype == FQ_F16) turbo_quant128_kernel<__half><<<grid16, 128, 0, st>>>(p);
            else turbo_quant128_kernel<__nv_bfloat16><<<grid16, 128, 0, st>>>(p);
            FQ_CHECK_LAUNCH(fn);
            return FQ_OK;
        }
    }
    dim3 grid((unsigned)((n_quant + 3) / 4), (unsigned)H, (unsigned)B);
    if (dtype == FQ_F32) launch_turbo<float>(p, grid, st);
    else if (dtype == FQ_F16) launch_turbo<__half>(p, grid, st);
    else launch_turbo<__nv_bfloat16>(p, grid, st);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" int fq_dequantize_turbo(
    const uint8_t* msb, int64_t ms_sb, int64_t ms_sh, int64_t ms_ss,
    const uint8_t* lsb, int64_t ls_sb, int64_t ls_sh, int64_t ls_ss,
    const void* scale, int64_t sc_sb, int64_t sc_sh, int64_t sc_ss,
    int B, int H, int S, int D, void* out, int64_t o_sb, int64_t o_sh, int64_t o_ss, void* stream) {
    using namespace fq;
    const char* fn = "fq_dequantize_turbo";
    FQ_CHECK_ARG(B > 0 && H > 0 && S >= 0, FQ_ERR_ARG, "%s: bad sizes", fn);
    FQ_CHECK_ARG(D >= 8 && (D & (D - 1)) == 0 && D <= 1024, FQ_ERR_UNSUPPORTED, "%s: head_dim %d must be a power of 2 in [8, 1024]", fn, D);
    if (S == 0) return FQ_OK;
    FQ_CHECK_ARG(msb && lsb && scale && out, FQ_ERR_ARG, "%s: null pointer", fn);
    FQ_CHECK_ARG(B <= 65535 && H <= 65535, FQ_ERR_ARG, "%s: B and H must be <= 65535", fn);
    dim3 grid((unsigned)((S + 3) / 4), (unsigned)H, (unsigned)B);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int epl = D >= 32 ? D / 32 : 1;
#define FQ_D(E) turbo_dequant_kernel<E><<<grid, 128, 0, st>>>(msb, ms_sb, ms_sh, ms_ss, lsb, ls_sb, ls_sh, ls_ss, \
        static_cast<const uint16_t*>(scale), sc_sb, sc_sh, sc_ss, S, D, static_cast<uint16_t*>(out), o_sb, o_sh, o_ss)
    switch (epl) {
        case 1: FQ_D(1); break;
        case 2: FQ_D(2); break;
        case 4: FQ_D(4); break;
        case 8: FQ_D(8); break;
        case 16: FQ_D(16); break;
        default: FQ_D(32); break;
    }
#undef FQ_D
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}
