// AWQ W4A16 GEMV for decode shapes (M <= 8 rows of activations), several projections that
// share the same input fused into one launch (QKV, gate/up), optionally with the element-wise
// operator in front of the linear (residual add + RMSNorm, or SwiGLU) computed while the input
// is staged and the rotary embedding applied to the outputs before they are stored.
//
// Layout (AutoAWQ GEMM format, flashquest/quant/awq_layout.py:18-44): qweight (K, N/8) int32
// with eight 4-bit codes per int32 along N, scales (K/G, N) fp16, qzeros (K/G, N/8) int32;
// w[k,n] = (code[k,n] - zero[k/G,n]) * scale[k/G,n].  In the interleaved order nibble i of an
// int32 holds column 8c + {0,2,4,6,1,3,5,7}[i].
//
// HBM-bound on the weights (0.5 byte per weight, read once) and, at these sizes (5-26 MB per
// launch), on latency: what matters is bytes in flight early and a short chain after the last
// byte.  A CTA owns a tile of 32 int32 column packs (128 B of a weight row, 256 outputs) of ONE
// projection and a range of quantisation groups; it streams the tile one group (<= 128 rows,
// 16 KiB) at a time through a 3- or 6-stage shared-memory ring with cp.async, the first stages requested
// before the dependency wait (weights never change).  Inside a group the kernel accumulates
// sum_k x*code in fp32 and applies scale and zero once: y += scale * (sum x*code - zero * sum x).
//   One row (M == 1), CUDA cores: a thread owns one pack (8 outputs), the 8 warps are 8 interleaved
//   row phases; the nibble is masked in place and reinterpreted as an fp32 (sub)normal, x is
//   pre-scaled by 2^100 and duplicated so that fma.rn.f32x2 handles two nibbles per issue slot.
//   2..8 rows, tensor cores (mma.sync m16n8k16, fp16 codes are exact, fp32 accumulation): the cost no
//   longer grows with the number of rows, which on the CUDA cores it does (8 fma per int32 and row).
// Split-K: the CTAs that share a tile form one thread-block cluster (<= 8); every CTA sends each
// column of its partial tile into the shared memory of the CTA that finishes that column, which adds
// the partial sums in rank order after one cluster barrier — no global round trip, no atomics, a
// fixed summation order, and the epilogue (bias, rounding, rotary embedding) spread over the cluster.
#include "fq_common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace fq {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int GEMV_PACKS = 32;          // int32 column packs per CTA (256 outputs)
constexpr int GEMV_TILE = GEMV_PACKS * 8;
constexpr int GEMV_MAX_PROJ = 4;
constexpr int GEMV_ROWS = 128;          // rows per stage = largest group size
constexpr int GEMV_STAGE_WORDS = GEMV_ROWS * GEMV_PACKS;
constexpr int GEMV_MAX_STAGES = 6;       // ring depth: 3 (short K ranges) or 6 (long ones: more bytes in flight per CTA)
constexpr int GEMV_MAX_CLUSTER = 8;

struct GemvProj {
    const int32_t* qweight; const __half* scales; const int32_t* qzeros; const __half* bias; __half* y;
    int N;              // outputs of this projection
    int tile0;          // first tile of this projection in the grid
    int rope;           // rotary embedding on the outputs of this projection
};

struct GemvParams {
    const __half* x; int M, K, group, n_groups;
    GemvProj proj[GEMV_MAX_PROJ]; int n_proj; int tiles_total;
    int interleaved;
    int vec16;          // every weight row starts 16-byte aligned and N % 32 == 0: 16-byte copies
    int k_split, groups_per_split;
    // operator in front of the linear
    int pro_kind;       // FQ_GEMV_PLAIN | FQ_GEMV_ADD_RMSNORM | FQ_GEMV_SWIGLU
    const __half* pro_b; const __half* pro_weight; float eps; __half* pro_out;
    // rotary embedding
    const int* pos_dev; int pos; float theta; int head_dim;
};

__device__ __forceinline__ float pow2f_i(int n) { return __int_as_float((127 + n) << 23); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// fixed-order sum over the CTA: lanes by butterfly, warps in index order
__device__ __forceinline__ float gemv_block_sum(float v, float* s_red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) t += s_red[w];
    return t;
}

__device__ __forceinline__ void gemv_mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// column (inside its pack of 8) of nibble i
__device__ __forceinline__ int gemv_nibble_col(int i, int interleaved) { return interleaved ? ((i & 3) * 2 + (i >> 2)) : i; }

// Shared memory (dynamic), in this order:
//   s_w    [STAGES][ROWS][WSTRIDE] u32    weight ring; after the main loop: row-phase partial sums, then the CTA's tile
//   s_x    M == 1: [range] float2 (x, x) * 2^100;  M > 1: [8][range + 8] fp16 (rows past the batch are zero)
//   s_slot [cluster][M][columns this CTA finishes] f32  one copy per CTA of the cluster (8 rows: TILE / cluster columns
//                                           in every CTA; fewer rows: the whole tile, used in the first CTA)
//   s_xsum [groups_per_split][M] f32       sum of x per group and row
// M == 1 multiplies on the CUDA cores (one thread per pack, 8 row phases).  M > 1 (2, 4 or 8 rows, padded to 8)
// multiplies on the tensor cores with mma.sync m16n8k16: the 16 "rows" of an A fragment are the low and the
// high nibble of one byte position of 8 neighbouring packs (lane group g owns pack 8*blk + g), its 16 k are 16
// weight rows, B holds the 8 activation rows; a warp owns 8 packs and every second 16-row step of the group.
template <int M, int GEMV_STAGES>
__global__ void __launch_bounds__(GEMV_THREADS) awq_gemv_kernel(GemvParams p) {
    constexpr bool MMA = M > 1;
    constexpr int WSTRIDE = MMA ? GEMV_PACKS + 4 : GEMV_PACKS;     // +4 words: the fragment loads of 4 rows x 8 packs hit 32 banks
    constexpr int STAGE_WORDS = GEMV_ROWS * WSTRIDE;
    extern __shared__ __align__(16) unsigned char s_raw[];
    cg::cluster_group cluster = cg::this_cluster();
    const int range = p.groups_per_split * p.group;
    const int xstride = range + 8;                                 // fp16 row stride of s_xh (M > 1)
    uint32_t* s_w = reinterpret_cast<uint32_t*>(s_raw);
    unsigned char* x_base = s_raw + (size_t)GEMV_STAGES * STAGE_WORDS * 4;
    float2* s_xs = reinterpret_cast<float2*>(x_base);              // M == 1
    __half* s_xh = reinterpret_cast<__half*>(x_base);              // M > 1
    const size_t x_bytes = MMA ? (size_t)8 * xstride * 2 : (size_t)range * 8;
    float* s_slot = reinterpret_cast<float*>(x_base + x_bytes);
    float* s_xsum = s_slot + (size_t)(M == 8 ? 1 : p.k_split) * M * GEMV_TILE;
    __shared__ float s_red8[GEMV_WARPS];
    __shared__ float s_rstd[M];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = blockIdx.x, split = blockIdx.y;       // split == rank in the cluster
    int pi = 0;
#pragma unroll
    for (int i = 1; i < GEMV_MAX_PROJ; ++i)
        if (i < p.n_proj && tile >= p.proj[i].tile0) pi = i;
    const GemvProj pr = p.proj[pi];
    const int npk = pr.N / 8;
    const int pk0 = (tile - pr.tile0) * GEMV_PACKS;          // first pack of the tile inside the projection
    const int g_begin = split * p.groups_per_split;
    const int g_end = min(p.n_groups, g_begin + p.groups_per_split);
    const int n_chunks = max(g_end - g_begin, 0);
    const int G = p.group;
    const int k0 = g_begin * G, k_len = n_chunks * G;

    // weights of a chunk (they never change: safe to request before the previous kernel is done)
    auto issue_w = [&](int chunk) {
        const int g = g_begin + chunk, st = chunk % GEMV_STAGES;
        uint32_t* dst = s_w + st * STAGE_WORDS;
        const int32_t* src = pr.qweight + (int64_t)g * G * npk + pk0;
        if (p.vec16) {
            // 256 threads = 32 rows x 8 pieces of 16 bytes: a thread keeps its piece and walks down the rows
            const int r0 = tid >> 3, q = tid & 7;
            if (pk0 + q * 4 < npk) {
                uint32_t* d = dst + r0 * WSTRIDE + q * 4;
                const int32_t* sp = src + (int64_t)r0 * npk + q * 4;
                for (int r = r0; r < G; r += 32, d += 32 * WSTRIDE, sp += 32 * (int64_t)npk) cp_async16(d, sp);
            }
        } else {
            const int r0 = tid >> 5, q = tid & 31;
            if (pk0 + q < npk) {
                uint32_t* d = dst + r0 * WSTRIDE + q;
                const int32_t* sp = src + (int64_t)r0 * npk + q;
                for (int r = r0; r < G; r += 8, d += 8 * WSTRIDE, sp += 8 * (int64_t)npk) cp_async4(d, sp);
            }
        }
    };
    // staged input element kk (inside the CTA's K range) of row m
    auto put_x = [&](int kk, int m, __half h) {
        if constexpr (MMA) s_xh[m * xstride + kk] = h;
        else { const float vs = __half2float(h) * 1.2676506002282294e30f; s_xs[kk] = make_float2(vs, vs); }
    };

    cluster.barrier_arrive();          // matched by the wait in front of the first access to another CTA's shared memory
#pragma unroll
    for (int s = 0; s < GEMV_STAGES; ++s) {
        if (s < n_chunks) issue_w(s);
        cp_async_commit();             // group s = chunk s
    }
    pdl_wait();        // x comes from the previous kernel
    pdl_trigger();

    // ---- the CTA's K range of the input, through the operator in front of the linear ----
    // 8 values (16 bytes) per thread and pass
    if constexpr (MMA) {               // rows past the batch multiply as zeros
        for (int i = tid; i < (8 - p.M) * (k_len / 8); i += GEMV_THREADS) {
            const int m = p.M + i / (k_len / 8), kk = (i % (k_len / 8)) * 8;
            *reinterpret_cast<uint4*>(s_xh + m * xstride + kk) = make_uint4(0, 0, 0, 0);
        }
    }
    const int kv8 = p.K / 8;
    if (p.pro_kind == FQ_GEMV_ADD_RMSNORM) {
        // h = x (+ b) in fp16; rstd = rsqrt(mean(h^2) + eps) over the whole row, computed by every CTA
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float ss = 0.f;
            if (m < p.M) {
                const uint4* xa = reinterpret_cast<const uint4*>(p.x + (int64_t)m * p.K);
                const uint4* xb = p.pro_b ? reinterpret_cast<const uint4*>(p.pro_b + (int64_t)m * p.K) : nullptr;
                for (int i = tid; i < kv8; i += GEMV_THREADS) {
                    uint4 a = __ldcg(xa + i);
                    __half2* ah = reinterpret_cast<__half2*>(&a);
                    if (xb) {
                        const uint4 b = __ldcg(xb + i);
                        const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
                        for (int j = 0; j < 4; ++j) ah[j] = __hadd2(ah[j], bh[j]);
                    }
                    const int kk = i * 8 - k0;
                    const bool mine = kk >= 0 && kk < k_len;
                    if (mine && tile == 0 && p.pro_out) *reinterpret_cast<uint4*>(p.pro_out + (int64_t)m * p.K + i * 8) = a;
                    if constexpr (MMA) {
                        if (mine) *reinterpret_cast<uint4*>(s_xh + m * xstride + kk) = a;     // h for now, normalised below
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(ah[j]);
                        ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
                        if constexpr (!MMA) {
                            if (mine) { s_xs[kk + 2 * j] = make_float2(f.x, 0.f); s_xs[kk + 2 * j + 1] = make_float2(f.y, 0.f); }
                        }
                    }
                }
            }
            const float tot = gemv_block_sum(ss, s_red8);
            if (tid == 0) s_rstd[m] = rsqrtf(tot / (float)p.K + p.eps);
        }
        __syncthreads();
        for (int i = tid; i < p.M * k_len; i += GEMV_THREADS) {
            const int m = i / k_len, kk = i - m * k_len;
            float hv;
            if constexpr (MMA) hv = __half2float(s_xh[m * xstride + kk]); else hv = s_xs[kk].x;
            const __half xh = __float2half_rn(hv * s_rstd[m]);
            put_x(kk, m, __hmul(p.pro_weight[k0 + kk], xh));
        }
    } else {
        const int kl8 = k_len / 8;
        for (int i = tid; i < p.M * kl8; i += GEMV_THREADS) {
            const int m = i / kl8, kk = (i % kl8) * 8;
            const int64_t gi = (int64_t)m * p.K + k0 + kk;
            uint4 a = __ldcg(reinterpret_cast<const uint4*>(p.x + gi));
            __half2* ah = reinterpret_cast<__half2*>(&a);
            if (p.pro_kind == FQ_GEMV_SWIGLU) {
                const uint4 u = __ldcg(reinterpret_cast<const uint4*>(p.pro_b + gi));
                const __half2* uh = reinterpret_cast<const __half2*>(&u);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 g2 = __half22float2(ah[j]);
                    ah[j] = __hmul2(__floats2half2_rn(g2.x / (1.0f + expf(-g2.x)), g2.y / (1.0f + expf(-g2.y))), uh[j]);
                }
                if (tile == 0 && p.pro_out) *reinterpret_cast<uint4*>(p.pro_out + gi) = a;
            }
            if constexpr (MMA) {
                *reinterpret_cast<uint4*>(s_xh + m * xstride + kk) = a;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) { put_x(kk + 2 * j, m, __low2half(ah[j])); put_x(kk + 2 * j + 1, m, __high2half(ah[j])); }
            }
        }
    }
    __syncthreads();
    // sum of x per group and row (fixed order): a warp per (group, row), lanes stride the group
    for (int gm = warp; gm < n_chunks * M; gm += GEMV_WARPS) {
        const int ch = gm / M, m = gm % M;
        float s = 0.f;
        for (int r = lane; r < G; r += 32) {
            if constexpr (MMA) s += __half2float(s_xh[m * xstride + ch * G + r]);
            else s += s_xs[ch * G + r].x * 7.888609052210118e-31f;            // * 2^-100 (exact)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) s_xsum[gm] = s;
    }

    // this thread's pack: one per lane (M == 1), one per lane group of the warp's 8-pack block (M > 1)
    const int g8 = lane >> 2, t4 = lane & 3;
    const int blk = warp & 3, kh = warp >> 2;
    const int lpk = MMA ? blk * 8 + g8 : lane;               // pack inside the tile
    const int c = pk0 + lpk;
    const bool valid = c < npk;
    constexpr int NACC = MMA ? 16 : 8;                       // M == 1: [nibble]; M > 1: [nibble][row 2*t4 + {0, 1}]
    float yacc[NACC];
#pragma unroll
    for (int j = 0; j < NACC; ++j) yacc[j] = 0.f;

    for (int ch = 0; ch < n_chunks; ++ch) {
        const int g = g_begin + ch, st = ch % GEMV_STAGES;
        // scale and zero of this group: issued before the wait so that they are in flight with it
        uint32_t z = 0; uint4 sc8 = make_uint4(0, 0, 0, 0);
        if (valid) {
            z = (uint32_t)__ldg(pr.qzeros + (int64_t)g * npk + c);
            sc8 = __ldg(reinterpret_cast<const uint4*>(pr.scales + (int64_t)g * pr.N + c * 8));
        }
        // groups committed so far: chunks 0 .. max(STAGES - 1, ch + STAGES - 2); chunk ch must have landed
        if (ch == 0) cp_async_wait<GEMV_STAGES - 1>(); else cp_async_wait<GEMV_STAGES - 2>();
        __syncthreads();                 // chunk ch has landed for everybody; chunk ch-1 is consumed; s_xsum is written
        if (ch >= 1) {
            if (ch + GEMV_STAGES - 1 < n_chunks) issue_w(ch + GEMV_STAGES - 1);    // into the stage chunk ch-1 has left
            cp_async_commit();
        }
        if constexpr (!MMA) {
            if (!valid) continue;      // (the tensor-core path keeps every lane: a pack past the end multiplies by scale 0)
        }
        const uint32_t* sw = s_w + st * STAGE_WORDS;
        // (scale and zero are first touched after the multiply loop, so their load stays in flight behind it)
        auto scales_f32 = [&](float (&scol)[8]) {
            const __half2* sch = reinterpret_cast<const __half2*>(&sc8);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 t = __half22float2(sch[j]); scol[2 * j] = t.x; scol[2 * j + 1] = t.y; }
        };
        if constexpr (!MMA) {
            float2 acc[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = make_float2(0.f, 0.f);
            const uint32_t* wcol = sw + lane;
            const float2* xs = s_xs + (size_t)ch * G;
#pragma unroll 4
            for (int r = warp; r < G; r += GEMV_WARPS) {
                const uint32_t w = wcol[r * WSTRIDE];
                float2 f[4];
                f[0] = make_float2(__uint_as_float(w & 0x0000000fu), __uint_as_float(w & 0x000000f0u));
                f[1] = make_float2(__uint_as_float(w & 0x00000f00u), __uint_as_float(w & 0x0000f000u));
                f[2] = make_float2(__uint_as_float(w & 0x000f0000u), __uint_as_float(w & 0x00f00000u));
                f[3] = make_float2(__uint_as_float(w >> 24), __uint_as_float(w >> 28));
                const float2 xx = xs[r];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] = __ffma2_rn(f[j], xx, acc[j]);
            }
            // undo the nibble-position powers of two, then apply zero and scale of this group
            float scol[8];
            scales_f32(scol);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float scv = p.interleaved ? scol[(i & 3) * 2 + (i >> 2)] : scol[i];   // a select of two registers, not an indexed array
                // zero of nibble i, same in-place trick: (z & mask) as fp32 is zero * 2^(4i-149)
                const float zero = i < 6 ? __uint_as_float(z & (0xfu << (4 * i))) * pow2f_i(100 - 4 * i) * pow2f_i(49)
                                         : __uint_as_float(i == 6 ? ((z >> 24) & 15u) : (z >> 28)) * pow2f_i(100) * pow2f_i(49);
                const float ai = (i & 1) ? acc[i >> 1].y : acc[i >> 1].x;
                float a;
                if (i <= 5) a = ai * pow2f_i(49 - 4 * i);
                else if (i == 6) a = fmaf(-16.f, acc[3].y, ai) * pow2f_i(49);
                else a = ai * pow2f_i(49);
                // the zero term belongs to the group once, not once per row phase
                const float zterm = warp == 0 ? zero * s_xsum[ch] : 0.f;
                yacc[i] = fmaf(scv, a - zterm, yacc[i]);     // kept in nibble order until the columns are written
            }
        } else {
            float cf[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) cf[j][e] = 0.f;
            const uint32_t* wp = sw + lpk;
            const __half* xrow = s_xh + g8 * xstride + ch * G + 2 * t4;
            for (int ks = kh; ks < G / 16; ks += 2) {
                const int r = ks * 16 + 2 * t4;
                const uint32_t wa = wp[r * WSTRIDE], wb = wp[(r + 1) * WSTRIDE], wc = wp[(r + 8) * WSTRIDE], wd = wp[(r + 9) * WSTRIDE];
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xrow + ks * 16);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(xrow + ks * 16 + 8);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // byte j of the two rows side by side: halves (row r, row r+1); low nibble = nibble 2j, high = 2j+1
                    const uint32_t sel = (uint32_t)((4 + j) << 12 | (4 + j) << 8 | j << 4 | j);
                    const uint32_t v1 = __byte_perm(wa, wb, sel), v2 = __byte_perm(wc, wd, sel);
                    const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400));
                    uint32_t a0 = (v1 & 0x000f000fu) | 0x64006400u, a1 = ((v1 >> 4) & 0x000f000fu) | 0x64006400u;
                    uint32_t a2 = (v2 & 0x000f000fu) | 0x64006400u, a3 = ((v2 >> 4) & 0x000f000fu) | 0x64006400u;
                    __half2 h0 = __hsub2(*reinterpret_cast<__half2*>(&a0), k1024), h1 = __hsub2(*reinterpret_cast<__half2*>(&a1), k1024);
                    __half2 h2 = __hsub2(*reinterpret_cast<__half2*>(&a2), k1024), h3 = __hsub2(*reinterpret_cast<__half2*>(&a3), k1024);
                    gemv_mma_16816(cf[j], *reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1),
                                   *reinterpret_cast<uint32_t*>(&h2), *reinterpret_cast<uint32_t*>(&h3), b0, b1);
                }
            }
            // cf[j] = {nibble 2j x rows (2t, 2t+1), nibble 2j+1 x rows (2t, 2t+1)}: sum over this warp's rows of x * code
            const float xs0 = kh == 0 ? s_xsum[ch * M + min(2 * t4, M - 1)] : 0.f;
            const float xs1 = kh == 0 ? s_xsum[ch * M + min(2 * t4 + 1, M - 1)] : 0.f;
            float scol[8];
            scales_f32(scol);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float scv = p.interleaved ? scol[(i & 3) * 2 + (i >> 2)] : scol[i];   // a select of two registers, not an indexed array
                const float zero = (float)((z >> (4 * i)) & 15u);
                yacc[2 * i] = fmaf(scv, cf[i >> 1][(i & 1) * 2] - zero * xs0, yacc[2 * i]);
                yacc[2 * i + 1] = fmaf(scv, cf[i >> 1][(i & 1) * 2 + 1] - zero * xs1, yacc[2 * i + 1]);
            }
        }
    }
    cp_async_wait<0>();
    // ---- the CTA's tile: add the row phases through shared memory, lay the columns out in order ----
    __syncthreads();
    float* s_red = reinterpret_cast<float*>(s_raw);                    // row-phase partial sums
    float* s_part = s_red + (GEMV_WARPS - 1) * 32 * NACC;              // [M][TILE] the CTA's partial tile
    constexpr int NRED = MMA ? 4 : GEMV_WARPS - 1;                     // warps that hand their sums over
    const int first_keep = MMA ? 4 : 1;                                // warps >= first_keep hand over (M > 1: the second k half)
    if (warp >= first_keep) {
#pragma unroll
        for (int j = 0; j < NACC; j += 4)
            *reinterpret_cast<float4*>(s_red + ((warp - first_keep) * 32 + lane) * NACC + j) = make_float4(yacc[j], yacc[j + 1], yacc[j + 2], yacc[j + 3]);
    }
    __syncthreads();
    cluster.barrier_wait();            // every CTA of the cluster runs: its shared memory may be addressed
    if (warp < first_keep) {
        if constexpr (!MMA) {
#pragma unroll
            for (int k = 0; k < NRED; ++k)
#pragma unroll
                for (int j = 0; j < NACC; ++j) yacc[j] += s_red[(k * 32 + lane) * NACC + j];
            // one row: the lane's 8 columns go straight from registers into slot [split] of the first CTA
            float cv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) cv[j] = p.interleaved ? yacc[(j >> 1) + (j & 1) * 4] : yacc[j];
            float4* d = reinterpret_cast<float4*>(cluster.map_shared_rank(s_slot, 0) + (size_t)split * GEMV_TILE + lane * 8);
            d[0] = make_float4(cv[0], cv[1], cv[2], cv[3]);
            d[1] = make_float4(cv[4], cv[5], cv[6], cv[7]);
        } else {
#pragma unroll
            for (int j = 0; j < NACC; ++j) yacc[j] += s_red[(warp * 32 + lane) * NACC + j];    // warp + 4 holds the other k half of this block
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int col = lpk * 8 + gemv_nibble_col(i, p.interleaved);
                if (2 * t4 < M) s_part[(2 * t4) * GEMV_TILE + col] = yacc[2 * i];
                if (2 * t4 + 1 < M) s_part[(2 * t4 + 1) * GEMV_TILE + col] = yacc[2 * i + 1];
            }
        }
    }
    // ---- merge over the cluster ----
    // 8 rows: rank r finishes the columns whose position inside half a head falls into its piece (the two partners
    // of a rotary pair meet in the same CTA), so a CTA holds 1/cluster of every partial tile.  Fewer rows: the partial
    // tiles are small and all go to the first CTA, which measured faster than the all-to-all exchange.
    constexpr bool SCATTER = M == 8;
    const int ks_n = p.k_split;
    const int period = (p.head_dim > 0 ? p.head_dim : 128) / 2;        // 64 unless the rotary embedding asks otherwise
    const int pw = SCATTER ? period / ks_n : period;                   // piece width (a multiple of 4, host-checked)
    const int own_n = SCATTER ? GEMV_TILE / ks_n : GEMV_TILE;          // columns finished per owner
    // local index of column col at its owner: (col / period) * pw + col % pw; four columns (16 bytes) per store
    if constexpr (MMA) __syncthreads();                                // s_part is complete
    for (int i = tid; MMA && i < M * (GEMV_TILE / 4); i += GEMV_THREADS) {
        const int m = i / (GEMV_TILE / 4), col = (i - m * (GEMV_TILE / 4)) * 4;
        const int within = col % period, owner = within / pw;
        const int loc = (col / period) * pw + within % pw;
        float* dst = cluster.map_shared_rank(s_slot, owner);
        *reinterpret_cast<float4*>(dst + ((size_t)split * M + m) * own_n + loc) = *reinterpret_cast<const float4*>(s_part + m * GEMV_TILE + col);
    }
    cluster.sync();                    // every partial sum has arrived at its owner
    if (!SCATTER && split != 0) return;
    // ---- owner: add the splits in rank order, bias, rounding, rotary embedding, store ----
    __half* s_y = reinterpret_cast<__half*>(s_raw);                    // [M][own_n] fp16 (the ring is free)
    for (int i = tid; i < M * own_n; i += GEMV_THREADS) {
        const int m = i / own_n, loc = i - m * own_n;
        const int col = (loc / pw) * period + split * pw + loc % pw;
        float v = 0.f;
        for (int s = 0; s < ks_n; ++s) v += s_slot[((size_t)s * M + m) * own_n + loc];
        const int n = pk0 * 8 + col;
        if (pr.bias && n < pr.N) v += __half2float(pr.bias[n]);
        const __half hv = __float2half_rn(v);
        if (pr.rope) s_y[i] = hv;
        else if (m < p.M && n < pr.N) pr.y[(int64_t)m * pr.N + n] = hv;
    }
    if (!pr.rope) return;
    __syncthreads();
    // Hugging Face "rotate_half" convention, cos/sin in fp32 from pos * theta^(-2i/D) rounded to fp16,
    // products and sum in fp16: the arithmetic of rope_kernel.  Local pieces alternate first half / second half of a head.
    const int D = p.head_dim;
    const int pos = p.pos_dev ? *p.pos_dev : p.pos;
    for (int i = tid; i < p.M * (own_n / 2); i += GEMV_THREADS) {
        const int m = i / (own_n / 2), j = i - m * (own_n / 2);
        const int hd = j / pw, e = j - hd * pw;                        // head inside the tile, element inside the piece
        const int idx = split * pw + e;                                // position inside the first half of the head
        const int n = pk0 * 8 + hd * D + idx;
        if (n >= pr.N) continue;
        const float inv_freq = 1.0f / powf(p.theta, (float)(2 * idx) / (float)D);
        const float ang = (float)pos * inv_freq;
        const __half cs = __float2half_rn(cosf(ang)), sn = __float2half_rn(sinf(ang));
        const __half x1 = s_y[m * own_n + (2 * hd) * pw + e], x2 = s_y[m * own_n + (2 * hd + 1) * pw + e];
        __half* yo = pr.y + (int64_t)m * pr.N + n;
        yo[0] = __hadd(__hmul(x1, cs), __hmul(__hneg(x2), sn));
        yo[period] = __hadd(__hmul(x2, cs), __hmul(x1, sn));
    }
}

}  // namespace fq

static inline int gemv_mp(int M) { return M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8)); }

extern "C" int fq_awq_gemv_default_splits(int K, int N_total, int group) {
    if (K <= 0 || N_total <= 0 || group <= 0) return 1;
    const int n_groups = K / group;
    const int tiles = (N_total / 8 + fq::GEMV_PACKS - 1) / fq::GEMV_PACKS;
    int want = (3 * 148 + tiles - 1) / tiles;       // about three CTAs per SM
    if (want > fq::GEMV_MAX_CLUSTER) want = fq::GEMV_MAX_CLUSTER;
    if (want > n_groups) want = n_groups;
    if (want < 1) want = 1;
    // cluster sizes are powers of two; every rank must own at least one group
    int ks = 1;
    while (ks * 2 <= want) ks *= 2;
    const int gps = (n_groups + ks - 1) / ks;
    while (ks > 1 && (ks - 1) * gps >= n_groups) ks /= 2;
    return ks;
}

extern "C" int fq_awq_gemv_fused(
    const void* x, int M, int K, int group, int n_proj,
    const int32_t* const* qweight, const void* const* scales, const int32_t* const* qzeros, const void* const* bias,
    const int* N, void* const* y, int interleaved, const fq_gemv_prologue* pro, const fq_gemv_rope* rope, int k_split, void* stream) {
    using namespace fq;
    const char* fn = "fq_awq_gemv";
    FQ_CHECK_ARG(M >= 1 && M <= 8, FQ_ERR_UNSUPPORTED, "%s: M=%d rows; the GEMV path takes 1..8 (larger M belongs to the GEMM path)", fn, M);
    FQ_CHECK_ARG(group == 32 || group == 64 || group == 128, FQ_ERR_UNSUPPORTED, "%s: group size %d; 32, 64 and 128 are built", fn, group);
    FQ_CHECK_ARG(K > 0 && K % group == 0, FQ_ERR_ARG, "%s: K=%d must be a multiple of the group size %d", fn, K, group);
    FQ_CHECK_ARG(n_proj >= 1 && n_proj <= GEMV_MAX_PROJ, FQ_ERR_ARG, "%s: 1..%d projections per call, got %d", fn, GEMV_MAX_PROJ, n_proj);
    FQ_CHECK_ARG(x && qweight && scales && qzeros && N && y, FQ_ERR_ARG, "%s: null pointer", fn);
    FQ_CHECK_ARG(aligned(x, 16), FQ_ERR_ALIGN, "%s: x must be 16-byte aligned", fn);
    FQ_CHECK_ARG(k_split >= 1 && k_split <= GEMV_MAX_CLUSTER && (k_split & (k_split - 1)) == 0, FQ_ERR_ARG,
                 "%s: k_split=%d must be 1, 2, 4 or 8 (the CTAs of one thread-block cluster)", fn, k_split);
    GemvParams p;
    p.x = static_cast<const __half*>(x); p.M = M; p.K = K; p.group = group; p.n_groups = K / group;
    p.n_proj = n_proj; p.interleaved = interleaved ? 1 : 0;
    p.pro_kind = FQ_GEMV_PLAIN; p.pro_b = nullptr; p.pro_weight = nullptr; p.eps = 0.f; p.pro_out = nullptr;
    if (pro && pro->kind != FQ_GEMV_PLAIN) {
        FQ_CHECK_ARG(pro->kind == FQ_GEMV_ADD_RMSNORM || pro->kind == FQ_GEMV_SWIGLU, FQ_ERR_ARG, "%s: prologue kind %d", fn, pro->kind);
        FQ_CHECK_ARG(K % 8 == 0, FQ_ERR_ARG, "%s: a fused prologue needs K %% 8 == 0", fn);
        if (pro->kind == FQ_GEMV_ADD_RMSNORM) FQ_CHECK_ARG(pro->weight, FQ_ERR_ARG, "%s: RMSNorm prologue without weight", fn);
        else FQ_CHECK_ARG(pro->b, FQ_ERR_ARG, "%s: SwiGLU prologue without the up projection", fn);
        FQ_CHECK_ARG(!pro->b || aligned(pro->b, 16), FQ_ERR_ALIGN, "%s: prologue operand must be 16-byte aligned", fn);
        FQ_CHECK_ARG(pro->out != x && (!pro->out || pro->out != pro->b), FQ_ERR_ARG, "%s: the prologue's output must not alias its inputs", fn);
        p.pro_kind = pro->kind; p.pro_b = static_cast<const __half*>(pro->b); p.pro_weight = static_cast<const __half*>(pro->weight);
        p.eps = pro->eps; p.pro_out = static_cast<__half*>(pro->out);
    }
    p.pos_dev = nullptr; p.pos = 0; p.theta = 0.f; p.head_dim = 0;
    if (rope) {
        FQ_CHECK_ARG(rope->head_dim > 0 && GEMV_TILE % rope->head_dim == 0 && rope->head_dim % 2 == 0, FQ_ERR_UNSUPPORTED,
                     "%s: rotary embedding needs a head_dim that divides %d (got %d)", fn, GEMV_TILE, rope->head_dim);
        FQ_CHECK_ARG(rope->theta > 0.f, FQ_ERR_ARG, "%s: rope theta", fn);
        p.pos_dev = rope->pos_dev; p.pos = rope->pos; p.theta = rope->theta; p.head_dim = rope->head_dim;
    }
    int tile0 = 0, vec16 = 1;
    for (int i = 0; i < n_proj; ++i) {
        FQ_CHECK_ARG(N[i] > 0 && N[i] % 8 == 0, FQ_ERR_ARG, "%s: N[%d]=%d must be a positive multiple of 8", fn, i, N[i]);
        FQ_CHECK_ARG(qweight[i] && scales[i] && qzeros[i] && y[i], FQ_ERR_ARG, "%s: null tensor in projection %d", fn, i);
        FQ_CHECK_ARG(aligned(y[i], 16) && aligned(scales[i], 16) && aligned(qweight[i], 4) && aligned(qzeros[i], 4), FQ_ERR_ALIGN,
                     "%s: y[%d] and scales[%d] must be 16-byte aligned", fn, i, i);
        if (N[i] % 32 != 0 || !aligned(qweight[i], 16)) vec16 = 0;
        GemvProj& q = p.proj[i];
        q.qweight = qweight[i]; q.scales = static_cast<const __half*>(scales[i]); q.qzeros = qzeros[i];
        q.bias = bias ? static_cast<const __half*>(bias[i]) : nullptr; q.y = static_cast<__half*>(y[i]);
        q.N = N[i]; q.tile0 = tile0;
        q.rope = rope && ((rope->proj_mask >> i) & 1) ? 1 : 0;
        if (q.rope) FQ_CHECK_ARG(N[i] % rope->head_dim == 0, FQ_ERR_ARG, "%s: N[%d]=%d is not a multiple of head_dim %d", fn, i, N[i], rope->head_dim);
        tile0 += (N[i] / 8 + GEMV_PACKS - 1) / GEMV_PACKS;
    }
    for (int i = n_proj; i < GEMV_MAX_PROJ; ++i) p.proj[i] = GemvProj{nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0};
    p.tiles_total = tile0; p.vec16 = vec16;
    const int tiles = tile0;
    if (k_split > p.n_groups) {
        k_split = 1;
        while (k_split * 2 <= p.n_groups) k_split *= 2;
    }
    // ranks past the last group get no chunks and send zeros
    const int Mp = gemv_mp(M);
    // the CTA keeps its whole K range of the input in shared memory: a range too long for it is split further
    size_t smem = 0;
    int stages = 3;
    const size_t stage_bytes = (size_t)GEMV_ROWS * (Mp > 1 ? GEMV_PACKS + 4 : GEMV_PACKS) * 4;
    for (;;) {
        p.groups_per_split = (p.n_groups + k_split - 1) / k_split;
        stages = p.groups_per_split > 3 ? GEMV_MAX_STAGES : 3;
        const size_t range = (size_t)p.groups_per_split * group;
        const size_t fixed = (Mp > 1 ? 8 * (range + 8) * 2 : range * 8) + (size_t)(Mp == 8 ? 1 : k_split) * Mp * GEMV_TILE * 4 +
                             (size_t)p.groups_per_split * Mp * 4;
        smem = stages * stage_bytes + fixed;
        // the deep ring only while two CTAs still fit on an SM
        if (smem > 113 * 1024 && stages > 3) { stages = 3; smem = stages * stage_bytes + fixed; }
        if (smem <= 226 * 1024 || k_split >= GEMV_MAX_CLUSTER || k_split * 2 > p.n_groups) break;
        k_split *= 2;
    }
    p.k_split = k_split;
    FQ_CHECK_ARG(((p.head_dim > 0 ? p.head_dim : 128) / 2) % (4 * (Mp == 8 ? k_split : 1)) == 0, FQ_ERR_UNSUPPORTED,
                 "%s: head_dim %d with %d-way split-K", fn, p.head_dim, k_split);
    FQ_CHECK_ARG(smem <= 226 * 1024, FQ_ERR_UNSUPPORTED, "%s: K=%d with %d rows needs %zu B of shared memory per CTA", fn, K, M, smem);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)tiles, (unsigned)k_split); cfg.blockDim = dim3(GEMV_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[2]{};
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = (unsigned)k_split; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl_enabled(PDL_GEMV) ? 2 : 1;
#define FQ_GEMV(MV, SV)                                                                                      \
    do {                                                                                                     \
        static std::atomic<size_t> attr_smem[64];                                                            \
        int dev = 0; cudaGetDevice(&dev);                                                                    \
        if (dev < 0 || dev >= 64 || attr_smem[dev].load(std::memory_order_acquire) < smem) {                 \
            cudaError_t e = cudaFuncSetAttribute(awq_gemv_kernel<MV, SV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: cannot reserve %zu B of shared memory: %s", fn, smem, cudaGetErrorString(e)); \
            if (dev >= 0 && dev < 64) attr_smem[dev].store(smem, std::memory_order_release);                 \
        }                                                                                                    \
        cudaLaunchKernelEx(&cfg, awq_gemv_kernel<MV, SV>, p);                                                \
    } while (0)
#define FQ_GEMV_M(MV) do { if (stages == 3) FQ_GEMV(MV, 3); else FQ_GEMV(MV, GEMV_MAX_STAGES); } while (0)
    if (Mp == 1) FQ_GEMV_M(1);
    else if (Mp == 2) FQ_GEMV_M(2);
    else if (Mp == 4) FQ_GEMV_M(4);
    else FQ_GEMV_M(8);
#undef FQ_GEMV_M
#undef FQ_GEMV
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" int fq_awq_gemv(
    const void* x, int M, int K, int group, int n_proj,
    const int32_t* const* qweight, const void* const* scales, const int32_t* const* qzeros, const void* const* bias,
    const int* N, void* const* y, int interleaved, int k_split, void* stream) {
    return fq_awq_gemv_fused(x, M, K, group, n_proj, qweight, scales, qzeros, bias, N, y, interleaved, nullptr, nullptr, k_split, stream);
}
