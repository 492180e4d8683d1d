// AWQ W4A16 GEMV for decode shapes (M <= 8 rows of activations), several projections that
// share the same input fused into one launch (QKV, gate/up).
//
// Layout (AutoAWQ GEMM format, flashquest/quant/awq_layout.py:18-44): qweight (K, N/8) int32
// with eight 4-bit codes per int32 along N, scales (K/G, N) fp16, qzeros (K/G, N/8) int32;
// w[k,n] = (code[k,n] - zero[k/G,n]) * scale[k/G,n].  In the interleaved order nibble i of an
// int32 holds column 8c + {0,2,4,6,1,3,5,7}[i].
//
// HBM-bound on the weights (0.5 byte per weight, read once), so what matters is bytes in
// flight: a CTA owns a tile of 64 int32 column packs (256 B of a weight row, 512 outputs) of ONE
// projection and a range of quantisation groups; it streams the tile one group (<= 128 rows,
// 32 KiB) at a time into a 3-stage shared-memory ring with cp.async, so up to 96 KiB per CTA are
// outstanding however many registers the arithmetic needs.  A thread owns one pack
// (8 outputs); the 8 warps are 2 column halves x 4 interleaved row phases.
// Inside a group the kernel accumulates sum_k x*code in fp32: the nibble is masked in place and
// reinterpreted as an fp32 (sub)normal, x is pre-scaled by 2^100 and duplicated so that
// fma.rn.f32x2 handles two nibbles per issue slot; the powers of two are undone once per group,
// where scale and zero are applied: y += scale * (sum x*code - zero * sum x).
// Split-K over ranges of groups: partial sums go to a workspace, the CTA that draws the last
// ticket of its tile adds them in split order and writes fp16.
#include "fq_common.cuh"

namespace fq {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_PACKS = 64;          // int32 column packs per CTA (512 outputs)
constexpr int GEMV_MAX_PROJ = 4;
constexpr int GEMV_STAGES = 3;
constexpr int GEMV_ROWS = 128;          // rows per stage = largest group size
constexpr int GEMV_STAGE_WORDS = GEMV_ROWS * GEMV_PACKS;

struct GemvProj {
    const int32_t* qweight; const __half* scales; const int32_t* qzeros; const __half* bias; __half* y;
    int N;              // outputs of this projection
    int tile0;          // first tile of this projection in the grid
};

struct GemvParams {
    const __half* x; int M, K, group, n_groups;
    GemvProj proj[GEMV_MAX_PROJ]; int n_proj; int tiles_total;
    int interleaved;
    int vec16;          // every weight row starts 16-byte aligned and N % 32 == 0: 16-byte copies
    int k_split, groups_per_split;
    float* partials;    // [k_split][M][tiles_total*512]
    int* tickets;       // per tile
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

// values held in nibble order -> 8 consecutive output columns as fp16.  In the interleaved
// order column j comes from nibble {0,4,1,5,2,6,3,7}[j].
__device__ __forceinline__ uint4 pack_columns(const float (&v)[8], int interleaved, const __half* bias) {
    float c[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) c[j] = interleaved ? v[(j >> 1) + (j & 1) * 4] : v[j];
    if (bias) {
#pragma unroll
        for (int j = 0; j < 8; ++j) c[j] += __half2float(bias[j]);
    }
    __half2 h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(c[2 * j], c[2 * j + 1]);
    return *reinterpret_cast<uint4*>(h);
}

template <int M>
__global__ void __launch_bounds__(GEMV_THREADS) awq_gemv_kernel(GemvParams p) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    uint32_t* s_w = reinterpret_cast<uint32_t*>(s_raw);                                   // [STAGES][ROWS][PACKS]
    __half* s_xh = reinterpret_cast<__half*>(s_raw + GEMV_STAGES * GEMV_STAGE_WORDS * 4);   // [STAGES][M][ROWS]
    float2* s_xs = reinterpret_cast<float2*>(s_xh + GEMV_STAGES * M * GEMV_ROWS);          // [ROWS][M] (x,x) * 2^100
    __shared__ float s_xsum[M];
    __shared__ int s_ticket;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wn = warp & 1, wk = warp >> 1;       // column half, row phase
    const int tile = blockIdx.x, split = blockIdx.y;
    int pi = 0;
#pragma unroll
    for (int i = 1; i < GEMV_MAX_PROJ; ++i)
        if (i < p.n_proj && tile >= p.proj[i].tile0) pi = i;
    const GemvProj pr = p.proj[pi];
    const int npk = pr.N / 8;
    const int pk0 = (tile - pr.tile0) * GEMV_PACKS;          // first pack of the tile inside the projection
    const int c = pk0 + wn * 32 + lane;                      // this thread's pack
    const bool valid = c < npk;
    const int g_begin = split * p.groups_per_split;
    const int g_end = min(p.n_groups, g_begin + p.groups_per_split);
    const int n_chunks = g_end - g_begin;
    const int G = p.group;

    // weights of a chunk (they never change: safe to request before the previous kernel is done)
    auto issue_w = [&](int chunk) {
        const int g = g_begin + chunk, st = chunk % GEMV_STAGES;
        uint32_t* dst = s_w + st * GEMV_STAGE_WORDS;
        const int32_t* src = pr.qweight + (int64_t)g * G * npk + pk0;
        if (p.vec16) {
            // 256 threads = 16 rows x 16 pieces of 16 bytes: a thread keeps its piece and walks down the rows
            const int r0 = tid >> 4, q = tid & 15;
            if (pk0 + q * 4 < npk) {
                uint32_t* d = dst + r0 * GEMV_PACKS + q * 4;
                const int32_t* sp = src + (int64_t)r0 * npk + q * 4;
                for (int r = r0; r < G; r += 16, d += 16 * GEMV_PACKS, sp += 16 * (int64_t)npk) cp_async16(d, sp);
            }
        } else {
            const int r0 = tid >> 6, q = tid & 63;
            if (pk0 + q < npk) {
                uint32_t* d = dst + r0 * GEMV_PACKS + q;
                const int32_t* sp = src + (int64_t)r0 * npk + q;
                for (int r = r0; r < G; r += 4, d += 4 * GEMV_PACKS, sp += 4 * (int64_t)npk) cp_async4(d, sp);
            }
        }
    };
    // activations of the group, fp16 as they are: M rows of G halves (16-byte pieces)
    auto issue_x = [&](int chunk) {
        const int g = g_begin + chunk, st = chunk % GEMV_STAGES;
        for (int i = tid; i < M * (G / 8); i += GEMV_THREADS) {
            const int m = i / (G / 8), q = i % (G / 8);
            if (m < p.M) cp_async16(s_xh + (st * M + m) * GEMV_ROWS + q * 8, p.x + (int64_t)m * p.K + (int64_t)g * G + q * 8);
        }
    };

#pragma unroll
    for (int s = 0; s < GEMV_STAGES - 1; ++s)
        if (s < n_chunks) issue_w(s);
    pdl_wait();        // x comes from the previous kernel
    pdl_trigger();
#pragma unroll
    for (int s = 0; s < GEMV_STAGES - 1; ++s) {
        if (s < n_chunks) issue_x(s);
        cp_async_commit();      // the first group also holds the weights of the later prologue stages: waits are only stricter
    }

    float yacc[M][8];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int j = 0; j < 8; ++j) yacc[m][j] = 0.f;

    for (int ch = 0; ch < n_chunks; ++ch) {
        const int g = g_begin + ch, st = ch % GEMV_STAGES;
        // scale and zero of this group: issued before the wait so that they are in flight with it
        uint32_t z = 0; uint4 sc8 = make_uint4(0, 0, 0, 0);
        if (valid) {
            z = (uint32_t)__ldg(pr.qzeros + (int64_t)g * npk + c);
            sc8 = __ldg(reinterpret_cast<const uint4*>(pr.scales + (int64_t)g * pr.N + c * 8));
        }
        cp_async_wait<GEMV_STAGES - 2>();
        __syncthreads();                 // chunk ch has landed for everybody; chunk ch-1 is consumed
        if (ch + GEMV_STAGES - 1 < n_chunks) { issue_w(ch + GEMV_STAGES - 1); issue_x(ch + GEMV_STAGES - 1); }
        cp_async_commit();
        // x of the group: fp16 -> fp32 * 2^100, duplicated; sum per row of x (fixed order)
        if (warp < M) {
            float s = 0.f;
            for (int r = lane; r < G; r += 32) {
                const float v = warp < p.M ? __half2float(s_xh[(st * M + warp) * GEMV_ROWS + r]) : 0.f;
                s += v;
                const float vs = v * 1.2676506002282294e30f;
                s_xs[r * M + warp] = make_float2(vs, vs);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) s_xsum[warp] = s;
        }
        __syncthreads();
        if (!valid) continue;
        float2 acc[M][4];
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[m][j] = make_float2(0.f, 0.f);
        const uint32_t* wcol = s_w + st * GEMV_STAGE_WORDS + wn * 32 + lane;
#pragma unroll 8
        for (int r = wk; r < G; r += 4) {
            const uint32_t w = wcol[r * GEMV_PACKS];
            float2 f[4];
            f[0] = make_float2(__uint_as_float(w & 0x0000000fu), __uint_as_float(w & 0x000000f0u));
            f[1] = make_float2(__uint_as_float(w & 0x00000f00u), __uint_as_float(w & 0x0000f000u));
            f[2] = make_float2(__uint_as_float(w & 0x000f0000u), __uint_as_float(w & 0x00f00000u));
            f[3] = make_float2(__uint_as_float(w >> 24), __uint_as_float(w >> 28));
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float2 xx = s_xs[r * M + m];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[m][j] = __ffma2_rn(f[j], xx, acc[m][j]);
            }
        }
        // undo the nibble-position powers of two, then apply zero and scale of this group
        const __half2* sch = reinterpret_cast<const __half2*>(&sc8);
        float scol[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 t = __half22float2(sch[j]); scol[2 * j] = t.x; scol[2 * j + 1] = t.y; }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float scv = p.interleaved ? scol[(i & 3) * 2 + (i >> 2)] : scol[i];   // column {0,2,4,6,1,3,5,7}[i]
            // zero of nibble i, same in-place trick: (z & mask) as fp32 is zero * 2^(4i-149)
            const float zero = i < 6 ? __uint_as_float(z & (0xfu << (4 * i))) * pow2f_i(100 - 4 * i) * pow2f_i(49)
                                     : __uint_as_float(i == 6 ? ((z >> 24) & 15u) : (z >> 28)) * pow2f_i(100) * pow2f_i(49);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float ai = (i & 1) ? acc[m][i >> 1].y : acc[m][i >> 1].x;
                float a;
                if (i <= 5) a = ai * pow2f_i(49 - 4 * i);
                else if (i == 6) a = fmaf(-16.f, acc[m][3].y, ai) * pow2f_i(49);
                else a = ai * pow2f_i(49);
                // the zero term belongs to the group once, not once per row phase
                const float zterm = wk == 0 ? zero * s_xsum[m] : 0.f;
                yacc[m][i] = fmaf(scv, a - zterm, yacc[m][i]);     // kept in nibble order until the store
            }
        }
    }
    cp_async_wait<0>();
    // reduce the 4 row phases through shared memory: s_red[wk-1][wn][lane][m][8]
    __syncthreads();
    float* s_red = reinterpret_cast<float*>(s_raw);
    if (wk > 0) {
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
            for (int j = 0; j < 8; ++j) s_red[((((wk - 1) * 2 + wn) * 32 + lane) * M + m) * 8 + j] = yacc[m][j];
    }
    __syncthreads();
    if (wk == 0) {
#pragma unroll
        for (int k = 0; k < 3; ++k)
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
                for (int j = 0; j < 8; ++j) yacc[m][j] += s_red[(((k * 2 + wn) * 32 + lane) * M + m) * 8 + j];
    }
    const __half* bias = pr.bias ? pr.bias + c * 8 : nullptr;
    if (p.k_split == 1) {
        if (wk == 0 && valid) {
#pragma unroll
            for (int m = 0; m < M; ++m)
                if (m < p.M) *reinterpret_cast<uint4*>(pr.y + (int64_t)m * pr.N + c * 8) = pack_columns(yacc[m], p.interleaved, bias);
        }
        return;
    }
    // split-K: publish, the CTA that draws the last ticket of the tile adds the splits in order
    constexpr int TILE_F = GEMV_PACKS * 8;                     // floats per tile row
    const int64_t n_pad = (int64_t)p.tiles_total * TILE_F;
    const int64_t tpos = (int64_t)tile * TILE_F;
    if (wk == 0 && valid) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float* dst = p.partials + ((int64_t)split * M + m) * n_pad + tpos + (wn * 32 + lane) * 8;
            __stcg(reinterpret_cast<float4*>(dst), make_float4(yacc[m][0], yacc[m][1], yacc[m][2], yacc[m][3]));
            __stcg(reinterpret_cast<float4*>(dst + 4), make_float4(yacc[m][4], yacc[m][5], yacc[m][6], yacc[m][7]));
        }
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        s_ticket = atomicAdd(&p.tickets[tile], 1);
        __threadfence();
    }
    __syncthreads();
    if (s_ticket != p.k_split - 1) return;
    // all 256 threads: a thread sums one float4 column piece of one row over the splits, eight
    // independent loads at a time; packs past the end of the projection hold garbage nobody reads
    float* s_out = reinterpret_cast<float*>(s_raw) + 3 * 2 * 32 * M * 8;      // [M][TILE_F], behind s_red
    {
        const int piece = tid & 127, mh = tid >> 7;
        for (int m = mh; m < p.M; m += 2) {
            const float* src = p.partials + (int64_t)m * n_pad + tpos + piece * 4;
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sp0 = 0; sp0 < p.k_split; sp0 += 8) {
                float4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    v[u] = sp0 + u < p.k_split ? __ldcg(reinterpret_cast<const float4*>(src + (int64_t)(sp0 + u) * M * n_pad))
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 8; ++u) { sum.x += v[u].x; sum.y += v[u].y; sum.z += v[u].z; sum.w += v[u].w; }
            }
            *reinterpret_cast<float4*>(s_out + m * TILE_F + piece * 4) = sum;
        }
    }
    __syncthreads();
    if (wk == 0 && valid) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (m >= p.M) break;
            float sv[8];
            const float4 a = *reinterpret_cast<const float4*>(s_out + m * TILE_F + (wn * 32 + lane) * 8);
            const float4 b2 = *reinterpret_cast<const float4*>(s_out + m * TILE_F + (wn * 32 + lane) * 8 + 4);
            sv[0] = a.x; sv[1] = a.y; sv[2] = a.z; sv[3] = a.w; sv[4] = b2.x; sv[5] = b2.y; sv[6] = b2.z; sv[7] = b2.w;
            *reinterpret_cast<uint4*>(pr.y + (int64_t)m * pr.N + c * 8) = pack_columns(sv, p.interleaved, bias);
        }
    }
    if (tid == 0) p.tickets[tile] = 0;
}

}  // namespace fq

static inline int gemv_mp(int M) { return M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8)); }
// upper bound of the tiles of a call whose projections sum to N_total outputs
static inline size_t gemv_tiles_bound(int N_total) { return (size_t)N_total / (fq::GEMV_PACKS * 8) + fq::GEMV_MAX_PROJ; }

extern "C" size_t fq_awq_gemv_workspace_bytes(int M, int N_total, int k_split) {
    if (M <= 0 || N_total <= 0 || k_split <= 1) return 0;
    const size_t tiles = gemv_tiles_bound(N_total);
    const size_t tickets = (tiles * 4 + 255) & ~(size_t)255;
    return tickets + (size_t)k_split * gemv_mp(M) * tiles * fq::GEMV_PACKS * 8 * 4;
}

extern "C" int fq_awq_gemv_default_splits(int K, int N_total, int group) {
    if (K <= 0 || N_total <= 0 || group <= 0) return 1;
    const int n_groups = K / group;
    const int tiles = (N_total / 8 + fq::GEMV_PACKS - 1) / fq::GEMV_PACKS;
    int want = (2 * 148 + tiles - 1) / tiles;       // about two CTAs per SM
    if (want > n_groups) want = n_groups;
    if (want < 1) want = 1;
    // groups per split must cover all groups: round the split count to ceil(n_groups / gps)
    const int gps = (n_groups + want - 1) / want;
    return (n_groups + gps - 1) / gps;
}

extern "C" int fq_awq_gemv(
    const void* x, int M, int K, int group, int n_proj,
    const int32_t* const* qweight, const void* const* scales, const int32_t* const* qzeros, const void* const* bias,
    const int* N, void* const* y, int interleaved, void* workspace, size_t workspace_bytes, int k_split, void* stream) {
    using namespace fq;
    const char* fn = "fq_awq_gemv";
    FQ_CHECK_ARG(M >= 1 && M <= 8, FQ_ERR_UNSUPPORTED, "%s: M=%d rows; the GEMV path takes 1..8 (larger M belongs to the GEMM path)", fn, M);
    FQ_CHECK_ARG(group == 32 || group == 64 || group == 128, FQ_ERR_UNSUPPORTED, "%s: group size %d; 32, 64 and 128 are built", fn, group);
    FQ_CHECK_ARG(K > 0 && K % group == 0, FQ_ERR_ARG, "%s: K=%d must be a multiple of the group size %d", fn, K, group);
    FQ_CHECK_ARG(n_proj >= 1 && n_proj <= GEMV_MAX_PROJ, FQ_ERR_ARG, "%s: 1..%d projections per call, got %d", fn, GEMV_MAX_PROJ, n_proj);
    FQ_CHECK_ARG(x && qweight && scales && qzeros && N && y, FQ_ERR_ARG, "%s: null pointer", fn);
    FQ_CHECK_ARG(aligned(x, 16), FQ_ERR_ALIGN, "%s: x must be 16-byte aligned", fn);
    FQ_CHECK_ARG(k_split >= 1, FQ_ERR_ARG, "%s: k_split=%d", fn, k_split);
    GemvParams p;
    p.x = static_cast<const __half*>(x); p.M = M; p.K = K; p.group = group; p.n_groups = K / group;
    p.n_proj = n_proj; p.interleaved = interleaved ? 1 : 0;
    int tile0 = 0, n_total = 0, vec16 = 1;
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
        tile0 += (N[i] / 8 + GEMV_PACKS - 1) / GEMV_PACKS;
        n_total += N[i];
    }
    for (int i = n_proj; i < GEMV_MAX_PROJ; ++i) p.proj[i] = GemvProj{nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0};
    p.tiles_total = tile0; p.vec16 = vec16;
    const int tiles = tile0;
    if (k_split > p.n_groups) k_split = p.n_groups;
    p.groups_per_split = (p.n_groups + k_split - 1) / k_split;
    k_split = (p.n_groups + p.groups_per_split - 1) / p.groups_per_split;
    p.k_split = k_split;
    FQ_CHECK_ARG(k_split <= 65535, FQ_ERR_ARG, "%s: k_split=%d", fn, k_split);
    p.partials = nullptr; p.tickets = nullptr;
    const int Mp = gemv_mp(M);
    if (k_split > 1) {
        const size_t need = fq_awq_gemv_workspace_bytes(M, n_total, k_split);
        FQ_CHECK_ARG(workspace && workspace_bytes >= need, FQ_ERR_WORKSPACE, "%s: workspace of %zu B needed, %zu given", fn, need, workspace_bytes);
        FQ_CHECK_ARG(aligned(workspace, 16), FQ_ERR_ALIGN, "%s: workspace must be 16-byte aligned", fn);
        p.tickets = static_cast<int*>(workspace);
        p.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + ((gemv_tiles_bound(n_total) * 4 + 255) & ~(size_t)255));
    }
    const size_t smem = (size_t)GEMV_STAGES * GEMV_STAGE_WORDS * 4 + (size_t)GEMV_STAGES * Mp * GEMV_ROWS * 2 + (size_t)GEMV_ROWS * Mp * 8;
    dim3 grid((unsigned)tiles, (unsigned)k_split);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define FQ_GEMV(MV)                                                                                          \
    do {                                                                                                     \
        static bool attr_set[64] = {};                                                                       \
        int dev = 0; cudaGetDevice(&dev);                                                                    \
        if (dev < 0 || dev >= 64 || !attr_set[dev]) {                                                        \
            cudaError_t e = cudaFuncSetAttribute(awq_gemv_kernel<MV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: cannot reserve %zu B of shared memory: %s", fn, smem, cudaGetErrorString(e)); \
            if (dev >= 0 && dev < 64) attr_set[dev] = true;                                                  \
        }                                                                                                    \
        launch_k(PDL_GEMV, awq_gemv_kernel<MV>, grid, dim3(GEMV_THREADS), smem, st, p);                                          \
    } while (0)
    if (Mp == 1) FQ_GEMV(1);
    else if (Mp == 2) FQ_GEMV(2);
    else if (Mp == 4) FQ_GEMV(4);
    else FQ_GEMV(8);
#undef FQ_GEMV
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}
