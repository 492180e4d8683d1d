// The small operators around the sparse-decode path in a Llama-shaped decode step: residual
// add + RMSNorm, rotary embedding of q and k, SwiGLU, the fp16 lm_head GEMV and argmax.
// They restate what the reference's patched forward inherits from the Hugging Face Llama
// modules it wraps (flashquest/eager/llama_persistent_patch.py:164-305 calls q/k/v_proj,
// apply_rotary_pos_emb, o_proj; the decoder layer around it adds the norms, residuals and the
// MLP), with the same intermediate roundings to fp16.  All are HBM- or latency-bound
// element-wise / reduction kernels; one launch each, programmatic dependent launch like the
// rest of the chain.
#include "fq_common.cuh"

#include <cooperative_groups.h>

namespace fq {

constexpr int NORM_THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float* s_red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < nw; ++w) t += s_red[w];
    return t;
}

// h = a (+ b) in fp16; sum_out = h; y = weight * fp16(h * rsqrt(mean(h^2) + eps))   (one CTA per row)
__global__ void __launch_bounds__(NORM_THREADS) add_rmsnorm_kernel(
    const __half* __restrict__ a, const __half* __restrict__ b, const __half* __restrict__ weight, float eps,
    int H, __half* __restrict__ sum_out, __half* __restrict__ y) {
    __shared__ float s_red[NORM_THREADS / 32];
    extern __shared__ __half s_row[];                 // the row after the add
    const int64_t row = blockIdx.x;
    pdl_wait();
    pdl_trigger();
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += NORM_THREADS) {
        __half h = a[row * H + i];
        if (b) h = __hadd(h, b[row * H + i]);
        s_row[i] = h;
        if (sum_out) sum_out[row * H + i] = h;
        const float f = __half2float(h);
        ss = fmaf(f, f, ss);
    }
    const float var = block_sum(ss, s_red) / (float)H;
    const float r = rsqrtf(var + eps);
    for (int i = threadIdx.x; i < H; i += NORM_THREADS) {
        const __half xh = __float2half_rn(__half2float(s_row[i]) * r);
        y[row * H + i] = __hmul(weight[i], xh);
    }
}

// Rotary embedding in place, Hugging Face "rotate_half" convention: for i < D/2
//   out[i]       = x[i]*cos_i       + (-x[i + D/2])*sin_i
//   out[i + D/2] = x[i + D/2]*cos_i + ( x[i])*sin_i
// with cos/sin computed in fp32 from pos * theta^(-2i/D) and rounded to fp16, products and sum in fp16.
__global__ void __launch_bounds__(128) rope_kernel(__half* __restrict__ q, int64_t q_sb, int64_t q_sh, int Hq,
                                                   __half* __restrict__ k, int64_t k_sb, int64_t k_sh, int Hkv,
                                                   int D, int pos, float theta, const int* __restrict__ pos_dev, int pos_step) {
    const int head = blockIdx.x, b = blockIdx.y;
    pdl_wait();
    pdl_trigger();
    if (pos_dev) pos = *pos_dev;      // position read on the device (graph-capturable step)
    pos += b * pos_step;              // rows are consecutive tokens of one sequence (prefill) when pos_step = 1
    __half* x = head < Hq ? q + b * q_sb + head * q_sh : k + b * k_sb + (head - Hq) * k_sh;
    const int half = D / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float inv_freq = 1.0f / powf(theta, (float)(2 * i) / (float)D);
        const float ang = (float)pos * inv_freq;
        const __half c = __float2half_rn(cosf(ang)), s = __float2half_rn(sinf(ang));
        const __half x1 = x[i], x2 = x[i + half];
        x[i] = __hadd(__hmul(x1, c), __hmul(__hneg(x2), s));
        x[i + half] = __hadd(__hmul(x2, c), __hmul(x1, s));
    }
}

// out = fp16(silu(gate)) * up, silu evaluated in fp32
__global__ void __launch_bounds__(256) swiglu_kernel(const __half2* __restrict__ gate, const __half2* __restrict__ up,
                                                     int64_t n2, __half2* __restrict__ out) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n2; i += (int64_t)gridDim.x * blockDim.x) {
        const float2 g = __half22float2(gate[i]);
        const __half2 a = __floats2half2_rn(g.x / (1.0f + expf(-g.x)), g.y / (1.0f + expf(-g.y)));
        out[i] = __hmul2(a, up[i]);
    }
}

// y[m, n] = sum_k x[m, k] * W[n, k]: fp16 weights (N, K) row-major read once, fp32 accumulation.
// One warp per output row, x (M <= 8 rows) staged in shared memory as fp32.
constexpr int GEMVH_WARPS = 8;
template <int M>
__global__ void __launch_bounds__(GEMVH_WARPS * 32) gemv_f16_kernel(const __half* __restrict__ x, const __half* __restrict__ W,
                                                                    int Mrows, int K, int N, __half* __restrict__ y) {
    extern __shared__ float s_x[];                    // [M][K]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * GEMVH_WARPS + warp;
    // the weights never change: request the first pieces of the row before the dependency wait
    uint4 w0 = make_uint4(0, 0, 0, 0);
    const uint4* wrow = reinterpret_cast<const uint4*>(W + (int64_t)min(n, N - 1) * K);
    if (lane * 8 < K) w0 = __ldg(wrow + lane);
    pdl_wait();
    pdl_trigger();
    for (int i = threadIdx.x; i < M * K; i += GEMVH_WARPS * 32) {
        const int m = i / K, kk = i % K;
        s_x[i] = m < Mrows ? __half2float(x[(int64_t)m * K + kk]) : 0.f;
    }
    __syncthreads();
    if (n >= N) return;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    for (int c = lane; c * 8 < K; c += 32) {
        const uint4 w = c == lane ? w0 : __ldg(wrow + c);
        const __half2* wh = reinterpret_cast<const __half2*>(&w);
        float wf[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __half22float2(wh[j]); wf[2 * j] = f.x; wf[2 * j + 1] = f.y; }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const float4 xa = *reinterpret_cast<const float4*>(s_x + m * K + c * 8);
            const float4 xb = *reinterpret_cast<const float4*>(s_x + m * K + c * 8 + 4);
            acc[m] = fmaf(wf[0], xa.x, fmaf(wf[1], xa.y, fmaf(wf[2], xa.z, fmaf(wf[3], xa.w, acc[m]))));
            acc[m] = fmaf(wf[4], xb.x, fmaf(wf[5], xb.y, fmaf(wf[6], xb.z, fmaf(wf[7], xb.w, acc[m]))));
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], off);
        if (lane == 0 && m < Mrows) y[(int64_t)m * N + n] = __float2half_rn(acc[m]);
    }
}

// The same product for 2..8 rows on the tensor cores (mma.sync m16n8k16, fp32 accumulation): on the CUDA cores every
// weight costs one fma per row and a shared-memory read of x, which for 8 rows is several times the HBM time of W.
// A warp owns 16 output rows (A = 16 rows of W, straight from global memory with 16-byte loads), B = the rows of x
// (staged once per CTA as fp16, padded to 8 rows); lane (g, t) reads W[n0+g][k0+8t .. +7] and W[n0+g+8][...], i.e. the
// k index inside an MMA is permuted the same way for A and B.  CTAs are persistent over tiles of 128 output rows.
constexpr int GEMVM_WARPS = 8;
constexpr int GEMVM_XPAD = 32;      // fp16 elements: row stride = 16 words mod 32, conflict-free 16-byte fragment loads

__global__ void __launch_bounds__(GEMVM_WARPS * 32) gemv_f16_mma_kernel(const __half* __restrict__ x, const __half* __restrict__ W,
                                                                        int Mrows, int K, int N, __half* __restrict__ y) {
    extern __shared__ __align__(16) __half s_xh[];      // [8][K + XPAD]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int xs = K + GEMVM_XPAD;
    pdl_wait();
    pdl_trigger();
    for (int i = threadIdx.x; i < 8 * (K / 8); i += GEMVM_WARPS * 32) {
        const int m = i / (K / 8), kk = (i - m * (K / 8)) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m < Mrows) v = __ldcg(reinterpret_cast<const uint4*>(x + (int64_t)m * K + kk));
        *reinterpret_cast<uint4*>(s_xh + m * xs + kk) = v;
    }
    __syncthreads();
    const int tiles = (N + 16 * GEMVM_WARPS - 1) / (16 * GEMVM_WARPS);
    const __half* xrow = s_xh + g * xs + 8 * t;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int n0 = tile * 16 * GEMVM_WARPS + warp * 16;
        if (n0 >= N) continue;
        const __half* wa = W + (int64_t)min(n0 + g, N - 1) * K + 8 * t;
        const __half* wb = W + (int64_t)min(n0 + g + 8, N - 1) * K + 8 * t;
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int k0 = 0; k0 < K; k0 += 32) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(wa + k0));
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(wb + k0));
            const uint4 xv = *reinterpret_cast<const uint4*>(xrow + k0);
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a.x), "r"(b.x), "r"(a.y), "r"(b.y), "r"(xv.x), "r"(xv.y));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a.z), "r"(b.z), "r"(a.w), "r"(b.w), "r"(xv.z), "r"(xv.w));
        }
        // c0, c1: output row n0+g for x rows 2t, 2t+1; c2, c3: output row n0+g+8
        if (2 * t < Mrows) {
            if (n0 + g < N) y[(int64_t)(2 * t) * N + n0 + g] = __float2half_rn(c[0]);
            if (n0 + g + 8 < N) y[(int64_t)(2 * t) * N + n0 + g + 8] = __float2half_rn(c[2]);
        }
        if (2 * t + 1 < Mrows) {
            if (n0 + g < N) y[(int64_t)(2 * t + 1) * N + n0 + g] = __float2half_rn(c[1]);
            if (n0 + g + 8 < N) y[(int64_t)(2 * t + 1) * N + n0 + g + 8] = __float2half_rn(c[3]);
        }
    }
}

// index of the first maximum of each row (torch.argmax): a cluster of ARGMAX_CTAS CTAs per row, each scans
// a contiguous slice and sends its best (value, index) to the first CTA through distributed shared memory
constexpr int ARGMAX_CTAS = 8;
constexpr int ARGMAX_THREADS = 512;

__device__ __forceinline__ bool argmax_better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_f16_kernel(const __half* __restrict__ x, int N, int32_t* __restrict__ out) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    __shared__ float s_cv[ARGMAX_CTAS];
    __shared__ int s_ci[ARGMAX_CTAS];
    const int64_t row = blockIdx.y;
    const int rank = blockIdx.x;
    cluster.barrier_arrive();
    pdl_wait();
    pdl_trigger();
    const int per = (N + ARGMAX_CTAS - 1) / ARGMAX_CTAS;
    const int lo = rank * per, hi = min(N, lo + per);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    const __half* xr = x + row * N;
    for (int i = lo + threadIdx.x; i < hi; i += ARGMAX_THREADS) {
        const float v = __half2float(xr[i]);
        if (bi == 0x7fffffff || argmax_better(v, i, best, bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (argmax_better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_v[warp] = best; s_i[warp] = bi; }
    __syncthreads();
    cluster.barrier_wait();            // every CTA of the cluster runs: the first one's shared memory may be addressed
    if (warp == 0) {
        constexpr int nw = ARGMAX_THREADS / 32;
        best = lane < nw ? s_v[lane] : -INFINITY;
        bi = lane < nw ? s_i[lane] : 0x7fffffff;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (argmax_better(ov, oi, best, bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) {
            cluster.map_shared_rank(s_cv, 0)[rank] = best;
            cluster.map_shared_rank(s_ci, 0)[rank] = bi;
        }
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x == 0) {
        best = s_cv[0]; bi = s_ci[0];
        for (int r = 1; r < ARGMAX_CTAS; ++r)
            if (argmax_better(s_cv[r], s_ci[r], best, bi)) { best = s_cv[r]; bi = s_ci[r]; }
        out[row] = bi;
    }
}

}  // namespace fq

extern "C" int fq_add_rmsnorm(const void* a, const void* b, const void* weight, float eps, int64_t rows, int H,
                              void* sum_out, void* y, void* stream) {
    using namespace fq;
    const char* fn = "fq_add_rmsnorm";
    FQ_CHECK_ARG(a && weight && y && rows >= 0 && H > 0, FQ_ERR_ARG, "%s: bad arguments", fn);
    FQ_CHECK_ARG((size_t)H * 2 <= 96 * 1024, FQ_ERR_UNSUPPORTED, "%s: hidden size %d too large", fn, H);
    if (rows == 0) return FQ_OK;
    const size_t smem = (size_t)H * 2;
    if (smem > 40 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: %s", fn, cudaGetErrorString(e));
    }
    launch_k(PDL_GEMV, add_rmsnorm_kernel, dim3((unsigned)rows), dim3(NORM_THREADS), smem, static_cast<cudaStream_t>(stream),
             static_cast<const __half*>(a), static_cast<const __half*>(b), static_cast<const __half*>(weight), eps, H,
             static_cast<__half*>(sum_out), static_cast<__half*>(y));
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

namespace fq {
int rope_launch(void* q, int64_t q_sb, int64_t q_sh, int Hq, void* k, int64_t k_sb, int64_t k_sh, int Hkv,
                int B, int D, int pos, float theta, void* stream, const int* pos_dev, int pos_step) {
    const char* fn = "fq_rope";
    FQ_CHECK_ARG(q && k && B > 0 && Hq > 0 && Hkv > 0 && D > 0 && D % 2 == 0 && pos >= 0 && theta > 0.f, FQ_ERR_ARG, "%s: bad arguments", fn);
    FQ_CHECK_ARG(B <= 65535, FQ_ERR_ARG, "%s: batch %d too large", fn, B);
    launch_k(PDL_GEMV, rope_kernel, dim3((unsigned)(Hq + Hkv), (unsigned)B), dim3(D / 2 < 128 ? (D / 2 + 31) / 32 * 32 : 128), 0,
             static_cast<cudaStream_t>(stream), static_cast<__half*>(q), q_sb, q_sh, Hq, static_cast<__half*>(k), k_sb, k_sh, Hkv,
             D, pos, theta, pos_dev, pos_step);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}
}  // namespace fq

extern "C" int fq_rope(void* q, int64_t q_sb, int64_t q_sh, int Hq, void* k, int64_t k_sb, int64_t k_sh, int Hkv,
                       int B, int D, int pos, float theta, void* stream) {
    return fq::rope_launch(q, q_sb, q_sh, Hq, k, k_sb, k_sh, Hkv, B, D, pos, theta, stream, nullptr, 0);
}

extern "C" int fq_rope_tokens(void* q, int64_t q_st, int64_t q_sh, int Hq, void* k, int64_t k_st, int64_t k_sh, int Hkv,
                              int n_tokens, int D, int pos0, float theta, void* stream) {
    return fq::rope_launch(q, q_st, q_sh, Hq, k, k_st, k_sh, Hkv, n_tokens, D, pos0, theta, stream, nullptr, 1);
}

extern "C" int fq_swiglu(const void* gate, const void* up, int64_t n, void* out, void* stream) {
    using namespace fq;
    const char* fn = "fq_swiglu";
    FQ_CHECK_ARG(gate && up && out && n >= 0 && n % 2 == 0, FQ_ERR_ARG, "%s: bad arguments (n must be even)", fn);
    FQ_CHECK_ARG(aligned(gate, 4) && aligned(up, 4) && aligned(out, 4), FQ_ERR_ALIGN, "%s: tensors must be 4-byte aligned", fn);
    if (n == 0) return FQ_OK;
    const int64_t n2 = n / 2;
    const unsigned blocks = (unsigned)((n2 + 255) / 256 < 148 * 8 ? (n2 + 255) / 256 : 148 * 8);
    launch_k(PDL_GEMV, swiglu_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
             static_cast<const __half2*>(gate), static_cast<const __half2*>(up), n2, static_cast<__half2*>(out));
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" int fq_gemv_f16(const void* x, const void* W, int M, int K, int N, void* y, void* stream) {
    using namespace fq;
    const char* fn = "fq_gemv_f16";
    FQ_CHECK_ARG(x && W && y && N > 0 && K > 0, FQ_ERR_ARG, "%s: bad arguments", fn);
    FQ_CHECK_ARG(M >= 1 && M <= 8, FQ_ERR_UNSUPPORTED, "%s: M=%d rows; 1..8 are built", fn, M);
    FQ_CHECK_ARG(K % 8 == 0 && aligned(W, 16) && aligned(x, 2), FQ_ERR_ALIGN, "%s: K must be a multiple of 8 and W 16-byte aligned", fn);
    cudaStream_t st0 = static_cast<cudaStream_t>(stream);
    if (M >= 2 && K % 32 == 0 && (size_t)8 * (K + GEMVM_XPAD) * 2 <= 100 * 1024) {
        const size_t smem_m = (size_t)8 * (K + GEMVM_XPAD) * 2;
        if (smem_m > 40 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(gemv_f16_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_m);
            if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: %s", fn, cudaGetErrorString(e));
        }
        const int tiles = (N + 16 * GEMVM_WARPS - 1) / (16 * GEMVM_WARPS);
        launch_k(PDL_GEMV, gemv_f16_mma_kernel, dim3((unsigned)(tiles < 2 * 148 ? tiles : 2 * 148)), dim3(GEMVM_WARPS * 32), smem_m, st0,
                 static_cast<const __half*>(x), static_cast<const __half*>(W), M, K, N, static_cast<__half*>(y));
        FQ_CHECK_LAUNCH(fn);
        return FQ_OK;
    }
    const int Mp = M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8));
    const size_t smem = (size_t)Mp * K * 4;
    FQ_CHECK_ARG(smem <= 200 * 1024, FQ_ERR_UNSUPPORTED, "%s: M x K = %d x %d does not fit in shared memory", fn, M, K);
    dim3 grid((unsigned)((N + GEMVH_WARPS - 1) / GEMVH_WARPS));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define FQ_GH(MV)                                                                                                  \
    do {                                                                                                           \
        if (smem > 40 * 1024) {                                                                                    \
            cudaError_t e = cudaFuncSetAttribute(gemv_f16_kernel<MV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: %s", fn, cudaGetErrorString(e));                   \
        }                                                                                                          \
        launch_k(PDL_GEMV, gemv_f16_kernel<MV>, grid, dim3(GEMVH_WARPS * 32), smem, st, static_cast<const __half*>(x), \
                 static_cast<const __half*>(W), M, K, N, static_cast<__half*>(y));                                 \
    } while (0)
    if (Mp == 1) FQ_GH(1);
    else if (Mp == 2) FQ_GH(2);
    else if (Mp == 4) FQ_GH(4);
    else FQ_GH(8);
#undef FQ_GH
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

extern "C" int fq_argmax_f16(const void* x, int64_t rows, int N, int32_t* out, void* stream) {
    using namespace fq;
    const char* fn = "fq_argmax_f16";
    FQ_CHECK_ARG(x && out && rows >= 0 && N > 0, FQ_ERR_ARG, "%s: bad arguments", fn);
    if (rows == 0) return FQ_OK;
    FQ_CHECK_ARG(rows <= 65535, FQ_ERR_ARG, "%s: at most 65535 rows", fn);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ARGMAX_CTAS, (unsigned)rows); cfg.blockDim = dim3(ARGMAX_THREADS); cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute at[2]{};
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = ARGMAX_CTAS; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 2;
    cudaLaunchKernelEx(&cfg, argmax_f16_kernel, static_cast<const __half*>(x), N, out);
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}

// seen: host positions (stream step) or nullptr with pos_dev: device positions (graph-capturable step)
static int llama_step_impl(const fq_llama_model* m, const fq_int4_cache* cache, const fq_decode_params* prm,
                           const int* seen, int* pos_dev, const void* x, int B, const fq_llama_scratch* s, void* stream) {
    using namespace fq;
    const char* fn = pos_dev ? "fq_llama_decode_step_dev" : "fq_llama_decode_step";
    FQ_CHECK_ARG(m && cache && prm && (seen || pos_dev) && x && s && m->layers, FQ_ERR_ARG, "%s: null argument", fn);
    FQ_CHECK_ARG(B >= 1 && B <= 8 && B == cache->B, FQ_ERR_ARG, "%s: batch %d (cache %d); 1..8 sequences are built", fn, B, cache->B);
    FQ_CHECK_ARG(m->n_layers >= 1 && m->n_layers <= cache->L && m->kv_heads == cache->Hkv && m->head_dim == cache->D &&
                 m->q_heads == prm->Hq, FQ_ERR_ARG, "%s: model and cache shapes differ", fn);
    FQ_CHECK_ARG(cache->kv_dtype == FQ_F16, FQ_ERR_DTYPE, "%s: the step computes in fp16; the cache stages dtype code %d", fn, cache->kv_dtype);
    const int H = m->hidden, D = m->head_dim, Hq = m->q_heads, Hkv = m->kv_heads;
    const int nq = Hq * D, nkv = Hkv * D;
    int rc;
    // split counts of the four GEMV shapes
    const int ks_qkv = fq_awq_gemv_default_splits(H, nq + 2 * nkv, m->group);
    const int ks_o = fq_awq_gemv_default_splits(nq, H, m->group);
    const int ks_gu = fq_awq_gemv_default_splits(H, 2 * m->ffn, m->group);
    const int ks_dn = fq_awq_gemv_default_splits(m->ffn, H, m->group);

    const void* xin = x;          // residual stream; alternates between the two buffers
    const void* delta = nullptr;  // output of the previous block, added by the next norm
    int flip = 0;
    // residual add + RMSNorm folded into the GEMV that consumes it: the prologue record and the buffer the sum goes to
    auto norm_prologue = [&](const void* w, fq_gemv_prologue& pro) -> const void* {
        pro.kind = FQ_GEMV_ADD_RMSNORM; pro.b = delta; pro.weight = w; pro.eps = m->rms_eps; pro.out = nullptr;
        const void* src = xin;
        if (delta) { pro.out = flip ? s->resid1 : s->resid0; flip ^= 1; xin = pro.out; }
        return src;
    };
    auto add_norm = [&](const void* w) -> int {
        void* out = nullptr;
        if (delta) { out = flip ? s->resid1 : s->resid0; flip ^= 1; }
        const int r = fq_add_rmsnorm(xin, delta, w, m->rms_eps, B, H, out, s->normed, stream);
        if (out) xin = out;
        return r;
    };
    for (int l = 0; l < m->n_layers; ++l) {
        const fq_llama_layer& L = m->layers[l];
        FQ_CHECK_ARG(L.q.K == H && L.q.N == nq && L.k.N == nkv && L.v.N == nkv && L.o.K == nq && L.o.N == H &&
                     L.gate.N == m->ffn && L.up.N == m->ffn && L.down.K == m->ffn && L.down.N == H, FQ_ERR_ARG,
                     "%s: layer %d has unexpected projection shapes", fn, l);
        void* Ol = static_cast<char*>(s->O) + (size_t)l * s->o_sl * 2;
        {
            // input_layernorm -> q/k/v -> rotary embedding of q and k: one launch
            const int32_t* qw[3] = {L.q.qweight, L.k.qweight, L.v.qweight};
            const void* sc[3] = {L.q.scales, L.k.scales, L.v.scales};
            const int32_t* qz[3] = {L.q.qzeros, L.k.qzeros, L.v.qzeros};
            const void* bs[3] = {L.q.bias, L.k.bias, L.v.bias};
            const int N[3] = {nq, nkv, nkv};
            void* y[3] = {s->q, s->k, s->v};
            fq_gemv_prologue pro;
            const void* src = norm_prologue(L.input_norm, pro);
            fq_gemv_rope rope;
            rope.proj_mask = 3u; rope.pos_dev = pos_dev ? pos_dev + l : nullptr; rope.pos = pos_dev ? 0 : seen[l];
            rope.theta = m->rope_theta; rope.head_dim = D;
            rc = fq_awq_gemv_fused(src, B, H, m->group, 3, qw, sc, qz, (bs[0] || bs[1] || bs[2]) ? bs : nullptr, N, y, m->interleaved,
                                   &pro, &rope, ks_qkv, stream);
            if (rc != FQ_OK) return rc;
        }
        if (pos_dev) {
            rc = decode_layer_int4_dyn(cache, l, pos_dev + l, s->k, s->v, nkv, D, D, 1, s->q, FQ_F16, nq, D, prm,
                                       s->scores + l * s->sc_sl, s->compact + l * s->cp_sl, Ol, nullptr,
                                       static_cast<char*>(s->attn_ws) + (size_t)l * s->attn_ws_sl, s->attn_ws_bytes, stream);
        } else {
            rc = fq_decode_layer_int4(cache, l, seen[l], s->k, s->v, nkv, D, D, 1, s->q, FQ_F16, nq, D, prm,
                                      s->scores + l * s->sc_sl, s->compact + l * s->cp_sl, Ol, nullptr,
                                      static_cast<char*>(s->attn_ws) + (size_t)l * s->attn_ws_sl, s->attn_ws_bytes, stream);
        }
        if (rc != FQ_OK) return rc;
        {
            const int32_t* qw[1] = {L.o.qweight}; const void* sc[1] = {L.o.scales}; const int32_t* qz[1] = {L.o.qzeros};
            const void* bs[1] = {L.o.bias}; const int N[1] = {H}; void* y[1] = {s->attn_out};
            rc = fq_awq_gemv(Ol, B, nq, m->group, 1, qw, sc, qz, bs[0] ? bs : nullptr, N, y, m->interleaved, ks_o, stream);
            if (rc != FQ_OK) return rc;
        }
        delta = s->attn_out;
        {
            // post_attention_layernorm -> gate/up: one launch
            const int32_t* qw[2] = {L.gate.qweight, L.up.qweight}; const void* sc[2] = {L.gate.scales, L.up.scales};
            const int32_t* qz[2] = {L.gate.qzeros, L.up.qzeros}; const void* bs[2] = {L.gate.bias, L.up.bias};
            const int N[2] = {m->ffn, m->ffn}; void* y[2] = {s->gate, s->up};
            fq_gemv_prologue pro;
            const void* src = norm_prologue(L.post_norm, pro);
            rc = fq_awq_gemv_fused(src, B, H, m->group, 2, qw, sc, qz, (bs[0] || bs[1]) ? bs : nullptr, N, y, m->interleaved,
                                   &pro, nullptr, ks_gu, stream);
            if (rc != FQ_OK) return rc;
        }
        {
            // act_fn(gate) * up -> down: one launch
            const int32_t* qw[1] = {L.down.qweight}; const void* sc[1] = {L.down.scales}; const int32_t* qz[1] = {L.down.qzeros};
            const void* bs[1] = {L.down.bias}; const int N[1] = {H}; void* y[1] = {s->down};
            fq_gemv_prologue pro;
            pro.kind = FQ_GEMV_SWIGLU; pro.b = s->up; pro.weight = nullptr; pro.eps = 0.f; pro.out = nullptr;
            rc = fq_awq_gemv_fused(s->gate, B, m->ffn, m->group, 1, qw, sc, qz, bs[0] ? bs : nullptr, N, y, m->interleaved,
                                   &pro, nullptr, ks_dn, stream);
            if (rc != FQ_OK) return rc;
        }
        delta = s->down;
    }
    if ((rc = add_norm(m->final_norm)) != FQ_OK) return rc;
    if ((rc = fq_gemv_f16(s->normed, m->lm_head, B, H, m->vocab, s->logits, stream)) != FQ_OK) return rc;
    if ((rc = fq_argmax_f16(s->logits, B, m->vocab, s->next_ids, stream)) != FQ_OK) return rc;
    return pos_dev ? advance_positions(pos_dev, m->n_layers, 1, cache->max_seq_len, stream) : FQ_OK;
}

extern "C" int fq_llama_decode_step(const fq_llama_model* m, const fq_int4_cache* cache, const fq_decode_params* prm,
                                    const int* seen, const void* x, int B, const fq_llama_scratch* s, void* stream) {
    return llama_step_impl(m, cache, prm, seen, nullptr, x, B, s, stream);
}

extern "C" int fq_llama_decode_step_dev(const fq_llama_model* m, const fq_int4_cache* cache, const fq_decode_params* prm,
                                        int* pos, const void* x, int B, const fq_llama_scratch* s, void* stream) {
    return llama_step_impl(m, cache, prm, nullptr, pos, x, B, s, stream);
}
