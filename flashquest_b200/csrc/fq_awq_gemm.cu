// AWQ W4A16 dequant-GEMM on the 5th-generation tensor cores (tcgen05) for prefill / batched
// shapes: y[M,N] = x[M,K] @ W, W in AutoAWQ's GEMM format (4-bit codes, group scales and zeros).
// The M <= 8 decode shapes stay with the GEMV (fq_awq_gemv.cu); this kernel is the dense
// contraction of the prefill branch (the q/k/v/o/gate/up/down linears over all prompt tokens).
//
// A CTA is persistent: it walks output tiles of 256 x 128 (two 128 x 128 accumulators in tensor memory
// that share every weight tile; two such sets, so that a finished tile is drained while the next one
// is multiplied) and, inside a tile, K in steps of 64:
//   warp 0       : one thread issues the TMA loads of a stage — two x tiles of 128 rows x 64 k
//                  (fp16, 128-byte swizzle, K-major) and the raw weight tile of 64 k x 16 int32;
//   warp 1       : one thread issues tcgen05.mma (M 128, N 128, K 16, fp16 x fp16 -> fp32 in TMEM),
//                  eight per stage, commits the stage back to the producer and the accumulator set
//                  to the epilogue; the warp also owns the tensor-memory allocation (512 columns);
//   warps 2..9   : dequantise the raw tile to fp16 in shared memory, (code - zero) * scale rounded
//                  once to fp16 like the reference's GEMM kernels, written N-contiguous in the
//                  canonical MN-major 128-byte-swizzle layout (AWQ's nibble order makes every
//                  masked word a pair of neighbouring columns, so a 32-bit word of codes becomes one
//                  16-byte store);
//   warps 10..13 : epilogue — drain an accumulator set (tcgen05.ld, lane quarter = warp id mod 4),
//                  add the bias, convert to fp16, store y, hand the set back.
// Stages and accumulator sets are handed over through mbarriers (TMA bytes -> dequantised ->
// consumed; multiplied -> drained); every wait is bounded and reports through the device status
// word instead of spinning forever.
#include <cuda.h>

#include "fq_common.cuh"

namespace fq {

constexpr int GM_BM = 128;          // rows per accumulator
constexpr int GM_BN = 256;          // columns per tile: one MMA of N = 256 per 16 k and accumulator
constexpr int GM_BK = 64;
constexpr int GM_TMEM_COLS = 512;   // all of an SM's tensor memory: MT = 1: two accumulator sets, MT = 2: one
constexpr int GM_DEQ_WARPS = 8;
constexpr int GM_EPI_WARPS = 4;
constexpr int GM_THREADS = (2 + GM_DEQ_WARPS + GM_EPI_WARPS) * 32;     // TMA warp, MMA warp, dequantise warps, epilogue warps

constexpr int GM_MAX_PROJ = 4;
constexpr unsigned GM_SPIN_LIMIT = 1u << 26;
constexpr int GM_A_BYTES = GM_BM * GM_BK * 2;             // 16 KiB per M tile
constexpr int GM_RAW_BYTES = GM_BK * (GM_BN / 8) * 4;     // 8 KiB
constexpr int GM_B_BYTES = GM_BK * GM_BN * 2;             // 32 KiB
// MT = accumulators (M tiles of 128 rows) per CTA tile.  MT = 2 (256 x 256 tiles, 3 stages): every byte fetched from L2
// feeds twice the MMAs, the tile for long M; MT = 1 (128 x 256 tiles, 4 stages, two accumulator sets so that a
// finished tile is drained while the next one is multiplied): more tiles, the one for short M.
template <int MT> struct GmCfg {
    static constexpr int STAGES = MT == 2 ? 3 : 4;
    static constexpr int ACC_SETS = GM_TMEM_COLS / (MT * GM_BN);
    static constexpr int STAGE_BYTES = MT * GM_A_BYTES + GM_B_BYTES + GM_RAW_BYTES;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers, tmem address */;
    static_assert((3 * STAGES + 2 * ACC_SETS) * 8 + 4 <= 256, "barrier block");
    static_assert(SMEM <= 227 * 1024, "shared memory");
};

struct GemmProj {
    const __half* scales; const int32_t* qzeros; const __half* bias; __half* y;
    int N, tile0;       // output columns; first N tile of this projection in the grid
};
struct GemmParams {
    GemmProj proj[GM_MAX_PROJ];
    int n_proj, M, K, group, interleaved;
    int n_tiles, m_tiles;   // N tiles over all projections, M tiles of 256 rows
    int* status;
};

__device__ __forceinline__ uint32_t gm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gm_mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gm_smem(bar)), "r"(count));
}
__device__ __forceinline__ void gm_mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(gm_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gm_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(gm_smem(bar)) : "memory");
}
__device__ __forceinline__ bool gm_mbar_try(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(gm_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait; false = gave up
__device__ __forceinline__ bool gm_wait(uint64_t* bar, unsigned parity) {
    unsigned spins = 0;
    while (!gm_mbar_try(bar, parity)) {
        if (++spins > GM_SPIN_LIMIT) return false;
    }
    return true;
}
__device__ __forceinline__ void gm_tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(gm_smem(dst)), "l"(map), "r"(gm_smem(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void gm_mma(uint32_t tmem_c, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_c), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void gm_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(gm_smem(bar)) : "memory");
}
// shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100); offsets in bytes
__device__ __forceinline__ uint64_t gm_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((smem_addr >> 4) & 0x3fff) | ((uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32) | (1ull << 46) | (2ull << 61);
}

template <bool INTERLEAVED, int GM_MT>
__global__ void __launch_bounds__(GM_THREADS, 1) awq_gemm_kernel(
    const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
    const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ CUtensorMap map_w3, const GemmParams p) {
    constexpr int GM_STAGES = GmCfg<GM_MT>::STAGES, GM_ACC_SETS = GmCfg<GM_MT>::ACC_SETS, GM_STAGE_BYTES = GmCfg<GM_MT>::STAGE_BYTES;
    extern __shared__ unsigned char gm_raw_smem[];
    // stage s: [A tiles | B (dequantised) | raw codes]; every tile 1024-byte aligned
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gm_raw_smem) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + GM_STAGES * GM_STAGE_BYTES);
    uint64_t* full_raw = bars;                       // [stages] TMA bytes landed (x tiles + raw codes)
    uint64_t* b_ready = bars + GM_STAGES;            // [stages] dequantised tile written (256 arrivals)
    uint64_t* empty = bars + 2 * GM_STAGES;          // [stages] the MMAs that read the stage have completed
    uint64_t* acc_ready = bars + 3 * GM_STAGES;      // [sets] all MMAs of a tile have completed
    uint64_t* acc_empty = acc_ready + GM_ACC_SETS;   // [sets] the epilogue has drained the set (128 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + GM_ACC_SETS);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int num_kb = p.K / GM_BK;
    const int total_tiles = p.n_tiles * p.m_tiles;

    if (tid == 0) {
        for (int s = 0; s < GM_STAGES; ++s) {
            gm_mbar_init(&full_raw[s], 1);
            gm_mbar_init(&b_ready[s], GM_DEQ_WARPS * 32);
            gm_mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < GM_ACC_SETS; ++a) {
            gm_mbar_init(&acc_ready[a], 1);
            gm_mbar_init(&acc_empty[a], GM_EPI_WARPS * 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {     // tensor memory: all 512 columns (ACC_SETS sets of MT accumulators of 256 fp32 columns)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gm_smem(tmem_slot)), "r"(GM_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    // tile index -> projection, first column inside it, first row (N tiles vary fastest: neighbouring CTAs share x rows)
    auto locate = [&](int tile, int& pj, int& n0, int& m0) {
        const int nt = tile % p.n_tiles;
        pj = 0;
#pragma unroll
        for (int i = 1; i < GM_MAX_PROJ; ++i)
            if (i < p.n_proj && nt >= p.proj[i].tile0) pj = i;
        n0 = (nt - p.proj[pj].tile0) * GM_BN;
        m0 = (tile / p.n_tiles) * (GM_BM * GM_MT);
    };

    if (warp == 0) {
        // =========================== TMA producer ===========================
        if (lane == 0) {
            int g = 0;                                  // k blocks issued so far, over all tiles
            for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x) {
                int pj, n0, m0;
                locate(tile, pj, n0, m0);
                const CUtensorMap* map_w = pj == 0 ? &map_w0 : (pj == 1 ? &map_w1 : (pj == 2 ? &map_w2 : &map_w3));
                for (int kb = 0; kb < num_kb; ++kb, ++g) {
                    const int s = g % GM_STAGES;
                    if (g >= GM_STAGES && !gm_wait(&empty[s], (unsigned)(g / GM_STAGES - 1) & 1u)) { failed = true; break; }
                    unsigned char* st = base + s * GM_STAGE_BYTES;
                    gm_mbar_expect_tx(&full_raw[s], GM_MT * GM_A_BYTES + GM_RAW_BYTES);
#pragma unroll
                    for (int mt = 0; mt < GM_MT; ++mt) gm_tma_2d(st + mt * GM_A_BYTES, &map_x, kb * GM_BK, m0 + mt * GM_BM, &full_raw[s]);
                    gm_tma_2d(st + GM_MT * GM_A_BYTES + GM_B_BYTES, map_w, n0 / 8, kb * GM_BK, &full_raw[s]);
                }
            }
        }
    } else if (warp == 1) {
        // =========================== MMA issuer ===========================
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, fp16 A (K-major) and B (MN-major), N = 128, M = 128
            const uint32_t idesc = (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (1u << 16) | ((uint32_t)(GM_BN >> 3) << 17) |
                                   ((uint32_t)(GM_BM >> 4) << 24);
            int g = 0, it = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x, ++it) {
                const int set = it % GM_ACC_SETS, use = it / GM_ACC_SETS;
                // the set must have been drained by the epilogue of the tile that used it last
                if (use >= 1 && !gm_wait(&acc_empty[set], (unsigned)(use - 1) & 1u)) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + (uint32_t)(set * GM_MT * GM_BN);
                for (int kb = 0; kb < num_kb; ++kb, ++g) {
                    const int s = g % GM_STAGES;
                    const unsigned ph = (unsigned)(g / GM_STAGES) & 1u;
                    if (!gm_wait(&full_raw[s], ph) || !gm_wait(&b_ready[s], ph)) { failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = gm_smem(base + s * GM_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + GM_MT * GM_A_BYTES;
#pragma unroll
                    for (int k = 0; k < GM_BK / 16; ++k) {
                        // B: MN-major; 64 columns x 8 k = one 1 KiB atom; atoms 1 KiB apart along K, BK*128 B apart along N (4 atoms)
                        const uint64_t db = gm_desc(b_addr + k * 2048, GM_BK * 128, 1024);
#pragma unroll
                        for (int mt = 0; mt < GM_MT; ++mt) {
                            // A: K-major; 8 rows x 64 k = one 1 KiB atom; 16 k = 32 B further inside the swizzled row
                            const uint64_t da = gm_desc(a_addr + mt * GM_A_BYTES + k * 32, 16, 1024);
                            gm_mma(acc + mt * GM_BN, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    gm_commit(&empty[s]);          // arrives when the MMAs issued so far have read their operands
                }
                if (!failed) gm_commit(&acc_ready[set]);
            }
        }
    } else if (warp < 2 + GM_DEQ_WARPS) {
        // =========================== dequantise ===========================
        const int t = tid - 64;                       // 0..255
        const int c = t & 31;                         // int32 column of the raw tile = 8 output columns n0 + 8c ..
        const int kr0 = t >> 5;                       // first k row of this thread; it takes rows kr0 + 8 i
        const int gpk = p.group / GM_BK;              // k blocks per quantisation group
        uint32_t zsub[4];                             // (1024 + zero) for the four column pairs, half2 bits
        __half2 sc2[4];                               // scales of the four column pairs
        const int a_n = c >> 3, chunk = c & 7;        // 64-column atom and 16-byte chunk inside its rows
        const int n_grp = (num_kb + gpk - 1) / gpk;
        int g = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x) {
            int pj, n0, m0;
            locate(tile, pj, n0, m0);
            const GemmProj& P = p.proj[pj];
            // scale and zero words of the NEXT group are requested one group ahead
            const bool col_ok = n0 + 8 * c < P.N;      // a projection of 128 (mod 256) columns ends inside its last tile
            auto load_meta = [&](int gi, uint32_t& zw, uint4& s4) {
                zw = 0; s4 = make_uint4(0, 0, 0, 0);
                if (col_ok) {
                    zw = (uint32_t)__ldg(P.qzeros + (int64_t)gi * (P.N / 8) + n0 / 8 + c);
                    s4 = __ldg(reinterpret_cast<const uint4*>(P.scales + (int64_t)gi * P.N + n0 + 8 * c));
                }
            };
            uint32_t zw_nx = 0; uint4 s4_nx = make_uint4(0, 0, 0, 0);
            load_meta(0, zw_nx, s4_nx);
            for (int kb = 0; kb < num_kb; ++kb, ++g) {
                const int s = g % GM_STAGES;
                if (kb % gpk == 0) {                      // new group: scale and zero of this thread's 8 columns
                    const int gi = kb / gpk;
                    const uint32_t zw = zw_nx;
                    const uint4 s4 = s4_nx;
                    if (gi + 1 < n_grp) load_meta(gi + 1, zw_nx, s4_nx);
                    const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) zsub[q] = ((zw >> (4 * q)) & 0x000f000fu) | 0x64006400u;
                    if constexpr (INTERLEAVED) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) sc2[q] = *reinterpret_cast<const __half2*>(&sw[q]);      // columns (2q, 2q+1)
                    } else {
                        // word q of the codes pairs columns (q, q+4)
                        const __half* sh = reinterpret_cast<const __half*>(sw);
#pragma unroll
                        for (int q = 0; q < 4; ++q) sc2[q] = __halves2half2(sh[q], sh[q + 4]);
                    }
                }
                if (!gm_wait(&full_raw[s], (unsigned)(g / GM_STAGES) & 1u)) { failed = true; break; }
                unsigned char* st = base + s * GM_STAGE_BYTES;
                const uint32_t* raw = reinterpret_cast<const uint32_t*>(st + GM_MT * GM_A_BYTES + GM_B_BYTES);
                unsigned char* bt = st + GM_MT * GM_A_BYTES + a_n * (GM_BK * 128);
#pragma unroll
                for (int i = 0; i < GM_BK / 8; ++i) {
                    const int kr = kr0 + 8 * i;
                    const uint32_t w = raw[kr * (GM_BN / 8) + c];
                    uint32_t o[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t h = ((w >> (4 * q)) & 0x000f000fu) | 0x64006400u;                   // (1024 + code) pairs
                        const __half2 d = __hsub2(*reinterpret_cast<const __half2*>(&h), *reinterpret_cast<const __half2*>(&zsub[q]));
                        const __half2 r = __hmul2(d, sc2[q]);
                        o[q] = *reinterpret_cast<const uint32_t*>(&r);
                    }
                    uint4 out;
                    if constexpr (INTERLEAVED) {
                        out = make_uint4(o[0], o[1], o[2], o[3]);
                    } else {      // pairs (q, q+4) -> column order
                        out = make_uint4(__byte_perm(o[0], o[1], 0x5410), __byte_perm(o[2], o[3], 0x5410),
                                         __byte_perm(o[0], o[1], 0x7632), __byte_perm(o[2], o[3], 0x7632));
                    }
                    // row kr of the atom column a_n: 128 B per row, 16-byte chunks swizzled by the row index
                    *reinterpret_cast<uint4*>(bt + kr * 128 + ((chunk ^ (kr & 7)) << 4)) = out;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> visible to the tensor core
                gm_mbar_arrive(&b_ready[s]);
            }
        }
    } else {
        // =========================== epilogue ===========================
        const int lq = warp & 3;                      // the TMEM lane quarter this warp may read
        int it = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x, ++it) {
            int pj, n0, m0;
            locate(tile, pj, n0, m0);
            const GemmProj& P = p.proj[pj];
            const int set = it % GM_ACC_SETS, use = it / GM_ACC_SETS;
            if (!gm_wait(&acc_ready[set], (unsigned)use & 1u)) { failed = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int mt = 0; mt < GM_MT; ++mt) {
                const int row = m0 + mt * GM_BM + lq * 32 + lane;
#pragma unroll 1
                for (int cb = 0; cb < GM_BN / 32; ++cb) {
                    uint32_t v[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(lq * 32) << 16) + (uint32_t)(set * GM_MT * GM_BN + mt * GM_BN + cb * 32);
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (row < p.M && n0 + cb * 32 < P.N) {
                        __half* yrow = P.y + (int64_t)row * P.N + n0 + cb * 32;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint32_t pk[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float f0 = __uint_as_float(v[j + 2 * e]), f1 = __uint_as_float(v[j + 2 * e + 1]);
                                if (P.bias) {
                                    f0 += __half2float(P.bias[n0 + cb * 32 + j + 2 * e]);
                                    f1 += __half2float(P.bias[n0 + cb * 32 + j + 2 * e + 1]);
                                }
                                const __half2 h = __floats2half2_rn(f0, f1);
                                pk[e] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                            *reinterpret_cast<uint4*>(yrow + j) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        }
                    }
                }
            }
            // the set's columns have been read: hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            gm_mbar_arrive(&acc_empty[set]);
        }
    }
    if (failed) atomicExch(p.status, FQ_ERR_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(GM_TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static std::atomic<void*> cached{nullptr};
    void* fn = cached.load(std::memory_order_relaxed);
    if (fn == nullptr) {
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess) return nullptr;
        cached.store(fn, std::memory_order_relaxed);
    }
    return reinterpret_cast<EncodeTiledFn>(fn);
}

}  // namespace fq

extern "C" int fq_awq_gemm(
    const void* x, int M, int K, int group, int n_proj,
    const int32_t* const* qweight, const void* const* scales, const int32_t* const* qzeros, const void* const* bias,
    const int* N, void* const* y, int interleaved, void* stream) {
    using namespace fq;
    const char* fn = "fq_awq_gemm";
    FQ_CHECK_ARG(M >= 1, FQ_ERR_ARG, "%s: M=%d", fn, M);
    FQ_CHECK_ARG(group == 64 || group == 128 || group == 256, FQ_ERR_UNSUPPORTED, "%s: group size %d; 64, 128 and 256 are built", fn, group);
    FQ_CHECK_ARG(K > 0 && K % group == 0, FQ_ERR_ARG, "%s: K=%d must be a multiple of the group size %d", fn, K, group);
    FQ_CHECK_ARG(n_proj >= 1 && n_proj <= GM_MAX_PROJ, FQ_ERR_ARG, "%s: 1..%d projections per call, got %d", fn, GM_MAX_PROJ, n_proj);
    FQ_CHECK_ARG(x && qweight && scales && qzeros && N && y, FQ_ERR_ARG, "%s: null pointer", fn);
    FQ_CHECK_ARG(aligned(x, 16), FQ_ERR_ALIGN, "%s: x must be 16-byte aligned", fn);
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return fail(FQ_ERR_CUDA, "%s: the driver does not export cuTensorMapEncodeTiled", fn);
    GemmParams p{};
    p.n_proj = n_proj; p.M = M; p.K = K; p.group = group; p.interleaved = interleaved ? 1 : 0;
    p.status = device_status_ptr();
    if (p.status == nullptr) return FQ_ERR_CUDA;
    CUtensorMap maps[1 + GM_MAX_PROJ];
    {
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
        const cuuint32_t box[2] = {(cuuint32_t)GM_BK, (cuuint32_t)GM_BM}, es[2] = {1, 1};
        CUresult r = encode(&maps[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(FQ_ERR_CUDA, "%s: tensor map for x: driver error %d", fn, (int)r);
    }
    int tile0 = 0;
    for (int i = 0; i < n_proj; ++i) {
        FQ_CHECK_ARG(N[i] > 0 && N[i] % 128 == 0, FQ_ERR_UNSUPPORTED, "%s: N[%d]=%d must be a positive multiple of 128", fn, i, N[i]);
        FQ_CHECK_ARG(qweight[i] && scales[i] && qzeros[i] && y[i], FQ_ERR_ARG, "%s: null tensor in projection %d", fn, i);
        FQ_CHECK_ARG(aligned(y[i], 16) && aligned(scales[i], 16) && aligned(qweight[i], 16) && aligned(qzeros[i], 4), FQ_ERR_ALIGN,
                     "%s: y[%d], scales[%d] and qweight[%d] must be 16-byte aligned", fn, i, i, i);
        p.proj[i] = GemmProj{static_cast<const __half*>(scales[i]), qzeros[i], bias ? static_cast<const __half*>(bias[i]) : nullptr,
                             static_cast<__half*>(y[i]), N[i], tile0};
        tile0 += (N[i] + GM_BN - 1) / GM_BN;
        const cuuint64_t dims[2] = {(cuuint64_t)(N[i] / 8), (cuuint64_t)K};
        const cuuint64_t strides[1] = {(cuuint64_t)(N[i] / 8) * 4};
        const cuuint32_t box[2] = {(cuuint32_t)(GM_BN / 8), (cuuint32_t)GM_BK}, es[2] = {1, 1};
        CUresult r = encode(&maps[1 + i], CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t*>(qweight[i]), dims, strides, box, es,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(FQ_ERR_CUDA, "%s: tensor map for qweight[%d]: driver error %d", fn, i, (int)r);
    }
    for (int i = n_proj; i < GM_MAX_PROJ; ++i) { maps[1 + i] = maps[1]; p.proj[i] = GemmProj{nullptr, nullptr, nullptr, nullptr, 0, 1 << 30}; }
    // one persistent CTA per SM (the shared memory of a CTA leaves room for no second one)
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    // 256-row tiles once they fill at least one wave of the SMs, 128-row tiles (twice as many CTAs) below that
    const int mt = ((int64_t)((M + 255) / 256) * tile0 >= (int64_t)sms) ? 2 : 1;
    const int m_tiles = (M + GM_BM * mt - 1) / (GM_BM * mt);
    FQ_CHECK_ARG((int64_t)m_tiles * tile0 <= 0x7fffffffLL, FQ_ERR_ARG, "%s: M=%d too large for one launch", fn, M);
    p.n_tiles = tile0; p.m_tiles = m_tiles;
    const int total = m_tiles * tile0;
    dim3 grid((unsigned)(total < sms ? total : sms));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define FQ_GM(IL, MTV)                                                                                                       \
    do {                                                                                                                     \
        cudaError_t e = cudaFuncSetAttribute(awq_gemm_kernel<IL, MTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, GmCfg<MTV>::SMEM); \
        if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: cannot reserve %d B of shared memory: %s", fn, GmCfg<MTV>::SMEM, cudaGetErrorString(e)); \
        awq_gemm_kernel<IL, MTV><<<grid, GM_THREADS, GmCfg<MTV>::SMEM, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], p);  \
    } while (0)
    if (interleaved) { if (mt == 2) FQ_GM(true, 2); else FQ_GM(true, 1); }
    else { if (mt == 2) FQ_GM(false, 2); else FQ_GM(false, 1); }
#undef FQ_GM
    FQ_CHECK_LAUNCH(fn);
    return FQ_OK;
}
