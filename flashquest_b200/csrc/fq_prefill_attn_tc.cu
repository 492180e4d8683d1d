// Dense causal attention of the prefill branch on the 5th-generation tensor cores (tcgen05), head_dim 128.
// Same contract as prefill_attn_kernel (fq_prefill_attn.cu): queries of the new tokens over the dequantised
// completed pages followed by the staged tail, grouped-query heads, causal mask aligned at the top left
// (query i sees keys 0..i), fp16 or bf16 operands, fp32 accumulation and softmax.
//
// One CTA = 128 queries of one query head, walking key tiles of 128:
//   warp 0      : two threads issue the TMA loads (4-D tensor maps over Q, K, V; 128-byte swizzle): Q once, then one
//                 thread the K tiles and one the V tiles, each into its own two-deep ring (a K stage is free again as
//                 soon as S has been computed, long before the V stage of the same tile);
//   warp 1      : one thread issues tcgen05.mma: S = Q K^T (M 128, N 128, K 16 x 8) into one of two S buffers in
//                 tensor memory, and O += P V into the one O accumulator in tensor memory, with P read from tensor
//                 memory as the A operand and V from shared memory as the MN-major B operand; S runs up to two key
//                 tiles ahead of P V;
//   warps 2..9  : softmax — two threads per query row (TMEM lane = row; warps 2..5 own the key columns 0..63, warps
//                 6..9 the columns 64..127): read S once (tcgen05.ld), scale, mask (diagonal tile only), agree on the
//                 row maximum through shared memory (one named barrier per pair of warps), write P as fp16/bf16, two
//                 values per 32-bit column, over the S columns they have just read (tcgen05.st).  The exponentials
//                 are taken against a reference maximum that follows the running maximum only when it has moved by
//                 more than 2^8; only then do the threads rescale their half row of O in tensor memory, so O is read
//                 back once, at the end, where it is normalised and stored.
// Every mbarrier wait is bounded and reports through the device status word.
#include <cuda.h>

#include "fq_common.cuh"

namespace fq {

constexpr int PT_BM = 128, PT_BN = 128, PT_D = 128;
constexpr int PT_SOFTMAX_WARPS = 8;      // two threads per query row: each owns 64 of the 128 columns
constexpr int PT_THREADS = (2 + PT_SOFTMAX_WARPS) * 32;
constexpr int PT_TILE_BYTES = 128 * PT_D * 2;                 // 32 KiB: two halves of [128 rows][64 elements]
constexpr int PT_HALF_BYTES = PT_TILE_BYTES / 2;
constexpr int PT_KV_STAGES = 2;
constexpr int PT_SMEM = PT_TILE_BYTES * (1 + 2 * PT_KV_STAGES) + 1024 + 256;   // Q, K ring, V ring, alignment slack, barriers
constexpr unsigned PT_SPIN_LIMIT = 1u << 26;
constexpr int PT_TMEM_COLS = 512;                              // S0 / P0 @0, S1 / P1 @128, O @256 (allocation sizes are powers of two)

struct PrefillTcParams {
    void* O; int64_t o_sb, o_sh, o_ss;
    int B, Hq, Hkv, Sq, Skv, bf16;
    float scale_log2;
    int* status;
};

__device__ __forceinline__ uint32_t pt_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pt_mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pt_smem(bar)), "r"(count));
}
__device__ __forceinline__ void pt_mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pt_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pt_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pt_smem(bar)) : "memory");
}
__device__ __forceinline__ bool pt_mbar_try(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(pt_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool pt_wait(uint64_t* bar, unsigned parity) {
    unsigned spins = 0;
    while (!pt_mbar_try(bar, parity)) {
        if (++spins > PT_SPIN_LIMIT) return false;
    }
    return true;
}
__device__ __forceinline__ void pt_tma_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(pt_smem(dst)), "l"(map), "r"(pt_smem(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void pt_mma(uint32_t tmem_c, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_c), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the A operand read from tensor memory (row m of A in lane m, two 16-bit elements per 32-bit column)
__device__ __forceinline__ void pt_mma_ta(uint32_t tmem_c, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_c), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void pt_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pt_smem(bar)) : "memory");
}
// shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100); offsets in bytes
__device__ __forceinline__ uint64_t pt_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((smem_addr >> 4) & 0x3fff) | ((uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void pt_tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void pt_tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
          "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
          "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float pt_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pt_pack(float lo, float hi, int bf16) {
    if (bf16) { __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&v); }
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(PT_THREADS, 1) prefill_attn_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
    const PrefillTcParams p) {
    extern __shared__ unsigned char pt_raw_smem[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(pt_raw_smem) + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = base;                                         // [2 halves][128 rows][128 B]
    unsigned char* sK = base + PT_TILE_BYTES;                         // [stages] same layout
    unsigned char* sV = sK + PT_KV_STAGES * PT_TILE_BYTES;            // [stages][2 halves of d][128 keys][128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + PT_KV_STAGES * PT_TILE_BYTES);
    uint64_t* q_full = bars;                 // Q landed
    uint64_t* k_full = bars + 1;             // [stages] K tile landed
    uint64_t* k_empty = bars + 3;            // [stages] S = Q K^T of the tile has completed
    uint64_t* v_full = bars + 5;             // [stages] V tile landed
    uint64_t* v_empty = bars + 7;            // [stages] O_tile = P V of the tile has completed
    uint64_t* s_ready = bars + 9;            // [2] S buffer written by the tensor core
    uint64_t* p_ready = bars + 11;           // [2] P buffer written (and the S buffer read) by the softmax threads
    uint64_t* pv_done = bars + 13;           // [2] O += P V of a tile has completed: its P buffer is free, O is up to date
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
    volatile int* s_fail = reinterpret_cast<volatile int*>(tmem_slot + 1);      // a wait gave up somewhere: nobody waits any more
    // exchange between the two threads of a row, private to each pair of warps that shares 32 rows (256 B per pair):
    // the tile maxima as bf16 [tile parity][column half][lane], at the end the denominators as fp32 [column half][lane]
    __shared__ __align__(16) unsigned char s_xch[4 * 256];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // the heaviest query tiles (most keys under the causal mask) are scheduled first
    const int qt = gridDim.x - 1 - blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (p.Hq / p.Hkv);
    const int q0 = qt * PT_BM;
    const int kv_tiles_all = (p.Skv + PT_BN - 1) / PT_BN;
    const int n_tiles = min(kv_tiles_all, qt + 1);                    // keys 0 .. q0 + 127

    if (tid == 0) {
        pt_mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            pt_mbar_init(&k_full[s], 1); pt_mbar_init(&k_empty[s], 1); pt_mbar_init(&v_full[s], 1); pt_mbar_init(&v_empty[s], 1);
            pt_mbar_init(&s_ready[s], 1); pt_mbar_init(&pv_done[s], 1);
            pt_mbar_init(&p_ready[s], PT_SOFTMAX_WARPS * 32);
        }
        *s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pt_smem(tmem_slot)), "r"(PT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    if (warp == 0) {
        // =========================== TMA producer ===========================
        if (lane == 0 && n_tiles > 0) {           // Q, then the K tiles
            pt_mbar_expect_tx(q_full, PT_TILE_BYTES);
            pt_tma_4d(sQ, &map_q, 0, q0, hq, b, q_full);
            pt_tma_4d(sQ + PT_HALF_BYTES, &map_q, 64, q0, hq, b, q_full);
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                if (j >= 2 && !pt_wait(&k_empty[s], (unsigned)((j >> 1) - 1) & 1u)) { failed = true; break; }
                pt_mbar_expect_tx(&k_full[s], PT_TILE_BYTES);
                pt_tma_4d(sK + s * PT_TILE_BYTES, &map_k, 0, j * PT_BN, hkv, b, &k_full[s]);
                pt_tma_4d(sK + s * PT_TILE_BYTES + PT_HALF_BYTES, &map_k, 64, j * PT_BN, hkv, b, &k_full[s]);
            }
        } else if (lane == 1 && n_tiles > 0) {    // the V tiles
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                if (j >= 2 && !pt_wait(&v_empty[s], (unsigned)((j >> 1) - 1) & 1u)) { failed = true; break; }
                pt_mbar_expect_tx(&v_full[s], PT_TILE_BYTES);
                pt_tma_4d(sV + s * PT_TILE_BYTES, &map_v, 0, j * PT_BN, hkv, b, &v_full[s]);
                pt_tma_4d(sV + s * PT_TILE_BYTES + PT_HALF_BYTES, &map_v, 64, j * PT_BN, hkv, b, &v_full[s]);
            }
        }
    } else if (warp == 1) {
        // =========================== MMA issuer ===========================
        if (lane == 0 && n_tiles > 0) {
            const uint32_t fmt = p.bf16 ? 1u : 0u;
            // fp32 accumulate; A K-major; B K-major (S = Q K^T) or MN-major (O = P V); N = 128, M = 128
            const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | (0u << 15) | (0u << 16) | ((uint32_t)(PT_BN >> 3) << 17) |
                                     ((uint32_t)(PT_BM >> 4) << 24);
            const uint32_t idesc_o = idesc_s | (1u << 16);
            const uint32_t q_addr = pt_smem(sQ);
            auto issue_s = [&](int j) -> bool {           // S[j & 1] = Q K_j^T; the buffer was read by the softmax of tile j-2
                const int s = j & 1;
                if (!pt_wait(&k_full[s], (unsigned)(j >> 1) & 1u)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t k_addr = pt_smem(sK + s * PT_TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < PT_D / 16; ++kk) {
                    // K-major, 128-byte swizzle: 8 rows x 64 elements = one 1 KiB atom; 16 k = 32 B inside the row; second half 16 KiB on
                    const uint32_t off = (uint32_t)(kk >> 2) * PT_HALF_BYTES + (uint32_t)(kk & 3) * 32;
                    pt_mma(tmem_base + (uint32_t)(s * PT_BN), pt_desc(q_addr + off, 16, 1024), pt_desc(k_addr + off, 16, 1024), idesc_s, kk != 0 ? 1u : 0u);
                }
                pt_commit(&s_ready[s]);
                pt_commit(&k_empty[s]);
                return true;
            };
            if (!pt_wait(q_full, 0u) || !issue_s(0)) failed = true;
            if (!failed && n_tiles > 1 && !issue_s(1)) failed = true;
            for (int j = 0; j < n_tiles && !failed; ++j) {
                const int s = j & 1;
                const unsigned ph = (unsigned)(j >> 1) & 1u;
                // p_ready also says that the softmax threads have rescaled O where a row's maximum moved
                if (!pt_wait(&p_ready[s], ph) || !pt_wait(&v_full[s], ph)) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t v_addr = pt_smem(sV + s * PT_TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < PT_BN / 16; ++kk) {
                    // A = P of tile j in tensor memory, written over the S buffer it came from: keys 0..63 in columns 0..31
                    // of the buffer, keys 64..127 in columns 64..95 (each half under the S columns its writer owns);
                    // B = V, MN-major: 64 channels x 8 keys = one atom, 16 keys = 2 KiB, channel halves 16 KiB apart
                    const uint32_t p_taddr = tmem_base + (uint32_t)(s * PT_BN + (kk >> 2) * 64 + (kk & 3) * 8);
                    pt_mma_ta(tmem_base + (uint32_t)(2 * PT_BN), p_taddr,
                              pt_desc(v_addr + (uint32_t)kk * 2048, PT_HALF_BYTES, 1024), idesc_o, (kk != 0 || j != 0) ? 1u : 0u);
                }
                pt_commit(&pv_done[s]);
                pt_commit(&v_empty[s]);
                // S two tiles ahead: its buffer has just been released by p_ready of tile j
                if (j + 2 < n_tiles && !issue_s(j + 2)) { failed = true; break; }
            }
        }
    } else {
        // =========================== softmax and output ===========================
        const int lq = warp & 3;                  // the TMEM lane quarter this warp may read
        const int hf = (warp - 2) >> 2;           // column half owned by this thread
        const int r = lq * 32 + lane;             // query row inside the tile
        const int qi = q0 + r;                    // global query index
        const uint32_t lane_addr = tmem_base + ((uint32_t)(lq * 32) << 16);
        // m_used is the maximum the row's probabilities and O are currently expressed against; it follows the true
        // running maximum only when that has moved by more than 8 (in base 2), so P stays below 2^8 and O in tensor
        // memory is rescaled rarely (the first few tiles of a row) instead of being read back after every tile
        float m_used = -INFINITY, l_run = 0.f;
        constexpr float PT_LAZY = 8.0f;
        // a wait that gives up is remembered by everybody: the loop then runs on without waiting, so that the
        // named barriers below still see both warps of every pair
        auto wait_ok = [&](uint64_t* bar, unsigned parity) {
            if (*s_fail) return;
            if (!pt_wait(bar, parity)) { failed = true; *s_fail = 1; }
        };
        const uint32_t o_addr = lane_addr + (uint32_t)(2 * PT_BN + hf * 64);      // this thread's half row of O
        __nv_bfloat16* xch_m = reinterpret_cast<__nv_bfloat16*>(s_xch + lq * 256);
        float* xch_l = reinterpret_cast<float*>(s_xch + lq * 256);
        const int pair_bar = 1 + lq;              // named barrier of the two warps that share these 32 rows
        for (int j = 0; j < n_tiles; ++j) {
            const int sb = j & 1;
            wait_ok(&s_ready[sb], (unsigned)(j >> 1) & 1u);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t s_addr = lane_addr + (uint32_t)(sb * PT_BN + hf * 64);
            const int k0 = j * PT_BN + hf * 64;           // first key of this thread's columns
            const int k_lim = min(qi, p.Skv - 1);         // last key this row may see
            const bool full = k0 + 63 <= min(q0, p.Skv - 1);     // no column of this half is masked for any row of the tile
            uint32_t v0[32], v1[32];
            pt_tmem_ld32(s_addr, v0);
            pt_tmem_ld32(s_addr + 32, v1);
            float m_tile = -INFINITY;
            if (full) {
#pragma unroll
                for (int i = 0; i < 32; ++i) m_tile = fmaxf(m_tile, fmaxf(__uint_as_float(v0[i]), __uint_as_float(v1[i])));
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (k0 + i > k_lim) v0[i] = 0xff800000u;          // -inf: masked
                    if (k0 + 32 + i > k_lim) v1[i] = 0xff800000u;
                    m_tile = fmaxf(m_tile, fmaxf(__uint_as_float(v0[i]), __uint_as_float(v1[i])));
                }
            }
            // The row's maximum over both halves, to bf16 precision (it only serves as the reference point of the
            // exponentials, and both threads must arrive at the same value).  One named barrier per pair of warps; the
            // slot alternates with the tile parity, so the write of tile j+2 cannot overtake the partner's read of tile j
            // (the partner reads before it arrives at the barrier of tile j+1).
            {
                const __nv_bfloat16 mine = __float2bfloat16_rn(m_tile);
                xch_m[(sb * 2 + hf) * 32 + lane] = mine;
                asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
                m_tile = fmaxf(__bfloat162float(mine), __bfloat162float(xch_m[(sb * 2 + (hf ^ 1)) * 32 + lane]));
            }
            // both threads of a row see the same m_tile and m_used, so they take the same decision
            const float m_true = m_tile * p.scale_log2;
            float alpha = 1.f;
            if (m_true > m_used + PT_LAZY || m_used == -INFINITY) {
                const float m_new = fmaxf(m_used, m_true);
                alpha = (m_used == -INFINITY) ? (m_new == -INFINITY ? 1.f : 0.f) : pt_ex2(m_used - m_new);
                m_used = m_new;
            }
            // rescale this thread's half row of O where the reference maximum moved (warp-collective tensor-memory
            // access: the whole warp goes when one lane must); O is complete only once P V of tile j-1 is
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                wait_ok(&pv_done[(j - 1) & 1], (unsigned)((j - 1) >> 1) & 1u);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t o[32];
                    pt_tmem_ld32(o_addr + (uint32_t)(c * 32), o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    pt_tmem_st32(o_addr + (uint32_t)(c * 32), o);
                }
            }
            const float m_sub = m_used == -INFINITY ? 0.f : m_used;
            // probabilities, two per 32-bit column, over the first half of this thread's own S columns (the S values
            // are in registers by now; the next S into this buffer is issued behind the P V that reads these)
            float l_tile = 0.f;
            uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const uint32_t (&v)[32] = c == 0 ? v0 : v1;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    // ex2(-inf) = 0 for masked columns
                    const float p0 = pt_ex2(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_sub));
                    const float p1 = pt_ex2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m_sub));
                    l_tile += p0 + p1;
                    pk[c * 16 + i / 2] = pt_pack(p0, p1, p.bf16);
                }
            }
            pt_tmem_st32(s_addr, pk);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            pt_mbar_arrive(&p_ready[sb]);
            l_run = l_run * alpha + l_tile;
        }
        // the row's denominator over both halves (the pair's exchange area again, as fp32)
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        xch_l[hf * 32 + lane] = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        l_run += xch_l[(hf ^ 1) * 32 + lane];
        // O is final once P V of the last tile has completed
        if (n_tiles > 0) wait_ok(&pv_done[(n_tiles - 1) & 1], (unsigned)((n_tiles - 1) >> 1) & 1u);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        {
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            const bool store = *s_fail == 0 && qi < p.Sq && n_tiles > 0;
            unsigned char* orow = static_cast<unsigned char*>(p.O) + ((int64_t)b * p.o_sb + (int64_t)hq * p.o_sh + (int64_t)qi * p.o_ss) * 2 + hf * 128;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t o[32];
                pt_tmem_ld32(o_addr + (uint32_t)(c * 32), o);       // warp-collective: every lane loads, the rows in range store
                if (store) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        *reinterpret_cast<uint4*>(orow + (c * 32 + i) * 2) =
                            make_uint4(pt_pack(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv, p.bf16),
                                       pt_pack(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv, p.bf16),
                                       pt_pack(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv, p.bf16),
                                       pt_pack(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv, p.bf16));
                    }
                }
            }
        }
    }
    if (failed) atomicExch(p.status, FQ_ERR_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(PT_TMEM_COLS) : "memory");
    }
}

typedef CUresult (*PtEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PtEncodeTiledFn pt_encode_fn() {
    static std::atomic<void*> cached{nullptr};
    void* fn = cached.load(std::memory_order_relaxed);
    if (fn == nullptr) {
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess) return nullptr;
        cached.store(fn, std::memory_order_relaxed);
    }
    return reinterpret_cast<PtEncodeTiledFn>(fn);
}

// (B, H, S, 128) tensor with element strides sb, sh, ss -> 4-D map {128, S, H, B}, boxes of 64 elements x 128 rows
static bool pt_make_map(PtEncodeTiledFn enc, CUtensorMap* map, const void* ptr, int bf16, int S, int H, int B, int64_t sb, int64_t sh, int64_t ss) {
    const cuuint64_t dims[4] = {(cuuint64_t)PT_D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
    const cuuint32_t box[4] = {64, 128, 1, 1}, es[4] = {1, 1, 1, 1};
    return enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, es,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// true when the launch was made; false: the shape is not served here (the caller falls back to the mma.sync kernel)
bool prefill_attention_tc_launch(const void* Q, int64_t q_sb, int64_t q_sh, int64_t q_ss, const void* K, int64_t k_sb, int64_t k_sh, int64_t k_ss,
                                 const void* V, int64_t v_sb, int64_t v_sh, int64_t v_ss, int bf16, int B, int Hq, int Hkv, int Sq, int Skv,
                                 float sm_scale, void* O, int64_t o_sb, int64_t o_sh, int64_t o_ss, cudaStream_t st, int* rc) {
    *rc = FQ_OK;
    // strides of a tensor map are 40-bit multiples of 16 bytes; a size-1 axis may carry any stride, so give it a valid one
    auto ok_stride = [](int64_t s) { return s > 0 && (s * 2) % 16 == 0 && s * 2 < (1ll << 40); };
    if (Sq < 1 || Skv < 1 || !aligned(O, 4) || o_ss % 2 != 0 || o_sh % 2 != 0 || o_sb % 2 != 0) return false;
    if (B == 1) { q_sb = (int64_t)Hq * q_sh; k_sb = (int64_t)Hkv * k_sh; v_sb = k_sb; }
    if (!ok_stride(q_ss) || !ok_stride(q_sh) || !ok_stride(q_sb) || !ok_stride(k_ss) || !ok_stride(k_sh) || !ok_stride(k_sb) ||
        !ok_stride(v_ss) || !ok_stride(v_sh) || !ok_stride(v_sb)) return false;
    PtEncodeTiledFn enc = pt_encode_fn();
    if (!enc) return false;
    CUtensorMap mq, mk, mv;
    if (!pt_make_map(enc, &mq, Q, bf16, Sq, Hq, B, q_sb, q_sh, q_ss) || !pt_make_map(enc, &mk, K, bf16, Skv, Hkv, B, k_sb, k_sh, k_ss) ||
        !pt_make_map(enc, &mv, V, bf16, Skv, Hkv, B, v_sb, v_sh, v_ss)) return false;
    PrefillTcParams p;
    p.O = O; p.o_sb = o_sb; p.o_sh = o_sh; p.o_ss = o_ss;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Skv = Skv; p.bf16 = bf16;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    p.status = device_status_ptr();
    if (p.status == nullptr) { *rc = FQ_ERR_CUDA; return true; }
    cudaError_t e = cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PT_SMEM);
    if (e != cudaSuccess) { *rc = fail(FQ_ERR_CUDA, "fq_prefill_attention: cannot reserve %d B of shared memory: %s", PT_SMEM, cudaGetErrorString(e)); return true; }
    dim3 grid((unsigned)((Sq + PT_BM - 1) / PT_BM), (unsigned)Hq, (unsigned)B);
    prefill_attn_tc_kernel<<<grid, PT_THREADS, PT_SMEM, st>>>(mq, mk, mv, p);
    return true;
}

}  // namespace fq
