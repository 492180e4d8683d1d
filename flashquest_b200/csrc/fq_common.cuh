// Shared device/host helpers for the flashquest_b200 kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <type_traits>

#include "../../include/flashquest_b200.h"

namespace fq {

// ---- error reporting (thread-local message behind fq_last_error_string) ----
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

#define FQ_CHECK_ARG(cond, code, ...)              \
    do {                                           \
        if (!(cond)) return fq::fail((code), __VA_ARGS__); \
    } while (0)

#define FQ_CHECK_LAUNCH(name)                                                        \
    do {                                                                             \
        cudaError_t e__ = cudaGetLastError();                                        \
        if (e__ != cudaSuccess)                                                      \
            return fq::fail(FQ_ERR_CUDA, "%s: launch failed: %s", (name), cudaGetErrorString(e__)); \
    } while (0)

// ---- programmatic dependent launch ----
// Every kernel of the decode chain is launched with programmatic stream serialisation: its
// CTAs may become resident while the previous kernel of the stream is still draining, run
// their prologue (index arithmetic, barrier set-up, loads of data that is older than the
// previous kernel) and block in pdl_wait() until the previous kernel has completed and its
// writes are visible.  pdl_trigger() comes right after the wait in every kernel, so at most
// two kernels of a chain overlap and whatever a kernel reads before its wait must have been
// written at least two kernels earlier.  All kernels get the attribute but the selection kernel,
// which measured 3 us slower per launch when it was made resident early beside the scoring kernel.
enum { PDL_SCORES = 1, PDL_SELECT = 2, PDL_ATTN = 4, PDL_QUANT = 8, PDL_GEMV = 16 };
constexpr bool pdl_enabled(int kind) { return kind != PDL_SELECT; }

template <typename... KP, typename... A>
inline cudaError_t launch_k(int kind, void (*kernel)(KP...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at{};
    at.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &at; cfg.numAttrs = pdl_enabled(kind) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<A&&>(args)...);
}

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// ---- token position read on the device ----
// The graph-capturable decode step (fq_decode_step_int4_dev) cannot bake the sequence length into
// its launches.  It hands this record to the launch functions below; a kernel that gets a non-null
// `pos` derives page count, tail length and append offsets from *pos (tokens cached before this
// step) instead of from its host-side arguments, which in that mode only size the grid (maximum
// values).  The public entry points pass an empty record.
// `early`: the kernel may read *pos BEFORE its dependency wait, overlapping the load with the wait.  Safe only for a
// kernel at least two launches behind the one that last wrote *pos: a dependent launch starts no earlier than its
// predecessor's own wait has returned, i.e. after the writer has completed.  The decode layer sets it for scores,
// selection and attention, which always follow the append launch; the append itself reads after its wait.
struct DynPos { const int* pos = nullptr; int n_new = 0; int page = 1; int max_tokens = 0; bool early = false; };

// Launch functions behind the public entry points of the same names, with the position record explicit.
int quantize_kv_int4_launch(
    const void* K_head, const void* V_head, int64_t hd_sb, int64_t hd_sh, int64_t hd_ss, int n_head,
    const void* K_new, const void* V_new, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    int dtype, int B, int H, int D, int page, int n_quant,
    uint8_t* K_packed, uint8_t* V_packed, int64_t pk_sb, int64_t pk_sh, int64_t pk_ss,
    void* K_scale, void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    void* V_scale, void* V_mn, int64_t vm_sb, int64_t vm_sh, int64_t vm_ss,
    void* stage_K, void* stage_V, int64_t st_sb, int64_t st_sh, int64_t st_ss, void* stream, const DynPos& dp);
int page_scores_int4_launch(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P, int D, float* scores, int64_t sc_sb, int64_t sc_sh, void* stream, const DynPos& dp,
    float levels = 15.0f);
bool score_select_fusable(int Hq, int Hkv, int P, int D);
int score_select_launch(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    int B, int Hq, int Hkv, int P, int D, float levels, float* scores, int64_t sc_sb, int64_t sc_sh,
    const float* retention_per_head, float retention, int k_max, int sinks, int window,
    int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket, int32_t* count, void* stream, const DynPos& dp, int first_fresh);
int select_pages_launch(
    const float* scores, int64_t sc_sb, int64_t sc_sh, int B, int H, int P,
    const float* retention_per_head, float retention, int k_max, int sinks, int window,
    uint8_t* mask, int64_t mk_sb, int64_t mk_sh, int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    int32_t* count, void* stream, const DynPos& dp);
int sparse_decode_int4_launch(
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const uint8_t* K_packed, int64_t kp_sb, int64_t kp_sh,
    const void* K_scale, const void* K_mn, int64_t km_sb, int64_t km_sh, int64_t km_sp,
    const uint8_t* V_packed, int64_t vp_sb, int64_t vp_sh,
    const void* V_scale, const void* V_mn, int64_t vm_sb, int64_t vm_sh,
    const int32_t* compact, int64_t cp_sb, int64_t cp_sh, int bucket,
    const void* K_tail, const void* V_tail, int tail_dtype, int64_t tl_sb, int64_t tl_sh, int64_t tl_ss, int tail_len,
    int B, int Hq, int Hkv, int S_kv, int P, int D, int page, float sm_scale,
    void* O, int64_t o_sb, int64_t o_sh, float* lse,
    void* workspace, size_t workspace_bytes, int n_split, void* stream, const DynPos& dp, const int32_t* list_count = nullptr);

// One layer of the graph-capturable step (append + score + select + attend with the sequence
// length read from *pos) and the closing increment of the positions; defined in fq_decode_layer.cu.
int decode_layer_int4_dyn(const fq_int4_cache* c, int layer, const int* pos, const void* K_new, const void* V_new,
                          int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new, const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
                          const fq_decode_params* prm, float* scores, int32_t* compact, void* O, float* lse,
                          void* workspace, size_t workspace_bytes, void* stream, bool append = true);
int advance_positions(int* pos, int n, int n_new, int max_tokens, void* stream);
int quant_append_layers_dyn(const fq_int4_cache* c, int n_layers, const int* pos, const void* K_new, const void* V_new,
                            int64_t nw_sl, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new, void* stream);
int rope_launch(void* q, int64_t q_sb, int64_t q_sh, int Hq, void* k, int64_t k_sb, int64_t k_sh, int Hkv, int B, int D, int pos,
                float theta, void* stream, const int* pos_dev, int pos_step);

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Device-side status word of the current device: kernels that wait (mbarrier) record a
// timeout there instead of spinning forever; fq_device_status() reads and clears it.
// Returns nullptr (with the error string set) if the address cannot be resolved.
int* device_status_ptr();

// ---- dtype traits ----
template <typename T> struct Dt;
template <> struct Dt<float> {
    static constexpr int code = FQ_F32;
    __device__ static float to_f32(float v) { return v; }
    __device__ static float rn(float v) { return v; }  // round to T, back to fp32
};
template <> struct Dt<__half> {
    static constexpr int code = FQ_F16;
    __device__ static float to_f32(__half v) { return __half2float(v); }
    __device__ static float rn(float v) { return __half2float(__float2half_rn(v)); }
};
template <> struct Dt<__nv_bfloat16> {
    static constexpr int code = FQ_BF16;
    __device__ static float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static float rn(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

__device__ __forceinline__ float bf16_lo(uint32_t x) { return __uint_as_float(x << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t x) { return __uint_as_float(x & 0xffff0000u); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// 16-byte read-only load of 8 16-bit elements / 4 fp32 elements.
__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// Convert 8 consecutive elements starting at p (16-byte aligned) to fp32.  Plain (coherent)
// loads: the quantiser reads a staging buffer that the same kernel later rewrites.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    v[0] = bf16_lo(u.x); v[1] = bf16_hi(u.x); v[2] = bf16_lo(u.y); v[3] = bf16_hi(u.y);
    v[4] = bf16_lo(u.z); v[5] = bf16_hi(u.z); v[6] = bf16_lo(u.w); v[7] = bf16_hi(u.w);
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

}  // namespace fq
