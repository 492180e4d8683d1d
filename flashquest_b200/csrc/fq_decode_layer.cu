// Host-side chaining of the four kernels of one decode step of one layer on a persistent
// INT4 cache: pack-on-append, page scores, top-k + compact index, sparse attention with the
// staged tail.  No device code of its own; it exists so that a caller pays one foreign call
// per layer instead of four plus the slicing arithmetic.
#include "fq_common.cuh"

extern "C" int fq_decode_layer_int4(
    const fq_int4_cache* c, int layer, int seen,
    const void* K_new, const void* V_new, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const fq_decode_params* prm,
    float* scores, int32_t* compact, void* O, float* lse,
    void* workspace, size_t workspace_bytes, void* stream) {
    using namespace fq;
    const char* fn = "fq_decode_layer_int4";
    FQ_CHECK_ARG(c && prm, FQ_ERR_ARG, "%s: null descriptor", fn);
    FQ_CHECK_ARG(layer >= 0 && layer < c->L, FQ_ERR_ARG, "%s: layer_idx %d out of range [0, %d)", fn, layer, c->L);
    FQ_CHECK_ARG(seen >= 0 && n_new >= 0 && seen + n_new <= c->max_seq_len, FQ_ERR_ARG,
                 "%s: seen+new=%d exceeds max_seq_len=%d", fn, seen + n_new, c->max_seq_len);
    FQ_CHECK_ARG(c->kv_dtype == FQ_F16 || c->kv_dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: cache dtype code %d", fn, c->kv_dtype);
    const int page = c->page, D = c->D, B = c->B, Hkv = c->Hkv, Hq = prm->Hq;
    const size_t esz = 2;
    const int partial_len = seen % page;
    const int total = partial_len + n_new;
    const int n_quant = (total / page) * page;
    const int tok_start = seen - partial_len;
    const int pg_start = tok_start / page;

    uint8_t* Kp = c->K_packed + layer * c->pk_sl;
    uint8_t* Vp = c->V_packed + layer * c->pk_sl;
    uint16_t* Ks = static_cast<uint16_t*>(c->K_scale) + layer * c->km_sl;
    uint16_t* Km = static_cast<uint16_t*>(c->K_mn) + layer * c->km_sl;
    uint16_t* Vs = static_cast<uint16_t*>(c->V_scale) + layer * c->vm_sl;
    uint16_t* Vm = static_cast<uint16_t*>(c->V_mn) + layer * c->vm_sl;
    char* Kt = static_cast<char*>(c->K_partial) + layer * c->pt_sl * esz;
    char* Vt = static_cast<char*>(c->V_partial) + layer * c->pt_sl * esz;

    int rc;
    if (n_new > 0) {
        rc = fq_quantize_kv_int4(
            Kt, Vt, c->pt_sb, c->pt_sh, c->pt_ss, partial_len,
            K_new, V_new, nw_sb, nw_sh, nw_ss, n_new,
            c->kv_dtype, B, Hkv, D, page, n_quant,
            Kp + (int64_t)tok_start * c->pk_ss, Vp + (int64_t)tok_start * c->pk_ss, c->pk_sb, c->pk_sh, c->pk_ss,
            Ks + (int64_t)pg_start * c->km_sp, Km + (int64_t)pg_start * c->km_sp, c->km_sb, c->km_sh, c->km_sp,
            Vs + tok_start, Vm + tok_start, c->vm_sb, c->vm_sh, 1,
            Kt, Vt, c->pt_sb, c->pt_sh, c->pt_ss, stream);
        if (rc != FQ_OK) return rc;
    }
    const int now = seen + n_new;
    const int tail = now % page;
    const int completed = now - tail;
    const int P = completed / page;
    if (P > 0) {
        rc = fq_page_scores_int4(Q, q_dtype, q_sb, q_sh, Ks, Km, c->km_sb, c->km_sh, c->km_sp,
                                 B, Hq, Hkv, P, D, scores, (int64_t)Hq * P, P, stream);
        if (rc != FQ_OK) return rc;
        const int k_max = prm->k_max_static < P ? prm->k_max_static : P;
        rc = fq_select_pages(scores, (int64_t)Hq * P, P, B, Hq, P, prm->retention_per_head, prm->retention,
                             k_max, prm->sinks, prm->window, nullptr, 0, 0,
                             compact, (int64_t)Hq * prm->bucket, prm->bucket, prm->bucket, nullptr, stream);
        if (rc != FQ_OK) return rc;
    }
    int n_split = prm->n_split > 0 ? prm->n_split : fq_sparse_decode_default_splits(B, Hq, prm->bucket, page);
    return fq_sparse_decode_int4(
        Q, q_dtype, q_sb, q_sh, Kp, c->pk_sb, c->pk_sh, Ks, Km, c->km_sb, c->km_sh, c->km_sp,
        Vp, c->pk_sb, c->pk_sh, Vs, Vm, c->vm_sb, c->vm_sh,
        compact, (int64_t)Hq * prm->bucket, prm->bucket, P > 0 ? prm->bucket : 0,
        tail ? Kt : nullptr, tail ? Vt : nullptr, c->kv_dtype, c->pt_sb, c->pt_sh, c->pt_ss, tail,
        B, Hq, Hkv, completed, P, D, page, prm->sm_scale,
        O, (int64_t)Hq * D, D, lse, workspace, workspace_bytes, n_split, stream);
}

extern "C" int fq_decode_step_int4(
    const fq_int4_cache* c, int n_layers, const int* seen,
    const void* K_new, const void* V_new, int64_t nw_sl, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    const void* Q, int q_dtype, int64_t q_sl, int64_t q_sb, int64_t q_sh,
    const fq_decode_params* prm, size_t prm_stride,
    float* scores, int64_t sc_sl, int32_t* compact, int64_t cp_sl, void* O, int64_t o_sl, float* lse, int64_t lse_sl,
    void* workspace, size_t ws_sl, size_t workspace_bytes, void* stream) {
    using namespace fq;
    const char* fn = "fq_decode_step_int4";
    FQ_CHECK_ARG(c && prm && seen, FQ_ERR_ARG, "%s: null descriptor", fn);
    FQ_CHECK_ARG(n_layers >= 0 && n_layers <= c->L, FQ_ERR_ARG, "%s: %d layers, the cache has %d", fn, n_layers, c->L);
    FQ_CHECK_ARG(n_layers <= 1 || ws_sl >= workspace_bytes, FQ_ERR_WORKSPACE,
                 "%s: the per-layer workspaces overlap (stride %zu B < %zu B)", fn, ws_sl, workspace_bytes);
    const size_t kv_esz = 2, q_esz = q_dtype == FQ_F32 ? 4 : 2;
    for (int l = 0; l < n_layers; ++l) {
        const fq_decode_params* pl = reinterpret_cast<const fq_decode_params*>(reinterpret_cast<const char*>(prm) + (size_t)l * prm_stride);
        const int rc = fq_decode_layer_int4(
            c, l, seen[l],
            K_new ? static_cast<const char*>(K_new) + (size_t)l * nw_sl * kv_esz : nullptr,
            V_new ? static_cast<const char*>(V_new) + (size_t)l * nw_sl * kv_esz : nullptr, nw_sb, nw_sh, nw_ss, n_new,
            static_cast<const char*>(Q) + (size_t)l * q_sl * q_esz, q_dtype, q_sb, q_sh, pl,
            scores + l * sc_sl, compact + l * cp_sl, static_cast<char*>(O) + (size_t)l * o_sl * q_esz,
            lse ? lse + l * lse_sl : nullptr,
            workspace ? static_cast<char*>(workspace) + (size_t)l * ws_sl : nullptr, workspace_bytes, stream);
        if (rc != FQ_OK) return rc;
    }
    return FQ_OK;
}

namespace fq {
__global__ void advance_pos_kernel(int* pos, int n, int n_new, int max_tokens) {
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && pos[i] + n_new <= max_tokens) pos[i] += n_new;
}

int advance_positions(int* pos, int n, int n_new, int max_tokens, void* stream) {
    launch_k(PDL_QUANT, advance_pos_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, static_cast<cudaStream_t>(stream),
             pos, n, n_new, max_tokens);
    FQ_CHECK_LAUNCH("advance_positions");
    return FQ_OK;
}

int decode_layer_int4_dyn(const fq_int4_cache* c, int l, const int* pos, const void* Kn, const void* Vn,
                          int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new, const void* Ql, int q_dtype, int64_t q_sb, int64_t q_sh,
                          const fq_decode_params* pl, float* sc, int32_t* cp, void* O, float* lse,
                          void* workspace, size_t workspace_bytes, void* stream, bool append) {
    const int page = c->page, D = c->D, B = c->B, Hkv = c->Hkv, Hq = pl->Hq;
    const int P_max = c->max_seq_len / page;
    const size_t kv_esz = 2;
    const DynPos dp{pos, n_new, page, c->max_seq_len};
    uint8_t* Kp = c->K_packed + l * c->pk_sl;
    uint8_t* Vp = c->V_packed + l * c->pk_sl;
    uint16_t* Ks = static_cast<uint16_t*>(c->K_scale) + l * c->km_sl;
    uint16_t* Km = static_cast<uint16_t*>(c->K_mn) + l * c->km_sl;
    uint16_t* Vs = static_cast<uint16_t*>(c->V_scale) + l * c->vm_sl;
    uint16_t* Vm = static_cast<uint16_t*>(c->V_mn) + l * c->vm_sl;
    char* Kt = static_cast<char*>(c->K_partial) + l * c->pt_sl * kv_esz;
    char* Vt = static_cast<char*>(c->V_partial) + l * c->pt_sl * kv_esz;
    // host-side sizes are the maxima (they size grids and pass validation); the kernels read *pos
    DynPos dp_early = dp;          // scores, selection and attention come at least two launches after any writer of *pos
    dp_early.early = true;
    int rc = FQ_OK;
    if (append)
        rc = quantize_kv_int4_launch(Kt, Vt, c->pt_sb, c->pt_sh, c->pt_ss, page - n_new, Kn, Vn, nw_sb, nw_sh, nw_ss, n_new,
                                     c->kv_dtype, B, Hkv, D, page, page,
                                     Kp, Vp, c->pk_sb, c->pk_sh, c->pk_ss, Ks, Km, c->km_sb, c->km_sh, c->km_sp,
                                     Vs, Vm, c->vm_sb, c->vm_sh, 1, Kt, Vt, c->pt_sb, c->pt_sh, c->pt_ss, stream, dp);
    if (rc != FQ_OK) return rc;
    rc = page_scores_int4_launch(Ql, q_dtype, q_sb, q_sh, Ks, Km, c->km_sb, c->km_sh, c->km_sp, B, Hq, Hkv, P_max, D,
                                 sc, (int64_t)Hq * P_max, P_max, stream, dp_early);
    if (rc != FQ_OK) return rc;
    rc = select_pages_launch(sc, (int64_t)Hq * P_max, P_max, B, Hq, P_max, pl->retention_per_head, pl->retention,
                             pl->k_max_static < P_max ? pl->k_max_static : P_max, pl->sinks, pl->window, nullptr, 0, 0,
                             cp, (int64_t)Hq * pl->bucket, pl->bucket, pl->bucket, nullptr, stream, dp_early);
    if (rc != FQ_OK) return rc;
    const int n_split = pl->n_split > 0 ? pl->n_split : fq_sparse_decode_default_splits(B, Hq, pl->bucket, page);
    return sparse_decode_int4_launch(
        Ql, q_dtype, q_sb, q_sh, Kp, c->pk_sb, c->pk_sh, Ks, Km, c->km_sb, c->km_sh, c->km_sp,
        Vp, c->pk_sb, c->pk_sh, Vs, Vm, c->vm_sb, c->vm_sh,
        cp, (int64_t)Hq * pl->bucket, pl->bucket, pl->bucket,
        Kt, Vt, c->kv_dtype, c->pt_sb, c->pt_sh, c->pt_ss, page - 1,
        B, Hq, Hkv, P_max * page, P_max, D, page, pl->sm_scale,
        O, (int64_t)Hq * D, D, lse, workspace, workspace_bytes, n_split, stream, dp_early);
}
}  // namespace fq

extern "C" int fq_decode_step_int4_dev(
    const fq_int4_cache* c, int n_layers, int* pos,
    const void* K_new, const void* V_new, int64_t nw_sl, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    const void* Q, int q_dtype, int64_t q_sl, int64_t q_sb, int64_t q_sh,
    const fq_decode_params* prm, size_t prm_stride,
    float* scores, int64_t sc_sl, int32_t* compact, int64_t cp_sl, void* O, int64_t o_sl, float* lse, int64_t lse_sl,
    void* workspace, size_t ws_sl, size_t workspace_bytes, void* stream) {
    using namespace fq;
    const char* fn = "fq_decode_step_int4_dev";
    FQ_CHECK_ARG(c && prm && pos && K_new && V_new && Q && scores && compact && O, FQ_ERR_ARG, "%s: null argument", fn);
    FQ_CHECK_ARG(n_layers >= 0 && n_layers <= c->L, FQ_ERR_ARG, "%s: %d layers, the cache has %d", fn, n_layers, c->L);
    FQ_CHECK_ARG(n_new >= 1 && n_new < c->page, FQ_ERR_ARG, "%s: n_new=%d must be in [1, page)", fn, n_new);
    FQ_CHECK_ARG(n_layers <= 1 || ws_sl >= workspace_bytes, FQ_ERR_WORKSPACE,
                 "%s: the per-layer workspaces overlap (stride %zu B < %zu B)", fn, ws_sl, workspace_bytes);
    FQ_CHECK_ARG(c->kv_dtype == FQ_F16 || c->kv_dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: cache dtype code %d", fn, c->kv_dtype);
    FQ_CHECK_ARG(c->max_seq_len / c->page >= 1, FQ_ERR_ARG, "%s: the cache holds less than one page", fn);
    const size_t kv_esz = 2, q_esz = q_dtype == FQ_F32 ? 4 : 2;
    // every layer's new tokens are known up front: one launch appends to all layers
    {
        const int rc = quant_append_layers_dyn(c, n_layers, pos, K_new, V_new, nw_sl, nw_sb, nw_sh, nw_ss, n_new, stream);
        if (rc != FQ_OK) return rc;
    }
    for (int l = 0; l < n_layers; ++l) {
        const fq_decode_params* pl = reinterpret_cast<const fq_decode_params*>(reinterpret_cast<const char*>(prm) + (size_t)l * prm_stride);
        const int rc = decode_layer_int4_dyn(
            c, l, pos + l, static_cast<const char*>(K_new) + (size_t)l * nw_sl * kv_esz,
            static_cast<const char*>(V_new) + (size_t)l * nw_sl * kv_esz, nw_sb, nw_sh, nw_ss, n_new,
            static_cast<const char*>(Q) + (size_t)l * q_sl * q_esz, q_dtype, q_sb, q_sh, pl,
            scores + l * sc_sl, compact + l * cp_sl, static_cast<char*>(O) + (size_t)l * o_sl * q_esz,
            lse ? lse + l * lse_sl : nullptr,
            workspace ? static_cast<char*>(workspace) + (size_t)l * ws_sl : nullptr, workspace_bytes, stream, false);
        if (rc != FQ_OK) return rc;
    }
    return advance_positions(pos, n_layers, n_new, c->max_seq_len, stream);
}
