// Host-side chaining of one decode step of one layer on a persistent TurboQuant (K3-V3) cache:
// pack-on-append (K planes, V planes, raw page metadata + staging), page scores from the raw
// metadata, top-k + compact index, rotation of Q, sparse attention over the selected planes in
// the rotated basis, rotation of O back, tail attention over the staged tokens and the LSE merge.
// No device code of its own: it exists so that a caller pays one foreign call per layer.
#include "fq_common.cuh"

extern "C" size_t fq_decode_layer_turbo_scratch_bytes(int B, int Hq, int D) {
    if (B <= 0 || Hq <= 0 || D <= 0) return 0;
    const size_t rows = (size_t)B * Hq;
    return ((rows * D * 2 * 4 + 255) & ~(size_t)255) + rows * 2 * 4;     // Q_rot, O_rot, two O parts (16-bit) | two lse parts
}

extern "C" int fq_decode_layer_turbo(
    const fq_turbo_cache* c, int layer, int seen,
    const void* K_new, const void* V_new, int64_t nw_sb, int64_t nw_sh, int64_t nw_ss, int n_new,
    const void* Q, int q_dtype, int64_t q_sb, int64_t q_sh,
    const fq_decode_params* prm,
    float* scores, int32_t* compact, void* scratch, size_t scratch_bytes, void* O, float* lse,
    void* workspace, size_t workspace_bytes, void* stream) {
    using namespace fq;
    const char* fn = "fq_decode_layer_turbo";
    FQ_CHECK_ARG(c && prm, FQ_ERR_ARG, "%s: null descriptor", fn);
    FQ_CHECK_ARG(layer >= 0 && layer < c->L, FQ_ERR_ARG, "%s: layer_idx %d out of range [0, %d)", fn, layer, c->L);
    FQ_CHECK_ARG(seen >= 0 && n_new >= 0 && seen + n_new <= c->max_seq_len, FQ_ERR_ARG,
                 "%s: seen+new=%d exceeds max_seq_len=%d", fn, seen + n_new, c->max_seq_len);
    FQ_CHECK_ARG(c->kv_dtype == FQ_F16 || c->kv_dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: cache dtype code %d", fn, c->kv_dtype);
    FQ_CHECK_ARG(q_dtype == FQ_F16 || q_dtype == FQ_BF16, FQ_ERR_DTYPE, "%s: Q must be fp16 or bf16 (code %d)", fn, q_dtype);
    const int page = c->page, D = c->D, B = c->B, Hkv = c->Hkv, Hq = prm->Hq;
    FQ_CHECK_ARG(Q && O && scratch && scratch_bytes >= fq_decode_layer_turbo_scratch_bytes(B, Hq, D), FQ_ERR_WORKSPACE,
                 "%s: scratch of %zu B needed, %zu given", fn, fq_decode_layer_turbo_scratch_bytes(B, Hq, D), scratch_bytes);
    FQ_CHECK_ARG(q_sh == D && q_sb == (int64_t)Hq * D, FQ_ERR_ARG, "%s: Q must be dense (B,H_q,D)", fn);
    const size_t esz = 2;
    const int partial_len = seen % page;
    const int n_quant = ((partial_len + n_new) / page) * page;
    const int tok_start = seen - partial_len;
    const int pg_start = tok_start / page;
    uint8_t* Kms = c->K_msb + layer * c->ms_sl; uint8_t* Kls = c->K_lsb + layer * c->ls_sl;
    uint8_t* Vms = c->V_msb + layer * c->ms_sl; uint8_t* Vls = c->V_lsb + layer * c->ls_sl;
    uint16_t* Kst = static_cast<uint16_t*>(c->K_scale_turbo) + layer * c->st_sl;
    uint16_t* Vst = static_cast<uint16_t*>(c->V_scale_turbo) + layer * c->st_sl;
    uint16_t* Ksr = static_cast<uint16_t*>(c->K_scale_raw) + layer * c->km_sl;
    uint16_t* Kmr = static_cast<uint16_t*>(c->K_mn_raw) + layer * c->km_sl;
    char* Kt = static_cast<char*>(c->K_partial) + layer * c->pt_sl * esz;
    char* Vt = static_cast<char*>(c->V_partial) + layer * c->pt_sl * esz;
    int rc;
    if (n_new > 0) {
        if (n_quant > 0) {
            rc = fq_quantize_turbo(Kt, c->pt_sb, c->pt_sh, c->pt_ss, partial_len, K_new, nw_sb, nw_sh, nw_ss, n_new, c->kv_dtype, B, Hkv, D, n_quant,
                                   Kms + (int64_t)tok_start * c->ms_ss, c->ms_sb, c->ms_sh, c->ms_ss,
                                   Kls + (int64_t)tok_start * c->ls_ss, c->ls_sb, c->ls_sh, c->ls_ss,
                                   Kst + tok_start, c->st_sb, c->st_sh, 1, stream);
            if (rc != FQ_OK) return rc;
            rc = fq_quantize_turbo(Vt, c->pt_sb, c->pt_sh, c->pt_ss, partial_len, V_new, nw_sb, nw_sh, nw_ss, n_new, c->kv_dtype, B, Hkv, D, n_quant,
                                   Vms + (int64_t)tok_start * c->ms_ss, c->ms_sb, c->ms_sh, c->ms_ss,
                                   Vls + (int64_t)tok_start * c->ls_ss, c->ls_sb, c->ls_sh, c->ls_ss,
                                   Vst + tok_start, c->st_sb, c->st_sh, 1, stream);
            if (rc != FQ_OK) return rc;
        }
        // raw per-page K metadata (for scoring) + staging of the left-over tokens, after the launches
        // above have read the staged head
        rc = fq_quantize_kv_int4(Kt, Vt, c->pt_sb, c->pt_sh, c->pt_ss, partial_len, K_new, V_new, nw_sb, nw_sh, nw_ss, n_new,
                                 c->kv_dtype, B, Hkv, D, page, n_quant, nullptr, nullptr, 0, 0, 0,
                                 Ksr + (int64_t)pg_start * c->km_sp, Kmr + (int64_t)pg_start * c->km_sp, c->km_sb, c->km_sh, c->km_sp,
                                 nullptr, nullptr, 0, 0, 0, Kt, Vt, c->pt_sb, c->pt_sh, c->pt_ss, stream);
        if (rc != FQ_OK) return rc;
    }
    const int now = seen + n_new;
    const int tail = now % page;
    const int completed = now - tail;
    const int P = completed / page;
    const int64_t rows = (int64_t)B * Hq;
    char* sb = static_cast<char*>(scratch);
    void* Q_rot = sb;
    void* O_rot = sb + rows * D * 2;
    char* O_parts = sb + rows * D * 4;
    float* lse_parts = reinterpret_cast<float*>(sb + ((rows * D * 8 + 255) & ~(int64_t)255));
    const bool sparse = P > 0, both = sparse && tail > 0;
    if (sparse) {
        rc = fq_page_scores_int4(Q, q_dtype, q_sb, q_sh, Ksr, Kmr, c->km_sb, c->km_sh, c->km_sp, B, Hq, Hkv, P, D, scores, (int64_t)Hq * P, P, stream);
        if (rc != FQ_OK) return rc;
        const int k_max = prm->k_max_static < P ? prm->k_max_static : P;
        rc = fq_select_pages(scores, (int64_t)Hq * P, P, B, Hq, P, prm->retention_per_head, prm->retention, k_max, prm->sinks, prm->window,
                             nullptr, 0, 0, compact, (int64_t)Hq * prm->bucket, prm->bucket, prm->bucket, nullptr, stream);
        if (rc != FQ_OK) return rc;
        if ((rc = fq_wht(Q, Q_rot, q_dtype, rows, D, stream)) != FQ_OK) return rc;
        int n_split = prm->n_split > 0 ? prm->n_split : fq_sparse_decode_default_splits(B, Hq, prm->bucket, page);
        if (n_split > 64) n_split = 64;
        rc = fq_sparse_decode_turbo(Q_rot, q_dtype, (int64_t)Hq * D, D,
                                    Kms, c->ms_sb, c->ms_sh, c->ms_ss, Kls, c->ls_sb, c->ls_sh, c->ls_ss, Kst, c->st_sb, c->st_sh,
                                    Vms, c->ms_sb, c->ms_sh, c->ms_ss, Vls, c->ls_sb, c->ls_sh, c->ls_ss, Vst, c->st_sb, c->st_sh,
                                    compact, (int64_t)Hq * prm->bucket, prm->bucket, prm->bucket,
                                    B, Hq, Hkv, completed, P, D, page, prm->sm_scale,
                                    O_rot, (int64_t)Hq * D, D, both ? lse_parts : lse, workspace, workspace_bytes, n_split, stream);
        if (rc != FQ_OK) return rc;
        if ((rc = fq_wht(O_rot, both ? static_cast<void*>(O_parts) : O, q_dtype, rows, D, stream)) != FQ_OK) return rc;
    }
    if (tail > 0 || !sparse) {
        // dense attention over the staged tokens: the tail-only case of the INT4 kernel (no pages)
        rc = fq_sparse_decode_int4(Q, q_dtype, q_sb, q_sh, nullptr, 0, 0, nullptr, nullptr, 0, 0, 0, nullptr, 0, 0, nullptr, nullptr, 0, 0,
                                   nullptr, 0, 0, 0, tail ? Kt : nullptr, tail ? Vt : nullptr, c->kv_dtype, c->pt_sb, c->pt_sh, c->pt_ss, tail,
                                   B, Hq, Hkv, 0, 0, D, page < 16 ? 16 : page, prm->sm_scale,
                                   both ? static_cast<void*>(O_parts + rows * D * 2) : O, (int64_t)Hq * D, D, both ? lse_parts + rows : lse,
                                   nullptr, 0, 1, stream);
        if (rc != FQ_OK) return rc;
    }
    if (both) return fq_lse_merge(O_parts, lse_parts, q_dtype, 2, rows, D, O, lse, stream);
    return FQ_OK;
}
