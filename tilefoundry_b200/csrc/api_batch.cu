// C ABI: the Qwen3-architecture decode step for several sequences at once.  See include/tfb200.h.
#include "api_internal.h"
#include "kernels.h"

#include <cstring>

using namespace tfb::host;

extern "C" {

int tfb_qwen3_batch_decode_step(const tfb_qwen3_batch_step_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->layers && a->n_layers > 0 && a->batch >= 1 && a->batch <= 32, TFB_EINVAL);
    TFB_REQUIRE(a->w_embed && a->gamma_final && a->w_head && a->tokens && a->pos && a->block_table, TFB_EINVAL);
    TFB_REQUIRE(a->hidden_buf && a->norm_buf && a->qkv_buf && a->attn_buf && a->act_buf && a->logits, TFB_EINVAL);
    TFB_REQUIRE(a->part_o && a->part_ml && a->counters && a->status, TFB_EINVAL);
    TFB_REQUIRE(a->pick_val && a->pick_idx, TFB_EINVAL);
    TFB_REQUIRE(a->hidden % 64 == 0 && a->inter % 64 == 0 && (a->hq * a->d) % 64 == 0 && a->hidden % 8 == 0, TFB_EINVAL);
    TFB_REQUIRE((long long)a->page_size * a->table_len >= a->max_ctx, TFB_ECAPACITY);
    TFB_REQUIRE(a->max_pos >= a->max_ctx && a->max_tokens <= a->max_ctx + 1, TFB_ECAPACITY);
    const bool pdl = a->pdl != 0;
    const int B = a->batch, H = a->hidden, QP = a->hq * a->d, KVP = a->hkv * a->d, I = a->inter;
    const int NQKV = QP + 2 * KVP;
    cudaStream_t st = S(stream);
    uint16_t* hid = static_cast<uint16_t*>(a->hidden_buf);
    uint16_t* nrm = static_cast<uint16_t*>(a->norm_buf);
    uint16_t* trace = static_cast<uint16_t*>(a->hidden_trace);

    auto project = [&](const void* w, const void* x, const void* residual, void* y, int n, int k, bool swiglu) -> int {
        tfb_gemm_small_m_args g;
        std::memset(&g, 0, sizeof g);
        g.w = w; g.x = x; g.residual = residual; g.y = y;
        g.status = a->status;
        g.m = B; g.n = n; g.k = k; g.pdl = pdl; g.swiglu = swiglu;
        return tfb_gemm_small_m(&g, stream);
    };
    auto norm = [&](const void* gamma) -> int {
        const cudaError_t e = tfb::rmsnorm_launch(hid, static_cast<const uint16_t*>(gamma), nrm, B, H, a->eps,
                                                  TFB_NORM_CAST_THEN_GAIN, st, pdl);
        return e == cudaSuccess ? TFB_OK : fail_launch(e);
    };

    // The step's first launch carries no programmatic dependency: it starts only when the previous step has
    // fully finished, so kernels of this step may read last step's positions before their own wait.
    cudaError_t e = tfb::embed_rows_launch(static_cast<const uint16_t*>(a->w_embed),
                                           reinterpret_cast<const long long*>(a->tokens), a->pos, a->max_tokens, hid, B, H,
                                           a->vocab, st, false);
    if (e != cudaSuccess) return fail_launch(e);

    for (int l = 0; l < a->n_layers; ++l) {
        const tfb_qwen3_batch_layer& L = a->layers[l];
        int rc = norm(L.gamma_in);
        if (rc) return rc;
        rc = project(L.w_qkv, nrm, nullptr, a->qkv_buf, NQKV, H, false);
        if (rc) return rc;
        tfb_attn_gqa_args t;
        std::memset(&t, 0, sizeof t);
        t.qkv = a->qkv_buf; t.gamma_q = L.gamma_q; t.gamma_k = L.gamma_k;
        t.cos_table = a->cos_table; t.sin_table = a->sin_table; t.pos = a->pos;
        t.k_pool = L.k_pool; t.v_pool = L.v_pool; t.block_table = a->block_table; t.out = a->attn_buf;
        t.part_o = a->part_o; t.part_ml = a->part_ml; t.counters = a->counters;
        t.hq = a->hq; t.hkv = a->hkv; t.d = a->d; t.rotary_dim = a->d;
        t.page_size = a->page_size; t.table_len = a->table_len; t.max_ctx = a->max_ctx; t.max_pos = a->max_pos;
        t.eps = a->eps; t.scale = a->scale; t.norm_mode = TFB_NORM_CAST_THEN_GAIN; t.pdl = pdl; t.batch = B;
        rc = tfb_attn_gqa_decode(&t, stream);
        if (rc) return rc;
        rc = project(L.w_o, a->attn_buf, hid, hid, H, QP, false);
        if (rc) return rc;
        rc = norm(L.gamma_post);
        if (rc) return rc;
        rc = project(L.w_gate_up, nrm, nullptr, a->act_buf, I, H, true);
        if (rc) return rc;
        rc = project(L.w_down, a->act_buf, hid, hid, H, I, false);
        if (rc) return rc;
        if (trace) {
            e = tfb::copy_launch(hid, trace + size_t(l) * B * H, B * H * 2, st, pdl);
            if (e != cudaSuccess) return fail_launch(e);
        }
    }
    int rc = norm(a->gamma_final);
    if (rc) return rc;
    if (trace) {
        e = tfb::copy_launch(nrm, trace + size_t(a->n_layers) * B * H, B * H * 2, st, pdl);
        if (e != cudaSuccess) return fail_launch(e);
    }
    rc = project(a->w_head, nrm, nullptr, a->logits, int(a->vocab), H, false);
    if (rc) return rc;
    e = tfb::pick_rows_launch(static_cast<const uint16_t*>(a->logits), B, int(a->vocab),
                              reinterpret_cast<long long*>(a->tokens), a->pos, a->n_prompt, a->max_tokens,
                              reinterpret_cast<long long*>(a->picked), a->pick_val, a->pick_idx,
                              a->counters + size_t(B) * a->hkv, a->temperature > 0.f ? a->temperature : 0.f, a->seed, st, pdl);
    return e == cudaSuccess ? TFB_OK : fail_launch(e);
}

int tfb_qwen3_prefill_chunk(const tfb_qwen3_prefill_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->layers && a->n_layers > 0 && a->m >= 2 && a->m <= 32, TFB_EINVAL);
    TFB_REQUIRE(a->w_embed && a->ids && a->pos_rows && a->block_table && a->cos_table && a->sin_table, TFB_EINVAL);
    TFB_REQUIRE(a->hidden_buf && a->norm_buf && a->qkv_buf && a->attn_buf && a->act_buf, TFB_EINVAL);
    TFB_REQUIRE(a->part_o && a->part_ml && a->counters && a->status, TFB_EINVAL);
    TFB_REQUIRE(a->hidden % 64 == 0 && a->inter % 64 == 0 && (a->hq * a->d) % 64 == 0, TFB_EINVAL);
    TFB_REQUIRE((long long)a->page_size * a->table_len >= a->max_ctx && a->max_pos >= a->max_ctx, TFB_ECAPACITY);
    const bool pdl = a->pdl != 0;
    const int M = a->m, H = a->hidden, QP = a->hq * a->d, KVP = a->hkv * a->d, I = a->inter;
    const int NQKV = QP + 2 * KVP;
    cudaStream_t st = S(stream);
    uint16_t* hid = static_cast<uint16_t*>(a->hidden_buf);
    uint16_t* nrm = static_cast<uint16_t*>(a->norm_buf);

    auto project = [&](const void* w, const void* x, const void* residual, void* y, int n, int k, bool swiglu) -> int {
        tfb_gemm_small_m_args g;
        std::memset(&g, 0, sizeof g);
        g.w = w; g.x = x; g.residual = residual; g.y = y; g.status = a->status;
        g.m = M; g.n = n; g.k = k; g.pdl = pdl; g.swiglu = swiglu;
        return tfb_gemm_small_m(&g, stream);
    };
    auto norm = [&](const void* gamma) -> int {
        return done(tfb::rmsnorm_launch(hid, static_cast<const uint16_t*>(gamma), nrm, M, H, a->eps,
                                        TFB_NORM_CAST_THEN_GAIN, st, pdl));
    };
    // first launch without a programmatic dependency, as in the decode steps
    cudaError_t e = tfb::embed_launch(static_cast<const uint16_t*>(a->w_embed), reinterpret_cast<const long long*>(a->ids),
                                      nullptr, nullptr, hid, M, H, a->vocab, 1.f, st, false);
    if (e != cudaSuccess) return fail_launch(e);
    for (int l = 0; l < a->n_layers; ++l) {
        const tfb_qwen3_batch_layer& L = a->layers[l];
        int rc = norm(L.gamma_in);
        if (rc) return rc;
        rc = project(L.w_qkv, nrm, nullptr, a->qkv_buf, NQKV, H, false);
        if (rc) return rc;
        tfb_attn_gqa_args t;
        std::memset(&t, 0, sizeof t);
        t.qkv = a->qkv_buf; t.gamma_q = L.gamma_q; t.gamma_k = L.gamma_k;
        t.cos_table = a->cos_table; t.sin_table = a->sin_table; t.pos = a->pos_rows;
        t.k_pool = L.k_pool; t.v_pool = L.v_pool; t.block_table = a->block_table; t.out = a->attn_buf;
        t.part_o = a->part_o; t.part_ml = a->part_ml; t.counters = a->counters;
        t.hq = a->hq; t.hkv = a->hkv; t.d = a->d; t.rotary_dim = a->d;
        t.page_size = a->page_size; t.table_len = a->table_len; t.max_ctx = a->max_ctx; t.max_pos = a->max_pos;
        t.eps = a->eps; t.scale = a->scale; t.norm_mode = TFB_NORM_CAST_THEN_GAIN; t.pdl = pdl; t.batch = M;
        t.chunk = 1;                                       // every token's K/V row into the cache ...
        rc = tfb_attn_gqa_decode(&t, stream);
        if (rc) return rc;
        t.chunk = 2;                                       // ... then each token attends to the rows before it
        rc = tfb_attn_gqa_decode(&t, stream);
        if (rc) return rc;
        rc = project(L.w_o, a->attn_buf, hid, hid, H, QP, false);
        if (rc) return rc;
        rc = norm(L.gamma_post);
        if (rc) return rc;
        rc = project(L.w_gate_up, nrm, nullptr, a->act_buf, I, H, true);
        if (rc) return rc;
        rc = project(L.w_down, a->act_buf, hid, hid, H, I, false);
        if (rc) return rc;
    }
    return TFB_OK;
}

}  // extern "C"
