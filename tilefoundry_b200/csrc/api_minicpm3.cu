// C ABI: MLA attention and the MiniCPM3-architecture decode step.  See include/tfb200.h.
#include "api_internal.h"
#include "kernels.h"

#include <cstring>

using namespace tfb::host;

extern "C" {

int tfb_attn_mla_decode(const tfb_attn_mla_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->q_up && a->kv_up && a->k_rope && a->cos_table && a->sin_table && a->pos, TFB_EINVAL);
    TFB_REQUIRE(a->k_pool && a->v_pool && a->block_table && a->out, TFB_EINVAL);
    TFB_REQUIRE(a->part_o && a->part_ml && a->counters, TFB_EINVAL);
    TFB_REQUIRE(a->heads > 0 && a->nope == 64 && a->rope == 32 && a->v == 64, TFB_EINVAL);
    TFB_REQUIRE(a->page_size > 0 && a->table_len > 0 && a->max_ctx > 0, TFB_EINVAL);
    TFB_REQUIRE((long long)a->page_size * a->table_len >= a->max_ctx && a->max_pos >= a->max_ctx, TFB_ECAPACITY);
    TFB_REQUIRE(aligned16(a->k_pool) && aligned16(a->v_pool), TFB_EALIGN);
    tfb::MlaParams p = {};
    p.q_up = static_cast<const uint16_t*>(a->q_up);
    p.kv_up = static_cast<const uint16_t*>(a->kv_up);
    p.k_rope = static_cast<const uint16_t*>(a->k_rope);
    p.cos_table = static_cast<const uint16_t*>(a->cos_table);
    p.sin_table = static_cast<const uint16_t*>(a->sin_table);
    p.pos = a->pos;
    p.rope_pos = a->rope_pos;
    p.k_pool = static_cast<uint16_t*>(a->k_pool);
    p.v_pool = static_cast<uint16_t*>(a->v_pool);
    p.block_table = a->block_table;
    p.out = static_cast<uint16_t*>(a->out);
    p.k_new_out = static_cast<uint16_t*>(a->k_new_out);
    p.v_new_out = static_cast<uint16_t*>(a->v_new_out);
    p.part_o = a->part_o;
    p.part_ml = a->part_ml;
    p.counters = a->counters;
    p.heads = a->heads; p.nope = a->nope; p.rope = a->rope; p.vd = a->v;
    p.page_size = a->page_size; p.max_ctx = a->max_ctx; p.nsplit = tfb::mla_splits(a->max_ctx);
    p.scale = a->scale;
    p.trace = next_trace();
    return done(tfb::attn_mla_dispatch(p, S(stream), a->pdl != 0));
}

int32_t tfb_mla_latent_splits(int32_t max_ctx) { return max_ctx > 0 ? tfb::mla_latent_splits(max_ctx) : 0; }

int tfb_mla_latent_decode(const tfb_mla_latent_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->qkv_a && a->gamma_q_a && a->gamma_kv_a && a->w_q_b && a->w_kv_b, TFB_EINVAL);
    TFB_REQUIRE(a->cos_table && a->sin_table && a->pos && a->pool && a->block_table && a->out, TFB_EINVAL);
    TFB_REQUIRE(a->q_lat && a->q_rope && a->part_o && a->part_ml, TFB_EINVAL);
    TFB_REQUIRE(a->tokens >= 0 && a->tokens <= 32 && (a->tokens <= 1 || a->no_early_rows), TFB_EINVAL);
    TFB_REQUIRE(a->page_size > 0 && a->table_len > 0 && a->max_ctx > 0, TFB_EINVAL);
    TFB_REQUIRE(tfb::mla_latent_supported(a->heads, a->q_lora, a->kv_lora, a->nope, a->rope, a->v, a->max_ctx), TFB_EINVAL);
    TFB_REQUIRE((long long)a->page_size * a->table_len >= a->max_ctx && a->max_pos >= a->max_ctx, TFB_ECAPACITY);
    TFB_REQUIRE(aligned16(a->pool) && aligned16(a->w_q_b) && aligned16(a->w_kv_b) && aligned16(a->qkv_a), TFB_EALIGN);
    tfb::MlaLatentParams p = {};
    p.qkv_a = static_cast<const uint16_t*>(a->qkv_a);
    p.gamma_q_a = static_cast<const uint16_t*>(a->gamma_q_a);
    p.gamma_kv_a = static_cast<const uint16_t*>(a->gamma_kv_a);
    p.w_q_b = static_cast<const uint16_t*>(a->w_q_b);
    p.w_kv_b = static_cast<const uint16_t*>(a->w_kv_b);
    p.cos_table = static_cast<const uint16_t*>(a->cos_table);
    p.sin_table = static_cast<const uint16_t*>(a->sin_table);
    p.pos = a->pos; p.rope_pos = a->rope_pos;
    p.pool = static_cast<uint16_t*>(a->pool);
    p.block_table = a->block_table;
    p.q_lat = a->q_lat; p.q_rope = a->q_rope; p.part_o = a->part_o; p.part_ml = a->part_ml;
    p.out = static_cast<uint16_t*>(a->out);
    p.latent_new_out = static_cast<uint16_t*>(a->latent_new_out);
    p.heads = a->heads; p.q_lora = a->q_lora; p.page_size = a->page_size; p.max_ctx = a->max_ctx;
    p.nsplit = tfb::mla_latent_splits(a->max_ctx);
    p.scale = a->scale; p.lora_eps = a->lora_eps; p.no_early_rows = a->no_early_rows != 0;
    p.tokens = a->tokens > 1 ? a->tokens : 1;
    p.qkv_stride = a->q_lora + a->kv_lora + a->rope;
    for (int i = 0; i < 3; ++i) p.trace3[i] = next_trace();
    return done(tfb::mla_latent_dispatch(p, S(stream), a->pdl != 0));
}

int tfb_minicpm3_prefill_chunk(const tfb_minicpm3_prefill_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->layers && a->n_layers > 0 && a->m >= 2 && a->m <= 32, TFB_EINVAL);
    TFB_REQUIRE(a->w_embed && a->ids && a->pos_rows && a->block_table && a->cos_table && a->sin_table, TFB_EINVAL);
    TFB_REQUIRE(a->hidden_buf && a->norm_buf && a->qkv_a_buf && a->attn_buf && a->act_buf, TFB_EINVAL);
    TFB_REQUIRE(a->q_lat_buf && a->q_rope_buf && a->part_o && a->part_ml && a->status, TFB_EINVAL);
    TFB_REQUIRE(a->hidden % 64 == 0 && a->inter % 64 == 0 && (a->heads * a->v) % 64 == 0, TFB_EINVAL);
    TFB_REQUIRE(tfb::mla_latent_supported(a->heads, a->q_lora, a->kv_lora, a->nope, a->rope, a->v, a->max_ctx), TFB_EINVAL);
    const bool pdl = a->pdl != 0;
    const int M = a->m, H = a->hidden, I = a->inter, NH = a->heads;
    const int NA = a->q_lora + a->kv_lora + a->rope, NO = NH * a->v;
    cudaStream_t st = S(stream);
    uint16_t* hid = static_cast<uint16_t*>(a->hidden_buf);
    uint16_t* nrm = static_cast<uint16_t*>(a->norm_buf);
    uint16_t* qkv_a = static_cast<uint16_t*>(a->qkv_a_buf);
    uint16_t* attn = static_cast<uint16_t*>(a->attn_buf);

    auto project = [&](const void* w, const void* x, const void* residual, void* y, int n, int k, bool swiglu) -> int {
        tfb_gemm_small_m_args g;
        std::memset(&g, 0, sizeof g);
        g.w = w; g.x = x; g.residual = residual; g.y = y; g.status = a->status;
        g.m = M; g.n = n; g.k = k; g.pdl = pdl; g.swiglu = swiglu; g.res_scale = a->residual_scale;
        return tfb_gemm_small_m(&g, stream);
    };
    auto norm = [&](const void* gamma) -> int {
        return done(tfb::rmsnorm_launch(hid, static_cast<const uint16_t*>(gamma), nrm, M, H, a->eps,
                                        TFB_NORM_CAST_THEN_GAIN, st, pdl));
    };
    // first launch without a programmatic dependency, as in the decode steps
    cudaError_t e = tfb::embed_launch(static_cast<const uint16_t*>(a->w_embed), reinterpret_cast<const long long*>(a->ids),
                                      nullptr, nullptr, hid, M, H, a->vocab, a->embed_scale, st, false);
    if (e != cudaSuccess) return fail_launch(e);
    for (int l = 0; l < a->n_layers; ++l) {
        const tfb_minicpm3_layer& L = a->layers[l];
        TFB_REQUIRE(static_cast<const uint16_t*>(L.w_up) == static_cast<const uint16_t*>(L.w_gate) + size_t(I) * H, TFB_EINVAL);
        int rc = norm(L.gamma_in);
        if (rc) return rc;
        if ((rc = project(L.w_qkv_a, nrm, nullptr, qkv_a, NA, H, false))) return rc;
        {                                                    // every token appends its latent row, then token t attends to rows <= its own
            tfb_mla_latent_args m;
            std::memset(&m, 0, sizeof m);
            m.qkv_a = qkv_a; m.gamma_q_a = L.gamma_q_a; m.gamma_kv_a = L.gamma_kv_a;
            m.w_q_b = L.w_q_b; m.w_kv_b = L.w_kv_b; m.cos_table = a->cos_table; m.sin_table = a->sin_table;
            m.pos = a->pos_rows; m.pool = L.k_pool; m.block_table = a->block_table; m.out = attn;
            m.q_lat = a->q_lat_buf; m.q_rope = a->q_rope_buf; m.part_o = a->part_o; m.part_ml = a->part_ml;
            m.heads = NH; m.q_lora = a->q_lora; m.kv_lora = a->kv_lora; m.nope = a->nope; m.rope = a->rope; m.v = a->v;
            m.page_size = a->page_size; m.table_len = a->table_len; m.max_ctx = a->max_ctx; m.max_pos = a->max_pos;
            m.scale = a->scale; m.lora_eps = a->lora_eps; m.pdl = pdl; m.no_early_rows = 1; m.tokens = M;
            if ((rc = tfb_mla_latent_decode(&m, stream))) return rc;
        }
        if ((rc = project(L.w_o, attn, hid, hid, H, NO, false))) return rc;
        if ((rc = norm(L.gamma_post))) return rc;
        if ((rc = project(L.w_gate, nrm, nullptr, a->act_buf, I, H, true))) return rc;
        if ((rc = project(L.w_down, a->act_buf, hid, hid, H, I, false))) return rc;
    }
    return TFB_OK;
}

int tfb_minicpm3_decode_step(const tfb_minicpm3_step_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->layers && a->n_layers > 0, TFB_EINVAL);
    TFB_REQUIRE(a->w_embed && a->gamma_final && a->w_head && a->tokens && a->pos, TFB_EINVAL);
    TFB_REQUIRE(a->hidden_buf && a->qkv_a_buf && a->attn_buf && a->act_buf, TFB_EINVAL);
    TFB_REQUIRE(a->cache_layout == TFB_MLA_CACHE_LATENT || (a->q_up_buf && a->kv_up_buf), TFB_EINVAL);
    TFB_REQUIRE(a->part_o && a->part_ml && a->counters && a->head_val && a->head_idx, TFB_EINVAL);
    TFB_REQUIRE(a->hidden % 256 == 0 && a->inter % 256 == 0 && a->q_lora % 256 == 0 && a->kv_lora % 256 == 0, TFB_EINVAL);
    TFB_REQUIRE((a->heads * a->v) % 256 == 0, TFB_EINVAL);
    TFB_REQUIRE(a->max_tokens <= a->max_ctx + 1, TFB_ECAPACITY);
    TFB_REQUIRE(a->cache_layout == TFB_MLA_CACHE_ASSEMBLED || a->cache_layout == TFB_MLA_CACHE_LATENT, TFB_EINVAL);
    const bool latent = a->cache_layout == TFB_MLA_CACHE_LATENT;
    TFB_REQUIRE(!latent || (a->q_lat_buf && a->q_rope_buf), TFB_EINVAL);
    const bool pdl = a->pdl != 0;
    const int H = a->hidden, I = a->inter, NH = a->heads;
    const int NA = a->q_lora + a->kv_lora + a->rope, NQ = NH * (a->nope + a->rope), NKV = NH * (a->nope + a->v);
    const int NO = NH * a->v;
    cudaStream_t st = S(stream);
    uint16_t* hid = static_cast<uint16_t*>(a->hidden_buf);
    uint16_t* qkv_a = static_cast<uint16_t*>(a->qkv_a_buf);
    uint16_t* trace = static_cast<uint16_t*>(a->hidden_trace);

    // The step's first launch carries no programmatic dependency: it starts only when the previous step has
    // fully finished, so kernels of this step may read last step's state and position before their own wait.
    cudaError_t e = tfb::embed_launch(static_cast<const uint16_t*>(a->w_embed), nullptr,
                                      reinterpret_cast<const long long*>(a->tokens), a->pos, hid, 1, H,
                                      a->vocab, a->embed_scale, st, false);
    if (e != cudaSuccess) return fail_launch(e);

    auto gemv = [&](const void* w, const void* w2, const void* x, const void* gamma, const void* res, void* y,
                    int n, int k, int pro, int epi, float eps, float res_scale) {
        tfb_gemv_args g;
        std::memset(&g, 0, sizeof g);
        g.w = w; g.w2 = w2; g.x = x; g.gamma = gamma; g.residual = res; g.y = y; g.n = n; g.k = k;
        g.prologue = pro; g.epilogue = epi; g.eps = eps; g.x_scale = 1.f; g.res_scale = res_scale; g.out_scale = 1.f;
        g.pdl = pdl;
        return gemv_checked(&g, stream);
    };

    for (int l = 0; l < a->n_layers; ++l) {
        const tfb_minicpm3_layer& L = a->layers[l];
        int rc;
        // 1. input norm + q down-projection | kv compression (one fused projection)
        if ((rc = gemv(L.w_qkv_a, nullptr, hid, L.gamma_in, nullptr, qkv_a, NA, H, TFB_NORM_CAST_THEN_GAIN,
                       TFB_EPI_STORE, a->eps, 1.f))) return rc;
        if (latent) {
            // 2-4. absorbed form: q_b + W_UK^T q / RoPE + latent append, attention over the latents, merge + W_UV
            tfb_mla_latent_args t;
            std::memset(&t, 0, sizeof t);
            t.qkv_a = qkv_a; t.gamma_q_a = L.gamma_q_a; t.gamma_kv_a = L.gamma_kv_a; t.w_q_b = L.w_q_b; t.w_kv_b = L.w_kv_b;
            t.cos_table = a->cos_table; t.sin_table = a->sin_table; t.pos = a->pos; t.pool = L.k_pool;
            t.block_table = a->block_table; t.out = a->attn_buf; t.q_lat = a->q_lat_buf; t.q_rope = a->q_rope_buf;
            t.part_o = a->part_o; t.part_ml = a->part_ml;
            t.heads = NH; t.q_lora = a->q_lora; t.kv_lora = a->kv_lora; t.nope = a->nope; t.rope = a->rope; t.v = a->v;
            t.page_size = a->page_size; t.table_len = a->table_len; t.max_ctx = a->max_ctx; t.max_pos = a->max_pos;
            t.scale = a->scale; t.lora_eps = a->lora_eps; t.pdl = pdl;
            if ((rc = tfb_mla_latent_decode(&t, stream))) return rc;
        } else {
        // 2 + 3. low-rank norms + q up-projection and kv up-projection (k_nope | v per head): independent of each
        // other, one launch
        {
            tfb_gemv_args gq, gkv;
            std::memset(&gq, 0, sizeof gq);
            gq.w = L.w_q_b; gq.x = qkv_a; gq.gamma = L.gamma_q_a; gq.y = a->q_up_buf; gq.n = NQ; gq.k = a->q_lora;
            gq.prologue = TFB_NORM_CAST_THEN_GAIN; gq.epilogue = TFB_EPI_STORE; gq.eps = a->lora_eps;
            gq.x_scale = 1.f; gq.res_scale = 1.f; gq.out_scale = 1.f; gq.pdl = pdl;
            gkv = gq;
            gkv.w = L.w_kv_b; gkv.x = qkv_a + a->q_lora; gkv.gamma = L.gamma_kv_a; gkv.y = a->kv_up_buf; gkv.n = NKV;
            gkv.k = a->kv_lora;
            if ((rc = tfb_gemv_pair(&gq, &gkv, stream))) return rc;
        }
        // 4. RoPE, assembly, cache append, attention
        tfb_attn_mla_args t;
        std::memset(&t, 0, sizeof t);
        t.q_up = a->q_up_buf; t.kv_up = a->kv_up_buf; t.k_rope = qkv_a + a->q_lora + a->kv_lora;
        t.cos_table = a->cos_table; t.sin_table = a->sin_table; t.pos = a->pos;
        t.k_pool = L.k_pool; t.v_pool = L.v_pool; t.block_table = a->block_table; t.out = a->attn_buf;
        t.part_o = a->part_o; t.part_ml = a->part_ml; t.counters = a->counters;
        t.heads = NH; t.nope = a->nope; t.rope = a->rope; t.v = a->v;
        t.page_size = a->page_size; t.table_len = a->table_len; t.max_ctx = a->max_ctx; t.max_pos = a->max_pos;
        t.scale = a->scale; t.pdl = pdl;
        if ((rc = tfb_attn_mla_decode(&t, stream))) return rc;
        }
        // 5. output projection + scaled residual
        if ((rc = gemv(L.w_o, nullptr, a->attn_buf, nullptr, hid, hid, H, NO, TFB_NORM_NONE, TFB_EPI_RESIDUAL,
                       a->eps, a->residual_scale))) return rc;
        // 6. post-attention norm + gate/up + SwiGLU
        if ((rc = gemv(L.w_gate, L.w_up, hid, L.gamma_post, nullptr, a->act_buf, I, H, TFB_NORM_CAST_THEN_GAIN,
                       TFB_EPI_SWIGLU, a->eps, 1.f))) return rc;
        // 7. down projection + scaled residual
        if ((rc = gemv(L.w_down, nullptr, a->act_buf, nullptr, hid, hid, H, I, TFB_NORM_NONE, TFB_EPI_RESIDUAL,
                       a->eps, a->residual_scale))) return rc;
        if (trace) {
            e = tfb::copy_launch(hid, trace + size_t(l) * H, H * 2, st, pdl);
            if (e != cudaSuccess) return fail_launch(e);
        }
    }
    if (trace) {
        e = tfb::rmsnorm_launch(hid, static_cast<const uint16_t*>(a->gamma_final),
                                trace + size_t(a->n_layers) * H, 1, H, a->eps, TFB_NORM_CAST_THEN_GAIN, st, pdl);
        if (e != cudaSuccess) return fail_launch(e);
    }
    tfb_lm_head_args h;
    std::memset(&h, 0, sizeof h);
    h.w = a->w_head; h.x = hid; h.gamma = a->gamma_final; h.logits = a->logits;
    h.scratch_val = a->head_val; h.scratch_idx = a->head_idx; h.counter = a->counters + NH;
    h.n = int(a->vocab); h.k = H; h.prologue = TFB_NORM_CAST_THEN_GAIN; h.eps = a->eps;
    h.x_scale = -a->logits_div; h.out_scale = 1.f; h.pdl = pdl;
    h.token_out = a->picked;
    h.tokens = a->tokens; h.pos = a->pos; h.n_prompt = a->n_prompt; h.max_tokens = a->max_tokens;
    h.temperature = a->temperature; h.seed = a->seed;
    h.eos_ids = a->eos_ids; h.n_eos = a->n_eos; h.stop_at = a->stop_at;
    return tfb_lm_head_argmax(&h, stream);
}

}  // extern "C"
