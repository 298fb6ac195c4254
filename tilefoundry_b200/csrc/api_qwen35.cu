// C ABI of the f32-activation family (Qwen3.5-35B-A3B): argument checks, then the launches.
#include "api_internal.h"
#include "kernels.h"

#include <cstring>

using namespace tfb::host;

extern "C" {

int tfb_gemv_f32(const tfb_gemv_f32_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->w && a->x && a->y, TFB_EINVAL);
    TFB_REQUIRE(a->n > 0 && a->k > 0 && a->k % 256 == 0 && a->k <= 8192, TFB_EINVAL);
    const int nm = a->prologue, ep = a->epilogue;
    TFB_REQUIRE(nm == TFB_NORM_NONE || nm == TFB_NORM_F32GAIN || nm == TFB_NORM_SEGMENT_GATED, TFB_EINVAL);
    TFB_REQUIRE(ep == TFB_EPI_STORE || ep == TFB_EPI_RESIDUAL || ep == TFB_EPI_SWIGLU, TFB_EINVAL);
    TFB_REQUIRE(nm == TFB_NORM_NONE || a->gamma, TFB_EINVAL);
    if (nm == TFB_NORM_SEGMENT_GATED) {
        const int s = a->seg;
        TFB_REQUIRE(a->gate && s >= 16 && s <= 256 && (s & (s - 1)) == 0 && a->k % s == 0, TFB_EINVAL);
    }
    TFB_REQUIRE(ep != TFB_EPI_RESIDUAL || a->residual, TFB_EINVAL);
    TFB_REQUIRE(ep != TFB_EPI_SWIGLU || a->w2, TFB_EINVAL);
    if (a->rows_per_expert > 0) {
        TFB_REQUIRE(a->rows_per_expert % 8 == 0 && a->routed_slots >= 0 &&
                        int64_t(a->routed_slots) * a->rows_per_expert <= a->n, TFB_EINVAL);   // the last extra slot may be partial
        TFB_REQUIRE(a->routed_slots == 0 || a->expert_idx, TFB_EINVAL);
        const bool extra = a->routed_slots * a->rows_per_expert < a->n;
        TFB_REQUIRE(!extra || (a->w_extra && (ep != TFB_EPI_SWIGLU || a->w2_extra)), TFB_EINVAL);
    }
    if (a->route_counter) {
        TFB_REQUIRE(ep == TFB_EPI_STORE && a->rows_per_expert == 0 && a->k <= 2048 && a->idx_out && a->w_out, TFB_EINVAL);
        TFB_REQUIRE(a->route_experts > 0 && a->route_experts <= 256 && a->route_experts <= a->n && a->route_top_k > 0 &&
                        a->route_top_k <= 32 && a->route_top_k <= a->route_experts, TFB_EINVAL);
    }
    TFB_REQUIRE(aligned16(a->w) && aligned16(a->x) && aligned16(a->y) && (!a->w2 || aligned16(a->w2)) &&
                    (!a->gamma || aligned16(a->gamma)) && (!a->gate || aligned16(a->gate)) &&
                    (!a->w_extra || aligned16(a->w_extra)) && (!a->w2_extra || aligned16(a->w2_extra)), TFB_EALIGN);
    tfb::GemvF32Params p = {};
    p.w = static_cast<const uint4*>(a->w); p.w2 = static_cast<const uint4*>(a->w2);
    p.w_extra = static_cast<const uint4*>(a->w_extra); p.w2_extra = static_cast<const uint4*>(a->w2_extra);
    p.x = a->x; p.gamma = a->gamma; p.gate = a->gate; p.residual = a->residual; p.y = a->y;
    p.n = a->n; p.k = a->k; p.seg = a->seg; p.eps = a->eps;
    p.expert_idx = reinterpret_cast<const long long*>(a->expert_idx);
    p.rows_per_expert = a->rows_per_expert; p.routed_slots = a->routed_slots;
    p.expert_rank = a->expert_rank; p.expert_world = a->expert_world;
    TFB_REQUIRE(a->expert_world <= 1 || (a->expert_rank >= 0 && a->expert_rank < a->expert_world), TFB_EINVAL);
    p.route_counter = a->route_counter; p.route_experts = a->route_experts; p.route_top_k = a->route_top_k;
    p.idx_out = reinterpret_cast<long long*>(a->idx_out); p.w_out = a->w_out;
    p.trace = next_trace();
    return done(tfb::gemv_f32_dispatch(p, nm, ep, S(stream), a->pdl != 0));
}

int tfb_gdn_step(const tfb_gdn_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->state && a->read, TFB_EINVAL);
    const bool direct = a->direct_q != nullptr;
    TFB_REQUIRE(!direct || (a->direct_k && a->direct_v && a->direct_g && a->direct_beta), TFB_EINVAL);
    TFB_REQUIRE(direct || (a->proj && a->conv_state && a->conv_w && a->a_log && a->dt_bias), TFB_EINVAL);
    TFB_REQUIRE(a->dk == 128 && a->kernel_width == 4 && a->hk > 0 && a->hv > 0 && a->hv % a->hk == 0 && a->dv > 0 &&
                    a->dv % 32 == 0, TFB_EINVAL);
    const uint64_t channels = 2ull * a->hk * a->dk + uint64_t(a->hv) * a->dv;
    TFB_REQUIRE(direct || a->conv_state_stride >= channels * (a->kernel_width - 1), TFB_EINVAL);
    tfb::GdnParams p = {};
    p.proj = a->proj; p.conv_state = a->conv_state; p.conv_state_stride = a->conv_state_stride; p.pos = a->pos;
    p.conv_w = a->conv_w; p.a_log = a->a_log; p.dt_bias = a->dt_bias; p.state = a->state; p.read = a->read;
    p.hk = a->hk; p.hv = a->hv; p.dk = a->dk; p.dv = a->dv; p.kernel_width = a->kernel_width; p.q_scale = a->q_scale;
    p.direct_q = a->direct_q; p.direct_k = a->direct_k; p.direct_v = a->direct_v; p.direct_g = a->direct_g;
    p.direct_beta = a->direct_beta;
    return done(tfb::gdn_step_launch(p, S(stream), a->pdl != 0));
}

int32_t tfb_attn_gated_splits(int32_t max_ctx) { return tfb::attn_gated_splits(max_ctx); }
int32_t tfb_attn_gated_groups(int32_t hq, int32_t hkv, int32_t d) {
    return (hq > 0 && hkv > 0 && hq % hkv == 0) ? tfb::attn_gated_groups(hq, hkv, d) : 0;
}

int tfb_attn_gated_decode(const tfb_attn_gated_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->proj && a->gamma_q && a->gamma_k && a->cos_table && a->sin_table && a->pos && a->k_pool &&
                    a->v_pool && a->block_table && a->out && a->part_o && a->part_ml && a->counters, TFB_EINVAL);
    TFB_REQUIRE(a->hq > 0 && a->hkv > 0 && a->hq % a->hkv == 0 && a->page_size > 0 && a->page_size % 64 == 0 &&
                    a->max_ctx > 0, TFB_EINVAL);
    TFB_REQUIRE(a->rotary_dim > 0 && a->rotary_dim % 64 == 0 && a->rotary_dim <= a->d, TFB_EINVAL);
    TFB_REQUIRE(int64_t(a->table_len) * a->page_size >= a->max_ctx && a->max_pos >= a->max_ctx, TFB_ECAPACITY);
    const int g = a->hq / a->hkv;
    TFB_REQUIRE((a->d == 256 && (g == 8 || g == 4)) || (a->d == 128 && (g == 2 || g == 4)), TFB_EINVAL);
    tfb::GatedAttnParams p = {};
    p.proj = a->proj; p.gamma_q = a->gamma_q; p.gamma_k = a->gamma_k; p.cos_table = a->cos_table; p.sin_table = a->sin_table;
    p.pos = a->pos; p.rope_pos = a->rope_pos; p.k_pool = a->k_pool; p.v_pool = a->v_pool; p.block_table = a->block_table;
    p.out = a->out; p.k_new_out = a->k_new_out; p.v_new_out = a->v_new_out;
    p.part_o = a->part_o; p.part_ml = a->part_ml; p.counters = a->counters;
    p.hq = a->hq; p.hkv = a->hkv; p.d = a->d; p.rotary_dim = a->rotary_dim; p.page_size = a->page_size;
    p.max_ctx = a->max_ctx; p.nsplit = tfb::attn_gated_splits(a->max_ctx); p.eps = a->eps; p.scale = a->scale;
    p.trace = next_trace();
    return done(tfb::attn_gated_dispatch(p, S(stream), a->pdl != 0));
}

int tfb_moe_batch_route(const tfb_moe_route_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->x && a->w_router && a->logits && a->indices && a->weights, TFB_EINVAL);
    TFB_REQUIRE(aligned16(a->x) && aligned16(a->w_router) && (!a->w_shared_scale || aligned16(a->w_shared_scale)), TFB_EALIGN);
    TFB_REQUIRE(a->mode == 0 || a->mode == 1, TFB_EINVAL);
    tfb::MoeRouteParams p;
    std::memset(&p, 0, sizeof p);
    p.x = a->x; p.w_router = static_cast<const uint16_t*>(a->w_router);
    p.w_shared_scale = static_cast<const uint16_t*>(a->w_shared_scale);
    p.logits = a->logits; p.indices = reinterpret_cast<long long*>(a->indices); p.weights = a->weights; p.shared_gate = a->shared_gate;
    p.tokens = a->tokens; p.hidden = a->hidden; p.experts = a->experts; p.top_k = a->top_k; p.mode = a->mode;
    const cudaError_t e = tfb::moe_batch_route_launch(p, S(stream), a->pdl != 0);
    return e == cudaErrorInvalidValue ? TFB_EINVAL : done(e);
}

int tfb_moe_batch(const tfb_moe_batch_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->x && a->indices && a->weights && a->w_gate && a->w_up && a->w_down && a->out, TFB_EINVAL);
    TFB_REQUIRE(a->x_bf16 && a->inner && a->y && a->counts && a->lists && a->status, TFB_EINVAL);
    TFB_REQUIRE(aligned16(a->w_gate) && aligned16(a->w_up) && aligned16(a->w_down) && aligned16(a->x_bf16) && aligned16(a->inner) &&
                    (!a->w_shared_gate || (aligned16(a->w_shared_gate) && aligned16(a->w_shared_up) && aligned16(a->w_shared_down))), TFB_EALIGN);
    tfb::MoeBatchParams p;
    std::memset(&p, 0, sizeof p);
    p.x = a->x; p.indices = reinterpret_cast<const long long*>(a->indices); p.weights = a->weights;
    p.shared_gate = a->shared_gate; p.residual = a->residual;
    auto c16 = [](const void* q) { return static_cast<const uint16_t*>(q); };
    p.w_gate = c16(a->w_gate); p.w_up = c16(a->w_up); p.w_down = c16(a->w_down);
    p.w_shared_gate = c16(a->w_shared_gate); p.w_shared_up = c16(a->w_shared_up); p.w_shared_down = c16(a->w_shared_down);
    p.out = a->out; p.x_bf16 = static_cast<uint16_t*>(a->x_bf16); p.inner = static_cast<uint16_t*>(a->inner);
    p.y = static_cast<uint16_t*>(a->y); p.counts = a->counts; p.lists = a->lists; p.status = a->status;
    p.tokens = a->tokens; p.hidden = a->hidden; p.inter = a->inter; p.experts = a->experts; p.top_k = a->top_k;
    TFB_REQUIRE(tfb::moe_batch_supported(p), TFB_EINVAL);
    return done(tfb::moe_batch_launch(p, S(stream), a->pdl != 0));
}

int tfb_moe_down_f32(const tfb_moe_down_f32_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->inner && a->out && a->top_k >= 0 && a->top_k <= 32, TFB_EINVAL);
    TFB_REQUIRE(a->top_k == 0 || (a->w_down && a->indices && a->weights), TFB_EINVAL);
    TFB_REQUIRE(a->top_k > 0 || a->w_shared, TFB_EINVAL);
    TFB_REQUIRE(a->hidden > 0 && a->inter > 0 && a->inter % 8 == 0, TFB_EINVAL);
    TFB_REQUIRE(!a->w_shared || (a->shared_inter > 0 && a->shared_inter % 8 == 0), TFB_EINVAL);
    TFB_REQUIRE((!a->w_down || aligned16(a->w_down)) && aligned16(a->inner) && (!a->w_shared || aligned16(a->w_shared)), TFB_EALIGN);
    const int is = a->w_shared ? a->shared_inter : 0;
    TFB_REQUIRE((size_t(a->top_k) * a->inter + is) * 4 <= 96 * 1024, TFB_ECAPACITY);
    tfb::MoeDownF32Params p = {};
    p.w_down = static_cast<const uint4*>(a->w_down); p.w_shared = static_cast<const uint4*>(a->w_shared);
    p.inner = a->inner; p.indices = reinterpret_cast<const long long*>(a->indices); p.weights = a->weights;
    p.shared_gate_logit = a->shared_gate_logit; p.residual = a->residual; p.out = a->out;
    p.hidden = a->hidden; p.inter = a->inter; p.shared_inter = is; p.top_k = a->top_k;
    p.expert_rank = a->expert_rank; p.expert_world = a->expert_world; p.partial = a->partial;
    TFB_REQUIRE(a->expert_world <= 1 || (a->expert_rank >= 0 && a->expert_rank < a->expert_world), TFB_EINVAL);
    return done(tfb::moe_down_f32_launch(p, S(stream), a->pdl != 0));
}

int tfb_conv_silu_f32(const float* state, const float* entry, const float* conv_w, float* mixed, int32_t channels,
                      int32_t width, int32_t pdl, tfb_stream_t stream) {
    TFB_REQUIRE(state && entry && conv_w && mixed && channels > 0 && width >= 2, TFB_EINVAL);
    return done(tfb::conv_silu_f32_launch(state, entry, conv_w, mixed, channels, width, S(stream), pdl != 0));
}

int tfb_l2norm_f32(const float* x, float* y, int32_t rows, int32_t width, float eps, int32_t pdl, tfb_stream_t stream) {
    TFB_REQUIRE(x && y && rows >= 0 && width > 0, TFB_EINVAL);
    if (rows == 0) return TFB_OK;
    return done(tfb::l2norm_f32_launch(x, y, rows, width, eps, S(stream), pdl != 0));
}

int tfb_partial_rope_f32(const float* x, const float* cos_table, const float* sin_table, const int32_t* pos, float* out,
                         int32_t heads, int32_t d, int32_t rotary_dim, int32_t pdl, tfb_stream_t stream) {
    TFB_REQUIRE(x && cos_table && sin_table && pos && out && heads > 0 && d > 0, TFB_EINVAL);
    TFB_REQUIRE(rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= d, TFB_EINVAL);
    return done(tfb::partial_rope_f32_launch(x, cos_table, sin_table, pos, out, heads, d, rotary_dim, S(stream), pdl != 0));
}

int tfb_embed_f32(const void* table, const int64_t* ids, float* out, int32_t rows, int32_t hidden, int64_t vocab,
                  int32_t pdl, tfb_stream_t stream) {
    TFB_REQUIRE(table && ids && out && rows >= 0 && hidden > 0 && vocab > 0, TFB_EINVAL);
    if (rows == 0) return TFB_OK;
    return done(tfb::embed_f32_launch(static_cast<const uint16_t*>(table), reinterpret_cast<const long long*>(ids), nullptr,
                                      nullptr, out, rows, hidden, vocab, S(stream), pdl != 0));
}

int tfb_rmsnorm_f32(const float* x, const float* gamma, float* y, int32_t rows, int32_t width, float eps, int32_t pdl,
                    tfb_stream_t stream) {
    TFB_REQUIRE(x && gamma && y && rows >= 0 && width > 0, TFB_EINVAL);
    if (rows == 0) return TFB_OK;
    return done(tfb::rmsnorm_f32_launch(x, gamma, y, rows, width, eps, S(stream), pdl != 0));
}

int tfb_residual_add_f32(const float* a, const float* b, float* out, int32_t n, int32_t pdl, tfb_stream_t stream) {
    TFB_REQUIRE(a && b && out && n >= 0, TFB_EINVAL);
    if (n == 0) return TFB_OK;
    return done(tfb::residual_add_f32_launch(a, b, out, n, S(stream), pdl != 0));
}

static int qwen35_part(const tfb_qwen35_step_args* a, int part, int layer, tfb_stream_t stream);

int tfb_qwen35_step_part(const tfb_qwen35_step_args* a, int32_t part, int32_t layer, tfb_stream_t stream) {
    TFB_REQUIRE(a && (part == 0 || part == 1 || part == 3), TFB_EINVAL);
    TFB_REQUIRE(part != 1 || (layer >= 0 && layer < a->n_layers), TFB_EINVAL);
    return qwen35_part(a, part, layer, stream);
}

int tfb_qwen35_decode_step(const tfb_qwen35_step_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->ep_world <= 1, TFB_EINVAL);          // sharded steps interleave exchange kernels: use the parts
    int rc = qwen35_part(a, 0, 0, stream);
    for (int l = 0; !rc && l < a->n_layers; ++l) rc = qwen35_part(a, 1, l, stream);
    return rc ? rc : qwen35_part(a, 3, 0, stream);
}

static int qwen35_part(const tfb_qwen35_step_args* a, int part, int layer, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->layers && a->n_layers > 0 && a->table && a->gamma_final && a->w_head && a->tokens && a->pos, TFB_EINVAL);
    TFB_REQUIRE(a->hidden_buf && a->attended_buf && a->proj_buf && a->mixed_buf && a->router_logits && a->router_idx &&
                    a->router_w && a->inner_buf && a->part_o && a->part_ml && a->counters && a->head_val && a->head_idx,
                TFB_EINVAL);
    TFB_REQUIRE(a->max_tokens <= a->max_ctx + 1, TFB_ECAPACITY);
    TFB_REQUIRE(a->inter > 0 && a->shared_inter % a->inter == 0, TFB_EINVAL);
    const bool sharded = a->ep_world > 1;
    TFB_REQUIRE(!sharded || (a->partial && a->pair && a->ep_rank >= 0 && a->ep_rank < a->ep_world &&
                             a->shared_inter % a->ep_world == 0 && a->vocab % a->ep_world == 0), TFB_EINVAL);
    const int pdl = a->pdl;
    const int H = a->hidden, KEY = a->hk * a->dk, VAL = a->hv * a->dv, CONV = 2 * KEY + VAL;
    const int N_GDN = CONV + VAL + 2 * a->hv, QD = a->hq * a->d, N_ATT = 2 * QD + 2 * a->hkv * a->d;
    const int E = a->experts, K = a->top_k, I = a->inter;
    const int IS = sharded ? a->shared_inter / a->ep_world : a->shared_inter;   // this rank's slice of the shared expert
    cudaStream_t st = S(stream);
    float* hid = a->hidden_buf;
    float* att = a->attended_buf;
    // The step's first launch carries no programmatic dependency: it starts only when the previous step has
    // fully finished, so kernels of this step may read last step's state and position before their own wait.
    cudaError_t e = cudaSuccess;
    if (part == 0) {
        e = tfb::embed_f32_launch(static_cast<const uint16_t*>(a->table), nullptr,
                                  reinterpret_cast<const long long*>(a->tokens), a->pos, hid, 1, H, a->vocab, st, false);
        return done(e);
    }
    int rc;
    tfb_gemv_f32_args g;
    auto base = [&](tfb_gemv_f32_args& x) { std::memset(&x, 0, sizeof x); x.eps = a->eps; x.pdl = pdl; };
    for (int l = layer; part == 1 && l <= layer; ++l) {
        const tfb_qwen35_layer& L = a->layers[l];
        base(g); g.w = L.w_in; g.x = hid; g.gamma = L.gamma_in; g.y = a->proj_buf; g.k = H;
        g.n = L.kind == 0 ? N_GDN : N_ATT; g.prologue = TFB_NORM_F32GAIN; g.epilogue = TFB_EPI_STORE;
        if ((rc = tfb_gemv_f32(&g, stream))) return rc;
        if (L.kind == 0) {
            tfb_gdn_args d;
            std::memset(&d, 0, sizeof d);
            d.proj = a->proj_buf; d.conv_state = L.conv_state; d.conv_state_stride = a->conv_state_stride; d.pos = a->pos;
            d.conv_w = L.conv_w; d.a_log = L.a_log; d.dt_bias = L.dt_bias; d.state = L.state; d.read = a->mixed_buf;
            d.hk = a->hk; d.hv = a->hv; d.dk = a->dk; d.dv = a->dv; d.kernel_width = a->conv_width; d.q_scale = a->q_scale;
            d.pdl = pdl;
            if ((rc = tfb_gdn_step(&d, stream))) return rc;
            base(g); g.w = L.w_out; g.x = a->mixed_buf; g.gamma = L.gamma_gdn; g.gate = a->proj_buf + CONV; g.seg = a->dv;
            g.residual = hid; g.y = att; g.n = H; g.k = VAL; g.prologue = TFB_NORM_SEGMENT_GATED; g.epilogue = TFB_EPI_RESIDUAL;
            if ((rc = tfb_gemv_f32(&g, stream))) return rc;
        } else {
            tfb_attn_gated_args t;
            std::memset(&t, 0, sizeof t);
            t.proj = a->proj_buf; t.gamma_q = L.gamma_q; t.gamma_k = L.gamma_k; t.cos_table = a->cos_table;
            t.sin_table = a->sin_table; t.pos = a->pos; t.k_pool = L.k_pool; t.v_pool = L.v_pool;
            t.block_table = a->block_table; t.out = a->mixed_buf; t.part_o = a->part_o; t.part_ml = a->part_ml;
            t.counters = a->counters; t.hq = a->hq; t.hkv = a->hkv; t.d = a->d; t.rotary_dim = a->rotary_dim;
            t.page_size = a->page_size; t.table_len = a->table_len; t.max_ctx = a->max_ctx; t.max_pos = a->max_ctx;
            t.eps = a->eps; t.scale = a->attn_scale; t.pdl = pdl;
            if ((rc = tfb_attn_gated_decode(&t, stream))) return rc;
            base(g); g.w = L.w_out; g.x = a->mixed_buf; g.residual = hid; g.y = att; g.n = H; g.k = QD;
            g.prologue = TFB_NORM_NONE; g.epilogue = TFB_EPI_RESIDUAL;
            if ((rc = tfb_gemv_f32(&g, stream))) return rc;
        }
        // ---- MoE block: router (+ the shared expert's scale row), selection, gate/up of 8 + 1 experts, down ----
        base(g); g.w = L.w_router; g.x = att; g.gamma = L.gamma_post; g.y = a->router_logits; g.n = E + 1; g.k = H;
        g.prologue = TFB_NORM_F32GAIN; g.epilogue = TFB_EPI_STORE;
        if ((rc = tfb_gemv_f32(&g, stream))) return rc;
        // the selection as a launch of its own measured 0.5 % faster per step than the last-CTA form of tfb_gemv_f32;
        // it also asks L2 for the selected experts' gate / up / down blocks while HBM is otherwise idle
        {
            tfb_router_select_args r;
            std::memset(&r, 0, sizeof r);
            r.logits_f32 = a->router_logits; r.indices = a->router_idx; r.weights_f32 = a->router_w;
            r.experts = E; r.top_k = K; r.mode = 1; r.pdl = pdl;
            r.slab[0] = L.w_gate; r.slab[1] = L.w_up; r.slab[2] = L.w_down;
            r.slab_bytes[0] = r.slab_bytes[1] = r.slab_bytes[2] = 2ull * I * H;
            r.n_slabs = a->expert_prefetch ? 3 : 0; r.expert_rank = a->ep_rank; r.expert_world = a->ep_world;
            if ((rc = tfb_router_select_prefetch(&r, stream))) return rc;
        }
        if (a->idx_trace) {
            e = tfb::copy_launch(a->router_idx, a->idx_trace + size_t(l) * K, K * 8, st, pdl != 0);
            if (e != cudaSuccess) return fail_launch(e);
        }
        base(g); g.w = L.w_gate; g.w2 = L.w_up; g.w_extra = L.w_shared_gate; g.w2_extra = L.w_shared_up; g.x = att;
        g.gamma = L.gamma_post; g.y = a->inner_buf; g.n = K * I + IS; g.k = H; g.prologue = TFB_NORM_F32GAIN;
        g.epilogue = TFB_EPI_SWIGLU; g.expert_idx = a->router_idx; g.rows_per_expert = I; g.routed_slots = K;
        g.expert_rank = a->ep_rank; g.expert_world = a->ep_world;
        if ((rc = tfb_gemv_f32(&g, stream))) return rc;
        tfb_moe_down_f32_args d;
        std::memset(&d, 0, sizeof d);
        d.w_down = L.w_down; d.w_shared = L.w_shared_down; d.inner = a->inner_buf; d.indices = a->router_idx;
        d.weights = a->router_w; d.shared_gate_logit = a->router_logits + E; d.residual = att; d.out = hid;
        d.hidden = H; d.inter = I; d.shared_inter = IS; d.top_k = K; d.pdl = pdl;
        d.expert_rank = a->ep_rank; d.expert_world = a->ep_world; d.partial = sharded ? a->partial : nullptr;
        if ((rc = tfb_moe_down_f32(&d, stream))) return rc;
        if (a->hidden_trace && !sharded) {
            e = tfb::copy_launch(hid, a->hidden_trace + size_t(l) * H, H * 4, st, pdl != 0);
            if (e != cudaSuccess) return fail_launch(e);
        }
    }
    if (part == 1) return TFB_OK;
    if (a->hidden_trace) {
        e = tfb::rmsnorm_f32_launch(hid, a->gamma_final, a->hidden_trace + size_t(a->n_layers) * H, 1, H, a->eps, st, pdl != 0);
        if (e != cudaSuccess) return fail_launch(e);
    }
    tfb_lm_head_args h;
    std::memset(&h, 0, sizeof h);
    h.w = a->w_head; h.x = hid; h.gamma = a->gamma_final; h.logits = a->logits;
    h.scratch_val = a->head_val; h.scratch_idx = a->head_idx; h.counter = a->counters + tfb::attn_gated_groups(a->hq, a->hkv, a->d);
    const int vslice = sharded ? int(a->vocab / a->ep_world) : int(a->vocab);
    if (sharded) {                                             // w_head already is this rank's slice
        if (a->logits) h.logits = static_cast<uint16_t*>(a->logits) + size_t(a->ep_rank) * vslice;
        h.pair_out = a->pair; h.index_offset = a->ep_rank * vslice;
    }
    h.n = vslice; h.k = H; h.prologue = TFB_NORM_F32_INPUT; h.eps = a->eps;
    h.x_scale = 1.f; h.out_scale = 1.f; h.pdl = pdl; h.token_out = a->picked;
    h.tokens = a->tokens; h.pos = a->pos; h.n_prompt = a->n_prompt; h.max_tokens = a->max_tokens;
    h.temperature = a->temperature; h.seed = a->seed;
    h.eos_ids = a->eos_ids; h.n_eos = a->n_eos; h.stop_at = a->stop_at;
    return tfb_lm_head_argmax(&h, stream);
}

}  // extern "C"
