// C ABI: Mamba-2 state update, MoE routing / down stage, and the granite-4.0-h decode step.
#include "api_internal.h"
#include "kernels.h"

#include <cstring>

using namespace tfb::host;
typedef const uint16_t* cu16;

extern "C" {

int tfb_residual_add(const void* a, const void* b, void* out, int32_t n, float scale, tfb_stream_t stream) {
    TFB_REQUIRE(a && b && out && n > 0, TFB_EINVAL);
    return done(tfb::residual_add_launch(cu16(a), cu16(b), static_cast<uint16_t*>(out), n, scale, S(stream), false));
}

int tfb_conv_step(const void* entry, const void* state_in, void* state_out, const void* conv_w,
                  const void* conv_b, void* mixed, void* entry_out, int32_t channels, int32_t kernel_width,
                  int32_t pdl, tfb_stream_t stream) {
    TFB_REQUIRE(entry && state_in && state_out && conv_w && mixed, TFB_EINVAL);
    TFB_REQUIRE(channels > 0 && kernel_width == 4, TFB_EINVAL);
    tfb::ConvParams p = {};
    p.entry = cu16(entry); p.state_in = cu16(state_in); p.state_out = static_cast<uint16_t*>(state_out);
    p.conv_w = cu16(conv_w); p.conv_b = cu16(conv_b); p.mixed = static_cast<uint16_t*>(mixed);
    p.entry_out = static_cast<uint16_t*>(entry_out); p.channels = channels; p.kernel_width = kernel_width;
    return done(tfb::conv_step_launch(p, S(stream), pdl != 0));
}

int tfb_ssm_step(const float* state_in, float* state_out, const void* x, const void* b_vec, const void* c_vec,
                 const void* dt_raw, const void* a_log, const void* dt_bias, const void* d_skip, void* y,
                 int32_t n_heads, int32_t head_dim, int32_t n_state, int32_t n_groups, int32_t pdl,
                 tfb_stream_t stream) {
    TFB_REQUIRE(state_in && state_out && x && b_vec && c_vec && dt_raw && a_log && dt_bias && d_skip && y, TFB_EINVAL);
    TFB_REQUIRE(n_heads > 0 && head_dim > 0 && head_dim % 8 == 0 && n_state == 128, TFB_EINVAL);
    TFB_REQUIRE(n_groups > 0 && n_heads % n_groups == 0, TFB_EINVAL);
    TFB_REQUIRE(aligned16(state_in) && aligned16(state_out), TFB_EALIGN);
    tfb::SsmParams p = {};
    p.state_in = state_in; p.state_out = state_out; p.x = cu16(x); p.b_vec = cu16(b_vec); p.c_vec = cu16(c_vec);
    p.dt_raw = cu16(dt_raw); p.a_log = cu16(a_log); p.dt_bias = cu16(dt_bias); p.d_skip = cu16(d_skip);
    p.y = static_cast<uint16_t*>(y); p.nh = n_heads; p.pd = head_dim; p.ns = n_state; p.ng = n_groups;
    return done(tfb::ssm_step_launch(p, S(stream), pdl != 0));
}

int tfb_router_select(const void* logits_bf16, const float* logits_f32, int64_t* indices, void* weights_bf16,
                      float* weights_f32, int32_t experts, int32_t top_k, int32_t mode, int32_t pdl,
                      tfb_stream_t stream) {
    TFB_REQUIRE((logits_bf16 || logits_f32) && indices && (weights_bf16 || weights_f32), TFB_EINVAL);
    TFB_REQUIRE(experts > 0 && experts <= 256 && top_k > 0 && top_k <= 32 && top_k <= experts, TFB_EINVAL);
    TFB_REQUIRE(mode == 0 || mode == 1, TFB_EINVAL);
    tfb::RouterParams p = {};
    p.logits_bf16 = cu16(logits_bf16); p.logits_f32 = logits_f32;
    p.indices = reinterpret_cast<long long*>(indices);
    p.weights_bf16 = static_cast<uint16_t*>(weights_bf16); p.weights_f32 = weights_f32;
    p.experts = experts; p.top_k = top_k; p.mode = mode;
    return done(tfb::router_select_launch(p, S(stream), pdl != 0));
}

int tfb_router_select_prefetch(const tfb_router_select_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && (a->logits_bf16 || a->logits_f32) && a->indices && (a->weights_bf16 || a->weights_f32), TFB_EINVAL);
    TFB_REQUIRE(a->experts > 0 && a->experts <= 256 && a->top_k > 0 && a->top_k <= 32 && a->top_k <= a->experts, TFB_EINVAL);
    TFB_REQUIRE((a->mode == 0 || a->mode == 1) && a->n_slabs >= 0 && a->n_slabs <= 4, TFB_EINVAL);
    TFB_REQUIRE(a->expert_world <= 1 || (a->expert_rank >= 0 && a->expert_rank < a->expert_world), TFB_EINVAL);
    tfb::RouterParams p = {};
    p.logits_bf16 = cu16(a->logits_bf16); p.logits_f32 = a->logits_f32;
    p.indices = reinterpret_cast<long long*>(a->indices);
    p.weights_bf16 = static_cast<uint16_t*>(a->weights_bf16); p.weights_f32 = a->weights_f32;
    p.experts = a->experts; p.top_k = a->top_k; p.mode = a->mode;
    for (int i = 0; i < a->n_slabs; ++i) {
        TFB_REQUIRE(a->slab[i] && aligned16(a->slab[i]) && a->slab_bytes[i] > 0 && a->slab_bytes[i] % 16 == 0, TFB_EALIGN);
        p.slab[i] = a->slab[i]; p.slab_bytes[i] = a->slab_bytes[i];
    }
    p.n_slabs = a->n_slabs; p.expert_rank = a->expert_rank; p.expert_world = a->expert_world;
    return done(tfb::router_select_launch(p, S(stream), a->pdl != 0));
}

int tfb_moe_down(const tfb_moe_down_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->w_down && a->inner && a->indices && a->weights && a->out, TFB_EINVAL);
    TFB_REQUIRE(a->hidden > 0 && a->inter > 0 && a->inter % 8 == 0 && a->top_k > 0 && a->top_k <= 32, TFB_EINVAL);
    TFB_REQUIRE(!a->w_shared || (a->shared_act && a->shared_inter > 0 && a->shared_inter % 8 == 0), TFB_EINVAL);
    TFB_REQUIRE(aligned16(a->w_down) && (!a->w_shared || aligned16(a->w_shared)) && aligned16(a->inner) &&
                    (!a->shared_act || aligned16(a->shared_act)), TFB_EALIGN);
    TFB_REQUIRE((size_t(a->top_k) * a->inter + a->shared_inter) * 4 <= 96 * 1024, TFB_ECAPACITY);
    tfb::MoeDownParams p = {};
    p.w_down = static_cast<const uint4*>(a->w_down); p.w_shared = static_cast<const uint4*>(a->w_shared);
    p.inner = cu16(a->inner); p.shared_act = cu16(a->shared_act);
    p.indices = reinterpret_cast<const long long*>(a->indices); p.weights = cu16(a->weights);
    p.shared_gate = a->shared_gate; p.residual = cu16(a->residual); p.out = static_cast<uint16_t*>(a->out);
    p.hidden = a->hidden; p.inter = a->inter; p.shared_inter = a->w_shared ? a->shared_inter : 0; p.top_k = a->top_k;
    p.res_scale = a->res_scale;
    p.expert_rank = a->expert_rank; p.expert_world = a->expert_world; p.partial = a->partial;
    TFB_REQUIRE(a->expert_world <= 1 || (a->expert_rank >= 0 && a->expert_rank < a->expert_world), TFB_EINVAL);
    return done(tfb::moe_down_launch(p, S(stream), a->pdl != 0));
}

int tfb_moe_finalize(const float* partial, const void* residual, void* out, int32_t hidden, float res_scale,
                     int32_t has_shared, int32_t pdl, tfb_stream_t stream) {
    TFB_REQUIRE(partial && out && hidden > 0, TFB_EINVAL);
    return done(tfb::moe_finalize_launch(partial, cu16(residual), static_cast<uint16_t*>(out), hidden, res_scale,
                                         has_shared != 0, S(stream), pdl != 0));
}

int tfb_pick_finalize(const float* pairs, int32_t world, int64_t* tokens, int32_t* pos, int32_t n_prompt,
                      int32_t max_tokens, int64_t* picked, int32_t pdl, tfb_stream_t stream) {
    TFB_REQUIRE(pairs && world > 0 && (picked || (tokens && pos)), TFB_EINVAL);
    return done(tfb::pick_finalize_launch(pairs, world, reinterpret_cast<long long*>(tokens), pos, n_prompt, max_tokens,
                                          reinterpret_cast<long long*>(picked), S(stream), pdl != 0));
}

int tfb_moe_allreduce_finalize(const tfb_moe_allreduce_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->partial && a->epoch && a->status && (a->out || a->out_f32) && a->hidden > 0, TFB_EINVAL);
    TFB_REQUIRE(a->world >= 2 && a->world <= tfb::kMaxPeers && a->rank >= 0 && a->rank < a->world, TFB_EINVAL);
    tfb::PeerReduceParams p = {};
    for (int r = 0; r < a->world; ++r) {
        TFB_REQUIRE(a->inbox[r] && a->flags[r], TFB_EINVAL);
        p.inbox[r] = a->inbox[r]; p.flags[r] = a->flags[r];
    }
    p.partial = a->partial; p.epoch = a->epoch; p.status = a->status; p.residual = cu16(a->residual);
    p.out = static_cast<uint16_t*>(a->out); p.hidden = a->hidden; p.rank = a->rank; p.world = a->world;
    p.has_shared = a->has_shared; p.res_scale = a->res_scale;
    p.residual_f32 = a->residual_f32; p.out_f32 = a->out_f32; p.gate_logit = a->gate_logit;
    return done(tfb::moe_allreduce_finalize_launch(p, S(stream), a->pdl != 0));
}

int tfb_pick_allgather(const tfb_pick_allgather_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->pair && a->epoch && a->status && (a->picked || (a->tokens && a->pos)), TFB_EINVAL);
    TFB_REQUIRE(a->world >= 2 && a->world <= tfb::kMaxPeers && a->rank >= 0 && a->rank < a->world, TFB_EINVAL);
    tfb::PeerPickParams p = {};
    for (int r = 0; r < a->world; ++r) {
        TFB_REQUIRE(a->inbox[r] && a->flags[r], TFB_EINVAL);
        p.inbox[r] = a->inbox[r]; p.flags[r] = a->flags[r];
    }
    p.pair = a->pair; p.epoch = a->epoch; p.status = a->status; p.tokens = reinterpret_cast<long long*>(a->tokens);
    p.pos = a->pos; p.picked = reinterpret_cast<long long*>(a->picked); p.n_prompt = a->n_prompt;
    p.max_tokens = a->max_tokens; p.rank = a->rank; p.world = a->world;
    return done(tfb::pick_allgather_launch(p, S(stream), a->pdl != 0));
}

static int granite_part(const tfb_granite_step_args* a, int part, int layer, tfb_stream_t stream);

int tfb_granite_step_part(const tfb_granite_step_args* a, int32_t part, int32_t layer, tfb_stream_t stream) {
    TFB_REQUIRE(a && part >= 0 && part <= 4, TFB_EINVAL);
    TFB_REQUIRE((part != 1 && part != 2) || (layer >= 0 && layer < a->n_layers), TFB_EINVAL);
    return granite_part(a, part, layer, stream);
}

int tfb_granite_decode_step(const tfb_granite_step_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->ep_world <= 1, TFB_EINVAL);        // sharded steps interleave collectives: use the parts
    int rc = granite_part(a, 0, 0, stream);
    for (int l = 0; !rc && l < a->n_layers; ++l) rc = granite_part(a, 1, l, stream);
    return rc ? rc : granite_part(a, 3, 0, stream);
}

// part 0: embed.  part 1: layer `layer` up to and including the MoE down stage (complete on one GPU; on
// several, it leaves this rank's un-rounded partial sums in a->partial for the caller to all-reduce).
// part 2: finish layer `layer` from the summed partials.  part 3: final norm + head (one GPU: with the
// greedy pick; several: this rank's vocabulary slice, leaving (logit, index) in a->pair for an all-gather).
// part 4: pick from the gathered pairs.
static int granite_part(const tfb_granite_step_args* a, int part, int layer, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->layers && a->n_layers > 0 && a->table && a->gamma_final && a->tokens && a->pos, TFB_EINVAL);
    TFB_REQUIRE(a->hidden_buf && a->proj_buf && a->mixed_buf && a->y_buf && a->router_logits && a->router_idx &&
                    a->router_w && a->inner_buf && a->shared_buf, TFB_EINVAL);
    TFB_REQUIRE(a->part_o && a->part_ml && a->counters && a->head_val && a->head_idx, TFB_EINVAL);
    TFB_REQUIRE(a->max_tokens <= a->max_ctx + 1, TFB_ECAPACITY);
    const bool sharded = a->ep_world > 1;
    TFB_REQUIRE(!sharded || (a->partial && a->pair && a->gathered && a->ep_rank >= 0 && a->ep_rank < a->ep_world), TFB_EINVAL);
    const bool pdl = a->pdl != 0;
    const int H = a->hidden, EXP = a->nh * a->pd, BC = a->ng * a->ns, CONVD = EXP + 2 * BC, PROJ = EXP + CONVD + a->nh;
    const int QP = a->hq * a->d, NQKV = (a->hq + 2 * a->hkv) * a->d;
    const int E = a->experts, K = a->top_k, I = a->inter;
    const int IS = sharded ? a->shared_inter / a->ep_world : a->shared_inter;   // this rank's slice of the shared expert
    cudaStream_t st = S(stream);
    uint16_t* hid = static_cast<uint16_t*>(a->hidden_buf);
    uint16_t* proj = static_cast<uint16_t*>(a->proj_buf);
    uint16_t* mixed = static_cast<uint16_t*>(a->mixed_buf);
    uint16_t* trace = static_cast<uint16_t*>(a->hidden_trace);

    cudaError_t e = cudaSuccess;
    if (part == 0) {
        // The step's first launch carries no programmatic dependency: it starts only when the previous step has
        // fully finished, so kernels of this step may read last step's state and position before their own wait.
        e = tfb::embed_launch(cu16(a->table), nullptr, reinterpret_cast<const long long*>(a->tokens), a->pos, hid, 1, H,
                              a->vocab, a->embed_scale, st, false);
        return done(e);
    }
    if (part == 2) {
        e = tfb::moe_finalize_launch(a->partial, hid, hid, H, a->res_scale, true, st, pdl);
        if (e != cudaSuccess) return fail_launch(e);
        if (trace) e = tfb::copy_launch(hid, trace + size_t(layer) * H, H * 2, st, pdl);
        return done(e);
    }
    if (part == 4)
        return done(tfb::pick_finalize_launch(a->gathered, a->ep_world, reinterpret_cast<long long*>(a->tokens), a->pos,
                                              a->n_prompt, a->max_tokens, reinterpret_cast<long long*>(a->picked), st, pdl));

    auto base = [&](tfb_gemv_args& g) {
        std::memset(&g, 0, sizeof g);
        g.eps = a->eps; g.x_scale = 1.f; g.res_scale = 1.f; g.out_scale = 1.f; g.pdl = pdl;
    };
    int rc;
    tfb_gemv_args g;
    for (int l = layer; part == 1 && l <= layer; ++l) {
        const tfb_granite_layer& L = a->layers[l];
        if (L.kind == 0) {
            // in_projection: gate | conv entry | dt
            base(g); g.w = L.w_in; g.x = hid; g.gamma = L.gamma_in; g.y = proj; g.n = PROJ; g.k = H;
            g.prologue = TFB_NORM_F32GAIN; g.epilogue = TFB_EPI_STORE;
            if ((rc = gemv_checked(&g, stream))) return rc;
            if ((rc = tfb_conv_step(proj + EXP, L.conv_state, L.conv_state, L.conv_w, L.conv_b, mixed, nullptr, CONVD,
                                    a->conv_width, pdl, stream))) return rc;
            if ((rc = tfb_ssm_step(L.ssm_state, L.ssm_state, mixed, mixed + EXP, mixed + EXP + BC, proj + EXP + CONVD,
                                   L.a_log, L.dt_bias, L.d_skip, a->y_buf, a->nh, a->pd, a->ns, a->ng, pdl, stream)))
                return rc;
            // gated norm + out_proj + scaled residual
            base(g); g.w = L.w_out; g.x = a->y_buf; g.x_gate = proj; g.gamma = L.gamma_ssm; g.residual = hid; g.y = hid;
            g.n = H; g.k = EXP; g.prologue = TFB_NORM_GATED; g.epilogue = TFB_EPI_RESIDUAL; g.res_scale = a->res_scale;
            if ((rc = gemv_checked(&g, stream))) return rc;
        } else {
            base(g); g.w = L.w_in; g.x = hid; g.gamma = L.gamma_in; g.y = proj; g.n = NQKV; g.k = H;
            g.prologue = TFB_NORM_F32GAIN; g.epilogue = TFB_EPI_STORE;
            if ((rc = gemv_checked(&g, stream))) return rc;
            tfb_attn_gqa_args t;
            std::memset(&t, 0, sizeof t);
            t.qkv = proj; t.pos = a->pos; t.k_pool = L.k_pool; t.v_pool = L.v_pool; t.block_table = a->block_table;
            t.out = a->y_buf; t.part_o = a->part_o; t.part_ml = a->part_ml; t.counters = a->counters;
            t.hq = a->hq; t.hkv = a->hkv; t.d = a->d; t.rotary_dim = 0; t.page_size = a->page_size;
            t.table_len = a->table_len; t.max_ctx = a->max_ctx; t.max_pos = a->max_ctx; t.eps = a->eps;
            t.scale = a->attn_scale; t.norm_mode = TFB_NORM_NONE; t.pdl = pdl;
            if ((rc = tfb_attn_gqa_decode(&t, stream))) return rc;
            base(g); g.w = L.w_out; g.x = a->y_buf; g.residual = hid; g.y = hid; g.n = H; g.k = QP;
            g.prologue = TFB_NORM_NONE; g.epilogue = TFB_EPI_RESIDUAL; g.res_scale = a->res_scale;
            if ((rc = gemv_checked(&g, stream))) return rc;
        }
        // ---- MoE block ----
        base(g); g.w = L.w_router; g.x = hid; g.gamma = L.gamma_post; g.y = a->router_logits; g.n = E; g.k = H;
        g.prologue = TFB_NORM_F32GAIN; g.epilogue = TFB_EPI_STORE;
        if ((rc = gemv_checked(&g, stream))) return rc;
        if ((rc = tfb_router_select(a->router_logits, nullptr, a->router_idx, a->router_w, nullptr, E, K, 0, pdl, stream)))
            return rc;
        if (a->idx_trace) {
            e = tfb::copy_launch(a->router_idx, a->idx_trace + size_t(l) * K, K * 8, st, pdl);
            if (e != cudaSuccess) return fail_launch(e);
        }
        base(g); g.w = L.w_gate; g.w2 = L.w_up; g.x = hid; g.gamma = L.gamma_post; g.y = a->inner_buf; g.n = K * I; g.k = H;
        g.prologue = TFB_NORM_F32GAIN; g.epilogue = TFB_EPI_SWIGLU; g.expert_idx = a->router_idx; g.rows_per_expert = I;
        g.expert_rank = a->ep_rank; g.expert_world = a->ep_world;
        if ((rc = gemv_checked(&g, stream))) return rc;
        base(g); g.w = L.w_shared_in; g.w2 = cu16(L.w_shared_in) + size_t(IS) * H; g.x = hid; g.gamma = L.gamma_post;
        g.y = a->shared_buf; g.n = IS; g.k = H; g.prologue = TFB_NORM_F32GAIN; g.epilogue = TFB_EPI_SWIGLU;
        if ((rc = gemv_checked(&g, stream))) return rc;
        tfb_moe_down_args d;
        std::memset(&d, 0, sizeof d);
        d.w_down = L.w_down; d.w_shared = L.w_shared_out; d.inner = a->inner_buf; d.shared_act = a->shared_buf;
        d.indices = a->router_idx; d.weights = a->router_w; d.residual = hid; d.out = hid;
        d.hidden = H; d.inter = I; d.shared_inter = IS; d.top_k = K; d.res_scale = a->res_scale; d.pdl = pdl;
        d.expert_rank = a->ep_rank; d.expert_world = a->ep_world; d.partial = sharded ? a->partial : nullptr;
        if ((rc = tfb_moe_down(&d, stream))) return rc;
        if (trace && !sharded) {
            e = tfb::copy_launch(hid, trace + size_t(l) * H, H * 2, st, pdl);
            if (e != cudaSuccess) return fail_launch(e);
        }
    }
    if (part == 1) return TFB_OK;
    if (trace) {
        e = tfb::rmsnorm_launch(hid, cu16(a->gamma_final), trace + size_t(a->n_layers) * H, 1, H, a->eps,
                                TFB_NORM_F32GAIN, st, pdl);
        if (e != cudaSuccess) return fail_launch(e);
    }
    tfb_lm_head_args h;
    std::memset(&h, 0, sizeof h);
    h.w = a->table; h.x = hid; h.gamma = a->gamma_final; h.logits = a->logits;
    h.scratch_val = a->head_val; h.scratch_idx = a->head_idx; h.counter = a->counters + a->hkv;
    const int vslice = sharded ? int(a->vocab / a->ep_world) : int(a->vocab);
    if (sharded) {
        h.w = cu16(a->table) + size_t(a->ep_rank) * vslice * H;
        if (a->logits) h.logits = static_cast<uint16_t*>(a->logits) + size_t(a->ep_rank) * vslice;
        h.pair_out = a->pair; h.index_offset = a->ep_rank * vslice;
    }
    h.n = vslice; h.k = H; h.prologue = TFB_NORM_F32GAIN; h.eps = a->eps;
    h.x_scale = 1.f; h.out_scale = a->logits_scale; h.pdl = pdl; h.token_out = a->picked;
    h.tokens = a->tokens; h.pos = a->pos; h.n_prompt = a->n_prompt; h.max_tokens = a->max_tokens;
    h.temperature = a->temperature; h.seed = a->seed;
    h.eos_ids = a->eos_ids; h.n_eos = a->n_eos; h.stop_at = a->stop_at;
    return tfb_lm_head_argmax(&h, stream);
}

}  // extern "C"
