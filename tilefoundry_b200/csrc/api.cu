// extern "C" entry points: host-side validation, then enqueue.  See include/tfb200.h.
#include "../../include/tfb200.h"
#include "kernels.h"
#include "api_internal.h"
#include <cstdlib>

#include <cstdio>
#include <cstring>

namespace tfb { namespace host {

thread_local char g_last_error[256] = "";

// debug timeline: 4 words per launch, handed out in launch order
unsigned long long* g_trace_buf = nullptr;
int g_trace_cap = 0, g_trace_next = 0;
unsigned long long* next_trace() {
    if (!g_trace_buf || g_trace_next >= g_trace_cap) return nullptr;
    return g_trace_buf + 8 * size_t(g_trace_next++);
}

int fail_launch(cudaError_t e) {
    std::snprintf(g_last_error, sizeof g_last_error, "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
    cudaGetLastError();  // clear the sticky-free error so later launches report their own
    return TFB_ELAUNCH;
}

} }  // namespace tfb::host

using namespace tfb::host;

extern "C" {

int tfb_version(void) { return 100; }

int tfb_debug_trace(void* device_buffer, int32_t capacity) {
    g_trace_buf = static_cast<unsigned long long*>(device_buffer);
    g_trace_cap = device_buffer ? capacity : 0;
    g_trace_next = 0;
    return TFB_OK;
}

int tfb_sample_top_p(const tfb_sample_top_p_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->logits && a->pos && a->prev_pos && a->tokens && a->hist, TFB_EINVAL);
    TFB_REQUIRE(a->vocab > 0 && a->temperature > 0.f && a->top_p > 0.f && a->top_p <= 1.f, TFB_EINVAL);
    TFB_REQUIRE(a->n_eos >= 0 && a->n_eos <= 16 && (a->n_eos == 0 || (a->eos_ids && a->stop_at)), TFB_EINVAL);
    tfb::TopPParams p;
    std::memset(&p, 0, sizeof p);
    p.logits = static_cast<const uint16_t*>(a->logits); p.vocab = a->vocab;
    p.temperature = a->temperature; p.top_p = a->top_p; p.seed = a->seed;
    p.pos = a->pos; p.prev_pos = a->prev_pos; p.tokens = reinterpret_cast<long long*>(a->tokens); p.n_prompt = a->n_prompt;
    p.picked = reinterpret_cast<long long*>(a->picked); p.threshold_out = a->threshold_out;
    p.eos_ids = reinterpret_cast<const long long*>(a->eos_ids); p.n_eos = a->eos_ids ? a->n_eos : 0; p.stop_at = a->stop_at;
    p.hist = a->hist;
    return done(tfb::sample_top_p_launch(p, S(stream), a->pdl != 0));
}

int tfb_graph_step_host(void* graph_exec, void* token_slot, const int64_t* token_in_host, const void* picked,
                        int64_t* token_out_host, tfb_stream_t stream) {
    TFB_REQUIRE(graph_exec && token_slot && token_in_host && picked && token_out_host, TFB_EINVAL);
    cudaStream_t st = S(stream);
    cudaError_t e = cudaMemcpyAsync(token_slot, token_in_host, sizeof(int64_t), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph_exec), st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(token_out_host, picked, sizeof(int64_t), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    return done(e);
}

int tfb_graph_generate_host(void* graph_exec, void* tokens, int64_t pos, int32_t steps, int64_t* token_io_host,
                            int64_t* out_host, tfb_stream_t stream) {
    TFB_REQUIRE(graph_exec && tokens && token_io_host && pos >= 0 && steps >= 0, TFB_EINVAL);
    int64_t* hist = static_cast<int64_t*>(tokens);
    for (int32_t i = 0; i < steps; ++i) {
        const int rc = tfb_graph_step_host(graph_exec, hist + pos + i, token_io_host, hist + pos + i + 1, token_io_host, stream);
        if (rc != TFB_OK) return rc;
        if (out_host) out_host[i] = *token_io_host;
    }
    return TFB_OK;
}

const char* tfb_status_string(int status) {
    switch (status) {
        case TFB_OK: return "ok";
        case TFB_EINVAL: return "invalid argument (size, null pointer or unsupported combination)";
        case TFB_EALIGN: return "pointer or row stride is not 16-byte aligned";
        case TFB_ECAPACITY: return "position or context exceeds the capacity given";
        case TFB_ELAUNCH: return "the CUDA runtime refused the launch (see tfb_last_error)";
        case TFB_ENODEVICE: return "no sm_100 device is current";
        default: return "unknown status";
    }
}

const char* tfb_last_error(void) { return g_last_error; }

int tfb_embed(const void* table, const int64_t* ids, void* out, int32_t rows, int32_t hidden,
              int64_t vocab, float scale, tfb_stream_t stream) {
    TFB_REQUIRE(table && ids && out, TFB_EINVAL);
    TFB_REQUIRE(rows >= 0 && hidden > 0 && vocab > 0 && hidden % 8 == 0, TFB_EINVAL);
    TFB_REQUIRE(aligned16(table) && aligned16(out), TFB_EALIGN);
    if (rows == 0) return TFB_OK;
    return done(tfb::embed_launch(static_cast<const uint16_t*>(table),
                                  reinterpret_cast<const long long*>(ids), nullptr, nullptr,
                                  static_cast<uint16_t*>(out), rows, hidden, vocab, scale, S(stream), false));
}

int tfb_rmsnorm(const void* x, const void* gamma, void* y, int32_t rows, int32_t width, float eps,
                int32_t mode, tfb_stream_t stream) {
    TFB_REQUIRE(x && gamma && y, TFB_EINVAL);
    TFB_REQUIRE(rows >= 0 && width > 0, TFB_EINVAL);
    TFB_REQUIRE(mode == TFB_NORM_F32GAIN || mode == TFB_NORM_CAST_THEN_GAIN, TFB_EINVAL);
    if (rows == 0) return TFB_OK;
    return done(tfb::rmsnorm_launch(static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(gamma),
                                    static_cast<uint16_t*>(y), rows, width, eps, mode, S(stream), false));
}

}  // extern "C"
// argument checks of one projection and its kernel parameters
static int gemv_params(const tfb_gemv_args* a, tfb::GemvParams& p) {
    TFB_REQUIRE(a && a->w && a->x && a->y, TFB_EINVAL);
    TFB_REQUIRE(a->n > 0 && a->k > 0 && a->k % 256 == 0 && a->k <= 16384, TFB_EINVAL);
    TFB_REQUIRE(a->prologue >= TFB_NORM_NONE && a->prologue <= TFB_NORM_GATED, TFB_EINVAL);
    TFB_REQUIRE(a->prologue != TFB_NORM_GATED || (a->x_gate && aligned16(a->x_gate) && a->k <= 8192 &&
                                                  a->epilogue <= TFB_EPI_RESIDUAL && a->kernel != TFB_KERNEL_RING), TFB_EINVAL);
    TFB_REQUIRE(!a->expert_idx || (a->rows_per_expert > 0 && a->rows_per_expert % 2 == 0 &&
                                   a->n % a->rows_per_expert == 0 && a->kernel != TFB_KERNEL_RING), TFB_EINVAL);
    TFB_REQUIRE(a->epilogue >= TFB_EPI_STORE && a->epilogue <= TFB_EPI_STORE_F32, TFB_EINVAL);
    TFB_REQUIRE(a->prologue == TFB_NORM_NONE || a->gamma, TFB_EINVAL);
    TFB_REQUIRE(a->epilogue != TFB_EPI_RESIDUAL || a->residual, TFB_EINVAL);
    TFB_REQUIRE(a->epilogue != TFB_EPI_SWIGLU || a->w2, TFB_EINVAL);
    TFB_REQUIRE(aligned16(a->w) && aligned16(a->x) && (!a->w2 || aligned16(a->w2)) &&
                    (!a->gamma || aligned16(a->gamma)), TFB_EALIGN);
    TFB_REQUIRE(!a->prefetch || (aligned16(a->prefetch) && a->prefetch_bytes % 16 == 0), TFB_EALIGN);
    p = {};
    p.w = static_cast<const uint4*>(a->w);
    p.w2 = static_cast<const uint4*>(a->w2);
    p.x = static_cast<const uint16_t*>(a->x);
    p.gamma = static_cast<const uint16_t*>(a->gamma);
    p.residual = static_cast<const uint16_t*>(a->residual);
    p.y = a->y;
    p.n = a->n;
    p.k = a->k;
    p.eps = a->eps;
    p.x_scale = a->x_scale;
    p.res_scale = a->res_scale;
    p.out_scale = a->out_scale;
    p.prefetch = a->prefetch;
    p.prefetch_bytes = a->prefetch_bytes;
    p.self_prefetch = a->self_prefetch;
    p.trace = next_trace();
    p.x2 = static_cast<const uint16_t*>(a->x_gate);
    p.expert_idx = reinterpret_cast<const long long*>(a->expert_idx);
    p.rows_per_expert = a->rows_per_expert;
    p.expert_rank = a->expert_rank;
    p.expert_world = a->expert_world;
    return TFB_OK;
}

int tfb::host::gemv_checked(const tfb_gemv_args* a, tfb_stream_t stream) {
    tfb::GemvParams p;
    if (const int rc = gemv_params(a, p)) return rc;
    if (a->kernel == TFB_KERNEL_RING && tfb::gemv_stream_supported(a->n, a->k))
        return done(tfb::gemv_stream_dispatch(p, a->prologue, a->epilogue, S(stream), a->pdl != 0));
    if (a->kernel == TFB_KERNEL_ASYNC && tfb::gemv_async_supported(p, a->prologue, a->epilogue))
        return done(tfb::gemv_async_dispatch(p, a->prologue, a->epilogue, S(stream), a->pdl != 0));
    // Measured on B200 (28 back-to-back launches over distinct 50 MB gate/up pairs): the persistent form with one
    // row pair per warp and both halves of the row in flight takes 11.7 us against 13.8 us for the one-shot
    // grid (66 MB at K = 2560: 15.5 against 17.6 us).  For the single-matrix projections the one-shot grid is as fast
    // or faster, and so it is for SwiGLU with fewer row pairs than resident warps (1536 x 4096: 6.9 against 8.1 us),
    // so only wide SwiGLU projections default to the persistent form.
    const bool auto_persist = a->kernel == TFB_KERNEL_AUTO && a->epilogue == TFB_EPI_SWIGLU && a->n >= 4096;
    if ((a->kernel == TFB_KERNEL_PERSIST || auto_persist) && a->epilogue <= TFB_EPI_SWIGLU &&
        tfb::gemv_persist_supported(p, a->prologue))
        return done(tfb::gemv_persist_dispatch(p, a->prologue, a->epilogue, S(stream), a->pdl != 0));
    return done(tfb::gemv_dispatch(p, a->prologue, a->epilogue, S(stream), a->pdl != 0));
}

extern "C" {
int tfb_gemv(const tfb_gemv_args* args, tfb_stream_t stream) { return gemv_checked(args, stream); }

int tfb_gemv_pair(const tfb_gemv_args* a, const tfb_gemv_args* b, tfb_stream_t stream) {
    tfb::GemvParams pa, pb;
    if (const int rc = gemv_params(a, pa)) return rc;
    if (const int rc = gemv_params(b, pb)) return rc;
    TFB_REQUIRE(a->prologue == b->prologue && a->epilogue == TFB_EPI_STORE && b->epilogue == TFB_EPI_STORE, TFB_EINVAL);
    TFB_REQUIRE(a->prologue != TFB_NORM_GATED && a->k <= 2048 && b->k <= 2048 && !a->expert_idx && !b->expert_idx, TFB_EINVAL);
    return done(tfb::gemv_pair_dispatch(pa, pb, a->prologue, a->epilogue, S(stream), a->pdl != 0));
}

int tfb_gemv_chain(const tfb_gemv_chain_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->n_phases >= 1 && a->n_phases <= 4 && a->sync, TFB_EINVAL);
    tfb::ChainParams p = {};
    p.n_phases = a->n_phases;
    p.barrier = a->sync;
    p.status = a->sync + 2;
    for (int q = 0; q < a->n_phases; ++q) {
        const tfb_gemv_args& g = a->phase[q];
        TFB_REQUIRE(g.w && g.x && g.y && g.n >= 256 && g.k > 0 && g.k % 256 == 0 && g.k <= 8192, TFB_EINVAL);
        TFB_REQUIRE(g.prologue >= TFB_NORM_NONE && g.prologue <= TFB_NORM_CAST_THEN_GAIN, TFB_EINVAL);
        TFB_REQUIRE(g.epilogue >= TFB_EPI_STORE && g.epilogue <= TFB_EPI_SWIGLU && !g.expert_idx, TFB_EINVAL);
        TFB_REQUIRE(g.prologue == TFB_NORM_NONE || g.gamma, TFB_EINVAL);
        TFB_REQUIRE(g.epilogue != TFB_EPI_RESIDUAL || g.residual, TFB_EINVAL);
        TFB_REQUIRE(g.epilogue != TFB_EPI_SWIGLU || g.w2, TFB_EINVAL);
        TFB_REQUIRE(aligned16(g.w) && aligned16(g.x) && (!g.w2 || aligned16(g.w2)) && (!g.gamma || aligned16(g.gamma)), TFB_EALIGN);
        tfb::ChainPhase& ph = p.ph[q];
        ph.w = static_cast<const uint4*>(g.w); ph.w2 = static_cast<const uint4*>(g.w2);
        ph.x = static_cast<const uint16_t*>(g.x); ph.gamma = static_cast<const uint16_t*>(g.gamma);
        ph.residual = static_cast<const uint16_t*>(g.residual); ph.y = static_cast<uint16_t*>(g.y);
        ph.n = g.n; ph.k = g.k; ph.norm = g.prologue; ph.epi = g.epilogue;
        ph.eps = g.eps; ph.x_scale = g.x_scale; ph.res_scale = g.res_scale;
    }
    return done(tfb::gemv_chain_launch(p, S(stream), a->pdl != 0, nullptr));
}

int32_t tfb_gemm_small_m_splits(int32_t n, int32_t k) {
    if (n <= 0 || k < 64) return 0;
    return tfb::gemm_tc_splits(n, k);
}
int32_t tfb_gemm_small_m_swiglu_splits(int32_t n, int32_t k) {
    if (n <= 0 || k < 64) return 0;
    return tfb::gemm_tc_splits_swiglu(n, k);
}

int tfb_gemm_small_m(const tfb_gemm_small_m_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->w && a->x && a->y && a->status, TFB_EINVAL);
    TFB_REQUIRE(a->m >= 1 && a->m <= 32 && a->n > 0 && a->k >= 64 && a->k % 64 == 0, TFB_EINVAL);
    TFB_REQUIRE(aligned16(a->w) && aligned16(a->x), TFB_EALIGN);
    TFB_REQUIRE(a->swiglu == 0 || (a->n % 64 == 0 && !a->residual), TFB_EINVAL);
    tfb::TcParams p = {};
    p.M = a->m; p.N = a->n; p.K = a->k; p.swiglu = a->swiglu != 0;
    p.splits = p.swiglu ? tfb::gemm_tc_splits_swiglu(a->n, a->k) : tfb::gemm_tc_splits(a->n, a->k);
    p.status = a->status;
    p.y = static_cast<uint16_t*>(a->y); p.residual = static_cast<const uint16_t*>(a->residual);
    p.res_scale = a->res_scale == 0.f ? 1.f : a->res_scale;
    return done(tfb::gemm_tc_launch(a->w, a->x, p, S(stream), a->pdl != 0));
}

int32_t tfb_lm_head_scratch_entries(int32_t n) {
    if (n <= 0) return 0;
    const int a = tfb::lm_head_ctas(n), b = tfb::lm_head_stream_ctas();
    return a > b ? a : b;
}

int tfb_lm_head_argmax(const tfb_lm_head_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->w && a->x && a->scratch_val && a->scratch_idx && a->counter, TFB_EINVAL);
    TFB_REQUIRE(a->token_out || a->pair_out || (a->tokens && a->pos), TFB_EINVAL);
    TFB_REQUIRE(a->n > 0 && a->k > 0 && a->k % 256 == 0 && a->k <= 8192, TFB_EINVAL);
    TFB_REQUIRE((a->prologue >= TFB_NORM_NONE && a->prologue <= TFB_NORM_CAST_THEN_GAIN) || a->prologue == TFB_NORM_F32_INPUT, TFB_EINVAL);
    TFB_REQUIRE(a->prologue == TFB_NORM_NONE || a->prologue == TFB_NORM_F32_INPUT || a->gamma, TFB_EINVAL);
    TFB_REQUIRE(aligned16(a->w) && aligned16(a->x) && (!a->gamma || aligned16(a->gamma)), TFB_EALIGN);
    if (a->kernel == TFB_KERNEL_RING && a->prologue != TFB_NORM_F32_INPUT && !a->pair_out && !(a->temperature > 0.f) &&
        tfb::gemv_stream_supported(a->n, a->k)) {
        tfb::GemvParams g = {};
        g.w = static_cast<const uint4*>(a->w);
        g.x = static_cast<const uint16_t*>(a->x);
        g.gamma = static_cast<const uint16_t*>(a->gamma);
        g.y = a->logits;
        g.n = a->n; g.k = a->k; g.eps = a->eps; g.x_scale = a->x_scale; g.res_scale = 1.f; g.out_scale = a->out_scale;
        g.scratch_val = a->scratch_val; g.scratch_idx = a->scratch_idx; g.counter = a->counter;
        g.token_out = reinterpret_cast<long long*>(a->token_out);
        g.tokens = reinterpret_cast<long long*>(a->tokens); g.pos = a->pos;
        g.n_prompt = a->n_prompt; g.max_tokens = a->max_tokens; g.self_prefetch = a->self_prefetch;
        return done(tfb::gemv_stream_dispatch(g, a->prologue, 4, S(stream), a->pdl != 0));
    }
    tfb::HeadParams p;
    p.w = static_cast<const uint4*>(a->w);
    p.x = static_cast<const uint16_t*>(a->x);
    p.gamma = static_cast<const uint16_t*>(a->gamma);
    p.logits = static_cast<uint16_t*>(a->logits);
    p.token_out = reinterpret_cast<long long*>(a->token_out);
    p.scratch_val = a->scratch_val;
    p.scratch_idx = a->scratch_idx;
    p.counter = a->counter;
    p.n = a->n;
    p.k = a->k;
    p.eps = a->eps;
    p.x_scale = a->x_scale;
    p.out_scale = a->out_scale;
    p.tokens = reinterpret_cast<long long*>(a->tokens);
    p.pos = a->pos;
    p.n_prompt = a->n_prompt;
    p.max_tokens = a->max_tokens;
    p.trace = next_trace();
    p.pair_out = a->pair_out;
    p.index_offset = a->index_offset;
    p.temperature = a->temperature > 0.f ? a->temperature : 0.f;
    p.seed = a->seed;
    TFB_REQUIRE(a->n_eos >= 0 && a->n_eos <= 16 && (a->eos_ids == nullptr || (a->stop_at && a->n_eos > 0)), TFB_EINVAL);
    p.eos_ids = reinterpret_cast<const long long*>(a->eos_ids);
    p.n_eos = a->eos_ids ? a->n_eos : 0;
    p.stop_at = a->stop_at;
    return done(tfb::lm_head_dispatch(p, a->prologue, S(stream), a->pdl != 0));
}

int32_t tfb_attn_splits(int32_t max_ctx) { return max_ctx > 0 ? tfb::attn_splits(max_ctx) : 0; }

// Every argument check of the attention entry points; `own_scratch`: the caller passes part_o / part_ml / counters.
// Runs before any stream work, so a refused call leaves nothing queued.
static int attn_gqa_validate(const tfb_attn_gqa_args* a, bool own_scratch) {
    TFB_REQUIRE(a && a->qkv && a->pos && a->k_pool && a->v_pool && a->block_table && a->out, TFB_EINVAL);
    TFB_REQUIRE(!own_scratch || (a->part_o && a->part_ml && a->counters), TFB_EINVAL);
    TFB_REQUIRE(a->hq > 0 && a->hkv > 0 && a->hkv <= a->hq && a->hq % a->hkv == 0, TFB_EINVAL);
    TFB_REQUIRE(a->d == 64 || a->d == 128, TFB_EINVAL);
    TFB_REQUIRE(a->rotary_dim >= 0 && a->rotary_dim <= a->d && a->rotary_dim % 64 == 0, TFB_EINVAL);
    TFB_REQUIRE(a->rotary_dim == 0 || (a->cos_table && a->sin_table), TFB_EINVAL);
    TFB_REQUIRE(a->page_size > 0 && a->table_len > 0 && a->max_ctx > 0, TFB_EINVAL);
    TFB_REQUIRE(a->norm_mode == TFB_NORM_NONE || a->norm_mode == TFB_NORM_CAST_THEN_GAIN, TFB_EINVAL);
    TFB_REQUIRE(a->norm_mode == TFB_NORM_NONE || (a->gamma_q && a->gamma_k), TFB_EINVAL);
    TFB_REQUIRE((long long)a->page_size * a->table_len >= a->max_ctx, TFB_ECAPACITY);
    TFB_REQUIRE(a->rotary_dim == 0 || a->max_pos >= a->max_ctx, TFB_ECAPACITY);
    TFB_REQUIRE(aligned16(a->k_pool) && aligned16(a->v_pool) && aligned16(a->qkv), TFB_EALIGN);
    TFB_REQUIRE(a->chunk >= 0 && a->chunk <= 2 && (a->chunk == 0 || a->batch > 1), TFB_EINVAL);
    TFB_REQUIRE(a->batch <= 65535, TFB_EINVAL);
    const int G = a->hq / a->hkv;
    TFB_REQUIRE(G == 1 || G == 2 || (G == 4 && a->d == 128), TFB_EINVAL);
    return TFB_OK;
}

static int attn_gqa_run(const tfb_attn_gqa_args* a, tfb_stream_t stream) {
    tfb::AttnParams p;
    p.qkv = static_cast<const uint16_t*>(a->qkv);
    p.gamma_q = static_cast<const uint16_t*>(a->gamma_q);
    p.gamma_k = static_cast<const uint16_t*>(a->gamma_k);
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
    p.hq = a->hq;
    p.hkv = a->hkv;
    p.d = a->d;
    p.rotary_dim = a->rotary_dim;
    p.page_size = a->page_size;
    p.max_ctx = a->max_ctx;
    p.nsplit = tfb::attn_splits(a->max_ctx);
    p.eps = a->eps;
    p.scale = a->scale;
    p.norm_mode = a->norm_mode;
    p.prefetch = a->prefetch;
    p.prefetch_bytes = a->prefetch_bytes;
    p.trace = next_trace();
    p.batch = a->batch > 1 ? a->batch : 1;
    p.qkv_stride = (a->hq + 2 * a->hkv) * a->d;
    p.out_stride = a->hq * a->d;
    p.bt_stride = a->chunk ? 0 : a->table_len;
    p.append_only = a->chunk;
    return done(tfb::attn_gqa_dispatch(p, S(stream), a->pdl != 0));
}

int tfb_attn_gqa_decode(const tfb_attn_gqa_args* a, tfb_stream_t stream) {
    const int v = attn_gqa_validate(a, true);
    return v != TFB_OK ? v : attn_gqa_run(a, stream);
}

int tfb_attn_gqa_decode_noalloc(const tfb_attn_gqa_args* a, tfb_stream_t stream) {
    const int v = attn_gqa_validate(a, false);               // everything is checked before any stream work
    if (v != TFB_OK) return v;
    TFB_REQUIRE(a->batch <= 1, TFB_ECAPACITY);               // the built-in scratch holds one sequence
    tfb_attn_gqa_args b = *a;
    bool fits = false;
    const cudaError_t e = tfb::attn_static_scratch(a->hq, tfb::attn_splits(a->max_ctx), a->d, &b.part_o, &b.part_ml,
                                                   &b.counters, &fits);
    if (e != cudaSuccess) return fail_launch(e);
    if (!fits) {
        std::snprintf(g_last_error, sizeof g_last_error,
                      "tfb_attn_gqa_decode_noalloc: %d heads x %d splits x %d dims exceeds the built-in scratch "
                      "(64 heads, 64 splits = 4096 positions, 128 dims)", a->hq, tfb::attn_splits(a->max_ctx), a->d);
        return TFB_ECAPACITY;
    }
    // the merge tickets must start at zero; everything else is written before it is read
    // (hkv <= hq <= 64 was checked above: the ticket region of the array holds 64 words)
    const cudaError_t m = cudaMemsetAsync(b.counters, 0, size_t(a->hkv) * sizeof(uint32_t), S(stream));
    if (m != cudaSuccess) return fail_launch(m);
    return attn_gqa_run(&b, stream);
}

int32_t tfb_qwen3_step_sync_words(int32_t n_layers, int32_t hkv) {
    return n_layers > 0 && hkv > 0 ? tfb::fused_step_sync_words(n_layers, hkv) : 0;
}
int64_t tfb_qwen3_step_xbuf_words(int32_t hidden, int32_t hq, int32_t hkv, int32_t d, int32_t inter) {
    return hidden > 0 && hq > 0 && hkv > 0 && d > 0 && inter > 0 ? tfb::fused_step_xbuf_words(hidden, hq, hkv, d, inter) : 0;
}
int32_t tfb_qwen3_step_splits(int32_t hkv) { return hkv > 0 ? tfb::fused_step_splits(hkv) : 0; }

// TFB_KERNEL_FUSED: the whole step as one cooperative launch.
static int qwen3_fused_step(const tfb_qwen3_step_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a->step_layers && a->step_sync && a->step_status && a->step_xbuf, TFB_EINVAL);
    TFB_REQUIRE(a->vocab > 0 && a->vocab < (1ll << 31), TFB_EINVAL);
    tfb::FusedParams p;
    std::memset(&p, 0, sizeof p);
    p.layers = static_cast<const tfb::FusedLayer*>(a->step_layers);
    p.n_layers = a->n_layers; p.hidden = a->hidden; p.hq = a->hq; p.hkv = a->hkv; p.d = a->d; p.inter = a->inter;
    p.vocab = int(a->vocab); p.eps = a->eps; p.scale = a->scale;
    p.w_embed = static_cast<const uint16_t*>(a->w_embed);
    p.gamma_final = static_cast<const uint16_t*>(a->gamma_final);
    p.w_head = static_cast<const uint16_t*>(a->w_head);
    p.cos_table = static_cast<const uint16_t*>(a->cos_table);
    p.sin_table = static_cast<const uint16_t*>(a->sin_table);
    p.page_size = a->page_size; p.max_ctx = a->max_ctx; p.block_table = a->block_table;
    p.tokens = reinterpret_cast<long long*>(a->tokens); p.pos = a->pos;
    p.n_prompt = a->n_prompt; p.max_tokens = a->max_tokens;
    p.logits = static_cast<uint16_t*>(a->logits);
    p.xbuf = a->step_xbuf;
    p.part_o = a->part_o; p.part_ml = a->part_ml;
    p.sync = a->step_sync; p.status = a->step_status;
    p.head_val = a->head_val; p.head_idx = a->head_idx;
    p.picked = reinterpret_cast<long long*>(a->picked);
    p.temperature = a->temperature > 0.f ? a->temperature : 0.f;
    p.seed = a->seed;
    p.hidden_trace = static_cast<uint16_t*>(a->hidden_trace);
    TFB_REQUIRE(a->n_eos >= 0 && a->n_eos <= 16 && (a->eos_ids == nullptr || (a->stop_at && a->n_eos > 0)), TFB_EINVAL);
    p.eos_ids = reinterpret_cast<const long long*>(a->eos_ids);
    p.n_eos = a->eos_ids ? a->n_eos : 0;
    p.stop_at = a->stop_at;
    p.timeline = g_trace_buf;                                              // tfb_debug_trace, else nullptr
    p.timeline_slots = g_trace_cap;
    TFB_REQUIRE(a->cos_table && a->sin_table && a->block_table, TFB_EINVAL);
    TFB_REQUIRE(tfb::fused_step_supported(p), TFB_EINVAL);
    return done(tfb::fused_step_launch(p, S(stream)));
}

int tfb_qwen3_decode_step(const tfb_qwen3_step_args* a, tfb_stream_t stream) {
    TFB_REQUIRE(a && a->layers && a->n_layers > 0, TFB_EINVAL);
    TFB_REQUIRE(a->w_embed && a->gamma_final && a->w_head && a->tokens && a->pos, TFB_EINVAL);
    TFB_REQUIRE(a->hidden_buf && a->qkv_buf && a->attn_buf && a->act_buf, TFB_EINVAL);
    TFB_REQUIRE(a->part_o && a->part_ml && a->counters && a->head_val && a->head_idx, TFB_EINVAL);
    TFB_REQUIRE(a->hidden % 256 == 0 && a->inter % 256 == 0 && (a->hq * a->d) % 256 == 0, TFB_EINVAL);
    TFB_REQUIRE((long long)a->page_size * a->table_len >= a->max_ctx, TFB_ECAPACITY);
    TFB_REQUIRE(a->max_pos >= a->max_ctx && a->max_tokens <= a->max_ctx + 1, TFB_ECAPACITY);
    if (a->kernel == TFB_KERNEL_FUSED) return qwen3_fused_step(a, stream);
    const bool pdl = a->pdl != 0;
    const bool pf = (a->l2_prefetch & 2) != 0;
    const int spf = a->l2_prefetch & 1;
    const int H = a->hidden, QP = a->hq * a->d, KVP = a->hkv * a->d, I = a->inter;
    const int NQKV = QP + 2 * KVP;
    cudaStream_t st = S(stream);
    uint16_t* hid = static_cast<uint16_t*>(a->hidden_buf);
    uint16_t* trace = static_cast<uint16_t*>(a->hidden_trace);

    // The step's first launch carries no programmatic dependency: it starts only when the previous step has
    // fully finished, so kernels of this step may read last step's state and position before their own wait.
    cudaError_t e = tfb::embed_launch(static_cast<const uint16_t*>(a->w_embed), nullptr,
                                      reinterpret_cast<const long long*>(a->tokens), a->pos, hid, 1, H,
                                      a->vocab, 1.f, st, false);
    if (e != cudaSuccess) return fail_launch(e);

    for (int l = 0; l < a->n_layers; ++l) {
        const tfb_qwen3_layer& L = a->layers[l];
        const tfb_qwen3_layer* next = (l + 1 < a->n_layers) ? &a->layers[l + 1] : nullptr;
        tfb_gemv_args g;
        // 1. input norm + q|k|v projection
        std::memset(&g, 0, sizeof g);
        g.w = L.w_qkv; g.x = hid; g.gamma = L.gamma_in; g.y = a->qkv_buf;
        g.n = NQKV; g.k = H; g.prologue = TFB_NORM_CAST_THEN_GAIN; g.epilogue = TFB_EPI_STORE;
        g.eps = a->eps; g.x_scale = 1.f; g.res_scale = 1.f; g.out_scale = 1.f; g.pdl = pdl; g.kernel = a->kernel; g.self_prefetch = spf;
        if (pf) { g.prefetch = L.w_o; g.prefetch_bytes = 2ull * H * QP; }
        const bool qkv_done = l > 0 && a->kernel == TFB_KERNEL_CHAIN && a->chain_sync != nullptr && !trace;
        if (a->kernel == TFB_KERNEL_CHAIN) g.kernel = TFB_KERNEL_AUTO;
        int rc = qkv_done ? TFB_OK : gemv_checked(&g, stream);
        if (rc) return rc;
        // 2. q/k norm, RoPE, KV append, attention
        tfb_attn_gqa_args t;
        std::memset(&t, 0, sizeof t);
        t.qkv = a->qkv_buf; t.gamma_q = L.gamma_q; t.gamma_k = L.gamma_k;
        t.cos_table = a->cos_table; t.sin_table = a->sin_table; t.pos = a->pos;
        t.k_pool = L.k_pool; t.v_pool = L.v_pool; t.block_table = a->block_table; t.out = a->attn_buf;
        t.part_o = a->part_o; t.part_ml = a->part_ml; t.counters = a->counters;
        t.hq = a->hq; t.hkv = a->hkv; t.d = a->d; t.rotary_dim = a->d;
        t.page_size = a->page_size; t.table_len = a->table_len; t.max_ctx = a->max_ctx; t.max_pos = a->max_pos;
        t.eps = a->eps; t.scale = a->scale; t.norm_mode = TFB_NORM_CAST_THEN_GAIN; t.pdl = pdl;
        if (pf) { t.prefetch = L.w_gate; t.prefetch_bytes = 2ull * I * H; }
        rc = tfb_attn_gqa_decode(&t, stream);
        if (rc) return rc;
        const bool chain = a->kernel == TFB_KERNEL_CHAIN && a->chain_sync != nullptr;
        tfb_gemv_chain_args ch;
        if (chain) std::memset(&ch, 0, sizeof ch);
        auto emit = [&](const tfb_gemv_args& x) -> int {        // one launch, or the next phase of the chain
            if (!chain) return gemv_checked(&x, stream);
            ch.phase[ch.n_phases] = x;
            ch.phase[ch.n_phases++].kernel = TFB_KERNEL_AUTO;
            return TFB_OK;
        };
        // 3. output projection + residual
        std::memset(&g, 0, sizeof g);
        g.w = L.w_o; g.x = a->attn_buf; g.residual = hid; g.y = hid;
        g.n = H; g.k = QP; g.prologue = TFB_NORM_NONE; g.epilogue = TFB_EPI_RESIDUAL;
        g.eps = a->eps; g.x_scale = 1.f; g.res_scale = 1.f; g.out_scale = 1.f; g.pdl = pdl; g.kernel = a->kernel; g.self_prefetch = spf;
        if (pf) { g.prefetch = L.w_up; g.prefetch_bytes = 2ull * I * H; }
        rc = emit(g);
        if (rc) return rc;
        // 4. post-attention norm + gate/up + SwiGLU
        std::memset(&g, 0, sizeof g);
        g.w = L.w_gate; g.w2 = L.w_up; g.x = hid; g.gamma = L.gamma_post; g.y = a->act_buf;
        g.n = I; g.k = H; g.prologue = TFB_NORM_CAST_THEN_GAIN; g.epilogue = TFB_EPI_SWIGLU;
        g.eps = a->eps; g.x_scale = 1.f; g.res_scale = 1.f; g.out_scale = 1.f; g.pdl = pdl; g.kernel = a->kernel; g.self_prefetch = spf;
        if (pf) { g.prefetch = L.w_down; g.prefetch_bytes = 2ull * I * H; }
        rc = emit(g);
        if (rc) return rc;
        // 5. down projection + residual
        std::memset(&g, 0, sizeof g);
        g.w = L.w_down; g.x = a->act_buf; g.residual = hid; g.y = hid;
        g.n = H; g.k = I; g.prologue = TFB_NORM_NONE; g.epilogue = TFB_EPI_RESIDUAL;
        g.eps = a->eps; g.x_scale = 1.f; g.res_scale = 1.f; g.out_scale = 1.f; g.pdl = pdl; g.kernel = a->kernel; g.self_prefetch = spf;
        if (pf && next) { g.prefetch = next->w_qkv; g.prefetch_bytes = 2ull * NQKV * H; }
        rc = emit(g);
        if (rc) return rc;
        if (chain) {
            if (next && !trace) {                              // the next layer's q|k|v reads what `down` just wrote
                std::memset(&g, 0, sizeof g);
                g.w = next->w_qkv; g.x = hid; g.gamma = next->gamma_in; g.y = a->qkv_buf;
                g.n = NQKV; g.k = H; g.prologue = TFB_NORM_CAST_THEN_GAIN; g.epilogue = TFB_EPI_STORE;
                g.eps = a->eps; g.x_scale = 1.f; g.res_scale = 1.f; g.out_scale = 1.f;
                ch.phase[ch.n_phases++] = g;
            }
            ch.pdl = pdl; ch.sync = a->chain_sync;
            rc = tfb_gemv_chain(&ch, stream);
            if (rc) return rc;
        }
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
    h.scratch_val = a->head_val; h.scratch_idx = a->head_idx; h.counter = a->counters + a->hkv;
    h.n = int(a->vocab); h.k = H; h.prologue = TFB_NORM_CAST_THEN_GAIN; h.eps = a->eps;
    h.x_scale = 1.f; h.out_scale = 1.f; h.pdl = pdl; h.kernel = a->kernel; h.self_prefetch = spf;
    h.token_out = a->picked;
    h.tokens = a->tokens; h.pos = a->pos; h.n_prompt = a->n_prompt; h.max_tokens = a->max_tokens;
    h.temperature = a->temperature; h.seed = a->seed;
    h.eos_ids = a->eos_ids; h.n_eos = a->n_eos; h.stop_at = a->stop_at;
    return tfb_lm_head_argmax(&h, stream);
}

}  // extern "C"
