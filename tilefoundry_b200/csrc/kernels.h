// Internal interface between the kernel translation units and the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tfb {

struct GemvParams {
    const uint4* w;
    const uint4* w2;
    const uint16_t* x;
    const uint16_t* gamma;
    const uint16_t* residual;
    void* y;
    int n, k;
    float eps, x_scale, res_scale, out_scale;
    const void* prefetch;
    unsigned long long prefetch_bytes;
    unsigned long long* trace;
    const uint16_t* x2;              // gate vector of the gated-norm prologue (mode 3)
    const long long* expert_idx;     // expert mode: expert of each slot of rows_per_expert output rows
    int rows_per_expert;
    int expert_rank, expert_world;   // expert e lives on rank e % world as local expert e / world (world <= 1: all local)
    // streaming kernel only
    int kc, nstages, self_prefetch;
    unsigned* status;
    // lm_head mode (epilogue 4) of the streaming kernel
    float* scratch_val;
    int* scratch_idx;
    unsigned* counter;
    long long* token_out;
    long long* tokens;
    int* pos;
    int n_prompt, max_tokens;
};
bool gemv_stream_supported(int n, int k);
cudaError_t gemv_stream_dispatch(const GemvParams& p, int norm_mode, int epi, cudaStream_t stream, bool pdl);
int lm_head_stream_ctas();
cudaError_t gemv_dispatch(const GemvParams& p, int norm_mode, int epi, cudaStream_t stream, bool pdl);
cudaError_t gemv_pair_dispatch(const GemvParams& a, const GemvParams& b, int norm_mode, int epi, cudaStream_t stream, bool pdl);
bool gemv_async_supported(const GemvParams& p, int norm_mode, int epi);
cudaError_t gemv_async_dispatch(const GemvParams& p, int norm_mode, int epi, cudaStream_t stream, bool pdl);
bool gemv_persist_supported(const GemvParams& p, int norm_mode);
cudaError_t gemv_persist_dispatch(const GemvParams& p, int norm_mode, int epi, cudaStream_t stream, bool pdl);

struct AttnParams {
    const uint16_t* qkv;
    const uint16_t* gamma_q;
    const uint16_t* gamma_k;
    const uint16_t* cos_table;
    const uint16_t* sin_table;
    const int* pos;
    const int* rope_pos;
    uint16_t* k_pool;
    uint16_t* v_pool;
    const int* block_table;
    uint16_t* out;
    uint16_t* k_new_out;
    uint16_t* v_new_out;
    float* part_o;
    float* part_ml;
    unsigned* counters;
    int hq, hkv, d, rotary_dim, page_size, max_ctx, nsplit;
    float eps, scale;
    int norm_mode;
    const void* prefetch;
    unsigned long long prefetch_bytes;
    unsigned long long* trace;
    // several sequences in one launch (blockIdx.z = sequence): element strides of qkv / out, row stride of the
    // block table; pos, rope_pos and the split scratch are indexed by sequence.  batch <= 1: one sequence.
    int batch, qkv_stride, out_stride, bt_stride;
    int append_only;             // batch form: 1 = only write each entry's new K/V row into the cache, 2 = attend without writing it
};
int attn_splits(int max_ctx);
cudaError_t attn_gqa_dispatch(const AttnParams& p, cudaStream_t stream, bool pdl);
// Scratch pointers inside the library's own static device array (no allocation); *fits = false when
// the shape is beyond its fixed capacity.
cudaError_t attn_static_scratch(int hq, int nsplit, int d, float** part_o, float** part_ml, unsigned** counters,
                                bool* fits);

struct HeadParams {
    const uint4* w;
    const uint16_t* x;
    const uint16_t* gamma;
    uint16_t* logits;
    long long* token_out;
    float* scratch_val;
    int* scratch_idx;
    unsigned* counter;
    int n, k;
    float eps, x_scale, out_scale;
    long long* tokens;
    int* pos;
    int n_prompt, max_tokens;
    unsigned long long* trace;
    float* pair_out;            // optional f32[2]: (best logit, index + index_offset) instead of the token update
    int index_offset;
    float temperature;          // > 0: Gumbel-max sample from softmax(logits / temperature); else greedy
    unsigned long long seed;
    const long long* eos_ids;   // end-of-sequence latch (nullptr: none): see tfb_lm_head_args
    int n_eos;
    int* stop_at;
};
struct TopPParams {
    const uint16_t* logits;     // bf16 [vocab]: the logits the step before kept
    int vocab;
    float temperature, top_p;
    unsigned long long seed;
    const int* pos;             // the position after that step
    const int* prev_pos;        // ... and before it
    long long* tokens;
    int n_prompt;
    long long* picked;          // optional
    float* threshold_out;       // optional: the smallest logit value inside the nucleus
    const long long* eos_ids;
    int n_eos;
    int* stop_at;
    int* hist;                  // scratch i32 [65664], zero between calls: value histogram, tickets, largest / threshold key, CTA picks
};
cudaError_t sample_top_p_launch(const TopPParams& p, cudaStream_t stream, bool pdl);
int lm_head_ctas(int n);
cudaError_t lm_head_dispatch(const HeadParams& p, int norm_mode, cudaStream_t stream, bool pdl);

cudaError_t embed_launch(const uint16_t* table, const long long* ids, const long long* ids_base,
                         const int* pos, uint16_t* out, int rows, int hidden, long long vocab,
                         float scale, cudaStream_t stream, bool pdl);
cudaError_t rmsnorm_launch(const uint16_t* x, const uint16_t* gamma, uint16_t* y, int rows, int width,
                           float eps, int mode, cudaStream_t stream, bool pdl);
cudaError_t copy_launch(const void* src, void* dst, int bytes, cudaStream_t stream, bool pdl);
cudaError_t moe_finalize_launch(const float* partial, const uint16_t* residual, uint16_t* out, int hidden,
                                float res_scale, bool has_shared, cudaStream_t stream, bool pdl);
cudaError_t pick_finalize_launch(const float* pairs, int world, long long* tokens, int* pos, int n_prompt,
                                 int max_tokens, long long* picked, cudaStream_t stream, bool pdl);
cudaError_t residual_add_launch(const uint16_t* a, const uint16_t* b, uint16_t* out, int n, float scale,
                                cudaStream_t stream, bool pdl);

struct MlaParams {
    const uint16_t* q_up;      // [heads][nope+rope]
    const uint16_t* kv_up;     // [heads][nope+v]
    const uint16_t* k_rope;    // [rope] shared rotary key slice
    const uint16_t* cos_table;
    const uint16_t* sin_table;
    const int* pos;
    const int* rope_pos;
    uint16_t* k_pool;          // [page][slot][heads][nope+rope]
    uint16_t* v_pool;          // [page][slot][heads][v]
    const int* block_table;
    uint16_t* out;             // [heads][v]
    uint16_t* k_new_out;
    uint16_t* v_new_out;
    float* part_o;
    float* part_ml;
    unsigned* counters;        // [heads]
    int heads, nope, rope, vd, page_size, max_ctx, nsplit;
    float scale;
    unsigned long long* trace;
};
// Latent-cache form (attn_mla_latent.cu): pool rows are [kv_lora | rope] per position.
struct MlaLatentParams {
    const uint16_t* qkv_a;       // [q_lora | kv_lora | rope]: the fused down-projection of this token
    const uint16_t* gamma_q_a;   // [q_lora]
    const uint16_t* gamma_kv_a;  // [kv_lora]
    const uint16_t* w_q_b;       // [heads*(nope+rope)][q_lora]
    const uint16_t* w_kv_b;      // [heads*(nope+v)][kv_lora]: k_nope rows then v rows per head
    const uint16_t* cos_table;
    const uint16_t* sin_table;
    const int* pos;
    const int* rope_pos;
    uint16_t* pool;              // [page][slot][kv_lora + rope]
    const int* block_table;
    float* q_lat;                // [heads][2][kv_lora] scratch
    float* q_rope;               // [heads][rope] scratch
    float* part_o;               // [heads][nsplit][kv_lora]
    float* part_ml;              // [heads][nsplit][2]
    uint16_t* out;               // [heads][v]
    uint16_t* latent_new_out;    // optional [kv_lora + rope]
    int heads, q_lora, page_size, max_ctx, nsplit;
    int no_early_rows;           // 1: fetch no cache row ahead of the dependency wait (rows may still be in flight)
    int tokens, qkv_stride;      // tokens of one sequence in this launch (prompt chunk; 0 or 1: one) and elements between their qkv_a rows
    float scale, lora_eps;
    unsigned long long* trace;   // debug timeline record of the launch this copy of the parameters goes to
    unsigned long long* trace3[3];
};
int mla_latent_splits(int max_ctx);
bool mla_latent_supported(int heads, int q_lora, int kv_lora, int nope, int rope, int vd, int max_ctx);
cudaError_t mla_latent_dispatch(const MlaLatentParams& p, cudaStream_t stream, bool pdl);
int mla_splits(int max_ctx);
cudaError_t attn_mla_dispatch(const MlaParams& p, cudaStream_t stream, bool pdl);


struct ConvParams {
    const uint16_t* entry;      // [channels] this token's column
    const uint16_t* state_in;   // [channels][width-1]
    uint16_t* state_out;        // may alias state_in
    const uint16_t* conv_w;     // [channels][width]
    const uint16_t* conv_b;     // [channels] or null
    uint16_t* mixed;            // [channels]
    uint16_t* entry_out;        // optional copy of the entry
    int channels, kernel_width;
};
cudaError_t conv_step_launch(const ConvParams& p, cudaStream_t stream, bool pdl);

struct SsmParams {
    const float* state_in;      // [nh][pd][ns] f32
    float* state_out;           // may alias state_in
    const uint16_t* x;          // [nh*pd]
    const uint16_t* b_vec;      // [ng][ns]
    const uint16_t* c_vec;      // [ng][ns]
    const uint16_t* dt_raw;     // [nh]
    const uint16_t* a_log;
    const uint16_t* dt_bias;
    const uint16_t* d_skip;
    uint16_t* y;                // [nh*pd]
    int nh, pd, ns, ng;
};
cudaError_t ssm_step_launch(const SsmParams& p, cudaStream_t stream, bool pdl);

struct RouterParams {
    const uint16_t* logits_bf16;
    const float* logits_f32;
    long long* indices;         // [top_k]
    uint16_t* weights_bf16;
    float* weights_f32;
    int experts, top_k, mode;
    // optional: ask L2 for the selected experts' weights (the kernels that read them cannot know the indices before
    // their own dependency wait, and HBM idles while this one-warp kernel runs)
    const void* slab[4];             // [experts][slab_bytes[i]] each
    unsigned long long slab_bytes[4];
    int n_slabs, expert_rank, expert_world;
};
cudaError_t router_select_launch(const RouterParams& p, cudaStream_t stream, bool pdl);

struct MoeDownParams {
    const uint4* w_down;        // [experts][hidden][inter]
    const uint4* w_shared;      // [hidden][shared_inter] or null
    const uint16_t* inner;      // [top_k][inter]
    const uint16_t* shared_act; // [shared_inter]
    const long long* indices;
    const uint16_t* weights;    // [top_k] bf16
    const float* shared_gate;   // optional scalar
    const uint16_t* residual;   // optional [hidden]
    uint16_t* out;              // [hidden]
    int hidden, inter, shared_inter, top_k;
    float res_scale;
    int expert_rank, expert_world;
    float* partial;             // optional f32 [2][hidden]: un-rounded routed sum and shared dot of this rank
};
cudaError_t moe_down_launch(const MoeDownParams& p, cudaStream_t stream, bool pdl);

// ---- f32-activation family (Qwen3.5) ----
struct GemvF32Params {
    const uint4* w;
    const uint4* w2;
    const uint4* w_extra;            // expert mode: rows of the slots past the routed ones (the shared expert)
    const uint4* w2_extra;
    const float* x;
    const float* gamma;
    const float* gate;               // prologue 4: the vector whose silu multiplies the normalised x
    const float* residual;
    float* y;
    int n, k, seg;
    float eps;
    const long long* expert_idx;
    int rows_per_expert, routed_slots;
    unsigned long long* trace;
    int expert_rank, expert_world;   // expert mode: expert e lives on rank e % world as local expert e / world
    // router launch (epilogue store, no expert mode), optional: the last CTA selects route_top_k of the first
    // route_experts outputs (softmax over all, top-k, renormalise) into idx_out / w_out
    unsigned* route_counter;         // u32, zero before the first launch; the kernel leaves it zero
    int route_experts, route_top_k;
    long long* idx_out;
    float* w_out;
};
cudaError_t gemv_f32_dispatch(const GemvF32Params& p, int norm_mode, int epi, cudaStream_t stream, bool pdl);

struct GdnParams {
    const float* proj;          // [2*hk*dk + hv*dv] conv entry | [hv*dv] z | [hv] b | [hv] a
    float* conv_state;          // two buffers of [channels][width-1], conv_state_stride floats apart
    size_t conv_state_stride;
    const int* pos;             // parity picks the buffer read; null: read buffer 0, write buffer 1
    const float* conv_w;        // [channels][width]
    const float* a_log;         // [hv]
    const float* dt_bias;       // [hv]
    float* state;               // [hv][dk][dv], updated in place
    float* read;                // [hv*dv]
    int hk, hv, dk, dv, kernel_width;
    float q_scale;
    // optional: q [hv][dk], k [hv][dk], v [hv][dv], g [hv], beta [hv] handed in (conv, norms and scalars skipped)
    const float* direct_q; const float* direct_k; const float* direct_v; const float* direct_g; const float* direct_beta;
};
cudaError_t conv_silu_f32_launch(const float* state, const float* entry, const float* conv_w, float* mixed, int channels,
                                 int width, cudaStream_t stream, bool pdl);
cudaError_t l2norm_f32_launch(const float* x, float* y, int rows, int width, float eps, cudaStream_t stream, bool pdl);
cudaError_t partial_rope_f32_launch(const float* x, const float* cos_table, const float* sin_table, const int* pos,
                                    float* out, int heads, int d, int rd, cudaStream_t stream, bool pdl);
cudaError_t gdn_step_launch(const GdnParams& p, cudaStream_t stream, bool pdl);

struct GatedAttnParams {
    const float* proj;          // [hq][2*d] q|gate per head, then [hkv][d] k, then [hkv][d] v
    const float* gamma_q;
    const float* gamma_k;
    const float* cos_table;     // [max_ctx][rotary_dim]
    const float* sin_table;
    const int* pos;
    const int* rope_pos;
    float* k_pool;              // [page][slot][hkv][d]
    float* v_pool;
    const int* block_table;
    float* out;                 // [hq*d] gated attention output
    float* k_new_out;
    float* v_new_out;
    float* part_o;
    float* part_ml;
    unsigned* counters;
    int hq, hkv, d, rotary_dim, page_size, max_ctx, nsplit;
    float eps, scale;
    unsigned long long* trace;
};
int attn_gated_splits(int max_ctx);
int attn_gated_groups(int hq, int hkv, int d);      // merge tickets the kernel needs
cudaError_t attn_gated_dispatch(const GatedAttnParams& p, cudaStream_t stream, bool pdl);

struct MoeDownF32Params {
    const uint4* w_down;        // [experts][hidden][inter]
    const uint4* w_shared;      // [hidden][shared_inter] or null
    const float* inner;         // [top_k][inter] then [shared_inter]
    const long long* indices;
    const float* weights;       // [top_k]
    const float* shared_gate_logit;
    const float* residual;
    float* out;
    int hidden, inter, shared_inter, top_k;
    int expert_rank, expert_world;   // expert e lives on rank e % world as local expert e / world (world <= 1: all local)
    float* partial;                  // optional f32 [2][hidden]: this rank's routed sum and un-rounded shared dot
};
cudaError_t moe_down_f32_launch(const MoeDownF32Params& p, cudaStream_t stream, bool pdl);

cudaError_t embed_f32_launch(const uint16_t* table, const long long* ids, const long long* tokens, const int* pos,
                             float* out, int rows, int hidden, long long vocab, cudaStream_t stream, bool pdl);
cudaError_t rmsnorm_f32_launch(const float* x, const float* gamma, float* y, int rows, int width, float eps,
                               cudaStream_t stream, bool pdl);
cudaError_t residual_add_f32_launch(const float* a, const float* b, float* out, int n, cudaStream_t stream, bool pdl);

// ---- a chain of dependent projections in one persistent launch (chain.cu) ----
struct ChainPhase {
    const uint4* w;
    const uint4* w2;
    const uint16_t* x;
    const uint16_t* gamma;
    const uint16_t* residual;
    uint16_t* y;
    int n, k, norm, epi;
    int ksplit, si;                  // filled by the launcher: K-slices per row, 256-element iterations per stage
    float eps, x_scale, res_scale;
};
struct ChainParams {
    ChainPhase ph[4];
    int n_phases;
    int kmax, part_floats;           // filled by the launcher
    unsigned* barrier;               // u32[2], zero before the first launch; the kernel leaves it zero
    unsigned* status;                // u32, set non-zero if a bounded wait gave up
};
cudaError_t gemv_chain_launch(ChainParams& p, cudaStream_t stream, bool pdl, size_t* smem_out);

// ---- small-batch projection on tcgen05 tensor cores (gemm_tc.cu) ----
struct TcParams {
    uint16_t* y;                 // bf16 [M][N]
    const uint16_t* residual;    // optional bf16 [M][N]
    unsigned* status;            // u32, set non-zero if a bounded wait gave up
    int M, N, K, ksteps, splits;
    int swiglu;                  // 1: w holds [gate rows; up rows] (2N rows), y[M][N] = bf16(silu(bf16 g)) * bf16 u
    float res_scale;             // with residual: y = residual + bf16(bf16(acc) * res_scale) (1: no multiply)
};
int gemm_tc_splits(int n, int k);
int gemm_tc_splits_swiglu(int n, int k);
cudaError_t gemm_tc_launch(const void* w, const void* x, TcParams p, cudaStream_t stream, bool pdl);

// ---- row-wise kernels of the several-sequence step (batch.cu) ----
cudaError_t embed_rows_launch(const uint16_t* table, const long long* tokens, const int* pos, int max_tokens,
                              uint16_t* out, int rows, int hidden, long long vocab, cudaStream_t stream, bool pdl);
int pick_rows_parts();
cudaError_t pick_rows_launch(const uint16_t* logits, int rows, int vocab, long long* tokens, int* pos, int n_prompt,
                             int max_tokens, long long* picked, float* part_val, int* part_idx, unsigned* tickets,
                             float temperature, unsigned long long seed, cudaStream_t stream, bool pdl);

// ---- mixture-of-experts block for a batch of tokens (moe_grouped.cu) ----
struct MoeBatchParams {
    const float* x;                  // f32 [tokens][hidden]: the block's input (post-attention norm applied)
    const long long* indices;        // [tokens][top_k]
    const float* weights;            // f32 [tokens][top_k]
    const float* shared_gate;        // optional f32 [tokens]: logit of the shared expert's sigmoid gate
    const float* residual;           // optional f32 [tokens][hidden], added to the result
    const uint16_t* w_gate;          // bf16 [experts][inter][hidden]
    const uint16_t* w_up;
    const uint16_t* w_down;          // bf16 [experts][hidden][inter]
    const uint16_t* w_shared_gate;   // optional shared expert, bf16 [inter][hidden] / [hidden][inter]
    const uint16_t* w_shared_up;
    const uint16_t* w_shared_down;
    float* out;                      // f32 [tokens][hidden]
    uint16_t* x_bf16;                // scratch bf16 [tokens][hidden]
    uint16_t* inner;                 // scratch bf16 [tokens][top_k + 1][inter]
    uint16_t* y;                     // scratch bf16 [tokens][top_k + 1][hidden]
    int* counts;                     // scratch i32 [2 * (experts + 1) + 1]: tokens per expert, number of experts with tokens, their ids
    int* lists;                      // scratch i32 [experts + 1][tokens]
    unsigned* status;                // u32, set non-zero if a bounded wait gave up
    int tokens, hidden, inter, experts, top_k;
};
struct MoeRouteParams {
    const float* x;                  // f32 [tokens][hidden]
    const uint16_t* w_router;        // bf16 [experts][hidden]
    const uint16_t* w_shared_scale;  // optional bf16 [hidden]: the row of the shared expert's gate
    float* logits;                   // scratch f32 [tokens][experts + 1]
    long long* indices;              // [tokens][top_k]
    float* weights;                  // f32 [tokens][top_k]
    float* shared_gate;              // optional f32 [tokens]
    int tokens, hidden, experts, top_k, mode;
};
cudaError_t moe_batch_route_launch(const MoeRouteParams& p, cudaStream_t stream, bool pdl);
bool moe_batch_supported(const MoeBatchParams& p);
cudaError_t moe_batch_launch(const MoeBatchParams& p, cudaStream_t stream, bool pdl);

// ---- exchange steps over NVLink peer memory (collective.cu) ----
constexpr int kMaxPeers = 8;
struct PeerReduceParams {
    const float* partial;            // local f32 [2][hidden]: this rank's routed sum and shared dot
    float* inbox[kMaxPeers];         // rank r's inbox (peer pointer): f32 [2 parities][world][2][hidden]
    unsigned* flags[kMaxPeers];      // rank r's flags (peer pointer): u32 [world][ceil(hidden/256)]
    unsigned* epoch;                 // local u32 [ceil(hidden/256)], zero at start
    unsigned* status;                // local u32
    const uint16_t* residual;
    uint16_t* out;
    int hidden, rank, world, has_shared;
    float res_scale;
    // f32 form (Qwen3.5): out_f32 = residual_f32 + sum(routed) + bf16(sum(shared)) * sigmoid(*gate_logit)
    const float* residual_f32;
    float* out_f32;
    const float* gate_logit;
};
cudaError_t moe_allreduce_finalize_launch(const PeerReduceParams& p, cudaStream_t stream, bool pdl);
struct PeerPickParams {
    const float* pair;               // local f32 [2]: (best logit, global index) of this rank's vocabulary slice
    float* inbox[kMaxPeers];         // rank r's inbox: f32 [2 parities][world][2]
    unsigned* flags[kMaxPeers];      // rank r's flags: u32 [world]
    unsigned* epoch;                 // local u32 [1]
    unsigned* status;
    long long* tokens;
    int* pos;
    long long* picked;
    int n_prompt, max_tokens, rank, world;
};
cudaError_t pick_allgather_launch(const PeerPickParams& p, cudaStream_t stream, bool pdl);

// ---- the whole Qwen3-architecture decode step as one cooperative launch (step_fused.cu) ------------------------
constexpr int kFusedMaxLayers = 128;
struct FusedLayer {                      // device-resident table, one entry per layer
    const uint16_t *gamma_in, *w_qkv, *gamma_q, *gamma_k, *w_o, *gamma_post, *w_gate, *w_up, *w_down;
    uint16_t *k_pool, *v_pool;
};
struct FusedParams {
    const FusedLayer* layers;            // device pointer
    int n_layers, hidden, hq, hkv, d, inter, vocab;
    float eps, scale;
    const uint16_t *w_embed, *gamma_final, *w_head, *cos_table, *sin_table;
    int page_size, max_ctx;
    const int* block_table;
    long long* tokens;
    int* pos;
    int n_prompt, max_tokens;
    uint16_t* logits;
    unsigned* xbuf;                      // fused_step_xbuf_words() tagged activation words, zero before the first launch
    float *part_o, *part_ml;             // [hq][fused_step_splits][d], [hq][fused_step_splits][2]
    unsigned* sync;                      // fused_step_sync_words() words, zero before the first launch
    unsigned* status;                    // [1]: non-zero after a wait gave up
    float* head_val;                     // [multiprocessors]
    int* head_idx;
    long long* picked;
    float temperature;                   // > 0: Gumbel-max sample from softmax(logits / temperature); else greedy
    unsigned long long seed;
    uint16_t* hidden_trace;
    const long long* eos_ids;            // end-of-sequence latch (nullptr: none): see tfb_lm_head_args
    int n_eos;
    int* stop_at;
    // debug timeline (nullptr normally): 8 words per phase -- earliest entry, earliest / latest end of the wait,
    // latest end of the phase over all CTAs (%globaltimer); phase 0 = embedding, 1 + 5*layer + {0..4}, then the head
    unsigned long long* timeline;
    int timeline_slots;
};
int fused_step_sync_words(int n_layers, int hkv);
long long fused_step_xbuf_words(int hidden, int hq, int hkv, int d, int inter);
int fused_step_splits(int hkv);
bool fused_step_supported(const FusedParams& p);
cudaError_t fused_step_launch(const FusedParams& p, cudaStream_t stream);

}  // namespace tfb
