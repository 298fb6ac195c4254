/* tfb200 -- C ABI of the B200 decode-step kernel library (libtfb200.so).
 *
 * Every entry point takes raw DEVICE pointers, sizes and a CUDA stream, validates
 * its arguments on the host, enqueues work on that stream and returns a status
 * (TFB_OK = 0).  Nothing here allocates device memory, synchronises or touches
 * torch types; buffers are the caller's.  All matrices are bf16 unless a comment
 * says otherwise.
 *
 * The entry points are what a TileFoundry runtime twin binds in place of its own
 * kernel library: the reference examples call per-function kernel launchers with
 * caller-owned outputs and no allocation or synchronisation
 * (examples/granite_4_0_h_small-cuda/kernels/granite.cu:804-808), selected through
 * @runtime_func bodies (src/tilefoundry/runtime/decorator.py:53-77).  Each
 * declaration cites the authored function or reference kernel it stands in for.
 */
#ifndef TFB200_H
#define TFB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define TFB_API __attribute__((visibility("default")))
#else
#define TFB_API
#endif

typedef void* tfb_stream_t; /* cudaStream_t */

enum {
    TFB_OK = 0,
    TFB_EINVAL = 1,      /* bad size, null pointer, unsupported combination */
    TFB_EALIGN = 2,      /* pointer or row stride not 16-byte aligned */
    TFB_ECAPACITY = 3,   /* position / context exceeds the cache or scratch capacity */
    TFB_ELAUNCH = 4,     /* the CUDA runtime refused the launch */
    TFB_ENODEVICE = 5    /* no sm_100 device is current */
};

TFB_API int tfb_version(void);
TFB_API const char* tfb_status_string(int status);
/* Text of the last CUDA runtime error a launch returned on this thread ("" if none). */
TFB_API const char* tfb_last_error(void);
/* Debug timeline.  While a device buffer of capacity*8 uint64 is registered, each projection,
 * attention and lm_head launch is given the next 8-word record and writes, in %globaltimer ns:
 * [0] earliest CTA start, [1] earliest and [2] latest return from the dependency wait, [3] latest exit,
 * [4..7] latest time any CTA passed each of up to four interior marks.  The caller presets the words to
 * (~0, ~0, 0, 0, 0, 0, 0, 0).  Pass NULL to stop.  Not for production use. */
TFB_API int tfb_debug_trace(void* device_buffer, int32_t capacity);

/* ---- one decode step with the token crossing the host -----------------------
 * What a host-driven generation loop does around the device step, in one call: copy this step's token id from
 * (pinned) host memory into its slot of the device token history, launch a captured step (a cudaGraphExec_t of any of
 * the four decode steps), copy the picked token back to (pinned) host memory and wait for the stream.
 * Stands in for one iteration of the reference's loop, which feeds `input_ids` from the host and reads the argmax
 * back every step: tests/models/orchestrator/causal_lm/generation.py:56-77.
 *   graph_exec: cudaGraphExec_t of the captured step        token_slot: device address of tokens[pos] (int64)
 *   picked:     device address the step writes its pick to (tokens[pos + 1], or the step's `picked` scalar)
 * Returns TFB_ELAUNCH with tfb_last_error() set if a CUDA call fails. */
TFB_API int tfb_graph_step_host(void* graph_exec, void* token_slot, const int64_t* token_in_host, const void* picked,
                                int64_t* token_out_host, tfb_stream_t stream);
/* `steps` such iterations from position `pos`: every step feeds *token_io_host (pinned) into tokens[pos + i], launches
 * the step, reads tokens[pos + i + 1] back into *token_io_host and waits -- the token crosses the host both ways every
 * step, as in the reference's loop -- and appends it to out_host[i] (plain host memory, may be NULL). */
TFB_API int tfb_graph_generate_host(void* graph_exec, void* tokens, int64_t pos, int32_t steps, int64_t* token_io_host,
                                    int64_t* out_host, tfb_stream_t stream);

/* ---- embedding row gather -------------------------------------------------
 * out[r, :] = table[ids[r], :] * scale (scale == 1 copies bits).
 * Stands in for `embed`: tests/models/qwen3_1_7b/model.py:311-318 (scale 1),
 * tests/models/minicpm3_4b/model.py:359 and
 * examples/granite_4_0_h_small-cuda/model.py:615 (scale 12, a bf16 multiply). */
TFB_API int tfb_embed(const void* table, const int64_t* ids, void* out, int32_t rows, int32_t hidden,
              int64_t vocab, float scale, tfb_stream_t stream);

/* ---- RMSNorm --------------------------------------------------------------
 * mode TFB_NORM_F32GAIN: y = bf16(x32 * rsqrt(mean(x32^2)+eps) * gamma32)      (tf.rms_norm,
 *      src/tilefoundry/ir/hir/nn/rms_norm.py:103-110)
 * mode TFB_NORM_CAST_THEN_GAIN: y = bf16(bf16(x32 * rsqrt(..)) * gamma)          (the spelled-out
 *      Qwen3RMSNorm, tests/models/qwen3_1_7b/model.py:127-138, :321-329) */
/* TFB_NORM_GATED (projections only): y = bf16(v * rsqrt(mean(v^2)+eps) * gamma32) with
 * v = f32(x) * silu(f32(x_gate)) -- granite's gated output norm,
 * examples/granite_4_0_h_small-cuda/model.py:223-236. */
enum { TFB_NORM_NONE = 0, TFB_NORM_F32GAIN = 1, TFB_NORM_CAST_THEN_GAIN = 2, TFB_NORM_GATED = 3,
       /* f32-activation family only: */
       TFB_NORM_SEGMENT_GATED = 4, /* per segment of `seg` elements: bf16(x * rsqrt(mean_seg(x^2)+eps) * gamma32[i % seg] * silu(gate[i])) */
       TFB_NORM_F32_INPUT = 5      /* tfb_lm_head_argmax: x and gamma are f32; y = bf16(x * rsqrt(mean(x^2)+eps) * gamma) */ };
TFB_API int tfb_rmsnorm(const void* x, const void* gamma, void* y, int32_t rows, int32_t width, float eps,
                int32_t mode, tfb_stream_t stream);

/* ---- weight-streaming projection (batch-1 GEMV) ----------------------------
 * y = epilogue( W . prologue(x) ),  W stored [n, k] row-major ("out, in": one
 * output's weights contiguous), x a length-k vector.
 *
 * prologue: TFB_NORM_* applied to x with `gamma`/`eps` (fused RMSNorm), then
 *           multiplied by x_scale if x_scale != 1 (bf16 multiply); a NEGATIVE x_scale divides
 *           by its magnitude instead (IEEE division, e.g. -10 for MiniCPM3's hidden / 10).
 * epilogue: TFB_EPI_STORE     y[i] = bf16(acc)
 *           TFB_EPI_RESIDUAL  y[i] = bf16(residual[i] + bf16(bf16(acc) * res_scale))
 *           TFB_EPI_SWIGLU    y[i] = bf16(bf16(silu(bf16(acc_gate))) * bf16(acc_up)), gate rows
 *                             from w, up rows from w2, both [n, k]
 *           TFB_EPI_STORE_F32 y[i] = acc * out_scale (f32 output)
 * Accumulation is f32.  `prefetch`/`prefetch_bytes` name a byte range (the next
 * projection's weights) that this launch asks the L2 to fetch while it runs.
 * pdl != 0 launches with programmatic stream serialisation: the kernel starts its
 * weight loads before the preceding kernel in the stream has finished and waits
 * for it only before reading x / residual.
 *
 * Stands in for the matmuls of self_attention / mlp (tests/models/qwen3_1_7b/
 * model.py:161-172,214-216,231-235) and their fused norms; reference kernels:
 * examples/qwen3_1_7b-tilelang/fast/kernels.py:124-260,
 * examples/granite_4_0_h_small-cuda/kernels/granite.cu:81-157. */
enum { TFB_EPI_STORE = 0, TFB_EPI_RESIDUAL = 1, TFB_EPI_SWIGLU = 2, TFB_EPI_STORE_F32 = 3 };
/* Two implementations compute the same thing: a warp-per-row kernel with direct 128-bit
 * streaming loads (what AUTO picks: it measured faster at every decode shape on B200), and a
 * persistent one-CTA-per-SM kernel that streams weights through a shared-memory ring filled by
 * bulk async copies (cp.async.bulk + mbarrier), kept selectable for A/B measurement. */
enum { TFB_KERNEL_AUTO = 0, TFB_KERNEL_ROWS = 1, TFB_KERNEL_RING = 2,
       TFB_KERNEL_PERSIST = 3, /* grid sized to residency, grid-stride tiles, two weight batches in flight */
       TFB_KERNEL_ASYNC = 4,   /* one CTA per SM, weights land in a shared-memory ring through cp.async */
       TFB_KERNEL_CHAIN = 5,   /* decode steps only: o / gate+up / down (/ next q|k|v) of a layer as ONE persistent launch */
       TFB_KERNEL_FUSED = 6    /* tfb_qwen3_decode_step only: the WHOLE step as one cooperative launch (step_* fields) */ };
typedef struct {
    const void* w;
    const void* w2;
    const void* x;
    const void* gamma;
    const void* residual;
    void* y;
    int32_t n, k;
    int32_t prologue;
    int32_t epilogue;
    float eps, x_scale, res_scale, out_scale;
    const void* prefetch;
    uint64_t prefetch_bytes;
    int32_t pdl;
    int32_t kernel;  /* TFB_KERNEL_AUTO, or force one implementation (for A/B measurement) */
    int32_t self_prefetch; /* streaming kernel: once its ring is full, ask the L2 for the rest of its own rows */
    int32_t rows_per_expert; /* expert mode: output rows come in slots of this many rows ... */
    const int64_t* expert_idx; /* ... and slot s reads the rows of expert expert_idx[s] (device array) from w / w2,
                                  which then hold [experts][rows_per_expert][k]; NULL = plain projection */
    const void* x_gate;    /* [k] bf16 gate vector of TFB_NORM_GATED */
    int32_t expert_rank;   /* expert parallel: with expert_world > 1, w / w2 hold only the experts e with */
    int32_t expert_world;  /* e % expert_world == expert_rank, as local expert e / expert_world; other slots give 0 */
} tfb_gemv_args;
TFB_API int tfb_gemv(const tfb_gemv_args* args, tfb_stream_t stream);
/* Two independent TFB_EPI_STORE projections (same prologue kind, k <= 2048 each) in one launch: MiniCPM3's q and kv
 * up-projections, which the reference also runs as one "pair" kernel (examples/minicpm3_4b-cutedsl/kernels/
 * reference_ops.py rmsnorm_gemv_pair).  Same results as two tfb_gemv calls. */
TFB_API int tfb_gemv_pair(const tfb_gemv_args* a, const tfb_gemv_args* b, tfb_stream_t stream);

/* ---- lm_head + greedy pick -------------------------------------------------
 * logits[i] = bf16( W[i,:] . prologue(x) * out_scale ), token = argmax over the bf16
 * logits with the lowest index winning ties (torch.argmax), all in one launch.
 * scratch_val/scratch_idx hold one (max, index) pair per CTA; `counter` is a
 * zero-initialised uint32 the kernel returns to zero.  Capacity needed:
 * tfb_lm_head_scratch_entries(n).  `logits` may be NULL to skip the store.
 * Stands in for lm_head + greedy: tests/models/qwen3_1_7b/model.py:332-336,
 * tests/models/orchestrator/causal_lm/generation.py:24-26; reference kernel
 * examples/qwen3_1_7b-tilelang/fast/kernels.py:261-328. */
typedef struct {
    const void* w;          /* [n, k] */
    const void* x;          /* [k] bf16 */
    const void* gamma;      /* [k] or NULL */
    void* logits;           /* [n] bf16 or NULL */
    int64_t* token_out;     /* [1] */
    float* scratch_val;
    int32_t* scratch_idx;
    uint32_t* counter;
    int32_t n, k;
    int32_t prologue;
    float eps, x_scale, out_scale;
    int32_t pdl;
    /* optional generation bookkeeping done by the same launch (all may be NULL):
     * tokens[pos+1] = (pos+1 < n_prompt) ? tokens[pos+1] : token;  pos += 1 */
    int64_t* tokens;
    int32_t* pos;
    int32_t n_prompt;
    int32_t max_tokens;
    int32_t kernel;         /* TFB_KERNEL_* */
    int32_t self_prefetch;  /* as in tfb_gemv_args */
    int32_t index_offset;   /* vocabulary parallel: w is rows [index_offset, index_offset + n) of the head */
    float* pair_out;        /* optional f32[2]: (best logit, global index) for an all-gather; suppresses the
                               token / position update, which tfb_pick_finalize then does */
    /* temperature > 0: the token is a draw from softmax(logits / temperature) by the Gumbel-max rule
     * (argmax of logit / T - log(-log u)), u from a counter-based generator keyed by (seed, *pos or 0, global
     * vocabulary index): reproducible, and the same token on any number of vocabulary shards.  With pair_out the
     * pair's value is the perturbed score.  temperature <= 0: greedy.  Not with TFB_KERNEL_RING (falls back to the
     * default kernel).  On-device sampling as in examples/granite_4_0_h_small-cuda/kernels/granite.cu:712-797
     * (own generator: the draw is keyed by the vocabulary index, not by a launch geometry). */
    float temperature;
    uint64_t seed;
    /* end-of-sequence latch, optional (eos_ids may be NULL): when the token this step picks is a NEW token (its slot
     * is past the prompt) and is one of eos_ids[0..n_eos), *stop_at becomes that slot's index in `tokens`; while
     * *stop_at != 0 a step leaves tokens and *pos untouched, so a caller may replay a fixed number of steps and
     * read where the sequence ended once, afterwards.  stop_at: int32[1], zeroed before a sequence starts.
     * Stands in for the `if token in eos: break` of tests/models/orchestrator/causal_lm/generation.py:70-72. */
    const int64_t* eos_ids;
    int32_t* stop_at;
    int32_t n_eos;
    int32_t reserved_eos;
} tfb_lm_head_args;
TFB_API int32_t tfb_lm_head_scratch_entries(int32_t n);
TFB_API int tfb_lm_head_argmax(const tfb_lm_head_args* args, tfb_stream_t stream);

/* ---- GQA decode attention over a paged KV cache ----------------------------
 * One launch: per-head q/k RMSNorm (optional) -> RoPE on the first rotary_dim
 * dims (rotate-half; 0 = none) -> append this token's K,V at position *pos ->
 * split-KV online-softmax attention over positions [0, *pos] -> merged bf16
 * output [hq*d].  Cache layout per layer: pool[page][slot][hkv][d], page_size
 * slots per page; logical position p lives in page block_table[p / page_size],
 * slot p % page_size.  k_new_out/v_new_out (optional) receive this token's entry
 * [hkv*d] as the authored function returns it.
 * q is scaled as the authored step does: q_s = bf16(q_rope * scale).
 * Scratch: part_o f32 [hq][splits][d], part_ml f32 [hq][splits][2], counters
 * uint32 [hkv] zero-initialised (returned to zero), where
 * splits = tfb_attn_splits(max_ctx).
 * Stands in for self_attention between the projections:
 * tests/models/qwen3_1_7b/model.py:173-213; reference kernels
 * examples/qwen3_1_7b-tilelang/fast/kernels.py:329-547. */
typedef struct {
    const void* qkv;        /* [hq*d | hkv*d | hkv*d] bf16, this token */
    const void* gamma_q;    /* [d] or NULL */
    const void* gamma_k;    /* [d] or NULL */
    const void* cos_table;  /* [max_pos, rotary_dim] bf16 (NULL if rotary_dim == 0) */
    const void* sin_table;
    const int32_t* pos;     /* device scalar: position of this token == prior context length */
    const int32_t* rope_pos;/* device scalar: row of the rotary tables to use; NULL = *pos */
    void* k_pool;
    void* v_pool;
    const int32_t* block_table;
    void* out;              /* [hq*d] bf16 */
    void* k_new_out;        /* optional [hkv*d] */
    void* v_new_out;        /* optional [hkv*d] */
    float* part_o;
    float* part_ml;
    uint32_t* counters;
    int32_t hq, hkv, d, rotary_dim;
    int32_t page_size, table_len, max_ctx, max_pos;
    float eps, scale;
    int32_t norm_mode;      /* TFB_NORM_NONE or TFB_NORM_CAST_THEN_GAIN */
    int32_t pdl;
    const void* prefetch;
    uint64_t prefetch_bytes;
    /* batch > 1: that many independent sequences in one launch.  qkv [batch][(hq+2hkv)*d], out [batch][hq*d],
     * pos (and rope_pos) [batch], block_table [batch][table_len] into the shared pools, k_new_out/v_new_out
     * [batch][hkv*d], part_o/part_ml/counters sized batch times the single-sequence scratch. */
    int32_t batch;
    /* chunk != 0 (with batch > 1): the `batch` entries are consecutive tokens of ONE sequence (prompt processing):
     * pos[i] = pos[0] + i, block_table is that sequence's single row.  A token attends to the rows before it, some of
     * which belong to the same chunk, so the chunk takes two launches: chunk = 1 writes every token's K/V row into the
     * cache and nothing else, chunk = 2 (after it) computes the attention. */
    int32_t chunk;
} tfb_attn_gqa_args;
TFB_API int32_t tfb_attn_splits(int32_t max_ctx);
TFB_API int tfb_attn_gqa_decode(const tfb_attn_gqa_args* args, tfb_stream_t stream);

/* The same attention with NO caller-provided scratch: a->part_o, a->part_ml and a->counters are
 * ignored and the split partials live in a fixed array inside the library image instead.  This
 * entry point has no counterpart in the reference.  It is for callers that cannot allocate device
 * memory themselves: a compiled TileFoundry entry is handed exactly the tensors its ABI declares
 * and nothing else, and a host that drives the step from inside a latency-critical loop cannot
 * afford cudaMalloc's device-wide synchronisation.  It calls no cudaMalloc / cudaFree and no
 * allocating library routine.
 *   Limits: hq <= 64 query heads, max_ctx <= 4096 positions (64 splits), d <= 128; anything larger
 * returns TFB_ECAPACITY with the reason in tfb_last_error.  The array (about 2.1 MB) is held by
 * every GPU that loads the library until the process exits.
 *   The first call on each device looks up the array's device address (one runtime query, no
 * allocation); make that first call before starting any stream capture.
 *   All calls on a device share the one array and it keeps the previous call's contents (the
 * merge tickets are cleared on the stream at the start of every call): two calls whose kernels can
 * overlap on the GPU -- different streams, or graph branches -- race on it.  Serialise them. */
TFB_API int tfb_attn_gqa_decode_noalloc(const tfb_attn_gqa_args* args, tfb_stream_t stream);

/* ---- a whole Qwen3-architecture decode step --------------------------------
 * embed -> layers x [norm+qkv, attention, o+residual, norm+gate/up+SwiGLU,
 * down+residual] -> final norm + lm_head + greedy pick + position advance, enqueued
 * back to back with programmatic dependent launch.  The caller owns every buffer
 * (weights packed [out, in]; w_qkv = q|k|v rows, w_gate / w_up separate).
 * Reads tokens[*pos]; leaves the picked token in tokens[*pos + 1] unless that slot
 * is still inside the prompt, and advances *pos.  Capturable in a CUDA graph.
 * Stands in for Qwen3_1_7B.forward + append_cache + greedy
 * (tests/models/qwen3_1_7b/model.py:338-383); reference driver
 * examples/qwen3_1_7b-tilelang/fast/engine.py:189-271. */
typedef struct {
    const void* gamma_in;
    const void* w_qkv;      /* [(hq+2hkv)*d, hidden] */
    const void* gamma_q;
    const void* gamma_k;
    const void* w_o;        /* [hidden, hq*d] */
    const void* gamma_post;
    const void* w_gate;     /* [inter, hidden] */
    const void* w_up;       /* [inter, hidden] */
    const void* w_down;     /* [hidden, inter] */
    void* k_pool;
    void* v_pool;
} tfb_qwen3_layer;
typedef struct {
    const tfb_qwen3_layer* layers; /* host array [n_layers] */
    int32_t n_layers, hidden, hq, hkv, d, inter;
    int64_t vocab;
    float eps, scale;
    const void* w_embed;    /* [vocab, hidden] */
    const void* gamma_final;
    const void* w_head;     /* [vocab, hidden] (may equal w_embed when tied) */
    const void* cos_table;
    const void* sin_table;
    int32_t max_pos, page_size, table_len, max_ctx;
    const int32_t* block_table;
    int64_t* tokens;
    int32_t* pos;
    int32_t n_prompt, max_tokens;
    /* activations and scratch */
    void* hidden_buf;       /* [hidden] bf16 residual stream */
    void* qkv_buf;          /* [(hq+2hkv)*d] */
    void* attn_buf;         /* [hq*d] */
    void* act_buf;          /* [inter] */
    void* logits;           /* [vocab] bf16 or NULL */
    float* part_o;
    float* part_ml;
    uint32_t* counters;     /* [hkv + 1] zero-initialised: attention + lm_head */
    float* head_val;
    int32_t* head_idx;
    void* hidden_trace;     /* optional [n_layers+1][hidden] bf16: residual stream after each layer, then final-normed */
    int32_t pdl;
    int32_t l2_prefetch;    /* bit 0: each projection prefetches its own remaining rows; bit 1: the next projection's */
    int32_t kernel;         /* TFB_KERNEL_* for every projection of the step */
    int64_t* picked;        /* optional [1]: the token this step picked, whatever the prompt says */
    uint32_t* chain_sync;   /* TFB_KERNEL_CHAIN: u32[4] zeroed once ([0..1] grid barrier, [2] status: non-zero if a wait gave up) */
    float temperature;      /* > 0: sample each token from softmax(logits / temperature) (see tfb_lm_head_args); else greedy */
    uint64_t seed;
    /* TFB_KERNEL_FUSED: the step as ONE cooperative launch, one CTA per multiprocessor; the weight stream runs
     * through a shared-memory ring across all phases and layers; phases hand activations over as tagged 32-bit
     * words (bf16 value + 16-bit tag of launch and phase) that the consumer polls, every wait bounded.  Needs
     * d = 128, hq = 2 hkv, hidden / hq*d / inter multiples of 1024 up to 6144; other shapes get TFB_EINVAL.  The matrix
     * phases run on the tcgen05 tensor cores (K folded into the MMA's N); temperature > 0 samples as the head kernel does.
     *   step_layers: DEVICE copy of the layer table, n_layers x 11 pointers in tfb_qwen3_layer's field order
     *   step_sync:   uint32 [tfb_qwen3_step_sync_words(n_layers, hkv)], zeroed once (words the kernel leaves zero, the
     *                head's arrival count and a launch counter, which it advances)
     *   step_xbuf:   uint32 [tfb_qwen3_step_xbuf_words(hidden, hq, hkv, d, inter)], zeroed once and again whenever
     *                step_sync is zeroed (the tagged activations: hidden | q|k|v | attention | MLP inner)
     *   step_status: uint32 [1], zeroed once; non-zero after a wait gave up (the step's results are then void)
     * and part_o / part_ml sized for tfb_qwen3_step_splits(hkv) splits, head_val / head_idx for one entry per
     * multiprocessor.  No reference counterpart: the reference's fast driver replays about 280 launches per
     * step (examples/qwen3_1_7b-tilelang/fast/engine.py:189-230). */
    const void* step_layers;
    uint32_t* step_sync;
    uint32_t* step_status;
    const int64_t* eos_ids;   /* end-of-sequence latch: see tfb_lm_head_args (NULL: none) */
    int32_t* stop_at;
    int32_t n_eos;
    int32_t reserved_eos;
    uint32_t* step_xbuf;
} tfb_qwen3_step_args;
TFB_API int tfb_qwen3_decode_step(const tfb_qwen3_step_args* args, tfb_stream_t stream);
TFB_API int32_t tfb_qwen3_step_sync_words(int32_t n_layers, int32_t hkv);
TFB_API int64_t tfb_qwen3_step_xbuf_words(int32_t hidden, int32_t hq, int32_t hkv, int32_t d, int32_t inter);
TFB_API int32_t tfb_qwen3_step_splits(int32_t hkv);   /* splits of the context the fused step may use (needs a CUDA device) */

/* ---- multi-head latent attention decode (MiniCPM3) ------------------------------
 * One launch: RoPE on the rotary slice of q and on the shared rotary key slice,
 * key = [k_nope | k_rope] and value assembly per head, append at position *pos, then
 * split-KV softmax attention over positions [0, *pos] of a paged cache of assembled
 * keys pool[page][slot][heads][nope+rope] and values pool[page][slot][heads][v].
 * q_s = bf16(query * scale) as the authored step does.  Scratch as for
 * tfb_attn_gqa_decode with hq = heads, d = v; counters uint32 [heads].
 * Stands in for steps 4-7 of mla_attention: examples/minicpm3_4b-cutedsl/model.py:250-290;
 * reference kernel examples/minicpm3_4b-cutedsl/kernels/cute_attention.py:60-200. */
typedef struct {
    const void* q_up;       /* [heads*(nope+rope)] bf16 */
    const void* kv_up;      /* [heads*(nope+v)] bf16: k_nope | v per head */
    const void* k_rope;     /* [rope] bf16 */
    const void* cos_table;  /* [max_pos, rope] */
    const void* sin_table;
    const int32_t* pos;
    const int32_t* rope_pos;
    void* k_pool;
    void* v_pool;
    const int32_t* block_table;
    void* out;              /* [heads*v] */
    void* k_new_out;        /* optional [heads*(nope+rope)] */
    void* v_new_out;        /* optional [heads*v] */
    float* part_o;
    float* part_ml;
    uint32_t* counters;
    int32_t heads, nope, rope, v;
    int32_t page_size, table_len, max_ctx, max_pos;
    float scale;
    int32_t pdl;
} tfb_attn_mla_args;
TFB_API int tfb_attn_mla_decode(const tfb_attn_mla_args* args, tfb_stream_t stream);

/* ---- multi-head latent attention over a cache of LATENTS ("absorbed" form) -------------------------
 * The cache holds, per position, the normalised compressed kv vector and the rotated shared rotary key:
 * pool[page][slot][kv_lora + rope] bf16 (576 bytes per position per layer for MiniCPM3-4B against 12,800 for
 * assembled keys and values).  W_kv_b is never applied to the cache: its key half is folded into the query
 * (q_lat[h] = W_UK[h]^T bf16(q_nope[h] * scale)) and its value half into the output (out[h] = W_UV[h] sum_t p_t c_t).
 * Three launches: (1) low-rank norm + q_b + absorption / RoPE, and the append of this token's latent row at *pos;
 * (2) split attention of all heads over the shared latent rows; (3) merge + W_UV.  Input is the fused
 * down-projection qkv_a = [q_a | kv_a] of the normalised hidden state; output is what mla_attention feeds to w_o.
 * kv_lora 256, nope 64, rope 32, v 64, heads a multiple of 4, q_lora a multiple of 256 up to 1024.
 * Scratch: q_lat f32 [heads*2*kv_lora], q_rope f32 [heads*rope], part_o f32 [heads*splits*kv_lora],
 * part_ml f32 [heads*splits*2] with splits = tfb_mla_latent_splits(max_ctx); nothing needs zeroing.
 * Same function as tfb_attn_mla_decode plus the two up-projections before it:
 * examples/minicpm3_4b-cutedsl/model.py:214-290 (the reference's kernel keeps the assembled cache,
 * kernels/cute_attention.py:60-200). */
typedef struct {
    const void* qkv_a;        /* [q_lora + kv_lora + rope] bf16 */
    const void* gamma_q_a;
    const void* gamma_kv_a;
    const void* w_q_b;        /* [heads*(nope+rope), q_lora] */
    const void* w_kv_b;       /* [heads*(nope+v), kv_lora] */
    const void* cos_table;    /* [max_pos, rope] */
    const void* sin_table;
    const int32_t* pos;
    const int32_t* rope_pos;  /* optional: rotary position when it differs from *pos */
    void* pool;
    const int32_t* block_table;
    void* out;                /* [heads*v] bf16 */
    void* latent_new_out;     /* optional [kv_lora + rope]: the row appended */
    float* q_lat;
    float* q_rope;
    float* part_o;
    float* part_ml;
    int32_t heads, q_lora, kv_lora, nope, rope, v;
    int32_t page_size, table_len, max_ctx, max_pos;
    float scale, lora_eps;
    int32_t pdl;
    int32_t no_early_rows;    /* 1: fetch no cache row before the dependency wait (set when rows below *pos may have been
                               * written by a launch that is still in the same dependency chain, as in a prompt chunk) */
    /* tokens > 1: a chunk of consecutive tokens of one sequence in the same three launches.  qkv_a is then
     * [tokens][q_lora+kv_lora+rope], pos (and rope_pos) [tokens], out [tokens][heads*v], latent_new_out
     * [tokens][kv_lora+rope], and every scratch buffer tokens times as long; all rows are appended by the first launch,
     * then token t attends to the rows up to pos[t].  no_early_rows must be set.  0 or 1: one token. */
    int32_t tokens, reserved;
} tfb_mla_latent_args;
TFB_API int tfb_mla_latent_decode(const tfb_mla_latent_args* args, tfb_stream_t stream);
TFB_API int32_t tfb_mla_latent_splits(int32_t max_ctx);

#define TFB_MLA_CACHE_ASSEMBLED 0   /* k_pool [..][heads][nope+rope], v_pool [..][heads][v] (the reference's format) */
#define TFB_MLA_CACHE_LATENT 1      /* k_pool [..][kv_lora+rope], v_pool unused */

/* ---- a whole MiniCPM3-architecture decode step ----------------------------------
 * embed*scale_emb -> layers x [norm + (q_a|kv_a), q_b, kv_b, MLA attention, o + scaled
 * residual, norm + gate/up + SwiGLU, down + scaled residual] -> final norm, hidden /
 * logits_scaling, lm_head, greedy pick, position advance.  Weights packed [out, in];
 * w_qkv_a = q_a rows then kv_a rows.  Stands in for MiniCPM3_4B.forward + append_cache
 * + greedy (examples/minicpm3_4b-cutedsl/model.py:396-470). */
typedef struct {
    const void* gamma_in;
    const void* w_qkv_a;    /* [q_lora + kv_lora + rope, hidden] */
    const void* gamma_q_a;
    const void* w_q_b;      /* [heads*(nope+rope), q_lora] */
    const void* gamma_kv_a;
    const void* w_kv_b;     /* [heads*(nope+v), kv_lora] */
    const void* w_o;        /* [hidden, heads*v] */
    const void* gamma_post;
    const void* w_gate;
    const void* w_up;
    const void* w_down;
    void* k_pool;
    void* v_pool;
} tfb_minicpm3_layer;
typedef struct {
    const tfb_minicpm3_layer* layers;
    int32_t n_layers, hidden, heads, q_lora, kv_lora, nope, rope, v, inter;
    int64_t vocab;
    float eps, lora_eps, scale, embed_scale, residual_scale, logits_div;
    const void* w_embed;
    const void* gamma_final;
    const void* w_head;
    const void* cos_table;
    const void* sin_table;
    int32_t max_pos, page_size, table_len, max_ctx;
    const int32_t* block_table;
    int64_t* tokens;
    int32_t* pos;
    int32_t n_prompt, max_tokens;
    void* hidden_buf;       /* [hidden] */
    void* qkv_a_buf;        /* [q_lora + kv_lora + rope] */
    void* q_up_buf;         /* [heads*(nope+rope)] */
    void* kv_up_buf;        /* [heads*(nope+v)] */
    void* attn_buf;         /* [heads*v] */
    void* act_buf;          /* [inter] */
    void* logits;
    float* part_o;
    float* part_ml;
    uint32_t* counters;     /* [heads + 1] */
    float* head_val;
    int32_t* head_idx;
    void* hidden_trace;     /* optional [n_layers+1][hidden] */
    int64_t* picked;
    int32_t pdl;
    float temperature;        /* > 0: sample each token from softmax(logits / temperature) (see tfb_lm_head_args); else greedy */
    uint64_t seed;
    const int64_t* eos_ids;   /* end-of-sequence latch: see tfb_lm_head_args (NULL: none) */
    int32_t* stop_at;
    int32_t n_eos;
    int32_t reserved_eos;
    /* cache_layout TFB_MLA_CACHE_LATENT: layers[i].k_pool is the latent pool, kv_b runs absorbed (tfb_mla_latent_decode
     * instead of kv_b + tfb_attn_mla_decode), part_o / part_ml sized by tfb_mla_latent_splits, and the two scratch
     * vectors below are required. */
    int32_t cache_layout;
    int32_t reserved_layout;
    float* q_lat_buf;         /* [heads*2*kv_lora] */
    float* q_rope_buf;        /* [heads*rope] */
} tfb_minicpm3_step_args;
TFB_API int tfb_minicpm3_decode_step(const tfb_minicpm3_step_args* args, tfb_stream_t stream);

/* ---- a chunk of up to 32 consecutive prompt tokens through the MiniCPM3 stack (latent cache) ----------------
 * Every projection streams its weights once per chunk on the tensor cores (tfb_gemm_small_m); the attention of the
 * chunk runs as one tfb_mla_latent_decode with tokens = m (every token appends its latent row, then token t attends
 * to the rows up to its own).  Nothing is picked.  Needs the gate and up projections of a layer
 * as one [2*inter, hidden] block (layers[i].w_up == layers[i].w_gate + inter*hidden elements) and
 * layers[i].k_pool = the latent pool.  Scratch as for the decode step with cache_layout TFB_MLA_CACHE_LATENT, every
 * buffer m times as long.  Replaces the prompt loop of tests/models/orchestrator/causal_lm/generation.py:56-61
 * for this model. */
typedef struct {
    const tfb_minicpm3_layer* layers;
    int32_t n_layers, m, hidden, heads, q_lora, kv_lora, nope, rope, v, inter;
    int64_t vocab;
    float eps, lora_eps, scale, embed_scale, residual_scale;
    int32_t pdl;
    const void* w_embed;
    const void* cos_table;
    const void* sin_table;
    int32_t max_pos, page_size, table_len, max_ctx;
    const int32_t* block_table;
    const int64_t* ids;       /* [m] token ids of the chunk */
    const int32_t* pos_rows;  /* [m] on the device: the chunk's positions (consecutive) */
    void* hidden_buf;         /* [m][hidden] */
    void* norm_buf;           /* [m][hidden] */
    void* qkv_a_buf;          /* [m][q_lora + kv_lora + rope] */
    void* attn_buf;           /* [m][heads*v] */
    void* act_buf;            /* [m][inter] */
    float* q_lat_buf;
    float* q_rope_buf;
    float* part_o;
    float* part_ml;
    uint32_t* status;         /* [1]: non-zero after a bounded wait of a projection gave up */
} tfb_minicpm3_prefill_args;
TFB_API int tfb_minicpm3_prefill_chunk(const tfb_minicpm3_prefill_args* args, tfb_stream_t stream);

/* out[i] = bf16(a[i] + bf16(b[i] * scale)).  Stands in for residual_add:
 * examples/granite_4_0_h_small-cuda/model.py:502-508; reference kernel granite.cu:159. */
TFB_API int tfb_residual_add(const void* a, const void* b, void* out, int32_t n, float scale, tfb_stream_t stream);

/* ---- Mamba-2 single-token state update --------------------------------------------
 * tfb_conv_step: depthwise causal convolution over [state | entry] (width 4), bf16 products and
 * sum, optional bias, SiLU; the window then slides by the entry (state_out may alias state_in).
 * tfb_ssm_step: dt = softplus(dt_raw + dt_bias); decay = exp(dt * -exp(a_log));
 * state = state * decay + bf16(bf16(dt*B) * x) (f32); y = bf16(sum bf16(state) * C) + x * d_skip.
 * Stand in for conv_step / ssm_step: examples/granite_4_0_h_small-cuda/model.py:154-220;
 * reference kernels examples/granite_4_0_h_small-cuda/kernels/granite.cu:302-410. */
TFB_API int tfb_conv_step(const void* entry, const void* state_in, void* state_out, const void* conv_w,
                          const void* conv_b, void* mixed, void* entry_out, int32_t channels,
                          int32_t kernel_width, int32_t pdl, tfb_stream_t stream);
TFB_API int tfb_ssm_step(const float* state_in, float* state_out, const void* x, const void* b_vec,
                         const void* c_vec, const void* dt_raw, const void* a_log, const void* dt_bias,
                         const void* d_skip, void* y, int32_t n_heads, int32_t head_dim, int32_t n_state,
                         int32_t n_groups, int32_t pdl, tfb_stream_t stream);

/* ---- MoE routing and the fused down stage -------------------------------------------
 * tfb_router_select: mode 0 = top-k of the (bf16) logits then softmax over the k (granite
 * `routing`, model.py:376-386); mode 1 = softmax over all experts in f32, top-k, renormalise
 * (Qwen3.5 `routing`, examples/qwen3_5_35b_a3b-tilelang/model.py:488-499).  indices int64[top_k]
 * by value descending, ties to the lower index; weights bf16 and/or f32.
 * tfb_moe_down: out = residual + bf16(res_scale * (sum_s weight[s] * (W_down[idx[s]] . inner[s])
 * + W_shared . shared_act)) with the authored rounding points (routed_experts / experts /
 * residual_add, granite model.py:406-470,502); reference kernels granite.cu:537-700. */
/* tfb_router_select_prefetch: the same selection; in addition lane j asks L2 (cp.async.bulk.prefetch.L2) for its
 * expert's block of each of up to 4 weight slabs [experts][slab_bytes[i]] (16-byte multiples), e.g. the gate, up and
 * down matrices: the kernels that read them cannot know the indices before their own dependency wait, and HBM is idle
 * while this one-warp kernel runs.  expert_world > 1: only experts with e % world == rank, at local index e / world. */
typedef struct {
    const void* logits_bf16; const float* logits_f32; int64_t* indices; void* weights_bf16; float* weights_f32;
    int32_t experts, top_k, mode, pdl;
    const void* slab[4]; uint64_t slab_bytes[4];
    int32_t n_slabs, expert_rank, expert_world, reserved;
} tfb_router_select_args;
TFB_API int tfb_router_select_prefetch(const tfb_router_select_args* args, tfb_stream_t stream);
TFB_API int tfb_router_select(const void* logits_bf16, const float* logits_f32, int64_t* indices,
                              void* weights_bf16, float* weights_f32, int32_t experts, int32_t top_k,
                              int32_t mode, int32_t pdl, tfb_stream_t stream);
typedef struct {
    const void* w_down;       /* [experts][hidden][inter] */
    const void* w_shared;     /* [hidden][shared_inter] or NULL */
    const void* inner;        /* [top_k][inter] bf16 */
    const void* shared_act;   /* [shared_inter] bf16 */
    const int64_t* indices;
    const void* weights;      /* [top_k] bf16 */
    const float* shared_gate; /* optional device scalar multiplying the shared expert's output */
    const void* residual;     /* optional [hidden] */
    void* out;                /* [hidden] bf16 */
    int32_t hidden, inter, shared_inter, top_k;
    float res_scale;
    int32_t pdl;
    int32_t expert_rank;      /* expert parallel, as in tfb_gemv_args */
    int32_t expert_world;
    float* partial;           /* optional f32 [2][hidden]: instead of `out`, this rank's un-rounded routed sum and
                                 shared-expert dot, to be all-reduced and finished by tfb_moe_finalize */
} tfb_moe_down_args;
TFB_API int tfb_moe_down(const tfb_moe_down_args* args, tfb_stream_t stream);
/* out = residual + bf16(res_scale * bf16(bf16(partial[0]) + bf16(partial[1]))): the roundings tfb_moe_down applies,
 * after the ranks' partials were summed (NCCL all-reduce).  No reference counterpart (the reference is one GPU). */
TFB_API int tfb_moe_finalize(const float* partial, const void* residual, void* out, int32_t hidden, float res_scale,
                             int32_t has_shared, int32_t pdl, tfb_stream_t stream);
/* Greedy pick over `world` gathered (logit, global index) pairs, lowest index on ties, then the token / position
 * bookkeeping of tfb_lm_head_argmax.  No reference counterpart. */
TFB_API int tfb_pick_finalize(const float* pairs, int32_t world, int64_t* tokens, int32_t* pos, int32_t n_prompt,
                              int32_t max_tokens, int64_t* picked, int32_t pdl, tfb_stream_t stream);

/* ---- a whole granite-4.0-h decode step ---------------------------------------------
 * embed*12 -> layers x [mixer (Mamba-2: in_proj, conv, ssm, gated norm + out_proj | attention:
 * qkv, nope GQA attention, o_proj) + 0.22 residual, MoE (router, top-10, gathered gate/up,
 * shared gate/up, fused down + shared out) + 0.22 residual] -> final norm, lm_head / 16, greedy
 * pick.  Recurrent and convolution state are updated in place.  Stands in for
 * Granite4_0_H_Small.forward + append_cache + greedy (granite model.py:640-719). */
typedef struct {
    int32_t kind;             /* 0 = Mamba-2 mixer, 1 = attention mixer */
    int32_t pad;
    const void* gamma_in;
    const void* w_in;         /* mamba: [proj, hidden]; attention: q|k|v rows [(hq+2hkv)*d, hidden] */
    const void* conv_w;
    const void* conv_b;
    const void* a_log;
    const void* dt_bias;
    const void* d_skip;
    const void* gamma_ssm;
    const void* w_out;        /* mamba: [hidden, expand]; attention: w_o [hidden, hq*d] */
    void* conv_state;         /* mamba: bf16 [conv_dim][3] */
    float* ssm_state;         /* mamba: f32 [nh][pd][ns] */
    void* k_pool;             /* attention */
    void* v_pool;
    const void* gamma_post;
    const void* w_router;     /* [experts, hidden] */
    const void* w_gate;       /* [experts, inter, hidden] */
    const void* w_up;
    const void* w_down;       /* [experts, hidden, inter] */
    const void* w_shared_in;  /* [2*shared_inter, hidden] */
    const void* w_shared_out; /* [hidden, shared_inter] */
} tfb_granite_layer;
typedef struct {
    const tfb_granite_layer* layers;
    int32_t n_layers, hidden;
    int32_t nh, pd, ns, ng, conv_width;          /* mamba */
    int32_t hq, hkv, d;                          /* attention */
    int32_t experts, top_k, inter, shared_inter; /* MoE */
    int64_t vocab;
    float eps, attn_scale, embed_scale, res_scale, logits_scale;
    const void* table;        /* [vocab, hidden]: embedding and tied head */
    const void* gamma_final;
    int32_t page_size, table_len, max_ctx;
    const int32_t* block_table;
    int64_t* tokens;
    int32_t* pos;
    int32_t n_prompt, max_tokens;
    void* hidden_buf;         /* [hidden] */
    void* proj_buf;           /* [max(proj, (hq+2hkv)*d)] */
    void* mixed_buf;          /* [conv_dim] */
    void* y_buf;              /* [max(expand, hq*d)] */
    void* router_logits;      /* [experts] bf16 */
    int64_t* router_idx;      /* [top_k] */
    void* router_w;           /* [top_k] bf16 */
    void* inner_buf;          /* [top_k*inter] */
    void* shared_buf;         /* [shared_inter] */
    void* logits;
    float* part_o;
    float* part_ml;
    uint32_t* counters;       /* [hkv + 1] */
    float* head_val;
    int32_t* head_idx;
    void* hidden_trace;       /* optional [n_layers+1][hidden] */
    int64_t* idx_trace;       /* optional [n_layers][top_k]: the routing indices of every layer */
    int64_t* picked;
    int32_t pdl;
    /* expert / tensor / vocabulary parallel over ep_world GPUs (one process each).  Routed experts: expert e on
     * rank e % ep_world; shared expert: column / row slices; head: vocabulary slices; mixers replicated.  The
     * layer slabs then hold only this rank's shard.  The caller all-reduces `partial` between parts 1 and 2 of
     * every layer and all-gathers `pair` into `gathered` between parts 3 and 4. */
    int32_t ep_rank, ep_world;
    float* partial;           /* f32 [2][hidden] */
    float* pair;              /* f32 [2] */
    float* gathered;          /* f32 [ep_world][2] */
    float temperature;        /* > 0: sample each token from softmax(logits / temperature) (see tfb_lm_head_args); else greedy */
    uint64_t seed;
    const int64_t* eos_ids;   /* end-of-sequence latch: see tfb_lm_head_args (NULL: none) */
    int32_t* stop_at;
    int32_t n_eos;
    int32_t reserved_eos;
} tfb_granite_step_args;
TFB_API int tfb_granite_decode_step(const tfb_granite_step_args* args, tfb_stream_t stream);
/* One piece of the step, so a sharded caller can interleave its collectives: part 0 embed; 1 layer `layer` up to
 * the MoE down stage; 2 finish layer `layer` from the summed partials; 3 final norm + head; 4 pick from the
 * gathered pairs.  With ep_world <= 1 parts 0, 1.., 3 are the whole step (what tfb_granite_decode_step runs). */
TFB_API int tfb_granite_step_part(const tfb_granite_step_args* args, int32_t part, int32_t layer, tfb_stream_t stream);

/* Up to 4 dependent projections (each reads the outputs of the one before) in one persistent cooperative launch of
 * one CTA per SM; same arithmetic as tfb_gemv with prologue NONE / F32GAIN / CAST_THEN_GAIN and epilogue STORE /
 * RESIDUAL / SWIGLU.  The weight stream runs ahead across the phase boundaries through a shared-memory ring.
 * sync: u32[4] zeroed once by the caller; sync[2] is set non-zero if a bounded grid-barrier wait gave up (the
 * outputs are then invalid; nothing hangs).  Every k a multiple of 256 and <= 8192; every n >= the SM count.
 * No reference counterpart: the reference launches these projections one by one
 * (examples/qwen3_1_7b-tilelang/fast/engine.py:189-271). */
typedef struct {
    tfb_gemv_args phase[4];
    int32_t n_phases, pdl;
    uint32_t* sync;
} tfb_gemv_chain_args;
TFB_API int tfb_gemv_chain(const tfb_gemv_chain_args* args, tfb_stream_t stream);

/* ---- small-batch projection on the tensor cores (tcgen05 + TMEM + TMA) -----------------------------------
 * y[M, N] = x[M, K] . w[N, K]^T (+ residual), 1 <= M <= 32 tokens, bf16 in / f32 accumulate / bf16 out; w in the
 * same [out, in] layout tfb_gemv reads.  With residual: y = bf16(residual + bf16(acc)) (TFB_EPI_RESIDUAL's
 * rounding).  K a multiple of 64; w, x 16-byte aligned.  K is split over the tfb_gemm_small_m_splits(N, K) CTAs
 * (1, 2, 4 or 8) of a thread-block cluster and the partial tiles are added in fixed order through distributed
 * shared memory: deterministic, nothing spins, no scratch in global memory (partial and tickets are not used and
 * may be NULL).  status: u32 set non-zero if a bounded mbarrier wait gave up (outputs then invalid; nothing hangs).
 * The batch-32 form of the projections of examples/qwen3_1_7b-tilelang/fast/kernels.py:124-260 (the reference
 * runs batch 1 only). */
typedef struct {
    const void* w; const void* x; const void* residual; void* y;
    float* partial; uint32_t* tickets; uint32_t* status;
    int32_t m, n, k, pdl;
    /* swiglu != 0: w is [2n, k] = n gate rows then n up rows, y[M, n] = bf16(silu(bf16(x.gate^T)) * bf16(x.up^T))
     * (TFB_EPI_SWIGLU's rounding); n a multiple of 64, no residual. */
    int32_t swiglu;
    /* with residual: y = bf16(residual + bf16(bf16(acc) * res_scale)), as tfb_gemv's res_scale; 0 means 1 */
    float res_scale;
} tfb_gemm_small_m_args;
TFB_API int32_t tfb_gemm_small_m_splits(int32_t n, int32_t k);
TFB_API int32_t tfb_gemm_small_m_swiglu_splits(int32_t n, int32_t k);
TFB_API int tfb_gemm_small_m(const tfb_gemm_small_m_args* args, tfb_stream_t stream);

/* ---- nucleus (top-p) sampling after a decode step ------------------------------------------------------------
 * Replaces the token a decode step has just written by a draw from the nucleus of softmax(logits / temperature): the
 * distinct logit values are walked from the largest down, adding count(value) * exp((value - max) / temperature) in
 * f64; the first value at which the running mass reaches top_p * total is the threshold, and every token whose logit
 * is at least that value belongs (ties included).  Inside the nucleus the pick is the Gumbel-max rule of
 * tfb_lm_head_args (same variates: top_p = 1 draws what the head kernel draws).  The reference's sampler has
 * temperature only (examples/granite_4_0_h_small-cuda/kernels/granite.cu:712-797); this is the filter its
 * generation loop would apply on the host.
 *   logits:   bf16 [vocab], kept by the step (its `logits` argument)
 *   pos:      the step's position scalar, after the step; prev_pos: a copy taken before the step
 *   tokens:   the history; tokens[*pos] is rewritten when *pos != *prev_pos and *pos >= n_prompt
 *   eos_ids / n_eos / stop_at: the end-of-sequence latch of tfb_lm_head_args, applied to the new token (give the step
 *             itself no end ids then); a latched sequence is left alone
 *   hist:     scratch int32 [65664], zeroed once (the two kernels of the call leave it zeroed)
 *   threshold_out: optional, the smallest logit value inside the nucleus */
typedef struct {
    const void* logits;
    const int32_t* pos;
    const int32_t* prev_pos;
    int64_t* tokens;
    int64_t* picked;            /* optional */
    float* threshold_out;       /* optional */
    const int64_t* eos_ids;
    int32_t* stop_at;
    int32_t* hist;
    int32_t vocab, n_prompt, n_eos, pdl;
    float temperature, top_p;
    uint64_t seed;
} tfb_sample_top_p_args;
TFB_API int tfb_sample_top_p(const tfb_sample_top_p_args* args, tfb_stream_t stream);

/* ---- mixture-of-experts block for a batch of tokens -----------------------------------------------------------
 * out[t] = residual[t] + sum_s weights[t,s] * bf16(W_down[e] . bf16(silu(bf16(W_gate[e] . bf16 x[t])) * bf16(W_up[e] . bf16 x[t])))
 *          + (the same through the shared expert) * sigmoid(shared_gate[t]),            e = indices[t,s]
 * for `tokens` tokens at once: every expert that a token selected is read once and meets all of its tokens on the
 * tensor cores (K folded into the MMA's N, eight tokens per tcgen05.mma; tilefoundry_b200/csrc/moe_grouped.cu).  The
 * batch form of `experts` of the authored Qwen3.5 block (examples/qwen3_5_35b_a3b-tilelang/model.py: routed_experts +
 * shared_expert; the reference's kernels, kernels/moe.py:368 `_h_kernel` and :527 `_down_kernel`, take one token).
 * Routing (indices, weights, the shared gate's logit) is the caller's: tfb_router_select per token.
 * Scratch (device, any contents): x_bf16 [tokens][hidden] bf16, inner [tokens][top_k+1][inter] bf16,
 * y [tokens][top_k+1][hidden] bf16, counts i32 [2*(experts+1)+1], lists i32 [experts+1][tokens]; status u32 zeroed once.
 * hidden and inter multiples of 128 (inter of 8, hidden of 16), (16 + 8) * max(hidden, inter) * 2 <= 200 KB. */
typedef struct {
    const float* x;             /* [tokens][hidden] f32 */
    const int64_t* indices;     /* [tokens][top_k] */
    const float* weights;       /* [tokens][top_k] f32 */
    const float* shared_gate;   /* optional [tokens] f32 */
    const float* residual;      /* optional [tokens][hidden] f32 */
    const void* w_gate;         /* bf16 [experts][inter][hidden] */
    const void* w_up;
    const void* w_down;         /* bf16 [experts][hidden][inter] */
    const void* w_shared_gate;  /* optional: bf16 [inter][hidden] */
    const void* w_shared_up;
    const void* w_shared_down;  /* bf16 [hidden][inter] */
    float* out;                 /* [tokens][hidden] f32 */
    void* x_bf16;
    void* inner;
    void* y;
    int32_t* counts;
    int32_t* lists;
    uint32_t* status;
    int32_t tokens, hidden, inter, experts, top_k, pdl;
} tfb_moe_batch_args;
TFB_API int tfb_moe_batch(const tfb_moe_batch_args* args, tfb_stream_t stream);
/* Routing for the same batch: logits[t][e] = bf16(W_router[e] . bf16 x[t]) (row `experts`: the shared expert's scale row),
 * then the selection of tfb_router_select (mode 0: top-k then softmax over the k; mode 1: softmax over all, top-k,
 * renormalise) for every token, one CTA per token.  `routing` + the gate logit of `shared_expert` of the authored
 * block for a batch (examples/qwen3_5_35b_a3b-tilelang/model.py: routing, shared_expert); weights are f32.
 * hidden a multiple of 256 up to 8192, experts <= 256, top_k <= 32. */
typedef struct {
    const float* x;              /* [tokens][hidden] f32 */
    const void* w_router;        /* bf16 [experts][hidden] */
    const void* w_shared_scale;  /* optional bf16 [hidden] */
    float* logits;               /* scratch [tokens][experts + 1] f32 */
    int64_t* indices;            /* [tokens][top_k] */
    float* weights;              /* [tokens][top_k] f32 */
    float* shared_gate;          /* optional [tokens] f32 */
    int32_t tokens, hidden, experts, top_k, mode, pdl;
} tfb_moe_route_args;
TFB_API int tfb_moe_batch_route(const tfb_moe_route_args* args, tfb_stream_t stream);

/* ---- Qwen3-architecture decode step for several sequences (batch <= 32) ------------------------------------
 * One token for each of `batch` independent sequences: every projection runs once on the tensor cores for the
 * whole batch (tfb_gemm_small_m), attention once per layer with one CTA set per sequence (tfb_attn_gqa_decode
 * with batch), norms / embedding / pick row-wise.  Per sequence the arithmetic and its rounding points are those
 * of tfb_qwen3_decode_step; only the order of the f32 sums inside a projection differs (tensor-core tiles).
 * The batch form of examples/qwen3_1_7b-tilelang/fast/engine.py:189-271 (the reference decodes one sequence).
 * Launches per step: 4 + 7 * n_layers. */
typedef struct {
    const void* gamma_in;
    const void* w_qkv;      /* [(hq+2hkv)*d, hidden] */
    const void* gamma_q;
    const void* gamma_k;
    const void* w_o;        /* [hidden, hq*d] */
    const void* gamma_post;
    const void* w_gate_up;  /* [2*inter, hidden]: gate rows, then up rows */
    const void* w_down;     /* [hidden, inter] */
    void* k_pool;           /* pages of every sequence */
    void* v_pool;
} tfb_qwen3_batch_layer;
typedef struct {
    const tfb_qwen3_batch_layer* layers; /* host array [n_layers] */
    int32_t n_layers, batch, hidden, hq, hkv, d, inter, pdl;
    int64_t vocab;
    float eps, scale;
    const void* w_embed;    /* [vocab, hidden] */
    const void* gamma_final;
    const void* w_head;     /* [vocab, hidden] */
    const void* cos_table;
    const void* sin_table;
    int32_t max_pos, page_size, table_len, max_ctx;
    const int32_t* block_table; /* [batch][table_len] */
    int64_t* tokens;        /* [batch][max_tokens]: prompt, then the picked tokens */
    int32_t* pos;           /* [batch]: advanced by the step */
    int32_t n_prompt, max_tokens;
    void* hidden_buf;       /* [batch][hidden] bf16 residual stream */
    void* norm_buf;         /* [batch][hidden] */
    void* qkv_buf;          /* [batch][(hq+2hkv)*d] */
    void* attn_buf;         /* [batch][hq*d] */
    void* act_buf;          /* [batch][inter] */
    void* logits;           /* [batch][vocab] bf16 (required: the pick reads it) */
    float* part_o;          /* attention split scratch, batch times the single-sequence size */
    float* part_ml;
    uint32_t* counters;     /* [batch*hkv + batch] zeroed once: attention tickets, then pick tickets */
    uint32_t* status;       /* u32 zeroed once; non-zero after a step: a bounded wait gave up, outputs invalid */
    float* pick_val;        /* f32 [batch * 8] */
    int32_t* pick_idx;      /* i32 [batch * 8] */
    int64_t* picked;        /* optional [batch]: the token each sequence picked, whatever its prompt says */
    void* hidden_trace;     /* optional [n_layers+1][batch][hidden] bf16 */
    float temperature;      /* > 0: every sequence samples from softmax(logits / temperature) by the Gumbel-max rule of
                             * tfb_lm_head_args, sequence b keyed by (seed + b, its position, vocabulary index); else greedy */
    int32_t reserved;
    uint64_t seed;
} tfb_qwen3_batch_step_args;
TFB_API int tfb_qwen3_batch_decode_step(const tfb_qwen3_batch_step_args* args, tfb_stream_t stream);

/* ---- Qwen3-architecture prompt processing, one chunk of <= 32 consecutive tokens of one sequence -----------
 * Runs the layer stack for the chunk's tokens at once: projections on the tensor cores (tfb_gemm_small_m, M = m),
 * attention in the chunk form of tfb_attn_gqa_decode (every token attends to the cached rows before it; two
 * launches per layer, see `chunk` there).  Leaves the tokens' K/V rows in the cache and the residual stream of
 * each token in hidden_buf; no head, no pick: a prompt's logits are not needed until its last token, which the
 * decode step processes.  The reference walks a prompt token by token
 * (tests/models/orchestrator/causal_lm/generation.py:56-61); per token the arithmetic and its rounding points are
 * those of that walk, only the order of the f32 sums inside a projection differs.  Launches: 1 + 8 * n_layers. */
typedef struct {
    const tfb_qwen3_batch_layer* layers; /* host array [n_layers] */
    int32_t n_layers, m, hidden, hq, hkv, d, inter, pdl;
    float eps, scale;
    int64_t vocab;
    const void* w_embed;
    const void* cos_table;
    const void* sin_table;
    int32_t max_pos, page_size, table_len, max_ctx;
    const int32_t* block_table; /* [table_len]: the sequence's pages */
    const int64_t* ids;         /* device [m]: the chunk's token ids */
    const int32_t* pos_rows;    /* device [m]: first position + i (first + m <= max_ctx) */
    void* hidden_buf;           /* [m][hidden] */
    void* norm_buf;             /* [m][hidden] */
    void* qkv_buf;              /* [m][(hq+2hkv)*d] */
    void* attn_buf;             /* [m][hq*d] */
    void* act_buf;              /* [m][inter] */
    float* part_o;              /* attention split scratch, m times the single-sequence size */
    float* part_ml;
    uint32_t* counters;         /* [m*hkv] zeroed once */
    uint32_t* status;           /* as in tfb_gemm_small_m */
} tfb_qwen3_prefill_args;
TFB_API int tfb_qwen3_prefill_chunk(const tfb_qwen3_prefill_args* args, tfb_stream_t stream);

/* ================= f32-activation family (Qwen3.5-35B-A3B) =================
 * The reference's Qwen3.5 example keeps activations, recurrent state and KV cache in f32 and its contracted
 * weights in bf16: a product casts its activation to bf16, runs at bf16 and casts the result back
 * (examples/qwen3_5_35b_a3b-tilelang/model.py:189,214-225; kernels/torch_ref.py:134-142).  Every f32 buffer
 * below follows that rule: values a product wrote are exactly representable in bf16. */

/* y = epilogue(bf16(W . bf16(prologue(x)))); W [n,k] bf16 row-major, x/gamma/gate/residual/y f32.
 * prologue TFB_NORM_NONE, TFB_NORM_F32GAIN (gamma [k]) or TFB_NORM_SEGMENT_GATED (gamma [seg], gate [k]);
 * epilogue TFB_EPI_STORE, TFB_EPI_RESIDUAL (y = residual + bf16(acc)) or TFB_EPI_SWIGLU
 * (y = bf16(silu(bf16(acc_gate)) * bf16(acc_up)), w = gate rows, w2 = up rows).
 * Expert mode (rows_per_expert > 0): output rows come in slots of rows_per_expert; slot s < routed_slots reads
 * the rows of expert expert_idx[s] of w (and w2), later rows (n need not end on a slot boundary) read consecutive
 * rows of w_extra (w2_extra).
 * Replaces the projections inside linear_attention / full_attention / routing / routed_experts / shared_expert
 * (examples/qwen3_5_35b_a3b-tilelang/model.py:214-228,380-417,488-499,540-590). */
typedef struct {
    const void* w; const void* w2; const void* w_extra; const void* w2_extra;
    const float* x; const float* gamma; const float* gate; const float* residual;
    float* y;
    int32_t n, k, seg;
    int32_t prologue, epilogue;
    float eps;
    const int64_t* expert_idx;
    int32_t rows_per_expert, routed_slots;
    int32_t pdl, reserved;
    /* Router launch (TFB_EPI_STORE, no expert mode), optional: when route_counter is set the last CTA to finish
     * selects route_top_k of the first route_experts outputs -- softmax over all, top-k, renormalise by the k (the
     * routing function, model.py:488-499) -- into idx_out [route_top_k] and w_out [route_top_k], so the selection
     * needs no launch of its own.  route_counter: u32 zeroed once by the caller; the kernel leaves it zero. */
    uint32_t* route_counter; int32_t route_experts, route_top_k;
    int64_t* idx_out; float* w_out;
    /* Expert mode on several GPUs: expert e lives on rank e % expert_world as local expert e / expert_world; slots
     * whose expert is another rank's are skipped (their outputs are left untouched).  0 or 1: all experts local. */
    int32_t expert_rank, expert_world;
} tfb_gemv_f32_args;
TFB_API int tfb_gemv_f32(const tfb_gemv_f32_args* args, tfb_stream_t stream);

/* One Gated DeltaNet token for all value heads: conv_step + SiLU, l2_normalise of q and k, the decay
 * g = -exp(a_log) * softplus(a + dt_bias) and write strength beta = sigmoid(b), and delta_step
 * (examples/qwen3_5_35b_a3b-tilelang/model.py:117-212).  proj = [2*hk*dk + hv*dv conv entry | hv*dv z | hv b | hv a]
 * (z is not read here).  conv_state is TWO buffers [channels][width-1], conv_state_stride floats apart: the
 * buffer (*pos & 1) is read and the other one receives the shifted window (pos null: read 0, write 1).
 * state [hv][dk][dv] is updated in place; read [hv*dv] is the un-normalised read-out. dk = 128, width = 4. */
typedef struct {
    const float* proj;
    float* conv_state; uint64_t conv_state_stride;
    const int32_t* pos;
    const float* conv_w; const float* a_log; const float* dt_bias;
    float* state; float* read;
    int32_t hk, hv, dk, dv, kernel_width;
    float q_scale;
    int32_t pdl, reserved;
    /* delta_step alone: when direct_q is set, q [hv][dk], k [hv][dk], v [hv][dv], g [hv], beta [hv] are taken
     * as given and proj / conv_state / conv_w / a_log / dt_bias are not read. */
    const float* direct_q; const float* direct_k; const float* direct_v; const float* direct_g; const float* direct_beta;
} tfb_gdn_args;
TFB_API int tfb_gdn_step(const tfb_gdn_args* args, tfb_stream_t stream);
/* The pieces of the mixer as functions of their own (conv_step, l2_normalise, partial_rope / partial_rope_kv;
 * examples/qwen3_5_35b_a3b-tilelang/model.py:117-150,293-330): mixed[c] = silu(sum_j window[c][j] * conv_w[c][j]) with
 * window = state [channels][width-1] followed by entry [channels]; y = x * rsqrt(sum(x^2) + eps) per row;
 * rotate-half RoPE at *pos on the leading rotary_dim of each of `heads` rows of d elements. */
TFB_API int tfb_conv_silu_f32(const float* state, const float* entry, const float* conv_w, float* mixed, int32_t channels,
                              int32_t width, int32_t pdl, tfb_stream_t stream);
TFB_API int tfb_l2norm_f32(const float* x, float* y, int32_t rows, int32_t width, float eps, int32_t pdl, tfb_stream_t stream);
TFB_API int tfb_partial_rope_f32(const float* x, const float* cos_table, const float* sin_table, const int32_t* pos,
                                 float* out, int32_t heads, int32_t d, int32_t rotary_dim, int32_t pdl, tfb_stream_t stream);

/* Gated GQA decode attention over a paged f32 cache: per-head RMSNorm of q and k with f32 gains, rotate-half
 * RoPE on the leading rotary_dim (a multiple of 64) of each head, append at *pos, softmax over positions
 * 0..*pos, output times sigmoid(gate) (examples/qwen3_5_35b_a3b-tilelang/model.py:293-417).
 * proj = [hq][2*d] (q then gate per head) | [hkv][d] k | [hkv][d] v.  Pools are [page][page_size][hkv][d] f32,
 * page_size a multiple of 64.
 * Scratch: part_o f32 [hq * nsplit * d], part_ml f32 [hq * nsplit * 2], counters u32 [tfb_attn_gated_groups(hq, hkv, d)]
 * zeroed once, with nsplit = tfb_attn_gated_splits(max_ctx). */
typedef struct {
    const float* proj; const float* gamma_q; const float* gamma_k;
    const float* cos_table; const float* sin_table;
    const int32_t* pos; const int32_t* rope_pos;
    float* k_pool; float* v_pool; const int32_t* block_table;
    float* out; float* k_new_out; float* v_new_out;
    float* part_o; float* part_ml; uint32_t* counters;
    int32_t hq, hkv, d, rotary_dim, page_size, table_len, max_ctx, max_pos;
    float eps, scale;
    int32_t pdl, reserved;
} tfb_attn_gated_args;
TFB_API int32_t tfb_attn_gated_splits(int32_t max_ctx);
TFB_API int32_t tfb_attn_gated_groups(int32_t hq, int32_t hkv, int32_t d);
TFB_API int tfb_attn_gated_decode(const tfb_attn_gated_args* args, tfb_stream_t stream);

/* out[j] = residual[j] + sum_s weights[s] * bf16(w_down[indices[s]][j,:] . inner[s,:])
 *                      + bf16(w_shared[j,:] . inner[top_k,:]) * sigmoid(*shared_gate_logit)
 * (routed_experts + shared_expert + experts + the layer's residual_add,
 * examples/qwen3_5_35b_a3b-tilelang/model.py:540-612,650-665). */
typedef struct {
    const void* w_down; const void* w_shared;
    const float* inner; const int64_t* indices; const float* weights; const float* shared_gate_logit;
    const float* residual; float* out;
    int32_t hidden, inter, shared_inter, top_k;
    int32_t pdl, reserved;
    /* Several GPUs: only this rank's experts (e % expert_world == expert_rank, stored as local expert
     * e / expert_world) and this rank's slice of the shared expert are here; with `partial` (f32 [2][hidden]) the
     * kernel writes its routed sum and its un-rounded shared dot there instead of `out`, for
     * tfb_moe_allreduce_finalize to add across ranks. */
    int32_t expert_rank, expert_world; float* partial;
} tfb_moe_down_f32_args;
TFB_API int tfb_moe_down_f32(const tfb_moe_down_f32_args* args, tfb_stream_t stream);

/* embed (bf16 table row widened to f32), tf.rms_norm on f32 with an f32 gain, plain f32 add
 * (examples/qwen3_5_35b_a3b-tilelang/model.py:760-800,650-665). */
TFB_API int tfb_embed_f32(const void* table, const int64_t* ids, float* out, int32_t rows, int32_t hidden, int64_t vocab,
                          int32_t pdl, tfb_stream_t stream);
TFB_API int tfb_rmsnorm_f32(const float* x, const float* gamma, float* y, int32_t rows, int32_t width, float eps,
                            int32_t pdl, tfb_stream_t stream);
TFB_API int tfb_residual_add_f32(const float* a, const float* b, float* out, int32_t n, int32_t pdl, tfb_stream_t stream);

/* One decoder layer's weights and state.  kind 0: Gated DeltaNet mixer, kind 1: gated attention mixer.
 * w_in  kind 0: [2*hk*dk + 2*hv*dv + 2*hv][hidden] rows of w_in_qkv | w_in_z | w_in_b | w_in_a
 *       kind 1: [hq*2*d + 2*hkv*d][hidden]        rows of w_qg | w_k | w_v
 * w_router [experts + 1][hidden]: the router's rows, then the shared expert's scale row. */
typedef struct {
    int32_t kind, reserved;
    const float* gamma_in; const void* w_in; const void* w_out;
    const float* conv_w; const float* a_log; const float* dt_bias; const float* gamma_gdn;
    float* conv_state; float* state;
    const float* gamma_q; const float* gamma_k; float* k_pool; float* v_pool;
    const float* gamma_post; const void* w_router;
    const void* w_gate; const void* w_up; const void* w_down;
    const void* w_shared_gate; const void* w_shared_up; const void* w_shared_down;
} tfb_qwen35_layer;

/* The whole captured step of the reference's engine for this model (embed -> layers -> final norm -> head ->
 * greedy pick -> bookkeeping; examples/qwen3_5_35b_a3b-tilelang/model.py:800-892 and runtime_model.py).
 * 7 launches per layer; token history
 * and position live on the device as in tfb_qwen3_decode_step. */
typedef struct {
    const tfb_qwen35_layer* layers; int32_t n_layers; int32_t pdl;
    const void* table; const float* gamma_final; const void* w_head;
    const float* cos_table; const float* sin_table;
    int64_t* tokens; int32_t* pos; int32_t n_prompt, max_tokens;
    const int32_t* block_table; int32_t page_size, table_len, max_ctx;
    int32_t hidden; int64_t vocab;
    int32_t hk, hv, dk, dv, conv_width;
    int32_t hq, hkv, d, rotary_dim;
    int32_t experts, top_k, inter, shared_inter;
    uint64_t conv_state_stride;
    float eps, attn_scale, q_scale;
    float* hidden_buf; float* attended_buf; float* proj_buf; float* mixed_buf;
    float* router_logits; int64_t* router_idx; float* router_w; float* inner_buf;
    float* part_o; float* part_ml; uint32_t* counters /* [tfb_attn_gated_groups(hq, hkv, d) + 1], zeroed once */; float* head_val; int32_t* head_idx;
    void* logits; int64_t* picked;
    float* hidden_trace;      /* optional f32 [(n_layers + 1)][hidden]: every layer's output, then the final norm */
    int64_t* idx_trace;       /* optional [n_layers][top_k] */
    /* several GPUs (expert / shared-expert / vocabulary parallel as in tfb_granite_step_args): the layers hold this
     * rank's experts, its slice of the shared expert (shared_inter is the FULL size) and w_head its vocabulary slice */
    int32_t ep_rank, ep_world;
    float* partial;           /* f32 [2][hidden] */
    float* pair;              /* f32 [2] */
    int32_t expert_prefetch;  /* non-zero: the selection kernel asks L2 for the selected experts' weights */
    int32_t reserved;
    float temperature;        /* > 0: sample each token from softmax(logits / temperature) (see tfb_lm_head_args); else greedy */
    uint64_t seed;
    const int64_t* eos_ids;   /* end-of-sequence latch: see tfb_lm_head_args (NULL: none) */
    int32_t* stop_at;
    int32_t n_eos;
    int32_t reserved_eos;
} tfb_qwen35_step_args;
TFB_API int tfb_qwen35_decode_step(const tfb_qwen35_step_args* args, tfb_stream_t stream);
/* One piece of the step, so a sharded caller can put its exchange kernels between them: part 0 embed; part 1 layer
 * `layer` up to the expert down stage (on several GPUs it leaves this rank's partial sums in args->partial and the
 * attended hidden state in attended_buf for tfb_moe_allreduce_finalize); part 3 final norm + head (several GPUs: this
 * rank's vocabulary slice, leaving (logit, index) in args->pair for tfb_pick_allgather). */
TFB_API int tfb_qwen35_step_part(const tfb_qwen35_step_args* args, int32_t part, int32_t layer, tfb_stream_t stream);

/* ---- exchange steps of the sharded MoE step as single kernels over NVLink peer memory ---------------------
 * tfb_moe_allreduce_finalize = all-reduce of the ranks' partial sums + tfb_moe_finalize in one launch;
 * tfb_pick_allgather = all-gather of the ranks' (logit, index) pairs + tfb_pick_finalize in one launch.
 * inbox[r] / flags[r] are pointers to rank r's buffers as mapped in THIS process (peer pointers for r != rank;
 * e.g. from torch.distributed._symmetric_memory).  Sizes, per rank: reduce inbox f32 [2][world][2][hidden], reduce
 * flags u32 [world][ceil(hidden/256)], pick inbox f32 [2][world][2], pick flags u32 [world]; all zeroed once before
 * the first call.  epoch: local u32 [ceil(hidden/256)] (reduce) / [1] (pick), zeroed once.  Every rank must make the
 * same sequence of calls.  Waits are bounded: on a timeout *status becomes non-zero and the outputs are invalid.
 * No reference counterpart: the reference runs on one GPU and has no collective of any kind. */
typedef struct {
    const float* partial; float* inbox[8]; uint32_t* flags[8]; uint32_t* epoch; uint32_t* status;
    const void* residual; void* out;
    int32_t hidden, rank, world, has_shared; float res_scale; int32_t pdl;
    /* f32-activation form (Qwen3.5), used when out_f32 is set:
     * out_f32 = residual_f32 + sum_r routed_r + bf16(sum_r shared_r) * sigmoid(*gate_logit). */
    const float* residual_f32; float* out_f32; const float* gate_logit;
} tfb_moe_allreduce_args;
TFB_API int tfb_moe_allreduce_finalize(const tfb_moe_allreduce_args* args, tfb_stream_t stream);
typedef struct {
    const float* pair; float* inbox[8]; uint32_t* flags[8]; uint32_t* epoch; uint32_t* status;
    int64_t* tokens; int32_t* pos; int64_t* picked;
    int32_t n_prompt, max_tokens, rank, world, pdl, reserved;
} tfb_pick_allgather_args;
TFB_API int tfb_pick_allgather(const tfb_pick_allgather_args* args, tfb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TFB200_H */
