// Small kernels around the projections: embedding gather, stand-alone RMSNorm,
// and the lm_head projection fused with the greedy pick.
#include "gemv.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

// ---- embedding ---------------------------------------------------------------
// Row r reads table[id] where id = ids[r], or tokens[*pos] when `tokens` is given
// (the generation loop keeps its token history and position on the device).
__global__ void embed_kernel(const uint16_t* __restrict__ table, const long long* __restrict__ ids,
                             const long long* __restrict__ tokens, const int* __restrict__ pos,
                             uint16_t* __restrict__ out, int hidden, long long vocab, float scale) {
    pdl_trigger();
    pdl_wait();
    long long id = tokens ? tokens[*pos] : ids[blockIdx.x];
    if (id < 0) id = 0;
    if (id >= vocab) id = vocab - 1;
    const uint4* src = reinterpret_cast<const uint4*>(table + size_t(id) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(out + size_t(blockIdx.x) * hidden);
    for (int c = threadIdx.x; c < (hidden >> 3); c += blockDim.x) {
        uint4 v = src[c];
        if (scale != 1.f) {
            uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t lo = f32_to_bf16_bits(bf16_lo(u[i]) * scale);
                const uint32_t hi = f32_to_bf16_bits(bf16_hi(u[i]) * scale);
                u[i] = lo | (hi << 16);
            }
            v = make_uint4(u[0], u[1], u[2], u[3]);
        }
        dst[c] = v;
    }
}

cudaError_t embed_launch(const uint16_t* table, const long long* ids, const long long* tokens,
                         const int* pos, uint16_t* out, int rows, int hidden, long long vocab,
                         float scale, cudaStream_t stream, bool pdl) {
    return launch_kernel(embed_kernel, dim3(rows), dim3(256), 0, stream, pdl, table, ids, tokens, pos,
                         out, hidden, vocab, scale);
}

// ---- RMSNorm -------------------------------------------------------------------
// One CTA per row.  Rows of up to 8 * blockDim elements (a multiple of 8) are read once with 16-byte loads and
// kept in registers between the sum of squares and the scaling; other widths take the two-pass form.
template <int MODE>
__global__ void rmsnorm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gamma,
                               uint16_t* __restrict__ y, int width, float eps) {
    __shared__ float red[32];
    const uint16_t* xr = x + size_t(blockIdx.x) * width;
    uint16_t* yr = y + size_t(blockIdx.x) * width;
    const bool one_pass = (width & 7) == 0 && width <= 8 * int(blockDim.x) &&
                          ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                            reinterpret_cast<uintptr_t>(gamma)) & 15) == 0;
    if (one_pass) {
        const int c = threadIdx.x;
        const bool mine = c * 8 < width;
        uint4 gv = make_uint4(0, 0, 0, 0);
        if (mine) gv = *(reinterpret_cast<const uint4*>(gamma) + c);     // the gain does not depend on the kernel before
        pdl_trigger();
        pdl_wait();
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = 0.f;
        if (mine) {
            const uint4 v = *(reinterpret_cast<const uint4*>(xr) + c);
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) { f[2 * i] = bf16_lo(u[i]); f[2 * i + 1] = bf16_hi(u[i]); }
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
        ss = block_sum(ss, red);
        const float rstd = rsqrtf(ss / float(width) + eps);
        if (mine) {
            const uint32_t gu[4] = {gv.x, gv.y, gv.z, gv.w};
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float g0 = bf16_lo(gu[i]), g1 = bf16_hi(gu[i]);
                const float a = (MODE == 2) ? round_bf16(f[2 * i] * rstd) * g0 : f[2 * i] * rstd * g0;
                const float b = (MODE == 2) ? round_bf16(f[2 * i + 1] * rstd) * g1 : f[2 * i + 1] * rstd * g1;
                o[i] = uint32_t(f32_to_bf16_bits(a)) | (uint32_t(f32_to_bf16_bits(b)) << 16);
            }
            *(reinterpret_cast<uint4*>(yr) + c) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        return;
    }
    pdl_trigger();
    pdl_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = bf16_bits_to_f32(xr[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / float(width) + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = bf16_bits_to_f32(xr[i]), g = bf16_bits_to_f32(gamma[i]);
        const float o = (MODE == 2) ? round_bf16(v * rstd) * g : v * rstd * g;
        yr[i] = f32_to_bf16_bits(o);
    }
}

cudaError_t rmsnorm_launch(const uint16_t* x, const uint16_t* gamma, uint16_t* y, int rows, int width,
                           float eps, int mode, cudaStream_t stream, bool pdl) {
    const int threads = (width > 2048 && width <= 4096 && (width & 7) == 0) ? 512 : 256;
    if (mode == 2)
        return launch_kernel(rmsnorm_kernel<2>, dim3(rows), dim3(threads), 0, stream, pdl, x, gamma, y, width, eps);
    return launch_kernel(rmsnorm_kernel<1>, dim3(rows), dim3(threads), 0, stream, pdl, x, gamma, y, width, eps);
}

__global__ void copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int n16) {
    pdl_trigger();
    pdl_wait();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += gridDim.x * blockDim.x) dst[i] = src[i];
}
cudaError_t copy_launch(const void* src, void* dst, int bytes, cudaStream_t stream, bool pdl) {
    return launch_kernel(copy_kernel, dim3(1), dim3(256), 0, stream, pdl,
                         static_cast<const uint4*>(src), static_cast<uint4*>(dst), bytes / 16);
}

// out = a + bf16(b * scale), element by element (granite's residual_add as a stand-alone function)
__global__ void residual_add_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b,
                                    uint16_t* __restrict__ out, int n, float scale) {
    pdl_trigger();
    pdl_wait();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        out[i] = f32_to_bf16_bits(bf16_bits_to_f32(a[i]) + round_bf16(bf16_bits_to_f32(b[i]) * scale));
}
cudaError_t residual_add_launch(const uint16_t* a, const uint16_t* b, uint16_t* out, int n, float scale,
                                cudaStream_t stream, bool pdl) {
    return launch_kernel(residual_add_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, pdl, a, b, out, n, scale);
}

// ---- lm_head + greedy pick (or Gumbel-max sample) ------------------------------
// Algorithmic bytes per launch = n*k*2 (the head matrix, read once).  Each CTA
// reduces its rows' bf16-rounded logits to one (max, lowest index) pair; the last
// CTA to finish (atomic ticket) reduces the pairs, writes the token and advances
// the generation state.  Ties resolve to the lowest index, as torch.argmax does.
// With temperature > 0 the pairs are over logit / T + Gumbel noise instead: a draw
// from softmax(logits / T) in the same single launch.
constexpr int kHeadRows = 4, kHeadWarps = 8, kHeadUnroll = 2;
int lm_head_ctas(int n) { return (n + kHeadRows * kHeadWarps - 1) / (kHeadRows * kHeadWarps); }

__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// f32 hidden state with an f32 gain, rounded to bf16 once on its way into the product (mode 5).
__device__ __forceinline__ void stage_head_f32(const float* __restrict__ x, const float* __restrict__ gamma, float* xs,
                                               float* red, int k, float eps) {
    if (gamma == nullptr) {                          // already normalised
        for (int i = threadIdx.x; i < k; i += blockDim.x) xs[xs_index(i)] = round_bf16(x[i]);
        return;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < k; i += blockDim.x) { const float v = x[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / float(k) + eps);
    for (int i = threadIdx.x; i < k; i += blockDim.x) xs[xs_index(i)] = round_bf16(x[i] * rstd * gamma[i]);
}

template <int NORM_MODE>
__global__ void __launch_bounds__(kHeadWarps * 32, 4) lm_head_kernel(const HeadParams p) {
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;
    float* red = smem + p.k;
    __shared__ float wv[kHeadWarps];
    __shared__ int wi[kHeadWarps];
    __shared__ int s_last;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = (blockIdx.x * kHeadWarps + warp) * kHeadRows;
    const int rows_valid = min(kHeadRows, p.n - row0);
    const int row_stride = p.k >> 3, its = p.k >> 8;

    trace_start(p.trace);
    RowsDot<kHeadRows, kHeadUnroll> a;
    const uint4* wrow = p.w + size_t(row0) * row_stride;
    a.load(wrow, row_stride, rows_valid, 0, its, lane);
    pdl_trigger();
    pdl_wait();
    trace_waited(p.trace);
    // the draw of a step is keyed by its position word (read before any CTA can have advanced it)
    const int sample_step = (p.temperature > 0.f && p.pos) ? *p.pos : 0;
    if (NORM_MODE == 5)
        stage_head_f32(reinterpret_cast<const float*>(p.x), reinterpret_cast<const float*>(p.gamma), xs, red, p.k, p.eps);
    else
        stage_activation<(NORM_MODE == 5 ? 0 : NORM_MODE)>(p.x, p.gamma, xs, red, p.k, p.eps, p.x_scale);
    __syncthreads();

    float acc[kHeadRows];
#pragma unroll
    for (int r = 0; r < kHeadRows; ++r) acc[r] = 0.f;
    for (int it0 = 0; it0 < its; it0 += kHeadUnroll) {
        a.fma(xs, it0, its, lane, acc);
        if (it0 + kHeadUnroll < its) a.load(wrow, row_stride, rows_valid, it0 + kHeadUnroll, its, lane);
    }
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    float gumbel = 0.f;                                   // lane r: the variate of this warp's row r
    if (p.temperature > 0.f && lane < rows_valid) gumbel = gumbel_variate(p.seed, sample_step, row0 + lane + p.index_offset);
#pragma unroll
    for (int r = 0; r < kHeadRows; ++r) {
        const float s = round_bf16(warp_sum(acc[r]) * p.out_scale);
        if (r < rows_valid) {
            if (lane == 0 && p.logits) p.logits[row0 + r] = f32_to_bf16_bits(s);
            float score = s;
            if (p.temperature > 0.f) score = __fdiv_rn(s, p.temperature) + __shfl_sync(0xffffffffu, gumbel, r);
            argmax_merge(best, best_i, score, row0 + r);
        }
    }
    if (lane == 0) { wv[warp] = best; wi[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kHeadWarps; ++w) argmax_merge(best, best_i, wv[w], wi[w]);
        p.scratch_val[blockIdx.x] = best;
        p.scratch_idx[blockIdx.x] = best_i;
        __threadfence();
        const unsigned ticket = atomicAdd(p.counter, 1u);
        s_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) { trace_end(p.trace); return; }
    __threadfence();
    best = -INFINITY;
    best_i = 0x7fffffff;
    for (int c = threadIdx.x; c < int(gridDim.x); c += blockDim.x)
        argmax_merge(best, best_i, __ldcg(p.scratch_val + c), __ldcg(p.scratch_idx + c));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        argmax_merge(best, best_i, ov, oi);
    }
    if (lane == 0) { wv[warp] = best; wi[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kHeadWarps; ++w) argmax_merge(best, best_i, wv[w], wi[w]);
        if (p.pair_out) {                       // vocabulary-parallel: hand (logit, global index) to the gather
            p.pair_out[0] = best;
            p.pair_out[1] = float(best_i + p.index_offset);
        }
        if (p.token_out) *p.token_out = best_i + p.index_offset;
        if (!p.pair_out && p.tokens && p.pos) {
            const int cur = *p.pos;
            const bool ended = p.stop_at != nullptr && *p.stop_at != 0;   // the sequence met an end token: nothing moves
            if (!ended && cur + 1 < p.max_tokens) {
                if (cur + 1 >= p.n_prompt) {
                    p.tokens[cur + 1] = best_i;
                    for (int e = 0; e < p.n_eos; ++e)
                        if (p.eos_ids[e] == (long long)(best_i + p.index_offset)) *p.stop_at = cur + 1;
                }
                *p.pos = cur + 1;
            }
        }
        *p.counter = 0;
    }
    trace_end(p.trace);
}

cudaError_t lm_head_dispatch(const HeadParams& p, int norm_mode, cudaStream_t stream, bool pdl) {
    const size_t smem = (size_t(p.k) + 32) * sizeof(float);
    const dim3 grid(lm_head_ctas(p.n)), block(kHeadWarps * 32);
    if (norm_mode == 0) return launch_kernel(lm_head_kernel<0>, grid, block, smem, stream, pdl, p);
    if (norm_mode == 1) return launch_kernel(lm_head_kernel<1>, grid, block, smem, stream, pdl, p);
    if (norm_mode == 2) return launch_kernel(lm_head_kernel<2>, grid, block, smem, stream, pdl, p);
    if (norm_mode == 5) return launch_kernel(lm_head_kernel<5>, grid, block, smem, stream, pdl, p);
    return cudaErrorInvalidValue;
}

// ---- f32-activation helpers (embedding rows widened, RMSNorm with an f32 gain, plain add) ----
__global__ void embed_f32_kernel(const uint16_t* __restrict__ table, const long long* __restrict__ ids,
                                 const long long* __restrict__ tokens, const int* __restrict__ pos,
                                 float* __restrict__ out, int hidden, long long vocab) {
    pdl_trigger();
    pdl_wait();
    long long id = tokens ? tokens[*pos] : ids[blockIdx.x];
    if (id < 0) id = 0;
    if (id >= vocab) id = vocab - 1;
    const uint16_t* src = table + size_t(id) * hidden;
    float* dst = out + size_t(blockIdx.x) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = bf16_bits_to_f32(src[i]);
}
cudaError_t embed_f32_launch(const uint16_t* table, const long long* ids, const long long* tokens, const int* pos,
                             float* out, int rows, int hidden, long long vocab, cudaStream_t stream, bool pdl) {
    return launch_kernel(embed_f32_kernel, dim3(rows), dim3(256), 0, stream, pdl, table, ids, tokens, pos, out, hidden, vocab);
}

__global__ void rmsnorm_f32_kernel(const float* __restrict__ x, const float* __restrict__ gamma, float* __restrict__ y,
                                   int width, float eps) {
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const float* xr = x + size_t(blockIdx.x) * width;
    float* yr = y + size_t(blockIdx.x) * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / float(width) + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) yr[i] = xr[i] * rstd * gamma[i];
}
cudaError_t rmsnorm_f32_launch(const float* x, const float* gamma, float* y, int rows, int width, float eps,
                               cudaStream_t stream, bool pdl) {
    return launch_kernel(rmsnorm_f32_kernel, dim3(rows), dim3(256), 0, stream, pdl, x, gamma, y, width, eps);
}

__global__ void residual_add_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int n) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}
cudaError_t residual_add_f32_launch(const float* a, const float* b, float* out, int n, cudaStream_t stream, bool pdl) {
    return launch_kernel(residual_add_f32_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, pdl, a, b, out, n);
}

// ---- nucleus (top-p) sampling over a row of bf16 logits -----------------------------------------------------------
// The nucleus: walk the distinct logit VALUES from the largest down, adding count(value) * exp((value - max) / T); the
// first value at which the running mass reaches top_p * (total mass) is the threshold, and every token whose logit is
// at least that value belongs (ties included).  bf16 logits have at most 65536 distinct values, so the walk is over a
// histogram of integer counts (exact, whatever the order of the atomics) and the masses are f64: the threshold does not
// depend on summation order beyond the last bit of a double.  Inside the nucleus the pick is the Gumbel-max rule of the
// head kernel (same variates), so top_p = 1 draws what the head kernel draws.
// The kernel follows a decode step that kept its logits; it replaces the token that step wrote.
__device__ __forceinline__ unsigned bf16_key(uint16_t b) { return (b & 0x8000u) ? (~unsigned(b) & 0xffffu) : (unsigned(b) | 0x8000u); }
__device__ __forceinline__ float bf16_of_key(unsigned key) {
    return bf16_bits_to_f32(uint16_t((key & 0x8000u) ? (key & 0x7fffu) : (~key & 0xffffu)));
}
constexpr int kTopPThreads = 1024;
constexpr int kTopPCtas = 32;

// Scratch words after the 65536 counts: [0] ticket of the first kernel, [1] largest key, [2] threshold key, [3] ticket of
// the second kernel, [4 ..] the CTAs' best (score bits, index) pairs.
constexpr int kTopPScratch = 65536;

// First kernel: every CTA counts its slice of the logits into the histogram (atomics from 32 multiprocessors at once);
// the last CTA to finish walks the values and leaves the threshold key.
__global__ void __launch_bounds__(kTopPThreads) top_p_threshold_kernel(const TopPParams p) {
    __shared__ double s_part[kTopPThreads];
    __shared__ unsigned s_maxkey;
    __shared__ int s_last;
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x;
    if (p.stop_at && *p.stop_at != 0) return;                  // the sequence has ended (the same for every CTA)
    const int slot = *p.pos, step = *p.prev_pos;               // the step before moved pos from `step` to `slot`
    if (slot == step || slot < p.n_prompt) return;             // it did not advance, or the slot belongs to the prompt
    int* const ticket = p.hist + kTopPScratch;
    unsigned* const gmax = reinterpret_cast<unsigned*>(p.hist + kTopPScratch + 1);
    if (tid == 0) s_maxkey = 0u;
    __syncthreads();
    unsigned mk = 0u;
    for (int i = blockIdx.x * kTopPThreads + tid; i < p.vocab; i += gridDim.x * kTopPThreads) {
        const unsigned key = bf16_key(p.logits[i]);
        atomicAdd(p.hist + key, 1);
        mk = max(mk, key);
    }
    atomicMax(&s_maxkey, mk);
    __syncthreads();
    if (tid == 0) {
        atomicMax(gmax, s_maxkey);
        __threadfence();
        s_last = atomicAdd(ticket, 1) == int(gridDim.x) - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const double m = double(bf16_of_key(__ldcg(gmax))), inv_t = 1.0 / double(p.temperature);
    // thread t owns keys 65535 - 64 t down to 65535 - 64 t - 63
    constexpr int PER = 65536 / kTopPThreads;
    double mine = 0.0;
    for (int q = 0; q < PER; ++q) {
        const unsigned key = 65535u - unsigned(tid * PER + q);
        const int c = __ldcg(p.hist + key);
        if (c) mine += double(c) * exp((double(bf16_of_key(key)) - m) * inv_t);
    }
    s_part[tid] = mine;
    __syncthreads();
    if (tid == 0) {                                            // the walk over the threads' masses, in key order
        double total = 0.0;
        for (int t = 0; t < kTopPThreads; ++t) total += s_part[t];
        const double target = double(p.top_p) * total;
        double run = 0.0;
        unsigned tau = 0u;
        bool found = false;
        for (int t = 0; t < kTopPThreads && !found; ++t) {
            if (run + s_part[t] < target) { run += s_part[t]; continue; }
            for (int q = 0; q < PER && !found; ++q) {          // the crossing lies among this thread's keys
                const unsigned key = 65535u - unsigned(t * PER + q);
                const int c = __ldcg(p.hist + key);
                if (c == 0) continue;
                run += double(c) * exp((double(bf16_of_key(key)) - m) * inv_t);
                if (run >= target) { tau = key; found = true; }
            }
            // (if rounding left the crossing to the next thread's keys, the walk goes on there)
        }
        p.hist[kTopPScratch + 2] = int(tau);                   // (0 if never reached: every token belongs)
        *ticket = 0;
        *gmax = 0u;
    }
}

// Second kernel: the Gumbel-max pick inside the nucleus, every CTA over its slice (two double-precision logarithms per
// token of the nucleus: too many for one multiprocessor); the last CTA to finish merges, writes the token, applies the
// end-of-sequence latch and zeroes the histogram for the next call.
__global__ void __launch_bounds__(kTopPThreads) top_p_pick_kernel(const TopPParams p) {
    __shared__ float s_val[kTopPThreads / 32];
    __shared__ int s_idx[kTopPThreads / 32];
    __shared__ int s_last;
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (p.stop_at && *p.stop_at != 0) return;
    const int slot = *p.pos, step = *p.prev_pos;
    if (slot == step || slot < p.n_prompt) return;
    const unsigned tau = unsigned(__ldcg(p.hist + kTopPScratch + 2));
    int* const ticket = p.hist + kTopPScratch + 3;
    int* const pairs = p.hist + kTopPScratch + 4;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = blockIdx.x * kTopPThreads + tid; i < p.vocab; i += gridDim.x * kTopPThreads) {
        const uint16_t b = p.logits[i];
        if (bf16_key(b) < tau) continue;
        const float sc = __fdiv_rn(bf16_bits_to_f32(b), p.temperature) + gumbel_variate(p.seed, step, i);
        if (sc > best || (sc == best && i < best_i)) { best = sc; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < kTopPThreads / 32; ++w)
            if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) { best = s_val[w]; best_i = s_idx[w]; }
        pairs[2 * blockIdx.x] = __float_as_int(best);
        pairs[2 * blockIdx.x + 1] = best_i;
        __threadfence();
        s_last = atomicAdd(ticket, 1) == int(gridDim.x) - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int k = tid; k < 65536; k += kTopPThreads) p.hist[k] = 0;      // clean for the next call
    if (tid == 0) {
        best = -INFINITY;
        best_i = 0x7fffffff;
        for (int c = 0; c < int(gridDim.x); ++c) {
            const float ov = __int_as_float(__ldcg(pairs + 2 * c));
            const int oi = __ldcg(pairs + 2 * c + 1);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        p.tokens[slot] = best_i;
        if (p.picked) *p.picked = best_i;
        if (p.threshold_out) *p.threshold_out = bf16_of_key(tau);
        for (int e = 0; e < p.n_eos; ++e)
            if (p.eos_ids[e] == (long long)best_i) *p.stop_at = slot;
        *ticket = 0;
    }
}

cudaError_t sample_top_p_launch(const TopPParams& p, cudaStream_t stream, bool pdl) {
    const cudaError_t e = launch_kernel(top_p_threshold_kernel, dim3(kTopPCtas), dim3(kTopPThreads), 0, stream, pdl, p);
    if (e != cudaSuccess) return e;
    return launch_kernel(top_p_pick_kernel, dim3(kTopPCtas), dim3(kTopPThreads), 0, stream, pdl, p);
}

}  // namespace tfb
