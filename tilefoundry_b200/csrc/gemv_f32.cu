// Batch-1 weight-streaming projections for models whose activations are f32 and whose contracted
// weights are bf16 (examples/qwen3_5_35b_a3b-tilelang/model.py:189,214-225): the activation is rounded
// to bf16 on its way into the product, the product's result is rounded to bf16 and carried on as f32.
//
//   y = epilogue(bf16(W . bf16(prologue(x))))
//
// prologue 0: x as is; 1: RMSNorm with an f32 gain over the whole vector; 4: RMSNorm per segment of
// `seg` elements (one head) with an f32 gain of `seg` elements, times silu(gate) -- the Gated DeltaNet
// output norm (model.py:224).  epilogue 0: store; 1: residual + y; 2: silu(y1) * y2 (one rounding).
//
// HBM-bound like the bf16 kernel: algorithmic bytes per launch = n*k*2 (x2 for SwiGLU).
// Expert mode: output rows are grouped in slots of rows_per_expert; the first routed_slots slots read the
// rows of expert expert_idx[slot], later slots read consecutive rows of w_extra (the shared expert).
#include "gemv.cuh"
#include "route.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

template <int MAXC, int NORM_MODE>
__device__ __forceinline__ void stage_f32(const float* __restrict__ x, const float* __restrict__ gate, const float* gs,
                                          float* xs, float* red, int k, float eps, int seg) {
    float4* dst = reinterpret_cast<float4*>(xs);
    const int pieces = k >> 3;
    float ss = 0.f;
#pragma unroll
    for (int m = 0; m < MAXC; ++m) {
        const int c = threadIdx.x + m * blockDim.x;
        if (c >= pieces) continue;                       // k is a multiple of 256: whole warps leave together
        const float4 lo = *reinterpret_cast<const float4*>(x + (c << 3)), hi = *reinterpret_cast<const float4*>(x + (c << 3) + 4);
        float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        if (NORM_MODE == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = round_bf16(f[i]);
        } else {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) s = fmaf(f[i], f[i], s);
            if (NORM_MODE == 1) ss += s;
            if (NORM_MODE == 4) {                        // seg/8 neighbouring lanes hold one segment
                for (int o = seg >> 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                const float rstd = rsqrtf(s / float(seg) + eps);
                const float4 ga = *reinterpret_cast<const float4*>(gate + (c << 3)), gb = *reinterpret_cast<const float4*>(gate + (c << 3) + 4);
                const float z[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
                const float* gm = gs + ((c << 3) % seg);
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = round_bf16(f[i] * rstd * gm[i] * silu_f32(z[i]));
            }
        }
        const int it = c >> 5, lane = c & 31;
        dst[(it * 2) * 32 + lane] = make_float4(f[0], f[1], f[2], f[3]);
        dst[(it * 2 + 1) * 32 + lane] = make_float4(f[4], f[5], f[6], f[7]);
    }
    if (NORM_MODE != 1) return;
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / float(k) + eps);
#pragma unroll
    for (int m = 0; m < MAXC; ++m) {                     // each thread rescales the pieces it wrote itself
        const int c = threadIdx.x + m * blockDim.x;
        if (c >= pieces) continue;
        const int it = c >> 5, lane = c & 31;
        const float4 lo = dst[(it * 2) * 32 + lane], hi = dst[(it * 2 + 1) * 32 + lane];
        const float* gm = gs + (c << 3);
        dst[(it * 2) * 32 + lane] = make_float4(round_bf16(lo.x * rstd * gm[0]), round_bf16(lo.y * rstd * gm[1]),
                                                round_bf16(lo.z * rstd * gm[2]), round_bf16(lo.w * rstd * gm[3]));
        dst[(it * 2 + 1) * 32 + lane] = make_float4(round_bf16(hi.x * rstd * gm[4]), round_bf16(hi.y * rstd * gm[5]),
                                                    round_bf16(hi.z * rstd * gm[6]), round_bf16(hi.w * rstd * gm[7]));
    }
}

template <int ROWS, int KSPLIT, int WARPS, int UNROLL, int NORM_MODE, int EPI>
__global__ void __launch_bounds__(WARPS * 32) gemv_f32_kernel(const GemvF32Params p) {
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;                         // k floats
    float* red = smem + p.k;                  // 32 floats
    float* part = red + 32;                   // WARPS * ROWS * 2
    float* gs = part + WARPS * ROWS * 2;      // parked norm gains: k floats (mode 1) or seg floats (mode 4)

    constexpr int GROUPS = WARPS / KSPLIT;
    constexpr int NMAT = (EPI == 2) ? 2 : 1;
    constexpr int MAXC = 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = warp / KSPLIT, ks = warp % KSPLIT;
    const int row0 = (blockIdx.x * GROUPS + group) * ROWS;
    const int rows_valid = max(0, min(ROWS, p.n - row0));
    const int row_stride = p.k >> 3;
    const int its = p.k >> 8;
    const int it_per = (its + KSPLIT - 1) / KSPLIT;
    const int it_begin = ks * it_per, it_end = min(its, it_begin + it_per);

    trace_start(p.trace);
    RowsDot<ROWS, UNROLL> a, b;
    const bool expert_mode = p.rows_per_expert > 0;
    const int r0c = min(row0, max(p.n - 1, 0));
    const int slot = expert_mode ? r0c / p.rows_per_expert : 0, within = expert_mode ? r0c % p.rows_per_expert : 0;
    const bool routed = expert_mode && slot < p.routed_slots;
    const uint4* wrow = p.w + size_t(r0c) * row_stride;
    const uint4* w2row = (EPI == 2) ? p.w2 + size_t(r0c) * row_stride : nullptr;
    if (expert_mode && !routed) {
        const size_t erow = size_t(slot - p.routed_slots) * p.rows_per_expert + within;
        wrow = p.w_extra + erow * row_stride;
        if (EPI == 2) w2row = p.w2_extra + erow * row_stride;
    }
    if (!routed) {                            // these rows do not depend on the kernel before: stream them now
        a.load(wrow, row_stride, rows_valid, it_begin, it_end, lane);
        if (EPI == 2) b.load(w2row, row_stride, rows_valid, it_begin, it_end, lane);
    }
    if (NORM_MODE != 0) {
        const int ng = (NORM_MODE == 1) ? p.k : p.seg;
        for (int i = threadIdx.x * 4; i < ng; i += blockDim.x * 4)
            *reinterpret_cast<float4*>(gs + i) = *reinterpret_cast<const float4*>(p.gamma + i);
    }
    pdl_trigger();
    pdl_wait();
    trace_waited(p.trace);

    int rows_live = rows_valid;
    if (routed) {
        long long e = p.expert_idx[slot];
        if (p.expert_world > 1) {                              // another rank owns this expert: nothing to read or write
            if (e % p.expert_world != p.expert_rank) rows_live = 0;
            e /= p.expert_world;
        }
        const size_t erow = size_t(rows_live ? e : 0) * p.rows_per_expert + within;
        wrow = p.w + erow * row_stride;
        if (EPI == 2) w2row = p.w2 + erow * row_stride;
        a.load(wrow, row_stride, rows_live, it_begin, it_end, lane);
        if (EPI == 2) b.load(w2row, row_stride, rows_live, it_begin, it_end, lane);
    }
    float res_early = 0.f;
    if (EPI == 1 && ks == 0 && lane < rows_valid) res_early = p.residual[row0 + lane];

    if (NORM_MODE != 0) __syncthreads();      // parked gains visible
    stage_f32<MAXC, NORM_MODE>(p.x, p.gate, gs, xs, red, p.k, p.eps, p.seg);
    __syncthreads();
    trace_mark(p.trace, 0);

    float acc[ROWS], acc2[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) { acc[r] = 0.f; acc2[r] = 0.f; }
    for (int it0 = it_begin; it0 < it_end; it0 += UNROLL) {
        a.fma(xs, it0, it_end, lane, acc);
        if (EPI == 2) b.fma(xs, it0, it_end, lane, acc2);
        if (it0 + UNROLL < it_end) {
            a.load(wrow, row_stride, rows_live, it0 + UNROLL, it_end, lane);
            if (EPI == 2) b.load(w2row, row_stride, rows_live, it0 + UNROLL, it_end, lane);
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        acc[r] = warp_sum(acc[r]);
        if (EPI == 2) acc2[r] = warp_sum(acc2[r]);
    }
    if (KSPLIT > 1) {
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                part[((group * KSPLIT + ks) * ROWS + r) * NMAT] = acc[r];
                if (EPI == 2) part[((group * KSPLIT + ks) * ROWS + r) * NMAT + 1] = acc2[r];
            }
        }
        __syncthreads();
        if (ks != 0) return;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float s = 0.f, s2 = 0.f;
#pragma unroll
            for (int q = 0; q < KSPLIT; ++q) {
                s += part[((group * KSPLIT + q) * ROWS + r) * NMAT];
                if (EPI == 2) s2 += part[((group * KSPLIT + q) * ROWS + r) * NMAT + 1];
            }
            acc[r] = s;
            acc2[r] = s2;
        }
    }
    if (lane < rows_live) {
        float v = 0.f, v2 = 0.f;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (lane == r) { v = acc[r]; v2 = acc2[r]; }
        const int row = row0 + lane;
        if (EPI == 0) p.y[row] = round_bf16(v);
        else if (EPI == 1) p.y[row] = res_early + round_bf16(v);
        else p.y[row] = round_bf16(silu_f32(round_bf16(v)) * round_bf16(v2));
    }
    if (EPI == 0 && KSPLIT == 1 && p.route_counter != nullptr) {
        // Router launch: the last CTA to finish (an atomic ticket, no spinning) selects the top-k from the logits
        // the grid has just written -- softmax over all experts, top-k, renormalise -- so the selection needs no
        // launch of its own.
        __shared__ int s_last;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_last = atomicAdd(p.route_counter, 1u) == gridDim.x - 1;
        __syncthreads();
        if (s_last && warp == 0) {
            __threadfence();
            float rw;
            int re;
            route_select<256>(p.y, nullptr, p.route_experts, p.route_top_k, 1, lane, rw, re);
            if (lane < p.route_top_k) { p.idx_out[lane] = re; p.w_out[lane] = rw; }
            if (lane == 0) *p.route_counter = 0;
        }
    }
    trace_end(p.trace);
}

template <int ROWS, int KSPLIT, int WARPS, int UNROLL, int NORM_MODE, int EPI>
static cudaError_t launch_cfg(const GemvF32Params& p, cudaStream_t stream, bool pdl) {
    constexpr int GROUPS = WARPS / KSPLIT;
    const int rows_per_cta = GROUPS * ROWS;
    const unsigned grid = (p.n + rows_per_cta - 1) / rows_per_cta;
    const size_t gains = NORM_MODE == 1 ? size_t(p.k) : NORM_MODE == 4 ? size_t(p.seg) : 0;
    const size_t smem = (size_t(p.k) + 32 + WARPS * ROWS * 2 + gains) * sizeof(float);
    auto kern = gemv_f32_kernel<ROWS, KSPLIT, WARPS, UNROLL, NORM_MODE, EPI>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
    }
    return launch_kernel(kern, dim3(grid), dim3(WARPS * 32), smem, stream, pdl, p);
}

template <int NORM_MODE, int EPI>
static cudaError_t pick_shape(const GemvF32Params& p, cudaStream_t stream, bool pdl) {
    // same shape choice as the bf16 kernel, measured there
    if (EPI == 2) return launch_cfg<2, 2, 4, 4, NORM_MODE, EPI>(p, stream, pdl);
    if (p.k >= 4096) return launch_cfg<2, 4, 8, 4, NORM_MODE, EPI>(p, stream, pdl);
    if (p.k > 2048) return launch_cfg<2, 2, 4, 4, NORM_MODE, EPI>(p, stream, pdl);
    return launch_cfg<1, 1, 8, 8, NORM_MODE, EPI>(p, stream, pdl);
}

cudaError_t gemv_f32_dispatch(const GemvF32Params& p, int norm_mode, int epi, cudaStream_t stream, bool pdl) {
#define TFB_CASE(NM, EP) \
    if (norm_mode == NM && epi == EP) return pick_shape<NM, EP>(p, stream, pdl);
    TFB_CASE(0, 0) TFB_CASE(1, 0) TFB_CASE(0, 1) TFB_CASE(4, 1) TFB_CASE(1, 2) TFB_CASE(0, 2) TFB_CASE(4, 0)
#undef TFB_CASE
    return cudaErrorInvalidValue;
}

}  // namespace tfb
