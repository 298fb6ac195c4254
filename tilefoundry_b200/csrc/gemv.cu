// Batch-1 weight-streaming projections: y = epilogue(W . prologue(x)).
//
// HBM-bound: per output row the kernel reads 2k bytes of weights once and does 2k
// flops.  Algorithmic bytes per launch = n*k*2 (x2 for SwiGLU) -- activations are
// a few KB and stay in L2.
#include "gemv.cuh"
#include "kernels.h"
#include "launch.h"

#include <cstdio>
#include <cstdlib>

namespace tfb {


// WARPS warps per CTA; KSPLIT of them share one group of ROWS rows, each taking a
// contiguous slice of K.  EPI: 0 store bf16, 1 residual, 2 SwiGLU, 3 store f32.
template <int ROWS, int KSPLIT, int WARPS, int UNROLL, int NORM_MODE, int EPI>
__device__ __forceinline__ void gemv_body(const GemvParams& p, const int bid, const int nblocks) {
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;                         // k floats
    float* red = smem + p.k;                  // 32 floats
    float* part = red + 32;                   // (WARPS/KSPLIT) * KSPLIT * ROWS * (EPI==2 ? 2 : 1)

    constexpr int GROUPS = WARPS / KSPLIT;
    constexpr int NMAT = (EPI == 2) ? 2 : 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = warp / KSPLIT, ks = warp % KSPLIT;
    const int row0 = (bid * GROUPS + group) * ROWS;
    const int rows_valid = min(ROWS, p.n - row0);
    const int row_stride = p.k >> 3;                       // uint4 per row
    const int its = p.k >> 8;                              // 256 elements per warp iteration
    const int it_per = (its + KSPLIT - 1) / KSPLIT;
    const int it_begin = ks * it_per, it_end = min(its, it_begin + it_per);

    trace_start(p.trace);
    // Weights do not depend on the preceding kernel: start streaming them now.
    RowsDot<ROWS, UNROLL> a, b;
    // Expert mode: output rows are grouped in slots of rows_per_expert; slot s reads the rows of
    // expert expert_idx[s] (a device array the router wrote), so its loads must follow the wait.
    const bool routed = p.expert_idx != nullptr;
    const uint4* wrow = p.w + size_t(max(row0, 0)) * row_stride;
    const uint4* w2row = (EPI == 2) ? p.w2 + size_t(row0) * row_stride : nullptr;
    if (!routed) {
        a.load(wrow, row_stride, rows_valid, it_begin, it_end, lane);
        if (EPI == 2) b.load(w2row, row_stride, rows_valid, it_begin, it_end, lane);
    }
    if (threadIdx.x == 0) l2_prefetch_slice(p.prefetch, p.prefetch_bytes, bid, nblocks);
    constexpr int MAXC = 4;
    const bool fast_stage = (p.k >> 3) <= MAXC * WARPS * 32;
    uint4* gs = reinterpret_cast<uint4*>(part + WARPS * ROWS * 2);     // parked norm gains
    if (fast_stage) StagedGain<MAXC>::template preload<NORM_MODE>(p.gamma, gs, p.k);

    pdl_trigger();
    pdl_wait();
    trace_waited(p.trace);

    bool skip_rows = false;
    if (routed) {
        const int slot = max(row0, 0) / p.rows_per_expert, within = max(row0, 0) % p.rows_per_expert;
        long long e = p.expert_idx[min(slot, p.n / p.rows_per_expert - 1)];
        if (p.expert_world > 1) {
            if (e % p.expert_world != p.expert_rank) skip_rows = true;       // another rank owns this expert
            e /= p.expert_world;
        }
        const size_t erow = size_t(e) * p.rows_per_expert + within;
        wrow = p.w + erow * row_stride;
        if (EPI == 2) w2row = p.w2 + erow * row_stride;
        a.load(wrow, row_stride, skip_rows ? 0 : rows_valid, it_begin, it_end, lane);
        if (EPI == 2) b.load(w2row, row_stride, skip_rows ? 0 : rows_valid, it_begin, it_end, lane);
    }
    // the residual is needed last but its load is issued first: one round trip less at the end
    float res_early = 0.f;
    if (EPI == 1 && KSPLIT == 1 && lane < rows_valid) res_early = bf16_bits_to_f32(p.residual[row0 + lane]);
    if (EPI == 1 && KSPLIT > 1 && ks == 0 && lane < rows_valid) res_early = bf16_bits_to_f32(p.residual[row0 + lane]);

    if (fast_stage) StagedGain<MAXC>::template stage<NORM_MODE>(p.x, p.x2, gs, xs, red, p.k, p.eps, p.x_scale);
    else stage_activation<NORM_MODE>(p.x, p.gamma, xs, red, p.k, p.eps, p.x_scale);
    __syncthreads();
    trace_mark(p.trace, 0);

    float acc[ROWS], acc2[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) { acc[r] = 0.f; acc2[r] = 0.f; }

    for (int it0 = it_begin; it0 < it_end; it0 += UNROLL) {
        a.fma(xs, it0, it_end, lane, acc);
        if (EPI == 2) b.fma(xs, it0, it_end, lane, acc2);
        if (it0 + UNROLL < it_end) {
            a.load(wrow, row_stride, skip_rows ? 0 : rows_valid, it0 + UNROLL, it_end, lane);
            if (EPI == 2) b.load(w2row, row_stride, skip_rows ? 0 : rows_valid, it0 + UNROLL, it_end, lane);
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
            for (int q = 0; q < KSPLIT; ++q) {         // fixed order: deterministic
                s += part[((group * KSPLIT + q) * ROWS + r) * NMAT];
                if (EPI == 2) s2 += part[((group * KSPLIT + q) * ROWS + r) * NMAT + 1];
            }
            acc[r] = s;
            acc2[r] = s2;
        }
    }

    if (lane < rows_valid) {
        float v = 0.f, v2 = 0.f;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (lane == r) { v = acc[r]; v2 = acc2[r]; }
        const int row = row0 + lane;
        if (EPI == 0) {
            static_cast<uint16_t*>(p.y)[row] = f32_to_bf16_bits(v);
        } else if (EPI == 1) {
            float o = round_bf16(v);
            if (p.res_scale != 1.f) o = round_bf16(o * p.res_scale);
            static_cast<uint16_t*>(p.y)[row] = f32_to_bf16_bits(res_early + o);
        } else if (EPI == 2) {
            const float g = round_bf16(v), u = round_bf16(v2);
            static_cast<uint16_t*>(p.y)[row] = f32_to_bf16_bits(round_bf16(silu_f32(g)) * u);
        } else {
            static_cast<float*>(p.y)[row] = v * p.out_scale;
        }
    }
    trace_end(p.trace);
}

template <int ROWS, int KSPLIT, int WARPS, int UNROLL, int NORM_MODE, int EPI>
__global__ void __launch_bounds__(WARPS * 32) gemv_kernel(const GemvParams p) {
    gemv_body<ROWS, KSPLIT, WARPS, UNROLL, NORM_MODE, EPI>(p, blockIdx.x, gridDim.x);
}

// Two independent projections in ONE launch: the first ctas_a CTAs work on `a`, the rest on `b` (MiniCPM3's q and kv
// up-projections both read the low-rank vector the launch before them wrote; examples/minicpm3_4b-cutedsl runs them
// as one "pair" kernel too, kernels/cute_gemv.py).  Same arithmetic as two launches, one launch latency.
template <int ROWS, int KSPLIT, int WARPS, int UNROLL, int NORM_MODE, int EPI>
__global__ void __launch_bounds__(WARPS * 32) gemv_pair_kernel(const GemvParams a, const GemvParams b, const int ctas_a) {
    if (int(blockIdx.x) < ctas_a) gemv_body<ROWS, KSPLIT, WARPS, UNROLL, NORM_MODE, EPI>(a, blockIdx.x, ctas_a);
    else gemv_body<ROWS, KSPLIT, WARPS, UNROLL, NORM_MODE, EPI>(b, blockIdx.x - ctas_a, gridDim.x - ctas_a);
}

template <int ROWS, int UNROLL, int NORM_MODE, int EPI>
static cudaError_t launch_pair_cfg(const GemvParams& a, const GemvParams& b, cudaStream_t stream, bool pdl) {
    constexpr int KSPLIT = 1, WARPS = 8;
    const unsigned ca = (a.n + WARPS * ROWS - 1) / (WARPS * ROWS), cb = (b.n + WARPS * ROWS - 1) / (WARPS * ROWS);
    const int kmax = a.k > b.k ? a.k : b.k;
    const size_t smem = (size_t(kmax) + 32 + WARPS * ROWS * 2) * sizeof(float) + (NORM_MODE ? size_t(kmax) * 2 : 0);
    auto kern = gemv_pair_kernel<ROWS, KSPLIT, WARPS, UNROLL, NORM_MODE, EPI>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
    }
    return launch_kernel(kern, dim3(ca + cb), dim3(WARPS * 32), smem, stream, pdl, a, b, int(ca));
}

template <int NORM_MODE, int EPI>
static cudaError_t launch_pair(const GemvParams& a, const GemvParams& b, cudaStream_t stream, bool pdl) {
    // Short rows (low-rank up-projections, 0.5-1.5 KB each): four rows per warp, so a CTA streams 16-48 KB instead of
    // 4-12 KB for the same staging and launch cost.  Otherwise the k <= 2048 shape of pick_shape.
    if (a.k <= 1024 && b.k <= 1024) return launch_pair_cfg<4, 4, NORM_MODE, EPI>(a, b, stream, pdl);
    return launch_pair_cfg<1, 8, NORM_MODE, EPI>(a, b, stream, pdl);
}

cudaError_t gemv_pair_dispatch(const GemvParams& a, const GemvParams& b, int norm_mode, int epi, cudaStream_t stream, bool pdl) {
    if (a.k > 2048 || b.k > 2048 || a.expert_idx || b.expert_idx) return cudaErrorInvalidValue;
    if (norm_mode == 0 && epi == 0) return launch_pair<0, 0>(a, b, stream, pdl);
    if (norm_mode == 1 && epi == 0) return launch_pair<1, 0>(a, b, stream, pdl);
    if (norm_mode == 2 && epi == 0) return launch_pair<2, 0>(a, b, stream, pdl);
    return cudaErrorInvalidValue;
}

template <int ROWS, int KSPLIT, int WARPS, int UNROLL, int NORM_MODE, int EPI>
static cudaError_t launch_cfg(const GemvParams& p, cudaStream_t stream, bool pdl) {
    constexpr int GROUPS = WARPS / KSPLIT;
    const int rows_per_cta = GROUPS * ROWS;
    const unsigned grid = (p.n + rows_per_cta - 1) / rows_per_cta;
    // x (f32) + reduce scratch + K-split partials (padded to WARPS*ROWS*2) + parked gains (bf16)
    const size_t smem = (size_t(p.k) + 32 + WARPS * ROWS * 2) * sizeof(float) + (NORM_MODE ? size_t(p.k) * 2 : 0);
    auto kern = gemv_kernel<ROWS, KSPLIT, WARPS, UNROLL, NORM_MODE, EPI>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
    }
    return launch_kernel(kern, dim3(grid), dim3(WARPS * 32), smem, stream, pdl, p);
}

template <int NORM_MODE, int EPI>
static cudaError_t pick_shape(const GemvParams& p, cudaStream_t stream, bool pdl) {
    // Shape choice: enough warps to cover 148 SMs several times over, rows per warp
    // and K-split chosen so one warp streams 4-8 KB.
    const long long bytes = 2ll * p.n * p.k * (EPI == 2 ? 2 : 1);
#ifdef TFB_TUNE
    if (const char* e = getenv("TFB_GEMV_CFG")) {
        int r = 0, ks = 0, w = 0, u = 0;
        if (sscanf(e, "%d,%d,%d,%d", &r, &ks, &w, &u) == 4) {
#define TFB_TRY(R, KS, W, U) \
    if (r == R && ks == KS && w == W && u == U) return launch_cfg<R, KS, W, U, NORM_MODE, EPI>(p, stream, pdl);
            TFB_TRY(1, 1, 4, 8) TFB_TRY(1, 2, 4, 4) TFB_TRY(1, 1, 8, 8) TFB_TRY(1, 2, 8, 4) TFB_TRY(1, 1, 2, 8)
            TFB_TRY(1, 3, 6, 8) TFB_TRY(1, 3, 3, 8) TFB_TRY(1, 6, 6, 4) TFB_TRY(2, 3, 6, 4) TFB_TRY(1, 4, 4, 2)
            TFB_TRY(1, 1, 4, 4) TFB_TRY(2, 1, 4, 4) TFB_TRY(2, 2, 4, 4) TFB_TRY(2, 4, 8, 4) TFB_TRY(2, 1, 4, 8)
#undef TFB_TRY
        }
    }
#endif
    // Measured on B200 (graph of 28 back-to-back launches, one per layer's weights): for k <= 2048
    // the whole row in flight in one batch (UNROLL 8) with 8-warp CTAs is fastest; the wide
    // SwiGLU and k >= 4096 shapes prefer two rows per warp with an in-CTA K split.
    (void)bytes;
    if (EPI == 2) {
        return launch_cfg<2, 2, 4, 4, NORM_MODE, EPI>(p, stream, pdl);
    }
    if (p.k >= 4096) {
        return launch_cfg<2, 4, 8, 4, NORM_MODE, EPI>(p, stream, pdl);
    }
    if (p.k > 2048) {
        return launch_cfg<2, 2, 4, 4, NORM_MODE, EPI>(p, stream, pdl);
    }
    return launch_cfg<1, 1, 8, 8, NORM_MODE, EPI>(p, stream, pdl);
}

cudaError_t gemv_dispatch(const GemvParams& p, int norm_mode, int epi, cudaStream_t stream, bool pdl) {
#define TFB_CASE(NM, EP) \
    if (norm_mode == NM && epi == EP) return pick_shape<NM, EP>(p, stream, pdl);
#ifdef TFB_TUNE
    TFB_CASE(0, 0) TFB_CASE(2, 0) TFB_CASE(0, 1) TFB_CASE(2, 2)
#else
    TFB_CASE(0, 0) TFB_CASE(1, 0) TFB_CASE(2, 0) TFB_CASE(3, 0)
    TFB_CASE(0, 1) TFB_CASE(1, 1) TFB_CASE(2, 1) TFB_CASE(3, 1)
    TFB_CASE(0, 2) TFB_CASE(1, 2) TFB_CASE(2, 2)
    TFB_CASE(0, 3) TFB_CASE(1, 3) TFB_CASE(2, 3)
#endif
#undef TFB_CASE
    return cudaErrorInvalidValue;
}

}  // namespace tfb
