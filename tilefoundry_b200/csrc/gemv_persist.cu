// Persistent form of the batch-1 weight-streaming projection y = epilogue(W . prologue(x)).
//
// Same arithmetic, rounding points and fixed reduction order as gemv_kernel (gemv.cu).  The difference is
// how rows are handed out: the grid is sized to what the GPU keeps resident (no partial last wave), a CTA
// stages the activation vector ONCE and then walks its tiles of GROUPS*ROWS output rows in a grid-stride
// loop, and every warp keeps two batches of weights in flight (while batch t is multiplied, batch t+1 is
// landing and batch t+2 is issued), so HBM requests never drain at a tile boundary.  The first two batches
// are issued before the dependency wait.
//
// HBM-bound: algorithmic bytes per launch = n*k*2 (x2 for SwiGLU).
#include "gemv.cuh"
#include "kernels.h"
#include "launch.h"


namespace tfb {

template <int ROWS, int KSPLIT, int WARPS, int UNROLL, int NORM_MODE, int EPI>
__global__ void __launch_bounds__(WARPS * 32) gemv_persist_kernel(const GemvParams p, const int tiles) {
    extern __shared__ __align__(16) float smem[];
    constexpr int GROUPS = WARPS / KSPLIT;
    constexpr int NMAT = (EPI == 2) ? 2 : 1;
    constexpr int PART = WARPS * ROWS * 2;
    float* xs = smem;                         // k floats
    float* red = smem + p.k;                  // 32 floats
    float* part = red + 32;                   // 2 * PART: K-split partials, double-buffered by tile parity
    uint4* gs = reinterpret_cast<uint4*>(part + 2 * PART);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = warp / KSPLIT, ks = warp % KSPLIT;
    const int row_stride = p.k >> 3;
    const int its = p.k >> 8;
    const int it_per = (its + KSPLIT - 1) / KSPLIT;
    const int it_begin = ks * it_per, it_end = min(its, it_begin + it_per);
    const int nch = (it_per + UNROLL - 1) / UNROLL;           // the same for every warp: barriers stay uniform
    const int my_tiles = (tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);
    const int T = my_tiles * nch;

    trace_start(p.trace);
    RowsDot<ROWS, UNROLL> a0, a1, b0, b1;
    auto issue = [&](int t, RowsDot<ROWS, UNROLL>& a, RowsDot<ROWS, UNROLL>& b) {
        const int j = t / nch, c = t - j * nch;
        const int row0 = ((int(blockIdx.x) + j * int(gridDim.x)) * GROUPS + group) * ROWS;
        const int rows_valid = max(0, min(ROWS, p.n - row0));
        const int r0 = min(row0, p.n - 1);
        a.load(p.w + size_t(r0) * row_stride, row_stride, rows_valid, it_begin + c * UNROLL, it_end, lane);
        if (EPI == 2) b.load(p.w2 + size_t(r0) * row_stride, row_stride, rows_valid, it_begin + c * UNROLL, it_end, lane);
    };
    if (T > 0) issue(0, a0, b0);
    if (T > 1) issue(1, a1, b1);
    constexpr int MAXC = 4;
    const bool fast_stage = (p.k >> 3) <= MAXC * WARPS * 32;
    if (fast_stage) StagedGain<MAXC>::template preload<NORM_MODE>(p.gamma, gs, p.k);

    pdl_trigger();
    pdl_wait();
    trace_waited(p.trace);
    if (fast_stage) StagedGain<MAXC>::template stage<NORM_MODE>(p.x, p.x2, gs, xs, red, p.k, p.eps, p.x_scale);
    else stage_activation<NORM_MODE>(p.x, p.gamma, xs, red, p.k, p.eps, p.x_scale);
    __syncthreads();
    trace_mark(p.trace, 0);

    float acc[ROWS], acc2[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) { acc[r] = 0.f; acc2[r] = 0.f; }

    auto consume = [&](int t, RowsDot<ROWS, UNROLL>& a, RowsDot<ROWS, UNROLL>& b) {
        const int j = t / nch, c = t - j * nch;
        a.fma(xs, it_begin + c * UNROLL, it_end, lane, acc);
        if (EPI == 2) b.fma(xs, it_begin + c * UNROLL, it_end, lane, acc2);
        if (c != nch - 1) return;
        // ---- this warp's share of tile j is complete ----
        const int row0 = ((int(blockIdx.x) + j * int(gridDim.x)) * GROUPS + group) * ROWS;
        const int rows_valid = max(0, min(ROWS, p.n - row0));
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            acc[r] = warp_sum(acc[r]);
            if (EPI == 2) acc2[r] = warp_sum(acc2[r]);
        }
        bool writer = true;
        if (KSPLIT > 1) {
            float* pt = part + (j & 1) * PART;
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    pt[((group * KSPLIT + ks) * ROWS + r) * NMAT] = acc[r];
                    if (EPI == 2) pt[((group * KSPLIT + ks) * ROWS + r) * NMAT + 1] = acc2[r];
                }
            }
            __syncthreads();
            writer = ks == 0;
            if (writer) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    float s = 0.f, s2 = 0.f;
#pragma unroll
                    for (int q = 0; q < KSPLIT; ++q) {         // fixed order: deterministic
                        s += pt[((group * KSPLIT + q) * ROWS + r) * NMAT];
                        if (EPI == 2) s2 += pt[((group * KSPLIT + q) * ROWS + r) * NMAT + 1];
                    }
                    acc[r] = s;
                    acc2[r] = s2;
                }
            }
        }
        if (writer && lane < rows_valid) {
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
                static_cast<uint16_t*>(p.y)[row] = f32_to_bf16_bits(bf16_bits_to_f32(p.residual[row]) + o);
            } else if (EPI == 2) {
                const float g = round_bf16(v), u = round_bf16(v2);
                static_cast<uint16_t*>(p.y)[row] = f32_to_bf16_bits(round_bf16(silu_f32(g)) * u);
            } else {
                static_cast<float*>(p.y)[row] = v * p.out_scale;
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) { acc[r] = 0.f; acc2[r] = 0.f; }
    };

    for (int t = 0; t < T; t += 2) {
        consume(t, a0, b0);
        if (t + 2 < T) issue(t + 2, a0, b0);
        if (t + 1 < T) {
            consume(t + 1, a1, b1);
            if (t + 3 < T) issue(t + 3, a1, b1);
        }
    }
    trace_end(p.trace);
}

template <int ROWS, int KSPLIT, int WARPS, int UNROLL, int NORM_MODE, int EPI>
static cudaError_t launch_cfg(const GemvParams& p, cudaStream_t stream, bool pdl) {
    constexpr int GROUPS = WARPS / KSPLIT;
    const int rows_per_tile = GROUPS * ROWS;
    const int tiles = (p.n + rows_per_tile - 1) / rows_per_tile;
    const size_t smem = (size_t(p.k) + 32 + 2 * WARPS * ROWS * 2) * sizeof(float) + (NORM_MODE ? size_t(p.k) * 2 : 0);
    auto kern = gemv_persist_kernel<ROWS, KSPLIT, WARPS, UNROLL, NORM_MODE, EPI>;
    static int occ_dev[kMaxDevices] = {};                 // occupancy and the opt-in it follows from are per device
    static size_t occ_smem_dev[kMaxDevices] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
    int& occ = occ_dev[dev];
    size_t& occ_smem = occ_smem_dev[dev];
    if (occ == 0 || smem > occ_smem) {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
            if (e != cudaSuccess) return e;
        }
        int o = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, kern, WARPS * 32, smem);
        if (e != cudaSuccess) return e;
        occ = o > 0 ? o : 1;
        occ_smem = smem;
    }
    const int cap = sm_count() * occ;
    const int per_cta = (tiles + cap - 1) / cap;                // tiles every CTA walks (the last may get fewer)
    const int grid = (tiles + per_cta - 1) / per_cta;
    return launch_kernel(kern, dim3(grid), dim3(WARPS * 32), smem, stream, pdl, p, tiles);
}

template <int NORM_MODE, int EPI>
static cudaError_t pick_shape(const GemvParams& p, cudaStream_t stream, bool pdl) {
    // One row (pair) per warp, no K split, the whole row in flight as two batches: the shape that measured best
    // for K = 2048 .. 2560.  Wider rows keep an in-CTA K split so a warp's batch stays 2-4 KB.
    if (p.k > 4096) return launch_cfg<1, 2, 8, 4, NORM_MODE, EPI>(p, stream, pdl);
    return launch_cfg<1, 1, 8, 4, NORM_MODE, EPI>(p, stream, pdl);
}

bool gemv_persist_supported(const GemvParams& p, int norm_mode) {
    return p.expert_idx == nullptr && norm_mode != 3;
}

cudaError_t gemv_persist_dispatch(const GemvParams& p, int norm_mode, int epi, cudaStream_t stream, bool pdl) {
#define TFB_CASE(NM, EP) \
    if (norm_mode == NM && epi == EP) return pick_shape<NM, EP>(p, stream, pdl);
    TFB_CASE(0, 0) TFB_CASE(1, 0) TFB_CASE(2, 0)
    TFB_CASE(0, 1) TFB_CASE(1, 1) TFB_CASE(2, 1)
    TFB_CASE(0, 2) TFB_CASE(1, 2) TFB_CASE(2, 2)
#undef TFB_CASE
    return cudaErrorInvalidValue;
}

}  // namespace tfb
