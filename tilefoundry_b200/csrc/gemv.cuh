// Weight-streaming GEMV building blocks shared by the projection and lm_head kernels.
//
// Data layout: W is [n, k] bf16 row-major, so one output's weights are one
// contiguous run of 2k bytes.  A warp owns ROWS consecutive outputs (times a
// K-slice when KSPLIT > 1); lane l reads the 16-byte pieces l, l+32, l+64, ... of
// each row, so every warp-wide load is 512 contiguous bytes.  The activation
// vector is staged once per CTA in shared memory as f32, permuted so that the two
// float4 a lane needs for one 16-byte weight piece are each a conflict-free
// warp-wide float4 read.
#pragma once
#include "common.cuh"

namespace tfb {

// Shared-memory float index of activation element k under the staging permutation:
// piece c = k/8 belongs to (iteration it = c/32, lane = c%32); its first 4 floats go
// to float4 slot (it*2+0)*32+lane, the last 4 to (it*2+1)*32+lane.
__device__ __forceinline__ int xs_index(int k) {
    const int c = k >> 3, j = k & 7;
    const int it = c >> 5, lane = c & 31;
    return (((it * 2 + (j >> 2)) * 32 + lane) << 2) + (j & 3);
}

// Stage x[0..k) (bf16) into xs (f32, permuted) applying the fused prologue.
// All threads of the CTA take part.  `red` is >= 32 floats of shared scratch.
template <int NORM_MODE>
__device__ __forceinline__ void stage_activation(const uint16_t* __restrict__ x,
                                                 const uint16_t* __restrict__ gamma, float* xs,
                                                 float* red, int k, float eps, float x_scale) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    float rstd = 1.f;
    if (NORM_MODE != 0) {
        float ss = 0.f;
        for (int c = tid; c < (k >> 3); c += nthr) {
            const uint4 v = *reinterpret_cast<const uint4*>(x + (c << 3));
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float a = bf16_lo(u[i]), b = bf16_hi(u[i]);
                ss = fmaf(a, a, ss);
                ss = fmaf(b, b, ss);
            }
        }
        ss = block_sum(ss, red);
        rstd = rsqrtf(ss / float(k) + eps);
    }
    for (int c = tid; c < (k >> 3); c += nthr) {
        const uint4 v = *reinterpret_cast<const uint4*>(x + (c << 3));
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[2 * i] = bf16_lo(u[i]); f[2 * i + 1] = bf16_hi(u[i]); }
        if (NORM_MODE != 0) {
            const uint4 gv = *reinterpret_cast<const uint4*>(gamma + (c << 3));
            const uint32_t g[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float g0 = bf16_lo(g[i]), g1 = bf16_hi(g[i]);
                if (NORM_MODE == 2) {          // round, then gain (a bf16 multiply)
                    f[2 * i] = round_bf16(round_bf16(f[2 * i] * rstd) * g0);
                    f[2 * i + 1] = round_bf16(round_bf16(f[2 * i + 1] * rstd) * g1);
                } else {                       // f32 through the gain, one rounding
                    f[2 * i] = round_bf16(f[2 * i] * rstd * g0);
                    f[2 * i + 1] = round_bf16(f[2 * i + 1] * rstd * g1);
                }
            }
        }
        if (x_scale != 1.f) {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = round_bf16(apply_scale(f[i], x_scale));
        }
        const int it = c >> 5, lane = c & 31;
        float4* dst = reinterpret_cast<float4*>(xs);
        dst[(it * 2) * 32 + lane] = make_float4(f[0], f[1], f[2], f[3]);
        dst[(it * 2 + 1) * 32 + lane] = make_float4(f[4], f[5], f[6], f[7]);
    }
}

// Same staging with one memory round trip between the dependency wait and the first dot product:
// the norm gains (weights, so readable before the wait) are parked in shared memory ahead of time,
// x is read from global memory exactly once, and normalisation happens in place in shared memory.
// Nothing is held in registers across the wait, so the weight-load buffers keep the register budget.
// Each thread owns up to MAXC 8-element pieces; callers fall back to stage_activation when
// k/8 > MAXC * blockDim.x.  `gs` is k/8 uint4 of shared memory.
// NORM_MODE 3 ("gated"): the vector normalised is f32(x) * silu(f32(gate)), kept in f32 through the
// gain and rounded once -- granite's gated output norm (rms_norm(y * silu(gate)) * gamma).
template <int MAXC>
struct StagedGain {
    template <int NORM_MODE>
    static __device__ __forceinline__ void preload(const uint16_t* __restrict__ gamma, uint4* gs, int k) {
        if constexpr (NORM_MODE != 0) {
#pragma unroll
            for (int m = 0; m < MAXC; ++m) {
                const int c = threadIdx.x + m * blockDim.x;
                if (c < (k >> 3)) gs[c] = *reinterpret_cast<const uint4*>(gamma + (c << 3));
            }
        }
    }
    template <int NORM_MODE>
    static __device__ __forceinline__ void stage(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate,
                                                 const uint4* gs, float* xs, float* red, int k, float eps,
                                                 float x_scale) {
        uint4 xv[MAXC], gv[NORM_MODE == 3 ? MAXC : 1];
#pragma unroll
        for (int m = 0; m < MAXC; ++m) {
            const int c = threadIdx.x + m * blockDim.x;
            xv[m] = (c < (k >> 3)) ? *reinterpret_cast<const uint4*>(x + (c << 3)) : make_uint4(0, 0, 0, 0);
            if (NORM_MODE == 3)
                gv[m] = (c < (k >> 3)) ? *reinterpret_cast<const uint4*>(gate + (c << 3)) : make_uint4(0, 0, 0, 0);
        }
        float4* dst = reinterpret_cast<float4*>(xs);
        float ss = 0.f;
#pragma unroll
        for (int m = 0; m < MAXC; ++m) {
            const int c = threadIdx.x + m * blockDim.x;
            if (c >= (k >> 3)) continue;
            const uint32_t u[4] = {xv[m].x, xv[m].y, xv[m].z, xv[m].w};
            float f[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) { f[2 * i] = bf16_lo(u[i]); f[2 * i + 1] = bf16_hi(u[i]); }
            if (NORM_MODE == 3) {
                const uint32_t q[4] = {gv[m].x, gv[m].y, gv[m].z, gv[m].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    f[2 * i] *= silu_f32(bf16_lo(q[i]));
                    f[2 * i + 1] *= silu_f32(bf16_hi(q[i]));
                }
            }
            if (NORM_MODE != 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
            } else if (x_scale != 1.f) {
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = round_bf16(apply_scale(f[i], x_scale));
            }
            const int it = c >> 5, lane = c & 31;
            dst[(it * 2) * 32 + lane] = make_float4(f[0], f[1], f[2], f[3]);
            dst[(it * 2 + 1) * 32 + lane] = make_float4(f[4], f[5], f[6], f[7]);
        }
        if (NORM_MODE == 0) return;
        ss = block_sum(ss, red);
        const float rstd = rsqrtf(ss / float(k) + eps);
#pragma unroll
        for (int m = 0; m < MAXC; ++m) {                 // each thread rescales the pieces it wrote itself
            const int c = threadIdx.x + m * blockDim.x;
            if (c >= (k >> 3)) continue;
            const int it = c >> 5, lane = c & 31;
            const float4 lo = dst[(it * 2) * 32 + lane], hi = dst[(it * 2 + 1) * 32 + lane];
            float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            const uint4 g = gs[c];
            const uint32_t gg[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (NORM_MODE == 2) {                    // round, then gain (a bf16 multiply)
                    f[2 * i] = round_bf16(round_bf16(f[2 * i] * rstd) * bf16_lo(gg[i]));
                    f[2 * i + 1] = round_bf16(round_bf16(f[2 * i + 1] * rstd) * bf16_hi(gg[i]));
                } else {                                 // f32 through the gain, one rounding
                    f[2 * i] = round_bf16(f[2 * i] * rstd * bf16_lo(gg[i]));
                    f[2 * i + 1] = round_bf16(f[2 * i + 1] * rstd * bf16_hi(gg[i]));
                }
            }
            if (x_scale != 1.f) {
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = round_bf16(apply_scale(f[i], x_scale));
            }
            dst[(it * 2) * 32 + lane] = make_float4(f[0], f[1], f[2], f[3]);
            dst[(it * 2 + 1) * 32 + lane] = make_float4(f[4], f[5], f[6], f[7]);
        }
    }
};

// Dot products of ROWS weight rows with the staged activation over the 16-byte
// pieces [it_begin, it_end) x 32 lanes.  `w` points at row 0, `row_stride` in
// uint4 units; rows at or beyond `rows_valid` are skipped (their acc stays 0).
// `first` holds pieces loaded ahead of time for iterations it_begin..it_begin+UNROLL-1.
template <int ROWS, int UNROLL>
struct RowsDot {
    uint4 buf[ROWS][UNROLL];

    __device__ __forceinline__ void load(const uint4* __restrict__ w, int row_stride, int rows_valid,
                                         int it0, int it_end, int lane) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int it = it0 + u;
                if (r < rows_valid && it < it_end)
                    buf[r][u] = ld_stream16(w + size_t(r) * row_stride + it * 32 + lane);
                else
                    buf[r][u] = make_uint4(0, 0, 0, 0);
            }
    }

    __device__ __forceinline__ void fma(const float* xs, int it0, int it_end, int lane, float (&acc)[ROWS]) {
        const float4* x4 = reinterpret_cast<const float4*>(xs);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int it = it0 + u;
            if (it < it_end) {
                const float4 xa = x4[(it * 2) * 32 + lane];
                const float4 xb = x4[(it * 2 + 1) * 32 + lane];
#pragma unroll
                for (int r = 0; r < ROWS; ++r) acc[r] = dot8(buf[r][u], xa, xb, acc[r]);
            }
        }
    }
};

}  // namespace tfb
