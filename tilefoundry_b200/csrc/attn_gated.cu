// Gated GQA decode attention over a paged f32 KV cache (examples/qwen3_5_35b_a3b-tilelang/model.py:293-417):
// per-head RMSNorm of q and k (f32 gains), rotate-half RoPE on the leading rotary_dim of each head, cache
// append, split-KV softmax, and the sigmoid output gate that the query projection carries beside q.
// Everything is f32; nothing is rounded (the o-projection rounds its input itself).
//
// HBM/L2-bound on the cache: algorithmic bytes per launch = (ctx+1) * hkv * d * 2 (K and V) * 4.
// Grid = (hkv, splits): a CTA owns one KV head and kGatedSplit consecutive positions and serves the
// G = hq/hkv query heads that share it.  The last CTA of a KV head to finish (an atomic ticket, no
// spinning) merges the splits.
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

constexpr int kGatedSplit = 64;
constexpr int kGatedThreads = 256;

int attn_gated_splits(int max_ctx) { return (max_ctx + kGatedSplit - 1) / kGatedSplit; }

template <int D, int G>
__global__ void __launch_bounds__(kGatedThreads) attn_gated_kernel(const GatedAttnParams p) {
    constexpr int NWARP = kGatedThreads / 32;
    constexpr int EPL = D / 32;                       // elements of one vector per lane
    constexpr int HG = (G * D) / kGatedThreads;       // heads per thread in the PV stage (thread owns one dim)
    static_assert((G * D) % kGatedThreads == 0 && HG >= 1 && kGatedThreads % D == 0 && EPL % 4 == 0, "shape");
    constexpr int NGRP = kGatedThreads / D;           // head groups in the PV stage
    static_assert(NGRP * HG == G, "shape");

    __shared__ __align__(16) float vec[G + 2][D];     // q_0..q_{G-1} (scaled), k_new, v_new
    __shared__ float sc[G][kGatedSplit];
    __shared__ float stat_m[G], stat_l[G];
    __shared__ float mrg_w[G][64];
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.x, split = blockIdx.y;
    const int p0 = split * kGatedSplit;

    pdl_trigger();
    pdl_wait();
    const int pos = *p.pos;
    const int total = pos + 1;
    const int n_active = (total + kGatedSplit - 1) / kGatedSplit;
    if (pos < 0 || pos >= p.max_ctx || split >= n_active) return;
    const bool owner = (split == n_active - 1);
    const int p1 = min(p0 + kGatedSplit, total);
    const int n = p1 - p0;                             // positions of this split, the new one included
    const int rd = p.rotary_dim, half = rd >> 1;
    const int rpos = p.rope_pos ? *p.rope_pos : pos;

    // ---- this token's q (G heads), k, v for KV head g: one warp per vector, all in registers ----
    for (int vi = warp; vi < G + 2; vi += NWARP) {
        const float* src;
        if (vi < G) src = p.proj + size_t(g * G + vi) * 2 * D;                       // q half of the q|gate pair
        else if (vi == G) src = p.proj + size_t(p.hq) * 2 * D + size_t(g) * D;
        else src = p.proj + size_t(p.hq) * 2 * D + size_t(p.hkv) * D + size_t(g) * D;
        float x[EPL];
#pragma unroll
        for (int i = 0; i < EPL; ++i) x[i] = src[lane + 32 * i];
        if (vi == G + 1) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) vec[vi][lane + 32 * i] = x[i];
            continue;
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / float(D) + p.eps);
        const float* gm = vi < G ? p.gamma_q : p.gamma_k;
#pragma unroll
        for (int i = 0; i < EPL; ++i) x[i] = x[i] * rstd * gm[lane + 32 * i];
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int e = lane + 32 * i;
            float r = x[i];
            if (e < rd) {                              // partner e +- half sits in the same lane (half % 32 == 0)
                const int pi = (e < half) ? i + half / 32 : i - half / 32;
                float partner = 0.f;
#pragma unroll
                for (int k2 = 0; k2 < EPL; ++k2) if (k2 == pi) partner = x[k2];
                if (e < half) partner = -partner;
                r = __fadd_rn(__fmul_rn(x[i], p.cos_table[size_t(rpos) * rd + e]),
                              __fmul_rn(partner, p.sin_table[size_t(rpos) * rd + e]));
            }
            if (vi < G) r *= p.scale;
            vec[vi][e] = r;
        }
    }
    __syncthreads();

    if (owner) {                                       // append this token's entry
        const int page = p.block_table[pos / p.page_size];
        const size_t base = ((size_t(page) * p.page_size + (pos % p.page_size)) * p.hkv + g) * D;
        for (int i = tid; i < D; i += kGatedThreads) {
            p.k_pool[base + i] = vec[G][i];
            p.v_pool[base + i] = vec[G + 1][i];
            if (p.k_new_out) p.k_new_out[size_t(g) * D + i] = vec[G][i];
            if (p.v_new_out) p.v_new_out[size_t(g) * D + i] = vec[G + 1][i];
        }
    }

    __syncthreads();                                   // the appended row is visible to the whole CTA
    // A split never straddles a page (the page size is a multiple of kGatedSplit): its rows are contiguous in the
    // pool, hkv*D floats apart.
    const int page = p.block_table[p0 / p.page_size];
    const size_t row_stride = size_t(p.hkv) * D;
    const size_t first = (size_t(page) * p.page_size + (p0 % p.page_size)) * p.hkv + g;
    const float* kbase = p.k_pool + first * D;
    const float* vbase = p.v_pool + first * D;

    // ---- scores: a warp takes 4 consecutive positions at a time (all their loads in flight together) ----
    {
        constexpr int V4 = EPL / 4;                    // float4 per lane per row
        float q[G][EPL];
#pragma unroll
        for (int j = 0; j < G; ++j)
#pragma unroll
            for (int i = 0; i < EPL; ++i) q[j][i] = vec[j][(i / 4) * 128 + lane * 4 + (i % 4)];
        for (int r0 = warp * 4; r0 < n; r0 += NWARP * 4) {
            float4 kf[4][V4];
#pragma unroll
            for (int t = 0; t < 4; ++t)
#pragma unroll
                for (int h = 0; h < V4; ++h)
                    kf[t][h] = (r0 + t < n) ? *reinterpret_cast<const float4*>(kbase + (r0 + t) * row_stride + h * 128 + lane * 4)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
#pragma unroll
                for (int j = 0; j < G; ++j) {
                    float s = 0.f;
#pragma unroll
                    for (int h = 0; h < V4; ++h) {
                        s = fmaf(q[j][h * 4 + 0], kf[t][h].x, s);
                        s = fmaf(q[j][h * 4 + 1], kf[t][h].y, s);
                        s = fmaf(q[j][h * 4 + 2], kf[t][h].z, s);
                        s = fmaf(q[j][h * 4 + 3], kf[t][h].w, s);
                    }
                    s = warp_sum(s);
                    if (lane == 0 && r0 + t < n) sc[j][r0 + t] = s;
                }
            }
        }
    }
    __syncthreads();

    for (int j = warp; j < G; j += NWARP) {            // softmax statistics of this split
        float m = -INFINITY;
        for (int i = lane; i < n; i += 32) m = fmaxf(m, sc[j][i]);
        m = warp_max(m);
        float l = 0.f;
        for (int i = lane; i < n; i += 32) {
            const float e = expf(sc[j][i] - m);
            sc[j][i] = e;
            l += e;
        }
        l = warp_sum(l);
        if (lane == 0) { stat_m[j] = m; stat_l[j] = l; }
    }
    __syncthreads();

    // ---- probability-weighted V: a thread owns dimension d of HG heads; each V element is loaded once ----
    const int d = tid % D, j0 = (tid / D) * HG;
    float o[HG];
#pragma unroll
    for (int t = 0; t < HG; ++t) o[t] = 0.f;
    for (int r0 = 0; r0 < n; r0 += 8) {                // 8 independent loads in flight per thread
        float v[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) v[t] = (r0 + t < n) ? vbase[(r0 + t) * row_stride + d] : 0.f;
#pragma unroll
        for (int t = 0; t < 8; ++t)
            if (r0 + t < n) {
#pragma unroll
                for (int h = 0; h < HG; ++h) o[h] = fmaf(sc[j0 + h][r0 + t], v[t], o[h]);
            }
    }
    const int nsplit = p.nsplit;
    if (n_active == 1) {
#pragma unroll
        for (int t = 0; t < HG; ++t) {
            const int head = g * G + j0 + t;
            const float gate = p.proj[size_t(head) * 2 * D + D + d];
            p.out[size_t(head) * D + d] = (o[t] / stat_l[j0 + t]) * (1.f / (1.f + expf(-gate)));
        }
        return;
    }
#pragma unroll
    for (int t = 0; t < HG; ++t) p.part_o[(size_t(g * G + j0 + t) * nsplit + split) * D + d] = o[t];
    if (tid < G) {
        p.part_ml[(size_t(g * G + tid) * nsplit + split) * 2] = stat_m[tid];
        p.part_ml[(size_t(g * G + tid) * nsplit + split) * 2 + 1] = stat_l[tid];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned ticket = atomicAdd(&p.counters[g], 1u);
        s_last = (ticket == unsigned(n_active - 1));
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();

    // ---- merge by the last CTA of this KV head ----
    float num[HG], den[HG], run_m[HG];
#pragma unroll
    for (int t = 0; t < HG; ++t) { num[t] = 0.f; den[t] = 0.f; run_m[t] = -INFINITY; }
    for (int s0 = 0; s0 < n_active; s0 += 64) {
        const int ns = min(64, n_active - s0);
        __syncthreads();
        for (int j = warp; j < G; j += NWARP) {
            const float* ml = p.part_ml + (size_t(g * G + j) * nsplit + s0) * 2;
            const float m0 = lane < ns ? __ldcg(ml + 2 * lane) : -INFINITY;
            const float m1 = lane + 32 < ns ? __ldcg(ml + 2 * (lane + 32)) : -INFINITY;
            const float M = warp_max(fmaxf(m0, m1));
            if (lane < ns) mrg_w[j][lane] = expf(m0 - M);
            if (lane + 32 < ns) mrg_w[j][lane + 32] = expf(m1 - M);
            if (lane == 0) stat_m[j] = M;
        }
        __syncthreads();
#pragma unroll
        for (int t = 0; t < HG; ++t) {
            const int j = j0 + t, head = g * G + j;
            const float* po = p.part_o + (size_t(head) * nsplit + s0) * D + d;
            const float* ml = p.part_ml + (size_t(head) * nsplit + s0) * 2;
            float a = 0.f, b = 0.f;
            for (int s = 0; s < ns; ++s) {
                a = fmaf(mrg_w[j][s], __ldcg(po + size_t(s) * D), a);
                b = fmaf(mrg_w[j][s], __ldcg(ml + 2 * s + 1), b);
            }
            const float M = stat_m[j];
            const float newm = fmaxf(run_m[t], M);
            const float c_old = run_m[t] == -INFINITY ? 0.f : expf(run_m[t] - newm);
            const float c_new = expf(M - newm);
            num[t] = num[t] * c_old + a * c_new;
            den[t] = den[t] * c_old + b * c_new;
            run_m[t] = newm;
        }
    }
#pragma unroll
    for (int t = 0; t < HG; ++t) {
        const int head = g * G + j0 + t;
        const float gate = p.proj[size_t(head) * 2 * D + D + d];
        p.out[size_t(head) * D + d] = (num[t] / den[t]) * (1.f / (1.f + expf(-gate)));
    }
    if (tid == 0) p.counters[g] = 0;
}

// rotate-half RoPE on the leading `rd` elements of each head, the tail copied (partial_rope / partial_rope_kv)
__global__ void partial_rope_f32_kernel(const float* __restrict__ x, const float* __restrict__ cos_table,
                                        const float* __restrict__ sin_table, const int* __restrict__ pos,
                                        float* __restrict__ out, int d, int rd) {
    pdl_trigger();
    pdl_wait();
    const float* xr = x + size_t(blockIdx.x) * d;
    const int half = rd >> 1, at = *pos;
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        float r = xr[e];
        if (e < rd) {
            const float partner = e < half ? -xr[e + half] : xr[e - half];
            r = __fadd_rn(__fmul_rn(xr[e], cos_table[size_t(at) * rd + e]), __fmul_rn(partner, sin_table[size_t(at) * rd + e]));
        }
        out[size_t(blockIdx.x) * d + e] = r;
    }
}
cudaError_t partial_rope_f32_launch(const float* x, const float* cos_table, const float* sin_table, const int* pos,
                                    float* out, int heads, int d, int rd, cudaStream_t stream, bool pdl) {
    return launch_kernel(partial_rope_f32_kernel, dim3(heads), dim3(128), 0, stream, pdl, x, cos_table, sin_table, pos, out, d, rd);
}

cudaError_t attn_gated_dispatch(const GatedAttnParams& p, cudaStream_t stream, bool pdl) {
    const int G = p.hq / p.hkv;
    if (p.rotary_dim % 64 != 0 || p.rotary_dim > p.d) return cudaErrorInvalidValue;
    const dim3 grid(p.hkv, p.nsplit), block(kGatedThreads);
#define TFB_ATTN(DD, GG) \
    if (p.d == DD && G == GG) return launch_kernel(attn_gated_kernel<DD, GG>, grid, block, 0, stream, pdl, p);
    TFB_ATTN(256, 8) TFB_ATTN(128, 2) TFB_ATTN(128, 4) TFB_ATTN(256, 4)
#undef TFB_ATTN
    return cudaErrorInvalidValue;
}

}  // namespace tfb
