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
constexpr int kGatedMergeBatch = 16;        // split partials one merging thread requests at once

int attn_gated_splits(int max_ctx) { return (max_ctx + kGatedSplit - 1) / kGatedSplit; }

// GH query heads per CTA: the G heads of a KV head are spread over G/GH CTAs so that a short context still
// occupies tens of SMs and no CTA carries more than GH heads x 64 positions of serial work.
template <int D, int G, int GH>
__global__ void __launch_bounds__(kGatedThreads) attn_gated_kernel(const GatedAttnParams p) {
    constexpr int NWARP = kGatedThreads / 32;
    constexpr int EPL = D / 32;                       // elements of one vector per lane
    constexpr int V4 = EPL / 4;                       // float4 per lane per row
    constexpr int HG = (GH * D) / kGatedThreads;      // heads per thread in the PV stage (thread owns one dim)
    constexpr int NGRP = kGatedThreads / D;           // head groups in the PV stage
    constexpr int NV = GH + 2;                        // vectors prepared: GH queries, the key, the value
    static_assert(G % GH == 0 && (GH * D) % kGatedThreads == 0 && HG >= 1 && kGatedThreads % D == 0 && EPL % 4 == 0 &&
                      NGRP * HG == GH && NV <= NWARP, "shape");

    __shared__ __align__(16) float vec[NV][D];        // q_0..q_{GH-1} (scaled), k_new, v_new
    __shared__ float sc[GH][kGatedSplit];
    __shared__ float stat_m[GH], stat_l[GH];
    __shared__ float mrg_w[GH][64];
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.x / (G / GH), hg = blockIdx.x % (G / GH), split = blockIdx.y;
    const int head0 = g * G + hg * GH;                // first query head of this CTA
    const int p0 = split * kGatedSplit;

    // ---- before the dependency wait: ask L2 for this split's cached rows.  Between two uses of a row a whole
    // step's weights (GBs) stream through L2, so the rows come from HBM; the position word may be a step behind
    // here, which only leaves one row un-prefetched. ----
    if (hg == 0) {
        const int pos_early = *reinterpret_cast<const volatile int*>(p.pos);
        if (pos_early >= 0 && pos_early < p.max_ctx && p0 < pos_early) {
            const int rows = min(kGatedSplit, pos_early - p0);
            const int page_e = p.block_table[p0 / p.page_size];
            const size_t first_e = (size_t(page_e) * p.page_size + (p0 % p.page_size)) * p.hkv + g;
            constexpr int LINES = D * 4 / 128;             // 128-byte lines per row
            for (int i = tid; i < rows * LINES * 2; i += kGatedThreads) {
                const int which = i / (rows * LINES), rest = i % (rows * LINES);
                const float* base = (which ? p.v_pool : p.k_pool) + (first_e + size_t(rest / LINES) * p.hkv) * D + (rest % LINES) * 32;
                asm volatile("prefetch.global.L2 [%0];" :: "l"(base));
            }
        }
    }
    trace_start(p.trace);
    pdl_trigger();
    pdl_wait();
    trace_waited(p.trace);
    // ---- this token's q (GH heads), k, v: one warp per vector; the loads go out before the position is read ----
    float x[EPL], gm[EPL], cs[EPL], sn[EPL];
    const int vi = warp;
    const int rd = p.rotary_dim, half = rd >> 1;
    const int rpos_early = p.rope_pos ? *p.rope_pos : *p.pos;          // issued together with the vector loads
    if (vi < NV) {
        const float* src;
        if (vi < GH) src = p.proj + size_t(head0 + vi) * 2 * D;                      // q half of the q|gate pair
        else if (vi == GH) src = p.proj + size_t(p.hq) * 2 * D + size_t(g) * D;
        else src = p.proj + size_t(p.hq) * 2 * D + size_t(p.hkv) * D + size_t(g) * D;
        const float* gsrc = vi < GH ? p.gamma_q : p.gamma_k;
#pragma unroll
        for (int i = 0; i < EPL; ++i) { x[i] = src[lane + 32 * i]; gm[i] = gsrc[lane + 32 * i]; }
    }
    const int pos = *p.pos;
    const int total = pos + 1;
    const int n_active = (total + kGatedSplit - 1) / kGatedSplit;
    if (pos < 0 || pos >= p.max_ctx || split >= n_active) return;
    const bool owner = (split == n_active - 1);
    const int p1 = min(p0 + kGatedSplit, total);
    const int n = p1 - p0;                             // positions of this split, the new one included
    const int rpos = rpos_early;

    if (vi < NV) {
        if (vi == GH + 1) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) vec[vi][lane + 32 * i] = x[i];
        } else {
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                const int e = lane + 32 * i;
                cs[i] = e < rd ? p.cos_table[size_t(rpos) * rd + e] : 1.f;
                sn[i] = e < rd ? p.sin_table[size_t(rpos) * rd + e] : 0.f;
            }
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < EPL; ++i) ss = fmaf(x[i], x[i], ss);
            ss = warp_sum(ss);
            const float rstd = rsqrtf(ss / float(D) + p.eps);
#pragma unroll
            for (int i = 0; i < EPL; ++i) x[i] = x[i] * rstd * gm[i];
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                const int e = lane + 32 * i;
                float r = x[i];
                if (e < rd) {                          // partner e +- half sits in the same lane (half % 32 == 0)
                    const int pi = (e < half) ? i + half / 32 : i - half / 32;
                    float partner = 0.f;
#pragma unroll
                    for (int k2 = 0; k2 < EPL; ++k2) if (k2 == pi) partner = x[k2];
                    if (e < half) partner = -partner;
                    r = __fadd_rn(__fmul_rn(x[i], cs[i]), __fmul_rn(partner, sn[i]));
                }
                if (vi < GH) r *= p.scale;
                vec[vi][e] = r;
            }
        }
    }
    __syncthreads();
    trace_mark(p.trace, 0);

    if (owner && hg == 0) {                            // append this token's entry (one CTA per KV head)
        const int page = p.block_table[pos / p.page_size];
        const size_t base = ((size_t(page) * p.page_size + (pos % p.page_size)) * p.hkv + g) * D;
        for (int i = tid; i < D; i += kGatedThreads) {
            p.k_pool[base + i] = vec[GH][i];
            p.v_pool[base + i] = vec[GH + 1][i];
            if (p.k_new_out) p.k_new_out[size_t(g) * D + i] = vec[GH][i];
            if (p.v_new_out) p.v_new_out[size_t(g) * D + i] = vec[GH + 1][i];
        }
    }
    // A split never straddles a page (the page size is a multiple of kGatedSplit): its rows are contiguous in the
    // pool, hkv*D floats apart.  The new row is taken from shared memory: the CTA that appends it may be another.
    const int page = p.block_table[p0 / p.page_size];
    const size_t row_stride = size_t(p.hkv) * D;
    const size_t first = (size_t(page) * p.page_size + (p0 % p.page_size)) * p.hkv + g;
    const float* kbase = p.k_pool + first * D;
    const float* vbase = p.v_pool + first * D;
    const int n_cached = owner ? n - 1 : n;            // rows of this split that are in the pool already
    const int r_new = owner ? n - 1 : -1;

    // ---- scores: a warp takes 4-8 consecutive positions at a time (all their loads in flight together) ----
    {
        float q[GH][EPL];
#pragma unroll
        for (int j = 0; j < GH; ++j)
#pragma unroll
            for (int i = 0; i < EPL; ++i) q[j][i] = vec[j][(i / 4) * 128 + lane * 4 + (i % 4)];
        constexpr int PB = 8 / V4;                     // positions a warp loads together (8 float4 per lane)
        for (int r0 = warp * PB; r0 < n; r0 += NWARP * PB) {
            float4 kf[PB][V4];
#pragma unroll
            for (int t = 0; t < PB; ++t)
#pragma unroll
                for (int h = 0; h < V4; ++h) {
                    const int r = r0 + t;
                    if (r < n_cached) kf[t][h] = *reinterpret_cast<const float4*>(kbase + r * row_stride + h * 128 + lane * 4);
                    else if (r == r_new) kf[t][h] = *reinterpret_cast<const float4*>(&vec[GH][h * 128 + lane * 4]);
                    else kf[t][h] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            float s[PB][GH];
#pragma unroll
            for (int t = 0; t < PB; ++t)
#pragma unroll
                for (int j = 0; j < GH; ++j) {
                    float a = 0.f;
#pragma unroll
                    for (int h = 0; h < V4; ++h) {
                        a = fmaf(q[j][h * 4 + 0], kf[t][h].x, a);
                        a = fmaf(q[j][h * 4 + 1], kf[t][h].y, a);
                        a = fmaf(q[j][h * 4 + 2], kf[t][h].z, a);
                        a = fmaf(q[j][h * 4 + 3], kf[t][h].w, a);
                    }
                    s[t][j] = a;
                }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)           // the PB x GH reductions interleaved
#pragma unroll
                for (int t = 0; t < PB; ++t)
#pragma unroll
                    for (int j = 0; j < GH; ++j) s[t][j] += __shfl_xor_sync(0xffffffffu, s[t][j], o);
            if (lane == 0) {
#pragma unroll
                for (int t = 0; t < PB; ++t)
#pragma unroll
                    for (int j = 0; j < GH; ++j)
                        if (r0 + t < n) sc[j][r0 + t] = s[t][j];
            }
        }
    }
    __syncthreads();
    trace_mark(p.trace, 1);

    // the value rows do not depend on the scores: all of the split's loads go out before the softmax
    const int d = tid % D, j0 = (tid / D) * HG;
    float va[32], vb[32];
#pragma unroll
    for (int t = 0; t < 32; ++t) {
        va[t] = t < n_cached ? vbase[t * row_stride + d] : (t == r_new ? vec[GH + 1][d] : 0.f);
        vb[t] = 32 + t < n_cached ? vbase[(32 + t) * row_stride + d] : (32 + t == r_new ? vec[GH + 1][d] : 0.f);
    }
    float gate[HG];                                    // needed last, requested first
#pragma unroll
    for (int t = 0; t < HG; ++t) gate[t] = p.proj[size_t(head0 + j0 + t) * 2 * D + D + d];

    for (int j = warp; j < GH; j += NWARP) {           // softmax statistics of this split
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

    // ---- probability-weighted V: a thread owns dimension d of HG heads ----
    float o[HG];
#pragma unroll
    for (int t = 0; t < HG; ++t) o[t] = 0.f;
#pragma unroll
    for (int t = 0; t < 32; ++t) {
        if (t < n) {
#pragma unroll
            for (int h = 0; h < HG; ++h) o[h] = fmaf(sc[j0 + h][t], va[t], o[h]);
        }
        if (32 + t < n) {
#pragma unroll
            for (int h = 0; h < HG; ++h) o[h] = fmaf(sc[j0 + h][32 + t], vb[t], o[h]);
        }
    }
    const int nsplit = p.nsplit;
    if (n_active == 1) {
#pragma unroll
        for (int t = 0; t < HG; ++t) {
            const int head = head0 + j0 + t;
            p.out[size_t(head) * D + d] = (o[t] / stat_l[j0 + t]) * (1.f / (1.f + expf(-gate[t])));
        }
        return;
    }
#pragma unroll
    for (int t = 0; t < HG; ++t) p.part_o[(size_t(head0 + j0 + t) * nsplit + split) * D + d] = o[t];
    if (tid < GH) {
        p.part_ml[(size_t(head0 + tid) * nsplit + split) * 2] = stat_m[tid];
        p.part_ml[(size_t(head0 + tid) * nsplit + split) * 2 + 1] = stat_l[tid];
    }
    trace_mark(p.trace, 2);
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned ticket = atomicAdd(&p.counters[blockIdx.x], 1u);
        s_last = (ticket == unsigned(n_active - 1));
    }
    __syncthreads();
    trace_mark(p.trace, 3);
    if (!s_last) return;
    __threadfence();

    // ---- merge by the last CTA of this head group ----
    float num[HG], den[HG], run_m[HG];
#pragma unroll
    for (int t = 0; t < HG; ++t) { num[t] = 0.f; den[t] = 0.f; run_m[t] = -INFINITY; }
    for (int s0 = 0; s0 < n_active; s0 += 64) {
        const int ns = min(64, n_active - s0);
        __syncthreads();
        for (int j = warp; j < GH; j += NWARP) {
            const float2* ml = reinterpret_cast<const float2*>(p.part_ml + (size_t(head0 + j) * nsplit + s0) * 2);
            const float2 a0 = lane < ns ? __ldcg(ml + lane) : make_float2(-INFINITY, 0.f);
            const float2 a1 = lane + 32 < ns ? __ldcg(ml + lane + 32) : make_float2(-INFINITY, 0.f);
            const float M = warp_max(fmaxf(a0.x, a1.x));
            const float w0 = lane < ns ? expf(a0.x - M) : 0.f;
            const float w1 = lane + 32 < ns ? expf(a1.x - M) : 0.f;
            mrg_w[j][lane] = w0;
            mrg_w[j][lane + 32] = w1;
            const float den_pass = warp_sum(fmaf(w0, a0.y, w1 * a1.y));
            if (lane == 0) { stat_m[j] = M; stat_l[j] = den_pass; }
        }
        __syncthreads();
#pragma unroll
        for (int t = 0; t < HG; ++t) {
            const int j = j0 + t, head = head0 + j;
            const float* po = p.part_o + (size_t(head) * nsplit + s0) * D + d;
            float a = 0.f;
            const float b = stat_l[j];
            for (int s = 0; s < ns; s += kGatedMergeBatch) {   // kGatedMergeBatch independent loads in flight
                float v[kGatedMergeBatch];
#pragma unroll
                for (int i = 0; i < kGatedMergeBatch; ++i) v[i] = (s + i < ns) ? __ldcg(po + size_t(s + i) * D) : 0.f;
#pragma unroll
                for (int i = 0; i < kGatedMergeBatch; ++i) a = fmaf(mrg_w[j][(s + i) & 63], v[i], a);
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
        const int head = head0 + j0 + t;
        p.out[size_t(head) * D + d] = (num[t] / den[t]) * (1.f / (1.f + expf(-gate[t])));
    }
    if (tid == 0) p.counters[blockIdx.x] = 0;
    trace_end(p.trace);
}

// CTAs along x for a shape: one per (KV head, group of GH query heads)
int attn_gated_groups(int hq, int hkv, int d) {
    const int G = hq / hkv;
    const int gh = (d == 256) ? 2 : (G >= 2 ? 2 : 1);
    return hkv * (G / gh);
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
    const dim3 grid(attn_gated_groups(p.hq, p.hkv, p.d), p.nsplit), block(kGatedThreads);
#define TFB_ATTN(DD, GG, HH) \
    if (p.d == DD && G == GG) return launch_kernel(attn_gated_kernel<DD, GG, HH>, grid, block, 0, stream, pdl, p);
    TFB_ATTN(256, 8, 2) TFB_ATTN(256, 4, 2) TFB_ATTN(128, 2, 2) TFB_ATTN(128, 4, 2)
#undef TFB_ATTN
    return cudaErrorInvalidValue;
}

}  // namespace tfb
