// GQA decode attention over a paged bf16 KV cache, one launch per layer:
// per-head q/k RMSNorm -> RoPE -> KV append -> split-KV online softmax -> merge.
//
// HBM-bound on the cache: algorithmic bytes per launch = (ctx+1) * hkv * d * 2 (K and V)
// * 2 bytes.  Grid = (hkv, splits): one CTA owns one KV head and SPLIT_LEN
// consecutive positions, and serves all G = hq/hkv query heads that share the KV
// head so each cache line is read once.  A sub-group of d/8 lanes reads one
// position's 2d-byte row with one 16-byte load per lane.  Partial (max, sum,
// weighted V) triples go to scratch; the last CTA of a KV head to finish (an atomic
// ticket, no spinning) merges them.
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

constexpr int kSplitLen = 128;
constexpr int kAttnThreads = 128;

int attn_splits(int max_ctx) { return (max_ctx + kSplitLen - 1) / kSplitLen; }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

template <int D, int G>
__global__ void __launch_bounds__(kAttnThreads) attn_gqa_kernel(const AttnParams p) {
    constexpr int LPP = D / 8;                 // lanes that share one position's row
    constexpr int PPW = 32 / LPP;              // positions a warp reads per load
    constexpr int NWARP = kAttnThreads / 32;
    constexpr int NG = NWARP * PPW;            // position sub-groups in the CTA
    constexpr int NV = G + 1;                  // vectors normalised + rotated: G queries and the key

    __shared__ __align__(16) float vec[NV + 1][D];       // q_0..q_{G-1}, k_new, v_new
    __shared__ __align__(16) float tmp[NV][D];
    __shared__ float sc[G][kSplitLen];
    __shared__ __align__(16) float red[NG][G][D];
    __shared__ float stat_m[G], stat_l[G];
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.x, split = blockIdx.y;

    if (tid == 0)
        l2_prefetch_slice(p.prefetch, p.prefetch_bytes, blockIdx.y * gridDim.x + blockIdx.x,
                          gridDim.x * gridDim.y);
    pdl_trigger();
    pdl_wait();

    const int pos = *p.pos;
    if (pos < 0 || pos >= p.max_ctx) return;
    const int total = pos + 1;
    const int n_active = (total + kSplitLen - 1) / kSplitLen;
    if (split >= n_active) return;
    const bool owner = (split == n_active - 1);
    const int p0 = split * kSplitLen;
    const int p1 = min(p0 + kSplitLen, total);
    const int pend = min(p1, pos);             // cache positions; the new token is handled from smem

    // ---- this token's q (G heads), k, v for KV head g -------------------------
    for (int vi = warp; vi < NV + 1; vi += NWARP) {
        const uint16_t* src;
        if (vi < G) src = p.qkv + size_t(g * G + vi) * D;
        else if (vi == G) src = p.qkv + size_t(p.hq) * D + size_t(g) * D;
        else src = p.qkv + size_t(p.hq + p.hkv) * D + size_t(g) * D;
        float x[D / 32];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < D / 32; ++i) {
            x[i] = bf16_bits_to_f32(src[lane + 32 * i]);
            ss = fmaf(x[i], x[i], ss);
        }
        if (vi == G + 1) {                     // v: no norm, no rotation
#pragma unroll
            for (int i = 0; i < D / 32; ++i) vec[vi][lane + 32 * i] = x[i];
            continue;
        }
        float rstd = 1.f;
        const uint16_t* gam = (vi < G) ? p.gamma_q : p.gamma_k;
        if (p.norm_mode != 0) {
            ss = warp_sum(ss);
            rstd = rsqrtf(ss / float(D) + p.eps);
        }
#pragma unroll
        for (int i = 0; i < D / 32; ++i) {
            float n = x[i];
            if (p.norm_mode != 0) n = round_bf16(round_bf16(n * rstd) * bf16_bits_to_f32(gam[lane + 32 * i]));
            tmp[vi][lane + 32 * i] = n;
        }
    }
    __syncthreads();
    const int rd = p.rotary_dim, half = rd >> 1;
    const int rpos = p.rope_pos ? *p.rope_pos : pos;
    for (int e = tid; e < NV * D; e += kAttnThreads) {
        const int vi = e / D, i = e % D;
        float r = tmp[vi][i];
        if (i < rd) {
            const float c = bf16_bits_to_f32(p.cos_table[size_t(rpos) * rd + i]);
            const float s = bf16_bits_to_f32(p.sin_table[size_t(rpos) * rd + i]);
            const float partner = (i < half) ? -tmp[vi][i + half] : tmp[vi][i - half];
            r = round_bf16(__fadd_rn(__fmul_rn(r, c), __fmul_rn(partner, s)));
        }
        if (vi < G) r = round_bf16(r * p.scale);
        vec[vi][i] = r;
    }
    __syncthreads();

    if (owner) {                                // append this token's entry to the cache
        const int page = p.block_table[pos / p.page_size];
        const size_t base = ((size_t(page) * p.page_size + (pos % p.page_size)) * p.hkv + g) * D;
        for (int i = tid; i < D; i += kAttnThreads) {
            const uint16_t kb = f32_to_bf16_bits(vec[G][i]), vb = f32_to_bf16_bits(vec[G + 1][i]);
            p.k_pool[base + i] = kb;
            p.v_pool[base + i] = vb;
            if (p.k_new_out) p.k_new_out[size_t(g) * D + i] = kb;
            if (p.v_new_out) p.v_new_out[size_t(g) * D + i] = vb;
        }
    }

    // ---- pass 1: scores ----------------------------------------------------------
    const int sg = warp * PPW + lane / LPP, sl = lane % LPP;
    float q[G][8];
#pragma unroll
    for (int j = 0; j < G; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) q[j][i] = vec[j][sl * 8 + i];

    constexpr int U = 4;
    // Every lane of a warp runs the same trip count (the shuffles below need the
    // full warp); only loads and stores are guarded by the position bound.
    for (int pb = p0; pb < pend; pb += NG * U) {
        uint4 kv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int pp = pb + u * NG + sg;
            if (pp < pend) {
                const int page = p.block_table[pp / p.page_size];
                const size_t off = ((size_t(page) * p.page_size + (pp % p.page_size)) * p.hkv + g) * D + sl * 8;
                kv[u] = *reinterpret_cast<const uint4*>(p.k_pool + off);
            } else {
                kv[u] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int pp = pb + u * NG + sg;
            float kf[8];
            unpack8(kv[u], kf);
#pragma unroll
            for (int j = 0; j < G; ++j) {
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) s = fmaf(q[j][i], kf[i], s);
#pragma unroll
                for (int o = LPP / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (sl == 0 && pp < pend) sc[j][pp - p0] = s;
            }
        }
    }
    if (owner && warp == 0) {                   // the token attends itself
#pragma unroll
        for (int j = 0; j < G; ++j) {
            float s = 0.f;
            for (int i = lane; i < D; i += 32) s = fmaf(vec[j][i], vec[G][i], s);
            s = warp_sum(s);
            if (lane == 0) sc[j][pos - p0] = s;
        }
    }
    __syncthreads();

    // ---- softmax statistics of this split ----------------------------------------
    const int n = p1 - p0;
    for (int j = warp; j < G; j += NWARP) {
        float m = -INFINITY;
        for (int i = lane; i < n; i += 32) m = fmaxf(m, sc[j][i]);
        m = warp_max(m);
        float l = 0.f;
        for (int i = lane; i < n; i += 32) {
            const float e = __expf(sc[j][i] - m);
            sc[j][i] = e;
            l += e;
        }
        l = warp_sum(l);
        if (lane == 0) { stat_m[j] = m; stat_l[j] = l; }
    }
    __syncthreads();

    // ---- pass 2: probability-weighted V --------------------------------------------
    float acc[G][8];
#pragma unroll
    for (int j = 0; j < G; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
    for (int pb = p0; pb < pend; pb += NG * U) {
        uint4 vv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int pp = pb + u * NG + sg;
            if (pp < pend) {
                const int page = p.block_table[pp / p.page_size];
                const size_t off = ((size_t(page) * p.page_size + (pp % p.page_size)) * p.hkv + g) * D + sl * 8;
                vv[u] = *reinterpret_cast<const uint4*>(p.v_pool + off);
            } else {
                vv[u] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int pp = pb + u * NG + sg;
            if (pp < pend) {
                float vf[8];
                unpack8(vv[u], vf);
#pragma unroll
                for (int j = 0; j < G; ++j) {
                    const float pr = sc[j][pp - p0];
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[j][i] = fmaf(pr, vf[i], acc[j][i]);
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < G; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) red[sg][j][sl * 8 + i] = acc[j][i];
    __syncthreads();

    const int nsplit = p.nsplit;
    for (int e = tid; e < G * D; e += kAttnThreads) {
        const int j = e / D, d = e % D;
        float o = 0.f;
#pragma unroll
        for (int s = 0; s < NG; ++s) o += red[s][j][d];
        if (owner) o = fmaf(sc[j][pos - p0], vec[G + 1][d], o);
        const int head = g * G + j;
        if (n_active == 1) {
            p.out[size_t(head) * D + d] = f32_to_bf16_bits(o / stat_l[j]);
        } else {
            p.part_o[(size_t(head) * nsplit + split) * D + d] = o;
        }
    }
    if (n_active == 1) return;
    if (tid < G) {
        const int head = g * G + tid;
        p.part_ml[(size_t(head) * nsplit + split) * 2] = stat_m[tid];
        p.part_ml[(size_t(head) * nsplit + split) * 2 + 1] = stat_l[tid];
    }

    // ---- merge by the last CTA of this KV head ---------------------------------------
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned ticket = atomicAdd(&p.counters[g], 1u);
        s_last = (ticket == unsigned(n_active - 1));
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int e = tid; e < G * D; e += kAttnThreads) {
        const int j = e / D, d = e % D;
        const int head = g * G + j;
        const float* ml = p.part_ml + size_t(head) * nsplit * 2;
        float M = -INFINITY;
        for (int s = 0; s < n_active; ++s) M = fmaxf(M, __ldcg(ml + 2 * s));
        float num = 0.f, den = 0.f;
        for (int s = 0; s < n_active; ++s) {
            const float w = __expf(__ldcg(ml + 2 * s) - M);
            num = fmaf(w, __ldcg(p.part_o + (size_t(head) * nsplit + s) * D + d), num);
            den = fmaf(w, __ldcg(ml + 2 * s + 1), den);
        }
        p.out[size_t(head) * D + d] = f32_to_bf16_bits(num / den);
    }
    if (tid == 0) p.counters[g] = 0;
}

cudaError_t attn_gqa_dispatch(const AttnParams& p, cudaStream_t stream, bool pdl) {
    const int G = p.hq / p.hkv;
    const dim3 grid(p.hkv, p.nsplit), block(kAttnThreads);
#define TFB_ATTN(DD, GG) \
    if (p.d == DD && G == GG) return launch_kernel(attn_gqa_kernel<DD, GG>, grid, block, 0, stream, pdl, p);
    TFB_ATTN(128, 1) TFB_ATTN(128, 2) TFB_ATTN(128, 4) TFB_ATTN(64, 2) TFB_ATTN(64, 1)
#undef TFB_ATTN
    return cudaErrorInvalidValue;
}

}  // namespace tfb
