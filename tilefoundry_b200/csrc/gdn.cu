// Gated DeltaNet recurrence for one token (examples/qwen3_5_35b_a3b-tilelang/model.py:117-228): the
// depthwise causal convolution of the q|k|v projection, SiLU, per-head L2 normalisation of q and k,
// the decay / write-strength scalars, and the delta-rule update and read of the per-head state.
//
// HBM-bound on the state: algorithmic bytes per launch = 2 * hv * dk * dv * 4 (read + write; Qwen3.5:
// 2 * 32 * 128 * 128 * 4 = 4.2 MB).  The recurrence is independent per state column, so the grid is
// (value heads, dv / 32): a CTA owns 32 columns of one head's dk x dv state, holds them in registers
// (loaded before the dependency wait -- the previous token wrote them), and needs two block-wide
// column reductions (the recall and the read).
//
// The convolution window of a channel is read by several CTAs (q and k channels serve every value head
// of their key head and every column slice), so the shifted window is written to the OTHER of two
// buffers, picked by the parity of the position word; no CTA ever reads what another is writing.
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

constexpr int kGdnCols = 32;
constexpr int kGdnThreads = 256;

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f32(float x) { return 1.f / (1.f + expf(-x)); }

// The delta rule on one CTA's 32 state columns; `s` holds the CTA's rows of the state (thread = column `lane`,
// rows warp, warp+8, ...), s_q / s_k the scaled query and the key of this head.
template <int DK>
__device__ __forceinline__ void delta_rule(const GdnParams& p, float (&s)[DK / (kGdnThreads / 32)], float* state,
                                           const float* s_q, const float* s_k, float (*s_red)[kGdnCols], float* s_col,
                                           float v_col, float beta, float decay) {
    constexpr int NWARP = kGdnThreads / 32;
    constexpr int RPW = DK / NWARP;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hv = blockIdx.x, c0 = blockIdx.y * kGdnCols;
    float recalled = 0.f;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        s[i] *= decay;
        recalled = fmaf(s[i], s_k[warp + i * NWARP], recalled);
    }
    s_red[warp][lane] = recalled;
    __syncthreads();
    if (tid < kGdnCols) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < NWARP; ++w) t += s_red[w][tid];
        s_col[tid] = (v_col - t) * beta;
    }
    __syncthreads();
    const float delta = s_col[lane];
    float read = 0.f;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        s[i] = fmaf(s_k[warp + i * NWARP], delta, s[i]);
        read = fmaf(s[i], s_q[warp + i * NWARP], read);
        state[size_t(warp + i * NWARP) * p.dv] = s[i];
    }
    __syncthreads();
    s_red[warp][lane] = read;
    __syncthreads();
    if (tid < kGdnCols) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < NWARP; ++w) t += s_red[w][tid];
        p.read[size_t(hv) * p.dv + c0 + tid] = t;
    }
}

template <int DK, int KW>
__global__ void __launch_bounds__(kGdnThreads) gdn_step_kernel(const GdnParams p) {
    constexpr int NWARP = kGdnThreads / 32;
    constexpr int RPW = DK / NWARP;                    // state rows per warp
    __shared__ float s_q[DK], s_k[DK];
    __shared__ float s_red[NWARP][kGdnCols];
    __shared__ float s_col[kGdnCols];
    __shared__ float s_norm[2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hv = blockIdx.x, c0 = blockIdx.y * kGdnCols;
    const int kh = hv / (p.hv / p.hk);
    const int key_dim = p.hk * DK, conv_dim = 2 * key_dim + p.hv * p.dv;

    // ---- before the wait: the state slice, the conv windows and weights (all from earlier tokens) ----
    float* state = p.state + (size_t(hv) * DK) * p.dv + c0 + lane;
    float s[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) s[i] = state[size_t(warp + i * NWARP) * p.dv];
    const bool direct = p.direct_q != nullptr;         // q, k, v, g, beta handed in: only the delta rule runs
    int parity = 0;
    if (p.pos) parity = *reinterpret_cast<const volatile int*>(p.pos) & 1;
    const float* win_in = p.conv_state + size_t(parity) * p.conv_state_stride;
    float* win_out = p.conv_state + size_t(parity ^ 1) * p.conv_state_stride;
    // channel of this thread: threads 0..DK-1 -> q of key head kh, DK..2DK-1 -> k; then a second role for v
    const int ch_qk = (tid < DK) ? kh * DK + tid : key_dim + kh * DK + (tid - DK);
    const int ch_v = 2 * key_dim + hv * p.dv + c0 + tid;          // threads < kGdnCols only
    float win[KW - 1], cw[KW], vwin[KW - 1], vcw[KW];
    if (!direct && tid < 2 * DK) {
#pragma unroll
        for (int j = 0; j < KW - 1; ++j) win[j] = win_in[size_t(ch_qk) * (KW - 1) + j];
#pragma unroll
        for (int j = 0; j < KW; ++j) cw[j] = p.conv_w[size_t(ch_qk) * KW + j];
    }
    if (!direct && tid < kGdnCols) {
#pragma unroll
        for (int j = 0; j < KW - 1; ++j) vwin[j] = win_in[size_t(ch_v) * (KW - 1) + j];
#pragma unroll
        for (int j = 0; j < KW; ++j) vcw[j] = p.conv_w[size_t(ch_v) * KW + j];
    }
    const float a_log = direct ? 0.f : p.a_log[hv], dt_bias = direct ? 0.f : p.dt_bias[hv];
    pdl_trigger();
    pdl_wait();
    if (direct) {
        if (tid < DK) s_q[tid] = p.direct_q[size_t(hv) * DK + tid] * p.q_scale;
        else if (tid < 2 * DK) s_k[tid - DK] = p.direct_k[size_t(hv) * DK + tid - DK];
        __syncthreads();
        delta_rule<DK>(p, s, state, s_q, s_k, s_red, s_col, tid < kGdnCols ? p.direct_v[size_t(hv) * p.dv + c0 + tid] : 0.f,
                       p.direct_beta[hv], expf(p.direct_g[hv]));
        return;
    }

    // ---- convolution + SiLU, L2 norms ----------------------------------------------------------
    const float* entry = p.proj;                                   // [conv_dim] then z [val] then b [hv] then a [hv]
    const bool qk_writer = (hv % (p.hv / p.hk) == 0) && blockIdx.y == 0;
    float mixed = 0.f;
    if (tid < 2 * DK) {
        const float e = entry[ch_qk];
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < KW - 1; ++j) acc += win[j] * cw[j];
        acc += e * cw[KW - 1];
        mixed = silu_f32(acc);
        if (qk_writer) {
#pragma unroll
            for (int j = 0; j < KW - 2; ++j) win_out[size_t(ch_qk) * (KW - 1) + j] = win[j + 1];
            win_out[size_t(ch_qk) * (KW - 1) + KW - 2] = e;
        }
    }
    float ssq = warp_sum(mixed * mixed);                           // warps 0..DK/32-1 hold q, the next DK/32 hold k
    if (lane == 0) s_red[0][warp] = ssq;
    float v_col = 0.f;
    if (tid < kGdnCols) {
        const float e = entry[ch_v];
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < KW - 1; ++j) acc += vwin[j] * vcw[j];
        acc += e * vcw[KW - 1];
        v_col = silu_f32(acc);
#pragma unroll
        for (int j = 0; j < KW - 2; ++j) win_out[size_t(ch_v) * (KW - 1) + j] = vwin[j + 1];
        win_out[size_t(ch_v) * (KW - 1) + KW - 2] = e;
    }
    __syncthreads();
    if (tid < 2) {
        float t = 0.f;
        for (int w = 0; w < DK / 32; ++w) t += s_red[0][tid * (DK / 32) + w];
        s_norm[tid] = rsqrtf(t + 1e-6f);
    }
    __syncthreads();
    if (tid < DK) s_q[tid] = mixed * s_norm[0] * p.q_scale;
    else if (tid < 2 * DK) s_k[tid - DK] = mixed * s_norm[1];
    const float beta = sigmoid_f32(entry[conv_dim + p.hv * p.dv + hv]);
    const float g = -expf(a_log) * softplus_f32(entry[conv_dim + p.hv * p.dv + p.hv + hv] + dt_bias);
    const float decay = expf(g);
    __syncthreads();

    delta_rule<DK>(p, s, state, s_q, s_k, s_red, s_col, v_col, beta, decay);
}

// ---- the same pieces as stand-alone functions (per-function checks of a runtime twin) ----
__global__ void conv_silu_f32_kernel(const float* __restrict__ state, const float* __restrict__ entry,
                                     const float* __restrict__ conv_w, float* __restrict__ mixed, int channels, int width) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float acc = 0.f;
    for (int j = 0; j < width - 1; ++j) acc += state[size_t(c) * (width - 1) + j] * conv_w[size_t(c) * width + j];
    acc += entry[c] * conv_w[size_t(c) * width + width - 1];
    mixed[c] = silu_f32(acc);
}
cudaError_t conv_silu_f32_launch(const float* state, const float* entry, const float* conv_w, float* mixed, int channels,
                                 int width, cudaStream_t stream, bool pdl) {
    return launch_kernel(conv_silu_f32_kernel, dim3((channels + 255) / 256), dim3(256), 0, stream, pdl, state, entry,
                         conv_w, mixed, channels, width);
}

__global__ void l2norm_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int width, float eps) {
    pdl_trigger();
    pdl_wait();
    const float* xr = x + size_t(blockIdx.x) * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += 32) ss = fmaf(xr[i], xr[i], ss);
    const float r = rsqrtf(warp_sum(ss) + eps);
    for (int i = threadIdx.x; i < width; i += 32) y[size_t(blockIdx.x) * width + i] = xr[i] * r;
}
cudaError_t l2norm_f32_launch(const float* x, float* y, int rows, int width, float eps, cudaStream_t stream, bool pdl) {
    return launch_kernel(l2norm_f32_kernel, dim3(rows), dim3(32), 0, stream, pdl, x, y, width, eps);
}

cudaError_t gdn_step_launch(const GdnParams& p, cudaStream_t stream, bool pdl) {
    if (p.dk != 128 || p.kernel_width != 4 || p.dv % kGdnCols != 0 || p.hv % p.hk != 0) return cudaErrorInvalidValue;
    const dim3 grid(p.hv, p.dv / kGdnCols), block(kGdnThreads);
    return launch_kernel(gdn_step_kernel<128, 4>, grid, block, 0, stream, pdl, p);
}

}  // namespace tfb
