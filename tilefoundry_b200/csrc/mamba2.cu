// Mamba-2 single-token state update (granite-4.0-h): depthwise causal convolution step and the
// selective-state recurrence, with every rounding point of the authored functions kept
// (examples/granite_4_0_h_small-cuda/model.py: conv_step :154-167, ssm_step :170-220).
//
// conv kernel: latency-bound, CONVD*(KRN*2+8) bytes.  ssm kernel: HBM-bound on the f32 state,
// algorithmic bytes per launch = 2 * NH*PD*NS*4 (state read + write) = 8 MB for granite.
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

// One thread per channel: window = [state | entry]; bf16 products, one bf16 sum, bias, SiLU;
// then the window slides by the entry.  state_in / state_out may be the same buffer.
template <int KRN>
__global__ void __launch_bounds__(256) conv_step_kernel(const ConvParams p) {
    constexpr int WIN = KRN - 1;
    float w[KRN], bias = 0.f;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < p.channels) {                       // weights first: they do not depend on the previous kernel
#pragma unroll
        for (int i = 0; i < KRN; ++i) w[i] = bf16_bits_to_f32(p.conv_w[size_t(c) * KRN + i]);
        if (p.conv_b) bias = bf16_bits_to_f32(p.conv_b[c]);
    }
    pdl_trigger();
    pdl_wait();
    if (c >= p.channels) return;
    float win[KRN];
#pragma unroll
    for (int i = 0; i < WIN; ++i) win[i] = bf16_bits_to_f32(p.state_in[size_t(c) * WIN + i]);
    const uint16_t entry = p.entry[c];
    win[WIN] = bf16_bits_to_f32(entry);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < KRN; ++i) s += round_bf16(win[i] * w[i]);      // bf16 products, f32 running sum
    s = round_bf16(s);                                                   // the reduce returns bf16
    if (p.conv_b) s = round_bf16(s + bias);
    p.mixed[c] = f32_to_bf16_bits(silu_f32(s));
#pragma unroll
    for (int i = 0; i + 1 < WIN; ++i) p.state_out[size_t(c) * WIN + i] = f32_to_bf16_bits(win[i + 1]);
    p.state_out[size_t(c) * WIN + WIN - 1] = entry;
    if (p.entry_out) p.entry_out[c] = entry;
}

cudaError_t conv_step_launch(const ConvParams& p, cudaStream_t stream, bool pdl) {
    const dim3 grid((p.channels + 255) / 256), block(256);
    if (p.kernel_width == 4) return launch_kernel(conv_step_kernel<4>, grid, block, 0, stream, pdl, p);
    return cudaErrorInvalidValue;
}

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// One warp per (head, row): NS states, NS/32 per lane.
template <int NS>
__global__ void __launch_bounds__(256) ssm_step_kernel(const SsmParams p) {
    constexpr int PER = NS / 32;
    __shared__ float sB[NS], sC[NS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * 8 + warp;                  // h * PD + pd
    const int h = row / p.pd;
    const bool live = row < p.nh * p.pd;

    // state and per-head constants do not depend on the previous kernel in the stream
    float st[PER];
    float a = 0.f, dtb = 0.f, dsk = 0.f;
    if (live) {
        const float4* src = reinterpret_cast<const float4*>(p.state_in + size_t(row) * NS + lane * PER);
#pragma unroll
        for (int i = 0; i < PER / 4; ++i) {
            const float4 v = __ldcs(src + i);
            st[4 * i] = v.x; st[4 * i + 1] = v.y; st[4 * i + 2] = v.z; st[4 * i + 3] = v.w;
        }
        a = -expf(bf16_bits_to_f32(p.a_log[h]));
        dtb = bf16_bits_to_f32(p.dt_bias[h]);
        dsk = bf16_bits_to_f32(p.d_skip[h]);
    }
    pdl_trigger();
    pdl_wait();

    const int group = live ? h / (p.nh / p.ng) : 0;
    for (int i = threadIdx.x; i < NS; i += blockDim.x) {     // one group per CTA (8 rows share a head)
        sB[i] = bf16_bits_to_f32(p.b_vec[size_t(group) * NS + i]);
        sC[i] = bf16_bits_to_f32(p.c_vec[size_t(group) * NS + i]);
    }
    __syncthreads();
    if (!live) return;

    const float dt = round_bf16(softplus_f32(round_bf16(bf16_bits_to_f32(p.dt_raw[h]) + dtb)));
    const float decay = expf(__fmul_rn(dt, a));
    const float x = bf16_bits_to_f32(p.x[row]);
    float read = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int n = lane * PER + i;
        const float dbx = round_bf16(round_bf16(dt * sB[n]) * x);
        st[i] = __fadd_rn(__fmul_rn(st[i], decay), dbx);
        read = fmaf(round_bf16(st[i]), sC[n], read);
    }
    float4* dst = reinterpret_cast<float4*>(p.state_out + size_t(row) * NS + lane * PER);
#pragma unroll
    for (int i = 0; i < PER / 4; ++i) dst[i] = make_float4(st[4 * i], st[4 * i + 1], st[4 * i + 2], st[4 * i + 3]);
    read = warp_sum(read);
    if (lane == 0) p.y[row] = f32_to_bf16_bits(round_bf16(read) + round_bf16(x * dsk));
}

cudaError_t ssm_step_launch(const SsmParams& p, cudaStream_t stream, bool pdl) {
    const dim3 grid((p.nh * p.pd + 7) / 8), block(256);
    if (p.ns == 128) return launch_kernel(ssm_step_kernel<128>, grid, block, 0, stream, pdl, p);
    return cudaErrorInvalidValue;
}

}  // namespace tfb
