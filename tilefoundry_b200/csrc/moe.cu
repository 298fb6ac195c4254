// Mixture-of-experts pieces for batch-1 decode: router selection (top-k + softmax) and the fused
// "down" stage (gathered expert down-projections, routing-weighted sum, shared expert, residual).
//
// Router select is one warp of latency.  The down kernel is HBM-bound: algorithmic bytes per
// launch = hidden * (top_k * inter + shared_inter) * 2 (each output row reads its top_k expert rows
// and its shared-expert row once); granite: 4096 * (10*768 + 1536) * 2 = 75.5 MB.
#include "common.cuh"
#include "route.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

// mode 0 (granite, examples/granite_4_0_h_small-cuda/model.py:376-386): logits (already bf16) -> top-k
//        -> softmax over the k -> bf16 weights.
// mode 1 (Qwen3.5, examples/qwen3_5_35b_a3b-tilelang/model.py:488-499): softmax over ALL experts in
//        f32 -> top-k -> renormalise by the sum of the k.
// Selection order is by value descending; equal values resolve to the lower index.
template <int MAXE>
__global__ void __launch_bounds__(32) router_select_kernel(const RouterParams p) {
    pdl_trigger();
    pdl_wait();
    float w;
    int e;
    route_select<MAXE>(p.logits_f32, p.logits_bf16, p.experts, p.top_k, p.mode, threadIdx.x, w, e);
    if (int(threadIdx.x) < p.top_k) {
        p.indices[threadIdx.x] = e;
        if (p.weights_bf16) p.weights_bf16[threadIdx.x] = f32_to_bf16_bits(w);
        if (p.weights_f32) p.weights_f32[threadIdx.x] = w;
        long long le = e;
        bool local = true;
        if (p.expert_world > 1) { local = (e % p.expert_world) == p.expert_rank; le = e / p.expert_world; }
        for (int i = 0; local && i < p.n_slabs; ++i) {
            const char* base = static_cast<const char*>(p.slab[i]) + size_t(le) * p.slab_bytes[i];
            for (unsigned long long off = 0; off < p.slab_bytes[i]; off += (1u << 20)) {
                const unsigned long long left = p.slab_bytes[i] - off;
                l2_prefetch_bulk(base + off, uint32_t(left < (1u << 20) ? left : (1u << 20)));
            }
        }
    }
}

cudaError_t router_select_launch(const RouterParams& p, cudaStream_t stream, bool pdl) {
    if (p.experts <= 128) return launch_kernel(router_select_kernel<128>, dim3(1), dim3(32), 0, stream, pdl, p);
    if (p.experts <= 256) return launch_kernel(router_select_kernel<256>, dim3(1), dim3(32), 0, stream, pdl, p);
    return cudaErrorInvalidValue;
}

// A warp owns kDownRows output rows: for each selected slot s, dot(w_down[idx[s]][j, :], inner[s, :]) rounded to
// bf16, times the routing weight (bf16), summed over slots with one rounding; plus the shared expert's row; then
// the layer's scaled residual.  All rounding points of routed_experts / experts / residual_add
// (examples/granite_4_0_h_small-cuda/model.py:406-470,502) are kept.
// Latency plan: the gathered activations are staged once per CTA with 16-byte loads and serve 16 rows; a warp has
// the rows of TWO slots for both of its output rows in flight at a time (12 x 16 bytes per lane), so the routed
// part takes top_k/2 memory round trips instead of top_k, each carrying four times the bytes.
constexpr int kDownWarps = 8;
constexpr int kDownRows = 2;
__global__ void __launch_bounds__(kDownWarps * 32) moe_down_kernel(const MoeDownParams p) {
    extern __shared__ __align__(16) float smem[];
    float* xin = smem;                                        // [top_k][inter] then [shared_inter]
    __shared__ long long s_idx[32];
    __shared__ float s_w[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j0 = (blockIdx.x * kDownWarps + warp) * kDownRows;
    const int I = p.inter, IS = p.shared_inter, K = p.top_k;

    // the shared expert's rows do not depend on the routing: fetch them before the wait
    const int sh_pieces = IS >> 3;                            // 16-byte pieces in a shared-expert row
    uint4 shw[kDownRows][4];
    const uint4* shrow[kDownRows];
#pragma unroll
    for (int r = 0; r < kDownRows; ++r) {
        shrow[r] = (p.w_shared && j0 + r < p.hidden) ? p.w_shared + size_t(j0 + r) * sh_pieces : nullptr;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            shw[r][u] = (shrow[r] && lane + 32 * u < sh_pieces) ? ld_stream16(shrow[r] + lane + 32 * u) : make_uint4(0, 0, 0, 0);
    }
    pdl_trigger();
    pdl_wait();

    float res[kDownRows];
#pragma unroll
    for (int r = 0; r < kDownRows; ++r) res[r] = (p.residual && j0 + r < p.hidden) ? bf16_bits_to_f32(p.residual[j0 + r]) : 0.f;
    if (threadIdx.x < K) { s_idx[threadIdx.x] = p.indices[threadIdx.x]; s_w[threadIdx.x] = bf16_bits_to_f32(p.weights[threadIdx.x]); }
    for (int c = threadIdx.x; c < (K * I + IS) >> 3; c += blockDim.x) {          // 8 activations per 16-byte load
        const int i = c << 3;
        const uint4 v = i < K * I ? *reinterpret_cast<const uint4*>(p.inner + i) : *reinterpret_cast<const uint4*>(p.shared_act + (i - K * I));
        *reinterpret_cast<float4*>(xin + i) = make_float4(bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y));
        *reinterpret_cast<float4*>(xin + i + 4) = make_float4(bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w));
    }
    __syncthreads();
    if (j0 >= p.hidden) return;

    float routed[kDownRows];
#pragma unroll
    for (int r = 0; r < kDownRows; ++r) routed[r] = 0.f;
    const int pieces = I >> 3;
    for (int s0 = 0; s0 < K; s0 += 2) {
        uint4 wb[2][kDownRows][3];
        bool live[2];
        const uint4* rows[2];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            live[t] = s0 + t < K;
            long long e = live[t] ? s_idx[s0 + t] : 0;
            if (live[t] && p.expert_world > 1) {               // expert parallel: only this rank's experts are here
                if (e % p.expert_world != p.expert_rank) live[t] = false;
                e /= p.expert_world;
            }
            rows[t] = p.w_down + (size_t(live[t] ? e : 0) * p.hidden + j0) * pieces;
#pragma unroll
            for (int r = 0; r < kDownRows; ++r)
#pragma unroll
                for (int u = 0; u < 3; ++u)
                    wb[t][r][u] = (live[t] && j0 + r < p.hidden && lane + 32 * u < pieces)
                                      ? ld_stream16(rows[t] + size_t(r) * pieces + lane + 32 * u) : make_uint4(0, 0, 0, 0);
        }
        float acc[2][kDownRows];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const float* x = xin + (s0 + t) * I;
#pragma unroll
            for (int r = 0; r < kDownRows; ++r) {
                acc[t][r] = 0.f;
                if (!live[t]) continue;
#pragma unroll
                for (int u = 0; u < 3; ++u) {
                    const int c = lane + 32 * u;
                    if (c < pieces) {
                        const float4 xa = *reinterpret_cast<const float4*>(x + c * 8), xb = *reinterpret_cast<const float4*>(x + c * 8 + 4);
                        acc[t][r] = dot8(wb[t][r][u], xa, xb, acc[t][r]);
                    }
                }
                for (int c = lane + 96; c < pieces; c += 32) {   // rows wider than 768 elements
                    const uint4 w = ld_stream16(rows[t] + size_t(r) * pieces + c);
                    const float4 xa = *reinterpret_cast<const float4*>(x + c * 8), xb = *reinterpret_cast<const float4*>(x + c * 8 + 4);
                    acc[t][r] = dot8(w, xa, xb, acc[t][r]);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int r = 0; r < kDownRows; ++r) acc[t][r] += __shfl_xor_sync(0xffffffffu, acc[t][r], o);
#pragma unroll
        for (int t = 0; t < 2; ++t)
            if (live[t]) {
#pragma unroll
                for (int r = 0; r < kDownRows; ++r) routed[r] += round_bf16(round_bf16(acc[t][r]) * s_w[s0 + t]);   // bf16 products, f32 running sum
            }
    }
#pragma unroll
    for (int r = 0; r < kDownRows; ++r) {
        const int j = j0 + r;
        if (j >= p.hidden) continue;
        float out = round_bf16(routed[r]);                     // the reduce over slots returns bf16
        float sh_raw = 0.f;
        if (shrow[r]) {
            const float* x = xin + K * I;
            float acc = 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = lane + 32 * u;
                if (c < sh_pieces) {
                    const float4 xa = *reinterpret_cast<const float4*>(x + c * 8), xb = *reinterpret_cast<const float4*>(x + c * 8 + 4);
                    acc = dot8(shw[r][u], xa, xb, acc);
                }
            }
            for (int c = lane + 128; c < sh_pieces; c += 32) {   // rows wider than 1024 elements
                const uint4 w = ld_stream16(shrow[r] + c);
                const float4 xa = *reinterpret_cast<const float4*>(x + c * 8), xb = *reinterpret_cast<const float4*>(x + c * 8 + 4);
                acc = dot8(w, xa, xb, acc);
            }
            sh_raw = warp_sum(acc);
            float sh = round_bf16(sh_raw);
            if (p.shared_gate) sh = round_bf16(sh * *p.shared_gate);  // a gate on the shared expert
            out = round_bf16(out + sh);
        }
        if (lane == 0) {
            if (p.partial) {                                     // sharded: the ranks' sums are added before any rounding
                p.partial[j] = routed[r];
                p.partial[p.hidden + j] = sh_raw;
            } else {
                if (p.residual) out = res[r] + round_bf16(out * p.res_scale);
                p.out[j] = f32_to_bf16_bits(out);
            }
        }
    }
}

// After the ranks' partials were summed: the roundings of routed_experts / experts / residual_add.
__global__ void moe_finalize_kernel(const float* __restrict__ partial, const uint16_t* __restrict__ residual,
                                    uint16_t* __restrict__ out, int hidden, float res_scale, int has_shared) {
    pdl_trigger();
    pdl_wait();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= hidden) return;
    float v = round_bf16(partial[j]);
    if (has_shared) v = round_bf16(v + round_bf16(partial[hidden + j]));
    if (residual) v = bf16_bits_to_f32(residual[j]) + round_bf16(v * res_scale);
    out[j] = f32_to_bf16_bits(v);
}
cudaError_t moe_finalize_launch(const float* partial, const uint16_t* residual, uint16_t* out, int hidden,
                                float res_scale, bool has_shared, cudaStream_t stream, bool pdl) {
    return launch_kernel(moe_finalize_kernel, dim3((hidden + 255) / 256), dim3(256), 0, stream, pdl, partial, residual,
                         out, hidden, res_scale, int(has_shared));
}

// Vocabulary-parallel greedy pick: every rank contributed (best logit, global index); highest logit wins,
// equal logits resolve to the lower index (torch.argmax over the whole vocabulary), then the generation
// bookkeeping of the single-GPU head kernel.
__global__ void pick_finalize_kernel(const float* __restrict__ pairs, int world, long long* tokens, int* pos,
                                     int n_prompt, int max_tokens, long long* picked) {
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x != 0) return;
    float best = -INFINITY;
    long long best_i = 0x7fffffff;
    for (int r = 0; r < world; ++r) {
        const float v = pairs[2 * r];
        const long long i = (long long)pairs[2 * r + 1];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
    if (picked) *picked = best_i;
    if (tokens && pos) {
        const int cur = *pos;
        if (cur + 1 < max_tokens) {
            if (cur + 1 >= n_prompt) tokens[cur + 1] = best_i;
            *pos = cur + 1;
        }
    }
}
cudaError_t pick_finalize_launch(const float* pairs, int world, long long* tokens, int* pos, int n_prompt,
                                 int max_tokens, long long* picked, cudaStream_t stream, bool pdl) {
    return launch_kernel(pick_finalize_kernel, dim3(1), dim3(32), 0, stream, pdl, pairs, world, tokens, pos, n_prompt,
                         max_tokens, picked);
}

cudaError_t moe_down_launch(const MoeDownParams& p, cudaStream_t stream, bool pdl) {
    const size_t smem = (size_t(p.top_k) * p.inter + p.shared_inter) * sizeof(float);
    if (smem > 48 * 1024) {
        static PerDeviceOnce once;
        if (once.first()) {
            cudaError_t e = cudaFuncSetAttribute(moe_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            if (e != cudaSuccess) return e;}
    }
    const dim3 grid((p.hidden + kDownWarps * kDownRows - 1) / (kDownWarps * kDownRows)), block(kDownWarps * 32);
    return launch_kernel(moe_down_kernel, grid, block, smem, stream, pdl, p);
}

// f32-activation form (examples/qwen3_5_35b_a3b-tilelang/model.py:502-612): each expert product is rounded
// to bf16 and carried on in f32; the routing weights, the weighted sum over slots, the shared expert's
// sigmoid gate and the residual are f32 with no further rounding.
//   out[j] = residual[j] + sum_s w[s] * bf16(w_down[idx[s]][j,:] . bf16(inner[s,:]))
//                        + bf16(w_shared[j,:] . bf16(inner[top_k,:])) * sigmoid(*shared_gate_logit)
// `inner` holds top_k routed slots followed by the shared expert's slot, already rounded to bf16 values.
__global__ void __launch_bounds__(kDownWarps * 32) moe_down_f32_kernel(const MoeDownF32Params p) {
    extern __shared__ __align__(16) float smem[];
    float* xin = smem;                                        // [top_k][inter] then [shared_inter]
    __shared__ long long s_idx[32];
    __shared__ float s_w[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = blockIdx.x * kDownWarps + warp;
    const int I = p.inter, IS = p.shared_inter, K = p.top_k;

    const int sh_pieces = IS >> 3;
    uint4 shw[4];
    const uint4* shrow = (p.w_shared && j < p.hidden) ? p.w_shared + size_t(j) * sh_pieces : nullptr;
#pragma unroll
    for (int u = 0; u < 4; ++u) shw[u] = (shrow && lane + 32 * u < sh_pieces) ? ld_stream16(shrow + lane + 32 * u) : make_uint4(0, 0, 0, 0);
    pdl_trigger();
    pdl_wait();

    const float res = (p.residual && j < p.hidden) ? p.residual[j] : 0.f;
    if (threadIdx.x < K) { s_idx[threadIdx.x] = p.indices[threadIdx.x]; s_w[threadIdx.x] = p.weights[threadIdx.x]; }
    for (int i = threadIdx.x * 4; i < K * I + IS; i += blockDim.x * 4)
        *reinterpret_cast<float4*>(xin + i) = *reinterpret_cast<const float4*>(p.inner + i);
    __syncthreads();
    if (j >= p.hidden) return;

    // every selected expert's row is requested before the first one is used: one memory round trip, not top_k
    float routed = 0.f;
    const int pieces = I >> 3;
    for (int s0 = 0; s0 < K; s0 += 8) {
        uint4 wb[8][2];
        bool alive[8];
        const uint4* rows[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            bool live = s0 + s < K;
            long long e = live ? s_idx[s0 + s] : 0;
            if (live && p.expert_world > 1) {                  // expert parallel: only this rank's experts are here
                if (e % p.expert_world != p.expert_rank) live = false;
                e /= p.expert_world;
            }
            alive[s] = live;
            const uint4* row = p.w_down + (size_t(live ? e : 0) * p.hidden + j) * pieces;
            rows[s] = row;
#pragma unroll
            for (int u = 0; u < 2; ++u)
                wb[s][u] = (live && lane + 32 * u < pieces) ? ld_stream16(row + lane + 32 * u) : make_uint4(0, 0, 0, 0);
        }
        float acc[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            acc[s] = 0.f;
            if (!alive[s]) continue;
            const float* x = xin + (s0 + s) * I;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int c = lane + 32 * u;
                if (c < pieces) {
                    const float4 xa = *reinterpret_cast<const float4*>(x + c * 8), xb = *reinterpret_cast<const float4*>(x + c * 8 + 4);
                    acc[s] = dot8(wb[s][u], xa, xb, acc[s]);
                }
            }
            for (int c = lane + 64; c < pieces; c += 32) {        // rows wider than 512 elements
                const uint4 w = ld_stream16(rows[s] + c);
                const float4 xa = *reinterpret_cast<const float4*>(x + c * 8), xb = *reinterpret_cast<const float4*>(x + c * 8 + 4);
                acc[s] = dot8(w, xa, xb, acc[s]);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int s = 0; s < 8; ++s) acc[s] += __shfl_xor_sync(0xffffffffu, acc[s], o);
#pragma unroll
        for (int s = 0; s < 8; ++s)
            if (alive[s]) routed = fmaf(round_bf16(acc[s]), s_w[s0 + s], routed);
    }
    float out = routed;
    if (shrow) {
        const float* x = xin + K * I;
        float acc = 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = lane + 32 * u;
            if (c < sh_pieces) {
                const float4 xa = *reinterpret_cast<const float4*>(x + c * 8), xb = *reinterpret_cast<const float4*>(x + c * 8 + 4);
                acc = dot8(shw[u], xa, xb, acc);
            }
        }
        for (int c = lane + 128; c < sh_pieces; c += 32) {
            const uint4 w = ld_stream16(shrow + c);
            const float4 xa = *reinterpret_cast<const float4*>(x + c * 8), xb = *reinterpret_cast<const float4*>(x + c * 8 + 4);
            acc = dot8(w, xa, xb, acc);
        }
        const float sh_raw = warp_sum(acc);
        if (p.partial) {                                         // sharded: the ranks' dots are added before the rounding
            if (lane == 0) p.partial[p.hidden + j] = sh_raw;
        } else {
            float sh = round_bf16(sh_raw);
            if (p.shared_gate_logit) sh *= 1.f / (1.f + expf(-*p.shared_gate_logit));
            out += sh;
        }
    }
    if (lane == 0) {
        if (p.partial) p.partial[j] = routed;
        else p.out[j] = res + out;
    }
}

cudaError_t moe_down_f32_launch(const MoeDownF32Params& p, cudaStream_t stream, bool pdl) {
    const size_t smem = (size_t(p.top_k) * p.inter + p.shared_inter) * sizeof(float);
    if (smem > 48 * 1024) {
        static PerDeviceOnce once;
        if (once.first()) {
            cudaError_t e = cudaFuncSetAttribute(moe_down_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            if (e != cudaSuccess) return e;}
    }
    const dim3 grid((p.hidden + kDownWarps - 1) / kDownWarps), block(kDownWarps * 32);
    return launch_kernel(moe_down_f32_kernel, grid, block, smem, stream, pdl, p);
}

}  // namespace tfb
