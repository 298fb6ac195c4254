// Top-k expert selection by one warp, shared by the stand-alone router kernel and the kernels that select in
// their own prologue.
#pragma once
#include "common.cuh"

namespace tfb {

// mode 0 (granite, examples/granite_4_0_h_small-cuda/model.py:376-386): logits -> top-k -> softmax over the k.
// mode 1 (Qwen3.5, examples/qwen3_5_35b_a3b-tilelang/model.py:488-499): softmax over ALL experts in f32 ->
//        top-k -> renormalise by the sum of the k.
// Selection order is by value descending; equal values resolve to the lower index.  On return lane j < top_k
// holds the j-th selection (expert index and routing weight).
template <int MAXE>
__device__ __forceinline__ void route_select(const float* __restrict__ logits_f32, const uint16_t* __restrict__ logits_bf16,
                                             int experts, int top_k, int mode, int lane, float& weight, int& expert) {
    constexpr int PER = MAXE / 32;
    float v[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        v[i] = -INFINITY;
        if (e < experts) v[i] = logits_f32 ? __ldcg(logits_f32 + e) : bf16_bits_to_f32(logits_bf16[e]);
    }
    if (mode == 1) {                           // probabilities over all experts
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < PER; ++i) m = fmaxf(m, v[i]);
        m = warp_max(m);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) { v[i] = (lane + 32 * i < experts) ? expf(v[i] - m) : -INFINITY; s += fmaxf(v[i], 0.f); }
        s = warp_sum(s);
#pragma unroll
        for (int i = 0; i < PER; ++i) if (lane + 32 * i < experts) v[i] = v[i] / s;
    }
    float top_v = 0.f;                          // lane j keeps the j-th selection
    int top_i = 0;
    for (int j = 0; j < top_k; ++j) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = lane + 32 * i;
            if (e < experts && (v[i] > best || (v[i] == best && e < best_e))) { best = v[i]; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
        }
        if (lane == j) { top_v = best; top_i = best_e; }
#pragma unroll
        for (int i = 0; i < PER; ++i) if (lane + 32 * i == best_e) v[i] = -INFINITY;
    }
    const bool mine = lane < top_k;
    if (mode == 0) {
        const float m = warp_max(mine ? top_v : -INFINITY);
        const float e = mine ? expf(top_v - m) : 0.f;
        weight = e / warp_sum(e);
    } else {
        weight = top_v / warp_sum(mine ? top_v : 0.f);
    }
    expert = top_i;
}

}  // namespace tfb
