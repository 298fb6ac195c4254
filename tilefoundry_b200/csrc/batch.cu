// Row-wise kernels of the several-sequence decode step (batch <= 32): each sequence keeps its own token history
// and position on the device, the projections between these kernels run on the tensor cores (gemm_tc.cu).
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

// ---- embedding: row b = table[tokens[b][pos[b]]] -------------------------------------------------
__global__ void embed_rows_kernel(const uint16_t* __restrict__ table, const long long* __restrict__ tokens,
                                  const int* __restrict__ pos, int max_tokens, uint16_t* __restrict__ out, int hidden,
                                  long long vocab) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    int cur = pos[b];
    cur = cur < 0 ? 0 : (cur >= max_tokens ? max_tokens - 1 : cur);
    long long id = tokens[size_t(b) * max_tokens + cur];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const uint4* src = reinterpret_cast<const uint4*>(table + size_t(id) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(out + size_t(b) * hidden);
    for (int c = threadIdx.x; c < (hidden >> 3); c += blockDim.x) dst[c] = src[c];
}

cudaError_t embed_rows_launch(const uint16_t* table, const long long* tokens, const int* pos, int max_tokens,
                              uint16_t* out, int rows, int hidden, long long vocab, cudaStream_t stream, bool pdl) {
    return launch_kernel(embed_rows_kernel, dim3(rows), dim3(256), 0, stream, pdl, table, tokens, pos, max_tokens, out,
                         hidden, vocab);
}

// ---- greedy pick per sequence: lowest index of the largest bf16 logit, then advance that sequence ------
// Grid (rows, kPickParts): each CTA scans one slice of a row; the last CTA of a row to finish (atomic ticket, no
// spinning) merges the kPickParts candidates, writes the token into the row's history unless the prompt still
// dictates it, and moves the row's position on.
constexpr int kPickParts = 8, kPickThreads = 512;

__device__ __forceinline__ void pick_merge(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__global__ void __launch_bounds__(kPickThreads) pick_rows_kernel(const uint16_t* __restrict__ logits, int vocab,
                                                                 long long* __restrict__ tokens, int* __restrict__ pos,
                                                                 int n_prompt, int max_tokens, long long* __restrict__ picked,
                                                                 float* __restrict__ part_val, int* __restrict__ part_idx,
                                                                 unsigned* __restrict__ tickets, float temperature,
                                                                 unsigned long long seed) {
    __shared__ float wv[kPickThreads / 32];
    __shared__ int wi[kPickThreads / 32];
    __shared__ int s_last;
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x, part = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint16_t* row = logits + size_t(b) * vocab;
    const int per = (((vocab + kPickParts - 1) / kPickParts) + 7) & ~7;     // slice length, a multiple of 8 elements
    const int begin = part * per, end = min(vocab, begin + per);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    if (temperature > 0.f) {
        // Gumbel-max sample of sequence b: the greedy pick over logit / T + noise (the rule and the generator of
        // lm_head_kernel); the draw is keyed by (seed + b, the sequence's position, vocabulary index)
        const int step = pos[b];
        for (int c = begin + threadIdx.x; c < end; c += kPickThreads)
            pick_merge(best, best_i, __fdiv_rn(bf16_bits_to_f32(row[c]), temperature) + gumbel_variate(seed + (unsigned long long)b, step, c), c);
    } else if ((vocab & 7) == 0) {     // 16-byte loads where the row allows it (vocab a multiple of 8 keeps every row aligned)
        for (int c = begin + threadIdx.x * 8; c < end; c += kPickThreads * 8) {
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(row + c));
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                pick_merge(best, best_i, bf16_lo(u[i]), c + 2 * i);
                pick_merge(best, best_i, bf16_hi(u[i]), c + 2 * i + 1);
            }
        }
    } else {
        for (int c = begin + threadIdx.x; c < end; c += kPickThreads) pick_merge(best, best_i, bf16_bits_to_f32(row[c]), c);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        pick_merge(best, best_i, ov, oi);
    }
    if (lane == 0) { wv[warp] = best; wi[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kPickThreads / 32; ++w) pick_merge(best, best_i, wv[w], wi[w]);
        part_val[b * kPickParts + part] = best;
        part_idx[b * kPickParts + part] = best_i;
        __threadfence();
        s_last = atomicAdd(&tickets[b], 1u) == unsigned(kPickParts - 1);
    }
    __syncthreads();
    if (!s_last || threadIdx.x != 0) return;
    __threadfence();
    best = -INFINITY;
    best_i = 0x7fffffff;
    for (int q = 0; q < kPickParts; ++q)
        pick_merge(best, best_i, __ldcg(part_val + b * kPickParts + q), __ldcg(part_idx + b * kPickParts + q));
    if (picked) picked[b] = best_i;
    const int cur = pos[b];
    if (cur + 1 < max_tokens) {
        if (cur + 1 >= n_prompt) tokens[size_t(b) * max_tokens + cur + 1] = best_i;
        pos[b] = cur + 1;
    }
    tickets[b] = 0;
}

int pick_rows_parts() { return kPickParts; }

cudaError_t pick_rows_launch(const uint16_t* logits, int rows, int vocab, long long* tokens, int* pos, int n_prompt,
                             int max_tokens, long long* picked, float* part_val, int* part_idx, unsigned* tickets,
                             float temperature, unsigned long long seed, cudaStream_t stream, bool pdl) {
    return launch_kernel(pick_rows_kernel, dim3(rows, kPickParts), dim3(kPickThreads), 0, stream, pdl, logits, vocab,
                         tokens, pos, n_prompt, max_tokens, picked, part_val, part_idx, tickets, temperature, seed);
}

}  // namespace tfb
