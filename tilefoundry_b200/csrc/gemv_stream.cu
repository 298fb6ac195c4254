// Persistent weight-streaming GEMV: y = epilogue(W . prologue(x)), one CTA per SM.
//
// HBM-bound.  Algorithmic bytes per launch = n*k*2 (x2 for SwiGLU, which reads a gate
// and an up matrix).  Each CTA owns a contiguous, balanced range of outputs and
// streams their weight rows through a shared-memory ring filled by bulk async copies
// (cp.async.bulk + mbarrier transaction counts), issued by a dedicated producer warp.
// The producer starts filling the ring before griddepcontrol.wait: weights never
// depend on the preceding kernel, so with programmatic dependent launch the next
// projection's first ~96 KB per SM are already in flight while the previous kernel
// drains, and HBM stays busy across kernel boundaries.
//
// A stage holds up to 16 row segments of kc elements (kc*2 bytes each, one bulk copy
// per segment).  Eight consumer warps each own two segments of the stage (two
// outputs, or one output's gate and up rows) and keep their partial dot products in
// registers across the k/kc stages of a tile, so no cross-warp reduction is needed
// and the summation order is fixed.  The activation vector is staged once per CTA as
// f32 in the conflict-free permuted layout of gemv.cuh.
//
// Every mbarrier wait is bounded: on exhaustion the thread records a status word (if
// the caller gave one) and leaves the kernel.
#include "gemv.cuh"
#include "kernels.h"
#include "launch.h"

#include <cstdlib>

namespace tfb {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kStreamThreads = kConsumerThreads + 32;   // + producer warp
constexpr int kSegs = 16;                               // row segments per stage
constexpr int kMaxStages = 8;
constexpr int kRingBytes = 96 * 1024;
constexpr unsigned kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; false = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (i > 64) __nanosleep(32);
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;" :: "n"(kConsumerThreads) : "memory");
}

// stage_activation for the consumer group only (named barrier instead of __syncthreads)
template <int NORM_MODE>
__device__ __forceinline__ void stage_activation_group(const uint16_t* __restrict__ x,
                                                       const uint16_t* __restrict__ gamma, float* xs,
                                                       float* red, int k, float eps, float x_scale) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float rstd = 1.f;
    if (NORM_MODE != 0) {
        float ss = 0.f;
        for (int c = tid; c < (k >> 3); c += kConsumerThreads) {
            const uint4 v = *reinterpret_cast<const uint4*>(x + (c << 3));
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float a = bf16_lo(u[i]), b = bf16_hi(u[i]);
                ss = fmaf(a, a, ss);
                ss = fmaf(b, b, ss);
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        consumer_sync();
        float t = lane < kConsumerWarps ? red[lane] : 0.f;
        t = warp_sum(t);
        rstd = rsqrtf(t / float(k) + eps);
    }
    for (int c = tid; c < (k >> 3); c += kConsumerThreads) {
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
                if (NORM_MODE == 2) {
                    f[2 * i] = round_bf16(round_bf16(f[2 * i] * rstd) * g0);
                    f[2 * i + 1] = round_bf16(round_bf16(f[2 * i + 1] * rstd) * g1);
                } else {
                    f[2 * i] = round_bf16(f[2 * i] * rstd * g0);
                    f[2 * i + 1] = round_bf16(f[2 * i + 1] * rstd * g1);
                }
            }
        }
        if (x_scale != 1.f) {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = round_bf16(apply_scale(f[i], x_scale));
        }
        const int it = c >> 5, ln = c & 31;
        float4* dst = reinterpret_cast<float4*>(xs);
        dst[(it * 2) * 32 + ln] = make_float4(f[0], f[1], f[2], f[3]);
        dst[(it * 2 + 1) * 32 + ln] = make_float4(f[4], f[5], f[6], f[7]);
    }
    consumer_sync();
}

__device__ __forceinline__ void argmax_take(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// EPI: 0 store bf16, 1 residual, 2 SwiGLU, 3 store f32, 4 lm_head (bf16 logits + greedy pick)
template <int NORM_MODE, int EPI>
__global__ void __launch_bounds__(kStreamThreads, 1) gemv_stream_kernel(const GemvParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int OUT_PER_TILE = (EPI == 2) ? kSegs / 2 : kSegs;
    const int kc = p.kc, nstages = p.nstages;
    const int seg_bytes = kc * 2, stage_bytes = kSegs * seg_bytes;
    unsigned char* ring = smem_raw;
    float* xs = reinterpret_cast<float*>(smem_raw + size_t(nstages) * stage_bytes);
    float* red = xs + p.k;
    uint64_t* full = reinterpret_cast<uint64_t*>(red + 32);
    uint64_t* empty = full + kMaxStages;
    __shared__ float wv[kConsumerWarps];
    __shared__ int wi[kConsumerWarps];
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long o_begin = (long long)p.n * blockIdx.x / gridDim.x;
    const long long o_end = (long long)p.n * (blockIdx.x + 1) / gridDim.x;
    const int n_out = int(o_end - o_begin);
    const int n_tiles = (n_out + OUT_PER_TILE - 1) / OUT_PER_TILE;
    const int kch = p.k / kc;                               // stages per tile
    const int total = n_tiles * kch;

    if (tid == 0) {
        for (int s = 0; s < nstages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, kConsumerWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();

    if (warp == kConsumerWarps) {
        // ---------------- producer warp: weights only, never waits on the previous kernel -----
        if (lane == 0) l2_prefetch_slice(p.prefetch, p.prefetch_bytes, blockIdx.x, gridDim.x);
        const unsigned char* wb = reinterpret_cast<const unsigned char*>(p.w);
        const unsigned char* w2b = reinterpret_cast<const unsigned char*>(p.w2);
        const size_t row_bytes = size_t(p.k) * 2;
        for (int q = 0; q < total; ++q) {
            const int slot = q % nstages;
            const unsigned phase = (q / nstages) & 1;
            if (!mbar_wait(empty + slot, phase ^ 1)) {
                if (lane == 0 && p.status) atomicExch(p.status, 1u);
                return;
            }
            const int tile = q / kch, chunk = q % kch;
            const long long o = o_begin + (long long)tile * OUT_PER_TILE;
            const int valid = min(OUT_PER_TILE, int(o_end - o));
            if (lane == 0) mbar_expect_tx(full + slot, unsigned(valid * (EPI == 2 ? 2 : 1) * seg_bytes));
            __syncwarp();
            unsigned char* stage = ring + size_t(slot) * stage_bytes;
            if (EPI == 2) {
                if (lane < kSegs) {
                    const int r = lane & 7;
                    if (r < valid) {
                        const unsigned char* src = (lane < 8 ? wb : w2b) + size_t(o + r) * row_bytes + size_t(chunk) * seg_bytes;
                        bulk_g2s(stage + lane * seg_bytes, src, seg_bytes, full + slot);
                    }
                }
            } else if (lane < valid) {
                bulk_g2s(stage + lane * seg_bytes, wb + size_t(o + lane) * row_bytes + size_t(chunk) * seg_bytes,
                         seg_bytes, full + slot);
            }
            // Once the ring is full for the first time the producer would stall until the consumers
            // (still waiting on the previous kernel) free a stage, and HBM would idle.  Ask the L2
            // to fetch the rest of this CTA's rows meanwhile; later ring fills then hit L2.
            if (p.self_prefetch && q == min(nstages, total) - 1 && lane == 0) {
                const size_t done_rows = size_t(min(nstages / kch, n_tiles)) * OUT_PER_TILE;
                if (done_rows < size_t(n_out)) {
                    const size_t off = size_t(o_begin + done_rows) * row_bytes;
                    size_t left = (size_t(n_out) - done_rows) * row_bytes;
                    for (int m = 0; m < (EPI == 2 ? 2 : 1); ++m) {
                        const unsigned char* src = (m == 0 ? wb : w2b) + off;
                        for (size_t b = 0; b < left; b += 65536)
                            l2_prefetch_bulk(src + b, unsigned(min(left - b, size_t(65536))));
                    }
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------------------------------------------------------
    pdl_wait();
    stage_activation_group<NORM_MODE>(p.x, p.gamma, xs, red, p.k, p.eps, p.x_scale);

    const int seg_a = (EPI == 2) ? warp : 2 * warp;          // first segment this warp reads
    const int seg_b = (EPI == 2) ? 8 + warp : 2 * warp + 1;
    const int its = kc >> 8;                                 // 256-element iterations per stage
    const float4* x4 = reinterpret_cast<const float4*>(xs);
    float best = -INFINITY;
    int best_i = 0x7fffffff;

    for (int tile = 0; tile < n_tiles; ++tile) {
        const long long o = o_begin + (long long)tile * OUT_PER_TILE;
        const int valid = min(OUT_PER_TILE, int(o_end - o));
        const int my_first = (EPI == 2) ? warp : 2 * warp;   // first output index within the tile
        const bool have_a = my_first < valid;
        const bool have_b = (EPI == 2) ? have_a : (my_first + 1 < valid);
        float acc_a = 0.f, acc_b = 0.f;
        for (int chunk = 0; chunk < kch; ++chunk) {
            const int q = tile * kch + chunk;
            const int slot = q % nstages;
            if (!mbar_wait(full + slot, (q / nstages) & 1)) {
                if (lane == 0 && p.status) atomicExch(p.status, 2u);
                return;
            }
            const unsigned char* stage = ring + size_t(slot) * stage_bytes;
            const uint4* sa = reinterpret_cast<const uint4*>(stage + seg_a * seg_bytes);
            const uint4* sb = reinterpret_cast<const uint4*>(stage + seg_b * seg_bytes);
            if (have_a) {
                const int it_base = chunk * its;
#pragma unroll 4
                for (int it = 0; it < its; ++it) {
                    const float4 xa = x4[((it_base + it) * 2) * 32 + lane];
                    const float4 xb = x4[((it_base + it) * 2 + 1) * 32 + lane];
                    const uint4 wa = sa[it * 32 + lane];
                    acc_a = dot8(wa, xa, xb, acc_a);
                    if (have_b) {
                        const uint4 wbv = sb[it * 32 + lane];
                        acc_b = dot8(wbv, xa, xb, acc_b);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + slot);
        }
        acc_a = warp_sum(acc_a);
        acc_b = warp_sum(acc_b);
        if (!have_a) continue;
        const long long row_a = o + my_first;
        if (EPI == 2) {
            if (lane == 0) {
                const float g = round_bf16(acc_a), u = round_bf16(acc_b);
                static_cast<uint16_t*>(p.y)[row_a] = f32_to_bf16_bits(round_bf16(silu_f32(g)) * u);
            }
        } else if (EPI == 4) {
            const float la = round_bf16(acc_a * p.out_scale);
            argmax_take(best, best_i, la, int(row_a));
            if (lane == 0 && p.y) static_cast<uint16_t*>(p.y)[row_a] = f32_to_bf16_bits(la);
            if (have_b) {
                const float lb = round_bf16(acc_b * p.out_scale);
                argmax_take(best, best_i, lb, int(row_a + 1));
                if (lane == 0 && p.y) static_cast<uint16_t*>(p.y)[row_a + 1] = f32_to_bf16_bits(lb);
            }
        } else if (lane < 2 && (lane == 0 || have_b)) {
            const float v = lane == 0 ? acc_a : acc_b;
            const long long row = row_a + lane;
            if (EPI == 0) {
                static_cast<uint16_t*>(p.y)[row] = f32_to_bf16_bits(v);
            } else if (EPI == 1) {
                float ov = round_bf16(v);
                if (p.res_scale != 1.f) ov = round_bf16(ov * p.res_scale);
                static_cast<uint16_t*>(p.y)[row] = f32_to_bf16_bits(bf16_bits_to_f32(p.residual[row]) + ov);
            } else {
                static_cast<float*>(p.y)[row] = v * p.out_scale;
            }
        }
    }

    if (EPI != 4) return;
    // ---------------- greedy pick: CTA pair -> scratch -> last CTA reduces ------------------------
    if (lane == 0) { wv[warp] = best; wi[warp] = best_i; }
    consumer_sync();
    if (tid == 0) {
        for (int w = 1; w < kConsumerWarps; ++w) argmax_take(best, best_i, wv[w], wi[w]);
        p.scratch_val[blockIdx.x] = best;
        p.scratch_idx[blockIdx.x] = best_i;
        __threadfence();
        s_last = (atomicAdd(p.counter, 1u) == gridDim.x - 1);
    }
    consumer_sync();
    if (!s_last) return;
    __threadfence();
    best = -INFINITY;
    best_i = 0x7fffffff;
    for (int c = tid; c < int(gridDim.x); c += kConsumerThreads)
        argmax_take(best, best_i, __ldcg(p.scratch_val + c), __ldcg(p.scratch_idx + c));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
        argmax_take(best, best_i, ov, oi);
    }
    consumer_sync();                         // wv/wi are about to be rewritten
    if (lane == 0) { wv[warp] = best; wi[warp] = best_i; }
    consumer_sync();
    if (tid == 0) {
        for (int w = 1; w < kConsumerWarps; ++w) argmax_take(best, best_i, wv[w], wi[w]);
        if (p.token_out) *p.token_out = best_i;
        if (p.tokens && p.pos) {
            const int cur = *p.pos;
            if (cur + 1 < p.max_tokens) {
                if (cur + 1 >= p.n_prompt) p.tokens[cur + 1] = best_i;
                *p.pos = cur + 1;
            }
        }
        *p.counter = 0;
    }
}

// ---- host side ---------------------------------------------------------------------------------

// Largest multiple of 256 (up to 1024) that divides k; 0 if k is not a multiple of 256.
static int pick_kc(int k) {
    for (int kc = 1024; kc >= 256; kc -= 256)
        if (k % kc == 0) return kc;
    return 0;
}

bool gemv_stream_supported(int n, int k) { return n > 0 && k > 0 && k % 256 == 0 && k <= 16384; }

template <int NORM_MODE, int EPI>
static cudaError_t launch_stream(GemvParams p, cudaStream_t stream, bool pdl) {
    p.kc = pick_kc(p.k);
    int ring_bytes = kRingBytes;
    if (const char* e = getenv("TFB_KC")) { const int v = atoi(e); if (v >= 256 && v % 256 == 0 && p.k % v == 0) p.kc = v; }
    if (const char* e = getenv("TFB_RING_KB")) { const int v = atoi(e); if (v >= 16 && v <= 190) ring_bytes = v * 1024; }
    const int stage_bytes = kSegs * p.kc * 2;
    p.nstages = max(1, min(kMaxStages, ring_bytes / stage_bytes));
    constexpr int OUT_PER_TILE = (EPI == 2) ? kSegs / 2 : kSegs;
    int grid = sm_count();
    const int max_useful = (p.n + OUT_PER_TILE / 2 - 1) / (OUT_PER_TILE / 2);
    if (grid > max_useful) grid = max_useful;
    const size_t smem = size_t(p.nstages) * stage_bytes + (size_t(p.k) + 32) * sizeof(float) +
                        2 * kMaxStages * sizeof(uint64_t);
    auto kern = gemv_stream_kernel<NORM_MODE, EPI>;
    static bool attr_set = false;                            // per instantiation
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        // Ask for the largest shared-memory carve-out: with the default, the SM is configured for
        // this kernel's ~105 KB alone and the next projection's CTA cannot move in beside it.
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    return launch_kernel(kern, dim3(grid), dim3(kStreamThreads), smem, stream, pdl, p);
}

cudaError_t gemv_stream_dispatch(const GemvParams& p, int norm_mode, int epi, cudaStream_t stream, bool pdl) {
#define TFB_CASE(NM, EP) \
    if (norm_mode == NM && epi == EP) return launch_stream<NM, EP>(p, stream, pdl);
    TFB_CASE(0, 0) TFB_CASE(1, 0) TFB_CASE(2, 0)
    TFB_CASE(0, 1) TFB_CASE(1, 1) TFB_CASE(2, 1)
    TFB_CASE(0, 2) TFB_CASE(1, 2) TFB_CASE(2, 2)
    TFB_CASE(0, 3) TFB_CASE(1, 3) TFB_CASE(2, 3)
    TFB_CASE(0, 4) TFB_CASE(1, 4) TFB_CASE(2, 4)
#undef TFB_CASE
    return cudaErrorInvalidValue;
}

int lm_head_stream_ctas() { return sm_count(); }

}  // namespace tfb
