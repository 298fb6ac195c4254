// Batch-1 weight-streaming projection y = epilogue(W . prologue(x)) with the weights landing in SHARED
// memory through per-thread 16-byte asynchronous copies (cp.async.cg), one persistent CTA per SM.
//
// Why: a B200 SM needs roughly bandwidth x latency = 44 GB/s x 2.5 us = 110 KB of loads in flight to hold
// its share of HBM bandwidth.  Loads that land in registers are capped by the register file (measured:
// ~80 KB in flight per SM, 4.5-5 TB/s); a ring in shared memory is not.  Each warp owns a private ring of
// STAGES stages; each LANE copies, and later reads back, only its own 16-byte pieces, so the only
// synchronisation on the data path is the lane's own cp.async.wait_group.  The ring is filled BEFORE the
// dependency wait, so about 100 KB per SM of the next projection's weights are already on chip when the
// kernel before it finishes.
//
// Work split: CTA b owns a contiguous block of output rows; a unit is (row, K-slice) and units go round-robin
// to the CTA's 8 warps, each unit in STAGE_ITS-iteration stages.  Unit results are parked in shared memory and
// one final pass adds the K-slices in fixed order (deterministic), applies the epilogue and writes the rows
// coalesced.  Same arithmetic and rounding points as gemv_kernel.
//
// HBM-bound: algorithmic bytes per launch = n*k*2 (x2 for SwiGLU).
#include "gemv.cuh"
#include "kernels.h"
#include "launch.h"


namespace tfb {

constexpr int kAsyncWarps = 8;
constexpr int kRingBytesPerWarp = 12 * 1024;

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

// NMAT 1 or 2 (SwiGLU streams gate and up rows together); SI = 256-element iterations per stage.
template <int NMAT, int SI, int NORM_MODE, int EPI>
__global__ void __launch_bounds__(kAsyncWarps * 32) gemv_async_kernel(const GemvParams p, const int ksplit) {
    constexpr int STAGE_BYTES = NMAT * SI * 512;
    constexpr int STAGES = kRingBytesPerWarp / STAGE_BYTES;
    static_assert(STAGES >= 2 && STAGES <= 16, "ring depth");
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;                                                   // k floats
    float* red = smem + p.k;                                            // 32 floats
    uint4* gs = reinterpret_cast<uint4*>(red + 32);                     // parked gains: k bf16 (norm modes)
    unsigned char* after = reinterpret_cast<unsigned char*>(gs) + (NORM_MODE ? size_t(p.k) * 2 : 0);
    unsigned char* ring = after;                                        // kAsyncWarps * kRingBytesPerWarp
    float* part = reinterpret_cast<float*>(ring + kAsyncWarps * kRingBytesPerWarp);   // rows_cta * ksplit * NMAT

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row_stride = p.k >> 3, its = p.k >> 8;
    const int it_per = (its + ksplit - 1) / ksplit;
    const int nst = (it_per + SI - 1) / SI;                             // stages per unit
    const int row_lo = int((long long)p.n * blockIdx.x / gridDim.x);
    const int row_hi = int((long long)p.n * (blockIdx.x + 1) / gridDim.x);
    const int units = (row_hi - row_lo) * ksplit;
    const int my_units = (units - warp + kAsyncWarps - 1) / kAsyncWarps;   // units warp, warp+8, ...
    const int Q = max(my_units, 0) * nst;
    const uint32_t ring_base = uint32_t(__cvta_generic_to_shared(ring + warp * kRingBytesPerWarp)) + lane * 16;

    trace_start(p.trace);
    auto issue = [&](int q) {
        if (q < Q) {
            const int j = q / nst, s = q - j * nst;
            const int u = warp + j * kAsyncWarps;
            const int row = row_lo + u / ksplit, ks = u % ksplit;
            const int it0 = ks * it_per + s * SI, it_end = min(its, (ks + 1) * it_per);
            const uint32_t dst = ring_base + (q % STAGES) * STAGE_BYTES;
            const uint4* src = p.w + size_t(row) * row_stride + lane;
            const uint4* src2 = (NMAT == 2) ? p.w2 + size_t(row) * row_stride + lane : nullptr;
#pragma unroll
            for (int i = 0; i < SI; ++i) {
                if (it0 + i < it_end) {
                    cp_async_16(dst + i * 512, src + (it0 + i) * 32);
                    if (NMAT == 2) cp_async_16(dst + (SI + i) * 512, src2 + (it0 + i) * 32);
                }
            }
        }
        cp_async_commit();                                              // always: keeps the group count uniform
    };
#pragma unroll 1
    for (int q = 0; q < STAGES; ++q) issue(q);                          // the whole ring before the wait
    constexpr int MAXC = 4;
    const bool fast_stage = (p.k >> 3) <= MAXC * kAsyncWarps * 32;
    if (fast_stage) StagedGain<MAXC>::template preload<NORM_MODE>(p.gamma, gs, p.k);

    pdl_trigger();
    pdl_wait();
    trace_waited(p.trace);
    if (fast_stage) StagedGain<MAXC>::template stage<NORM_MODE>(p.x, p.x2, gs, xs, red, p.k, p.eps, p.x_scale);
    else stage_activation<NORM_MODE>(p.x, p.gamma, xs, red, p.k, p.eps, p.x_scale);
    __syncthreads();
    trace_mark(p.trace, 0);

    const float4* x4 = reinterpret_cast<const float4*>(xs);
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;              // (matrix 0 even/odd piece), (matrix 1 even/odd)
#pragma unroll 1
    for (int q = 0; q < Q; ++q) {
        cp_async_wait<STAGES - 1>();                                    // this lane's copies of stage q have landed
        const int j = q / nst, s = q - j * nst;
        const int u = warp + j * kAsyncWarps;
        const int ks = u % ksplit;
        const int it0 = ks * it_per + s * SI, it_end = min(its, (ks + 1) * it_per);
        const uint32_t src = ring_base + (q % STAGES) * STAGE_BYTES;
#pragma unroll
        for (int i = 0; i < SI; ++i) {
            if (it0 + i < it_end) {
                const float4 xa = x4[((it0 + i) * 2) * 32 + lane], xb = x4[((it0 + i) * 2 + 1) * 32 + lane];
                const uint4 w = lds128(src + i * 512);
                if (i & 1) acc1 = dot8(w, xa, xb, acc1); else acc0 = dot8(w, xa, xb, acc0);
                if (NMAT == 2) {
                    const uint4 w2 = lds128(src + (SI + i) * 512);
                    if (i & 1) acc3 = dot8(w2, xa, xb, acc3); else acc2 = dot8(w2, xa, xb, acc2);
                }
            }
        }
        issue(q + STAGES);                                              // refill the slot just read
        if (s == nst - 1) {
            const float v = warp_sum(acc0 + acc1);
            const float v2 = (NMAT == 2) ? warp_sum(acc2 + acc3) : 0.f;
            if (lane == 0) {
                part[u * NMAT] = v;
                if (NMAT == 2) part[u * NMAT + 1] = v2;
            }
            acc0 = acc1 = acc2 = acc3 = 0.f;
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- K-slices added in fixed order, epilogue, coalesced stores ----
    for (int r = threadIdx.x; r < row_hi - row_lo; r += blockDim.x) {
        float v = 0.f, v2 = 0.f;
        for (int ks = 0; ks < ksplit; ++ks) {
            v += part[(r * ksplit + ks) * NMAT];
            if (NMAT == 2) v2 += part[(r * ksplit + ks) * NMAT + 1];
        }
        const int row = row_lo + r;
        if (EPI == 0) {
            static_cast<uint16_t*>(p.y)[row] = f32_to_bf16_bits(v);
        } else if (EPI == 1) {
            float o = round_bf16(v);
            if (p.res_scale != 1.f) o = round_bf16(o * p.res_scale);
            static_cast<uint16_t*>(p.y)[row] = f32_to_bf16_bits(bf16_bits_to_f32(p.residual[row]) + o);
        } else if (EPI == 2) {
            const float g = round_bf16(v), u = round_bf16(v2);
            static_cast<uint16_t*>(p.y)[row] = f32_to_bf16_bits(round_bf16(silu_f32(g)) * u);
        } else {
            static_cast<float*>(p.y)[row] = v * p.out_scale;
        }
    }
    trace_end(p.trace);
}

static int async_sm_count() { return sm_count(); }

template <int NMAT, int SI, int NORM_MODE, int EPI>
static cudaError_t launch_async(const GemvParams& p, cudaStream_t stream, bool pdl) {
    int grid = 2 * async_sm_count();                    // two CTAs (16 warps, 192 KB of ring) per SM measured best
    if (grid > p.n) grid = p.n;
    const int rows_cta = (p.n + grid - 1) / grid + 1;
    // K-slices per row: enough units for ~10 per warp, but never thinner than one stage
    const int its = p.k >> 8;
    int ksplit = 1;
    while (rows_cta * ksplit < 10 * kAsyncWarps && (its / (ksplit * 2)) >= SI && its % (ksplit * 2) == 0) ksplit *= 2;
    if (ksplit < 1) ksplit = 1;
    const size_t smem = (size_t(p.k) + 32) * sizeof(float) + (NORM_MODE ? size_t(p.k) * 2 : 0) +
                        size_t(kAsyncWarps) * kRingBytesPerWarp + size_t(rows_cta) * ksplit * NMAT * sizeof(float);
    auto kern = gemv_async_kernel<NMAT, SI, NORM_MODE, EPI>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    return launch_kernel(kern, dim3(grid), dim3(kAsyncWarps * 32), smem, stream, pdl, p, ksplit);
}

bool gemv_async_supported(const GemvParams& p, int norm_mode, int epi) {
    return p.expert_idx == nullptr && norm_mode != 3 && epi <= 2 && p.n >= 1024 && p.k <= 8192;
}

cudaError_t gemv_async_dispatch(const GemvParams& p, int norm_mode, int epi, cudaStream_t stream, bool pdl) {
#define TFB_CASE(NM, EP) \
    if (norm_mode == NM && epi == EP) return launch_async<(EP == 2 ? 2 : 1), 2, NM, EP>(p, stream, pdl);
    TFB_CASE(0, 0) TFB_CASE(1, 0) TFB_CASE(2, 0)
    TFB_CASE(0, 1) TFB_CASE(1, 1) TFB_CASE(2, 1)
    TFB_CASE(0, 2) TFB_CASE(1, 2) TFB_CASE(2, 2)
#undef TFB_CASE
    return cudaErrorInvalidValue;
}

}  // namespace tfb
