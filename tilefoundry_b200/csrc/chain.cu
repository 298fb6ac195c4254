// A chain of dependent batch-1 projections in ONE persistent launch (one CTA per SM):
//   phase 0: o-projection + residual -> phase 1: norm + gate/up + SwiGLU -> phase 2: down + residual
//   (-> phase 3: the next layer's norm + q|k|v projection)
// Each phase needs every output of the one before, so phases are separated by a grid-wide barrier.  What
// the single launch buys: the weight stream never stops at a phase boundary.  Every warp owns a ring in
// shared memory that it fills with per-thread 16-byte cp.async copies, and its copy cursor runs through the
// units of ALL phases in order -- weights do not depend on activations -- so while a CTA waits at the
// barrier and restages the activation vector, about 160 KB per SM of the next phase's weights keep
// arriving.  Separate launches instead pay (measured) about 4 us per boundary in which HBM idles.
//
// Unit = (output row, K-slice of one 2 KB stage); units of a phase go round-robin to the CTA's 16 warps;
// each lane copies and later reads only its own 16-byte pieces, so the data path needs no barrier besides
// the lane's own cp.async.wait_group.  Unit sums are parked in shared memory; at the end of a phase the
// K-slices of a row are added in fixed order (deterministic), the epilogue applied and the rows written.
// Rounding points are those of gemv_kernel (gemv.cu).
//
// The grid barrier is a monotonic counter in global memory; every spin on it is bounded and a timeout
// sets *status instead of hanging.  All CTAs must be co-resident: the launch is cooperative.
//
// HBM-bound: algorithmic bytes per launch = sum over phases of n*k*2 (x2 for SwiGLU).
#include "common.cuh"
#include "gemv.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

constexpr int kChainWarps = 16;
constexpr int kChainThreads = kChainWarps * 32;
constexpr int kSlotBytes = 2048;
constexpr int kChainStages = 5;
constexpr int kChainRing = kSlotBytes * kChainStages;          // per warp
constexpr unsigned kSpinLimit = 1u << 18;                      // x (20 ns sleep + one L2 read): a fraction of a second

__device__ __forceinline__ void chain_cp16(uint32_t smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void chain_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ uint4 chain_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Activation of a phase into xs (f32, the staging permutation of gemv.cuh), read through L2: another SM wrote it
// during this launch, so L1 must not serve it.
__device__ void chain_stage(const ChainPhase& ph, float* xs, float* red) {
    const int pieces = ph.k >> 3;
    float4* dst = reinterpret_cast<float4*>(xs);
    float ss = 0.f;
    for (int c = threadIdx.x; c < pieces; c += blockDim.x) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(ph.x) + c);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[2 * i] = bf16_lo(u[i]); f[2 * i + 1] = bf16_hi(u[i]); }
        if (ph.norm != 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
        } else if (ph.x_scale != 1.f) {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = round_bf16(apply_scale(f[i], ph.x_scale));
        }
        const int it = c >> 5, lane = c & 31;
        dst[(it * 2) * 32 + lane] = make_float4(f[0], f[1], f[2], f[3]);
        dst[(it * 2 + 1) * 32 + lane] = make_float4(f[4], f[5], f[6], f[7]);
    }
    if (ph.norm == 0) return;
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / float(ph.k) + ph.eps);
    for (int c = threadIdx.x; c < pieces; c += blockDim.x) {   // each thread rescales the pieces it wrote itself
        const int it = c >> 5, lane = c & 31;
        const float4 lo = dst[(it * 2) * 32 + lane], hi = dst[(it * 2 + 1) * 32 + lane];
        float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        const uint4 g = *(reinterpret_cast<const uint4*>(ph.gamma) + c);
        const uint32_t gg[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (ph.norm == 2) {                              // round, then gain (a bf16 multiply)
                f[2 * i] = round_bf16(round_bf16(f[2 * i] * rstd) * bf16_lo(gg[i]));
                f[2 * i + 1] = round_bf16(round_bf16(f[2 * i + 1] * rstd) * bf16_hi(gg[i]));
            } else {                                         // f32 through the gain, one rounding
                f[2 * i] = round_bf16(f[2 * i] * rstd * bf16_lo(gg[i]));
                f[2 * i + 1] = round_bf16(f[2 * i + 1] * rstd * bf16_hi(gg[i]));
            }
        }
        if (ph.x_scale != 1.f) {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = round_bf16(apply_scale(f[i], ph.x_scale));
        }
        dst[(it * 2) * 32 + lane] = make_float4(f[0], f[1], f[2], f[3]);
        dst[(it * 2 + 1) * 32 + lane] = make_float4(f[4], f[5], f[6], f[7]);
    }
}

__global__ void __launch_bounds__(kChainThreads, 1) gemv_chain_kernel(const ChainParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* xs = reinterpret_cast<float*>(smem_raw);                         // kmax floats
    float* red = xs + p.kmax;                                               // 32 floats
    float* part = red + 32;                                                 // part_floats
    unsigned char* ring = reinterpret_cast<unsigned char*>(part + p.part_floats);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int P = p.n_phases;
    const uint32_t ring_base = uint32_t(__cvta_generic_to_shared(ring + warp * kChainRing)) + lane * 16;

    // per-phase geometry of this CTA
    __shared__ int row_lo[4], units[4];
    if (threadIdx.x < 4) {
        const int q = threadIdx.x;
        row_lo[q] = 0; units[q] = 0;
        if (q < P) {
            const ChainPhase& ph = p.ph[q];
            row_lo[q] = int((long long)ph.n * blockIdx.x / gridDim.x);
            const int hi = int((long long)ph.n * (blockIdx.x + 1) / gridDim.x);
            units[q] = (hi - row_lo[q]) * ph.ksplit;
        }
    }
    __syncthreads();

    // ---- copy cursor: runs through the units of all phases, kChainStages stages ahead of the arithmetic ----
    int ip = 0, iu = warp;
    unsigned issued = 0;
    auto issue = [&]() {
        while (ip < P && iu >= units[ip]) { ++ip; iu = warp; }
        if (ip < P) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (q == ip) {
                    const ChainPhase& ph = p.ph[q];
                    const int row = row_lo[q] + iu / ph.ksplit, ks = iu % ph.ksplit;
                    const int it0 = ks * ph.si;
                    const uint32_t dst = ring_base + (issued % kChainStages) * kSlotBytes;
                    const uint4* src = ph.w + size_t(row) * (ph.k >> 3) + it0 * 32 + lane;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (i < ph.si) chain_cp16(dst + i * 512, src + i * 32);
                    if (ph.epi == 2) {
                        const uint4* src2 = ph.w2 + size_t(row) * (ph.k >> 3) + it0 * 32 + lane;
#pragma unroll
                        for (int i = 0; i < 2; ++i)
                            if (i < ph.si) chain_cp16(dst + (ph.si + i) * 512, src2 + i * 32);
                    }
                }
            }
            iu += kChainWarps;
        }
        chain_commit();                                        // always: keeps the group count uniform
        ++issued;
    };
#pragma unroll 1
    for (int s = 0; s < kChainStages; ++s) issue();
    pdl_trigger();
    pdl_wait();

    unsigned consumed = 0;
    const float4* x4 = reinterpret_cast<const float4*>(xs);
#pragma unroll 1
    for (int q = 0; q < P; ++q) {
        const ChainPhase& ph = p.ph[q];
        if (q > 0) {                                           // every CTA has written the phase before
            if (threadIdx.x == 0) {
                const unsigned target = unsigned(q) * gridDim.x;
                unsigned spins = 0;
                while (ld_acquire_u32(p.barrier) < target) {
                    if (++spins > kSpinLimit) { atomicExch(p.status, 0x100u + q); break; }
                    __nanosleep(20);
                }
            }
            __syncthreads();
        }
        chain_stage(ph, xs, red);
        __syncthreads();

        const int nmat = ph.epi == 2 ? 2 : 1, si = ph.si;
        for (int u = warp; u < units[q]; u += kChainWarps) {
            asm volatile("cp.async.wait_group %0;" :: "n"(kChainStages - 1) : "memory");
            const int it0 = (u % ph.ksplit) * si;
            const uint32_t src = ring_base + (consumed % kChainStages) * kSlotBytes;
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (i < si) {
                    const float4 xa = x4[((it0 + i) * 2) * 32 + lane], xb = x4[((it0 + i) * 2 + 1) * 32 + lane];
                    const uint4 w = chain_lds128(src + i * 512);
                    if (i & 1) a1 = dot8(w, xa, xb, a1); else a0 = dot8(w, xa, xb, a0);
                    if (nmat == 2 && i < 2) {
                        const uint4 w2 = chain_lds128(src + (si + i) * 512);
                        if (i & 1) b1 = dot8(w2, xa, xb, b1); else b0 = dot8(w2, xa, xb, b0);
                    }
                }
            }
            ++consumed;
            issue();                                           // refill the slot just read
            const float v = warp_sum(a0 + a1);
            const float v2 = nmat == 2 ? warp_sum(b0 + b1) : 0.f;
            if (lane == 0) {
                part[u * nmat] = v;
                if (nmat == 2) part[u * nmat + 1] = v2;
            }
        }
        __syncthreads();

        // ---- K-slices added in fixed order, epilogue, coalesced stores ----
        const int rows = units[q] / ph.ksplit;
        for (int r = threadIdx.x; r < rows; r += blockDim.x) {
            float v = 0.f, v2 = 0.f;
            for (int ks = 0; ks < ph.ksplit; ++ks) {
                v += part[(r * ph.ksplit + ks) * nmat];
                if (nmat == 2) v2 += part[(r * ph.ksplit + ks) * nmat + 1];
            }
            const int row = row_lo[q] + r;
            if (ph.epi == 0) {
                ph.y[row] = f32_to_bf16_bits(v);
            } else if (ph.epi == 1) {
                float o = round_bf16(v);
                if (ph.res_scale != 1.f) o = round_bf16(o * ph.res_scale);
                ph.y[row] = f32_to_bf16_bits(bf16_bits_to_f32(__ldcg(ph.residual + row)) + o);
            } else {
                const float g = round_bf16(v), uu = round_bf16(v2);
                ph.y[row] = f32_to_bf16_bits(round_bf16(silu_f32(g)) * uu);
            }
        }
        if (q + 1 < P) {                                       // arrive: this CTA's rows of phase q are visible
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) atomicAdd(p.barrier, 1u);
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    // the last CTA to leave puts the counters back for the next launch
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(p.barrier + 1, 1u);
        if (t == gridDim.x - 1) { p.barrier[0] = 0; p.barrier[1] = 0; __threadfence(); }
    }
}

cudaError_t gemv_chain_launch(ChainParams& p, cudaStream_t stream, bool pdl, size_t* smem_out) {
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    int kmax = 0, part = 0;
    for (int q = 0; q < p.n_phases; ++q) {
        ChainPhase& ph = p.ph[q];
        const int nmat = ph.epi == 2 ? 2 : 1;
        const int its = ph.k >> 8;
        const int rows_cta = (ph.n + sms - 1) / sms + 1;
        // stage = 2 KB per warp: 4 iterations of one matrix or 2 of two; thinner stages when the phase is
        // too small to give every warp a few units
        int si = nmat == 2 ? 2 : 4;
        while (si > 1 && (its % si != 0 || rows_cta * (its / si) < 4 * kChainWarps)) si >>= 1;
        ph.si = si;
        ph.ksplit = its / si;
        if (ph.k > kmax) kmax = ph.k;
        const int need = rows_cta * ph.ksplit * nmat;
        if (need > part) part = need;
    }
    p.kmax = kmax;
    p.part_floats = (part + 3) & ~3;
    const size_t smem = (size_t(kmax) + 32 + p.part_floats) * sizeof(float) + size_t(kChainWarps) * kChainRing;
    if (smem_out) *smem_out = smem;
    if (smem > 227 * 1024) return cudaErrorInvalidValue;
    static size_t set_smem_dev[kMaxDevices] = {};          // the opt-in is per device
    size_t& set_smem = set_smem_dev[dev >= 0 && dev < kMaxDevices ? dev : 0];
    if (smem > set_smem) {
        e = cudaFuncSetAttribute(gemv_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        set_smem = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms);
    cfg.blockDim = dim3(kChainThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;              // every CTA resident: the grid barrier needs it
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, gemv_chain_kernel, p);
}

}  // namespace tfb
