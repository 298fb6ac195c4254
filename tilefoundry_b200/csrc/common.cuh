// Shared device helpers for the decode kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tfb {

constexpr int kWarp = 32;

// ---- bf16 <-> f32 ---------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }
// round-to-nearest-even f32 -> bf16, returned as f32 (a value bf16 holds exactly)
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float x) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}

// ---- streaming loads ------------------------------------------------------
// Weights are read once per token: keep them out of L1.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// Read through L2 (data another SM has just written).
__device__ __forceinline__ float ld_cg_f32(const float* p) { return __ldcg(p); }

// ---- programmatic dependent launch ----------------------------------------
// wait: blocks until every grid this one depends on has completed and its writes
// are visible; a no-op when the launch carried no programmatic dependency.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// trigger: lets the next grid in the stream begin its own pre-wait part.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Ask the L2 to fetch [p, p+bytes) from HBM; p 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void l2_prefetch_bulk(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(p), "r"(bytes) : "memory");
}
// Slice `total` bytes at `base` evenly over the grid; one thread per CTA issues its slice.
__device__ __forceinline__ void l2_prefetch_slice(const void* base, unsigned long long total,
                                                  unsigned cta, unsigned n_cta) {
    if (base == nullptr || total == 0) return;
    unsigned long long per = ((total / n_cta) + 15ull) & ~15ull;
    if (per == 0) per = 16;
    unsigned long long off = per * cta;
    if (off >= total) return;
    unsigned long long len = total - off < per ? total - off : per;
    len &= ~15ull;
    const char* p = static_cast<const char*>(base) + off;
    while (len) {
        uint32_t piece = len > (1u << 20) ? (1u << 20) : uint32_t(len);
        l2_prefetch_bulk(p, piece);
        p += piece;
        len -= piece;
    }
}

// ---- optional timeline trace (debug): 8 words per launch -------------------------------
// [0] earliest CTA start, [1] earliest / [2] latest return from the dependency wait, [3] latest exit
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void trace_start(unsigned long long* t) {
    if (t && threadIdx.x == 0) atomicMin(t, global_ns());
}
__device__ __forceinline__ void trace_waited(unsigned long long* t) {
    if (t && threadIdx.x == 0) { const unsigned long long g = global_ns(); atomicMin(t + 1, g); atomicMax(t + 2, g); }
}
// words 4..7: latest time any CTA passed an interior mark
__device__ __forceinline__ void trace_mark(unsigned long long* t, int which) {
    if (t && threadIdx.x == 0) atomicMax(t + 4 + which, global_ns());
}
__device__ __forceinline__ void trace_end(unsigned long long* t) {
    if (t && threadIdx.x == 0) atomicMax(t + 3, global_ns());
}

// ---- reductions -----------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over the whole CTA; every thread gets the result. `scratch` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = lane < nwarp ? scratch[lane] : 0.f;
    t = warp_sum(t);
    __syncthreads();
    return t;
}

// 8 bf16 weights (one 16-byte load) times 8 f32 activations.
__device__ __forceinline__ float dot8(const uint4& w, const float4& xa, const float4& xb, float acc) {
    acc = fmaf(bf16_lo(w.x), xa.x, acc);
    acc = fmaf(bf16_hi(w.x), xa.y, acc);
    acc = fmaf(bf16_lo(w.y), xa.z, acc);
    acc = fmaf(bf16_hi(w.y), xa.w, acc);
    acc = fmaf(bf16_lo(w.z), xb.x, acc);
    acc = fmaf(bf16_hi(w.z), xb.y, acc);
    acc = fmaf(bf16_lo(w.w), xb.z, acc);
    acc = fmaf(bf16_hi(w.w), xb.w, acc);
    return acc;
}

// Activation pre-scale of the projections: a positive factor multiplies, a negative one divides by
// its magnitude (IEEE division: "hidden / 10" is not "hidden * 0.1" in the last bit).
__device__ __forceinline__ float apply_scale(float x, float s) {
    return s < 0.f ? __fdiv_rn(x, -s) : x * s;
}

__device__ __forceinline__ float silu_f32(float x) { return x / (1.f + __expf(-x)); }

// Gumbel-max sampling: argmax_i(logit_i / T + G_i) with G_i = -log(-log(u_i)) is a draw from softmax(logits / T),
// so sampling is the greedy pick over perturbed scores -- no normalisation pass.  u_i comes from a counter-based
// generator (the splitmix64 finaliser over seed, step and the GLOBAL vocabulary index), so a vocabulary-parallel
// head draws the same token as one GPU.  u = (k + 0.5) / 2^23 with k the top 23 bits: never 0 or 1.  The two
// logarithms run in double precision (one lane per row, so their cost does not matter): the fast single-precision
// log loses the tail u -> 1 where the winning variates live.
static __device__ __noinline__ float gumbel_variate(unsigned long long seed, int step, int index) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (unsigned long long)(unsigned(index) + 1u) +
                           0xD1B54A32D192ED03ull * (unsigned long long)(unsigned(step) + 1u);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    const double u = (double(unsigned(z >> 41)) + 0.5) * (1.0 / 8388608.0);
    return float(-log(-log(u)));
}

}  // namespace tfb
