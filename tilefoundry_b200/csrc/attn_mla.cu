// Multi-head latent attention decode (MiniCPM3): RoPE on the rotary slice, key/value assembly,
// cache append and split-KV softmax over a paged cache of ASSEMBLED keys [heads][nope+rope] and
// values [heads][v], one launch per layer.
//
// HBM/L2-bound on the cache: algorithmic bytes per launch = (ctx+1) * heads * (nope+rope+v) * 2.
// Grid = (heads, splits): one CTA owns one head and 128 positions (two pages).  Same latency plan as the GQA
// kernel: cached rows stream into shared memory with cp.async before griddepcontrol.wait; after the
// wait this token's query is rotated and scaled, its key/value row joins the shared tile, and the
// last CTA of a head to finish (atomic ticket, no spinning) merges the split partials.
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

constexpr int kMlaSplit = 128;                     // positions per CTA: two 64-row pages (fewer, fatter CTAs launch faster
                                                   // and leave half as many partials to merge)
constexpr int kMlaThreads = 256;

__device__ __forceinline__ void mla_cp16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 :: "r"(uint32_t(__cvta_generic_to_shared(smem_dst))), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void mla_cp_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <int NOPE, int R, int VD>
__global__ void __launch_bounds__(kMlaThreads) attn_mla_kernel(const MlaParams p) {
    constexpr int DK = NOPE + R;
    constexpr int KP = DK / 8, VP = VD / 8;            // 16-byte pieces per row
    constexpr int NWARP = kMlaThreads / 32;
    static_assert(DK % 32 == 0 && kMlaThreads % VD == 0 && DK <= kMlaThreads, "layout");

    __shared__ __align__(16) uint16_t kbuf[kMlaSplit][DK];
    __shared__ __align__(16) uint16_t vbuf[kMlaSplit][VD];
    __shared__ float qraw[DK], qs[DK], kraw[R];
    __shared__ float sc[kMlaSplit];
    __shared__ float pv_part[kMlaThreads / VD][VD];
    __shared__ float stat[2];
    __shared__ float mrg_w[64];
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.x, split = blockIdx.y, p0 = split * kMlaSplit;
    const int NH = p.heads;

    trace_start(p.trace);
    int pre_end = p0;
    {
        const int pos_early = *reinterpret_cast<const volatile int*>(p.pos);
        if (pos_early >= 0 && pos_early < p.max_ctx) {
            pre_end = max(p0, min(p0 + kMlaSplit, pos_early));
            for (int c = tid; c < (pre_end - p0) * (KP + VP); c += kMlaThreads) {
                const int r = c / (KP + VP), piece = c % (KP + VP);
                const int pp = p0 + r;
                const size_t row = size_t(p.block_table[pp / p.page_size]) * p.page_size + (pp % p.page_size);
                if (piece < KP) mla_cp16(&kbuf[r][piece * 8], p.k_pool + (row * NH + h) * DK + piece * 8);
                else mla_cp16(&vbuf[r][(piece - KP) * 8], p.v_pool + (row * NH + h) * VD + (piece - KP) * 8);
            }
        }
    }
    pdl_trigger();
    pdl_wait();
    trace_waited(p.trace);

    const int pos = *p.pos;
    const int total = pos + 1;
    const int n_active = (total + kMlaSplit - 1) / kMlaSplit;
    if (pos < 0 || pos >= p.max_ctx || split >= n_active) { mla_cp_wait(); return; }
    const bool owner = (split == n_active - 1);
    const int p1 = min(p0 + kMlaSplit, total);
    const int pend = min(p1, pos);
    for (int c = tid; c < max(pend - pre_end, 0) * (KP + VP); c += kMlaThreads) {
        const int r = (pre_end - p0) + c / (KP + VP), piece = c % (KP + VP);
        const int pp = p0 + r;
        const size_t row = size_t(p.block_table[pp / p.page_size]) * p.page_size + (pp % p.page_size);
        if (piece < KP) mla_cp16(&kbuf[r][piece * 8], p.k_pool + (row * NH + h) * DK + piece * 8);
        else mla_cp16(&vbuf[r][(piece - KP) * 8], p.v_pool + (row * NH + h) * VD + (piece - KP) * 8);
    }

    // ---- this token: query [nope | rope], shared rotary key slice --------------------------------
    const int rpos = p.rope_pos ? *p.rope_pos : pos;
    if (tid < DK) qraw[tid] = bf16_bits_to_f32(p.q_up[size_t(h) * DK + tid]);
    if (tid < R) kraw[tid] = bf16_bits_to_f32(p.k_rope[tid]);
    __syncthreads();
    float k_rot = 0.f;
    if (tid < DK) {
        float q = qraw[tid];
        if (tid >= NOPE) {
            const int i = tid - NOPE, half = R / 2;
            const float c = bf16_bits_to_f32(p.cos_table[size_t(rpos) * R + i]);
            const float s = bf16_bits_to_f32(p.sin_table[size_t(rpos) * R + i]);
            const float qp = (i < half) ? -qraw[NOPE + i + half] : qraw[NOPE + i - half];
            const float kp = (i < half) ? -kraw[i + half] : kraw[i - half];
            q = round_bf16(__fadd_rn(__fmul_rn(q, c), __fmul_rn(qp, s)));
            k_rot = round_bf16(__fadd_rn(__fmul_rn(kraw[i], c), __fmul_rn(kp, s)));
        }
        qs[tid] = round_bf16(q * p.scale);
    }
    if (owner) {                                  // assemble and append this token's key / value row
        const size_t row = size_t(p.block_table[pos / p.page_size]) * p.page_size + (pos % p.page_size);
        if (tid < DK) {
            const uint16_t kb = (tid < NOPE) ? p.kv_up[size_t(h) * (NOPE + VD) + tid] : f32_to_bf16_bits(k_rot);
            p.k_pool[(row * NH + h) * DK + tid] = kb;
            kbuf[pos - p0][tid] = kb;
            if (p.k_new_out) p.k_new_out[size_t(h) * DK + tid] = kb;
        }
        if (tid < VD) {
            const uint16_t vb = p.kv_up[size_t(h) * (NOPE + VD) + NOPE + tid];
            p.v_pool[(row * NH + h) * VD + tid] = vb;
            vbuf[pos - p0][tid] = vb;
            if (p.v_new_out) p.v_new_out[size_t(h) * VD + tid] = vb;
        }
    }
    mla_cp_wait();
    __syncthreads();
    trace_mark(p.trace, 0);

    // ---- scores: a warp takes four rows at a time (their reductions interleave), DK/32 elements per lane -------
    const int n = p1 - p0;
    {
        float q[DK / 32];
#pragma unroll
        for (int i = 0; i < DK / 32; ++i) q[i] = qs[lane + 32 * i];
        for (int r0 = warp * 4; r0 < n; r0 += NWARP * 4) {
            float sv[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                sv[t] = 0.f;
                if (r0 + t < n) {
#pragma unroll
                    for (int i = 0; i < DK / 32; ++i) sv[t] = fmaf(q[i], bf16_bits_to_f32(kbuf[r0 + t][lane + 32 * i]), sv[t]);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int t = 0; t < 4; ++t) sv[t] += __shfl_xor_sync(0xffffffffu, sv[t], o);
            if (lane < 4 && r0 + lane < n) sc[r0 + lane] = lane == 0 ? sv[0] : lane == 1 ? sv[1] : lane == 2 ? sv[2] : sv[3];
        }
    }
    __syncthreads();
    if (warp == 0) {
        float m = -INFINITY;
        for (int i = lane; i < n; i += 32) m = fmaxf(m, sc[i]);
        m = warp_max(m);
        float l = 0.f;
        for (int i = lane; i < n; i += 32) {
            const float e = __expf(sc[i] - m);
            sc[i] = e;
            l += e;
        }
        l = warp_sum(l);
        if (lane == 0) { stat[0] = m; stat[1] = l; }
    }
    __syncthreads();

    trace_mark(p.trace, 1);
    const int nsplit = p.nsplit;
    {
        // kMlaThreads / VD groups of threads share the rows: thread (d, grp) sums rows grp, grp + NG, ...
        constexpr int NG = kMlaThreads / VD;
        const int d = tid % VD, grp = tid / VD;
        float o = 0.f;
        for (int r = grp; r < n; r += NG) o = fmaf(sc[r], bf16_bits_to_f32(vbuf[r][d]), o);
        pv_part[grp][d] = o;
    }
    __syncthreads();
    if (tid < VD) {
        float o = 0.f;
#pragma unroll
        for (int g2 = 0; g2 < kMlaThreads / VD; ++g2) o += pv_part[g2][tid];          // fixed order
        if (n_active == 1) p.out[size_t(h) * VD + tid] = f32_to_bf16_bits(o / stat[1]);
        else p.part_o[(size_t(h) * nsplit + split) * VD + tid] = o;
    }
    if (n_active == 1) { trace_end(p.trace); return; }
    if (tid == 0) {
        p.part_ml[(size_t(h) * nsplit + split) * 2] = stat[0];
        p.part_ml[(size_t(h) * nsplit + split) * 2 + 1] = stat[1];
    }
    trace_mark(p.trace, 2);
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&p.counters[h], 1u) == unsigned(n_active - 1));
    __syncthreads();
    trace_mark(p.trace, 3);
    if (!s_last) { trace_end(p.trace); return; }
    __threadfence();

    float num = 0.f, den = 0.f, run_m = -INFINITY;
    for (int s0 = 0; s0 < n_active; s0 += 64) {
        const int ns = min(64, n_active - s0);
        const float* ml = p.part_ml + (size_t(h) * nsplit + s0) * 2;
        __syncthreads();
        if (warp == 0) {
            const float m0 = lane < ns ? __ldcg(ml + 2 * lane) : -INFINITY;
            const float m1 = lane + 32 < ns ? __ldcg(ml + 2 * (lane + 32)) : -INFINITY;
            const float M = warp_max(fmaxf(m0, m1));
            if (lane < ns) mrg_w[lane] = __expf(m0 - M);
            if (lane + 32 < ns) mrg_w[lane + 32] = __expf(m1 - M);
            if (lane == 0) stat[0] = M;
        }
        __syncthreads();
        if (tid < VD) {
            const float* po = p.part_o + (size_t(h) * nsplit + s0) * VD + tid;
            float a = 0.f, b = 0.f;
            int s = 0;
            for (; s + 4 <= ns; s += 4) {                      // independent loads, four in flight
                const float v0 = __ldcg(po + size_t(s) * VD), v1 = __ldcg(po + size_t(s + 1) * VD);
                const float v2 = __ldcg(po + size_t(s + 2) * VD), v3 = __ldcg(po + size_t(s + 3) * VD);
                const float l0 = __ldcg(ml + 2 * s + 1), l1 = __ldcg(ml + 2 * s + 3);
                const float l2 = __ldcg(ml + 2 * s + 5), l3 = __ldcg(ml + 2 * s + 7);
                a = fmaf(mrg_w[s], v0, a); a = fmaf(mrg_w[s + 1], v1, a); a = fmaf(mrg_w[s + 2], v2, a); a = fmaf(mrg_w[s + 3], v3, a);
                b = fmaf(mrg_w[s], l0, b); b = fmaf(mrg_w[s + 1], l1, b); b = fmaf(mrg_w[s + 2], l2, b); b = fmaf(mrg_w[s + 3], l3, b);
            }
            for (; s < ns; ++s) {
                a = fmaf(mrg_w[s], __ldcg(po + size_t(s) * VD), a);
                b = fmaf(mrg_w[s], __ldcg(ml + 2 * s + 1), b);
            }
            const float M = stat[0], newm = fmaxf(run_m, M);
            const float c_old = run_m == -INFINITY ? 0.f : __expf(run_m - newm), c_new = __expf(M - newm);
            num = num * c_old + a * c_new;
            den = den * c_old + b * c_new;
            run_m = newm;
        }
    }
    if (tid < VD) p.out[size_t(h) * VD + tid] = f32_to_bf16_bits(num / den);
    if (tid == 0) p.counters[h] = 0;
    trace_end(p.trace);
}

int mla_splits(int max_ctx) { return (max_ctx + kMlaSplit - 1) / kMlaSplit; }

cudaError_t attn_mla_dispatch(const MlaParams& p, cudaStream_t stream, bool pdl) {
    const dim3 grid(p.heads, p.nsplit), block(kMlaThreads);
    if (p.nope == 64 && p.rope == 32 && p.vd == 64)
        return launch_kernel(attn_mla_kernel<64, 32, 64>, grid, block, 0, stream, pdl, p);
    return cudaErrorInvalidValue;
}

}  // namespace tfb
