// Mixture-of-experts block for a batch of tokens: every expert that at least one token selected is read ONCE, and its
// rows meet all of its tokens on the tensor cores.
//
//   inner[t, s, :] = bf16( silu(bf16(W_gate[e] . x_t)) * bf16(W_up[e] . x_t) )        e = indices[t, s]  (x_t rounded to bf16)
//   y[t, s, :]     = bf16( W_down[e] . inner[t, s, :] )
//   out[t, :]      = sum_s weights[t, s] * y[t, s, :]  +  y[t, K, :] * sigmoid(shared_gate[t])      (slot K: the shared expert)
//
// the rounding points of Qwen3_5SparseMoeBlock as authored (every matmul takes bf16 operands and returns bf16).
//
// A batch of 64 tokens with 8 of 256 experts each touches ~222 experts with two or three tokens apiece: a GEMM per
// expert has no M to speak of and a GEMV per (token, expert) reads every expert several times.  Here a CTA owns 16 rows
// of one expert and up to eight of its tokens at a time: K is folded into the MMA's N as in the one-launch Qwen3 step
// (256 contiguous bytes of a weight row are an 8 x 16 K-major block; the stride between 8-row groups is the row pitch;
// the B operand is the same fold of each token's activation chunk, one 8-row group per token, so N = 8 x tokens), one
// tcgen05.mma (M 128, N 64, K 16) per 128 elements of K whatever the number of tokens, accumulating in tensor memory;
// token b's dot product with row g is the diagonal sum D[8g + r][8b + r].  HBM-bound: the touched experts' bytes once.
#include "common.cuh"
#include "route.cuh"
#include "kernels.h"
#include "launch.h"

#include <algorithm>

namespace tfb {
namespace {

constexpr int kGRows = 16;                       // weight rows of a CTA (M = 128: eight tensor-memory lanes per row)
constexpr int kGTok = 8;                         // tokens per pass (N = 64)
constexpr int kGThreads = 128;
constexpr int kGCols = 64;                       // tensor-memory columns of the accumulator
constexpr unsigned kSpinLimit = 1u << 22;        // bound of every barrier wait (each try may suspend for a while)

__device__ __forceinline__ uint32_t s_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mb_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(s_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mb_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(s_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mb_try(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(s_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// false: the wait gave up (the caller records it; the results of the CTA are void)
__device__ __forceinline__ bool mb_wait(unsigned long long* bar, unsigned parity) {
    for (unsigned i = 0; i < kSpinLimit; ++i)
        if (mb_try(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(s_u32(dst)), "l"(src), "r"(bytes), "r"(s_u32(bar)) : "memory");
}
__device__ __forceinline__ uint64_t folded_desc(uint32_t smem_addr, uint32_t group_pitch) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr & 0x3FFFF) >> 4);               // start address, 16-byte units
    d |= uint64_t(128 >> 4) << 16;                            // byte offset between core matrices along K
    d |= uint64_t(group_pitch >> 4) << 32;                    // byte offset between 8-row groups
    d |= uint64_t(1) << 46;                                   // descriptor version of this architecture
    return d;                                                  // (layout type 0: no swizzle)
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_arrive(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(s_u32(bar)) : "memory");
}
// D f32, A and B bf16, both K-major, N = 64, M = 128
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(kGTok * 8 >> 3) << 17) | (uint32_t(128 >> 4) << 24);

// one expert list entry: token in the high bits, slot (0 .. K) in the low eight
__device__ __forceinline__ int entry_token(int e) { return e >> 8; }
__device__ __forceinline__ int entry_slot(int e) { return e & 255; }

// ---- routing of a batch: router logits, top-k, the shared expert's gate logit -- one CTA per token ----------------
// logits[t][e] = bf16(W_router[e] . bf16 x_t) (the authored matmul: bf16 in, bf16 out), row `experts` = the shared
// expert's scale row; then the selection of route_select (the rule of the one-token router kernel).
template <int MAXE>
__global__ void __launch_bounds__(256) moe_batch_route_kernel(const MoeRouteParams p) {
    extern __shared__ __align__(16) float xr[];                // x_t rounded to bf16, as f32
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int H = p.hidden, E = p.experts;
    for (int i = threadIdx.x; i < H; i += blockDim.x) xr[i] = round_bf16(p.x[size_t(t) * H + i]);
    __syncthreads();
    float* logits = p.logits + size_t(t) * (E + 1);
    const int rows = E + (p.w_shared_scale ? 1 : 0);
    // a warp takes four rows at a time (rows r, r + 8, r + 16, r + 24): four independent chains of loads in flight
    for (int r0 = warp; r0 < rows; r0 += 32) {
        const uint4* w[4];
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int r = min(r0 + 8 * q, rows - 1);            // (a row past the end repeats the last one; not stored)
            w[q] = reinterpret_cast<const uint4*>(r < E ? p.w_router + size_t(r) * H : p.w_shared_scale);
        }
#pragma unroll 8
        for (int c = lane; c < (H >> 3); c += 32) {            // (unrolled: the loads of eight steps are requested together)
            uint4 wv[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) wv[q] = __ldg(w[q] + c);
            const float4 xa = *reinterpret_cast<const float4*>(xr + c * 8), xb = *reinterpret_cast<const float4*>(xr + c * 8 + 4);
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[q] = dot8(wv[q], xa, xb, acc[q]);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float sum = warp_sum(acc[q]);
            if (lane == 0 && r0 + 8 * q < rows) logits[r0 + 8 * q] = round_bf16(sum);
        }
    }
    __syncthreads();                                           // (the logits were written by this CTA: visible to it in L2)
    if (warp == 0) {
        float w;
        int e;
        route_select<MAXE>(logits, nullptr, E, p.top_k, p.mode, lane, w, e);
        if (lane < p.top_k) {
            p.indices[size_t(t) * p.top_k + lane] = e;
            p.weights[size_t(t) * p.top_k + lane] = w;
        }
        if (lane == 0 && p.shared_gate) p.shared_gate[t] = p.w_shared_scale ? __ldcg(logits + E) : 0.f;
    }
}

// ---- tokens f32 -> bf16 rows, and the experts' token lists ------------------------------------------------------
__global__ void __launch_bounds__(1024) moe_batch_prepare_kernel(const MoeBatchParams p) {
    pdl_trigger();
    pdl_wait();
    if (blockIdx.x > 0) {                                      // CTAs 1..: the rounding of the activations
        const size_t n = size_t(p.tokens) * p.hidden;
        for (size_t i = size_t(blockIdx.x - 1) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x - 1) * blockDim.x)
            p.x_bf16[i] = f32_to_bf16_bits(p.x[i]);
        return;
    }
    // CTA 0: lists in token order (deterministic), one WARP per expert: the routing table passes through shared memory in
    // pieces, a warp compares 32 entries at a time and the matching lanes write at their rank among the matches.  (One
    // thread per expert reading the table from global memory took 70 us, from shared memory 30.)
    __shared__ short ids[1024];
    __shared__ int s_cnt[513];
    const int T = p.tokens, K = p.top_k, E = p.experts;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int e = threadIdx.x; e <= E; e += blockDim.x) s_cnt[e] = 0;
    for (int a0 = 0; a0 < T * K; a0 += 1024) {
        const int na = min(1024, T * K - a0);
        __syncthreads();
        for (int i = threadIdx.x; i < na; i += blockDim.x) ids[i] = short(p.indices[a0 + i]);
        __syncthreads();
        for (int e = warp; e < E; e += nwarps) {
            int* lst = p.lists + size_t(e) * T;
            int n = s_cnt[e];                                  // (this warp alone touches expert e's count)
            for (int i0 = 0; i0 < na; i0 += 32) {
                const bool hit = i0 + lane < na && ids[i0 + lane] == short(e);
                const unsigned m = __ballot_sync(0xffffffffu, hit);
                if (hit) { const int a = a0 + i0 + lane; lst[n + __popc(m & ((1u << lane) - 1u))] = ((a / K) << 8) | (a % K); }
                n += __popc(m);
            }
            __syncwarp();
            if (lane == 0) s_cnt[e] = n;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) p.counts[e] = s_cnt[e];
    // the shared expert takes every token, in slot K
    const int n_shared = p.w_shared_gate ? T : 0;
    for (int t = threadIdx.x; t < n_shared; t += blockDim.x) p.lists[size_t(E) * T + t] = (t << 8) | K;
    if (threadIdx.x == 0) { p.counts[E] = n_shared; s_cnt[E] = n_shared; }
    __syncthreads();
    if (threadIdx.x == 0) {
        // the experts that have tokens: the shared expert first (every token is its: its items take the most passes, and
        // items are dealt round-robin, so the longest go out first), then the routed ones in index order
        int* active = p.counts + E + 2;
        int na = 0;
        if (s_cnt[E] > 0) active[na++] = E;
        for (int e = 0; e < E; ++e)
            if (s_cnt[e] > 0) active[na++] = e;
        p.counts[E + 1] = na;
    }
}

// ---- the grouped products -----------------------------------------------------------------------------------------
// STAGE 0: gate/up + SwiGLU -- inter / 8 row groups per expert, tile rows 2i / 2i + 1 = gate / up row r0 + i, k = hidden,
//          activations x_bf16[token], result inner[token, slot, r0 + i].
// Persistent: a CTA allocates its accumulator once and takes every gridDim.x-th (expert with tokens, row group).
// STAGE 1: down -- hidden / 16 row groups per expert, tile rows = rows j0 .. j0 + 15 of W_down[e], k = inter,
//          activations inner[token, slot], result y[token, slot, j0 + g].
template <int STAGE>
__global__ void __launch_bounds__(kGThreads) moe_grouped_kernel(const MoeBatchParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bar_w, bar_x, bar_mma;
    __shared__ uint32_t tmem_base;
    __shared__ int s_fail;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int E = p.experts, K = p.top_k, T = p.tokens;
    const int k = STAGE == 0 ? p.hidden : p.inter;              // reduction length
    const int row_bytes = k * 2;
    const int RG = STAGE == 0 ? p.inter / (kGRows / 2) : p.hidden / kGRows;      // row groups of an expert
    pdl_trigger();
    pdl_wait();
    const int n_items = p.counts[E + 1] * RG;                  // (experts with tokens) x (row groups): a CTA takes every
    if (int(blockIdx.x) >= n_items) return;                    //  gridDim.x-th item (uniform over the CTA, nothing allocated yet)
    const int* active = p.counts + E + 2;
    unsigned char* tile = smem;                                // [16 rows][k] bf16
    unsigned char* xs = smem + kGRows * row_bytes;             // [8 tokens][k] bf16

    if (tid == 0) {
        mb_init(&bar_w, 1); mb_init(&bar_x, 1); mb_init(&bar_mma, 1);
        s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(s_u32(&tmem_base)), "n"(kGCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base;
    const int trow = warp * 4 + (lane >> 3);                    // the tile row of this lane's team of eight
    unsigned wpar = 0, xpar = 0, mpar = 0;

    // the weight rows of an item: lane r of warp 0 copies tile row r
    auto issue_tile = [&](int item) {
        if (warp != 0) return;
        const int e = active[item / RG], rg = item % RG;
        if (lane == 0) mb_expect_tx(&bar_w, unsigned(kGRows) * row_bytes);
        __syncwarp();
        if (lane < kGRows) {
            const uint16_t* src;
            if (STAGE == 0) {
                const int r = rg * (kGRows / 2) + (lane >> 1);
                const uint16_t* base = e < E ? ((lane & 1) ? p.w_up : p.w_gate) + size_t(e) * p.inter * p.hidden
                                             : ((lane & 1) ? p.w_shared_up : p.w_shared_gate);
                src = base + size_t(r) * p.hidden;
            } else {
                const int j = rg * kGRows + lane;
                src = (e < E ? p.w_down + size_t(e) * p.hidden * p.inter : p.w_shared_down) + size_t(j) * p.inter;
            }
            bulk_load(tile + lane * row_bytes, src, row_bytes, &bar_w);
        }
    };
    // the activations of one pass over an item's tokens: lane b of warp 1 copies token b's row
    auto issue_x = [&](int item, int p0) {
        if (warp != 1) return;
        const int e = active[item / RG];
        const int nb = min(kGTok, p.counts[e] - p0);
        const int* lst = p.lists + size_t(e) * T;
        if (lane == 0) mb_expect_tx(&bar_x, unsigned(nb) * row_bytes);
        __syncwarp();
        if (lane < nb) {
            const int ent = lst[p0 + lane];
            const uint16_t* src = STAGE == 0 ? p.x_bf16 + size_t(entry_token(ent)) * p.hidden
                                             : p.inner + (size_t(entry_token(ent)) * (K + 1) + entry_slot(ent)) * p.inter;
            bulk_load(xs + lane * row_bytes, src, row_bytes, &bar_x);
        }
    };
    issue_tile(blockIdx.x);
    issue_x(blockIdx.x, 0);
    for (int item = blockIdx.x; item < n_items && !s_fail; item += gridDim.x) {
        const int e = active[item / RG], rg = item % RG;
        const int n = p.counts[e];
        const int* lst = p.lists + size_t(e) * T;
        for (int p0 = 0; p0 < n; p0 += kGTok) {
            const int nb = min(kGTok, n - p0);
            if (p0 > 0) issue_x(item, p0);                      // (the first pass's were asked for while the last item finished)
            if (tid == 0) {
                // the MMAs of the pass: one per 128 elements of K, all tokens at once
                const bool ok = (p0 > 0 || mb_wait(&bar_w, wpar)) && mb_wait(&bar_x, xpar);
                if (ok) {
                    const uint64_t da = folded_desc(s_u32(tile), row_bytes), db = folded_desc(s_u32(xs), row_bytes);
                    for (int t = 0; t < k / 128; ++t)
                        umma_f16(tmem, da + uint64_t((t * 256) >> 4), db + uint64_t((t * 256) >> 4), kIdesc, t ? 1u : 0u);
                } else {
                    s_fail = 1;
                }
                umma_arrive(&bar_mma);
            }
            xpar ^= 1u;
            if (!mb_wait(&bar_mma, mpar)) s_fail = 1;          // everyone waits for the accumulator
            mpar ^= 1u;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            __syncthreads();
            if (s_fail) break;                                  // (uniform after the barrier)
            // The rows and the activations have been read: the next item's can land while this pass's results are
            // taken out of tensor memory.
            if (p0 + kGTok >= n && item + int(gridDim.x) < n_items) {
                issue_tile(item + gridDim.x);
                issue_x(item + gridDim.x, 0);
            }

            // epilogue: lane 8g + r of the quadrant wants, for token b, column 8b + r; a team of eight lanes sums the
            // diagonal.  Four tokens (32 columns) at a time: 64 values in registers cost the down stage three of its
            // eight resident CTAs.
            const bool b4 = lane & 4, b2 = lane & 2, b1 = lane & 1;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                if (half * 4 >= nb) break;                      // (uniform: no token in the second half)
                uint32_t v[32];
                const uint32_t taddr = tmem + (uint32_t(warp * 32) << 16) + uint32_t(half * 32);
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                             "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                               "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                             : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int bb = 0; bb < 4; ++bb) {
                    const int b = half * 4 + bb;
                    const uint32_t t0 = b4 ? v[8 * bb + 4] : v[8 * bb], t1 = b4 ? v[8 * bb + 5] : v[8 * bb + 1];
                    const uint32_t t2 = b4 ? v[8 * bb + 6] : v[8 * bb + 2], t3 = b4 ? v[8 * bb + 7] : v[8 * bb + 3];
                    const uint32_t q0 = b2 ? t2 : t0, q1 = b2 ? t3 : t1;
                    float d = __uint_as_float(b1 ? q1 : q0);
                    d += __shfl_xor_sync(0xffffffffu, d, 1);
                    d += __shfl_xor_sync(0xffffffffu, d, 2);
                    d += __shfl_xor_sync(0xffffffffu, d, 4);
                    if (STAGE == 0) {
                        const float up = round_bf16(__shfl_xor_sync(0xffffffffu, d, 8));     // (the team next door holds the up row)
                        if (b < nb && (lane & 15) == 0) {
                            const int ent = lst[p0 + b];
                            const int col = rg * (kGRows / 2) + (trow >> 1);
                            p.inner[(size_t(entry_token(ent)) * (K + 1) + entry_slot(ent)) * p.inter + col] =
                                f32_to_bf16_bits(silu_f32(round_bf16(d)) * up);
                        }
                    } else {
                        if (b < nb && (lane & 7) == 0) {
                            const int ent = lst[p0 + b];
                            p.y[(size_t(entry_token(ent)) * (K + 1) + entry_slot(ent)) * p.hidden + rg * kGRows + trow] = f32_to_bf16_bits(d);
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();                                    // (the next pass overwrites the activations and the accumulator)
        }
        wpar ^= 1u;
    }
    if (s_fail && tid == 0) {
        atomicOr(p.status, 0x1000u);
        umma_arrive(&bar_mma);                                  // MMAs may still be in flight: they end by themselves, and this
        mb_wait(&bar_mma, mpar);                                //  fresh completion is waited for (bounded) before the release;
        mb_wait(&bar_w, wpar);                                  //  so are copies that were asked for ahead (bounded: if none
        mb_wait(&bar_x, xpar);                                  //  is in flight these give up after their limit)
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "n"(kGCols) : "memory");
    }
}

// ---- out[t] = residual[t] + sum of the routed slots by weight + shared slot by its gate --------------------------
__global__ void __launch_bounds__(256) moe_batch_finalize_kernel(const MoeBatchParams p) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y, K = p.top_k;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= p.hidden) return;
    const uint16_t* y = p.y + size_t(t) * (K + 1) * p.hidden + j;
    float routed = 0.f;
    for (int s = 0; s < K; ++s) routed = fmaf(bf16_bits_to_f32(y[size_t(s) * p.hidden]), p.weights[size_t(t) * K + s], routed);
    float out = routed;
    if (p.w_shared_gate) {
        float sh = bf16_bits_to_f32(y[size_t(K) * p.hidden]);
        if (p.shared_gate) sh *= 1.f / (1.f + expf(-p.shared_gate[t]));
        out += sh;
    }
    if (p.residual) out += p.residual[size_t(t) * p.hidden + j];
    p.out[size_t(t) * p.hidden + j] = out;
}

}  // namespace

cudaError_t moe_batch_route_launch(const MoeRouteParams& p, cudaStream_t stream, bool pdl) {
    if (p.tokens < 1 || p.hidden < 256 || p.hidden % 256 != 0 || p.hidden > 8192 || p.experts < 1 || p.experts > 256 ||
        p.top_k < 1 || p.top_k > 32 || p.top_k > p.experts)
        return cudaErrorInvalidValue;
    const size_t smem = size_t(p.hidden) * 4;
    if (p.experts <= 128) return launch_kernel(moe_batch_route_kernel<128>, dim3(p.tokens), dim3(256), smem, stream, pdl, p);
    return launch_kernel(moe_batch_route_kernel<256>, dim3(p.tokens), dim3(256), smem, stream, pdl, p);
}

size_t moe_grouped_smem(int k) { return size_t(kGRows + kGTok) * k * 2; }

bool moe_batch_supported(const MoeBatchParams& p) {
    auto ok_k = [](int k) { return k >= 128 && k % 128 == 0 && moe_grouped_smem(k) <= 200 * 1024; };
    return p.tokens >= 1 && p.tokens <= 4096 && p.top_k >= 1 && p.top_k < 255 && p.experts >= 1 && p.experts <= 512 && ok_k(p.hidden) &&
           ok_k(p.inter) && p.inter % (kGRows / 2) == 0 && p.hidden % kGRows == 0 &&
           (!p.w_shared_gate || (p.w_shared_up && p.w_shared_down));
}

cudaError_t moe_batch_launch(const MoeBatchParams& p, cudaStream_t stream, bool pdl) {
    if (!moe_batch_supported(p)) return cudaErrorInvalidValue;
    static PerDeviceOnce once;
    static int s_regs[2] = {96, 96};                           // registers per thread of the two stages (the same on every device)
    if (once.first()) {
        cudaError_t e = cudaFuncSetAttribute(moe_grouped_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(moe_grouped_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncAttributes fa;
        if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, moe_grouped_kernel<0>);
        if (e == cudaSuccess) s_regs[0] = fa.numRegs;
        if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, moe_grouped_kernel<1>);
        if (e == cudaSuccess) s_regs[1] = fa.numRegs;
        if (e != cudaSuccess) return e;
    }
    cudaError_t e = launch_kernel(moe_batch_prepare_kernel, dim3(1 + 32), dim3(1024), 0, stream, pdl, p);
    if (e != cudaSuccess) return e;
    // persistent grids: as many CTAs as stay resident (two per multiprocessor by the 96 KB of the gate/up stage, eight by
    // the 64 tensor-memory columns of the down stage), each taking every gridDim.x-th (expert, row group)
    const int sms = sm_count();
    const int max0 = p.inter / (kGRows / 2) * (p.experts + 1), max1 = p.hidden / kGRows * (p.experts + 1);
    // CTAs that stay resident on a multiprocessor: by registers, shared memory and the 512 columns of tensor memory
    auto resident = [](int regs, size_t smem) {
        const int by_regs = 65536 / (((regs + 7) / 8 * 8) * kGThreads);
        const int by_smem = int((227 * 1024) / (smem + 1024));
        return std::max(1, std::min({by_regs, by_smem, 512 / kGCols}));
    };
    const int per0 = resident(s_regs[0], moe_grouped_smem(p.hidden)), per1 = resident(s_regs[1], moe_grouped_smem(p.inter));
    e = launch_kernel(moe_grouped_kernel<0>, dim3(std::min(max0, sms * per0)), dim3(kGThreads), moe_grouped_smem(p.hidden), stream, pdl, p);
    if (e != cudaSuccess) return e;
    e = launch_kernel(moe_grouped_kernel<1>, dim3(std::min(max1, sms * per1)), dim3(kGThreads), moe_grouped_smem(p.inter), stream, pdl, p);
    if (e != cudaSuccess) return e;
    return launch_kernel(moe_batch_finalize_kernel, dim3((p.hidden + 255) / 256, p.tokens), dim3(256), 0, stream, pdl, p);
}

}  // namespace tfb
