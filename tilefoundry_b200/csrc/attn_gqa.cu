// GQA decode attention over a paged bf16 KV cache, one launch per layer:
// per-head q/k RMSNorm -> RoPE -> KV append -> split-KV softmax -> merge.
//
// HBM/L2-bound on the cache: algorithmic bytes per launch = (ctx+1) * hkv * d * 2 (K and V)
// * 2 bytes.  Grid = (hkv, splits): one CTA owns one KV head and kSplitLen (= one
// page of) consecutive positions, and serves all G = hq/hkv query heads that share
// the KV head, so each cache row is read once.
//
// Latency is what matters at batch 1, so the kernel is built around one round trip:
//  * cached rows are immutable, so the CTA starts copying its K and V rows into
//    shared memory (16-byte cp.async, all in flight at once) BEFORE
//    griddepcontrol.wait, while the q|k|v projection before it is still running.
//    The position word may still be the previous step's at that moment; it can only
//    be smaller, and the rows it leaves out are fetched after the wait.
//  * after the wait: this token's q/k/v are normalised, rotated, and the new K/V row
//    is dropped into the same shared tile, so the score and PV loops have no special
//    case.
//  * PV gives each thread whole output elements (no cross-thread reduction).
//  * partial (max, sum, weighted V) go to scratch; the last CTA of a KV head to
//    finish (an atomic ticket, no spinning) merges them with all loads independent.
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

constexpr int kSplitLen = 64;
constexpr int kAttnThreads = 256;
constexpr int kMergeBatch = 16;             // split partials one merging thread requests at once

int attn_splits(int max_ctx) { return (max_ctx + kSplitLen - 1) / kSplitLen; }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 :: "r"(uint32_t(__cvta_generic_to_shared(smem_dst))), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <int D, int G>
__global__ void __launch_bounds__(kAttnThreads) attn_gqa_kernel(const AttnParams p) {
    constexpr int LPP = D / 8;                 // lanes that share one position's row (16 B each)
    constexpr int NSG = kAttnThreads / LPP;    // position sub-groups in the CTA
    constexpr int NWARP = kAttnThreads / 32;
    constexpr int NV = G + 1;                  // vectors normalised + rotated: G queries and the key
    constexpr int OUT_PER_THREAD = (G * D + kAttnThreads - 1) / kAttnThreads;

    __shared__ __align__(16) uint16_t kbuf[kSplitLen][D];
    __shared__ __align__(16) uint16_t vbuf[kSplitLen][D];
    __shared__ __align__(16) float vec[NV + 1][D];       // q_0..q_{G-1} (scaled), k_new, v_new
    __shared__ float gain[2][D];                         // q and k norm gains
    __shared__ float rot[2][D];                          // cos / sin row of this position
    __shared__ float sc[G][kSplitLen];
    __shared__ float stat_m[G], stat_l[G];
    __shared__ float mrg_w[G][64];                       // merge weights per split (64 splits per pass)
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.x, split = blockIdx.y;
    const int p0 = split * kSplitLen;
    trace_start(p.trace);
    // ---- before the dependency wait: start fetching the cached rows ---------------------
    // Rows below the position word are final whatever step wrote that word last.
    int pre_end = p0, rot_pos = -1;
    {
        const int pos_early = *reinterpret_cast<const volatile int*>(p.pos);
        if (pos_early >= 0 && pos_early < p.max_ctx) {
            pre_end = max(p0, min(p0 + kSplitLen, pos_early));
            const int rows = pre_end - p0;
            for (int c = tid; c < rows * LPP; c += kAttnThreads) {
                const int r = c / LPP, piece = c % LPP;
                const int pp = p0 + r;
                const int page = p.block_table[pp / p.page_size];
                const size_t off = ((size_t(page) * p.page_size + (pp % p.page_size)) * p.hkv + g) * D + piece * 8;
                cp_async16(&kbuf[r][piece * 8], p.k_pool + off);
                cp_async16(&vbuf[r][piece * 8], p.v_pool + off);
            }
        }
        if (tid == 0)
            l2_prefetch_slice(p.prefetch, p.prefetch_bytes, blockIdx.y * gridDim.x + blockIdx.x,
                              gridDim.x * gridDim.y);
        // weights and (most likely) the rotary row do not depend on the previous kernel either
        if (tid < D) {
            gain[0][tid] = p.norm_mode ? bf16_bits_to_f32(p.gamma_q[tid]) : 1.f;
            gain[1][tid] = p.norm_mode ? bf16_bits_to_f32(p.gamma_k[tid]) : 1.f;
        }
        rot_pos = (p.rope_pos == nullptr && pos_early >= 0 && pos_early < p.max_ctx) ? pos_early : -1;
        if (rot_pos >= 0 && tid < p.rotary_dim) {
            rot[0][tid] = bf16_bits_to_f32(p.cos_table[size_t(rot_pos) * p.rotary_dim + tid]);
            rot[1][tid] = bf16_bits_to_f32(p.sin_table[size_t(rot_pos) * p.rotary_dim + tid]);
        }
    }
    pdl_trigger();
    pdl_wait();
    trace_waited(p.trace);

    // this token's q/k/v do not depend on the position word: request them before reading it
    uint16_t xraw[2][D / 32];                    // up to two vectors per warp (NV + 1 <= 2 * NWARP)
    int vis[2] = {warp, warp + NWARP};
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2) {
        const int vi = vis[s2];
        if (vi < NV + 1) {
            const uint16_t* src;
            if (vi < G) src = p.qkv + size_t(g * G + vi) * D;
            else if (vi == G) src = p.qkv + size_t(p.hq) * D + size_t(g) * D;
            else src = p.qkv + size_t(p.hq + p.hkv) * D + size_t(g) * D;
#pragma unroll
            for (int i = 0; i < D / 32; ++i) xraw[s2][i] = src[lane + 32 * i];
        }
    }

    const int pos = *p.pos;
    const int total = pos + 1;
    const int n_active = (total + kSplitLen - 1) / kSplitLen;
    if (pos < 0 || pos >= p.max_ctx || split >= n_active) {
        cp_async_wait_all();                   // nothing may still be landing in smem when the CTA exits
        return;
    }
    const bool owner = (split == n_active - 1);
    const int p1 = min(p0 + kSplitLen, total);
    const int pend = min(p1, pos);             // cached rows of this split are [p0, pend)
    for (int c = tid; c < max(pend - pre_end, 0) * LPP; c += kAttnThreads) {   // rows the early look missed
        const int r = (pre_end - p0) + c / LPP, piece = c % LPP;
        const int pp = p0 + r;
        const int page = p.block_table[pp / p.page_size];
        const size_t off = ((size_t(page) * p.page_size + (pp % p.page_size)) * p.hkv + g) * D + piece * 8;
        cp_async16(&kbuf[r][piece * 8], p.k_pool + off);
        cp_async16(&vbuf[r][piece * 8], p.v_pool + off);
    }

    // ---- this token's q (G heads), k, v for KV head g -------------------------------------
    // One warp per vector, everything in registers: lane l holds elements l, l+32, ...; the
    // rotate-half partner of element i is i +- rotary_dim/2, a multiple of 32 away, so it sits in
    // the same lane and norm -> RoPE -> scale needs no shared-memory round trip.
    const int rd = p.rotary_dim, half = rd >> 1;
    const int rpos = p.rope_pos ? *p.rope_pos : pos;
    if (rpos != rot_pos && tid < rd) {            // the early look was a step behind (or not allowed)
        rot[0][tid] = bf16_bits_to_f32(p.cos_table[size_t(rpos) * rd + tid]);
        rot[1][tid] = bf16_bits_to_f32(p.sin_table[size_t(rpos) * rd + tid]);
    }
    float xv[2][D / 32];
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
        for (int i = 0; i < D / 32; ++i) xv[s2][i] = (vis[s2] < NV + 1) ? bf16_bits_to_f32(xraw[s2][i]) : 0.f;
    __syncthreads();                             // rot[] / gain[] visible
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2) {
        const int vi = vis[s2];
        if (vi >= NV + 1) continue;
        float* x = xv[s2];
        if (vi == G + 1) {                       // v: no norm, no rotation
#pragma unroll
            for (int i = 0; i < D / 32; ++i) vec[vi][lane + 32 * i] = x[i];
            continue;
        }
        if (p.norm_mode != 0) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < D / 32; ++i) ss = fmaf(x[i], x[i], ss);
            ss = warp_sum(ss);
            const float rstd = rsqrtf(ss / float(D) + p.eps);
            const float* gm = gain[vi < G ? 0 : 1];
#pragma unroll
            for (int i = 0; i < D / 32; ++i) x[i] = round_bf16(round_bf16(x[i] * rstd) * gm[lane + 32 * i]);
        }
        float r[D / 32];
#pragma unroll
        for (int i = 0; i < D / 32; ++i) {
            const int e = lane + 32 * i;
            r[i] = x[i];
            if (e < rd) {
                // partner index e +- half; half is a multiple of 32, so it is register i +- half/32
                const int pi = (e < half) ? i + half / 32 : i - half / 32;
                float partner = 0.f;
#pragma unroll
                for (int k2 = 0; k2 < D / 32; ++k2) if (k2 == pi) partner = x[k2];
                if (e < half) partner = -partner;
                r[i] = round_bf16(__fadd_rn(__fmul_rn(x[i], rot[0][e]), __fmul_rn(partner, rot[1][e])));
            }
            if (vi < G) r[i] = round_bf16(r[i] * p.scale);
            vec[vi][e] = r[i];
        }
    }
    __syncthreads();
    trace_mark(p.trace, 0);

    if (owner) {                                // append this token's entry: cache, outputs, shared tile
        const int page = p.block_table[pos / p.page_size];
        const size_t base = ((size_t(page) * p.page_size + (pos % p.page_size)) * p.hkv + g) * D;
        for (int i = tid; i < D; i += kAttnThreads) {
            const uint16_t kb = f32_to_bf16_bits(vec[G][i]), vb = f32_to_bf16_bits(vec[G + 1][i]);
            p.k_pool[base + i] = kb;
            p.v_pool[base + i] = vb;
            kbuf[pos - p0][i] = kb;
            vbuf[pos - p0][i] = vb;
            if (p.k_new_out) p.k_new_out[size_t(g) * D + i] = kb;
            if (p.v_new_out) p.v_new_out[size_t(g) * D + i] = vb;
        }
    }
    cp_async_wait_all();
    __syncthreads();
    trace_mark(p.trace, 1);

    // ---- scores --------------------------------------------------------------------------------
    const int n = p1 - p0;                      // rows in the shared tile, the new one included
    {
        const int sg = tid / LPP, sl = tid % LPP;
        float q[G][8];
#pragma unroll
        for (int j = 0; j < G; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) q[j][i] = vec[j][sl * 8 + i];
        // every lane runs the same trip count (the shuffles need the full warp)
#pragma unroll
        for (int r0 = 0; r0 < kSplitLen; r0 += NSG) {
            const int r = r0 + sg;
            float kf[8];
            if (r < n) {
                unpack8(*reinterpret_cast<const uint4*>(&kbuf[r][sl * 8]), kf);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) kf[i] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < G; ++j) {
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) s = fmaf(q[j][i], kf[i], s);
#pragma unroll
                for (int o = LPP / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (sl == 0 && r < n) sc[j][r] = s;
            }
        }
    }
    __syncthreads();

    // ---- softmax statistics of this split ----------------------------------------------------
    for (int j = warp; j < G; j += NWARP) {
        float m = -INFINITY;
        for (int i = lane; i < n; i += 32) m = fmaxf(m, sc[j][i]);
        m = warp_max(m);
        float l = 0.f;
        for (int i = lane; i < n; i += 32) {
            const float e = __expf(sc[j][i] - m);
            sc[j][i] = e;
            l += e;
        }
        l = warp_sum(l);
        if (lane == 0) { stat_m[j] = m; stat_l[j] = l; }
    }
    __syncthreads();

    // ---- probability-weighted V: each thread owns whole output elements -----------------------
    const int nsplit = p.nsplit;
#pragma unroll
    for (int t = 0; t < OUT_PER_THREAD; ++t) {
        const int e = tid + t * kAttnThreads;
        if (e < G * D) {
            const int j = e / D, d = e % D;
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
            int r = 0;
            for (; r + 3 < n; r += 4) {
                o0 = fmaf(sc[j][r], bf16_bits_to_f32(vbuf[r][d]), o0);
                o1 = fmaf(sc[j][r + 1], bf16_bits_to_f32(vbuf[r + 1][d]), o1);
                o2 = fmaf(sc[j][r + 2], bf16_bits_to_f32(vbuf[r + 2][d]), o2);
                o3 = fmaf(sc[j][r + 3], bf16_bits_to_f32(vbuf[r + 3][d]), o3);
            }
            for (; r < n; ++r) o0 = fmaf(sc[j][r], bf16_bits_to_f32(vbuf[r][d]), o0);
            const float o = (o0 + o1) + (o2 + o3);
            const int head = g * G + j;
            if (n_active == 1) p.out[size_t(head) * D + d] = f32_to_bf16_bits(o / stat_l[j]);
            else p.part_o[(size_t(head) * nsplit + split) * D + d] = o;
        }
    }
    if (n_active == 1) { trace_end(p.trace); return; }
    if (tid < G) {
        const int head = g * G + tid;
        p.part_ml[(size_t(head) * nsplit + split) * 2] = stat_m[tid];
        p.part_ml[(size_t(head) * nsplit + split) * 2 + 1] = stat_l[tid];
    }

    trace_mark(p.trace, 2);
    // ---- merge by the last CTA of this KV head ---------------------------------------------------
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned ticket = atomicAdd(&p.counters[g], 1u);
        s_last = (ticket == unsigned(n_active - 1));
    }
    __syncthreads();
    trace_mark(p.trace, 3);
    if (!s_last) { trace_end(p.trace); return; }
    __threadfence();

    float num[OUT_PER_THREAD], den[OUT_PER_THREAD], run_m[OUT_PER_THREAD];
#pragma unroll
    for (int t = 0; t < OUT_PER_THREAD; ++t) { num[t] = 0.f; den[t] = 0.f; run_m[t] = -INFINITY; }
    for (int s0 = 0; s0 < n_active; s0 += 64) {              // 64 splits per pass (4096 positions)
        const int ns = min(64, n_active - s0);
        __syncthreads();
        // per head: max over this pass, weights exp(m_s - M) into shared, and the pass's denominator
        for (int j = warp; j < G; j += NWARP) {
            const float* ml = p.part_ml + (size_t(g * G + j) * nsplit + s0) * 2;
            const float2 a0 = lane < ns ? __ldcg(reinterpret_cast<const float2*>(ml) + lane) : make_float2(-INFINITY, 0.f);
            const float2 a1 = lane + 32 < ns ? __ldcg(reinterpret_cast<const float2*>(ml) + lane + 32)
                                             : make_float2(-INFINITY, 0.f);
            const float M = warp_max(fmaxf(a0.x, a1.x));
            const float w0 = lane < ns ? __expf(a0.x - M) : 0.f;
            const float w1 = lane + 32 < ns ? __expf(a1.x - M) : 0.f;
            mrg_w[j][lane] = w0;
            mrg_w[j][lane + 32] = w1;
            const float den_pass = warp_sum(fmaf(w0, a0.y, w1 * a1.y));
            if (lane == 0) { stat_m[j] = M; stat_l[j] = den_pass; }
        }
        __syncthreads();
#pragma unroll
        for (int t = 0; t < OUT_PER_THREAD; ++t) {
            const int e = tid + t * kAttnThreads;
            if (e < G * D) {
                const int j = e / D, d = e % D;
                const int head = g * G + j;
                const float* po = p.part_o + (size_t(head) * nsplit + s0) * D + d;
                float a = 0.f;
                const float b = stat_l[j];
                for (int s = 0; s < ns; s += kMergeBatch) {    // kMergeBatch independent loads in flight
                    float v[kMergeBatch];
#pragma unroll
                    for (int i = 0; i < kMergeBatch; ++i) v[i] = (s + i < ns) ? __ldcg(po + size_t(s + i) * D) : 0.f;
#pragma unroll
                    for (int i = 0; i < kMergeBatch; ++i) a = fmaf(mrg_w[j][(s + i) & 63], v[i], a);
                }
                // fold this pass into the running (max, num, den)
                const float M = stat_m[j];
                const float newm = fmaxf(run_m[t], M);
                const float c_old = run_m[t] == -INFINITY ? 0.f : __expf(run_m[t] - newm);
                const float c_new = __expf(M - newm);
                num[t] = num[t] * c_old + a * c_new;
                den[t] = den[t] * c_old + b * c_new;
                run_m[t] = newm;
            }
        }
    }
#pragma unroll
    for (int t = 0; t < OUT_PER_THREAD; ++t) {
        const int e = tid + t * kAttnThreads;
        if (e < G * D) {
            const int j = e / D, d = e % D;
            p.out[size_t(g * G + j) * D + d] = f32_to_bf16_bits(num[t] / den[t]);
        }
    }
    if (tid == 0) p.counters[g] = 0;
    trace_end(p.trace);
}

// ---- several sequences per launch ----------------------------------------------------------------------
// At batch 32 the cache is the larger half of a step's bytes (32 sequences x context x 4 KB per KV head pair and
// layer), so this form is built for bandwidth rather than for one round trip: grid (hkv, chunks, sequences),
// a CTA walks up to kBatchTiles consecutive 64-position tiles of one KV head of one sequence through a
// double-buffered cp.async ring (the next tile lands while this one is scored), carrying a running (max, sum)
// and rescaled PV accumulators, so the q/k normalisation + rotation is paid once per 512 positions and a
// context of 2048 leaves 4 partials per head to merge instead of 32 (measured: 2, 4, 6, 8, 16 tiles per CTA give
// 2.90, 2.70, 2.67, 2.67, 2.75 ms per batch-32 step).  Arithmetic and rounding points per
// element are those of attn_gqa_kernel; only the grouping of the softmax partials differs.
constexpr int kBatchTiles = 8;

int attn_batch_chunks(int max_ctx) { return (attn_splits(max_ctx) + kBatchTiles - 1) / kBatchTiles; }

template <int D, int G>
__global__ void __launch_bounds__(kAttnThreads, 3) attn_gqa_batch_kernel(AttnParams p) {
    constexpr int LPP = D / 8;
    constexpr int NSG = kAttnThreads / LPP;
    constexpr int NWARP = kAttnThreads / 32;
    constexpr int NV = G + 1;
    constexpr int OUT_PER_THREAD = (G * D + kAttnThreads - 1) / kAttnThreads;
    constexpr int TILE = kSplitLen * D;                  // elements of one K (or V) tile

    extern __shared__ __align__(16) unsigned char batch_smem[];
    uint16_t* kbuf = reinterpret_cast<uint16_t*>(batch_smem);            // [2][kSplitLen][D]
    uint16_t* vbuf = kbuf + 2 * TILE;                                     // [2][kSplitLen][D]
    __shared__ __align__(16) float vec[NV + 1][D];
    __shared__ float gain[2][D];
    __shared__ float rot[2][D];
    __shared__ __align__(16) float sc[G][kSplitLen];
    __shared__ __align__(16) float prob[(kAttnThreads / 32) * G * kSplitLen];   // each warp's copy of a tile's probabilities
    __shared__ float stat_m[G], stat_l[G];
    __shared__ float mrg_w[G][64];
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.x, chunk = blockIdx.y;
    {
        const size_t b = blockIdx.z;
        p.qkv += b * p.qkv_stride;
        p.out += b * p.out_stride;
        p.block_table += b * p.bt_stride;
        p.pos += b;
        if (p.rope_pos) p.rope_pos += b;
        p.part_o += b * p.hq * p.nsplit * D;
        p.part_ml += b * p.hq * p.nsplit * 2;
        p.counters += b * p.hkv;
        if (p.k_new_out) p.k_new_out += b * p.hkv * D;
        if (p.v_new_out) p.v_new_out += b * p.hkv * D;
    }
    if (tid < D) {                                       // weights: independent of the kernel before
        gain[0][tid] = p.norm_mode ? bf16_bits_to_f32(p.gamma_q[tid]) : 1.f;
        gain[1][tid] = p.norm_mode ? bf16_bits_to_f32(p.gamma_k[tid]) : 1.f;
    }
    pdl_trigger();
    pdl_wait();

    const int pos = *p.pos;
    const int total = pos + 1;
    const int n_tiles = (total + kSplitLen - 1) / kSplitLen;
    const int t0 = chunk * kBatchTiles;
    if (pos < 0 || pos >= p.max_ctx || t0 >= n_tiles) return;
    const int t1 = min(t0 + kBatchTiles, n_tiles);
    const int n_chunks = (n_tiles + kBatchTiles - 1) / kBatchTiles;
    const bool owner = (t1 == n_tiles);                  // this CTA's last tile holds the new position
    if (p.append_only == 1 && !owner) return;

    // A thread copies the same 16-byte piece of rows r_first, r_first + NSG, ...; when a page holds whole tiles
    // (page_size a multiple of 64) the tile has one page and the source address is one multiply-add per row.
    const int piece = tid % LPP, r_first = tid / LPP;
    const size_t row_stride = size_t(p.hkv) * D;
    const bool tile_in_page = (p.page_size % kSplitLen) == 0;
    auto fetch = [&](int tile, int buf) {                // cached rows of a tile -> ring slot (the new row comes from vec[])
        const int base = tile * kSplitLen;
        const int rows = min(kSplitLen, pos - base);     // rows below pos are in the cache
        // K rows are stored with their 16-byte pieces XOR-swizzled by the row's low three bits, so the score MMA's
        // 4-byte operand loads (eight rows, one piece) fall on 32 different banks
        uint16_t* kd = kbuf + buf * TILE;
        uint16_t* vd = vbuf + buf * TILE + piece * 8;
        if (tile_in_page) {
            const int page = p.block_table[base / p.page_size];
            const size_t off0 = (size_t(page) * p.page_size + (base % p.page_size)) * row_stride + size_t(g) * D + piece * 8;
#pragma unroll
            for (int r = r_first; r < kSplitLen; r += NSG)
                if (r < rows) {
                    cp_async16(kd + r * D + ((piece ^ (r & 7)) * 8), p.k_pool + off0 + r * row_stride);
                    cp_async16(vd + r * D, p.v_pool + off0 + r * row_stride);
                }
        } else {
            for (int r = r_first; r < rows; r += NSG) {
                const int pp = base + r;
                const int page = p.block_table[pp / p.page_size];
                const size_t off = (size_t(page) * p.page_size + (pp % p.page_size)) * row_stride + size_t(g) * D + piece * 8;
                cp_async16(kd + r * D + ((piece ^ (r & 7)) * 8), p.k_pool + off);
                cp_async16(vd + r * D, p.v_pool + off);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (p.append_only != 1) fetch(t0, 0);

    // ---- this token's q (G heads), k, v for KV head g: as in attn_gqa_kernel ----
    const int rd = p.rotary_dim, half = rd >> 1;
    const int rpos = p.rope_pos ? *p.rope_pos : pos;
    if (tid < rd) {
        rot[0][tid] = bf16_bits_to_f32(p.cos_table[size_t(rpos) * rd + tid]);
        rot[1][tid] = bf16_bits_to_f32(p.sin_table[size_t(rpos) * rd + tid]);
    }
    int vis[2] = {warp, warp + NWARP};
    float xv[2][D / 32];
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2) {
        const int vi = vis[s2];
#pragma unroll
        for (int i = 0; i < D / 32; ++i) xv[s2][i] = 0.f;
        if (vi < NV + 1) {
            const uint16_t* src;
            if (vi < G) src = p.qkv + size_t(g * G + vi) * D;
            else if (vi == G) src = p.qkv + size_t(p.hq) * D + size_t(g) * D;
            else src = p.qkv + size_t(p.hq + p.hkv) * D + size_t(g) * D;
#pragma unroll
            for (int i = 0; i < D / 32; ++i) xv[s2][i] = bf16_bits_to_f32(src[lane + 32 * i]);
        }
    }
    __syncthreads();                                     // rot[] / gain[] visible
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2) {
        const int vi = vis[s2];
        if (vi >= NV + 1) continue;
        float* x = xv[s2];
        if (vi == G + 1) {
#pragma unroll
            for (int i = 0; i < D / 32; ++i) vec[vi][lane + 32 * i] = x[i];
            continue;
        }
        if (p.norm_mode != 0) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < D / 32; ++i) ss = fmaf(x[i], x[i], ss);
            ss = warp_sum(ss);
            const float rstd = rsqrtf(ss / float(D) + p.eps);
            const float* gm = gain[vi < G ? 0 : 1];
#pragma unroll
            for (int i = 0; i < D / 32; ++i) x[i] = round_bf16(round_bf16(x[i] * rstd) * gm[lane + 32 * i]);
        }
#pragma unroll
        for (int i = 0; i < D / 32; ++i) {
            const int e = lane + 32 * i;
            float r = x[i];
            if (e < rd) {
                const int pi = (e < half) ? i + half / 32 : i - half / 32;
                float partner = 0.f;
#pragma unroll
                for (int k2 = 0; k2 < D / 32; ++k2) if (k2 == pi) partner = x[k2];
                if (e < half) partner = -partner;
                r = round_bf16(__fadd_rn(__fmul_rn(x[i], rot[0][e]), __fmul_rn(partner, rot[1][e])));
            }
            if (vi < G) r = round_bf16(r * p.scale);
            vec[vi][e] = r;
        }
    }
    __syncthreads();

    if (owner && p.append_only != 2) {                   // append this token's entry to the cache
        const int page = p.block_table[pos / p.page_size];
        const size_t base = ((size_t(page) * p.page_size + (pos % p.page_size)) * p.hkv + g) * D;
        for (int i = tid; i < D; i += kAttnThreads) {
            const uint16_t kb = f32_to_bf16_bits(vec[G][i]), vb = f32_to_bf16_bits(vec[G + 1][i]);
            p.k_pool[base + i] = kb;
            p.v_pool[base + i] = vb;
            if (p.k_new_out) p.k_new_out[size_t(g) * D + i] = kb;
            if (p.v_new_out) p.v_new_out[size_t(g) * D + i] = vb;
        }
    }
    if (p.append_only == 1) return;

    // PV mapping: thread (dp, rg) owns the output pair d = 2dp, 2dp+1 of every query head for the rows of row
    // group rg of each tile (one 4-byte V load feeds 2G products); the RG partial sums meet once, after the last
    // tile, through shared memory in fixed order.
    constexpr int PAIRS = D / 2, RG = kAttnThreads / PAIRS, ROWS_PER_RG = kSplitLen / RG;
    const int dp = tid % PAIRS, rg = tid / PAIRS;
    float o_acc[G][2];
#pragma unroll
    for (int j = 0; j < G; ++j) { o_acc[j][0] = 0.f; o_acc[j][1] = 0.f; }
    // Scores on the tensor cores (mma.sync m16n8k16, bf16 in, f32 out): the G query heads are rows 0..G-1 of the
    // 16-row A operand (the rest zero), a warp owns 8 positions of the tile as the B operand's columns.  A fragment
    // of k-step ks, lane (gq, tq): a0 = q[gq][16ks + 2tq, +1], a2 = q[gq][16ks + 8 + 2tq, +1]; a1 = a3 = 0.
    constexpr int KS = D / 16;
    static_assert(kAttnThreads / 32 * 8 == kSplitLen, "one warp per 8 positions of a tile");
    const int gq = lane >> 2, tq = lane & 3;
    uint32_t qa[KS][2];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        qa[ks][0] = 0u; qa[ks][1] = 0u;
        if (gq < G) {
            const float* qv = vec[gq];
            qa[ks][0] = uint32_t(f32_to_bf16_bits(qv[16 * ks + 2 * tq])) | (uint32_t(f32_to_bf16_bits(qv[16 * ks + 2 * tq + 1])) << 16);
            qa[ks][1] = uint32_t(f32_to_bf16_bits(qv[16 * ks + 8 + 2 * tq])) |
                        (uint32_t(f32_to_bf16_bits(qv[16 * ks + 8 + 2 * tq + 1])) << 16);
        }
    }

    // Two barriers per tile.  #1: this tile's copies have landed (and every warp has left the tile before, so the
    // other ring slot, sc[] and each warp's prob[] may be rewritten) -- the next tile's copies are requested right
    // after it.  #2: the scores of all 64 positions are in sc[].  The softmax statistics are then computed by every
    // warp for itself (lane-uniform registers, its own copy of the probabilities), which saves the third barrier and
    // the phase in which only G warps worked.
    float m_run[G], l_run[G];
#pragma unroll
    for (int j = 0; j < G; ++j) { m_run[j] = -INFINITY; l_run[j] = 0.f; }
    float* my_prob = prob + warp * (G * kSplitLen);
    for (int tile = t0; tile < t1; ++tile) {
        const int buf = (tile - t0) & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        const int base = tile * kSplitLen;
        const int n = min(kSplitLen, total - base);      // rows of this tile, the new one included
        if (tile == n_tiles - 1)                         // the new entry goes straight into the ring slot
            for (int i = tid; i < D; i += kAttnThreads) {
                const int rn = pos - base;
                kbuf[buf * TILE + rn * D + (((i >> 3) ^ (rn & 7)) << 3) + (i & 7)] = f32_to_bf16_bits(vec[G][i]);
                vbuf[buf * TILE + rn * D + i] = f32_to_bf16_bits(vec[G + 1][i]);
            }
        __syncthreads();                                 // #1
        if (tile + 1 < t1) fetch(tile + 1, buf ^ 1);
        const uint16_t* kt = kbuf + buf * TILE;
        const uint16_t* vt = vbuf + buf * TILE;
        // scores: warp w, positions 8w .. 8w+7.  B fragment of k-step ks, lane (gq, tq): b0 = K[8w + gq][16ks + 2tq, +1],
        // b1 = K[8w + gq][16ks + 8 + 2tq, +1]; C fragment c0, c1 = score of head gq at positions 8w + 2tq, +1.
        // Rows past n hold stale bytes; they only reach columns the statistics pass zeroes.
        {
            const int nrow = warp * 8 + gq;
            const uint16_t* krow = kt + nrow * D + 2 * tq;
            const int sw = nrow & 7;
            float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + (((2 * ks) ^ sw) << 3));
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + (((2 * ks + 1) ^ sw) << 3));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                             "{%0, %1, %2, %3};"
                             : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
                             : "r"(qa[ks][0]), "r"(0u), "r"(qa[ks][1]), "r"(0u), "r"(b0), "r"(b1));
            }
            if (gq < G) {
                sc[gq][warp * 8 + 2 * tq] = c0;
                sc[gq][warp * 8 + 2 * tq + 1] = c1;
            }
        }
        __syncthreads();                                 // #2
        // running softmax statistics, per warp; rows past n get probability 0 so the PV loop needs no bound
        float resc[G];
#pragma unroll
        for (int j = 0; j < G; ++j) {
            const float s0 = lane < n ? sc[j][lane] : -INFINITY;
            const float s1 = lane + 32 < n ? sc[j][lane + 32] : -INFINITY;
            const float new_m = fmaxf(m_run[j], warp_max(fmaxf(s0, s1)));
            const float e0 = lane < n ? __expf(s0 - new_m) : 0.f;
            const float e1 = lane + 32 < n ? __expf(s1 - new_m) : 0.f;
            my_prob[j * kSplitLen + lane] = e0;
            my_prob[j * kSplitLen + lane + 32] = e1;
            const float l = warp_sum(e0 + e1);
            resc[j] = m_run[j] == -INFINITY ? 0.f : __expf(m_run[j] - new_m);
            l_run[j] = l_run[j] * resc[j] + l;
            m_run[j] = new_m;
        }
        __syncwarp();
        // probability-weighted V
        {
            float a[G][2];
#pragma unroll
            for (int j = 0; j < G; ++j) { a[j][0] = 0.f; a[j][1] = 0.f; }
            const int r_begin = rg * ROWS_PER_RG;
            if (r_begin < n) {
#pragma unroll 2
                for (int i = 0; i < ROWS_PER_RG; i += 4) {
                    const int r = r_begin + i;
                    // rows past n hold stale bytes: read them as zero bits, their probability is zero too
                    float v_lo[4], v_hi[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t v2 = r + u < n ? *reinterpret_cast<const uint32_t*>(&vt[(r + u) * D + 2 * dp]) : 0u;
                        v_lo[u] = bf16_lo(v2);
                        v_hi[u] = bf16_hi(v2);
                    }
#pragma unroll
                    for (int j = 0; j < G; ++j) {
                        const float4 pr = *reinterpret_cast<const float4*>(&my_prob[j * kSplitLen + r]);   // four rows
                        a[j][0] = fmaf(pr.x, v_lo[0], a[j][0]); a[j][1] = fmaf(pr.x, v_hi[0], a[j][1]);
                        a[j][0] = fmaf(pr.y, v_lo[1], a[j][0]); a[j][1] = fmaf(pr.y, v_hi[1], a[j][1]);
                        a[j][0] = fmaf(pr.z, v_lo[2], a[j][0]); a[j][1] = fmaf(pr.z, v_hi[2], a[j][1]);
                        a[j][0] = fmaf(pr.w, v_lo[3], a[j][0]); a[j][1] = fmaf(pr.w, v_hi[3], a[j][1]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < G; ++j) {
                o_acc[j][0] = o_acc[j][0] * resc[j] + a[j][0];
                o_acc[j][1] = o_acc[j][1] * resc[j] + a[j][1];
            }
        }
    }
    __syncthreads();                                     // every warp has left the ring: it becomes pv_red
    if (warp == 0 && lane == 0) {
#pragma unroll
        for (int j = 0; j < G; ++j) { stat_m[j] = m_run[j]; stat_l[j] = l_run[j]; }
    }

    // the row groups' partial sums meet in the (now idle) ring: pv_red[rg][j][d]
    float* pv_red = reinterpret_cast<float*>(batch_smem);
#pragma unroll
    for (int j = 0; j < G; ++j) {
        pv_red[(rg * G + j) * D + 2 * dp] = o_acc[j][0];
        pv_red[(rg * G + j) * D + 2 * dp + 1] = o_acc[j][1];
    }
    __syncthreads();
    const int nsplit = p.nsplit;
#pragma unroll
    for (int t = 0; t < OUT_PER_THREAD; ++t) {
        const int e = tid + t * kAttnThreads;
        if (e < G * D) {
            const int j = e / D, d = e % D;
            const int head = g * G + j;
            float o = 0.f;
#pragma unroll
            for (int r2 = 0; r2 < RG; ++r2) o += pv_red[(r2 * G + j) * D + d];
            if (n_chunks == 1) p.out[size_t(head) * D + d] = f32_to_bf16_bits(o / stat_l[j]);
            else p.part_o[(size_t(head) * nsplit + chunk) * D + d] = o;
        }
    }
    if (n_chunks == 1) return;
    if (tid < G) {
        const int head = g * G + tid;
        p.part_ml[(size_t(head) * nsplit + chunk) * 2] = stat_m[tid];
        p.part_ml[(size_t(head) * nsplit + chunk) * 2 + 1] = stat_l[tid];
    }
    // ---- merge by the last CTA of this (sequence, KV head) ----
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&p.counters[g], 1u) == unsigned(n_chunks - 1));
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // n_chunks <= 64 is checked on the host: one pass
    for (int j = warp; j < G; j += NWARP) {
        const float* ml = p.part_ml + size_t(g * G + j) * nsplit * 2;
        const float2 a0 = lane < n_chunks ? __ldcg(reinterpret_cast<const float2*>(ml) + lane) : make_float2(-INFINITY, 0.f);
        const float2 a1 = lane + 32 < n_chunks ? __ldcg(reinterpret_cast<const float2*>(ml) + lane + 32)
                                               : make_float2(-INFINITY, 0.f);
        const float M = warp_max(fmaxf(a0.x, a1.x));
        const float w0 = lane < n_chunks ? __expf(a0.x - M) : 0.f;
        const float w1 = lane + 32 < n_chunks ? __expf(a1.x - M) : 0.f;
        mrg_w[j][lane] = w0;
        mrg_w[j][lane + 32] = w1;
        const float den = warp_sum(fmaf(w0, a0.y, w1 * a1.y));
        if (lane == 0) stat_l[j] = den;
    }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < OUT_PER_THREAD; ++t) {
        const int e = tid + t * kAttnThreads;
        if (e < G * D) {
            const int j = e / D, d = e % D;
            const int head = g * G + j;
            const float* po = p.part_o + size_t(head) * nsplit * D + d;
            float a = 0.f;
            for (int s = 0; s < n_chunks; s += kMergeBatch) {
                float v[kMergeBatch];
#pragma unroll
                for (int i = 0; i < kMergeBatch; ++i) v[i] = (s + i < n_chunks) ? __ldcg(po + size_t(s + i) * D) : 0.f;
#pragma unroll
                for (int i = 0; i < kMergeBatch; ++i) a = fmaf(mrg_w[j][(s + i) & 63], v[i], a);
            }
            p.out[size_t(head) * D + d] = f32_to_bf16_bits(a / stat_l[j]);
        }
    }
    if (tid == 0) p.counters[g] = 0;
}

cudaError_t attn_gqa_dispatch(const AttnParams& p, cudaStream_t stream, bool pdl) {
    const int G = p.hq / p.hkv;
    if (p.batch > 1) {
        const int chunks = attn_batch_chunks(p.max_ctx);
        if (chunks > 64) return cudaErrorInvalidValue;
        const dim3 bgrid(p.hkv, chunks, p.batch), bblock(kAttnThreads);
#define TFB_ATTN_BATCH(DD, GG)                                                                                 \
        if (p.d == DD && G == GG) {                                                                            \
            const size_t smem = size_t(4) * kSplitLen * DD * sizeof(uint16_t);                                 \
            static PerDeviceOnce once;                                                                          \
            if (once.first()) {                                                                                       \
                cudaError_t e = cudaFuncSetAttribute(attn_gqa_batch_kernel<DD, GG>,                            \
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); \
                if (e != cudaSuccess) return e;                                                                \
            }                                                                                                  \
            return launch_kernel(attn_gqa_batch_kernel<DD, GG>, bgrid, bblock, smem, stream, pdl, p);         \
        }
        TFB_ATTN_BATCH(128, 1) TFB_ATTN_BATCH(128, 2) TFB_ATTN_BATCH(128, 4) TFB_ATTN_BATCH(64, 2) TFB_ATTN_BATCH(64, 1)
#undef TFB_ATTN_BATCH
        return cudaErrorInvalidValue;
    }
    const dim3 grid(p.hkv, p.nsplit), block(kAttnThreads);
#define TFB_ATTN(DD, GG)                                                                                  \
    if (p.d == DD && G == GG) {                                                                           \
        static PerDeviceOnce once;                                                                         \
        if (once.first()) {                                                                                      \
            cudaFuncSetAttribute(attn_gqa_kernel<DD, GG>, cudaFuncAttributePreferredSharedMemoryCarveout, \
                                 cudaSharedmemCarveoutMaxShared);                                         \
        }                                                                                                 \
        return launch_kernel(attn_gqa_kernel<DD, GG>, grid, block, 0, stream, pdl, p);                    \
    }
    TFB_ATTN(128, 1) TFB_ATTN(128, 2) TFB_ATTN(128, 4) TFB_ATTN(64, 2) TFB_ATTN(64, 1)
#undef TFB_ATTN
    return cudaErrorInvalidValue;
}

}  // namespace tfb

// ---- scratch that lives in the library image -----------------------------------------------------
// Some callers may not call cudaMalloc at all (see tfb_attn_gqa_decode_noalloc in the header).  For
// them the split-KV partials, their (max, sum) pairs and the merge tickets live in this file-scope
// array: 64 query heads x 64 splits (4096 positions) x 128 dims of f32, about 2.1 MB that every GPU
// which loads the library holds until the process exits.
namespace tfb {

constexpr int kStaticHeads = 64, kStaticSplits = 64, kStaticDim = 128;
constexpr size_t kStaticPartO = size_t(kStaticHeads) * kStaticSplits * kStaticDim * sizeof(float);
constexpr size_t kStaticPartMl = size_t(kStaticHeads) * kStaticSplits * 2 * sizeof(float);
constexpr size_t kStaticCounters = 256;                       // 64 tickets, padded
static __device__ __align__(256) unsigned char g_attn_scratch[kStaticPartO + kStaticPartMl + kStaticCounters];

// In host code `g_attn_scratch` is only a handle for the runtime, not a device address, so the
// address is asked for once per device (with that device current) and remembered.
cudaError_t attn_static_scratch(int hq, int nsplit, int d, float** part_o, float** part_ml, unsigned** counters,
                                bool* fits) {
    *fits = hq <= kStaticHeads && nsplit <= kStaticSplits && d <= kStaticDim && hq > 0 && nsplit > 0 && d > 0;
    if (!*fits) return cudaSuccess;
    constexpr int kMaxDevices = 64;
    static unsigned char* base[kMaxDevices] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (base[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_attn_scratch);
        if (e != cudaSuccess) return e;
        base[dev] = static_cast<unsigned char*>(p);
    }
    *part_o = reinterpret_cast<float*>(base[dev]);
    *part_ml = reinterpret_cast<float*>(base[dev] + kStaticPartO);
    *counters = reinterpret_cast<unsigned*>(base[dev] + kStaticPartO + kStaticPartMl);
    return cudaSuccess;
}

}  // namespace tfb
