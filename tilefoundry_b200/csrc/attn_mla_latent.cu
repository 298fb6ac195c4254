// Multi-head latent attention decode over a cache of LATENTS (MiniCPM3): what is kept per position is the
// normalised compressed key/value vector (kv_lora = 256 values) and the rotated shared rotary key (32 values) --
// 576 bytes per position per layer instead of the 12,800 of assembled per-head keys and values.  The
// up-projection W_kv_b = [W_UK | W_UV] per head is never applied to the cache: W_UK is folded into the query
// ("absorbed": q_lat[h] = W_UK[h]^T q_nope[h], so q_lat . c == q_nope . (W_UK c)) and W_UV into the output
// (out[h] = W_UV[h] (sum_t p_t c_t)).  Every head attends over the same 288-wide rows.
//
// Three launches per layer, chained by programmatic dependent launch:
//   mla_q_absorb_kernel   grid (3, heads): low-rank norm + this head's 96 rows of q_b (32 rows per CTA, weights
//                         in registers before the dependency wait), then either the CTA's share of W_UK^T q
//                         (two CTAs per head, 32 nope rows each) or RoPE on the rotary query slice.  CTA (2, 0)
//                         also norms the compressed kv vector, rotates the shared key slice and APPENDS the
//                         latent row at *pos.
//   mla_latent_attn_kernel grid (heads / 4, splits of 32 positions): the 32 latent rows stream into shared
//                         memory once (cp.async, cached rows before the dependency wait) and serve 4 heads;
//                         warp (head, half of the 288 columns) x lane (position) takes half a dot product, a warp
//                         owns a head's softmax, then the probabilities weight the 256 latent columns.  Partials
//                         (f32) go to part_o / part_ml.  Many small CTAs (340 at context 1088) spread evenly
//                         over the multiprocessors; with 8 heads per CTA 170 CTAs left 22 of 148 with double work.
//   mla_v_absorb_kernel   grid (heads), 512 threads: merges the split partials of a head (every (max, sum) pair in
//                         one load per thread, up to 32 partial columns per thread in flight), applies W_UV[h]
//                         (64 rows x 256, in registers before the wait) and rounds the 64 outputs to bf16.
//
// Algorithmic bytes per layer: (ctx+1) * 576 (cache) + heads*(96*q_lora + 128*256)*2 (q_b and W_kv_b).
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

constexpr int kLatThreads = 256;
constexpr int kLatSplit = 32;                      // positions per attention CTA
constexpr int kKvl = 256, kNope = 64, kRope = 32, kVd = 64;
constexpr int kLatRow = kKvl + kRope;              // 288 values per cached position
constexpr int kLatPad = kLatRow + 8;               // shared-memory row stride: 16-byte reads of 8 threads hit 32 banks

__device__ __forceinline__ void lat_cp16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 :: "r"(uint32_t(__cvta_generic_to_shared(smem_dst))), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void lat_cp_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---- 1. q_b rows + absorption of W_UK / RoPE / latent append --------------------------------------------------
// A launch may carry several tokens of one sequence (a prompt chunk): the last grid axis is the token, each with its
// own position word, input row and scratch; one token (decode) is the same code with that axis 1 long.
__device__ __forceinline__ MlaLatentParams for_token(const MlaLatentParams& q, int tok) {
    MlaLatentParams p = q;
    p.qkv_a += size_t(tok) * q.qkv_stride;
    p.pos += tok;
    if (p.rope_pos) p.rope_pos += tok;
    p.q_lat += size_t(tok) * q.heads * 2 * kKvl;
    p.q_rope += size_t(tok) * q.heads * kRope;
    p.part_o += size_t(tok) * q.heads * q.nsplit * kKvl;
    p.part_ml += size_t(tok) * q.heads * q.nsplit * 2;
    p.out += size_t(tok) * q.heads * kVd;
    if (p.latent_new_out) p.latent_new_out += size_t(tok) * kLatRow;
    return p;
}

template <int QC>                                  // q_lora = 256 * QC
__global__ void __launch_bounds__(kLatThreads) mla_q_absorb_kernel(const MlaLatentParams pq) {
    const MlaLatentParams p = for_token(pq, blockIdx.z);
    constexpr int QL = 256 * QC;
    __shared__ float xs[QL];
    __shared__ float red[32];
    __shared__ float qv[32];
    __shared__ float part[2][kKvl];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j = blockIdx.x, h = blockIdx.y;      // j: 0,1 = nope rows [32j, 32j+32); 2 = the rotary rows
    trace_start(p.trace);

    // weights first: they depend on nothing, so they travel while the projection before this one finishes
    const size_t q_row0 = size_t(h) * (kNope + kRope) + size_t(j) * 32 + size_t(warp) * 4;
    uint4 wq[4][QC];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int i = 0; i < QC; ++i) wq[r][i] = ld_stream16(p.w_q_b + (q_row0 + r) * QL + (lane + 32 * i) * 8);
    // W_UK rows of this CTA: thread (pair of columns, half of the 32 rows)
    const int pair = tid & 127, half = tid >> 7;
    uint32_t wk[16];
    if (j < 2) {
        const uint16_t* base = p.w_kv_b + (size_t(h) * (kNope + kVd) + size_t(j) * 32 + size_t(half) * 16) * kKvl + pair * 2;
#pragma unroll
        for (int r = 0; r < 16; ++r) wk[r] = __ldg(reinterpret_cast<const uint32_t*>(base + size_t(r) * kKvl));
    }
    // The position does not change inside a step (the head kernel advances it, and a step's first launch waits for
    // the whole previous step), so it and the rotary row it selects are read ahead of the wait as well.
    const int pos = *reinterpret_cast<const volatile int*>(p.pos);
    const bool pos_ok = pos >= 0 && pos < p.max_ctx;
    constexpr int HALF = kRope / 2;
    float rc = 0.f, rs = 0.f;
    if (pos_ok && j == 2 && tid < kRope) {
        const int rpos = p.rope_pos ? *reinterpret_cast<const volatile int*>(p.rope_pos) : pos;
        rc = bf16_bits_to_f32(p.cos_table[size_t(rpos) * kRope + tid]);
        rs = bf16_bits_to_f32(p.sin_table[size_t(rpos) * kRope + tid]);
    }
    pdl_trigger();
    pdl_wait();
    trace_waited(p.trace);
    if (!pos_ok) return;

    // low-rank norm of the compressed query: cast, then gain
    {
        float v[QC], ss = 0.f;
#pragma unroll
        for (int i = 0; i < QC; ++i) { v[i] = bf16_bits_to_f32(p.qkv_a[tid + 256 * i]); ss = fmaf(v[i], v[i], ss); }
        const float rstd = rsqrtf(block_sum(ss, red) / float(QL) + p.lora_eps);
#pragma unroll
        for (int i = 0; i < QC; ++i)
            xs[tid + 256 * i] = round_bf16(round_bf16(v[i] * rstd) * bf16_bits_to_f32(p.gamma_q_a[tid + 256 * i]));
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < QC; ++i) {
            const float4* x4 = reinterpret_cast<const float4*>(xs + (lane + 32 * i) * 8);
            acc = dot8(wq[r][i], x4[0], x4[1], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) qv[warp * 4 + r] = round_bf16(acc);
    }
    __syncthreads();

    if (j < 2) {
        // q_lat[c] += sum over this CTA's 32 nope rows of bf16(q * scale) * W_UK[row][c]
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const float q = round_bf16(qv[half * 16 + r] * p.scale);
            a0 = fmaf(q, bf16_lo(wk[r]), a0);
            a1 = fmaf(q, bf16_hi(wk[r]), a1);
        }
        part[half][pair * 2] = a0;
        part[half][pair * 2 + 1] = a1;
        __syncthreads();
        p.q_lat[(size_t(h) * 2 + j) * kKvl + tid] = part[0][tid] + part[1][tid];
        trace_end(p.trace);
        return;
    }

    if (tid < kRope) {
        const float qp = (tid < HALF) ? -qv[tid + HALF] : qv[tid - HALF];
        const float q = round_bf16(__fadd_rn(__fmul_rn(qv[tid], rc), __fmul_rn(qp, rs)));
        p.q_rope[size_t(h) * kRope + tid] = round_bf16(q * p.scale);
    }
    if (h != 0) { trace_end(p.trace); return; }

    // this token's latent row: norm of the compressed kv vector | rotated shared key slice
    const uint16_t* kv_c = p.qkv_a + QL;
    const float v = bf16_bits_to_f32(kv_c[tid]);
    const float rstd = rsqrtf(block_sum(v * v, red) / float(kKvl) + p.lora_eps);
    const uint16_t lat = f32_to_bf16_bits(round_bf16(v * rstd) * bf16_bits_to_f32(p.gamma_kv_a[tid]));
    const size_t row = size_t(p.block_table[pos / p.page_size]) * p.page_size + (pos % p.page_size);
    uint16_t* dst = p.pool + row * kLatRow;
    dst[tid] = lat;
    if (p.latent_new_out) p.latent_new_out[tid] = lat;
    if (tid < kRope) {
        const uint16_t* kr = kv_c + kKvl;
        const float k0 = bf16_bits_to_f32(kr[tid]);
        const float kp = (tid < HALF) ? -bf16_bits_to_f32(kr[tid + HALF]) : bf16_bits_to_f32(kr[tid - HALF]);
        const uint16_t rot = f32_to_bf16_bits(__fadd_rn(__fmul_rn(k0, rc), __fmul_rn(kp, rs)));
        dst[kKvl + tid] = rot;
        if (p.latent_new_out) p.latent_new_out[kKvl + tid] = rot;
    }
    trace_end(p.trace);
}

// ---- 2. attention of 4 heads over 32 latent rows ----------------------------------------------------------------
constexpr int kLatHG = 4;

__global__ void __launch_bounds__(kLatThreads) mla_latent_attn_kernel(const MlaLatentParams pq) {
    const MlaLatentParams p = for_token(pq, blockIdx.z);
    constexpr int HG = kLatHG;
    __shared__ __align__(16) uint16_t kv[kLatSplit][kLatPad];
    __shared__ __align__(16) float qf[HG][kLatRow];
    __shared__ float sp[2 * HG][kLatSplit];        // partial scores of a (head, column half) warp
    __shared__ float sc[HG][kLatSplit];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h0 = blockIdx.x * HG, split = blockIdx.y, p0 = split * kLatSplit;
    constexpr int PIECES = kLatRow / 8;            // 16-byte pieces per row

    trace_start(p.trace);
    // the position is fixed for the whole step (see mla_q_absorb_kernel): rows below it are final already
    const int pos = *reinterpret_cast<const volatile int*>(p.pos);
    const int total = pos + 1;
    const int n_active = (total + kLatSplit - 1) / kLatSplit;
    const bool active = pos >= 0 && pos < p.max_ctx && split < n_active;
    const int n = active ? min(p0 + kLatSplit, total) - p0 : 0;
    const int n_cached = active ? min(p0 + kLatSplit, pos) - p0 : 0;      // all but this token's own row
    // (a chunk of prompt tokens runs this kernel once per token in one dependency chain: rows of the chunk's earlier
    // tokens may still be on their way then, so nothing is fetched ahead of the wait)
    const int n_early = p.no_early_rows ? 0 : n_cached;
    for (int c = tid; c < n_early * PIECES; c += kLatThreads) {
        const int r = c / PIECES, piece = c % PIECES, pp = p0 + r;
        const size_t row = size_t(p.block_table[pp / p.page_size]) * p.page_size + (pp % p.page_size);
        lat_cp16(&kv[r][piece * 8], p.pool + row * kLatRow + piece * 8);
    }
    pdl_trigger();
    pdl_wait();
    trace_waited(p.trace);
    if (!active) { lat_cp_wait(); return; }

    for (int c = tid; c < (n_cached - n_early) * PIECES; c += kLatThreads) {
        const int r = n_early + c / PIECES, piece = c % PIECES, pp = p0 + r;
        const size_t row = size_t(p.block_table[pp / p.page_size]) * p.page_size + (pp % p.page_size);
        lat_cp16(&kv[r][piece * 8], p.pool + row * kLatRow + piece * 8);
    }
    if (n > n_cached && tid < PIECES) {            // the row appended by the kernel before this one
        const size_t row = size_t(p.block_table[pos / p.page_size]) * p.page_size + (pos % p.page_size);
        lat_cp16(&kv[n_cached][tid * 8], p.pool + row * kLatRow + tid * 8);
    }
    if (warp >= HG) {                              // warp 4 + i fetches head i's query: both partial absorbed queries and
        const int hh = warp - HG;                  // the rotary slice, every load issued before the first is used
        const size_t h = size_t(h0 + hh);
        const float4* a = reinterpret_cast<const float4*>(p.q_lat + h * 2 * kKvl);
        const float4* b = a + kKvl / 4;
        const float4 a0 = __ldcg(a + lane), a1 = __ldcg(a + lane + 32), b0 = __ldcg(b + lane), b1 = __ldcg(b + lane + 32);
        const float r = __ldcg(p.q_rope + h * kRope + lane);
        float4* q4 = reinterpret_cast<float4*>(&qf[hh][0]);
        q4[lane] = make_float4(a0.x + b0.x, a0.y + b0.y, a0.z + b0.z, a0.w + b0.w);
        q4[lane + 32] = make_float4(a1.x + b1.x, a1.y + b1.y, a1.z + b1.z, a1.w + b1.w);
        qf[hh][kKvl + lane] = r;
    }
    lat_cp_wait();
    __syncthreads();
    trace_mark(p.trace, 0);

    // scores: warp = (column half, head), lane = position; 18 pieces of 8 columns each
    {
        const int hh = warp & (HG - 1), kh = warp / HG;
        float acc = 0.f;
        if (lane < n) {
            const uint4* krow = reinterpret_cast<const uint4*>(&kv[lane][0]) + kh * (PIECES / 2);
            const float4* q4 = reinterpret_cast<const float4*>(&qf[hh][0]) + kh * PIECES;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f;
#pragma unroll
            for (int c = 0; c < PIECES / 2; c += 3) {
                a0 = dot8(krow[c], q4[2 * c], q4[2 * c + 1], a0);
                a1 = dot8(krow[c + 1], q4[2 * c + 2], q4[2 * c + 3], a1);
                a2 = dot8(krow[c + 2], q4[2 * c + 4], q4[2 * c + 5], a2);
            }
            acc = a0 + a1 + a2;
        }
        sp[warp][lane] = acc;
    }
    __syncthreads();
    if (warp < HG) {
        const float s = lane < n ? sp[warp][lane] + sp[warp + HG][lane] : -INFINITY;
        const float m = warp_max(s);
        const float e = lane < n ? __expf(s - m) : 0.f;
        const float l = warp_sum(e);
        sc[warp][lane] = e;
        if (lane == 0)
            *reinterpret_cast<float2*>(p.part_ml + (size_t(h0 + warp) * p.nsplit + split) * 2) = make_float2(m, l);
    }
    __syncthreads();
    trace_mark(p.trace, 1);

    // weighted latents: thread (pair of columns, half of the heads)
    {
        constexpr int HH = HG / 2;
        const int pair = tid & 127, hb = (tid >> 7) * HH;
        float acc[HH][2];
#pragma unroll
        for (int i = 0; i < HH; ++i) acc[i][0] = acc[i][1] = 0.f;
#pragma unroll 4
        for (int r = 0; r < n; ++r) {
            const uint32_t u = *reinterpret_cast<const uint32_t*>(&kv[r][pair * 2]);
            const float c0 = bf16_lo(u), c1 = bf16_hi(u);
#pragma unroll
            for (int i = 0; i < HH; ++i) {
                const float w = sc[hb + i][r];
                acc[i][0] = fmaf(w, c0, acc[i][0]);
                acc[i][1] = fmaf(w, c1, acc[i][1]);
            }
        }
#pragma unroll
        for (int i = 0; i < HH; ++i)
            *reinterpret_cast<float2*>(p.part_o + (size_t(h0 + hb + i) * p.nsplit + split) * kKvl + pair * 2) =
                make_float2(acc[i][0], acc[i][1]);
    }
    trace_end(p.trace);
}

// ---- 3. merge of the splits + W_UV -------------------------------------------------------------------------------
constexpr int kLatMaxSplits = 1024;                // 32,768 positions
constexpr int kVaThreads = 512;

__global__ void __launch_bounds__(kVaThreads) mla_v_absorb_kernel(const MlaLatentParams pq) {
    const MlaLatentParams p = for_token(pq, blockIdx.y);
    __shared__ float w[kLatMaxSplits];
    __shared__ __align__(16) float ol[2][kKvl];
    __shared__ float red[32];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, h = blockIdx.x;
    trace_start(p.trace);
    // W_UV[h]: 64 rows x 256; a warp takes 4 rows, a lane 8 columns of each
    uint4 wv[4];
    const uint16_t* base = p.w_kv_b + (size_t(h) * (kNope + kVd) + kNope + size_t(warp) * 4) * kKvl + lane * 8;
#pragma unroll
    for (int r = 0; r < 4; ++r) wv[r] = ld_stream16(base + size_t(r) * kKvl);
    const int pos = *reinterpret_cast<const volatile int*>(p.pos);      // fixed for the whole step
    pdl_trigger();
    pdl_wait();
    trace_waited(p.trace);
    if (pos < 0 || pos >= p.max_ctx) return;
    const int n_active = (pos + kLatSplit) / kLatSplit;
    // the first 64 splits' partial columns of this thread are requested together with the (max, sum) pairs below:
    // one round trip to L2 for everything the merge needs
    const int mc = tid & (kKvl - 1), mhalf = tid >> 8;
    const float* po = p.part_o + size_t(h) * p.nsplit * kKvl + mc;
    float v0[32];
#pragma unroll
    for (int q = 0; q < 32; ++q) v0[q] = __ldcg(po + size_t(min(mhalf + 2 * q, n_active - 1)) * kKvl);
    // (max, sum) of every split: one load per thread (two beyond 512 splits), kept in registers
    const float2* ml = reinterpret_cast<const float2*>(p.part_ml + size_t(h) * p.nsplit * 2);
    float2 st[kLatMaxSplits / kVaThreads];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kLatMaxSplits / kVaThreads; ++i) {
        const int sidx = tid + i * kVaThreads;
        st[i] = sidx < n_active ? __ldcg(ml + sidx) : make_float2(-INFINITY, 0.f);
        m = fmaxf(m, st[i].x);
    }
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int i = 1; i < kVaThreads / 32; ++i) m = fmaxf(m, red[i]);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < kLatMaxSplits / kVaThreads; ++i) {
        const int sidx = tid + i * kVaThreads;
        if (sidx < n_active) {
            const float ws = __expf(st[i].x - m);
            w[sidx] = ws;
            den = fmaf(ws, st[i].y, den);
        }
    }
    __syncthreads();                               // everyone has read red; w is complete
    den = block_sum(den, red);
    {
        // thread (column, parity of the split)
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int q = 0; q < 32; q += 2) {
            a = fmaf(mhalf + 2 * q < n_active ? w[mhalf + 2 * q] : 0.f, v0[q], a);
            b = fmaf(mhalf + 2 * q + 2 < n_active ? w[mhalf + 2 * q + 2] : 0.f, v0[q + 1], b);
        }
        for (int s0 = mhalf + 64; s0 < n_active; s0 += 64) {   // contexts beyond 2048 positions
            float v[32];
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = __ldcg(po + size_t(min(s0 + 2 * q, n_active - 1)) * kKvl);
#pragma unroll
            for (int q = 0; q < 32; q += 2) {
                a = fmaf(s0 + 2 * q < n_active ? w[s0 + 2 * q] : 0.f, v[q], a);
                b = fmaf(s0 + 2 * q + 2 < n_active ? w[s0 + 2 * q + 2] : 0.f, v[q + 1], b);
            }
        }
        ol[mhalf][mc] = a + b;
    }
    __syncthreads();
    if (tid < kKvl) ol[0][tid] = (ol[0][tid] + ol[1][tid]) / den;
    __syncthreads();
    const float4* x4 = reinterpret_cast<const float4*>(&ol[0][lane * 8]);
    const float4 xa = x4[0], xb = x4[1];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const float acc = warp_sum(dot8(wv[r], xa, xb, 0.f));
        if (lane == 0) p.out[size_t(h) * kVd + warp * 4 + r] = f32_to_bf16_bits(acc);
    }
    trace_end(p.trace);
}

int mla_latent_splits(int max_ctx) { return (max_ctx + kLatSplit - 1) / kLatSplit; }

bool mla_latent_supported(int heads, int q_lora, int kv_lora, int nope, int rope, int vd, int max_ctx) {
    return kv_lora == kKvl && nope == kNope && rope == kRope && vd == kVd && heads > 0 && heads % 4 == 0 &&
           q_lora % 256 == 0 && q_lora >= 256 && q_lora <= 1024 && max_ctx > 0 &&
           mla_latent_splits(max_ctx) <= kLatMaxSplits;
}

cudaError_t mla_latent_dispatch(const MlaLatentParams& params, cudaStream_t stream, bool pdl) {
    MlaLatentParams p = params;
    p.trace = p.trace3[0];
    cudaError_t e;
    const int T = p.tokens > 0 ? p.tokens : 1;
    const dim3 block(kLatThreads), g1(3, p.heads, T);
    switch (p.q_lora / 256) {
        case 1: e = launch_kernel(mla_q_absorb_kernel<1>, g1, block, 0, stream, pdl, p); break;
        case 2: e = launch_kernel(mla_q_absorb_kernel<2>, g1, block, 0, stream, pdl, p); break;
        case 3: e = launch_kernel(mla_q_absorb_kernel<3>, g1, block, 0, stream, pdl, p); break;
        case 4: e = launch_kernel(mla_q_absorb_kernel<4>, g1, block, 0, stream, pdl, p); break;
        default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return e;
    p.trace = p.trace3[1];
    e = launch_kernel(mla_latent_attn_kernel, dim3(p.heads / kLatHG, p.nsplit, T), block, 0, stream, pdl, p);
    if (e != cudaSuccess) return e;
    p.trace = p.trace3[2];
    return launch_kernel(mla_v_absorb_kernel, dim3(p.heads, T), dim3(kVaThreads), 0, stream, pdl, p);
}

}  // namespace tfb
