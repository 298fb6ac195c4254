// One decode step of the Qwen3 architecture as ONE cooperative launch (one CTA per SM):
//   embed -> layers x [norm + q|k|v, q/k norm + RoPE + KV append + split-KV attention + merge, o + residual,
//   norm + gate/up + SwiGLU, down + residual] -> final norm + head + greedy pick + position advance.
//
// Why one launch: as separate launches the step is bound by the chain of dependent launches (about 4 us of
// release + activation staging + first-byte latency + tail per kernel, five per layer), not by bytes.  Here the
// weight stream never stops at a dependency: weights do not depend on activations, so the producer warp of a CTA
// walks a STATIC schedule of tiles through all phases of all layers and lands them in a 196 KB shared-memory ring
// with bulk asynchronous copies (cp.async.bulk, mbarrier transaction counts), as far ahead of the arithmetic as
// the ring allows.  While the consumer warps wait for an activation vector, the ring takes up to 4.5 us of HBM
// traffic.
//
// Data layout: matrix rows are dealt to the CTAs in contiguous blocks (CTA c owns rows [c*n/G, (c+1)*n/G)), taken
// in groups of at most 14 rows (gate/up: 7 row pairs, interleaved); a tile is 1024 consecutive K elements of a
// group's rows, 2 KB per row.  The dot products run on the tensor cores although the batch is one: K is folded
// into the MMA's N (see "tensor-core pieces" below), one tcgen05.mma per 16 rows x 128 elements, accumulating over
// a group's tiles in tensor memory; four epilogue warps read the accumulators back, a team of eight lanes per
// row.  Everything is summed in a fixed order (deterministic); rounding points are those of gemv_kernel /
// attn_gqa_kernel / lm_head_kernel.
//
// Dependencies between phases travel WITH the data: every activation element is a 32-bit word, bf16 value in
// the low half and a 16-bit tag in the high half that names the launch and the phase that wrote it.  A consumer
// polls the words themselves (relaxed gpu-scope loads; each word of a vector is fetched by exactly one thread
// of the CTA and shared through shared memory) and proceeds when every tag matches, so a hand-over costs one
// trip through L2 -- no fence, no counter, no second read.  (With counters it cost fence + atomic + counter poll
// + vector read, about 3.5 us per phase, five phases per layer.)  A word is single-copy atomic, the tag of a
// phase differs from the tag of whatever the word held before (launch counter * phases + phase, mod 65535, +1;
// zero is never a tag), and a word is rewritten only after every reader of its old value has produced something
// that the writer has already consumed (the data dependences of the step guarantee it).
// Attention: KV head h, split s of the context on CTA s*hkv + h (the context is cut into at most G/hkv splits,
// so no CTA has two); cached K/V rows are requested before this token's q|k|v is waited on; split 0 of a KV
// head merges the partials, which reach it as tagged 64-bit words.  Every wait is bounded: a timeout sets
// *status, and every later wait of that CTA returns at once, so the launch always ends.
//
// HBM-bound: algorithmic bytes per launch = all weights once + the KV rows of positions [0, pos].
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {
namespace {

constexpr int kCW = 12;                          // consumer warps
constexpr int kCT = kCW * 32;                    // consumer threads
constexpr int kFusedThreads = kCT + 32;          // + the producer warp (warp 0)
constexpr int kSliceLen = 1024;                  // K elements of a weight row in one tile
constexpr int kGroupRows = 16;                   // weight rows one accumulator has room for (8 tensor-memory lanes each)
#ifndef TFB_GROUP_CAP
#define TFB_GROUP_CAP 14
#endif
constexpr int kGroupCap = TFB_GROUP_CAP;         // ... and how many a tile takes (even; 2048 / 148 = 13.8 rows fit one tile)
constexpr int kRowBytes = kSliceLen * 2;         // a tile row: 2 KB, one bulk copy
constexpr int kTileBytes = kGroupCap * kRowBytes;
static_assert(kGroupCap % 2 == 0 && kGroupCap <= kGroupRows, "a tile's rows must fit one accumulator");
constexpr int kStages = (210 * 1024) / kTileBytes;   // seven 28 KB stages
constexpr int kChunkBytes = 256;                 // of every tile row, what one MMA consumes (128 elements)
constexpr int kAccBufs = 4;                      // accumulators in flight between the MMA thread and the epilogue warps
constexpr int kAccCols = 32;                     // tensor-memory columns per hand-over: 16 per issuing thread
constexpr int kTmemCols = kAccBufs * kAccCols;
constexpr int kEpiWarps = 4;                     // consumer warps 0..3 read tensor memory (one lane quadrant each)
constexpr int kMmaWarp = 4;                      // first of the consumer warps whose lane 0 issues MMAs
constexpr int kMmaThreads = 2;                   // ... each takes its share of every tile's chunks, into its own accumulator
constexpr unsigned long long kWaitNs = 200ull * 1000 * 1000;   // every wait gives up after 0.2 s
constexpr int kD = 128, kGQ = 2;                 // head dim and query heads per KV head of this build
constexpr int kBatchRows = 8;                    // cache rows one warp holds in registers at a time
constexpr int kMergeLoads = 6;                   // 16-byte pieces of split partials one merging thread requests at once

struct FusedSmem {
    alignas(128) unsigned char ring[kStages][kTileBytes];
    alignas(8) unsigned long long full[kStages];
    unsigned long long empty[kStages];
    unsigned long long acc_full[kAccBufs], acc_empty[kAccBufs], mma_done;
    uint32_t tmem_base;
    float head_v[kEpiWarps];                     // the epilogue warps' best logit and its row, for the pick
    int head_i[kEpiWarps];
    float red[16];
    alignas(16) float q[kGQ][kD];
    alignas(16) float knew[kD];
    alignas(16) float vnew[kD];
    float wm[kCW][kGQ], wl[kCW][kGQ];
    alignas(16) float wo[kCW][kGQ][kD];
    int flag;
    volatile int abort;
    float mrg_m[kGQ][64], mrg_l[kGQ][64];        // (max, sum) of every split of this KV head's query heads, for the merge
    unsigned koff[kCW][kBatchRows];              // element offset of warp w's cached row t of its first batch, or ~0u
    unsigned new_off;                            // where this token's own row goes (the owner split)
};

__device__ __forceinline__ uint32_t s_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mb_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(s_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mb_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(s_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mb_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(s_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mb_try(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(s_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(s_u32(dst)), "l"(src), "r"(bytes), "r"(s_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" :: "n"(kCT) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint4 ld_relaxed16(const unsigned* p) {
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_relaxed32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_tagged(unsigned* p, unsigned tag, uint16_t bits) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" :: "l"(p), "r"((tag << 16) | unsigned(bits)) : "memory");
}
// f32 partials travel the same way in 64-bit words: value in the low half, tag in the high half.
__device__ __forceinline__ void st_tagged64(unsigned long long* p, unsigned tag, float v) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ ulonglong2 ld_relaxed64x2(const unsigned long long* p) {
    ulonglong2 v;
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool tags_ok(const uint4& w, unsigned tag) {
    return (w.x >> 16) == tag && (w.y >> 16) == tag && (w.z >> 16) == tag && (w.w >> 16) == tag;
}

// Bounded waits.  After the first timeout of a CTA every wait returns at once (the results are void, *status says so).
__device__ __forceinline__ void wait_bar(FusedSmem& s, unsigned long long* bar, unsigned parity, unsigned* status, unsigned code) {
    if (mb_try(bar, parity)) return;
    if (s.abort) return;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mb_try(bar, parity)) return;
        if (s.abort) return;
        if (global_ns() - t0 > kWaitNs) break;
    }
    s.abort = 1;
    atomicOr(status, code);
}
// One thread of the CTA polls; the consumer barrier that follows hands the acquired view to the others.
__device__ __forceinline__ void wait_count(FusedSmem& s, const unsigned* ctr, unsigned target, unsigned* status, unsigned code) {
    if (s.abort) return;
    if (ld_acquire(ctr) >= target) return;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 16; ++i)
            if (ld_acquire(ctr) >= target) return;
        if (global_ns() - t0 > kWaitNs) break;
    }
    s.abort = 1;
    atomicOr(status, code);
}
// Inside a polling loop: true when the loop has to give up (another wait of the CTA already did, or this one has
// made kPollLimit trips to L2: a trip takes 0.3 us at the least, so the bound is a tenth of a second or more).
constexpr int kPollLimit = 1 << 19;
__device__ __forceinline__ bool poll_expired(FusedSmem& s, int& spins, unsigned* status, unsigned code) {
    if (s.abort) return true;
    if (++spins < kPollLimit) return false;
    s.abort = 1;
    atomicOr(status, code);
    return true;
}
// A CTA's outputs of a phase are written (by the threads of one warp, or before a consumer_sync): publish them.
__device__ __forceinline__ void arrive(unsigned* ctr) {
    __threadfence();
    atomicAdd(ctr, 1u);
}

// debug timeline of phase `ph` (one thread per CTA calls these)
__device__ __forceinline__ void tl_enter(const FusedParams& p, int ph) {
    if (p.timeline && ph < p.timeline_slots) atomicMin(p.timeline + 8 * ph, global_ns());
}
__device__ __forceinline__ void tl_waited(const FusedParams& p, int ph) {
    if (p.timeline && ph < p.timeline_slots) {
        const unsigned long long t = global_ns();
        atomicMin(p.timeline + 8 * ph + 1, t);
        atomicMax(p.timeline + 8 * ph + 2, t);
    }
}
__device__ __forceinline__ void tl_done(const FusedParams& p, int ph) {
    if (p.timeline && ph < p.timeline_slots) atomicMax(p.timeline + 8 * ph + 3, global_ns());
}

__device__ __forceinline__ void span(int n, int c, int G, int& u0, int& u1) {
    u0 = int((long long)n * c / G);
    u1 = int((long long)n * (c + 1) / G);
}

struct RingPos {
    int stage;
    unsigned parity;
    __device__ __forceinline__ void next() {
        if (++stage == kStages) { stage = 0; parity ^= 1u; }
    }
    __device__ __forceinline__ void advance(int n) {
        const int t = stage + n;
        stage = t % kStages;
        parity ^= unsigned(t / kStages) & 1u;
    }
};

// A CTA's rows of a matrix are taken in groups of at most `cap` units (rows, or gate/up pairs), evenly sized.
__device__ __forceinline__ void groups_of(int units, int cap, int& ng, int& per) {
    ng = (units + cap - 1) / cap;
    per = ng > 0 ? (units + ng - 1) / ng : 0;
}

// ---- producer: the tiles of one matrix phase, in the order the consumers take them ------------------------------
// A tile is kSliceLen consecutive K elements of up to kGroupCap rows, one 2 KB bulk copy per row (lane r copies
// tile row r); gate/up phases interleave the rows: tile row 2i is gate row i of the group, 2i + 1 its up row.
__device__ __forceinline__ void produce(FusedSmem& s, RingPos& rp, const uint16_t* w, const uint16_t* w2, int n, int k,
                                        int c, int G, int lane, unsigned* status) {
    const int KT = k / kSliceLen;
    int u0, u1, ng, per;
    span(n, c, G, u0, u1);
    groups_of(u1 - u0, w2 ? kGroupCap / 2 : kGroupCap, ng, per);
    for (int g = 0; g < ng; ++g) {
        const int u = u0 + g * per, nu = min(per, u1 - u);
        const int nrows = w2 ? 2 * nu : nu;
        const uint16_t* src = w;
        if (lane < nrows) src = w2 ? ((lane & 1) ? w2 : w) + size_t(u + (lane >> 1)) * k : w + size_t(u + lane) * k;
        for (int kt = 0; kt < KT; ++kt) {
            if (lane == 0) {
                wait_bar(s, &s.empty[rp.stage], rp.parity ^ 1u, status, 0x10000u);
                mb_expect_tx(&s.full[rp.stage], unsigned(nrows) * kRowBytes);
            }
            __syncwarp();
            if (lane < nrows)
                bulk_load(s.ring[rp.stage] + lane * kRowBytes, src + kt * kSliceLen, kRowBytes, &s.full[rp.stage]);
            rp.next();
        }
    }
}

enum { kStore = 0, kResidual = 1, kSwiglu = 2, kHead = 3 };

struct HeadBest {
    float v;
    int i;
};

// ---- tensor-core pieces of the matrix phases ---------------------------------------------------------------------
// Batch 1 has no N dimension to give the MMA, so K is FOLDED into it.  A K-major operand without swizzle is made of core
// matrices of 8 rows x 16 bytes, each 128 contiguous bytes.  Read 256 contiguous bytes of a weight row (128 elements)
// as ONE 8 x 16 block -- "row" r, column 8h + c is element h * 64 + r * 8 + c (two core matrices, 128 bytes apart along
// K) -- and let the stride between 8-row groups be the pitch of the tile's rows: the A operand of an M = 128 MMA is then
// the same 128-element chunk of 16 weight rows, straight from the row-major tile.  The B operand is the matching chunk
// of the activation vector, folded the same way (8 x 16; N = 16 is the least M = 128 takes, the second eight are never
// read).  D[8g + r][r'] = sum over (h, c) of W[g][(r, h, c)] * x[(r', h, c)]: the diagonal r = r' of each 8 x 8 block
// carries the products that belong together, and successive chunks ACCUMULATE in tensor memory, so after k / 128 MMAs
// row g's dot product is D[8g][0] + D[8g + 1][1] + ... + D[8g + 7][7].  Seven of eight products are thrown away, and
// the tensor core still takes 4 KB of weights every ~50 cycles, four times what HBM delivers to one SM: the CUDA cores
// (64 unpack + multiply-add instructions per 2 KB per warp, and a barrier per handful of rows) did not keep up.
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
__device__ __forceinline__ void umma_arrive(unsigned long long* bar) {     // arrives when every MMA issued so far is done
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(s_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
// D f32, A and B bf16, both K-major, N = 16, M = 128
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(16 >> 3) << 17) | (uint32_t(128 >> 4) << 24);

struct AccPos {                                   // which accumulator a hand-over uses, and its barrier parity
    int buf;
    unsigned parity;
    __device__ __forceinline__ void next() {
        if (++buf == kAccBufs) { buf = 0; parity ^= 1u; }
    }
    __device__ __forceinline__ void advance(int n) {
        const int t = buf + n;
        buf = t % kAccBufs;
        parity ^= unsigned(t / kAccBufs) & 1u;
    }
};

// The dot product of the weight row that this lane's team of eight lanes holds in the accumulators of hand-over `buf`
// (row i of an M = 128 accumulator sits in tensor-memory lane i; lane l of the quadrant wants column l % 8 of each).  Every lane of a team
// returns the row's sum (a fixed shuffle tree: deterministic).  `release` is arrived on as soon as the load has landed.
__device__ __forceinline__ float team_dot(uint32_t tmem, int buf, int quad, int lane, unsigned long long* release) {
    uint32_t v[8], w[8];
    const uint32_t taddr = tmem + (uint32_t(quad * 32) << 16) + uint32_t(buf * kAccCols);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "r"(taddr + uint32_t(kAccCols / kMmaThreads)) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mb_arrive(release);                        // this warp has read the accumulators
    const bool b4 = lane & 4, b2 = lane & 2, b1 = lane & 1;
    const uint32_t t0 = b4 ? v[4] : v[0], t1 = b4 ? v[5] : v[1], t2 = b4 ? v[6] : v[2], t3 = b4 ? v[7] : v[3];
    const uint32_t s0 = b4 ? w[4] : w[0], s1 = b4 ? w[5] : w[1], s2 = b4 ? w[6] : w[2], s3 = b4 ? w[7] : w[3];
    const uint32_t q0 = b2 ? t2 : t0, q1 = b2 ? t3 : t1, r0 = b2 ? s2 : s0, r1 = b2 ? s3 : s1;
    float d = __uint_as_float(b1 ? q1 : q0) + __uint_as_float(b1 ? r1 : r0);      // the two issuing threads' halves
    d += __shfl_xor_sync(0xffffffffu, d, 1);
    d += __shfl_xor_sync(0xffffffffu, d, 2);
    d += __shfl_xor_sync(0xffffffffu, d, 4);
    return d;
}

// ---- consumers: one matrix phase --------------------------------------------------------------------------------
// y = epilogue(W . prologue(x)) for this CTA's rows.  x: tagged words, complete when every tag is in_tag; y: tagged
// words written with out_tag (the head writes plain bf16 logits to y_plain instead).
template <int KIND, bool NORM>
__device__ __forceinline__ void consume(FusedSmem& s, RingPos& rp, AccPos& ap, const FusedParams& p, int n, int k,
                                        const unsigned* x, unsigned in_tag, const uint16_t* gamma, unsigned* y,
                                        unsigned out_tag, uint16_t* y_plain, uint16_t* trace_row,
                                        int c, int G, int cw, int lane, HeadBest* best, int ph) {
    const int KT = k / kSliceLen;
    int u0, u1, ng, per;
    span(n, c, G, u0, u1);
    groups_of(u1 - u0, KIND == kSwiglu ? kGroupCap / 2 : kGroupCap, ng, per);
    const int tid = cw * 32 + lane;
    const int nvec = k >> 2;                                  // <= 4 * kCT (k <= 6144)

    // norm gains are weights: ask for the ones of this thread's pieces before the wait
    uint2 gv[4];
    if (NORM) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            gv[i] = tid + i * kCT < nvec ? *reinterpret_cast<const uint2*>(gamma + 4 * (tid + i * kCT)) : make_uint2(0u, 0u);
    }
    if (tid == 0) tl_enter(p, ph);
    // The activation vector: each tagged word is fetched by exactly one thread of the CTA, polled until its tag says
    // this phase's input has landed, normalised where the phase asks for it, and parked as bf16 in shared memory (the
    // attention scratch, idle here) in natural order: the MMAs' other operand.
    uint16_t* xs = reinterpret_cast<uint16_t*>(&s.wo[0][0][0]);
    {
        uint4 w[4];
        int spins = 0;
        for (;;) {                                            // (a thread without an i-th piece re-reads its first)
            bool ok = true;
#pragma unroll
            for (int i = 0; i < 4; ++i) w[i] = ld_relaxed16(x + 4 * (tid + i * kCT < nvec ? tid + i * kCT : tid % nvec));
#pragma unroll
            for (int i = 0; i < 4; ++i) ok = ok && tags_ok(w[i], in_tag);
            if (ok || poll_expired(s, spins, p.status, 0x100u)) break;
        }
        float rstd = 1.f;
        if (NORM) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (tid + i * kCT < nvec) {
                    const float a = bf16_lo(w[i].x), b = bf16_lo(w[i].y), cc = bf16_lo(w[i].z), d = bf16_lo(w[i].w);
                    ss = fmaf(a, a, ss); ss = fmaf(b, b, ss); ss = fmaf(cc, cc, ss); ss = fmaf(d, d, ss);
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) s.red[cw] = ss;
            consumer_sync();
            float tot = 0.f;
#pragma unroll
            for (int q = 0; q < kCW; ++q) tot += s.red[q];
            rstd = rsqrtf(tot / float(k) + p.eps);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (tid + i * kCT < nvec) {
                uint32_t lo = (w[i].x & 0xffffu) | (w[i].y << 16), hi = (w[i].z & 0xffffu) | (w[i].w << 16);
                if (NORM) {                                   // Qwen3RMSNorm: round, then gain (a bf16 multiply)
                    const float a = round_bf16(round_bf16(bf16_lo(w[i].x) * rstd) * bf16_lo(gv[i].x));
                    const float b = round_bf16(round_bf16(bf16_lo(w[i].y) * rstd) * bf16_hi(gv[i].x));
                    const float cc = round_bf16(round_bf16(bf16_lo(w[i].z) * rstd) * bf16_lo(gv[i].y));
                    const float d = round_bf16(round_bf16(bf16_lo(w[i].w) * rstd) * bf16_hi(gv[i].y));
                    lo = uint32_t(f32_to_bf16_bits(a)) | (uint32_t(f32_to_bf16_bits(b)) << 16);
                    hi = uint32_t(f32_to_bf16_bits(cc)) | (uint32_t(f32_to_bf16_bits(d)) << 16);
                    if (trace_row && KIND == kHead && c == 0)  // the final-normed hidden state, for the trace
                        *reinterpret_cast<uint2*>(trace_row + 4 * (tid + i * kCT)) = make_uint2(lo, hi);
                }
                *reinterpret_cast<uint2*>(xs + 4 * (tid + i * kCT)) = make_uint2(lo, hi);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // these writes are read by the MMAs (async proxy)
    }
    consumer_sync();
    if (tid == 0) tl_waited(p, ph);

    const int sample_step = (KIND == kHead && p.temperature > 0.f) ? *p.pos : 0;   // (the draw is keyed by the position)
    const uint32_t tmem = s.tmem_base;
    RingPos r = rp;
    AccPos a = ap;
    if (cw >= kMmaWarp && cw < kMmaWarp + kMmaThreads) {
        // ---- the MMA issuers (lane 0 of two warps): a tensor-core instruction of this size occupies the pipe for ~45
        // cycles however it is shaped, and the waits and commits around a tile cost the issuing thread as much again;
        // two threads, each with half of every tile's chunks and an accumulator of its own, keep the pipe busy ----
        if (lane == 0) {
            const int j = cw - kMmaWarp;
            constexpr int CPT = kRowBytes / kChunkBytes / kMmaThreads;          // chunks of a tile per thread
            const uint64_t xdesc = folded_desc(s_u32(xs) + uint32_t(j * CPT * kChunkBytes), kChunkBytes);
            for (int g = 0; g < ng; ++g) {
                wait_bar(s, &s.acc_empty[a.buf], a.parity ^ 1u, p.status, 0x40000u);
                tc_fence_after();
                const uint32_t d_tmem = tmem + uint32_t(a.buf * kAccCols + j * (kAccCols / kMmaThreads));
                for (int kt = 0; kt < KT; ++kt) {
                    wait_bar(s, &s.full[r.stage], r.parity, p.status, 0x20000u);
                    const uint64_t da = folded_desc(s_u32(s.ring[r.stage]) + uint32_t(j * CPT * kChunkBytes), kRowBytes);
                    const uint64_t db = xdesc + uint64_t((kt * kRowBytes) >> 4);
#pragma unroll
                    for (int t = 0; t < CPT; ++t)
                        umma_f16(d_tmem, da + uint64_t((t * kChunkBytes) >> 4), db + uint64_t((t * kChunkBytes) >> 4), kIdesc,
                                 (kt | t) != 0 ? 1u : 0u);
                    umma_arrive(&s.empty[r.stage]);               // the stage is free when the MMAs that read it are done
                    r.next();
                }
                umma_arrive(&s.acc_full[a.buf]);
                a.next();
            }
        }
        __syncwarp();
    } else if (cw < kEpiWarps) {
        // ---- the epilogue warps: a team of eight lanes per weight row, four rows per warp, no step across warps ----
        const int quad = (cw + 1) & 3;                        // the tensor-memory lane quadrant this warp may read
        const int trow = quad * 4 + (lane >> 3);              // the tile row of this lane's team
        const int unit = KIND == kSwiglu ? trow >> 1 : trow;  // (gate/up: tile rows 2i and 2i + 1 make unit i)
        const bool writer = KIND == kSwiglu ? (lane & 15) == 0 : (lane & 7) == 0;
        for (int g = 0; g < ng; ++g) {
            const int u = u0 + g * per, nu = min(per, u1 - u);
            const int row = u + unit;
            const bool live = writer && unit < nu;
            float res = 0.f;                                   // (written by this CTA itself in an earlier phase)
            if (KIND == kResidual && live) res = bf16_lo(ld_relaxed32(y + row));
            wait_bar(s, &s.acc_full[a.buf], a.parity, p.status, 0x80000u);
            tc_fence_after();
            const float v = team_dot(tmem, a.buf, quad, lane, &s.acc_empty[a.buf]);
            if (KIND == kStore) {
                if (live) st_tagged(y + row, out_tag, f32_to_bf16_bits(v));
            } else if (KIND == kSwiglu) {
                const float up = round_bf16(__shfl_xor_sync(0xffffffffu, v, 8));
                if (live) st_tagged(y + row, out_tag, f32_to_bf16_bits(round_bf16(silu_f32(round_bf16(v))) * up));
            } else if (KIND == kHead) {
                float sc = round_bf16(v);
                if (live) {
                    if (y_plain) y_plain[row] = f32_to_bf16_bits(sc);
                    // sampling: the greedy pick over logit / T + Gumbel noise (the rule of lm_head_kernel, same variates)
                    if (p.temperature > 0.f) sc = __fdiv_rn(sc, p.temperature) + gumbel_variate(p.seed, sample_step, row);
                    if (sc > best->v || (sc == best->v && row < best->i)) { best->v = sc; best->i = row; }
                }
            } else {
                if (live) {
                    const uint16_t out = f32_to_bf16_bits(res + round_bf16(v));
                    st_tagged(y + row, out_tag, out);
                    if (trace_row) trace_row[row] = out;
                }
            }
            a.next();
        }
    }
    // every thread tracks the ring and the accumulators, whatever its role in this phase
    rp.advance(ng * KT);
    ap.advance(ng);
    consumer_sync();                                            // (every MMA of the phase is complete: its accumulator was
                                                                //  waited for; s.red / xs may be reused)
    if (tid == 0) tl_done(p, ph);
}

__device__ __forceinline__ size_t kv_offset(const FusedParams& p, int pos, int h) {
    const int page = p.block_table[pos / p.page_size];
    return ((size_t(page) * p.page_size + (pos % p.page_size)) * p.hkv + h) * kD;
}

// A layer's cached K/V rows of this CTA's split (first batch: the rows of s.koff) asked into L2 well before attention
// wants them.  A DRAM read issued when attention starts queues behind the weight stream -- every CTA keeps up to 196 KB
// of tile copies in flight, 29 MB over the GPU, 4 us of HBM time -- and attention then sat waiting for its rows.
// The warps that have nothing to do in the matrix phases issue the hints, one row half (128 bytes) of K and of V each.
__device__ __forceinline__ void ask_cache_rows(const FusedSmem& s, const FusedLayer& L, int cw, int lane) {
    if (cw < kCW / 2) return;
    const int i = (cw - kCW / 2) * 32 + lane;                   // 0 .. 191 = kCW * kBatchRows * 2 row halves
    const unsigned off = s.koff[i >> 4][(i >> 1) & (kBatchRows - 1)];
    if (off == ~0u) return;
    asm volatile("prefetch.global.L2 [%0];" :: "l"(L.k_pool + off + (i & 1) * (kD / 2)));
    asm volatile("prefetch.global.L2 [%0];" :: "l"(L.v_pool + off + (i & 1) * (kD / 2)));
}

// ---- consumers: attention of one layer ------------------------------------------------------------------------
__device__ __forceinline__ void attend(FusedSmem& s, const FusedParams& p, const FusedLayer& L, const unsigned* xqkv,
                                       unsigned in_tag, unsigned* xattn, unsigned out_tag, unsigned long long* xpart, int pos,
                                       int c, int G, int cw, int lane, int ph) {
    const int total = pos + 1;
    const int ns_max = min(G / p.hkv, 64);
    const int SL = max(16, ((total + ns_max - 1) / ns_max + 15) & ~15);
    const int NS = (total + SL - 1) / SL;
    const int h = c % p.hkv, sp = c / p.hkv;
    if (sp >= NS || c >= p.hkv * ns_max) return;
    const int p0 = sp * SL, p1 = min(p0 + SL, total), n = p1 - p0;
    const bool owner = sp == NS - 1;
    const uint16_t* kpool = L.k_pool;
    const uint16_t* vpool = L.v_pool;

    // cached rows do not depend on this token: the first batch is requested before the q|k|v counter is waited on
    uint2 kreg[kBatchRows], vreg[kBatchRows];
    // (the page table belongs to the sequence, not to a layer: the offsets were worked out once, at the start)
#pragma unroll
    for (int t = 0; t < kBatchRows; ++t) {
        const unsigned off = s.koff[cw][t];
        kreg[t] = make_uint2(0, 0);
        vreg[t] = make_uint2(0, 0);
        if (off != ~0u) {
            kreg[t] = __ldg(reinterpret_cast<const uint2*>(kpool + off + lane * 4));
            vreg[t] = __ldg(reinterpret_cast<const uint2*>(vpool + off + lane * 4));
        }
    }
    // norm gains and the rotary row of this position are known too
    const int nvec = kGQ + 2;
    float gm[4], rc[4], rs[4];
    if (cw <= kGQ) {
        const uint16_t* gsrc = cw < kGQ ? L.gamma_q : L.gamma_k;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            gm[i] = bf16_bits_to_f32(gsrc[lane + 32 * i]);
            rc[i] = bf16_bits_to_f32(p.cos_table[size_t(pos) * kD + lane + 32 * i]);
            rs[i] = bf16_bits_to_f32(p.sin_table[size_t(pos) * kD + lane + 32 * i]);
        }
    }
    if (cw == 0 && lane == 0) tl_enter(p, ph);

    // this token's q (2 heads), k, v of KV head h: one warp per vector, lane l holds elements l, l+32, l+64, l+96,
    // so the rotate-half partner (64 away) sits in the same lane; the tagged words are polled until they are this
    // layer's
    if (cw < nvec) {
        const unsigned* src = cw < kGQ ? xqkv + size_t(h * kGQ + cw) * kD
                              : cw == kGQ ? xqkv + size_t(p.hq) * kD + size_t(h) * kD
                                          : xqkv + size_t(p.hq + p.hkv) * kD + size_t(h) * kD;
        unsigned wd[4];
        int spins = 0;
        for (;;) {
#pragma unroll
            for (int i = 0; i < 4; ++i) wd[i] = ld_relaxed32(src + lane + 32 * i);
            const bool ok = (wd[0] >> 16) == in_tag && (wd[1] >> 16) == in_tag && (wd[2] >> 16) == in_tag && (wd[3] >> 16) == in_tag;
            if (__all_sync(0xffffffffu, ok)) break;
            if (poll_expired(s, spins, p.status, 0x200u)) break;
        }
        if (cw == 0 && lane == 0) tl_waited(p, ph);
        float xv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) xv[i] = bf16_lo(wd[i]);
        if (cw == kGQ + 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) s.vnew[lane + 32 * i] = xv[i];
        } else {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) ss = fmaf(xv[i], xv[i], ss);
            ss = warp_sum(ss);
            const float rstd = rsqrtf(ss / float(kD) + p.eps);
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = round_bf16(round_bf16(xv[i] * rstd) * gm[i]);
            float out[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float partner = i < 2 ? -xv[i + 2] : xv[i - 2];
                out[i] = round_bf16(__fadd_rn(__fmul_rn(xv[i], rc[i]), __fmul_rn(partner, rs[i])));
                if (cw < kGQ) out[i] = round_bf16(out[i] * p.scale);
            }
            float* dst = cw < kGQ ? s.q[cw] : s.knew;
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = out[i];
        }
    }
    consumer_sync();
    if (owner && (cw == kGQ || cw == kGQ + 1)) {                // append this token's row to the cache
        uint16_t* dst = (cw == kGQ ? L.k_pool : L.v_pool) + s.new_off;
        const float* src = cw == kGQ ? s.knew : s.vnew;
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = f32_to_bf16_bits(src[lane + 32 * i]);
    }

    float qv[kGQ][4];
#pragma unroll
    for (int jh = 0; jh < kGQ; ++jh) {
        const float4 t4 = *reinterpret_cast<const float4*>(&s.q[jh][lane * 4]);
        qv[jh][0] = t4.x; qv[jh][1] = t4.y; qv[jh][2] = t4.z; qv[jh][3] = t4.w;
    }
    float m[kGQ], l[kGQ], o[kGQ][4];
#pragma unroll
    for (int jh = 0; jh < kGQ; ++jh) { m[jh] = -INFINITY; l[jh] = 0.f; o[jh][0] = o[jh][1] = o[jh][2] = o[jh][3] = 0.f; }

    for (int b0 = 0; b0 < n; b0 += kCW * kBatchRows) {
        if (b0 > 0) {                                           // later batches of a long split: request them now
#pragma unroll
            for (int t = 0; t < kBatchRows; ++t) {
                const int pp = p0 + b0 + cw + kCW * t;
                kreg[t] = make_uint2(0, 0);
                vreg[t] = make_uint2(0, 0);
                if (pp < p1 && pp < pos) {
                    const size_t off = kv_offset(p, pp, h) + lane * 4;
                    kreg[t] = __ldg(reinterpret_cast<const uint2*>(kpool + off));
                    vreg[t] = __ldg(reinterpret_cast<const uint2*>(vpool + off));
                }
            }
        }
        float sc[kGQ][kBatchRows], vf[kBatchRows][4];
        float bm[kGQ];
#pragma unroll
        for (int jh = 0; jh < kGQ; ++jh) bm[jh] = -INFINITY;
#pragma unroll
        for (int t = 0; t < kBatchRows; ++t) {
            const int pp = p0 + b0 + cw + kCW * t;
            const bool valid = pp < p1;
            float kf[4];
            if (valid && pp == pos) {                            // this token's own row comes from shared memory
                const float4 k4 = *reinterpret_cast<const float4*>(&s.knew[lane * 4]);
                const float4 v4 = *reinterpret_cast<const float4*>(&s.vnew[lane * 4]);
                kf[0] = k4.x; kf[1] = k4.y; kf[2] = k4.z; kf[3] = k4.w;
                vf[t][0] = v4.x; vf[t][1] = v4.y; vf[t][2] = v4.z; vf[t][3] = v4.w;
            } else {
                kf[0] = bf16_lo(kreg[t].x); kf[1] = bf16_hi(kreg[t].x); kf[2] = bf16_lo(kreg[t].y); kf[3] = bf16_hi(kreg[t].y);
                vf[t][0] = bf16_lo(vreg[t].x); vf[t][1] = bf16_hi(vreg[t].x); vf[t][2] = bf16_lo(vreg[t].y); vf[t][3] = bf16_hi(vreg[t].y);
            }
#pragma unroll
            for (int jh = 0; jh < kGQ; ++jh) {
                float d = qv[jh][0] * kf[0];
                d = fmaf(qv[jh][1], kf[1], d);
                d = fmaf(qv[jh][2], kf[2], d);
                d = fmaf(qv[jh][3], kf[3], d);
                d = warp_sum(d);
                sc[jh][t] = valid ? d : -INFINITY;
                bm[jh] = fmaxf(bm[jh], sc[jh][t]);
            }
        }
#pragma unroll
        for (int jh = 0; jh < kGQ; ++jh) {
            if (bm[jh] == -INFINITY) continue;                   // no row of this warp in the batch
            const float nm = fmaxf(m[jh], bm[jh]);
            const float resc = m[jh] == -INFINITY ? 0.f : __expf(m[jh] - nm);
            l[jh] *= resc;
#pragma unroll
            for (int e = 0; e < 4; ++e) o[jh][e] *= resc;
#pragma unroll
            for (int t = 0; t < kBatchRows; ++t) {
                const float pr = sc[jh][t] == -INFINITY ? 0.f : __expf(sc[jh][t] - nm);
                l[jh] += pr;
#pragma unroll
                for (int e = 0; e < 4; ++e) o[jh][e] = fmaf(pr, vf[t][e], o[jh][e]);
            }
            m[jh] = nm;
        }
    }
#pragma unroll
    for (int jh = 0; jh < kGQ; ++jh) {
        if (lane == 0) { s.wm[cw][jh] = m[jh]; s.wl[cw][jh] = l[jh]; }
        *reinterpret_cast<float4*>(&s.wo[cw][jh][lane * 4]) = make_float4(o[jh][0], o[jh][1], o[jh][2], o[jh][3]);
    }
    consumer_sync();

    // the warps' partial (max, sum, weighted V) of this split, folded in warp order
    const int tid = cw * 32 + lane;
    const int jh = tid / kD, d = tid % kD;                       // threads 0..255: one output element each
    const bool col = tid < kGQ * kD;
    const int head = h * kGQ + (col ? jh : 0);
    constexpr int PW = kD + 2;                                   // words of a partial: kD weighted sums, max, sum
    float M = -INFINITY, num = 0.f, den = 0.f;
    if (col) {
        for (int w = 0; w < kCW; ++w) M = fmaxf(M, s.wm[w][jh]);
        for (int w = 0; w < kCW; ++w) {
            const float wgt = s.wm[w][jh] == -INFINITY ? 0.f : __expf(s.wm[w][jh] - M);
            num = fmaf(wgt, s.wo[w][jh][d], num);
            den = fmaf(wgt, s.wl[w][jh], den);
        }
        if (NS == 1) {
            st_tagged(xattn + size_t(head) * kD + d, out_tag, f32_to_bf16_bits(num / den));
        } else if (sp != 0) {                                    // handed to split 0 of this KV head as tagged words
            unsigned long long* dst = xpart + (size_t(head) * ns_max + sp) * PW;
            st_tagged64(dst + d, out_tag, num);
            if (d == 0) {
                st_tagged64(dst + kD, out_tag, M);
                st_tagged64(dst + kD + 1, out_tag, den);
            }
        }
    }
    if (NS > 1 && sp == 0) {
        // Split 0 merges.  Every word it needs is requested at once and polled until its tag is this phase's: one
        // trip through L2 after the last split has written, with no fence and no ticket on the way.  The other
        // splits' columns are dealt over all 384 threads -- thread (pair of columns, third of the splits) -- so
        // that a thread holds at most kMergeLoads 16-byte loads in registers.
        const int others = NS - 1;
        const int pr = tid & 127, g = tid >> 7;                  // pr: head pr / 64, columns 2 * (pr % 64) and the next
        const int pj = pr >> 6, pd = (pr & 63) * 2;
        const unsigned long long* src = xpart + (size_t(h * kGQ + pj) * ns_max) * PW + pd;
        ulonglong2 nv[kMergeLoads];
        auto split_of = [others, g](int i) { return min(1 + g + 3 * i, others); };      // (clamped: re-reads the last one)
#pragma unroll
        for (int i = 0; i < kMergeLoads; ++i) nv[i] = ld_relaxed64x2(src + size_t(split_of(i)) * PW);
        if (tid < kGQ * others * 2) {                            // (max, sum) of the other splits: one word per thread
            const int j2 = tid / (others * 2), rem = tid % (others * 2), q = 1 + (rem >> 1), which = rem & 1;
            const unsigned long long* a = xpart + (size_t(h * kGQ + j2) * ns_max + q) * PW + kD + which;
            unsigned long long w;
            int spins = 0;
            for (;;) {
                w = ld_relaxed64(a);
                if (unsigned(w >> 32) == out_tag || poll_expired(s, spins, p.status, 0x800u)) break;
            }
            (which ? s.mrg_l : s.mrg_m)[j2][q] = __uint_as_float(unsigned(w));
        }
        if (col && d == 0) { s.mrg_m[jh][0] = M; s.mrg_l[jh][0] = den; }
        consumer_sync();                                         // (also: every thread is done with s.wo)
        float gm = -INFINITY;
        for (int q = 0; q < NS; ++q) gm = fmaxf(gm, s.mrg_m[pj][q]);
        float t0 = 0.f, t1 = 0.f;
        for (int i0 = 0; 1 + g + 3 * i0 <= others; i0 += kMergeLoads) {
            if (i0 > 0) {                                        // more splits than one batch holds
#pragma unroll
                for (int i = 0; i < kMergeLoads; ++i) nv[i] = ld_relaxed64x2(src + size_t(split_of(i0 + i)) * PW);
            }
            int spins = 0;
            for (;;) {                                           // until the whole batch carries this phase's tag
                bool ok = true;
#pragma unroll
                for (int i = 0; i < kMergeLoads; ++i)
                    ok = ok && unsigned(nv[i].x >> 32) == out_tag && unsigned(nv[i].y >> 32) == out_tag;
                if (ok || poll_expired(s, spins, p.status, 0x800u)) break;
#pragma unroll
                for (int i = 0; i < kMergeLoads; ++i) nv[i] = ld_relaxed64x2(src + size_t(split_of(i0 + i)) * PW);
            }
#pragma unroll
            for (int i = 0; i < kMergeLoads; ++i) {
                const int q = 1 + g + 3 * (i0 + i);
                if (q <= others) {
                    const float wq = __expf(s.mrg_m[pj][q] - gm);
                    t0 = fmaf(wq, __uint_as_float(unsigned(nv[i].x)), t0);
                    t1 = fmaf(wq, __uint_as_float(unsigned(nv[i].y)), t1);
                }
            }
        }
        float* acc = &s.wo[0][0][0];                             // [3][kGQ][kD]
        *reinterpret_cast<float2*>(acc + (g * kGQ + pj) * kD + pd) = make_float2(t0, t1);
        consumer_sync();
        if (col) {
            float gmc = -INFINITY, td = 0.f;
            for (int q = 0; q < NS; ++q) gmc = fmaxf(gmc, s.mrg_m[jh][q]);
            for (int q = 0; q < NS; ++q) td = fmaf(__expf(s.mrg_m[jh][q] - gmc), s.mrg_l[jh][q], td);
            const float tn = fmaf(__expf(M - gmc), num, acc[(0 * kGQ + jh) * kD + d] + acc[(1 * kGQ + jh) * kD + d] + acc[(2 * kGQ + jh) * kD + d]);
            st_tagged(xattn + size_t(head) * kD + d, out_tag, f32_to_bf16_bits(tn / td));
        }
    }
    consumer_sync();                                             // (s.wo is the next phase's activation staging)
    if (tid == 0) tl_done(p, ph);
}

__global__ void __launch_bounds__(kFusedThreads, 1) qwen3_step_kernel(const FusedParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    FusedSmem& s = *reinterpret_cast<FusedSmem*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x, G = gridDim.x;
    const int pos = *p.pos;
    if (pos < 0 || pos >= p.max_ctx) return;                      // (uniform over the grid: nothing waits on anything)
    if (p.stop_at != nullptr && *p.stop_at != 0) return;          // the sequence met an end token: the step is a no-op
    const int H = p.hidden, L = p.n_layers, QP = p.hq * kD, NQKV = (p.hq + 2 * p.hkv) * kD;
    const int per_layer = 5 + p.hkv;                               // (a layer's words: unused since hand-overs travel with the data)
    unsigned* const glob = p.sync + L * per_layer;                 // [1] head pairs written, [2] exit tickets, [3] launch counter
    // tags: launch counter * phases + phase, mod 65535, + 1 (phase 0 embedding, 1 + 5*layer + {0..4}, then the head)
    const unsigned epoch = glob[3];                                // written by the previous launch's last CTA
    const unsigned tag_base = unsigned((unsigned long long)epoch * unsigned(5 * L + 2) % 65535ull);
    auto tag = [tag_base](int ph) { return (tag_base + unsigned(ph)) % 65535u + 1u; };
    unsigned* const xh = p.xbuf;                                   // tagged activations: hidden | q|k|v | attention | MLP inner
    unsigned* const xqkv = xh + H;
    unsigned* const xattn = xqkv + NQKV;
    unsigned* const xact = xattn + QP;
    unsigned long long* const xpart = reinterpret_cast<unsigned long long*>(xact + ((p.inter + 1) & ~1));   // split partials

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) { mb_init(&s.full[i], 1); mb_init(&s.empty[i], kMmaThreads); }
        for (int i = 0; i < kAccBufs; ++i) { mb_init(&s.acc_full[i], kMmaThreads); mb_init(&s.acc_empty[i], kEpiWarps); }
        mb_init(&s.mma_done, kMmaThreads);
        s.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1 + kMmaWarp) {                                     // tensor memory for the accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(s_u32(&s.tmem_base)), "n"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp == 0) {
        // ---- producer: every weight tile of the step, in consumption order (lane r: row r of every tile) ----
        RingPos rp{0, 0};
        for (int l = 0; l < L; ++l) {
            const FusedLayer Ly = p.layers[l];
            produce(s, rp, Ly.w_qkv, nullptr, NQKV, H, c, G, lane, p.status);
            produce(s, rp, Ly.w_o, nullptr, H, QP, c, G, lane, p.status);
            produce(s, rp, Ly.w_gate, Ly.w_up, p.inter, H, c, G, lane, p.status);
            produce(s, rp, Ly.w_down, nullptr, H, p.inter, c, G, lane, p.status);
        }
        produce(s, rp, p.w_head, nullptr, p.vocab, H, c, G, lane, p.status);
        return;
    }

    // ---- consumers ----
    const int cw = warp - 1;
    const int tid = cw * 32 + lane;
    RingPos rp{0, 0};
    AccPos ap{0, 0};
    {   // where this CTA's attention rows sit in every layer's pools (same split arithmetic as attend())
        const int total = pos + 1, ns_max = min(G / p.hkv, 64);
        const int SL = max(16, ((total + ns_max - 1) / ns_max + 15) & ~15), NS = (total + SL - 1) / SL;
        const int h = c % p.hkv, sp = c / p.hkv;
        const bool active = sp < NS && c < p.hkv * ns_max;
        const int p0 = sp * SL, p1 = min(p0 + SL, total);
        if (lane < kBatchRows) {
            const int pp = p0 + cw + kCW * lane;
            s.koff[cw][lane] = (active && pp < p1 && pp < pos) ? unsigned(kv_offset(p, pp, h)) : ~0u;
        }
        if (tid == 0) s.new_off = (active && sp == NS - 1) ? unsigned(kv_offset(p, pos, h)) : 0u;
    }
    {   // the embedding row of this step's token, dealt like the rows of the projections that update it
        long long id = p.tokens[pos];
        id = id < 0 ? 0 : (id >= p.vocab ? p.vocab - 1 : id);
        int u0, u1;
        span(H, c, G, u0, u1);
        for (int i = u0 + tid; i < u1; i += kCT) st_tagged(xh + i, tag(0), p.w_embed[size_t(id) * H + i]);
        if (tid == 0) tl_done(p, 0);
    }
    int hidden_ph = 0;                                             // the phase that wrote the current hidden state
    consumer_sync();                                               // (s.koff is read across warps below)
    ask_cache_rows(s, p.layers[0], cw, lane);
    for (int l = 0; l < L; ++l) {
        const FusedLayer& Ly = p.layers[l];
        const int ph = 1 + 5 * l;
        consume<kStore, true>(s, rp, ap, p, NQKV, H, xh, tag(hidden_ph), Ly.gamma_in, xqkv, tag(ph), nullptr, nullptr,
                              c, G, cw, lane, nullptr, ph);
        attend(s, p, Ly, xqkv, tag(ph), xattn, tag(ph + 1), xpart, pos, c, G, cw, lane, ph + 1);
        consume<kResidual, false>(s, rp, ap, p, H, QP, xattn, tag(ph + 1), nullptr, xh, tag(ph + 2), nullptr, nullptr,
                                  c, G, cw, lane, nullptr, ph + 2);
        consume<kSwiglu, true>(s, rp, ap, p, p.inter, H, xh, tag(ph + 2), Ly.gamma_post, xact, tag(ph + 3), nullptr, nullptr,
                               c, G, cw, lane, nullptr, ph + 3);
        if (l + 1 < L) ask_cache_rows(s, p.layers[l + 1], cw, lane);   // (two phases and two hand-overs ahead of its use)
        consume<kResidual, false>(s, rp, ap, p, H, p.inter, xact, tag(ph + 3), nullptr, xh, tag(ph + 4), nullptr,
                                  p.hidden_trace ? p.hidden_trace + size_t(l) * H : nullptr, c, G, cw, lane, nullptr, ph + 4);
        hidden_ph = ph + 4;
    }
    HeadBest best{-INFINITY, 0x7fffffff};
    consume<kHead, true>(s, rp, ap, p, p.vocab, H, xh, tag(hidden_ph), p.gamma_final, nullptr, 0u, p.logits,
                         p.hidden_trace ? p.hidden_trace + size_t(L) * H : nullptr, c, G, cw, lane, &best, 1 + 5 * L);
    if (cw > kMmaWarp && cw < kMmaWarp + kMmaThreads && lane == 0) umma_arrive(&s.mma_done);
    if (cw == kMmaWarp) {
        // Tensor memory goes back once nothing can touch it: the head phase's last barrier is behind every consumer, and
        // every MMA this CTA issued has completed (after a timeout some may still be in flight: wait for them, bounded).
        if (lane == 0) {
            umma_arrive(&s.mma_done);
            const unsigned long long t0 = global_ns();
            while (!mb_try(&s.mma_done, 0u) && global_ns() - t0 < kWaitNs) {}
        }
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(s.tmem_base), "n"(kTmemCols) : "memory");
    }
    if (cw < kEpiWarps) {                                           // each epilogue warp's (best logit, lowest index)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best.v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best.i, o);
            if (ov > best.v || (ov == best.v && oi < best.i)) { best.v = ov; best.i = oi; }
        }
        if (lane == 0) { s.head_v[cw] = best.v; s.head_i[cw] = best.i; }
    }
    consumer_sync();
    if (cw == 0) {
        // this CTA's best, then the pick over all CTAs by CTA 0
        best.v = s.head_v[0];
        best.i = s.head_i[0];
#pragma unroll
        for (int q = 1; q < kEpiWarps; ++q) {
            const float ov = s.head_v[q];
            const int oi = s.head_i[q];
            if (ov > best.v || (ov == best.v && oi < best.i)) { best.v = ov; best.i = oi; }
        }
        if (lane == 0) {
            p.head_val[c] = best.v;
            p.head_idx[c] = best.i;
            arrive(&glob[1]);
        }
        if (c == 0) {
            if (lane == 0) wait_count(s, &glob[1], unsigned(G), p.status, 0x400u);
            __syncwarp();
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int q = lane; q < G; q += 32) {
                const float ov = __ldcg(p.head_val + q);
                const int oi = __ldcg(p.head_idx + q);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) {
                if (p.picked) *p.picked = bi;
                if (pos + 1 < p.max_tokens) {
                    if (pos + 1 >= p.n_prompt) {
                        p.tokens[pos + 1] = bi;
                        for (int e = 0; e < p.n_eos; ++e)
                            if (p.eos_ids[e] == (long long)bi) *p.stop_at = pos + 1;
                    }
                    *p.pos = pos + 1;
                }
            }
        }
        // the last CTA to leave puts every counter back to zero for the next launch
        if (lane == 0) s.flag = atomicAdd(&glob[2], 1u) == unsigned(G - 1);
        __syncwarp();
        if (s.flag) {
            __threadfence();
            for (int i = lane; i < L * per_layer + 3; i += 32) p.sync[i] = 0u;
            if (lane == 0) glob[3] = epoch + 1u;
        }
    }
}

}  // namespace

int fused_step_sync_words(int n_layers, int hkv) { return n_layers * (5 + hkv) + 4; }
long long fused_step_xbuf_words(int hidden, int hq, int hkv, int d, int inter) {
    const long long vectors = (long long)hidden + (long long)(hq + 2 * hkv) * d + (long long)hq * d + ((inter + 1) & ~1);
    return vectors + 2ll * hq * fused_step_splits(hkv) * (d + 2);       // + the split partials as 64-bit words
}
int fused_step_splits(int hkv) { const int s = sm_count() / (hkv > 0 ? hkv : 1); return s < 64 ? s : 64; }

bool fused_step_supported(const FusedParams& p) {
    const int QP = p.hq * kD;
    // (k <= 6144: an activation vector is staged as bf16 in the 12 KB attention scratch, four 16-byte pieces per thread)
    auto ok_k = [](int k) { return k >= kSliceLen && k % kSliceLen == 0 && k <= 4 * 4 * kCT; };
    const int G = sm_count();
    return p.n_layers >= 1 && p.n_layers <= kFusedMaxLayers && p.d == kD && p.hkv >= 1 && p.hq == kGQ * p.hkv &&
           ok_k(p.hidden) && ok_k(QP) && ok_k(p.inter) &&
           p.hidden <= 32 * G && p.hkv <= G && p.inter >= 1 && p.vocab >= 1 && p.xbuf != nullptr;
}

cudaError_t fused_step_launch(const FusedParams& p, cudaStream_t stream) {
    if (!fused_step_supported(p)) return cudaErrorInvalidValue;
    const size_t smem = sizeof(FusedSmem);
    static PerDeviceOnce once;
    if (once.first()) {
        cudaError_t e = cudaFuncSetAttribute(qwen3_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count());
    cfg.blockDim = dim3(kFusedThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;               // every CTA resident: they wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, qwen3_step_kernel, p);
}

}  // namespace tfb
