// Small-batch projection on the 5th-generation tensor cores: Y[M, N] = X[M, K] . W[N, K]^T (+ residual) for
// M <= 32 tokens, bf16 in, f32 accumulate, bf16 out.
//
// At batch 32 a projection is still HBM-bound (64 flop per weight byte against a ridge near 290), but the
// CUDA cores can no longer keep up with the weight stream (it would need ~200 TFLOP/s of FMA), so the
// products move to tcgen05.mma with the operands swapped: the WEIGHT tile is the MMA's 128-row A operand
// and the token block its N = 32 B operand, both K-major in shared memory, the 128 x 32 f32 accumulator in
// tensor memory.  The weight stream is what matters: a producer thread keeps TC_STAGES TMA tiles of
// 128 rows x 64 columns (16 KB, 128-byte swizzle) in flight per CTA, two CTAs per SM (one fills its ring while the
// other streams), completion counted by mbarriers.
//
// Roles in a CTA of 6 warps: warp 0 (one lane) issues TMA loads; warp 1 allocates tensor memory and (one lane)
// issues the MMAs, four per stage (K = 16 each), releasing a stage with tcgen05.commit; warps 2-5 read the
// accumulator back (tcgen05.ld, one TMEM lane quadrant each) and write it out.  K is split over the 1, 2, 4 or 8
// CTAs of a thread-block cluster so that a 2048 x 2048 projection (16 row tiles) still reaches most SMs.  The
// splits' f32 partials never leave the chip: every CTA parks its 128 x 32 tile in its own shared memory, and
// after a cluster barrier CTA c adds, in fixed split order (deterministic), the 32/S token rows it owns from all
// S CTAs through distributed shared memory and writes them out.
//
// SwiGLU form (p.swiglu): a row tile holds 64 gate rows and the 64 up rows of the same outputs (two 64-row TMA
// boxes from a [gate; up] matrix), so one accumulator carries both halves; the up half crosses to the gate half's
// threads through shared memory and y = bf16(silu(bf16 g)) * bf16 u is written, rounding as the batch-1 epilogue.
//
// The weight tiles of the first ring pass do not depend on the kernel before: the producer requests them before
// griddepcontrol.wait and only the token tiles after it.
//
// Every mbarrier wait is bounded; a timeout sets *status, and the CTA still frees its tensor memory.
//
// HBM-bound: algorithmic bytes per launch = N*K*2 (weights) + M*K*2 per row tile from L2.
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

#include <cuda.h>

namespace tfb {

constexpr int TC_BM = 128, TC_BN = 32, TC_BK = 64, TC_STAGES = 5, TC_THREADS = 192;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2, TC_B_BYTES = TC_BN * TC_BK * 2;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase of the given parity; false if it gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < TC_WAIT_LIMIT; ++spin) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* tile) {
    uint64_t d = 0;
    d |= uint64_t((smem_u32(tile) & 0x3FFFF) >> 4);          // start address, 16-byte units
    d |= uint64_t(1) << 16;                                   // leading-dimension byte offset: unused with swizzle
    d |= uint64_t(1024 >> 4) << 32;                           // stride-dimension byte offset: one 8-row group
    d |= uint64_t(1) << 46;                                   // descriptor version of this architecture
    d |= uint64_t(2) << 61;                                   // 128-byte swizzle
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}

struct TcSmemTail {
    uint64_t full[TC_STAGES], empty[TC_STAGES], accum;
    uint32_t tmem_base;
    int aborted;
    float exch[64][33];                                                 // SwiGLU, unsplit: the up half of a finished tile
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;\nbarrier.cluster.wait.acquire;" ::: "memory");
}
// 16 bytes of CTA `rank`'s shared memory at the address `local` has in this CTA's window
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}

// The finished f32 sums of tile row r (0..127) for the M tokens -> y (unsplit launch).  Called by all 128
// epilogue threads.
__device__ __forceinline__ void tc_finish_row(const TcParams& p, TcSmemTail* t, int tile, int r, const float (&acc)[32]) {
    if (p.swiglu) {
        if (r >= 64) {
#pragma unroll
            for (int m = 0; m < 32; ++m) t->exch[r - 64][m] = acc[m];
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");                  // the four epilogue warps only
        const int j = tile * 64 + r;
        if (r < 64 && j < p.N) {
#pragma unroll
            for (int m = 0; m < 32; ++m)
                if (m < p.M) {
                    const float g = round_bf16(acc[m]), u = round_bf16(t->exch[r][m]);
                    p.y[size_t(m) * p.N + j] = f32_to_bf16_bits(round_bf16(silu_f32(g)) * u);
                }
        }
        return;
    }
    const int n = tile * TC_BM + r;
    if (n >= p.N) return;
#pragma unroll
    for (int m = 0; m < 32; ++m)
        if (m < p.M) {
            float o = acc[m];
            if (p.residual) {                              // TFB_EPI_RESIDUAL's rounding: bf16(acc), bf16(. * scale), then the add
                float t = round_bf16(acc[m]);
                if (p.res_scale != 1.f) t = round_bf16(t * p.res_scale);
                o = bf16_bits_to_f32(p.residual[size_t(m) * p.N + n]) + t;
            }
            p.y[size_t(m) * p.N + n] = f32_to_bf16_bits(o);
        }
}

// Split launch: token row m, tile rows 4q .. 4q+3 summed over the splits -> y.  Called by whole warps (the SwiGLU
// form moves the up half to the gate half's lanes by shuffle: lane q holds gate rows 4q.., lane q + 16 the up rows
// of the same outputs).
__device__ __forceinline__ void tc_finish_quad(const TcParams& p, int tile, int m, int q, float4 acc) {
    const float a[4] = {acc.x, acc.y, acc.z, acc.w};
    if (p.swiglu) {
        float u[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) u[i] = __shfl_down_sync(0xffffffffu, a[i], 16);
        if (q < 16 && m < p.M) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j = tile * 64 + 4 * q + i;
                if (j < p.N)
                    p.y[size_t(m) * p.N + j] = f32_to_bf16_bits(round_bf16(silu_f32(round_bf16(a[i]))) * round_bf16(u[i]));
            }
        }
        return;
    }
    if (m >= p.M) return;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int n = tile * TC_BM + 4 * q + i;
        if (n < p.N) {
            float o = a[i];
            if (p.residual) {
                float t = round_bf16(a[i]);
                if (p.res_scale != 1.f) t = round_bf16(t * p.res_scale);
                o = bf16_bits_to_f32(p.residual[size_t(m) * p.N + n]) + t;
            }
            p.y[size_t(m) * p.N + n] = f32_to_bf16_bits(o);
        }
    }
}

__global__ void __launch_bounds__(TC_THREADS, 2) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x, const TcParams p) {
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* a_tiles = base;                                      // TC_STAGES x 16 KB, 1024-byte aligned
    unsigned char* b_tiles = base + TC_STAGES * TC_A_BYTES;             // TC_STAGES x 4 KB
    TcSmemTail* t = reinterpret_cast<TcSmemTail*>(b_tiles + TC_STAGES * TC_B_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = p.splits > 1 ? int(cluster_ctarank()) : 0;
    const int per = (p.ksteps + p.splits - 1) / p.splits;
    const int k_begin = split * per, k_end = min(p.ksteps, k_begin + per);
    const int nsteps = max(k_end - k_begin, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&t->full[s], 1); mbar_init(&t->empty[s], 1); }
        mbar_init(&t->accum, 1);
        t->aborted = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                                    // 32 columns of tensor memory: the 128 x 32 f32 tile
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&t->tmem_base)), "r"(32u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = t->tmem_base;
    pdl_trigger();
    const bool producer = (warp == 0 && lane == 0);
    if (!producer) pdl_wait();

    if (warp == 0) {
        if (lane == 0) {                                                // ---- TMA producer ----
            auto load_w = [&](int i, int s) {
                const int kx = (k_begin + i) * TC_BK;
                if (p.swiglu) {                                         // 64 gate rows, then the 64 up rows of the same outputs
                    tma_load_2d(a_tiles + s * TC_A_BYTES, &map_w, &t->full[s], kx, tile * 64);
                    tma_load_2d(a_tiles + s * TC_A_BYTES + TC_A_BYTES / 2, &map_w, &t->full[s], kx, p.N + tile * 64);
                } else {
                    tma_load_2d(a_tiles + s * TC_A_BYTES, &map_w, &t->full[s], kx, tile * TC_BM);
                }
            };
            const int pre = min(nsteps, TC_STAGES);
            for (int i = 0; i < pre; ++i) {                             // weights never depend on the kernel before
                mbar_expect_tx(&t->full[i], TC_A_BYTES + TC_B_BYTES);
                load_w(i, i);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i)
                tma_load_2d(b_tiles + i * TC_B_BYTES, &map_x, &t->full[i], (k_begin + i) * TC_BK, 0);
            for (int i = pre; i < nsteps; ++i) {
                const int s = i % TC_STAGES;
                if (!mbar_wait(&t->empty[s], ((i / TC_STAGES) & 1) ^ 1)) { t->aborted = 1; atomicExch(p.status, 1u); break; }
                mbar_expect_tx(&t->full[s], TC_A_BYTES + TC_B_BYTES);
                load_w(i, s);
                tma_load_2d(b_tiles + s * TC_B_BYTES, &map_x, &t->full[s], (k_begin + i) * TC_BK, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                                // ---- MMA issuer ----
            // instruction descriptor: D f32, A and B bf16, both K-major, N = 32, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(TC_BN >> 3) << 17) | (uint32_t(TC_BM >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < nsteps && ok; ++i) {
                const int s = i % TC_STAGES;
                ok = mbar_wait(&t->full[s], (i / TC_STAGES) & 1);
                if (!ok) { t->aborted = 1; atomicExch(p.status, 2u); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = umma_desc_sw128(a_tiles + s * TC_A_BYTES), db = umma_desc_sw128(b_tiles + s * TC_B_BYTES);
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk)                 // 16 bf16 = 32 bytes = 2 descriptor units per step
                    umma_bf16(tmem, da + 2 * kk, db + 2 * kk, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&t->empty[s]);                              // arrives when these MMAs have read the stage
            }
            if (ok) umma_commit(&t->accum);                             // arrives when the accumulator is complete
        }
    } else {                                                            // ---- epilogue: warps 2..5 ----
        const int quad = warp & 3;                                      // the TMEM lane quadrant this warp may read
        bool ok = nsteps > 0 ? mbar_wait(&t->accum, 0) : true;
        if (!ok) { t->aborted = 1; atomicExch(p.status, 3u); }
        uint32_t v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
        if (ok && nsteps > 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem + (uint32_t(quad * 32) << 16);
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                         "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                         "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                         : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                           "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                           "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                           "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                         : "r"(taddr) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        }
        if (p.splits == 1) {
            float acc[32];
#pragma unroll
            for (int m = 0; m < 32; ++m) acc[m] = __uint_as_float(v[m]);
            tc_finish_row(p, t, tile, quad * 32 + lane, acc);
        } else {
            // park this split's tile as red[m][r] in the first weight stage: every load into it has landed and
            // every MMA that read it has completed once the accumulator barrier fires
            float* red = reinterpret_cast<float*>(a_tiles);
#pragma unroll
            for (int m = 0; m < 32; ++m) red[m * TC_BM + quad * 32 + lane] = __uint_as_float(v[m]);
        }
    }

    // ---- teardown, and the split-K reduction through distributed shared memory ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(32u) : "memory");
    }
    if (p.splits > 1) {
        cluster_sync_all();                                             // every split's tile is parked
        if (warp >= 2) {
            const int tq = threadIdx.x - 64, q = tq & 31, mg = tq >> 5; // 4 token rows at a time, 32 row quads each
            const int m_per = 32 / p.splits;                            // token rows this CTA finishes (>= 4)
            const uint32_t red = smem_u32(a_tiles);
            for (int j = 0; j < m_per; j += 4) {
                const int m = split * m_per + j + mg;
                const uint32_t local = red + uint32_t((m * TC_BM + 4 * q) * 4);
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                float4 part[8];
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    if (s < p.splits) part[s] = ld_dsmem_f4(local, uint32_t(s));
#pragma unroll
                for (int s = 0; s < 8; ++s)                             // fixed order
                    if (s < p.splits) { acc.x += part[s].x; acc.y += part[s].y; acc.z += part[s].z; acc.w += part[s].w; }
                tc_finish_quad(p, tile, m, q, acc);
            }
        }
        cluster_sync_all();                                             // nobody leaves while its tile is still being read
    }
}

// ---- host side: tensor maps and launch ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

static bool make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(cols) * 2};
    const cuuint32_t box[2] = {cuuint32_t(TC_BK), cuuint32_t(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int splits_for_tiles(int tiles, int k);
int gemm_tc_splits(int n, int k) { return splits_for_tiles((n + TC_BM - 1) / TC_BM, k); }
int gemm_tc_splits_swiglu(int n, int k) { return splits_for_tiles((n + 63) / 64, k); }
// K splits = CTAs of one cluster: the largest power of two (at most 8, the portable cluster size) that keeps the
// grid within the two CTAs an SM holds.
static int splits_for_tiles(int tiles, int k) {
    const int sms = sm_count();
    const int ksteps = k / TC_BK;
    int splits = 1;
    while (splits < 8 && tiles * splits * 2 <= 2 * sms && ksteps % (splits * 2) == 0) splits *= 2;
    return splits;
}

cudaError_t gemm_tc_launch(const void* w, const void* x, TcParams p, cudaStream_t stream, bool pdl) {
    CUtensorMap map_w, map_x;
    const int w_rows = p.swiglu ? 2 * p.N : p.N;
    if (!make_map(&map_w, w, w_rows, p.K, p.swiglu ? 64 : TC_BM) || !make_map(&map_x, x, p.M, p.K, TC_BN))
        return cudaErrorInvalidValue;
    p.ksteps = p.K / TC_BK;
    const int tiles = p.swiglu ? (p.N + 63) / 64 : (p.N + TC_BM - 1) / TC_BM;
    const size_t smem = 1024 + size_t(TC_STAGES) * (TC_A_BYTES + TC_B_BYTES) + sizeof(TcSmemTail);
    static PerDeviceOnce once;
    if (once.first()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;}
    const dim3 grid(tiles, p.splits), block(TC_THREADS);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (p.splits > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = unsigned(p.splits);
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, gemm_tc_kernel, map_w, map_x, p);
}

}  // namespace tfb
