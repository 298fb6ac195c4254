// The two exchange steps of the sharded MoE decode step, each as ONE kernel over NVLink peer memory instead of
// an NCCL collective followed by a finishing kernel:
//
//  * moe_allreduce_finalize_kernel: every rank holds the un-rounded partial sums of its experts / its slice of the
//    shared expert ([2][hidden] f32).  A CTA PUSHES its 256-element slice into every peer's inbox with plain peer
//    stores, publishes an epoch flag (st.release.sys) in the peer's memory, waits for the peers' flags in its OWN
//    memory (so the polling never crosses NVLink), adds the inboxes in rank order (every rank computes the same
//    sum) and applies the roundings of routed_experts / experts / residual_add.  One NVLink traversal on the
//    critical path; NCCL's launch + protocol for 32 KB measured ~20 us per MoE block inside a captured step.
//  * pick_allgather_kernel: the same pattern for the (best logit, index) pairs of the vocabulary-parallel head.
//
// Inboxes are double-buffered by epoch parity: a peer can write epoch e+2 only after it has seen this rank's
// flag for e+1, which is published after the reads of epoch e.  Every CTA slice has its own flag and its own
// epoch counter, so there is no grid-wide coordination.  Every wait is bounded; a timeout sets *status.
// No multimem, no TMA: plain loads and stores on peer pointers.
#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace tfb {

// A peer's flag is waited for at most this long (a healthy exchange takes microseconds); the clock is read every
// 64th poll, and a poll count bounds the loop as well should the clock not advance.
constexpr unsigned long long kPeerWaitNs = 1000ull * 1000 * 1000;
constexpr unsigned kPeerSpinLimit = 1u << 24;

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// wait until *flag has reached epoch (epochs only grow; the comparison is wrap-safe)
__device__ __forceinline__ bool wait_epoch(const unsigned* flag, unsigned epoch) {
    unsigned long long t0 = 0;
    for (unsigned spin = 0; spin < kPeerSpinLimit; ++spin) {
        if (int(ld_acquire_sys(flag) - epoch) >= 0) return true;
        __nanosleep(40);
        if ((spin & 63u) == 63u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > kPeerWaitNs) return false;
        }
    }
    return false;
}

__global__ void __launch_bounds__(256) moe_allreduce_finalize_kernel(const PeerReduceParams p) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x, tid = threadIdx.x, j = b * 256 + tid, H = p.hidden, W = p.world;
    const unsigned e = p.epoch[b] + 1;
    const int parity = e & 1;
    const bool live = j < H;
    const float mine_r = live ? p.partial[j] : 0.f, mine_s = live ? p.partial[H + j] : 0.f;
    for (int r = 0; r < W; ++r) {
        if (r == p.rank || !live) continue;
        float* box = p.inbox[r] + size_t(parity * W + p.rank) * 2 * H;          // my slot in rank r's inbox
        box[j] = mine_r;
        box[H + j] = mine_s;
    }
    __threadfence_system();
    __syncthreads();
    if (tid < W && tid != p.rank) {
        st_release_sys(p.flags[tid] + p.rank * gridDim.x + b, e);                // "slice b of epoch e from me has landed"
        if (!wait_epoch(p.flags[p.rank] + tid * gridDim.x + b, e)) atomicExch(p.status, 0x200u + tid);
    }
    __syncthreads();
    if (live) {
        float routed = 0.f, shared = 0.f;
        const float* boxes = p.inbox[p.rank] + size_t(parity * W) * 2 * H;
        for (int r = 0; r < W; ++r) {                                            // rank order: the same sum on every rank
            routed += (r == p.rank) ? mine_r : __ldcg(boxes + size_t(r) * 2 * H + j);
            shared += (r == p.rank) ? mine_s : __ldcg(boxes + size_t(r) * 2 * H + H + j);
        }
        if (p.out_f32) {                                                         // f32 activations (Qwen3.5)
            float sh = round_bf16(shared);
            if (p.gate_logit) sh *= 1.f / (1.f + expf(-*p.gate_logit));
            p.out_f32[j] = (p.residual_f32 ? p.residual_f32[j] : 0.f) + (routed + sh);
        } else {
            float v = round_bf16(routed);
            if (p.has_shared) v = round_bf16(v + round_bf16(shared));
            if (p.residual) v = bf16_bits_to_f32(p.residual[j]) + round_bf16(v * p.res_scale);
            p.out[j] = f32_to_bf16_bits(v);
        }
    }
    if (tid == 0) p.epoch[b] = e;
}

cudaError_t moe_allreduce_finalize_launch(const PeerReduceParams& p, cudaStream_t stream, bool pdl) {
    return launch_kernel(moe_allreduce_finalize_kernel, dim3((p.hidden + 255) / 256), dim3(256), 0, stream, pdl, p);
}

__global__ void __launch_bounds__(32) pick_allgather_kernel(const PeerPickParams p) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x, W = p.world;
    const unsigned e = p.epoch[0] + 1;
    const int parity = e & 1;
    const float my_v = p.pair[0], my_i = p.pair[1];
    if (lane < W && lane != p.rank) {
        float* box = p.inbox[lane] + size_t(parity * W + p.rank) * 2;
        box[0] = my_v;
        box[1] = my_i;
        __threadfence_system();
        st_release_sys(p.flags[lane] + p.rank, e);
        if (!wait_epoch(p.flags[p.rank] + lane, e)) atomicExch(p.status, 0x300u + lane);
    }
    __syncwarp();
    if (lane == 0) {
        float best = -INFINITY;
        long long best_i = 0x7fffffff;
        const float* boxes = p.inbox[p.rank] + size_t(parity * W) * 2;
        for (int r = 0; r < W; ++r) {
            const float v = (r == p.rank) ? my_v : __ldcg(boxes + 2 * r);
            const long long i = (long long)((r == p.rank) ? my_i : __ldcg(boxes + 2 * r + 1));
            if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
        }
        if (p.picked) *p.picked = best_i;
        if (p.tokens && p.pos) {
            const int cur = *p.pos;
            if (cur + 1 < p.max_tokens) {
                if (cur + 1 >= p.n_prompt) p.tokens[cur + 1] = best_i;
                *p.pos = cur + 1;
            }
        }
        p.epoch[0] = e;
    }
}

cudaError_t pick_allgather_launch(const PeerPickParams& p, cudaStream_t stream, bool pdl) {
    return launch_kernel(pick_allgather_kernel, dim3(1), dim3(32), 0, stream, pdl, p);
}

}  // namespace tfb
