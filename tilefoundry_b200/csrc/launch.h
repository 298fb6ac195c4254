// Host-side launch helper: one place that sets the programmatic-dependent-launch
// attribute, so every kernel in a decode step can overlap its weight prefetch with
// the tail of the kernel before it.
#pragma once
#include <cuda_runtime.h>

namespace tfb {

constexpr int kMaxDevices = 64;

// Function attributes (dynamic shared memory opt-in, carve-out) belong to a device: a process that drives several
// GPUs has to set them on each.  `first()` is true the first time it is asked with a given device current.
struct PerDeviceOnce {
    bool done[kMaxDevices] = {};
    bool first() {
        int d = 0;
        if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return true;
        if (done[d]) return false;
        done[d] = true;
        return true;
    }
};

// Multiprocessor count of the current device, asked once per device.
inline int sm_count() {
    static int n[kMaxDevices] = {};
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return 148;
    if (n[d] == 0) {
        if (cudaDeviceGetAttribute(&n[d], cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n[d] <= 0) n[d] = 148;
    }
    return n[d];
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

}  // namespace tfb
