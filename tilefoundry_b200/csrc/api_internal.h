// Helpers shared by the translation units that implement the C ABI.
#pragma once
#include "../../include/tfb200.h"
#include <cuda_runtime.h>
#include <stdint.h>

namespace tfb { namespace host {

int fail_launch(cudaError_t e);                 // records the text, returns TFB_ELAUNCH
unsigned long long* next_trace();               // next debug-timeline record or nullptr
int gemv_checked(const tfb_gemv_args* a, tfb_stream_t stream);

inline int done(cudaError_t e) { return e == cudaSuccess ? TFB_OK : fail_launch(e); }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline cudaStream_t S(tfb_stream_t s) { return static_cast<cudaStream_t>(s); }

} }  // namespace tfb::host

#define TFB_REQUIRE(cond, code)      \
    do {                             \
        if (!(cond)) return (code);  \
    } while (0)
