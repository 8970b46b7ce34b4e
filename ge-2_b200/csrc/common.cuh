// Shared helpers for the sm_100a kernels behind the C ABI in include/ge2_b200.h.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../include/ge2_b200.h"

namespace ge2 {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids of streaming kernels are sized in multiples of this

extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e, const char* what = nullptr, const char* file = nullptr, int line = 0) {
    g_last_cuda_error = (int)e;
    if (what != nullptr && getenv("GE2_DEBUG_ERRORS") != nullptr)
        fprintf(stderr, "[ge2] %s failed with cudaError %d (%s) at %s:%d\n", what, (int)e, cudaGetErrorString(e), file, line);
    return GE2_ERR_CUDA;
}

// GE2_DEBUG_ERRORS=1 in the environment: the failing call site is printed to stderr before the status is returned
#define GE2_CUDA_TRY(expr)                                                          \
    do {                                                                            \
        cudaError_t _e = (expr);                                                    \
        if (_e != cudaSuccess) return ::ge2::cuda_fail(_e, #expr, __FILE__, __LINE__); \
    } while (0)

#define GE2_LAUNCH_CHECK()                                                                  \
    do {                                                                                    \
        cudaError_t _e = cudaGetLastError();                                                \
        if (_e != cudaSuccess) return ::ge2::cuda_fail(_e, "kernel launch", __FILE__, __LINE__); \
    } while (0)

inline cudaStream_t as_stream(ge2_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

template <typename T>
__host__ __device__ constexpr T ceil_div(T a, T b) {
    return (a + b - 1) / b;
}
template <typename T>
__host__ __device__ constexpr T round_up(T a, T b) {
    return ceil_div(a, b) * b;
}

// number of CTAs for a grid-stride kernel over `work` items, `per_cta` items per CTA per sweep
inline int stream_grid(int64_t work, int per_cta, int ctas_per_sm = 8) {
    int64_t need = ceil_div<int64_t>(work, per_cta);
    int64_t cap = (int64_t)kNumSMs * ctas_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

// Programmatic dependent launch: a kernel launched with launch_after() may start while the kernel before it on the stream is
// still running (its CTAs become resident as SMs free up, and its prologue -- shared-memory set-up, barrier initialisation,
// tensor-memory allocation -- overlaps the predecessor's tail).  griddep_wait() returns once the predecessor grid has completed
// and its memory is visible; every thread calls it before its first access to global memory.  Without the launch attribute
// (or with a predecessor that is not a kernel) it returns at once.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// GE2_PDL=0 in the environment turns the attribute off (plain stream order)
inline bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("GE2_PDL");
        return e == nullptr || atoi(e) != 0;
    }();
    return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_after(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ void or_status(int32_t* status, int32_t bit) {
    if (status != nullptr) atomicOr(status, bit);
}

// ceil(B / C) the way the reference computes it (float division, decoder_methods.cpp:772 of the reference project)
inline int rows_per_chunk(int B, int C) {
    float q = (float)B / (float)C;
    int r = (int)q;
    return ((float)r < q) ? r + 1 : r;
}

}  // namespace ge2
