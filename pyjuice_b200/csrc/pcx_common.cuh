// Shared device helpers for the probabilistic-circuit kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <math_constants.h>

#define PCX_NEG_INF (-CUDART_INF_F)

#define PCX_LAUNCH_CHECK()                              \
    do {                                                \
        cudaError_t _e = cudaGetLastError();            \
        if (_e != cudaSuccess) return (int)_e;          \
    } while (0)

static inline int64_t pcx_cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

// A "done once" flag PER DEVICE for set-up that CUDA keeps per device (kernel attributes such as the dynamic
// shared-memory limit): reads and writes refer to the flag of the current device, so a process that drives several
// GPUs configures every kernel on each of them.  Used as `static PcxOnce done; if (!done) { ...; done = true; }`.
struct PcxOnce {
    bool flags[64] = {};
    bool& here() {
        int d = 0;
        if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) d = 0;
        return flags[d];
    }
    operator bool() { return here(); }
    PcxOnce& operator=(bool v) { here() = v; return *this; }
    bool* operator&() { return &here(); }
};

// log(exp(a) + exp(b)) with -inf handled (no NaN from inf - inf).
__device__ __forceinline__ float pcx_logaddexp(float a, float b) {
    float hi = fmaxf(a, b), lo = fminf(a, b);
    if (hi == PCX_NEG_INF) return PCX_NEG_INF;
    return hi + log1pf(__expf(lo - hi));
}

// Read one category id from a [V, B] table whose element size is 1, 2, 4 or 8 bytes.
__device__ __forceinline__ int pcx_load_cat(const void* data, int elsize, int64_t idx) {
    switch (elsize) {
        case 1: return (int)((const uint8_t*)data)[idx];
        case 2: return (int)((const int16_t*)data)[idx];
        case 4: return ((const int32_t*)data)[idx];
        default: return (int)((const int64_t*)data)[idx];
    }
}
