// Shared device helpers and the problem descriptor used by every SSD kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ssd {

// Problem dimensions; c = T / l, hpg = heads per group.
struct Dims {
    int b, T, h, p, n, g, l, c, hpg;
};

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Element offsets of the dense layouts.
__device__ __forceinline__ size_t x_off(const Dims& d, int bb, int t, int hh) {  // (b,T,h,p) row start
    return ((size_t)((size_t)bb * d.T + t) * d.h + hh) * d.p;
}
__device__ __forceinline__ size_t bc_off(const Dims& d, int bb, int t, int gg) {  // (b,T,g,n) row start
    return ((size_t)((size_t)bb * d.T + t) * d.g + gg) * d.n;
}
__device__ __forceinline__ size_t cum_off(const Dims& d, int bb, int hh, int k) {  // (b,h,c,l) chunk start
    return ((size_t)((size_t)bb * d.h + hh) * d.c + k) * d.l;
}
__device__ __forceinline__ size_t st_off(const Dims& d, int bb, int k, int hh) {  // (b,c,h,p,n) state start
    return ((size_t)((size_t)bb * d.c + k) * d.h + hh) * (size_t)d.p * d.n;
}

namespace prof {
// Kernel slots for launch accounting / optional per-kernel timing (definitions in ssd_b200_api.cu).
enum Kernel {
    K_CUMSUM = 0, K_CHUNK_STATE, K_STATE_PASS, K_CHUNK_SCAN, K_CHUNK_DSTATE, K_STATE_PASS_REV, K_BWD_ROW, K_BWD_COL,
    K_DECAY, K_REDUCE, K_CACHE_L, K_CACHE_DC, K_PREFIX, K_TC_FWD, K_TC_BWD_STATE, K_TC_BWD, K_TC_AUX, K_TC_SUMMARY,
    K_TC_BWD_ALT, K_TC_FWD_ALT, K_EXCHANGE, K_COUNT
};
void begin(int k, cudaStream_t st);
void end(cudaStream_t st);
}  // namespace prof

// Wrap one kernel launch statement: counts it and, when profiling is on, brackets it with events.
#define SSD_LAUNCH(kidx, st, ...)     \
    do {                              \
        ::ssd::prof::begin(kidx, st); \
        __VA_ARGS__;                  \
        ::ssd::prof::end(st);         \
    } while (0)

}  // namespace ssd
