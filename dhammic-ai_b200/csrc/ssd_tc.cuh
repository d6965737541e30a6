// Tensor-core (tcgen05 / TMEM / TMA) path of the SSD chunked scan.
#pragma once
#include "ssd_common.cuh"
struct ssd_b200_fwd_args;
struct ssd_b200_bwd_args;
namespace ssd {
namespace tc {
inline bool supported(int, int, int, int, int, int, int) { return false; }
inline size_t workspace_bytes(const Dims&, int) { return 0; }
inline int forward(const ssd_b200_fwd_args*, const Dims&, cudaStream_t, char*, size_t) { return -2; }
inline int backward(const ssd_b200_bwd_args*, const Dims&, cudaStream_t, char*, size_t) { return -2; }
}  // namespace tc
}  // namespace ssd
