// Placeholder replaced below.
#pragma once
#include "common.cuh"
namespace nvfp4n {
struct ActivationLayout {
    uint64_t scale_offset, global_offset, bytes;
    uint32_t pad;
    __host__ __device__ ActivationLayout(uint32_t rows, uint32_t k) {
        const uint64_t kp = ((uint64_t)k + 127u) / 128u * 128u;
        pad = (rows + 127u) / 128u * 128u;
        scale_offset = ((uint64_t)rows * 2u * (kp / 2u) + 255u) & ~255ull;
        global_offset = (scale_offset + (kp / 128u) * 2u * pad * 8ull + 255u) & ~255ull;
        bytes = global_offset + 4ull * rows;
    }
};
inline cudaError_t initialize() { return cudaSuccess; }
inline cudaError_t run(const void*, const void*, void*, void*, uint32_t, uint32_t, uint32_t, int, cudaStream_t, bool, uint32_t*) {
    return cudaErrorNotSupported;
}
}  // namespace nvfp4n
