// The trellis-tile16-v1 decode arithmetic (the format is exllamav3's EXL3 with the "mul1" codebook; the reference
// keeps it in native/src/trellis/codebook.cuh:18-113, NumPy twin native/tests/trellis_reference.py:9-76).
//
// A 16 x 16 tile is a tail-biting ring of w 16-bit words (w = 16 * bits per weight, multiples of 8 from 16 to 128).
// The ring is read as 32-bit little-endian words, most significant bit first. Position p (0..255) decodes the 16-bit
// window that ENDS at ring bit
//     S(p) = (p / 16) * w + (w / 16) * (p % 16 + 1) + [w % 16 == 8] * (number of odd j <= p % 16),
// the window's value ("state") goes through
//     value = fp16_fma(fp16_bits(0x6400 + sum of the four bytes of (state * 0x83DCD12D)), 0x1EEE, 0xC931),
// and position p = 8 * lane + j is element (k, n) of the tile with, for g = lane / 4 and q = lane % 4,
//     k = 2 q + 8 * ((j / 2) % 2) + j % 2,  n = g + 8 * (j / 4):
// a lane's eight positions are exactly its m16n8k16 A fragment when the tile's n runs along the MMA's 16 rows.
#pragma once

#include "common.cuh"

namespace trellis {

constexpr float kInvSqrt128 = 0.08838834764831845f;

// FP16 bits of the codebook value of one state.
__device__ __forceinline__ uint16_t value_bits(uint32_t state) {
    const uint32_t sum = __dp4a(state * 0x83DCD12Du, 0x01010101u, 0x6400u);
    return __half_as_ushort(__hfma(__ushort_as_half((unsigned short)sum), __ushort_as_half((unsigned short)0x1EEE),
            __ushort_as_half((unsigned short)0xC931)));
}

// Two values at once as a packed half2 (low half from state0).
__device__ __forceinline__ uint32_t value_pair(uint32_t state0, uint32_t state1) {
    const uint32_t s0 = __dp4a(state0 * 0x83DCD12Du, 0x01010101u, 0x6400u);
    const uint32_t s1 = __dp4a(state1 * 0x83DCD12Du, 0x01010101u, 0x6400u);
    const uint32_t packed = __byte_perm(s0, s1, 0x5410);
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&packed), __half2half2(__ushort_as_half((unsigned short)0x1EEE)),
            __half2half2(__ushort_as_half((unsigned short)0xC931)));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// Ring bit at which the window of position p ends.
__host__ __device__ __forceinline__ int window_end(int p, int w) {
    const int m = p & 15;
    return (p >> 4) * w + (w >> 4) * (m + 1) + (((w & 15) == 8) ? (m + 1) / 2 : 0);
}

// The state of position p of a tile given as w 16-bit words in global or shared memory (slow path: scalar kernels).
__device__ __forceinline__ uint32_t window_of_tile(const uint16_t* tile, int w, int p) {
    const int ring = 16 * w;
    int start = (window_end(p, w) - 16) % ring;
    if (start < 0) start += ring;
    const uint32_t* words = reinterpret_cast<const uint32_t*>(tile);
    const int nw = w >> 1, wi = start >> 5, o = start & 31;
    const uint32_t hi = words[wi], lo = words[wi + 1 == nw ? 0 : wi + 1];
    const uint64_t both = ((uint64_t)hi << 32) | lo;
    return (uint32_t)(both >> (48 - o)) & 0xFFFFu;
}

// Position whose element is (k = rl, n = cl) of the tile: the inverse of the map in the header comment.
__host__ __device__ __forceinline__ int position_of(int rl, int cl) {
    const int j = (rl & 1) | (((rl >> 3) & 1) << 1) | ((cl >> 3) << 2);
    const int lane = ((cl & 7) << 2) | ((rl >> 1) & 3);
    return (lane << 3) | j;
}

// 128-point Sylvester Hadamard of s[0..127] (shared memory) by the 128 threads of a block: stages h = 1, 2, .., 64 in
// that order (pair i, i + h becomes a + b, a - b), then * 1/sqrt(128). Synchronizes the block.
__device__ __forceinline__ void hadamard128_block(float* s, int t) {
    __syncthreads();
    for (int h = 1; h < 128; h <<= 1) {
        if (t < 64) {
            const int i = (t / h) * 2 * h + (t % h);
            const float a = s[i], b = s[i + h];
            s[i] = __fadd_rn(a, b);
            s[i + h] = __fsub_rn(a, b);
        }
        __syncthreads();
    }
    s[t] = __fmul_rn(s[t], kInvSqrt128);
    __syncthreads();
}

// The same transform on 128 floats held by one warp, element 4 * lane + j in v[j]: the two lowest stages are inside a
// lane, the other five exchange with lane ^ (h / 4). Every stage forms the same a + b and a - b as the block version,
// so the results are bitwise equal.
__device__ __forceinline__ void hadamard128_warp(float (&v)[4], int lane) {
    const float a0 = __fadd_rn(v[0], v[1]), a1 = __fsub_rn(v[0], v[1]), a2 = __fadd_rn(v[2], v[3]), a3 = __fsub_rn(v[2], v[3]);
    v[0] = __fadd_rn(a0, a2);
    v[1] = __fadd_rn(a1, a3);
    v[2] = __fsub_rn(a0, a2);
    v[3] = __fsub_rn(a1, a3);
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
        const bool upper = (lane & h) != 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float other = __shfl_xor_sync(0xFFFFFFFFu, v[j], h);
            v[j] = upper ? __fsub_rn(other, v[j]) : __fadd_rn(v[j], other);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __fmul_rn(v[j], kInvSqrt128);
}

}  // namespace trellis
