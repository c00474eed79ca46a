// Scalar FP32 kernels: what euhedral_cuda_select_exact_numerics(1) routes every quantized linear to, and what shapes
// or alignments no fast kernel takes fall back to. They follow the arithmetic and the summation order of the
// reference's oracles (native/src/reference/kernels.cu:17-48,125-159 and native/src/reference/trellis.cuh:14-55): 128
// threads stride K, a 7-step pairwise tree joins them, one output element per CTA iteration.
#pragma once

#include "common.cuh"
#include "trellis_codebook.cuh"

namespace exact {

__device__ __forceinline__ float tree128(float value, float* scratch) {
    scratch[threadIdx.x] = value;
    __syncthreads();
    for (uint32_t stride = 64; stride > 0; stride >>= 1) {
        if (threadIdx.x < stride) scratch[threadIdx.x] = __fadd_rn(scratch[threadIdx.x], scratch[threadIdx.x + stride]);
        __syncthreads();
    }
    const float total = scratch[0];
    __syncthreads();
    return total;
}

__device__ __forceinline__ float e2m1(uint32_t code) {
    const uint32_t m = code & 7u;
    const float v = m < 4u ? 0.5f * (float)m : (float)(2u << (m - 4u >> 1)) * ((m & 1u) ? 1.5f : 1.0f);
    return (code & 8u) ? -v : v;
}

__device__ __forceinline__ float e4m3(uint32_t code) {
    // E4M3 is FP16 with bias 7 instead of 15: shift into an FP16 and multiply by 2^8 (exact, subnormals included).
    return __half2float(__ushort_as_half((unsigned short)((code & 0x7fu) << 7))) * 256.0f;
}

// NVFP4: partial = fma(x, e2m1 * e4m3, partial); (tree sum) * global; BF16. Grid-stride over rows * n outputs.
// kTable: the block scales are 4-bit indices (two per byte, the even block in the low nibble) into the tensor's table of
// 16 E4M3 codes (layout row-split-k128-sd4-v1; the reference's twin kernels, native/src/nvfp4/scale_table.cuh:4-15).
template <bool kTable>
__global__ void __launch_bounds__(128) nvfp4_linear(const uint16_t* __restrict__ x, const uint8_t* __restrict__ w,
        uint16_t* __restrict__ y, uint32_t rows, uint32_t k, uint32_t n) {
    __shared__ float scratch[128];
    const uint64_t kp = ((uint64_t)k + 127u) / 128u * 128u;
    const uint64_t row_bytes = kp / 2u, row_scales = kTable ? kp / 32u : kp / 16u;
    const uint64_t scale_offset = ((uint64_t)n * row_bytes + 255u) & ~255ull;
    const uint64_t table_offset = (scale_offset + (uint64_t)n * row_scales + 255u) & ~255ull;
    const uint64_t global_offset = kTable ? table_offset + 16u : table_offset;
    const float global = *reinterpret_cast<const float*>(w + global_offset);
    const uint64_t count = (uint64_t)rows * n;
    for (uint64_t index = blockIdx.x; index < count; index += gridDim.x) {
        const uint32_t row = (uint32_t)(index / n), col = (uint32_t)(index % n);
        float partial = 0.0f;
        for (uint32_t i = threadIdx.x; i < k; i += 128u) {
            const uint32_t code = (w[(uint64_t)col * row_bytes + i / 2u] >> ((i & 1u) * 4u)) & 15u;
            uint32_t scale_code;
            if (kTable) {
                const uint32_t block = i / 16u;
                scale_code = w[table_offset + ((w[scale_offset + (uint64_t)col * row_scales + block / 2u] >> ((block & 1u) * 4u)) & 15u)];
            } else {
                scale_code = w[scale_offset + (uint64_t)col * row_scales + i / 16u];
            }
            partial = __fmaf_rn(eb::bf16_bits_to_float(x[(uint64_t)row * k + i]), __fmul_rn(e2m1(code), e4m3(scale_code)), partial);
        }
        const float total = tree128(partial, scratch);
        if (threadIdx.x == 0) y[index] = eb::float_to_bf16_bits(__fmul_rn(total, global));
    }
}

// FP16 -> FP32 keeping NaN payloads (the reference's scalar Q3 oracle does, native/src/q3/numeric.cuh:9-16).
__device__ __forceinline__ float half_bits_to_float(uint16_t bits) {
    if ((bits & 0x7c00u) == 0x7c00u && (bits & 0x03ffu) != 0u)
        return __uint_as_float(((uint32_t)(bits & 0x8000u) << 16) | 0x7f800000u | ((uint32_t)(bits & 0x03ffu) << 13));
    return __half2float(__ushort_as_half(bits));
}

// Q3G64_F16S: partial += (x * code) * scale, each operation rounded; tree sum; BF16.
__global__ void __launch_bounds__(128) q3_linear(const uint16_t* __restrict__ x, const uint8_t* __restrict__ w,
        uint16_t* __restrict__ y, uint32_t rows, uint32_t k, uint32_t n, uint64_t scale_offset) {
    __shared__ float scratch[128];
    const uint64_t groups = ((uint64_t)k + 127u) / 128u * 2u;
    const uint16_t* scales = reinterpret_cast<const uint16_t*>(w + scale_offset);
    const uint64_t count = (uint64_t)rows * n;
    for (uint64_t index = blockIdx.x; index < count; index += gridDim.x) {
        const uint32_t row = (uint32_t)(index / n), col = (uint32_t)(index % n);
        float partial = 0.0f;
        for (uint32_t i = threadIdx.x; i < k; i += 128u) {
            const uint64_t group = (uint64_t)col * groups + i / 64u;
            const uint8_t* bytes = w + group * 24u;
            const uint32_t bit = (i % 64u) * 3u, at = bit >> 3;
            const uint32_t pair = (uint32_t)bytes[at] | (at + 1u < 24u ? (uint32_t)bytes[at + 1u] << 8 : 0u);
            const uint32_t field = (pair >> (bit & 7u)) & 7u;
            const float code = (float)((int)field - (field >= 4u ? 8 : 0));
            const float term = __fmul_rn(__fmul_rn(eb::bf16_bits_to_float(x[(uint64_t)row * k + i]), code), half_bits_to_float(scales[group]));
            partial = __fadd_rn(partial, term);
        }
        const float total = tree128(partial, scratch);
        if (threadIdx.x == 0) y[index] = eb::float_to_bf16_bits(total);
    }
}

// Trellis, FP32 throughout and no FP16 rounding of the activations: one CTA per output element (r, c); the rotated
// input u = H128(x * suh[seg(c)]) lives in dynamic shared memory (4 * k bytes), thread t sums column c0 + t of the 128
// column block holding c, the block applies the output Hadamard and thread (c & 127) writes svh[c] * H(z)[c].
__global__ void __launch_bounds__(128) trellis_linear(const uint16_t* __restrict__ x, const uint16_t* __restrict__ words,
        const uint16_t* __restrict__ suh, const uint16_t* __restrict__ svh, const int* __restrict__ ends, int s,
        uint16_t* __restrict__ out, int rows, int k, int n, int w) {
    extern __shared__ float u[];
    __shared__ float z[128];
    const int t = threadIdx.x;
    const size_t index = blockIdx.x;
    const int r = (int)(index / (size_t)n), c = (int)(index % (size_t)n);
    if (r >= rows) return;
    const int c0 = c & ~127;
    int seg = 0;
    while (seg + 1 < s && c0 >= ends[seg]) ++seg;
    for (int b = 0; b < k / 128; ++b) {
        const size_t col = (size_t)b * 128 + t;
        z[t] = __fmul_rn(eb::bf16_bits_to_float(x[(size_t)r * k + col]), __half2float(__ushort_as_half(suh[(size_t)seg * k + col])));
        trellis::hadamard128_block(z, t);
        u[b * 128 + t] = z[t];
        __syncthreads();
    }
    const int col = c0 + t, tj = col >> 4, cl = col & 15;
    const int tiles_n = n >> 4;
    float sum = 0.0f;
    for (int row = 0; row < k; ++row) {
        const int ti = row >> 4, rl = row & 15;
        const int p = trellis::position_of(rl, cl);
        const uint16_t* tile = words + ((size_t)ti * tiles_n + tj) * w;
        const float q = __half2float(__ushort_as_half(trellis::value_bits(trellis::window_of_tile(tile, w, p))));
        sum = __fadd_rn(sum, __fmul_rn(u[row], q));
    }
    z[t] = sum;
    trellis::hadamard128_block(z, t);
    if (t == (c & 127))
        out[(size_t)r * n + c] = eb::float_to_bf16_bits(__fmul_rn(__half2float(__ushort_as_half(svh[c])), z[t]));
}

}  // namespace exact
