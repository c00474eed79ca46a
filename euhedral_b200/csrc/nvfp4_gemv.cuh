// NVFP4 decode GEMV for 1 to 8 BF16 activation rows on sm_100a: y[M, N] = x[M, K] . W^T with W in the converter's
// row-split NVFP4 layout (E2M1 codes two per byte, one E4M3 scale per 16 values, one FP32 scale per tensor).
//
// Replaces the reference's decode kernels native/src/nvfp4/kernels.cu:8-36 (body native/src/nvfp4/nvfp4.cuh:97-198)
// behind euhedral_cuda_linear_nvfp4_bf16 (native/src/host/nvfp4_linear.c:124-146). Same contract: products
// x * (e2m1 * e4m3) are exact, accumulation is FP32, the FP32 tensor scale multiplies the sum, the output is BF16
// round-to-nearest-even, and every activation row is computed independently of the others (row exactness).
//
// Design (bandwidth-bound, no tensor-map, no scratch):
//   * A CTA owns RB = 16 * RT weight rows and one K slice; the S CTAs of a thread-block cluster own the S slices of
//     the same rows. S depends on K only and RT on the launch geometry only, so a row's summation order is a function
//     of K alone: N-sharded copies of a tensor give bitwise the unsharded result.
//   * The whole tile (codes, scales, the activation slice) is made resident in shared memory by bulk asynchronous
//     copies issued before anything else, one mbarrier per 16-row tile. All bytes of the tile are in flight at once,
//     and with two or three CTAs per SM the memory system always has > 100 KB outstanding per SM.
//   * Weights do not depend on the previous kernel, so they are requested before griddepcontrol.wait: under
//     programmatic dependent launch the weight stream of call i+1 overlaps the tail of call i.
//   * Decode in registers: a lane owns 32 consecutive K values (16 code bytes) of rows g and g+8. Nibbles i and i+4 of
//     a 32-bit word become one BF16x2 register by two shifts and two masks (the E2M1 bits are placed where BF16 keeps
//     its two low exponent bits and its top mantissa bit, which reads as e2m1 * 2^-126, subnormal included), and one
//     packed multiply by (e4m3 * 2^110) gives e2m1 * e4m3 * 2^-16 exactly. The activations are staged in shared memory
//     in the matching (x[i], x[i+4]) pairing, so no further shuffling is needed.
//   * mma.sync.m16n8k16 (BF16, FP32 accumulate) with weights as the 16-row operand and the activation rows as the 8
//     columns, two warps per 16-row tile splitting the slice's chunks, summed in warp order, then in cluster-rank
//     order through distributed shared memory. The 2^16 and the tensor scale are applied to the final sum.
#pragma once

#include "common.cuh"

namespace nvfp4 {

constexpr uint32_t kChunk = 128;         // K values per chunk: 64 code bytes and 8 scale bytes per row
constexpr uint32_t kMaxRows = 8;         // activation rows per launch
constexpr uint32_t kMaxSplit = 8;        // portable cluster size

__host__ __device__ inline uint64_t align256(uint64_t v) { return (v + 255ull) & ~255ull; }

// Byte geometry of a tensor (tools/euhedral_artifacts/nvfp4.py:49-57; native/src/host/nvfp4_linear.c:79-91).
struct Geometry {
    uint64_t row_bytes, row_scales, scale_offset, global_offset, size;
    __host__ __device__ Geometry(uint32_t rows, uint32_t k) {
        const uint64_t kp = ((uint64_t)k + 127u) / 128u * 128u;
        row_bytes = kp / 2u;
        row_scales = kp / 16u;
        scale_offset = align256((uint64_t)rows * row_bytes);
        global_offset = align256(scale_offset + (uint64_t)rows * row_scales);
        size = global_offset + 4u;
    }
};

// Shared-memory layout of one CTA. Strides are 64 modulo 128 so that the eight rows a quarter-warp reads with 16-byte
// loads fall in distinct banks.
struct Tile {
    uint32_t stride_codes, stride_scales, stride_x;
    uint32_t off_scales, off_x, off_zero, off_partial, off_gather, off_bars, bytes;
    __host__ __device__ Tile(uint32_t rt, uint32_t chunks_max, uint32_t rows, uint32_t split) {
        const uint32_t rb = 16u * rt;
        stride_codes = chunks_max * 64u;
        if ((stride_codes & 127u) == 0u) stride_codes += 64u;
        stride_scales = chunks_max * 8u;
        stride_x = chunks_max * 256u + 64u;
        off_scales = rb * stride_codes;
        off_x = (off_scales + rb * stride_scales + 127u) & ~127u;
        off_zero = off_x + rows * stride_x;   // 256 zero bytes: the activations of lanes beyond the last row
        off_partial = off_zero + 256u;
        off_gather = off_partial + 2u * rt * 16u * 8u * 4u;
        off_bars = off_gather + (split > 1u ? split * rb * 8u * 4u : 0u);
        bytes = off_bars + 8u * rt;
    }
};

// K slices per row (cluster size): a function of K alone.
__host__ __device__ inline uint32_t split_of(uint32_t k) {
    const uint32_t chunks = k / kChunk;
    return chunks <= 12u ? 1u : chunks <= 24u ? 2u : chunks <= 48u ? 4u : 8u;
}

// Two E2M1 codes of `v` (nibbles `lo` and `lo + 4`) as BF16x2 holding e2m1 * 2^-126 each.
template <int LO>
__device__ __forceinline__ uint32_t raw_pair(uint32_t v) {
    constexpr int sign_shift = 12 - 4 * LO;   // nibble sign bit (4 LO + 3) to bit 15
    constexpr int mag_shift = 6 - 4 * LO;     // nibble magnitude (4 LO .. 4 LO + 2) to bits 6..8
    const uint32_t s = sign_shift > 0 ? v << sign_shift : v;
    const uint32_t m = mag_shift >= 0 ? v << mag_shift : v >> (-mag_shift);
    return (s & 0x80008000u) | (m & 0x01C001C0u);
}

// (e4m3 * 2^110) of the two scale bytes in `bits` as BF16x2 (low byte in the low half). The byte shifted left by 4 is
// a BF16 holding e4m3 * 2^-120 (subnormal codes included; bit 7 of the byte is ignored); two exact multiplies rescale it.
__device__ __forceinline__ uint32_t scale_pair(uint32_t bits) {
    const uint32_t raw = ((bits << 4) & 0x000007F0u) | ((bits << 12) & 0x07F00000u);
    const uint32_t unit = eb::bf16x2_mul(raw, 0x7B807B80u);   // * 2^120 -> e4m3
    return eb::bf16x2_mul(unit, 0x76807680u);                  // * 2^110
}

template <int RT>
__global__ void __launch_bounds__(64 * RT) gemv_kernel(const uint16_t* __restrict__ x, const uint8_t* __restrict__ w,
        uint16_t* __restrict__ y, uint32_t rows, uint32_t k, uint32_t n, uint32_t split, uint32_t* __restrict__ error) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t kRb = 16u * RT, kThreads = 64u * RT;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, q = lane & 3u;
    const uint32_t rank = split > 1u ? eb::cluster_rank() : 0u;
    const uint32_t row0 = (blockIdx.x / split) * kRb;
    const uint32_t chunks = k / kChunk;
    const uint32_t c_begin = (uint32_t)((uint64_t)rank * chunks / split), c_end = (uint32_t)((uint64_t)(rank + 1u) * chunks / split);
    const uint32_t nc = c_end - c_begin, nc_max = (chunks + split - 1u) / split;
    const Tile tile(RT, nc_max, rows, split);
    const Geometry geo(n, k);
    uint8_t* codes = smem;
    uint8_t* scales = smem + tile.off_scales;
    uint8_t* xs = smem + tile.off_x;
    float* partial = reinterpret_cast<float*>(smem + tile.off_partial);
    float* gather = reinterpret_cast<float*>(smem + tile.off_gather);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + tile.off_bars);

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < RT; ++i) eb::mbar_init(&bars[i], 16);
        eb::mbar_fence_init();
    }
    __syncthreads();

    // Weight bytes first: one bulk copy per row of the tile, then the scale bytes in 8-byte pieces.
    if (tid < kRb) {
        uint64_t* bar = &bars[tid >> 4];
        eb::mbar_arrive_expect_tx(bar, nc * 64u);
        eb::bulk_g2s(codes + tid * tile.stride_codes, w + (uint64_t)(row0 + tid) * geo.row_bytes + (uint64_t)c_begin * 64u,
                nc * 64u, bar);
    }
    for (uint32_t i = tid; i < kRb * nc; i += kThreads) {
        const uint32_t r = i / nc, c = i - r * nc;
        eb::cp_async_8(scales + r * tile.stride_scales + c * 8u,
                w + geo.scale_offset + (uint64_t)(row0 + r) * geo.row_scales + (uint64_t)(c_begin + c) * 8u);
    }
    const float global = *reinterpret_cast<const float*>(w + geo.global_offset);

    // The activations may come from the kernel before this one.
    eb::pdl_launch_dependents();
    eb::pdl_wait();
    if (tid < 64u) reinterpret_cast<uint32_t*>(smem + tile.off_zero)[tid] = 0u;
    for (uint32_t u = tid; u < rows * nc * 16u; u += kThreads) {
        const uint32_t t = u / (nc * 16u), j = u - t * (nc * 16u);
        const uint32_t c = j >> 4, qq = (j >> 2) & 3u, i = j & 3u;
        const uint4 v = *reinterpret_cast<const uint4*>(x + (uint64_t)t * k + (uint64_t)(c_begin + c) * kChunk + qq * 32u + i * 8u);
        uint4 p;
        p.x = __byte_perm(v.x, v.z, 0x5410);   // (x0, x4)
        p.y = __byte_perm(v.x, v.z, 0x7632);   // (x1, x5)
        p.z = __byte_perm(v.y, v.w, 0x5410);   // (x2, x6)
        p.w = __byte_perm(v.y, v.w, 0x7632);   // (x3, x7)
        *reinterpret_cast<uint4*>(xs + t * tile.stride_x + c * 256u + i * 64u + qq * 16u) = p;
    }
    eb::cp_async_wait_all();
    __syncthreads();

    // Two warps per 16-row tile: warp 2 rt + h takes the h-th half of the slice's chunks.
    const uint32_t rt = warp >> 1, half = warp & 1u;
    const uint32_t first = nc * half / 2u, last = nc * (half + 1u) / 2u;
    if (!eb::mbar_wait(&bars[rt], 0) && lane == 0) atomicOr(error, 1u);
    const uint8_t* code_g = codes + (rt * 16u + g) * tile.stride_codes + q * 16u + first * 64u;
    const uint8_t* code_h = code_g + 8u * tile.stride_codes;
    const uint8_t* scale_g = scales + (rt * 16u + g) * tile.stride_scales + q * 2u + first * 8u;
    const uint8_t* scale_h = scale_g + 8u * tile.stride_scales;
    // Lanes beyond the last activation row read the zero block and never advance.
    const bool live = g < rows;
    const uint8_t* x_lane = live ? xs + g * tile.stride_x + q * 16u + first * 256u : smem + tile.off_zero + q * 16u;
    const uint32_t x_step = live ? 256u : 0u;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (uint32_t c = first; c < last; ++c) {
        const uint4 cg = *reinterpret_cast<const uint4*>(code_g);
        const uint4 ch = *reinterpret_cast<const uint4*>(code_h);
        const uint32_t sg = scale_pair(*reinterpret_cast<const uint16_t*>(scale_g));
        const uint32_t sh = scale_pair(*reinterpret_cast<const uint16_t*>(scale_h));
        const uint32_t sg_block[2] = {__byte_perm(sg, sg, 0x1010), __byte_perm(sg, sg, 0x3232)};
        const uint32_t sh_block[2] = {__byte_perm(sh, sh, 0x1010), __byte_perm(sh, sh, 0x3232)};
        const uint32_t wg[4] = {cg.x, cg.y, cg.z, cg.w}, wh[4] = {ch.x, ch.y, ch.z, ch.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 xv = *reinterpret_cast<const uint4*>(x_lane + i * 64u);
            const uint32_t fg = sg_block[i >> 1], fh = sh_block[i >> 1];
            const uint32_t g0 = eb::bf16x2_mul(raw_pair<0>(wg[i]), fg), h0 = eb::bf16x2_mul(raw_pair<0>(wh[i]), fh);
            const uint32_t g1 = eb::bf16x2_mul(raw_pair<1>(wg[i]), fg), h1 = eb::bf16x2_mul(raw_pair<1>(wh[i]), fh);
            eb::mma_bf16_16816(acc, g0, h0, g1, h1, xv.x, xv.y);
            const uint32_t g2 = eb::bf16x2_mul(raw_pair<2>(wg[i]), fg), h2 = eb::bf16x2_mul(raw_pair<2>(wh[i]), fh);
            const uint32_t g3 = eb::bf16x2_mul(raw_pair<3>(wg[i]), fg), h3 = eb::bf16x2_mul(raw_pair<3>(wh[i]), fh);
            eb::mma_bf16_16816(acc, g2, h2, g3, h3, xv.z, xv.w);
        }
        code_g += 64u;
        code_h += 64u;
        scale_g += 8u;
        scale_h += 8u;
        x_lane += x_step;
    }
    // partial[warp][row in tile][activation row]
    float* mine = partial + warp * 128u;
    mine[g * 8u + 2u * q] = acc[0];
    mine[g * 8u + 2u * q + 1u] = acc[1];
    mine[(g + 8u) * 8u + 2u * q] = acc[2];
    mine[(g + 8u) * 8u + 2u * q + 1u] = acc[3];
    __syncthreads();

    if (split == 1u) {
        for (uint32_t i = tid; i < kRb * rows; i += kThreads) {
            const uint32_t t = i / kRb, r = i - t * kRb;
            const float sum = partial[(r >> 4) * 256u + (r & 15u) * 8u + t] + partial[(r >> 4) * 256u + 128u + (r & 15u) * 8u + t];
            y[(uint64_t)t * n + row0 + r] = eb::float_to_bf16_bits(sum * 65536.0f * global);
        }
        return;
    }
    // Every rank deposits its tile of sums in rank 0's gather buffer; rank 0 adds them in rank order.
    const uint32_t gather0 = eb::map_to_rank(eb::smem_u32(gather), 0);
    for (uint32_t i = tid; i < kRb * 8u; i += kThreads) {
        const uint32_t r = i >> 3, t = i & 7u;
        const float sum = partial[(r >> 4) * 256u + (r & 15u) * 8u + t] + partial[(r >> 4) * 256u + 128u + (r & 15u) * 8u + t];
        eb::st_cluster_f32(gather0 + ((rank * kRb + r) * 8u + t) * 4u, sum);
    }
    eb::cluster_sync();
    if (rank != 0u) return;
    for (uint32_t i = tid; i < kRb * rows; i += kThreads) {
        const uint32_t t = i / kRb, r = i - t * kRb;
        float sum = gather[r * 8u + t];
        for (uint32_t s = 1; s < split; ++s) sum += gather[(s * kRb + r) * 8u + t];
        y[(uint64_t)t * n + row0 + r] = eb::float_to_bf16_bits(sum * 65536.0f * global);
    }
}

}  // namespace nvfp4
