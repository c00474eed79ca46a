// Q3G64_F16S decode GEMV for 1 to 8 BF16 activation rows on sm_100a: y[M, N] = x[M, K] . W^T with W in the
// converter's row-split layout (groups of 64 three-bit codes in 24 bytes, one FP16 scale per group in a second plane).
//
// Replaces the reference's contiguous decode kernels native/src/q3/kernels.cu:11-41 (body
// native/src/q3/contiguous.cuh:55-223) behind euhedral_cuda_linear_q3_bf16 (native/src/host/q3_linear_bf16.c:73-102).
// Same contract: products x * code are exact, a group's 64 products are summed in FP32 and multiplied once by the FP32
// value of the FP16 group scale, the output is BF16 round-to-nearest-even, and every activation row is computed
// independently of the others (row exactness).
//
// The reference spends one FP32 FMA per weight and activation row, which B200's ratio of ALU rate to HBM bandwidth
// cannot pay for. Here the codes become BF16 integers (-4..3) and the sums run on the tensor core: one
// mma.sync.m16n8k16 covers 16 weight rows x 16 K values x 8 activation rows, four MMAs with a fresh accumulator cover
// one group, and the group's FP32 scale is applied to that accumulator (an FP16 scale is not exact in BF16, so it
// cannot be folded into the operand).
//
// Tile residency, cluster K split and programmatic-dependent-launch ordering are those of the NVFP4 GEMV
// (nvfp4_gemv.cuh). A lane owns 16 consecutive codes (48 bits) of a group for rows g and g+8: lane q's bits start
// at bit 48 q of the group's 192. Codes j and j+5 (j < 5) and codes 10+j and 13+j (j < 3) are brought 16 bits apart
// so that one shift and one mask yield both halves of a BF16x2 register; the activations are staged in shared
// memory in the same pairing.
#pragma once

#include "common.cuh"

namespace q3 {

constexpr uint32_t kChunk = 128;   // K values per chunk: two groups, 48 code bytes and two FP16 scales per row

// Byte geometry (tools/euhedral_artifacts/grouped.py:24-36; native/src/host/q3_linear_bf16.c:82-84).
struct Geometry {
    uint64_t groups, row_bytes, scale_offset, size;
    __host__ __device__ Geometry(uint32_t rows, uint32_t k) {
        groups = ((uint64_t)k + 127u) / 128u * 2u;
        row_bytes = groups * 24u;
        scale_offset = ((uint64_t)rows * row_bytes + 255ull) & ~255ull;
        size = scale_offset + (uint64_t)rows * groups * 2u;
    }
};

struct Tile {
    uint32_t stride_codes, stride_scales, stride_x;
    uint32_t off_scales, off_x, off_zero, off_xsum, off_partial, off_gather, off_bars, bytes;
    __host__ __device__ Tile(uint32_t rt, uint32_t chunks_max, uint32_t rows, uint32_t split) {
        const uint32_t rb = 16u * rt;
        // 16 bytes modulo 128: the eight rows of a warp's 32-bit loads start four banks apart.
        stride_codes = chunks_max * 48u;
        while ((stride_codes & 127u) != 16u) stride_codes += 16u;
        stride_scales = chunks_max * 4u;
        stride_x = chunks_max * 256u + 64u;
        off_scales = rb * stride_codes;
        off_x = (off_scales + rb * stride_scales + 127u) & ~127u;
        off_zero = off_x + rows * stride_x;          // 256 zero bytes: the activations of lanes beyond the last row
        off_xsum = off_zero + 256u;                   // float [chunk][group][8 rows]: -132 * sum of the group's activations
        off_partial = off_xsum + chunks_max * 64u;
        off_gather = off_partial + 2u * rt * 16u * 8u * 4u;
        off_bars = off_gather + (split > 1u ? split * rb * 8u * 4u : 0u);
        bytes = off_bars + 8u * rt;
    }
};

// Pair p of a lane's 16 codes: (low code, high code).
__host__ __device__ constexpr int pair_lo(int p) { return p < 5 ? p : p + 5; }
__host__ __device__ constexpr int pair_hi(int p) { return p < 5 ? p + 5 : p + 8; }

// The (x[lo], x[hi]) register of pair P from 16 consecutive BF16 activations held in s[0..7] (two per register).
template <int P>
__device__ __forceinline__ uint32_t pair_x(const uint32_t (&s)[8]) {
    constexpr int lo = pair_lo(P), hi = pair_hi(P);
    constexpr uint32_t selector = (uint32_t)((lo & 1) * 2) | (uint32_t)((lo & 1) * 2 + 1) << 4 | (uint32_t)(4 + (hi & 1) * 2) << 8
            | (uint32_t)(4 + (hi & 1) * 2 + 1) << 12;
    return __byte_perm(s[lo >> 1], s[hi >> 1], selector);
}

// A value the compiler must keep in a register (LOP3 takes one immediate only; masks and magic are both needed).
__device__ __forceinline__ uint32_t in_register(uint32_t v) {
    asm volatile("mov.b32 %0, %0;" : "+r"(v));
    return v;
}

// Eight BF16x2 registers for the 16 codes of the 48 bits (a32 | b16 << 32), in pair order. Each half is the BF16
// 132 + code (0x4300 | (field ^ 4)): the kernel starts a group's accumulator at -132 * (sum of the group's
// activations), so the MMAs leave sum x * code without a per-weight subtraction. Bits of b16 above 16 are ignored.
__device__ __forceinline__ void decode16(uint32_t a32, uint32_t b16, uint32_t mask7, uint32_t magic, uint32_t (&out)[8]) {
    // Codes 0..4 at bits 0,3,..,12 of the low half and codes 5..9 at the same bits of the high half (bits 15 and 31 hold
    // leftovers that the 3-bit masks below never select).
    const uint32_t z = eb::lop3<eb::kLutSelect>(a32, a32 << 1, 0x00007FFFu);
    // Codes 10..15 start at bit 30: bring them to bit 0, then 10..12 low and 13..15 high.
    const uint32_t y = __funnelshift_r(a32, b16, 30);
    const uint32_t z2 = eb::lop3<eb::kLutSelect>(y, y << 7, 0x000001FFu);
#pragma unroll
    for (int t = 0; t < 5; ++t) out[t] = eb::lop3<eb::kLutAndXor>(z >> (3 * t), mask7, magic);
#pragma unroll
    for (int t = 0; t < 3; ++t) out[5 + t] = eb::lop3<eb::kLutAndXor>(z2 >> (3 * t), mask7, magic);
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
    float* xsum = reinterpret_cast<float*>(smem + tile.off_xsum);
    float* partial = reinterpret_cast<float*>(smem + tile.off_partial);
    float* gather = reinterpret_cast<float*>(smem + tile.off_gather);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + tile.off_bars);

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < RT; ++i) eb::mbar_init(&bars[i], 16);
        eb::mbar_fence_init();
    }
    __syncthreads();

#ifndef EB_SKIP_LOADS
    if (tid < kRb) {
        uint64_t* bar = &bars[tid >> 4];
        eb::mbar_arrive_expect_tx(bar, nc * 48u);
        eb::bulk_g2s(codes + tid * tile.stride_codes, w + (uint64_t)(row0 + tid) * geo.row_bytes + (uint64_t)c_begin * 48u,
                nc * 48u, bar);
    }
#endif
    for (uint32_t i = tid; i < kRb * nc; i += kThreads) {
        const uint32_t r = i / nc, c = i - r * nc;
        eb::cp_async_4(scales + r * tile.stride_scales + c * 4u,
                w + geo.scale_offset + ((uint64_t)(row0 + r) * geo.groups + (uint64_t)(c_begin + c) * 2u) * 2u);
    }

    eb::pdl_launch_dependents();
    eb::pdl_wait();
    // One unit = 16 consecutive activations of one row, (row, chunk, group, quarter): stored in the decode's pairing for
    // the lane quartet that reads it. The four quarters of a group sit in four neighbouring lanes, which add their sums
    // in a fixed order ((q0 + q1) + (q2 + q3)) and store -132 * that. Rows beyond `rows` read zero bytes and get a zero sum.
    if (tid < 64u) reinterpret_cast<uint32_t*>(smem + tile.off_zero)[tid] = 0u;
#ifndef EB_SKIP_STAGING
    for (uint32_t unit = tid; unit < 8u * nc * 8u; unit += kThreads) {
        const uint32_t t = unit / (nc * 8u), j = unit - t * (nc * 8u);
        const uint32_t c = j >> 3, grp = (j >> 2) & 1u, qq = j & 3u;
        float total = 0.0f;
        if (t < rows) {
            const uint4* src = reinterpret_cast<const uint4*>(x + (uint64_t)t * k + (uint64_t)(c_begin + c) * kChunk + grp * 64u + qq * 16u);
            const uint4 v0 = src[0], v1 = src[1];
            const uint32_t s[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            uint8_t* dst = xs + t * tile.stride_x + c * 256u + grp * 128u + qq * 16u;
            *reinterpret_cast<uint4*>(dst) = make_uint4(pair_x<0>(s), pair_x<1>(s), pair_x<2>(s), pair_x<3>(s));
            *reinterpret_cast<uint4*>(dst + 64u) = make_uint4(pair_x<4>(s), pair_x<5>(s), pair_x<6>(s), pair_x<7>(s));
            float even = 0.0f, odd = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                even = __fadd_rn(even, eb::bf16_bits_to_float(s[e] & 0xFFFFu));
                odd = __fadd_rn(odd, __uint_as_float(s[e] & 0xFFFF0000u));
            }
            total = __fadd_rn(even, odd);
        }
        // kThreads and the unit count are multiples of 4, so a quartet is always whole.
        total = __fadd_rn(total, __shfl_xor_sync(0xFFFFFFFFu, total, 1));
        total = __fadd_rn(total, __shfl_xor_sync(0xFFFFFFFFu, total, 2));
        if (qq == 0u) xsum[(c * 2u + grp) * 8u + t] = __fmul_rn(total, -132.0f);
    }
#endif
    eb::cp_async_wait_all();
    __syncthreads();

    const uint32_t rt = warp >> 1, half = warp & 1u;
    const uint32_t first = nc * half / 2u, last = nc * (half + 1u) / 2u;
#ifndef EB_SKIP_LOADS
    if (!eb::mbar_wait(&bars[rt], 0) && lane == 0) atomicOr(error, 2u);
#endif
    // Lane q's 48 bits of a group start at 32-bit word {0, 1, 3, 4}[q], at bit 16 of it for odd q.
    const uint32_t word = (q >> 1) * 3u + (q & 1u), shift = (q & 1u) * 16u;
    const uint8_t* code_g = codes + (rt * 16u + g) * tile.stride_codes + word * 4u + first * 48u;
    const uint8_t* code_h = code_g + 8u * tile.stride_codes;
    const uint8_t* scale_g = scales + (rt * 16u + g) * tile.stride_scales + first * 4u;
    const uint8_t* scale_h = scale_g + 8u * tile.stride_scales;
    // Lanes beyond the last activation row read the zero block and never advance.
    const bool live = g < rows;
    const uint8_t* x_lane = live ? xs + g * tile.stride_x + q * 16u + first * 256u : smem + tile.off_zero + q * 16u;
    const uint32_t x_step = live ? 256u : 0u;
    const float2* offset_lane = reinterpret_cast<const float2*>(xsum) + first * 8u + q;   // rows 2q, 2q + 1
    const uint32_t mask7 = in_register(0x00070007u), magic = in_register(0x43044304u);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#ifdef EB_SKIP_COMPUTE
    for (uint32_t c = last; c < last; ++c) {
#else
    for (uint32_t c = first; c < last; ++c) {
#endif
#pragma unroll
        for (uint32_t grp = 0; grp < 2u; ++grp) {
            const uint32_t* pg = reinterpret_cast<const uint32_t*>(code_g + grp * 24u);
            const uint32_t* ph = reinterpret_cast<const uint32_t*>(code_h + grp * 24u);
            const uint32_t ga = pg[0], gb = pg[1], ha = ph[0], hb = ph[1];
            uint32_t wg[8], wh[8];
            decode16(__funnelshift_r(ga, gb, shift), gb >> shift, mask7, magic, wg);
            decode16(__funnelshift_r(ha, hb, shift), hb >> shift, mask7, magic, wh);
            const uint4 x0 = *reinterpret_cast<const uint4*>(x_lane + grp * 128u);
            const uint4 x1 = *reinterpret_cast<const uint4*>(x_lane + grp * 128u + 64u);
            const float2 offset = offset_lane[grp * 4u];
            float sum[4] = {offset.x, offset.y, offset.x, offset.y};
            eb::mma_bf16_16816(sum, wg[0], wh[0], wg[1], wh[1], x0.x, x0.y);
            eb::mma_bf16_16816(sum, wg[2], wh[2], wg[3], wh[3], x0.z, x0.w);
            eb::mma_bf16_16816(sum, wg[4], wh[4], wg[5], wh[5], x1.x, x1.y);
            eb::mma_bf16_16816(sum, wg[6], wh[6], wg[7], wh[7], x1.z, x1.w);
            const float sg = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(scale_g + grp * 2u)));
            const float sh = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(scale_h + grp * 2u)));
            acc[0] = fmaf(sum[0], sg, acc[0]);
            acc[1] = fmaf(sum[1], sg, acc[1]);
            acc[2] = fmaf(sum[2], sh, acc[2]);
            acc[3] = fmaf(sum[3], sh, acc[3]);
        }
        code_g += 48u;
        code_h += 48u;
        scale_g += 4u;
        scale_h += 4u;
        x_lane += x_step;
        offset_lane += 8u;
    }
    float* mine = partial + warp * 128u;
    mine[g * 8u + 2u * q] = acc[0];
    mine[g * 8u + 2u * q + 1u] = acc[1];
    mine[(g + 8u) * 8u + 2u * q] = acc[2];
    mine[(g + 8u) * 8u + 2u * q + 1u] = acc[3];
    __syncthreads();

    if (split == 1u) {
        for (uint32_t i = tid; i < kRb * rows; i += kThreads) {
            const uint32_t t = i / kRb, r = i - t * kRb;
            const float total = partial[(r >> 4) * 256u + (r & 15u) * 8u + t] + partial[(r >> 4) * 256u + 128u + (r & 15u) * 8u + t];
            y[(uint64_t)t * n + row0 + r] = eb::float_to_bf16_bits(total);
        }
        return;
    }
    const uint32_t gather0 = eb::map_to_rank(eb::smem_u32(gather), 0);
    for (uint32_t i = tid; i < kRb * 8u; i += kThreads) {
        const uint32_t r = i >> 3, t = i & 7u;
        const float total = partial[(r >> 4) * 256u + (r & 15u) * 8u + t] + partial[(r >> 4) * 256u + 128u + (r & 15u) * 8u + t];
        eb::st_cluster_f32(gather0 + ((rank * kRb + r) * 8u + t) * 4u, total);
    }
    eb::cluster_sync();
    if (rank != 0u) return;
    for (uint32_t i = tid; i < kRb * rows; i += kThreads) {
        const uint32_t t = i / kRb, r = i - t * kRb;
        float total = gather[r * 8u + t];
        for (uint32_t s = 1; s < split; ++s) total += gather[(s * kRb + r) * 8u + t];
        y[(uint64_t)t * n + row0 + r] = eb::float_to_bf16_bits(total);
    }
}

}  // namespace q3
