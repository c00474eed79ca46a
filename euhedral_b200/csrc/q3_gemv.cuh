// Q3G64_F16S policy of the decode GEMV (gemv_stream.cuh): W in the converter's row-split layout (groups of 64 three-bit
// codes in 24 bytes, one FP16 scale per group in a second plane).
//
// Replaces the reference's contiguous decode kernels native/src/q3/kernels.cu:11-41 (body
// native/src/q3/contiguous.cuh:55-223) behind euhedral_cuda_linear_q3_bf16 (native/src/host/q3_linear_bf16.c:73-102).
// Same contract: products x * code are exact, a group's 64 products are summed in FP32 and multiplied once by the FP32
// value of the FP16 group scale, the output is BF16 round-to-nearest-even, and every activation row is computed
// independently of the others (row exactness).
//
// The reference spends one FP32 FMA per weight and activation row, which B200's ratio of ALU rate to HBM bandwidth
// cannot pay for. Here the sums run on the tensor core: one mma.sync.m16n8k16 covers 16 weight rows x 16 K values x 8
// activation rows, four MMAs cover one group, and the group's FP32 scale is applied to the group's accumulator (an
// FP16 scale is not exact in BF16, so it cannot be folded into the operand).
//
// The cost that matters is integer instructions per code, so a code is never moved to a fixed bit position and never
// has its bias subtracted:
//   * A lane owns 16 consecutive codes (48 bits) of a group for rows g and g+8: lane q's bits start at bit 48 q of the
//     group's 192. Codes j and j+5 (j < 5) and codes 10+j and 13+j (j < 3) are brought 16 bits apart, so one mask
//     yields both halves of a BF16x2 register.
//   * A 3-bit field f sitting at mantissa bits 0..2 of the BF16 0x4300 reads 128 + f, and at mantissa bits 3..5 it reads
//     128 + 8 f. Two codes are therefore taken per shift; the activations that meet a field at bits 3..5 are staged
//     pre-multiplied by 1/8 (exact in BF16).
//   * f = code XOR 4 is the stored code plus 4 (the XOR rides in the same logic instruction as the mask). The bias, 132
//     per plain activation and 16 + 4 per pre-divided one, is removed by starting the group's accumulator at minus the
//     biased sum of the group's activations, computed once per CTA when the activations are staged.
#pragma once

#include "gemv_stream.cuh"

namespace q3 {

constexpr uint32_t kChunk = gemv::kChunk;   // K values per chunk: two groups, 48 code bytes and two FP16 scales per row

// Byte geometry (tools/euhedral_artifacts/grouped.py:24-36; native/src/host/q3_linear_bf16.c:82-84).
struct Geometry {
    uint64_t groups, row_bytes, scale_row_bytes, scale_offset, size;
    __host__ __device__ Geometry(uint32_t rows, uint32_t k) {
        groups = ((uint64_t)k + 127u) / 128u * 2u;
        row_bytes = groups * 24u;
        scale_row_bytes = groups * 2u;
        scale_offset = ((uint64_t)rows * row_bytes + 255ull) & ~255ull;
        size = scale_offset + (uint64_t)rows * groups * 2u;
    }
};

// Pair p of a lane's 16 codes: (low code, high code). Pairs 1, 3 and 6 are decoded at mantissa bits 3..5 (times 8).
__host__ __device__ constexpr int pair_lo(int p) { return p < 5 ? p : p + 5; }
__host__ __device__ constexpr int pair_hi(int p) { return p < 5 ? p + 5 : p + 8; }
__host__ __device__ constexpr bool pair_times8(int p) { return p == 1 || p == 3 || p == 6; }

// The (x[lo], x[hi]) register of pair P from 16 consecutive BF16 activations held in s[0..7] (two per register),
// multiplied by 1/8 for the pairs whose codes are decoded times 8.
template <int P>
__device__ __forceinline__ uint32_t pair_x(const uint32_t (&s)[8]) {
    constexpr int lo = pair_lo(P), hi = pair_hi(P);
    constexpr uint32_t selector = (uint32_t)((lo & 1) * 2) | (uint32_t)((lo & 1) * 2 + 1) << 4 | (uint32_t)(4 + (hi & 1) * 2) << 8
            | (uint32_t)(4 + (hi & 1) * 2 + 1) << 12;
    const uint32_t v = __byte_perm(s[lo >> 1], s[hi >> 1], selector);
    return pair_times8(P) ? eb::bf16x2_mul(v, 0x3E003E00u) : v;
}

// The bias weight of activation e (0..15) of a lane's 16: 132 where its code is decoded plain, 16 + 4 where times 8.
__host__ __device__ constexpr bool element_times8(int e) { return e == 1 || e == 3 || e == 6 || e == 8 || e == 11 || e == 14; }

struct Masks {
    uint32_t field1, magic1, field8, magic8;
    __device__ Masks()
        : field1(eb::pinned(0x00070007u)), magic1(eb::pinned(0x43044304u)), field8(eb::pinned(0x00380038u)),
          magic8(eb::pinned(0x43204320u)) {}
};

// Eight BF16x2 registers for the 16 codes of the 48 bits (a32 | b16 << 32), in pair order: 128 + (code ^ 4) for the
// plain pairs, 128 + 8 (code ^ 4) for pairs 1, 3 and 6. Bits of b16 above 16 are ignored.
__device__ __forceinline__ void decode16(uint32_t a32, uint32_t b16, const Masks& m, uint32_t (&out)[8]) {
    // Codes 0..4 at bits 0,3,..,12 of the low half and codes 5..9 at the same bits of the high half (bits 15 and 31 hold
    // leftovers that the masks below never select).
    const uint32_t z = eb::lop3_imm<eb::kLutSelect, 0x00007FFFu>(a32, a32 << 1);
    // Codes 10..15 start at bit 30: bring them to bit 0, then 10..12 low and 13..15 high.
    const uint32_t y = __funnelshift_r(a32, b16, 30);
    const uint32_t z2 = eb::lop3_imm<eb::kLutSelect, 0x000001FFu>(y, y << 7);
    const uint32_t z6 = z >> 6;
    out[0] = eb::lop3<eb::kLutAndXor>(z, m.field1, m.magic1);
    out[1] = eb::lop3<eb::kLutAndXor>(z, m.field8, m.magic8);
    out[2] = eb::lop3<eb::kLutAndXor>(z6, m.field1, m.magic1);
    out[3] = eb::lop3<eb::kLutAndXor>(z6, m.field8, m.magic8);
    out[4] = eb::lop3<eb::kLutAndXor>(z >> 12, m.field1, m.magic1);
    out[5] = eb::lop3<eb::kLutAndXor>(z2, m.field1, m.magic1);
    out[6] = eb::lop3<eb::kLutAndXor>(z2, m.field8, m.magic8);
    out[7] = eb::lop3<eb::kLutAndXor>(z2 >> 6, m.field1, m.magic1);
}

struct Format {
    using Geometry = q3::Geometry;
    static constexpr uint32_t kCodeBytes = 48, kScaleBytes = 4, kErrorBit = 2;
    // A piece is at most 5 chunks (3.75 KB of codes per 16 rows). The scale box, 48 bytes per row, covers 5 chunks' scales
    // plus the 12 bytes a piece can start after a 16-byte boundary, and is an odd multiple of 16.
    static constexpr bool kAddingWarp = false;
    static constexpr uint32_t kPieceChunks = 5, kMaxPiece = 5, kScaleBox = 48;
    // float [chunk][group][lane q][4]: minus the biased sum of the group's activations of rows 2q and 2q+1, twice over
    // (x, y, x, y), which is the accumulator quad lane q starts a group with.
    __host__ __device__ static constexpr uint32_t extra_bytes(uint32_t chunks) { return chunks * 128u; }
    __device__ static uint32_t lane_scale_offset(uint32_t) { return 0; }

    // One unit = 16 consecutive activations of one row, (row, chunk, group, quarter): stored in the decode's pairing for
    // the lane quartet that reads it. The four quarters of a group sit in four neighbouring lanes, which add their
    // biased sums in a fixed order ((q0 + q1) + (q2 + q3)).
    __device__ static void stage(uint8_t* xs, uint8_t* extra, const uint16_t* __restrict__ x, uint32_t rows, uint32_t k,
            uint32_t c_begin, uint32_t nc, uint32_t stride_x, uint32_t tid, uint32_t threads) {
        float* bias = reinterpret_cast<float*>(extra);
        // Activation rows beyond `rows` have no bias: their MMA columns are never stored. A thread takes up to kTurns units
        // per pass and issues the loads of all of them before it touches the first, so that one memory latency covers them.
        constexpr uint32_t kTurns = 4;
        const uint32_t per_row = nc * 8u, total = rows * per_row;
        for (uint32_t base = 0; base < total; base += kTurns * threads) {
            uint4 v0[kTurns], v1[kTurns];
#pragma unroll
            for (uint32_t turn = 0; turn < kTurns; ++turn) {
                const uint32_t unit = base + turn * threads + tid;
                if (unit < total) {
                    const uint32_t t = unit / per_row, j = unit - t * per_row;
                    const uint32_t c = j >> 3, grp = (j >> 2) & 1u, qq = j & 3u;
                    const uint4* src = reinterpret_cast<const uint4*>(x + (uint64_t)t * k + (uint64_t)(c_begin + c) * kChunk + grp * 64u + qq * 16u);
                    v0[turn] = src[0];
                    v1[turn] = src[1];
                }
            }
#pragma unroll
            for (uint32_t turn = 0; turn < kTurns; ++turn) {
                const uint32_t unit = base + turn * threads + tid;
                if (unit < total) {   // whole quartets of neighbouring lanes take the branch together (the unit count is a multiple of 4)
                    const uint32_t t = unit / per_row, j = unit - t * per_row;
                    const uint32_t c = j >> 3, grp = (j >> 2) & 1u, qq = j & 3u;
                    const uint32_t s[8] = {v0[turn].x, v0[turn].y, v0[turn].z, v0[turn].w, v1[turn].x, v1[turn].y, v1[turn].z, v1[turn].w};
                    uint8_t* dst = xs + t * stride_x + c * 256u + grp * 128u + qq * 16u;
                    *reinterpret_cast<uint4*>(dst) = make_uint4(pair_x<0>(s), pair_x<1>(s), pair_x<2>(s), pair_x<3>(s));
                    *reinterpret_cast<uint4*>(dst + 64u) = make_uint4(pair_x<4>(s), pair_x<5>(s), pair_x<6>(s), pair_x<7>(s));
                    // Two chains of eight additions in element order (plain elements, elements met times 8), then the lanes
                    // of the quartet in the order ((q0 + q1) + (q2 + q3)).
                    float plain = 0.0f, eighth = 0.0f;
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const float value = (e & 1) ? __uint_as_float(s[e >> 1] & 0xFFFF0000u) : eb::bf16_bits_to_float(s[e >> 1] & 0xFFFFu);
                        if (element_times8(e)) eighth = __fadd_rn(eighth, value);
                        else plain = __fadd_rn(plain, value);
                    }
                    float sum = __fmaf_rn(20.0f, eighth, __fmul_rn(132.0f, plain));
                    sum = __fadd_rn(sum, __shfl_xor_sync(__activemask(), sum, 1));
                    sum = __fadd_rn(sum, __shfl_xor_sync(__activemask(), sum, 2));
                    if (qq == 0u) {
                        float* quad = bias + ((c * 2u + grp) * 4u + (t >> 1)) * 4u + (t & 1u);
                        quad[0] = quad[2] = -sum;
                    }
                }
            }
        }
    }

    template <int P>
    struct State {
        float acc[4];
        uint32_t bias_lane;   // shared address of the bias of activation rows 2q, 2q + 1 of the piece's first chunk
        uint32_t first_word, second_word, select_low, select_high;
        Masks masks;
        // Lane q's 48 bits of a group start at 32-bit word {0, 1, 3, 4}[q] of the group's six, at bit 16 of it for odd q,
        // and end in the next word. The two words are fetched by two loads whose lane-to-word maps, {0, 2, 3, 5} and
        // {1, 1, 4, 4}, keep a warp's 32 addresses in 32 distinct banks when the box rows are 4 words apart modulo 32 (a
        // piece of 3 or 5 chunks): even lanes get their lower word first, odd lanes their upper word. One byte permute
        // with a lane constant then yields bits 0..31 of the lane's 48, another bits 32..47.
        __device__ State(uint32_t extra, uint32_t q)
            : bias_lane(eb::pinned(extra + q * 16u)), first_word(eb::pinned(((q >> 1) * 3u + (q & 1u) * 2u) * 4u)),
              second_word(eb::pinned(((q >> 1) * 3u + 1u) * 4u)), select_low(eb::pinned((q & 1u) ? 0x1076u : 0x3210u)),
              select_high(eb::pinned((q & 1u) ? 0x3232u : 0x7654u)) {}
        __device__ __forceinline__ void tensor(const uint8_t*, const Geometry&) {}   // nothing is kept per tensor
        // codes: shared address of row g of the piece's code box (rows are W chunks wide, row g + 8 eight rows further);
        // scales: of the two FP16 scales of row g and the piece's first chunk (row g + 8: 8 * kScaleBox further);
        // x: of the lane's activations of the piece's first chunk.
        template <int I, int W>
        __device__ __forceinline__ void chunk(uint32_t codes, uint32_t scales, uint32_t x) {
            constexpr int kRow8 = 8 * W * (int)kCodeBytes, kAt = I * (int)kCodeBytes;
            const uint32_t scales_g = eb::lds_u32<I * 4>(scales), scales_h = eb::lds_u32<I * 4 + 8 * (int)kScaleBox>(scales);
            const float2 sg2 = __half22float2(*reinterpret_cast<const __half2*>(&scales_g));
            const float2 sh2 = __half22float2(*reinterpret_cast<const __half2*>(&scales_h));
            const uint32_t first = codes + first_word, second = codes + second_word;
            uint32_t ga[2], gb[2], ha[2], hb[2];   // a: the word fetched first, b: second (which is lower depends on the lane)
            ga[0] = eb::lds_u32<kAt>(first);
            gb[0] = eb::lds_u32<kAt>(second);
            ha[0] = eb::lds_u32<kAt + kRow8>(first);
            hb[0] = eb::lds_u32<kAt + kRow8>(second);
            ga[1] = eb::lds_u32<kAt + 24>(first);
            gb[1] = eb::lds_u32<kAt + 24>(second);
            ha[1] = eb::lds_u32<kAt + kRow8 + 24>(first);
            hb[1] = eb::lds_u32<kAt + kRow8 + 24>(second);
            const uint4 xv[4] = {eb::lds_v4<I * 256>(x), eb::lds_v4<I * 256 + 64>(x), eb::lds_v4<I * 256 + 128>(x), eb::lds_v4<I * 256 + 192>(x)};
            const float4 bias[2] = {eb::lds_f4<I * 128>(bias_lane), eb::lds_f4<I * 128 + 64>(bias_lane)};
#pragma unroll
            for (int grp = 0; grp < 2; ++grp) {
                uint32_t wg[8], wh[8];
                decode16(__byte_perm(ga[grp], gb[grp], select_low), __byte_perm(ga[grp], gb[grp], select_high), masks, wg);
                decode16(__byte_perm(ha[grp], hb[grp], select_low), __byte_perm(ha[grp], hb[grp], select_high), masks, wh);
                float sum[4];
                eb::mma_bf16_16816_from(sum, wg[0], wh[0], wg[1], wh[1], xv[2 * grp].x, xv[2 * grp].y, bias[grp]);
                eb::mma_bf16_16816(sum, wg[2], wh[2], wg[3], wh[3], xv[2 * grp].z, xv[2 * grp].w);
                eb::mma_bf16_16816(sum, wg[4], wh[4], wg[5], wh[5], xv[2 * grp + 1].x, xv[2 * grp + 1].y);
                eb::mma_bf16_16816(sum, wg[6], wh[6], wg[7], wh[7], xv[2 * grp + 1].z, xv[2 * grp + 1].w);
                const float sg = grp == 0 ? sg2.x : sg2.y, sh = grp == 0 ? sh2.x : sh2.y;
                acc[0] = fmaf(sum[0], sg, acc[0]);
                acc[1] = fmaf(sum[1], sg, acc[1]);
                acc[2] = fmaf(sum[2], sh, acc[2]);
                acc[3] = fmaf(sum[3], sh, acc[3]);
            }
        }
        __device__ __forceinline__ void result(float (&out)[4]) const {
#pragma unroll
            for (int i = 0; i < 4; ++i) out[i] = acc[i];
        }
        __device__ __forceinline__ void reset() {
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = 0.0f;
        }
    };

    struct Finish {
        __device__ Finish(const uint8_t*, const Geometry&) {}
        __device__ __forceinline__ float apply(float sum) const { return sum; }
    };
};

}  // namespace q3
