// NVFP4 policy of the decode GEMV (gemv_stream.cuh): W in the converter's row-split NVFP4 layout (E2M1 codes two per
// byte, one E4M3 scale per 16 values, one FP32 scale per tensor).
//
// Replaces the reference's decode kernels native/src/nvfp4/kernels.cu:8-36 (body native/src/nvfp4/nvfp4.cuh:97-198)
// behind euhedral_cuda_linear_nvfp4_bf16 (native/src/host/nvfp4_linear.c:124-146). Same contract: products
// x * (e2m1 * e4m3) are exact, accumulation is FP32, the FP32 tensor scale multiplies the sum, the output is BF16
// round-to-nearest-even, and every activation row is computed independently of the others (row exactness).
//
// Decode in registers: a lane owns 32 consecutive K values (16 code bytes) of rows g and g+8. Nibbles i and i+4 of a
// 32-bit word become one BF16x2 register by a mask, one integer multiply and a mask: the multiply by 2^12 + 2^6 lays
// two copies of each nibble down, one with its sign on the BF16 sign bit and one with its three magnitude bits where
// BF16 keeps its two low exponent bits and its top mantissa bit, which reads as e2m1 * 2^-126 (subnormal included).
// The multiply runs on the FMA pipe, which leaves the integer pipe - the scarce one on sm_100 - two logic operations
// per register. One packed multiply by (e4m3 * 2^110) then gives e2m1 * e4m3 * 2^-16 exactly. The activations are
// staged in shared memory in the matching (x[i], x[i+4]) pairing. Even and odd MMAs of a chunk feed two accumulators
// that are added at the end; the 2^16 and the tensor scale multiply the final sum.
#pragma once

#include "gemv_stream.cuh"

namespace nvfp4 {

constexpr uint32_t kChunk = gemv::kChunk;   // K values per chunk: 64 code bytes and 8 scale bytes per row

__host__ __device__ inline uint64_t align256(uint64_t v) { return (v + 255ull) & ~255ull; }

// Byte geometry of a tensor (tools/euhedral_artifacts/nvfp4.py:49-57; native/src/host/nvfp4_linear.c:79-91).
struct Geometry {
    uint64_t row_bytes, row_scales, scale_row_bytes, scale_offset, global_offset, size;
    __host__ __device__ Geometry(uint32_t rows, uint32_t k) {
        const uint64_t kp = ((uint64_t)k + 127u) / 128u * 128u;
        row_bytes = kp / 2u;
        row_scales = scale_row_bytes = kp / 16u;
        scale_offset = align256((uint64_t)rows * row_bytes);
        global_offset = align256(scale_offset + (uint64_t)rows * row_scales);
        size = global_offset + 4u;
    }
};

// The four BF16x2 registers of a code word: register i holds nibbles i and i+4 as e2m1 * 2^-126 each.
__device__ __forceinline__ void raw_word(uint32_t v, uint32_t (&r)[4]) {
    const uint32_t u = v >> 8;
    r[0] = ((v & 0x000F000Fu) * 4160u) & 0x81C081C0u;   // nibble at bit 0: copies at bits 12 and 6
    r[1] = ((v & 0x00F000F0u) * 260u) & 0x81C081C0u;    // nibble at bit 4: copies at bits 12 and 6
    r[2] = ((u & 0x000F000Fu) * 4160u) & 0x81C081C0u;
    r[3] = ((u & 0x00F000F0u) * 260u) & 0x81C081C0u;
}

// (e4m3 * 2^110) of the two scale bytes in `bits` as BF16x2 (low byte in the low half). A byte shifted left by 4 is a
// BF16 holding e4m3 * 2^-120 (subnormal codes included; bit 7 of the byte is ignored); two exact multiplies rescale it.
__device__ __forceinline__ uint32_t scale_pair(uint32_t bits) {
    const uint32_t t = bits & 0x00007F7Fu;
    const uint32_t raw = ((t * 16u) | (t * 4096u)) & 0x07F007F0u;   // low byte to bits 4..10, high byte to bits 20..26
    const uint32_t unit = eb::bf16x2_mul(raw, 0x7B807B80u);   // * 2^120 -> e4m3
    return eb::bf16x2_mul(unit, 0x76807680u);                  // * 2^110
}

// Byte geometry of a tensor whose block scales are 4-bit indices into a table of 16 E4M3 codes (layout
// row-split-k128-sd4-v1, tools/euhedral_artifacts/nvfp4.py:60-69): the index plane is half the scale plane (two indices
// per byte, the even block in the low nibble), then the table, then the FP32 tensor scale.
struct GeometrySd4 {
    uint64_t row_bytes, scale_row_bytes, scale_offset, table_offset, global_offset, size;
    __host__ __device__ GeometrySd4(uint32_t rows, uint32_t k) {
        const uint64_t kp = ((uint64_t)k + 127u) / 128u * 128u;
        row_bytes = kp / 2u;
        scale_row_bytes = kp / 32u;
        scale_offset = align256((uint64_t)rows * row_bytes);
        table_offset = align256(scale_offset + (uint64_t)rows * scale_row_bytes);
        global_offset = table_offset + 16u;
        size = table_offset + 20u;
    }
};

// Where a lane's block scales come from. Plain: two E4M3 bytes per lane and chunk, read as they are.
struct PlainScales {
    using Geometry = nvfp4::Geometry;
    static constexpr uint32_t kScaleBytes = 8, kScaleBox = 80;   // 80 bytes per row: an odd multiple of 16
    __device__ static uint32_t lane_scale_offset(uint32_t q) { return 2u * q; }
    __device__ __forceinline__ void tensor(const uint8_t*, const Geometry&) {}
    // The lane's two E4M3 bytes (low byte: its first block of 16) of chunk I at shared address `scales` + OFFSET rows' bytes.
    template <int I, int OFFSET>
    __device__ __forceinline__ uint32_t read(uint32_t scales) const { return eb::lds_u16<I * 8 + OFFSET>(scales); }
};

// Table-indexed (SD4): one byte per lane and chunk holds the two 4-bit indices; the tensor's 16 codes sit in four
// registers and one byte permute per half of the table plus a select on each index's top bit looks both up at once
// (the reference's twin kernels look four up at a time the same way, native/src/nvfp4/scale_table.cuh:4-15).
struct TableScales {
    using Geometry = GeometrySd4;
    static constexpr uint32_t kScaleBytes = 4, kScaleBox = 48;
    __device__ static uint32_t lane_scale_offset(uint32_t q) { return q; }
    uint4 table;
    __device__ __forceinline__ void tensor(const uint8_t* w, const Geometry& geo) { table = *reinterpret_cast<const uint4*>(w + geo.table_offset); }
    template <int I, int OFFSET>
    __device__ __forceinline__ uint32_t read(uint32_t scales) const {
        uint32_t pair;
        asm volatile("ld.shared.u8 %0, [%1 + %2];" : "=r"(pair) : "r"(scales), "n"(I * 4 + OFFSET));
        const uint32_t within = pair & 0x77u;   // per nibble: which of the eight codes of a table half
        const uint32_t low = __byte_perm(table.x, table.y, within), high = __byte_perm(table.z, table.w, within);
        // byte 0 all ones when index 0 is 8 or more, byte 1 when index 1 is: a byte of ones (selector 4) or of zeros (0)
        const uint32_t upper = __byte_perm(0u, 0xFFFFFFFFu, (pair >> 1) & 0x44u);
        return eb::lop3<eb::kLutSelect>(high, low, upper) & 0xFFFFu;
    }
};

template <class Scales>
struct FormatOf {
    using Geometry = typename Scales::Geometry;
    static constexpr uint32_t kCodeBytes = 64, kScaleBytes = Scales::kScaleBytes, kErrorBit = 1;
    // A piece is at most 4 chunks (4 KB of codes per 16 rows): with sixteen warps and a ring of two slots each that leaves
    // room for the activations of 5 rows at K = 5120. The scale box, 80 bytes per row, is an odd multiple of 16.
    static constexpr bool kAddingWarp = true;
    static constexpr uint32_t kPieceChunks = 3, kMaxPiece = 4, kScaleBox = Scales::kScaleBox;
    __host__ __device__ static constexpr uint32_t extra_bytes(uint32_t) { return 0; }
    __device__ static uint32_t lane_scale_offset(uint32_t q) { return Scales::lane_scale_offset(q); }

    // x[t][c][i][qq] <- the (x0,x4) (x1,x5) (x2,x6) (x3,x7) pairs of the eight activations 8 i .. 8 i + 7 of quarter qq.
    __device__ static void stage(uint8_t* xs, uint8_t*, const uint16_t* __restrict__ x, uint32_t rows, uint32_t k, uint32_t c_begin,
            uint32_t nc, uint32_t stride_x, uint32_t tid, uint32_t threads) {
        // A thread takes up to kTurns 16-byte units per pass and issues all their loads before the first store.
        constexpr uint32_t kTurns = 4;
        const uint32_t total = rows * nc * 16u;
        for (uint32_t base = 0; base < total; base += kTurns * threads) {
            uint4 v[kTurns];
#pragma unroll
            for (uint32_t turn = 0; turn < kTurns; ++turn) {
                const uint32_t u = base + turn * threads + tid;
                if (u < total) {
                    const uint32_t t = u / (nc * 16u), j = u - t * (nc * 16u);
                    const uint32_t c = j >> 4, qq = (j >> 2) & 3u, i = j & 3u;
                    v[turn] = *reinterpret_cast<const uint4*>(x + (uint64_t)t * k + (uint64_t)(c_begin + c) * kChunk + qq * 32u + i * 8u);
                }
            }
#pragma unroll
            for (uint32_t turn = 0; turn < kTurns; ++turn) {
                const uint32_t u = base + turn * threads + tid;
                if (u < total) {
                    const uint32_t t = u / (nc * 16u), j = u - t * (nc * 16u);
                    const uint32_t c = j >> 4, qq = (j >> 2) & 3u, i = j & 3u;
                    uint4 p;
                    p.x = __byte_perm(v[turn].x, v[turn].z, 0x5410);   // (x0, x4)
                    p.y = __byte_perm(v[turn].x, v[turn].z, 0x7632);   // (x1, x5)
                    p.z = __byte_perm(v[turn].y, v[turn].w, 0x5410);   // (x2, x6)
                    p.w = __byte_perm(v[turn].y, v[turn].w, 0x7632);   // (x3, x7)
                    *reinterpret_cast<uint4*>(xs + t * stride_x + c * 256u + i * 64u + qq * 16u) = p;
                }
            }
        }
    }

    template <int P>
    struct State {
        float even[4], odd[4];
        uint32_t lane_codes;   // byte offset of the lane's 16 code bytes within a chunk
        Scales source;         // what turns the slot's scale bytes into E4M3 codes (per tensor: the table, if any)
        __device__ State(uint32_t, uint32_t q) : lane_codes(eb::pinned(q * 16u)) {}
        __device__ __forceinline__ void tensor(const uint8_t* w, const Geometry& geo) { source.tensor(w, geo); }
        // codes: shared address of row g of the piece's code box (rows are W chunks wide, row g + 8 eight rows further);
        // scales: of the lane's two scale bytes of row g and the piece's first chunk (row g + 8: 8 * kScaleBox further);
        // x: of the lane's activations of the piece's first chunk.
        template <int I, int W>
        __device__ __forceinline__ void chunk(uint32_t codes, uint32_t scales, uint32_t x) {
            constexpr int kRow8 = 8 * W * (int)kCodeBytes, kAt = I * (int)kCodeBytes;
            const uint4 cg = eb::lds_v4<kAt>(codes + lane_codes);
            const uint4 ch = eb::lds_v4<kAt + kRow8>(codes + lane_codes);
            const uint32_t sg = scale_pair(source.template read<I, 0>(scales)), sh = scale_pair(source.template read<I, 8 * (int)kScaleBox>(scales));
            const uint32_t sg_block[2] = {__byte_perm(sg, sg, 0x1010), __byte_perm(sg, sg, 0x3232)};
            const uint32_t sh_block[2] = {__byte_perm(sh, sh, 0x1010), __byte_perm(sh, sh, 0x3232)};
            const uint32_t wg[4] = {cg.x, cg.y, cg.z, cg.w}, wh[4] = {ch.x, ch.y, ch.z, ch.w};
            const uint4 xv[4] = {eb::lds_v4<I * 256>(x), eb::lds_v4<I * 256 + 64>(x), eb::lds_v4<I * 256 + 128>(x), eb::lds_v4<I * 256 + 192>(x)};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t fg = sg_block[i >> 1], fh = sh_block[i >> 1];
                uint32_t rg[4], rh[4];
                raw_word(wg[i], rg);
                raw_word(wh[i], rh);
                eb::mma_bf16_16816(even, eb::bf16x2_mul(rg[0], fg), eb::bf16x2_mul(rh[0], fh), eb::bf16x2_mul(rg[1], fg),
                        eb::bf16x2_mul(rh[1], fh), xv[i].x, xv[i].y);
                eb::mma_bf16_16816(odd, eb::bf16x2_mul(rg[2], fg), eb::bf16x2_mul(rh[2], fh), eb::bf16x2_mul(rg[3], fg),
                        eb::bf16x2_mul(rh[3], fh), xv[i].z, xv[i].w);
            }
        }
        __device__ __forceinline__ void result(float (&out)[4]) const {
#pragma unroll
            for (int i = 0; i < 4; ++i) out[i] = even[i] + odd[i];
        }
        __device__ __forceinline__ void reset() {
#pragma unroll
            for (int i = 0; i < 4; ++i) even[i] = odd[i] = 0.0f;
        }
    };

    struct Finish {
        float global;
        __device__ Finish(const uint8_t* w, const Geometry& geo) : global(*reinterpret_cast<const float*>(w + geo.global_offset)) {}
        __device__ __forceinline__ float apply(float sum) const { return sum * 65536.0f * global; }
    };
};

using Format = FormatOf<PlainScales>;      // row-split-k128-v1
using FormatSd4 = FormatOf<TableScales>;   // row-split-k128-sd4-v1

}  // namespace nvfp4
