// Trellis (trellis-tile16-v1) linear for decode-sized row counts on sm_100a.
//
// What the format and the reference's host fix (native/src/host/linear_kernels.c:7-24 names the table entries; the Java
// host plans them, core/.../artifact/format/TrellisFormat.java:484-567):
//   entry 0 "prepass":  act[g][r] = fp16(H128(bf16 x[r] * fp16 suh[g])), FP16 in the MMA fragment order of the scratch
//   entry 1 "mma":      z = act . Q over K split i = tile rows [i T / S, (i + 1) T / S), FP16 x FP16 -> FP32
//   entry 4 "epilogue": y = bf16(svh * H128(sum of the splits in split order))
//   entry 5 "decode":   the rotated weight as BF16 [n][k]
// and the scratch layout between them (activations, then FP32 partials [split][row][n]).
//
// How it runs here: ONE kernel does a whole linear. A CTA owns 128 output columns and one K split.
//   * Warp 8 only requests payload: one tiled TMA copy per stage (16 tile rows x the CTA's 8 tiles), a ring of stages
//     with a full and an empty mbarrier each, so the eight decoding warps drift apart by up to a ring instead of meeting
//     at a CTA barrier every stage.
//   * Warps 0-7 each own one tile column. The rotated activations of the CTA's K range are made here, as many tile rows at
//     a time as fit (all of them for the usual split), straight into shared memory (from x and suh, or copied from the scratch when the caller ran entry 0), in the
//     order the decode below wants them; nothing goes through global memory between "prepass" and "mma".
//   * A lane decodes its eight consecutive trellis states from registers; the byte sums of the codebook hash are taken by
//     the tensor core (two m16n8k32 u8 MMAs against a 0/1 selector, accumulator preset to the FP16 bit pattern 0x6400),
//     which also hands each lane the values in the order of its FP16 A fragment; the 16 k of a tile reach the FP16 MMA in
//     a fixed permutation that the activations in shared memory follow.
//   * The K splits meet without a second launch and without a counter that would need clearing: a CTA stores its FP32
//     partials, publishes a flag holding this call's tag, and reads the flags of its column block; whoever sees all of
//     them set adds the partials in split order, rotates, scales and writes BF16, then unsets the flags (a launch replayed
//     from a CUDA graph carries the same tag again). Two CTAs that finish together may both do that; they write the same bits.
// Table entries 0, 1, 4 stay callable one by one (their outputs and the scratch layout are the contract); entry 1 is the
// same kernel reading the activations from the scratch and leaving the partials to entry 4.
#pragma once

#include "common.cuh"
#include "trellis_codebook.cuh"

namespace trellis {

// The stored tile widths (16-bit words per tile): X(w) for each.
#define EB_TRELLIS_WIDTHS(X) X(16) X(24) X(32) X(40) X(48) X(56) X(64) X(72) X(80) X(88) X(96) X(104) X(112) X(120) X(128)

constexpr int kStageTiles = 16;                       // tile rows (k16 steps) per streaming stage
constexpr int kStages = 3;
constexpr int kResident = 3;                          // CTAs of up to 8 rows an SM holds (72 registers a thread)
constexpr int kUnroll = 8;                            // tiles decoded per trip of the inner loop
constexpr int kChunkLimit = 512;                      // most tile rows whose activations are in shared memory at once
constexpr int kDecodeWarps = 8;                       // one per tile column of the CTA's 128 output columns
constexpr int kThreads = 32 * (kDecodeWarps + 1);     // and the warp that requests the payload
// Shared memory for the activations of a chunk: the live rows only, each chunk * 32 + 32 bytes long (32 modulo 128: the
// 8 rows x 4 quads of one load tile the banks). 8 rows get 64 tile rows, 5 rows 96, one row 512; 32 rows get 32.
__host__ __device__ constexpr uint32_t act_bytes(int groups) { return groups == 1 ? 8u * (64u * 32u + 32u) : 32u * (32u * 32u + 32u); }
__host__ __device__ inline int chunk_tiles(int groups, int live) {
    const int fit = (int)((act_bytes(groups) / (uint32_t)live - 32u) / 32u) & ~7;
    return fit < kChunkLimit ? fit : kChunkLimit;
}
constexpr int kBatch = 4;                             // tiles a warp of the BF16 decode takes side by side
constexpr uint32_t kWaitFailed = 4u;                  // error bit: a stage did not arrive (or was never freed)

// ---- pieces shared by the one-kernel linear and the table entries -------------------------------------------------------

// One warp: 128 columns of x (BF16) times suh (FP16), rotated; the lane keeps columns 4 lane .. 4 lane + 3.
__device__ __forceinline__ void rotate128(const uint16_t* __restrict__ x, const uint16_t* __restrict__ suh, int lane, float (&v)[4]) {
    const uint2 xb = *reinterpret_cast<const uint2*>(x + 4 * lane);
    const uint2 sb = *reinterpret_cast<const uint2*>(suh + 4 * lane);
    const uint32_t xw[2] = {xb.x, xb.y}, sw[2] = {sb.x, sb.y};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t xs = (xw[j >> 1] >> (16 * (j & 1))) & 0xFFFFu, ss = (sw[j >> 1] >> (16 * (j & 1))) & 0xFFFFu;
        v[j] = __fmul_rn(eb::bf16_bits_to_float(xs), __half2float(__ushort_as_half((unsigned short)ss)));
    }
    hadamard128_warp(v, lane);
}

// Two floats rounded to nearest even into one BF16 pair by the hardware conversion (low half from `low`); for finite values
// the bits of eb::float_to_bf16_bits.
__device__ __forceinline__ uint32_t bf16_pair(float low, float high) {
    const __nv_bfloat162 both = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&both);
}

__device__ __forceinline__ uint32_t half_pair(float low, float high) {
    return (uint32_t)__half_as_ushort(__float2half_rn(low)) | (uint32_t)__half_as_ushort(__float2half_rn(high)) << 16;
}

// One warp: the lane's four sums of a 128-column block -> rotated, times svh (FP16), BF16 to out.
__device__ __forceinline__ void finish128(float (&v)[4], const uint16_t* __restrict__ svh, uint16_t* __restrict__ out, int lane) {
    hadamard128_warp(v, lane);
    const uint2 sb = *reinterpret_cast<const uint2*>(svh + 4 * lane);
    const uint32_t sw[2] = {sb.x, sb.y};
    uint32_t bits[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float scale = __half2float(__ushort_as_half((unsigned short)(sw[j >> 1] >> (16 * (j & 1)))));
        bits[j] = eb::float_to_bf16_bits(__fmul_rn(scale, v[j]));
    }
    *reinterpret_cast<uint2*>(out + 4 * lane) = make_uint2(bits[0] | bits[1] << 16, bits[2] | bits[3] << 16);
}

// One warp: partials[i * stride + 4 lane ..] of splits i = 0 .. splits - 1 added in that order (read past L1: other SMs
// wrote them), then finish128.
__device__ __forceinline__ void add_and_finish128(const float* __restrict__ partials, size_t stride, int splits,
        const uint16_t* __restrict__ svh, uint16_t* __restrict__ out, int lane) {
    float4 sum = __ldcg(reinterpret_cast<const float4*>(partials) + lane);
    for (int i = 1; i < splits; ++i) {
        const float4 part = __ldcg(reinterpret_cast<const float4*>(partials + (size_t)i * stride) + lane);
        sum.x = __fadd_rn(sum.x, part.x);
        sum.y = __fadd_rn(sum.y, part.y);
        sum.z = __fadd_rn(sum.z, part.z);
        sum.w = __fadd_rn(sum.w, part.w);
    }
    float v[4] = {sum.x, sum.y, sum.z, sum.w};
    finish128(v, svh, out, lane);
}

// ---- table entries 0, 4, 5 as launches of their own --------------------------------------------------------------------

// x bf16 [rows][k], suh f16 [s][k] -> out [s][rows][k]. layout 0: FP16 in the scratch's fragment order (of every 16 columns,
// columns 2q, 2q+1, 2q+8, 2q+9 sit together at 4q); layout 1: BF16 in column order. A warp per (segment, row, 128 columns).
//   grid ceil(s * rows * (k / 128) / 8), block 256.
__global__ void __launch_bounds__(256) rotate_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ suh,
        uint16_t* __restrict__ out, int rows, int k, int s, int layout) {
    const int lane = threadIdx.x & 31;
    const uint32_t blocks = (uint32_t)k >> 7, task = blockIdx.x * 8u + (threadIdx.x >> 5);   // the launch holds fewer than 2^31 tasks
    eb::pdl_launch_dependents();
    eb::pdl_wait();
    if (task >= (uint32_t)s * (uint32_t)rows * blocks) return;
    const uint32_t block = task % blocks, above = task / blocks, row = above % (uint32_t)rows, seg = above / (uint32_t)rows;
    float v[4];
    rotate128(x + (size_t)row * k + (size_t)block * 128, suh + (size_t)seg * k + (size_t)block * 128, lane, v);
    uint16_t* to = out + ((size_t)seg * rows + row) * k + (size_t)block * 128;
    if (layout == 0) {
        const int a = lane & 3;   // the lane's columns are 4a .. 4a+3 of group lane / 4: (4a, 4a+1) and (4a+2, 4a+3) are pairs
        uint32_t* group = reinterpret_cast<uint32_t*>(to + 16 * (lane >> 2));
        group[4 * (a & 1) + (a >> 1)] = half_pair(v[0], v[1]);
        group[4 * (a & 1) + (a >> 1) + 2] = half_pair(v[2], v[3]);
    } else {
        *reinterpret_cast<uint2*>(to + 4 * lane) = make_uint2(
                (uint32_t)eb::float_to_bf16_bits(v[0]) | (uint32_t)eb::float_to_bf16_bits(v[1]) << 16,
                (uint32_t)eb::float_to_bf16_bits(v[2]) | (uint32_t)eb::float_to_bf16_bits(v[3]) << 16);
    }
}

// The same rotation in the BF16 column layout for many rows (the prefill plan's prepass): a CTA of 128 threads takes 128
// consecutive 128-column blocks of one segment - 32 KB of x, which is contiguous - through shared memory: coalesced 16-byte
// loads in, a thread per block (the 128 values in registers, the seven butterfly stages without a shuffle: every a + b and
// a - b as hadamard128_warp forms them, so the bits are the same), coalesced 16-byte stores out.
//   grid (ceil(rows * (k / 128) / 128), s), block 128, static shared 128 x 272 bytes.
constexpr int kRotateRowsThreads = 128;
__global__ void __launch_bounds__(kRotateRowsThreads) rotate_rows_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ suh,
        uint16_t* __restrict__ out, uint32_t rows, uint32_t k) {
    constexpr uint32_t kPitch = 272;   // bytes of a block's row in shared memory: 256 + 16, so that 8 threads' 16-byte loads tile the banks
    __shared__ __align__(16) uint8_t stage[kRotateRowsThreads * kPitch];
    const uint32_t t = threadIdx.x, blocks = k >> 7, seg = blockIdx.y;
    const uint32_t total = rows * blocks, first = blockIdx.x * (uint32_t)kRotateRowsThreads;   // < 2^31 blocks per segment
    const uint32_t count = min((uint32_t)kRotateRowsThreads, total - first);
    eb::pdl_launch_dependents();
    eb::pdl_wait();
    const uint4* from = reinterpret_cast<const uint4*>(x + (size_t)first * 128);
#pragma unroll
    for (uint32_t i = 0; i < 16u; ++i) {
        const uint32_t chunk = i * kRotateRowsThreads + t;   // 16-byte chunk of the CTA's span: block chunk / 16, piece chunk % 16
        if (chunk < count * 16u) *reinterpret_cast<uint4*>(stage + (chunk >> 4) * kPitch + (chunk & 15u) * 16u) = from[chunk];
    }
    __syncthreads();
    if (t < count) {
        const uint32_t block = (first + t) % blocks;
        const uint4* scales = reinterpret_cast<const uint4*>(suh + (size_t)seg * k + (size_t)block * 128);
        uint8_t* mine = stage + t * kPitch;
        float v[128];
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const uint4 xb = *reinterpret_cast<const uint4*>(mine + 16 * c), sb = scales[c];
            const uint32_t xw[4] = {xb.x, xb.y, xb.z, xb.w}, sw[4] = {sb.x, sb.y, sb.z, sb.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t xs = (xw[j >> 1] >> (16 * (j & 1))) & 0xFFFFu, ss = (sw[j >> 1] >> (16 * (j & 1))) & 0xFFFFu;
                v[8 * c + j] = __fmul_rn(eb::bf16_bits_to_float(xs), __half2float(__ushort_as_half((unsigned short)ss)));
            }
        }
#pragma unroll
        for (int h = 1; h < 128; h <<= 1) {
#pragma unroll
            for (int p = 0; p < 64; ++p) {
                const int i = (p / h) * 2 * h + (p % h);
                const float a = v[i], b = v[i + h];
                v[i] = __fadd_rn(a, b);
                v[i + h] = __fsub_rn(a, b);
            }
        }
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            uint32_t packed[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) packed[i] = bf16_pair(__fmul_rn(v[8 * c + 2 * i], kInvSqrt128), __fmul_rn(v[8 * c + 2 * i + 1], kInvSqrt128));
            *reinterpret_cast<uint4*>(mine + 16 * c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
    }
    __syncthreads();
    uint4* to = reinterpret_cast<uint4*>(out + ((size_t)seg * rows * k) + (size_t)first * 128);
#pragma unroll
    for (uint32_t i = 0; i < 16u; ++i) {
        const uint32_t chunk = i * kRotateRowsThreads + t;
        if (chunk < count * 16u) to[chunk] = *reinterpret_cast<const uint4*>(stage + (chunk >> 4) * kPitch + (chunk & 15u) * 16u);
    }
}

// partials f32 [splits][rows][n] -> out bf16 [rows][n]. A warp per (row, 128 columns).
//   grid ceil(rows * (n / 128) / 8), block 256.
__global__ void __launch_bounds__(256) finish_kernel(const float* __restrict__ partials, int splits, const uint16_t* __restrict__ svh,
        uint16_t* __restrict__ out, int rows, int n) {
    const int lane = threadIdx.x & 31, blocks = n >> 7;
    const long long task = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    eb::pdl_launch_dependents();
    eb::pdl_wait();
    if (task >= (long long)rows * blocks) return;
    const size_t at = (size_t)(task / blocks) * n + (size_t)(task % blocks) * 128;
    add_and_finish128(partials + at, (size_t)rows * n, splits, svh + (size_t)(task % blocks) * 128, out + at, lane);
}

// rotated bf16: the product of segment g starts at element rows * start_g with row stride width_g (start_g, width_g from the
// exclusive segment ends) -> out bf16 [rows][n] = bf16(svh * H128(rotated)). A warp per (row, 128 columns).
//   grid ceil(rows * (n / 128) / 8), block 256.
__global__ void __launch_bounds__(256) finish_bf16_kernel(const uint16_t* __restrict__ rotated, const int* __restrict__ ends, int s,
        const uint16_t* __restrict__ svh, uint16_t* __restrict__ out, int rows, int n) {
    const int lane = threadIdx.x & 31, blocks = n >> 7;
    const long long task = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    eb::pdl_launch_dependents();
    eb::pdl_wait();
    if (task >= (long long)rows * blocks) return;
    const int row = (int)(task / blocks), block_start = (int)(task % blocks) * 128;
    int g = 0;
    while (g + 1 < s && block_start >= ends[g]) ++g;
    const int start = g == 0 ? 0 : ends[g - 1], width = ends[g] - start;
    const uint2 bits = *reinterpret_cast<const uint2*>(rotated + (size_t)rows * start + (size_t)row * width + (block_start - start) + 4 * lane);
    float v[4] = {eb::bf16_bits_to_float(bits.x & 0xFFFFu), eb::bf16_bits_to_float(bits.x >> 16), eb::bf16_bits_to_float(bits.y & 0xFFFFu),
            eb::bf16_bits_to_float(bits.y >> 16)};
    finish128(v, svh + block_start, out + (size_t)row * n + block_start, lane);
}

// ---- the linear ------------------------------------------------------------------------------------------------------

// The 16 k of a tile enter the FP16 MMA in this order of its k index c: k = 2 (c % 4) + (c % 8) / 4 + 8 (c / 8). It is
// where the u8 MMA's output lands: lane (g, q) gets the sums of columns 2q and 2q + 1 of its 8, and column 4 b + q' is the
// product lane (g, q') put into its A register pair b. With it, lane q of a quad reads its B fragment of a tile as one
// 8-byte load when the activations of 16 k are stored as k = 0 2 8 10 | 4 6 12 14 | 1 3 9 11 | 5 7 13 15.

// How one lane reads its eight states out of a tile's ring of W 16-bit words.
template <int W>
struct Lane {
    static constexpr int kRingWords = W / 2;                // 32-bit words of a tile
    static constexpr int kStep = W / 16;                    // whole bits from one position's window to the next
    static constexpr bool kHalfStep = (W % 16) == 8;        // and one more bit before every odd position
    __host__ __device__ static constexpr int start(int j) { return kStep * j + (kHalfStep ? (j + 1) / 2 : 0); }   // window j after window 0
    // The first window starts up to 31 bits into the first word; the last one ends start(7) + 16 bits after that.
    static constexpr int kWords = (31 + start(7) + 16 + 31) / 32;

    uint32_t at[kWords];   // byte offsets of the lane's ring words inside a tile
    uint32_t shift;        // bits in front of its first window in the first of them
    uint32_t select[2];    // B operand of the byte-sum MMA: ones where this lane's column takes its k group

    __device__ __forceinline__ void init(int lane) {
        int bit = window_end(lane * 8, W) - 16;             // tail-biting: the first windows start before the ring's bit 0
        if (bit < 0) bit += kRingWords * 32;
        shift = (uint32_t)bit & 31u;
#pragma unroll
        for (int i = 0; i < kWords; ++i) at[i] = 4u * (uint32_t)(((bit >> 5) + i) % kRingWords);
        const int g = lane >> 2, q = lane & 3;
        select[0] = g == q ? 0x01010101u : 0u;
        select[1] = g == q + 4 ? 0x01010101u : 0u;
    }

    // State of window J, the words already shifted so that window 0 starts at the top bit of u[0].
    template <int J>
    __device__ __forceinline__ static uint32_t state(const uint32_t (&u)[kWords + 1]) {
        constexpr int o = start(J), i = o >> 5, b = o & 31;
        if constexpr (b == 0) {
            return u[i] >> 16;
        } else if constexpr (b == 16) {
            return u[i] & 0xFFFFu;
        } else if constexpr (b < 16) {
            return (u[i] >> (16 - b)) & 0xFFFFu;
        } else {
            return __funnelshift_l(u[i + 1], u[i], b) >> 16;
        }
    }

    // The lane's FP16 A fragment of the tile OFFSET bytes after shared address `tile`.
    template <int OFFSET>
    __device__ __forceinline__ void fragment(uint32_t tile, uint32_t (&a)[4]) const {
        uint32_t u[kWords + 1];
#pragma unroll
        for (int i = 0; i < kWords; ++i) u[i] = eb::lds_u32<OFFSET>(tile + at[i]);
        u[kWords] = 0u;
#pragma unroll
        for (int i = 0; i < kWords; ++i) u[i] = __funnelshift_l(u[i + 1], u[i], shift);
        constexpr uint32_t kHash = 0x83DCD12Du;
        const uint32_t p0 = state<0>(u) * kHash, p1 = state<1>(u) * kHash, p2 = state<2>(u) * kHash, p3 = state<3>(u) * kHash;
        const uint32_t p4 = state<4>(u) * kHash, p5 = state<5>(u) * kHash, p6 = state<6>(u) * kHash, p7 = state<7>(u) * kHash;
        // Positions 0..3 are tile row g (k = 2q, 2q+1, 2q+8, 2q+9), 4..7 the same k of row g + 8.
        uint32_t low[4], high[4];
        eb::mma_u8_16832_from(low, p0, p4, p1, p5, select[0], select[1], 0x6400u);    // k = 2q' and 2q'+1 of every lane q'
        eb::mma_u8_16832_from(high, p2, p6, p3, p7, select[0], select[1], 0x6400u);   // k = 2q'+8 and 2q'+9
        const __half2 slope = __half2half2(__ushort_as_half((unsigned short)0x1EEE)), offset = __half2half2(__ushort_as_half((unsigned short)0xC931));
        const uint32_t packed[4] = {__byte_perm(low[0], low[1], 0x5410), __byte_perm(low[2], low[3], 0x5410),
                __byte_perm(high[0], high[1], 0x5410), __byte_perm(high[2], high[3], 0x5410)};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 value = __hfma2(*reinterpret_cast<const __half2*>(&packed[i]), slope, offset);
            a[i] = *reinterpret_cast<const uint32_t*>(&value);
        }
    }
};

// Payload -> BF16 rotated weight [n][k] (row-major weights of a BF16 linear). A warp takes kBatch tiles side by side: a lane
// reads its ring words of all of them from global memory first, then takes its eight states of each as the linear does and
// stores 16 contiguous bytes of one weight row (the quad's pairs regrouped through shared memory).
//   grid ceil((k / 16) * (n / 16) / (8 kBatch)), block 256.
template <int W>
__global__ void __launch_bounds__(256) decode_bf16_kernel(const uint16_t* __restrict__ words, uint16_t* __restrict__ out, int k, int n) {
    using L = Lane<W>;
    const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    constexpr int kExchangePitch = 40;   // words of an exchange row: 32 lanes + 8, so that a quarter warp's 16-byte loads tile the banks
    __shared__ __align__(16) uint32_t exchange_rows[8][4 * kExchangePitch];
    uint32_t* exchange = exchange_rows[threadIdx.x >> 5];
    const uint32_t first = (blockIdx.x * 8u + (threadIdx.x >> 5)) * (uint32_t)kBatch, tiles = (uint32_t)(k >> 4) * (uint32_t)(n >> 4);   // < 2^31
    if (first >= tiles) return;
    L me;
    me.init(lane);
    uint32_t u[kBatch][L::kWords + 1];
#pragma unroll
    for (int t = 0; t < kBatch; ++t) {
        const uint32_t tile = first + t < tiles ? first + t : tiles - 1u;
        const uint8_t* ring = reinterpret_cast<const uint8_t*>(words + (size_t)tile * W);
#pragma unroll
        for (int i = 0; i < L::kWords; ++i) u[t][i] = __ldg(reinterpret_cast<const uint32_t*>(ring + me.at[i]));
        u[t][L::kWords] = 0u;
    }
#pragma unroll
    for (int t = 0; t < kBatch; ++t) {
        const uint32_t tile = first + t;
        if (tile >= tiles) break;
        const int ti = (int)(tile / (uint32_t)(n >> 4)), tj = (int)(tile % (uint32_t)(n >> 4));
#pragma unroll
        for (int i = 0; i < L::kWords; ++i) u[t][i] = __funnelshift_l(u[t][i + 1], u[t][i], me.shift);
        const uint32_t state[8] = {L::template state<0>(u[t]), L::template state<1>(u[t]), L::template state<2>(u[t]), L::template state<3>(u[t]),
                L::template state<4>(u[t]), L::template state<5>(u[t]), L::template state<6>(u[t]), L::template state<7>(u[t])};
        uint32_t pair[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t values = value_pair(state[2 * j], state[2 * j + 1]);   // two FP16 codebook values
            const float2 wide = __half22float2(*reinterpret_cast<const __half2*>(&values));
            pair[j] = bf16_pair(wide.x, wide.y);
        }
        // positions 0..3 are tile row g at k = 2q, 2q+1, 2q+8, 2q+9; positions 4..7 the same k of row g + 8. The four lanes of a
        // quad trade their pairs through shared memory so that each stores 16 contiguous bytes: lane q gets pair q of all
        // four, i.e. k 0..7 (q = 0) or 8..15 (q = 1) of row g, or the same of row g + 8 (q = 2, 3).
        __syncwarp();   // the tile before has been read out of the exchange rows
#pragma unroll
        for (int j = 0; j < 4; ++j) exchange[j * kExchangePitch + lane] = pair[j];
        __syncwarp();
        const uint4 mine = *reinterpret_cast<const uint4*>(exchange + q * kExchangePitch + 4 * g);
        *reinterpret_cast<uint4*>(out + (size_t)(tj * 16 + g + 8 * (q >> 1)) * k + ti * 16 + 8 * (q & 1)) = mine;
    }
}

// What a launch of the linear works on. `activations` (the scratch's fragment-order FP16 [s][rows][k], written by a
// rotate launch) or, when it is null, x and suh. `flags` null: the partials of a split K are left for a finish launch.
struct Job {
    const uint16_t* activations;
    const uint16_t* x;
    const uint16_t* suh;
    const int* ends;              // exclusive column ends of the s segments
    const uint16_t* svh;
    float* partials;              // [splits][rows][n], used when splits > 1
    uint16_t* out;                // bf16 [rows][n]
    unsigned long long* flags;    // [n / 128][splits]
    unsigned long long tag;       // this call's flag value
    int rows, k, n, splits, s;
};

__device__ __forceinline__ void decoders_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * kDecodeWarps) : "memory"); }

// P = groups of 8 activation rows held at once (rows beyond 8 P take another pass over the payload).
//   grid (n / 128, splits), block kThreads, dynamic shared kStages * kStageTiles * 16 W + act_bytes(P) bytes.
template <int W, int P>
__global__ void __launch_bounds__(kThreads, P == 1 ? kResident : 2) linear_kernel(const __grid_constant__ CUtensorMap payload_map,
        const __grid_constant__ Job job, uint32_t* __restrict__ error) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t kTileBytes = 2u * W, kTileRowBytes = 8u * kTileBytes, kStageBytes = kStageTiles * kTileRowBytes;
    __shared__ __align__(8) uint64_t full[kStages], empty[kStages];
    __shared__ int last_arrival;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q = lane & 3;
    const int rows = job.rows, k = job.k, n = job.n, splits = job.splits;
    const int column0 = blockIdx.x * 128, split = blockIdx.y;
    const int tiles = k >> 4;
    const int first = (int)(((long long)split * tiles) / splits), last = (int)(((long long)(split + 1) * tiles) / splits);
    const int stages = (last - first + kStageTiles - 1) / kStageTiles;
    const int passes = (rows + 8 * P - 1) / (8 * P);
    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            eb::mbar_init(&full[i], 1);
            eb::mbar_init(&empty[i], kDecodeWarps);
        }
        eb::mbar_fence_init();
    }
    __syncthreads();
    eb::pdl_launch_dependents();

    if (warp == kDecodeWarps) {
        // Stage number i over all passes holds tile rows [first + (i % stages) * 16, ..) in ring buffer i % kStages. The box is
        // always whole (rows past the tensor arrive as zeros, rows past the split are not decoded), so is the byte count.
        if (lane == 0) {
            const int total = passes * stages;
            for (int i = 0; i < total; ++i) {
                const int slot = i % kStages;
                // a stage lasts microseconds: the poll sleeps between tries and leaves the issue slots to the decoding warps
                if (i >= kStages && !eb::mbar_wait_at<256>(eb::smem_u32(&empty[slot]), (uint32_t)(i / kStages - 1) & 1u)) {
                    atomicOr(error, kWaitFailed);
                    break;
                }
                eb::mbar_arrive_expect_tx(&full[slot], kStageBytes);
                eb::tma_load_2d(smem + slot * kStageBytes, &payload_map, (column0 >> 4) * (W / 4), first + (i % stages) * kStageTiles, &full[slot]);
            }
        }
        return;
    }

    uint8_t* act = smem + kStages * kStageBytes;   // [live rows][stride]: tile row t of the chunk at 32 (t - 8 block0)
    int seg = 0;   // the segment of this column block: the first whose end lies beyond it
    while (seg + 1 < job.s && column0 >= job.ends[seg]) ++seg;
    Lane<W> decoder;
    decoder.init(lane);
    const uint32_t ring = eb::smem_u32(smem) + warp * kTileBytes;
    bool alive = true;   // false once a stage failed to arrive: no further waits, the error bit is set

    eb::pdl_wait();   // x, or the activations of a rotate launch, come from the launch before

    for (int pass = 0; pass < passes; ++pass) {
        const int row_base = pass * 8 * P, live = min(8 * P, rows - row_base);
        const int chunk = chunk_tiles(P, live);
        const uint32_t stride = (uint32_t)chunk * 32u + 32u;
        // Lane (g, q) reads activation row 8 p + g; a row that is not there reads the last one (its sums are never stored).
        uint32_t act_lane[P];
#pragma unroll
        for (int p = 0; p < P; ++p) act_lane[p] = eb::smem_u32(act) + (uint32_t)min(8 * p + g, live - 1) * stride + q * 8u;
        float acc[P][4];
#pragma unroll
        for (int p = 0; p < P; ++p) acc[p][0] = acc[p][1] = acc[p][2] = acc[p][3] = 0.0f;
        for (int c0 = first; c0 < last;) {
            const int c1 = min(last, (c0 / chunk + 1) * chunk);
            const int block0 = c0 >> 3, blocks = ((c1 + 7) >> 3) - block0;
            decoders_sync();   // nobody reads the chunk before any more
            for (int task = warp; task < live * blocks; task += kDecodeWarps) {
                const int r = task % live, block = block0 + task / live;
                uint8_t* to = act + r * stride + (block - block0) * 256 + (lane >> 2) * 32;   // this lane's group of 16 k
                const int a = lane & 3;
                if (job.activations == nullptr) {
                    float v[4];
                    rotate128(job.x + (size_t)(row_base + r) * k + (size_t)block * 128, job.suh + (size_t)seg * k + (size_t)block * 128, lane, v);
                    // the lane's k are 4a .. 4a+3 of its group: (4a, 4a+2) are neighbours in the order above, (4a+1, 4a+3) 8 further
                    uint32_t* pair = reinterpret_cast<uint32_t*>(to) + 2 * (a & 1) + (a >> 1);
                    pair[0] = half_pair(v[0], v[2]);
                    pair[4] = half_pair(v[1], v[3]);
                } else {
                    // the scratch holds k = 2a, 2a+1, 2a+8, 2a+9 of the group at 4a
                    const uint2 from = *reinterpret_cast<const uint2*>(
                            job.activations + ((size_t)seg * rows + row_base + r) * k + (size_t)block * 128 + 4 * lane);
                    uint16_t* half = reinterpret_cast<uint16_t*>(to) + 4 * (a >> 1) + (a & 1);
                    half[0] = (uint16_t)(from.x & 0xFFFFu);
                    half[8] = (uint16_t)(from.x >> 16);
                    half[2] = (uint16_t)(from.y & 0xFFFFu);
                    half[10] = (uint16_t)(from.y >> 16);
                }
            }
            decoders_sync();
            for (int t0 = c0; t0 < c1;) {   // the pieces of the chunk that lie in one stage
                const int stage = (t0 - first) / kStageTiles, stage_end = first + (stage + 1) * kStageTiles;
                const int t1 = min(c1, stage_end), number = pass * stages + stage, slot = number % kStages;
                if (alive && !eb::mbar_wait(&full[slot], (uint32_t)(number / kStages) & 1u)) {
                    alive = false;
                    if (lane == 0) atomicOr(error, kWaitFailed);
                }
                uint32_t tile = ring + slot * kStageBytes + (t0 - first - stage * kStageTiles) * kTileRowBytes;
                const uint32_t b_offset = (uint32_t)(t0 - 8 * block0) * 32u;
                uint32_t b_at[P];
#pragma unroll
                for (int p = 0; p < P; ++p) b_at[p] = act_lane[p] + b_offset;
                auto one = [&](auto index) {   // tile `index` after the current one
                    constexpr int kAhead = decltype(index)::value;
                    uint32_t a[4];
                    decoder.template fragment<kAhead * kTileRowBytes>(tile, a);
#pragma unroll
                    for (int p = 0; p < P; ++p) {
                        const float2 b = eb::lds_f2<kAhead * 32>(b_at[p]);
                        eb::mma_f16_16816(acc[p], a[0], a[1], a[2], a[3], __float_as_uint(b.x), __float_as_uint(b.y));
                    }
                };
                int t = t0;
                for (; t + kUnroll <= t1; t += kUnroll) {
                    eb::static_for<kUnroll>(one);
                    tile += kUnroll * kTileRowBytes;
#pragma unroll
                    for (int p = 0; p < P; ++p) b_at[p] += 32u * kUnroll;
                }
                for (; t < t1; ++t) {
                    one(std::integral_constant<int, 0>{});
                    tile += kTileRowBytes;
#pragma unroll
                    for (int p = 0; p < P; ++p) b_at[p] += 32u;
                }
                if (t1 == stage_end || t1 == last) {   // done with the stage's buffer
                    __syncwarp();
                    if (lane == 0) eb::mbar_arrive(&empty[slot]);
                }
                t0 = t1;
            }
            c0 = c1;
        }
        // acc[p][i]: column g (i < 2) or g + 8 of this warp's 16, row row_base + 8 p + 2 q + (i & 1).
        if (splits > 1) {
#pragma unroll
            for (int p = 0; p < P; ++p)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = row_base + 8 * p + 2 * q + (i & 1);
                    if (row < rows) job.partials[((size_t)split * rows + row) * n + column0 + warp * 16 + g + 8 * (i >> 1)] = acc[p][i];
                }
        } else {
            // One split: rotate and scale here. The sums of 8 rows x 128 columns meet in the activation buffer, which nobody
            // reads any more; warp w finishes row w of the 8.
            float(*tile_out)[128] = reinterpret_cast<float(*)[128]>(act);
#pragma unroll
            for (int p = 0; p < P; ++p) {
                decoders_sync();
#pragma unroll
                for (int i = 0; i < 4; ++i) tile_out[2 * q + (i & 1)][warp * 16 + g + 8 * (i >> 1)] = acc[p][i];
                decoders_sync();
                const int row = row_base + 8 * p + warp;
                if (row < rows) {
                    float v[4] = {tile_out[warp][lane * 4], tile_out[warp][lane * 4 + 1], tile_out[warp][lane * 4 + 2], tile_out[warp][lane * 4 + 3]};
                    finish128(v, job.svh + column0, job.out + (size_t)row * n + column0, lane);
                }
            }
        }
    }

    if (splits > 1 && job.flags != nullptr) {
        decoders_sync();   // every thread's partials are stored; the fence of thread 0 below orders them before the flag
        if (warp == 0) {
            volatile unsigned long long* flags = job.flags + (size_t)blockIdx.x * splits;
            if (lane == 0) {
                __threadfence();
                flags[split] = job.tag;
            }
            __syncwarp();
            __threadfence();   // sequentially consistent: of two CTAs that finish together at least one sees the other's flag
            bool all = true;   // the lanes read the block's flags side by side
            for (int i = lane; i < splits; i += 32) all = all && flags[i] == job.tag;
            all = __all_sync(0xFFFFFFFFu, all);
            __threadfence();
            if (lane == 0) last_arrival = all ? 1 : 0;
        }
        decoders_sync();
        if (last_arrival != 0) {
            for (int row = warp; row < rows; row += kDecodeWarps)
                add_and_finish128(job.partials + (size_t)row * n + column0, (size_t)rows * n, splits, job.svh + column0,
                        job.out + (size_t)row * n + column0, lane);
            // The block is done: its flags stop carrying the tag, so that the same launch replayed from a CUDA graph (same
            // tag) starts from flags that are not set. A CTA that reads them only now sees them unset and leaves the block
            // to this one.
            if (warp == 0)
                for (int i = lane; i < splits; i += 32) job.flags[(size_t)blockIdx.x * splits + i] = ~job.tag;
        }
    }
}

}  // namespace trellis
