// Trellis (trellis-tile16-v1) linear for decode-sized row counts on sm_100a, as three stream-ordered launches behind
// the reference's table launcher euhedral_cuda_linear_launch (native/src/host/linear_kernels.c:7-24):
//   prepass  (table entry 0, native/src/trellis/prepass.cuh:17-81):  act[g][r] = fp16(H128(bf16 x[r] * fp16 suh[g]))
//   mma      (table entry 1, native/src/trellis/mma.cuh:434-455):    z = act . Q per K split (FP16 x FP16 -> FP32)
//   epilogue (table entry 4, native/src/trellis/epilogue.cuh:13-41): y = bf16(svh * H128(sum of the splits in order))
// plus decode_bf16 (table entry 5, native/src/trellis/decode.cuh:15-29). Arguments, scratch layout (activations then
// FP32 partials [split][row][n]) and the split ranges [i T / S, (i + 1) T / S) of the T = k / 16 tile rows are the
// reference's, because its Java host plans them (core/.../artifact/format/TrellisFormat.java:484-567).
//
// The mma kernel: a CTA owns 128 output columns (8 tiles of 16) and one K split; warp i owns tile column i. The CTA
// streams its tile rows through a ring of stages in shared memory with bulk asynchronous copies (the 8 tiles of a tile
// row are contiguous in the payload), all requested before griddepcontrol.wait. A lane decodes its eight consecutive
// positions of a tile - exactly its m16n8k16 A fragment - from the ring words in registers and issues one MMA per
// group of 8 activation rows, k16 tiles in increasing order, so a row's bits depend on its own data and the K range only.
#pragma once

#include "common.cuh"
#include "trellis_codebook.cuh"

namespace trellis {

// x bf16 [rows][k], suh f16 [s][k] -> out [s][rows][k]: layout 0 = FP16 in MMA fragment order (in each group of 16,
// elements 2q, 2q+1, 2q+8, 2q+9 contiguous at 4q), layout 1 = BF16 in column order. One warp per 128-column block.
//   grid (ceil(k / 512), rows, s), block 128.
__global__ void __launch_bounds__(128) prepass_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ suh,
        uint16_t* __restrict__ out, int rows, int k, int s, int layout) {
    const int lane = threadIdx.x & 31, r = blockIdx.y, seg = blockIdx.z;
    const int block = blockIdx.x * 4 + (threadIdx.x >> 5);
    eb::pdl_launch_dependents();
    eb::pdl_wait();
    if (block * 128 >= k) return;
    const size_t column = (size_t)block * 128 + lane * 4;
    const uint2 xb = *reinterpret_cast<const uint2*>(x + (size_t)r * k + column);
    const uint2 sb = *reinterpret_cast<const uint2*>(suh + (size_t)seg * k + column);
    float v[4];
    v[0] = __fmul_rn(eb::bf16_bits_to_float(xb.x & 0xFFFFu), __half2float(__ushort_as_half((unsigned short)(sb.x & 0xFFFFu))));
    v[1] = __fmul_rn(eb::bf16_bits_to_float(xb.x >> 16), __half2float(__ushort_as_half((unsigned short)(sb.x >> 16))));
    v[2] = __fmul_rn(eb::bf16_bits_to_float(xb.y & 0xFFFFu), __half2float(__ushort_as_half((unsigned short)(sb.y & 0xFFFFu))));
    v[3] = __fmul_rn(eb::bf16_bits_to_float(xb.y >> 16), __half2float(__ushort_as_half((unsigned short)(sb.y >> 16))));
    hadamard128_warp(v, lane);
    uint16_t* row = out + ((size_t)seg * rows + r) * k;
    if (layout == 0) {
#pragma unroll
        for (int pair = 0; pair < 2; ++pair) {
            const int e = (lane * 4 + pair * 2) & 15;
            const size_t at = (column & ~(size_t)15) + 4 * ((e & 7) >> 1) + 2 * (e >> 3);
            const uint32_t bits = (uint32_t)__half_as_ushort(__float2half_rn(v[2 * pair]))
                    | (uint32_t)__half_as_ushort(__float2half_rn(v[2 * pair + 1])) << 16;
            *reinterpret_cast<uint32_t*>(row + at) = bits;
        }
    } else {
        const uint32_t lo = (uint32_t)eb::float_to_bf16_bits(v[0]) | (uint32_t)eb::float_to_bf16_bits(v[1]) << 16;
        const uint32_t hi = (uint32_t)eb::float_to_bf16_bits(v[2]) | (uint32_t)eb::float_to_bf16_bits(v[3]) << 16;
        *reinterpret_cast<uint2*>(row + column) = make_uint2(lo, hi);
    }
}

// partials f32 [splits][rows][n] summed in split order, H128 per 128 columns, * f32(fp16 svh), BF16.
//   grid (ceil(n / 512), rows), block 128.
__global__ void __launch_bounds__(128) epilogue_kernel(const float* __restrict__ partials, int splits,
        const uint16_t* __restrict__ svh, uint16_t* __restrict__ out, int rows, int n) {
    const int lane = threadIdx.x & 31, r = blockIdx.y;
    const int block = blockIdx.x * 4 + (threadIdx.x >> 5);
    eb::pdl_launch_dependents();
    eb::pdl_wait();
    if (block * 128 >= n) return;
    const size_t column = (size_t)block * 128 + lane * 4;
    float4 sum = *reinterpret_cast<const float4*>(partials + (size_t)r * n + column);
    for (int i = 1; i < splits; ++i) {
        const float4 part = *reinterpret_cast<const float4*>(partials + ((size_t)i * rows + r) * n + column);
        sum.x = __fadd_rn(sum.x, part.x);
        sum.y = __fadd_rn(sum.y, part.y);
        sum.z = __fadd_rn(sum.z, part.z);
        sum.w = __fadd_rn(sum.w, part.w);
    }
    float v[4] = {sum.x, sum.y, sum.z, sum.w};
    hadamard128_warp(v, lane);
    const uint2 sb = *reinterpret_cast<const uint2*>(svh + column);
    const uint32_t sw[2] = {sb.x, sb.y};
    uint32_t bits[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float scale = __half2float(__ushort_as_half((unsigned short)(sw[j >> 1] >> (16 * (j & 1)))));
        bits[j] = eb::float_to_bf16_bits(__fmul_rn(scale, v[j]));
    }
    *reinterpret_cast<uint2*>(out + (size_t)r * n + column) = make_uint2(bits[0] | bits[1] << 16, bits[2] | bits[3] << 16);
}

// Payload -> BF16 rotated weight [n][k] (row-major weights of a BF16 linear). One CTA per tile, one thread per position.
//   grid (k / 16) * (n / 16), block 256.
__global__ void __launch_bounds__(256) decode_bf16_kernel(const uint16_t* __restrict__ words, uint16_t* __restrict__ out,
        int k, int n, int w) {
    const int tiles_n = n >> 4;
    const int ti = blockIdx.x / tiles_n, tj = blockIdx.x % tiles_n;
    const int p = threadIdx.x;
    const float value = __half2float(__ushort_as_half(value_bits(window_of_tile(words + (size_t)blockIdx.x * w, w, p))));
    const int lane = p >> 3, j = p & 7;
    const int kk = 2 * (lane & 3) + 8 * ((j >> 1) & 1) + (j & 1), nn = (lane >> 2) + 8 * (j >> 2);
    out[(size_t)(tj * 16 + nn) * k + ti * 16 + kk] = eb::float_to_bf16_bits(value);
}

// ---- the tensor-core GEMM -------------------------------------------------------------------------------------------

// The stored tile widths (16-bit words per tile): X(w) for each.
#define EB_TRELLIS_WIDTHS(X) X(16) X(24) X(32) X(40) X(48) X(56) X(64) X(72) X(80) X(88) X(96) X(104) X(112) X(120) X(128)

constexpr int kStageTiles = 16;   // tile rows (k16 steps) per ring stage
constexpr int kStages = 3;

// Per-width constants of a lane's eight windows: window j starts offset(j) bits after window 0, whatever the lane
// (8 * lane is 0 or 8 modulo 16 and the half-step layout adds its extra bit on odd positions only).
template <int W>
struct Width {
    static constexpr int kWords32 = W / 2, kBits = W / 16;
    static constexpr bool kHalf = (W & 15) == 8;
    __host__ __device__ static constexpr int offset(int j) { return kBits * j + (kHalf ? (j + 1) / 2 : 0); }
    // Window 0 starts up to 31 bits into the first word; window 7 ends offset(7) + 16 bits later.
    static constexpr int kWords = (31 + offset(7) + 16 + 31) / 32;
};

// Window j of words normalised so that window 0 starts at the top bit of u[0].
template <int W, int J>
__device__ __forceinline__ uint32_t window(const uint32_t* u) {
    constexpr int o = Width<W>::offset(J), i = o >> 5, b = o & 31;
    if constexpr (b <= 16) {
        return (u[i] >> (16 - b)) & 0xFFFFu;
    } else {
        return __funnelshift_l(u[i + 1], u[i], b) >> 16;
    }
}

// act f16 [s][rows][k] in fragment order; words [k/16][n/16][W]; ends the exclusive column ends of the s segments;
// svh f16 [n]. splits == 1: out (BF16 [rows][n]) is written here with the output Hadamard applied; otherwise the raw
// FP32 sums of split blockIdx.y go to partials[split][rows][n]. P = groups of 8 activation rows held at once.
//   grid (n / 128, splits), block 256, dynamic shared kStages * kStageTiles * 8 * W * 2 bytes (+ barriers).
template <int W, int P>
__global__ void __launch_bounds__(256) mma_kernel(const __grid_constant__ CUtensorMap payload_map, const uint16_t* __restrict__ act,
        const uint16_t* __restrict__ words, const int* __restrict__ ends, const uint16_t* __restrict__ svh, float* __restrict__ partials,
        uint16_t* __restrict__ out, int rows, int k, int n, int splits, int s, uint32_t* __restrict__ error) {
    extern __shared__ __align__(128) uint8_t smem[];
    using Wd = Width<W>;
    constexpr uint32_t kTileRowBytes = 8u * W * 2u;                 // 8 tiles of one tile row
    constexpr uint32_t kStageBytes = kStageTiles * kTileRowBytes;
    __shared__ float tile_out[8][128];
    __shared__ __align__(8) uint64_t bars[kStages];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q = lane & 3;
    const int column0 = blockIdx.x * 128;
    const int tiles = k >> 4;
    const int first = (int)(((long long)blockIdx.y * tiles) / splits), last = (int)(((long long)(blockIdx.y + 1) * tiles) / splits);
    const int count = last - first;
    const int stages_total = (count + kStageTiles - 1) / kStageTiles;
    (void)words;   // read through payload_map
    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) eb::mbar_init(&bars[i], 1);
        eb::mbar_fence_init();
    }
    __syncthreads();
    // Streaming stage number gst (over all passes over the activation rows) holds the tile rows
    // [first + (gst % stages_total) * kStageTiles, ...) in ring buffer gst % kStages: one bulk copy per tile row.
    const int passes = (rows + 8 * P - 1) / (8 * P);
    const int stream_total = passes * stages_total;
    // One tiled TMA copy per stage: a box of kStageTiles tile rows x this block's 8 tiles (16 W bytes) of the payload seen
    // as [k / 16 rows][n / 16 * 2 W bytes]. A last stage that reaches past the split brings rows that are never decoded
    // (zeros past the tensor); the box is always whole, so is the byte count the barrier expects.
    auto request = [&](int gst) {
        const int base = first + (gst % stages_total) * kStageTiles;
        if (lane == 0) {
            uint64_t* bar = &bars[gst % kStages];
            eb::mbar_arrive_expect_tx(bar, kStageBytes);
            eb::tma_load_2d(smem + (gst % kStages) * kStageBytes, &payload_map, (column0 >> 4) * (W / 4), base, bar);
        }
    };
    if (warp == 0)
        for (int gst = 0; gst < min(kStages, stream_total); ++gst) request(gst);

    // Segment of this column block: the first whose end is beyond it.
    int seg = 0;
    while (seg + 1 < s && column0 >= ends[seg]) ++seg;

    // This lane's ring words of a tile and the bit where its first window starts in the first of them.
    int at = window_end(lane * 8, W) - 16;
    if (at < 0) at += Wd::kWords32 * 32;
    const int shift = at & 31;
    int word[Wd::kWords];
#pragma unroll
    for (int i = 0; i < Wd::kWords; ++i) word[i] = ((at >> 5) + i) % Wd::kWords32;

    eb::pdl_launch_dependents();
    eb::pdl_wait();   // the activations come from the prepass launch

    for (int row_base = 0; row_base < rows; row_base += 8 * P) {
        float acc[P][4];
#pragma unroll
        for (int p = 0; p < P; ++p) acc[p][0] = acc[p][1] = acc[p][2] = acc[p][3] = 0.0f;
        // Lane's activations of k16 tile ti for row (row_base + 8 p + g): 8 bytes at a_lane + 16 * ti (+ 8 p rows).
        const uint16_t* a_lane = act + ((size_t)seg * rows + row_base + g) * k + 4 * q;
        const int pass = row_base / (8 * P);
        for (int st = 0; st < stages_total; ++st) {
            const int gst = pass * stages_total + st;   // stage number over all passes
            if (!eb::mbar_wait(&bars[gst % kStages], (uint32_t)(gst / kStages) & 1u) && lane == 0) atomicOr(error, 4u);
            const uint8_t* stage = smem + (gst % kStages) * kStageBytes + warp * (W * 2u);
            const int base = first + st * kStageTiles;
            const int rows_here = min(kStageTiles, last - base);
            for (int t = 0; t < rows_here; ++t) {
                const uint32_t* ring = reinterpret_cast<const uint32_t*>(stage + t * kTileRowBytes);
                uint32_t u[Wd::kWords + 1];
#pragma unroll
                for (int i = 0; i < Wd::kWords; ++i) u[i] = ring[word[i]];
                u[Wd::kWords] = 0u;
#pragma unroll
                for (int i = 0; i < Wd::kWords; ++i) u[i] = __funnelshift_l(u[i + 1], u[i], shift);
                const uint32_t a0 = value_pair(window<W, 0>(u), window<W, 1>(u));
                const uint32_t a2 = value_pair(window<W, 2>(u), window<W, 3>(u));
                const uint32_t a1 = value_pair(window<W, 4>(u), window<W, 5>(u));
                const uint32_t a3 = value_pair(window<W, 6>(u), window<W, 7>(u));
                const int ti = base + t;
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    uint2 xv = make_uint2(0u, 0u);
                    if (row_base + 8 * p + g < rows) xv = *reinterpret_cast<const uint2*>(a_lane + (size_t)(8 * p) * k + (size_t)ti * 16);
                    eb::mma_f16_16816(acc[p], a0, a1, a2, a3, xv.x, xv.y);
                }
            }
            __syncthreads();   // every warp is done with this stage's buffer
            // Refill the buffer with the stage kStages ahead (wrapping into the next pass over the rows).
            if (warp == 0 && gst + kStages < stream_total) request(gst + kStages);
        }
        // acc[p][i]: column g (i < 2) or g + 8 of this warp's 16, row row_base + 8 p + 2 q + (i & 1).
        if (splits > 1) {
#pragma unroll
            for (int p = 0; p < P; ++p)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = row_base + 8 * p + 2 * q + (i & 1);
                    if (row < rows)
                        partials[((size_t)blockIdx.y * rows + row) * n + column0 + warp * 16 + g + 8 * (i >> 1)] = acc[p][i];
                }
        } else {
#pragma unroll
            for (int p = 0; p < P; ++p) {
                __syncthreads();
#pragma unroll
                for (int i = 0; i < 4; ++i) tile_out[2 * q + (i & 1)][warp * 16 + g + 8 * (i >> 1)] = acc[p][i];
                __syncthreads();
                // Warp `warp` finishes row `warp` of the 8: Hadamard in registers, svh, BF16.
                const int row = row_base + 8 * p + warp;
                float v[4] = {tile_out[warp][lane * 4], tile_out[warp][lane * 4 + 1], tile_out[warp][lane * 4 + 2], tile_out[warp][lane * 4 + 3]};
                hadamard128_warp(v, lane);
                if (row < rows) {
                    const uint2 sb = *reinterpret_cast<const uint2*>(svh + column0 + lane * 4);
                    const uint32_t sw[2] = {sb.x, sb.y};
                    uint32_t bits[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        bits[j] = eb::float_to_bf16_bits(__fmul_rn(__half2float(__ushort_as_half((unsigned short)(sw[j >> 1] >> (16 * (j & 1))))), v[j]));
                    *reinterpret_cast<uint2*>(out + (size_t)row * n + column0 + lane * 4) = make_uint2(bits[0] | bits[1] << 16, bits[2] | bits[3] << 16);
                }
            }
        }
    }
}

}  // namespace trellis
