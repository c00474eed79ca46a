// BF16 x BF16 -> BF16 linear on tcgen05 (kind::f16, FP32 accumulators in tensor memory) for the trellis prefill route:
// out[r][j] = bf16(sum_k a[r][k] * b[j][k]) for a [rows][k] and b [n][k], both BF16 and K-major. It stands where the
// reference's trellis prefill calls its row-exact BF16 linear on the decoded weights
// (core/.../artifact/format/TrellisFormat.java:560-604, RowExactBf16.java:52-84): every output is one FP32 sum over K in
// K order whatever the row count, so a row's bits do not depend on the rows beside it.
//
// The engine is the NVFP4 prefill kernel's (nvfp4_native.cuh) without scales: a persistent CTA per SM walks 128 x 256
// output tiles; warp 0 requests the stages by TMA (64 K of the 128 activation rows and of the 256 weight rows: 48 KB,
// 128-byte swizzle, four stages), one thread of warp 1 issues four K = 16 MMAs per stage and commits the stage back, eight
// epilogue warps drain a 128 x 256 accumulator into registers, hand it back and round and store, while the MMAs of the next
// tile fill the other accumulator (two of 256 columns: all of tensor memory). Every wait is bounded.
#pragma once

#include <atomic>

#include "nvfp4_native.cuh"
#include "trellis_codebook.cuh"

namespace bf16n {

using nvfp4n::kThreads;
using nvfp4n::kTileM;
using nvfp4n::kTileN;
using nvfp4n::kTmemColumns;

constexpr uint32_t kStepK = 64;                                   // BF16 values of K per stage: 128 bytes a row
constexpr uint32_t kATile = kTileM * 128u, kBTile = kTileN * 128u;
constexpr uint32_t kStageBytes = kATile + kBTile;
constexpr uint32_t kStages = 4;
constexpr uint32_t kSharedBytes = kStages * kStageBytes + 128u + 1024u;   // + barriers + slack to align to 1024
constexpr uint32_t kWaitFailed = 16u;                             // error bit: a bounded wait of this kernel gave up

// kind::f16 instruction descriptor: FP32 accumulator, BF16 x BF16, both operands K-major, M 128, N 256.
constexpr uint32_t kInstruction = (1u << 4) | (1u << 7) | (1u << 10) | ((kTileN >> 3) << 17) | ((kTileM >> 4) << 24);

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(kInstruction), "r"(accumulate)
            : "memory");
}

// A thread's 128 consecutive sums of one row (one 128-column block of the trellis output) -> the block's final values:
// the sums rounded to BF16 as the plan's BF16 linear stores them, the block's Hadamard transform in FP32 by the format's
// butterflies (stage h pairs i with i + h; every a + b and a - b as trellis::hadamard128_warp forms them, so the bits are
// those of the plan's epilogue kernel), times 1/sqrt(128), times svh, BF16. No other thread is needed.
__device__ __forceinline__ void store_rotated(uint32_t (&r)[4][32], uint16_t* __restrict__ out, const uint16_t* __restrict__ svh) {
    float* v = reinterpret_cast<float*>(&r[0][0]);
#pragma unroll
    for (int i = 0; i < 128; ++i) v[i] = eb::bf16_bits_to_float(eb::float_to_bf16_bits(v[i]));
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
        const uint4 scales = *reinterpret_cast<const uint4*>(svh + 8 * c);
        const uint32_t sw[4] = {scales.x, scales.y, scales.z, scales.w};
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t bits[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float scale = __half2float(__ushort_as_half((unsigned short)(sw[i] >> (16 * e))));
                bits[e] = eb::float_to_bf16_bits(__fmul_rn(scale, __fmul_rn(v[8 * c + 2 * i + e], trellis::kInvSqrt128)));
            }
            packed[i] = bits[0] | bits[1] << 16;
        }
        *reinterpret_cast<uint4*>(out + 8 * c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

//   grid: min(tiles, SMs), block nvfp4n::kThreads, dynamic shared kSharedBytes. map_a: [rows][k] BF16, box 64 x 128;
//   map_b: [n][k] BF16, box 64 x 128 (a B tile is two boxes). n a multiple of 128. out: row stride `stride` elements.
//   svh null: out[r][j] = bf16(sum); else out[r][j] = the trellis output of the 128-column block j belongs to (svh [n]).
//   a_period: K of map_a (k is a multiple of it). pair_tiles: see below (svh must be null then).
__global__ void __launch_bounds__(kThreads, 1) bf16_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
        uint16_t* __restrict__ out, const uint16_t* __restrict__ svh, uint32_t stride, uint32_t rows, uint32_t n, uint32_t k,
        uint32_t a_period, uint32_t pair_tiles, uint32_t* __restrict__ error) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;    // two accumulators of 256 columns: the MMAs of a tile run while the tile before is drained
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    // pair_tiles != 0: the gate/up region. `n` is the output width (half of the weight rows); an output tile of 128 columns
    // takes the 128 gate rows at its own place and the 128 up rows pair_tiles * 128 further down as the halves of its B tile.
    const bool paired = pair_tiles != 0u;
    const nvfp4n::TileWalk walk(rows, n, paired ? 128u : kTileN);
    const uint32_t k_steps = k / kStepK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            eb::mbar_init(&full[s], 1);
            eb::mbar_init(&empty[s], 1);
        }
        for (uint32_t b = 0; b < 2u; ++b) {
            eb::mbar_init(&acc_full[b], 1);
            eb::mbar_init(&acc_empty[b], 8);
        }
        eb::mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(eb::smem_u32(tmem_holder)), "r"(kTmemColumns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    nvfp4n::tcgen05_fence_before();
    __syncthreads();
    nvfp4n::tcgen05_fence_after();
    const uint32_t tmem = *tmem_holder;
    eb::pdl_launch_dependents();
    eb::pdl_wait();   // both operands come from the launches before this one

    if (warp == 0) {
        if (lane == 0) {
            uint32_t step = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < walk.total && ok; tile += gridDim.x) {
                uint32_t tm, tn;
                walk.at(tile, &tm, &tn);
                for (uint32_t ks = 0; ks < k_steps; ++ks, ++step) {
                    const uint32_t s = step % kStages, round = step / kStages;
                    if (round > 0 && !eb::mbar_wait(&empty[s], (round - 1u) & 1u)) {
                        atomicOr(error, kWaitFailed);
                        ok = false;
                        break;
                    }
                    uint8_t* stage = smem + s * kStageBytes;
                    eb::mbar_arrive_expect_tx(&full[s], kStageBytes);
                    // rows past the end of a matrix read as zeros (and the transaction still counts the whole box)
                    // the activations' K index wraps at a_period (the weight's K holds several terms of the same activations)
                    eb::tma_load_2d(stage, &map_a, (int)((ks * kStepK) % a_period), (int)(tm * kTileM), &full[s]);
                    const uint32_t low = paired ? tn : 2u * tn, high = paired ? pair_tiles + tn : 2u * tn + 1u;
                    eb::tma_load_2d(stage + kATile, &map_b, (int)(ks * kStepK), (int)(low * 128u), &full[s]);
                    eb::tma_load_2d(stage + kATile + kBTile / 2u, &map_b, (int)(ks * kStepK), (int)(high * 128u), &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t step = 0, local = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < walk.total && ok; tile += gridDim.x, ++local) {
                const uint32_t buffer = local & 1u, use = local >> 1;
                if (use > 0 && !eb::mbar_wait(&acc_empty[buffer], (use - 1u) & 1u)) {
                    atomicOr(error, kWaitFailed);
                    break;
                }
                nvfp4n::tcgen05_fence_after();
                const uint32_t accumulator = tmem + buffer * kTileN;
                for (uint32_t ks = 0; ks < k_steps; ++ks, ++step) {
                    const uint32_t s = step % kStages, round = step / kStages;
                    if (!eb::mbar_wait(&full[s], round & 1u)) {
                        atomicOr(error, kWaitFailed);
                        ok = false;
                        break;
                    }
                    nvfp4n::tcgen05_fence_after();
                    const uint8_t* stage = smem + s * kStageBytes;
                    const uint64_t a = nvfp4n::tile_descriptor(stage), b = nvfp4n::tile_descriptor(stage + kATile);
#pragma unroll
                    for (uint32_t j = 0; j < 4u; ++j) mma_bf16(accumulator, a + 2u * j, b + 2u * j, (uint32_t)((ks | j) != 0u));   // 32 bytes of K further
                    nvfp4n::mma_commit(&empty[s]);
                }
                if (ok) nvfp4n::mma_commit(&acc_full[buffer]);
            }
        }
    } else {
        // warp w reads the 32 accumulator rows of lane quarter w % 4; warps 2..5 take columns 0..127, warps 6..9 128..255
        const uint32_t quarter = warp & 3u, half = (warp - 2u) >> 2;
        uint32_t local = 0;
        for (uint32_t tile = blockIdx.x; tile < walk.total; tile += gridDim.x, ++local) {
            uint32_t tm, tn;
            walk.at(tile, &tm, &tn);
            const uint32_t buffer = local & 1u;
            if (!eb::mbar_wait(&acc_full[buffer], (local >> 1) & 1u)) {
                if (lane == 0) atomicOr(error, kWaitFailed);
                break;
            }
            nvfp4n::tcgen05_fence_after();
            uint32_t r[4][32];
            // plain: 128 consecutive columns; paired: 64 gate columns (r[0], r[1]) and the 64 up columns that match them (r[2], r[3])
            const uint32_t from = tmem + ((quarter * 32u) << 16) + buffer * kTileN + (paired ? half * 64u : half * 128u);
            const uint32_t other = paired ? from + 128u : from + 64u;
            nvfp4n::tmem_load_32(r[0], from);
            nvfp4n::tmem_load_32(r[1], from + 32u);
            nvfp4n::tmem_load_32(r[2], other);
            nvfp4n::tmem_load_32(r[3], other + 32u);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            nvfp4n::tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) eb::mbar_arrive(&acc_empty[buffer]);
            const uint32_t row = tm * kTileM + quarter * 32u + lane, col = paired ? tn * 128u + half * 64u : tn * kTileN + half * 128u;
            if (svh == nullptr) {
                nvfp4n::store_block(r, out, row, rows, n, col, 1.0f, paired);   // row stride n
            } else if (row < rows && col < n) {
                store_rotated(r, out + (uint64_t)row * stride + col, svh + col);
            }
        }
    }
    nvfp4n::tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns) : "memory");
    }
}

// ---- the same GEMM on CTA pairs -----------------------------------------------------------------------------------------
// Two CTAs of a cluster share an output tile of 256 rows x 256 columns: each holds its own 128 activation rows and HALF of
// the weight tile (128 weight rows); one thread of the even CTA issues tcgen05.mma.cta_group::2 (M 256, N 256, K 16), which
// reads both CTAs' shared memory and accumulates each CTA's 128 rows in its own tensor memory. A stage is 32 KB per CTA
// instead of 48 KB for the same FLOP: a third fewer operand bytes from L2 per FLOP and six stages in flight instead of four.
// No multicast loads: each CTA requests its own tiles, and both CTAs' loads are counted on the even CTA's stage barrier
// (the pair form of the TMA load may signal a barrier of the peer), so no thread relays arrivals between the CTAs. Used for calls of kPairRows rows and more.
constexpr uint32_t kPairStages = 6;
constexpr uint32_t kPairStageBytes = kATile + 128u * 128u;
constexpr uint32_t kPairShared = kPairStages * kPairStageBytes + 256u + 1024u;
constexpr uint32_t kPairInstruction = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((256u >> 4) << 24);
constexpr uint32_t kPairRows = 512;

// A tiled TMA load of a CTA of a pair whose completion is counted on a barrier of either CTA of the pair (`bar`: a
// shared::cluster address). No multicast: the box lands in the executing CTA's shared memory only.
__device__ __forceinline__ void pair_tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                         eb::smem_u32(dst)),
            "l"(map), "r"(c0), "r"(c1), "r"(bar)
            : "memory");
}

__device__ __forceinline__ void pair_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(kPairInstruction), "r"(accumulate)
            : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1) bf16_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a,
        const __grid_constant__ CUtensorMap map_b, uint16_t* __restrict__ out, const uint16_t* __restrict__ svh, uint32_t stride, uint32_t rows,
        uint32_t n, uint32_t k, uint32_t a_period, uint32_t pair_tiles, uint32_t* __restrict__ error) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
    uint64_t* empty = full + kPairStages;
    uint64_t* acc_full = empty + kPairStages;    // two accumulators of 256 columns: a tile's MMAs run while the tile before is drained
    uint64_t* acc_empty = acc_full + 2;          // even CTA: both CTAs' epilogue warps have drained the accumulator
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = eb::cluster_rank(), pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    // pair_tiles != 0: the gate/up region; the even CTA's half of the weight tile is the gate rows, the odd CTA's the up rows.
    const bool paired = pair_tiles != 0u;
    const uint32_t tiles_m = (rows + 255u) / 256u, tiles_n = paired ? pair_tiles : (n + 255u) / 256u, items = tiles_m * tiles_n;
    const uint32_t k_steps = k / kStepK;
    // Panels of kPanel tile columns; inside a panel the row index runs fastest across the panel's columns.
    auto place = [&](uint32_t item, uint32_t* tm, uint32_t* tn) {
        const uint32_t per_panel = tiles_m * nvfp4n::kPanel, panel = item / per_panel, rest = item - panel * per_panel;
        const uint32_t width = min(nvfp4n::kPanel, tiles_n - panel * nvfp4n::kPanel);
        *tm = rest / width;
        *tn = panel * nvfp4n::kPanel + rest % width;
    };

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kPairStages; ++s) {
            eb::mbar_init(&full[s], 1);
            eb::mbar_init(&empty[s], 1);
        }
        for (uint32_t b = 0; b < 2u; ++b) {
            eb::mbar_init(&acc_full[b], 1);
            eb::mbar_init(&acc_empty[b], 16);
        }
        eb::mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(eb::smem_u32(tmem_holder)), "r"(kTmemColumns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    nvfp4n::tcgen05_fence_before();
    __syncthreads();
    eb::cluster_sync();   // both CTAs' barriers exist before anything arrives on them from the other CTA
    nvfp4n::tcgen05_fence_after();
    const uint32_t tmem = *tmem_holder;
    eb::pdl_launch_dependents();
    eb::pdl_wait();   // both operands come from the launches before this one

    if (warp == 0) {
        if (lane == 0) {
            uint32_t step = 0;
            bool ok = true;
            for (uint32_t item = pair; item < items && ok; item += pairs) {
                uint32_t tm, tn;
                place(item, &tm, &tn);
                const uint32_t row_tile = 2u * tm + rank;                      // this CTA's 128 rows
                const uint32_t weight_tile = paired ? (rank == 0u ? tn : pair_tiles + tn) : 2u * tn + rank;   // its 128 weight rows
                for (uint32_t ks = 0; ks < k_steps; ++ks, ++step) {
                    const uint32_t s = step % kPairStages, round = step / kPairStages;
                    if (round > 0 && !eb::mbar_wait(&empty[s], (round - 1u) & 1u)) {
                        atomicOr(error, kWaitFailed);
                        ok = false;
                        break;
                    }
                    uint8_t* stage = smem + s * kPairStageBytes;
                    // both CTAs' boxes are counted on the even CTA's barrier, where the thread that issues the MMAs waits
                    if (rank == 0u) eb::mbar_arrive_expect_tx(&full[s], 2u * kPairStageBytes);
                    const uint32_t bar = eb::map_to_rank(eb::smem_u32(&full[s]), 0u);
                    pair_tma_load_2d(stage, &map_a, (int)((ks * kStepK) % a_period), (int)(row_tile * kTileM), bar);
                    pair_tma_load_2d(stage + kATile, &map_b, (int)(ks * kStepK), (int)(weight_tile * 128u), bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0u) {   // the odd CTA issues nothing: its tiles are read by the even CTA's MMAs
            uint32_t step = 0, local = 0;
            bool ok = true;
            for (uint32_t item = pair; item < items && ok; item += pairs, ++local) {
                const uint32_t buffer = local & 1u, use = local >> 1;
                if (use > 0 && !eb::mbar_wait(&acc_empty[buffer], (use - 1u) & 1u)) {
                    atomicOr(error, kWaitFailed);
                    break;
                }
                nvfp4n::tcgen05_fence_after();
                const uint32_t accumulator = tmem + buffer * kTileN;
                for (uint32_t ks = 0; ks < k_steps; ++ks, ++step) {
                    const uint32_t s = step % kPairStages, round = step / kPairStages;
                    if (!eb::mbar_wait(&full[s], round & 1u)) {
                        atomicOr(error, kWaitFailed);
                        ok = false;
                        break;
                    }
                    nvfp4n::tcgen05_fence_after();
                    const uint8_t* stage = smem + s * kPairStageBytes;
                    const uint64_t a = nvfp4n::tile_descriptor(stage), b = nvfp4n::tile_descriptor(stage + kATile);
#pragma unroll
                    for (uint32_t j = 0; j < 4u; ++j) pair_mma_bf16(accumulator, a + 2u * j, b + 2u * j, (uint32_t)((ks | j) != 0u));
                    nvfp4n::pair_commit(&empty[s]);
                }
                if (ok) nvfp4n::pair_commit(&acc_full[buffer]);
            }
        }
    } else {
        // Epilogue, in both CTAs, each over its own 128 rows: as in bf16_gemm_kernel.
        const uint32_t quarter = warp & 3u, half = (warp - 2u) >> 2;
        uint32_t local = 0;
        for (uint32_t item = pair; item < items; item += pairs, ++local) {
            uint32_t tm, tn;
            place(item, &tm, &tn);
            const uint32_t buffer = local & 1u;
            if (!eb::mbar_wait(&acc_full[buffer], (local >> 1) & 1u)) {
                if (lane == 0) atomicOr(error, kWaitFailed);
                break;
            }
            nvfp4n::tcgen05_fence_after();
            uint32_t r[4][32];
            const uint32_t from = tmem + ((quarter * 32u) << 16) + buffer * kTileN + (paired ? half * 64u : half * 128u);
            const uint32_t other = paired ? from + 128u : from + 64u;
            nvfp4n::tmem_load_32(r[0], from);
            nvfp4n::tmem_load_32(r[1], from + 32u);
            nvfp4n::tmem_load_32(r[2], other);
            nvfp4n::tmem_load_32(r[3], other + 32u);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            nvfp4n::tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) nvfp4n::arrive_at_rank(&acc_empty[buffer], 0u);
            const uint32_t row = (2u * tm + rank) * kTileM + quarter * 32u + lane, col = paired ? tn * 128u + half * 64u : tn * kTileN + half * 128u;
            if (svh == nullptr) {
                nvfp4n::store_block(r, out, row, rows, n, col, 1.0f, paired);   // row stride n
            } else if (row < rows && col < n) {
                store_rotated(r, out + (uint64_t)row * stride + col, svh + col);
            }
        }
    }
    nvfp4n::tcgen05_fence_before();
    __syncthreads();
    eb::cluster_sync();   // neither CTA leaves while the other may still read its shared memory or arrive on its barriers
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns) : "memory");
    }
}

// Q3G64_F16S tensor -> two BF16 planes side by side along K, [n][2 k]: columns [0, k) hold hi = bf16(code * scale), columns
// [k, 2 k) lo = code * scale - hi. code * f32(scale) has at most 14 significant bits, hi keeps 8 and the rest fits BF16:
// hi + lo is the weight exactly, and both products with a BF16 activation are exact in FP32. Eight threads per group of 64:
// a thread takes 8 codes (24 bits) and writes 16 bytes of each plane, so a warp's stores are whole 128-byte lines.
//   grid ceil(n * (k / 64) * 8 / 256), block 256. k a multiple of 128.
__global__ void __launch_bounds__(256) q3_terms_kernel(const uint8_t* __restrict__ w, uint64_t scale_offset, uint16_t* __restrict__ out,
        uint32_t n, uint32_t k) {
    const uint32_t groups = k / 64u;
    const uint64_t index = (uint64_t)blockIdx.x * 256u + threadIdx.x, group_index = index >> 3;
    if (group_index >= (uint64_t)n * groups) return;
    const uint32_t sub = (uint32_t)index & 7u, row = (uint32_t)(group_index / groups), group = (uint32_t)(group_index % groups);
    const uint32_t* words = reinterpret_cast<const uint32_t*>(w + group_index * 24u);
    const uint32_t byte = 3u * sub, word = byte >> 2;              // the thread's 24 bits start at this byte of the group's 24
    const uint32_t bits = __funnelshift_r(__ldg(words + word), __ldg(words + min(word + 1u, 5u)), 8u * (byte & 3u));
    const float scale = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const uint16_t*>(w + scale_offset) + group_index)));
    uint32_t high[4], low[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float value[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            // the 3-bit two's complement code as a float without an integer conversion: code + 4 = field ^ 4 sits in the
            // mantissa of 2^23, and 2^23 + 4 is subtracted (exact)
            const uint32_t field = (bits >> (3 * (2 * i + e))) & 7u;
            value[e] = __fmul_rn(__fsub_rn(__uint_as_float(0x4B000000u | (field ^ 4u)), 8388612.0f), scale);
        }
        // round to nearest even in one conversion per pair; the values are finite
        const __nv_bfloat162 top = __floats2bfloat162_rn(value[0], value[1]);
        const float2 back = __bfloat1622float2(top);
        const __nv_bfloat162 rest = __floats2bfloat162_rn(__fsub_rn(value[0], back.x), __fsub_rn(value[1], back.y));
        high[i] = *reinterpret_cast<const uint32_t*>(&top);
        low[i] = *reinterpret_cast<const uint32_t*>(&rest);
    }
    uint16_t* hi = out + (uint64_t)row * 2u * k + (uint64_t)group * 64u + 8u * sub;
    *reinterpret_cast<uint4*>(hi) = make_uint4(high[0], high[1], high[2], high[3]);
    *reinterpret_cast<uint4*>(hi + k) = make_uint4(low[0], low[1], low[2], low[3]);
}

inline cudaError_t initialize() {
    const cudaError_t e = cudaFuncSetAttribute(bf16_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSharedBytes);
    return e != cudaSuccess ? e : cudaFuncSetAttribute(bf16_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPairShared);
}

// Whether calls of kPairRows rows and more run on CTA pairs (process-wide; same bits either way).
inline std::atomic<bool> g_pairs{true};

// a [rows][k], b [n][k] -> out [rows][n] at row stride `stride`, all BF16 in device memory, 16-byte aligned; k % 64 == 0,
// n % 128 == 0. svh (FP16 [n], may be null): finish the trellis output in the epilogue instead of storing the sums.
// a_k: K of a (k = terms x a_k: b's K holds `terms` planes that all multiply the same activations). paired: b is a gate/up
// object of n rows (gate first) and out is [rows][n / 2] SwiGLU values.
inline cudaError_t linear(const void* a, const void* b, void* out, const void* svh, uint32_t stride, uint32_t rows, uint32_t k, uint32_t n, int sms,
        cudaStream_t stream, bool pdl, uint32_t* error, uint32_t a_k = 0, bool paired = false) {
    if (a_k == 0) a_k = k;
    const eb::EncodeTiled encode = eb::encoder();
    if (encode == nullptr) return cudaErrorNotSupported;
    CUtensorMap map_a, map_b;
    const cuuint32_t ones[2] = {1u, 1u}, box[2] = {kStepK, 128u};
    const cuuint64_t a_dims[2] = {a_k, rows}, b_dims[2] = {k, n}, strides[1] = {(cuuint64_t)k * 2u}, a_strides[1] = {(cuuint64_t)a_k * 2u};
    CUresult r = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a), a_dims, a_strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS)
        r = encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(b), b_dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    const uint32_t pair_tiles = paired ? n / 256u : 0u, width = paired ? n / 2u : n;
    if (rows >= kPairRows && g_pairs.load()) {
        const uint32_t items = ((rows + 255u) / 256u) * (paired ? pair_tiles : (n + 255u) / 256u);
        const uint32_t ctas = 2u * std::max(1u, std::min((uint32_t)sms / 2u, items));
        return nvfp4n::launch_on(stream, pdl, bf16_gemm_pair_kernel, dim3(ctas), dim3(kThreads), kPairShared, map_a, map_b, static_cast<uint16_t*>(out),
                static_cast<const uint16_t*>(svh), stride, rows, width, k, a_k, pair_tiles, error);
    }
    const uint32_t tiles = ((rows + kTileM - 1u) / kTileM) * (paired ? pair_tiles : (n + kTileN - 1u) / kTileN);
    return nvfp4n::launch_on(stream, pdl, bf16_gemm_kernel, dim3(tiles < (uint32_t)sms ? tiles : (uint32_t)sms), dim3(kThreads), kSharedBytes, map_a, map_b,
            static_cast<uint16_t*>(out), static_cast<const uint16_t*>(svh), stride, rows, width, k, a_k, pair_tiles, error);
}

}  // namespace bf16n
