// NVFP4 prefill GEMM on sm_100a: both operands NVFP4, tcgen05 block-scaled MMA (kind::mxf4nvf4, one UE4M3 scale per 16
// values) with the accumulator in tensor memory.
//
// Replaces the reference's native route behind euhedral_cuda_linear_nvfp4_native_bf16
// (native/src/host/nvfp4_linear.c:299-361): its activation quantizer native/src/nvfp4_native/native.cuh:105-168 and its
// 128x128 warp-MMA tile native/src/nvfp4_native/native.cuh:265-432. Same arithmetic contract: each BF16 activation row
// becomes two NVFP4 terms (the value and the quantized residual) under one FP32 scale per row; per output the K steps
// run in increasing order with one MMA per term into the same FP32 accumulator; the result is
// bf16(acc * row scale * tensor scale).
//
// Three launches per call, all on the selected stream, no allocation (everything lives in the caller's scratch):
//   1. quantize_rows: BF16 rows -> code planes [term][row][K/2], block scales already in the layout tcgen05 wants
//      (512-byte atoms of 128 rows x 4 scales, byte (r % 32) * 16 + (r / 32) * 4 + s), one FP32 scale per row. One warp
//      per row; a lane's unit is a K block of 64 values, whose four scales are one 4-byte store into the atom.
//   2. repack_weight_scales: the tensor's row-major E4M3 scale plane -> the same atom layout (the scales are 1/9 of
//      the weight bytes; the codes are consumed in place through a tensor map).
//   3. gemm: persistent CTAs, one per SM, 128 x 256 output tiles, K in steps of 256 through a 3-stage ring.
//      warp 0 (one lane) issues the TMA loads (codes as 128-byte-swizzled tiles, scale atoms as bulk copies),
//      warp 1 (one lane) copies the scale atoms to tensor memory (tcgen05.cp) and issues the MMAs
//      (M 128, N 256, K 64; two terms x four K blocks per stage) and commits to the ring's and the accumulator's
//      mbarriers, warps 2..9 drain the accumulator into registers (tcgen05.ld), hand it back at once, then scale, round
//      and store BF16 while the next tile's MMAs already run.
// Tiles are walked in panels of eight tile columns with the row index fastest, so that CTAs running together share
// weight tiles and re-read activation tiles from L2. Every CTA issues its own loads; there is no cluster.
#pragma once

#include <cuda.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <algorithm>

#include "common.cuh"

namespace nvfp4n {

constexpr uint32_t kTerms = 2;
constexpr uint32_t kTileM = 128, kTileN = 256, kStepK = 256, kBlockK = 64;
constexpr uint32_t kStages = 3;
constexpr uint32_t kATile = kTileM * 128u;                 // one term's codes of a stage: 128 rows x 128 bytes
constexpr uint32_t kBTile = kTileN * 128u;
constexpr uint32_t kAtom = 512u;                           // 128 rows x 4 scales
constexpr uint32_t kSfaStage = (kStepK / kBlockK) * kTerms * kAtom;
constexpr uint32_t kSfbStage = (kStepK / kBlockK) * (kTileN / 128u) * kAtom;
constexpr uint32_t kStageBytes = kTerms * kATile + kBTile + kSfaStage + kSfbStage;
constexpr uint32_t kBarrierBytes = 128u;
constexpr uint32_t kSharedBytes = kStages * kStageBytes + kBarrierBytes + 1024u;   // + slack to align to 1024
constexpr uint32_t kThreads = 320u;                         // TMA warp, MMA warp, eight epilogue warps
constexpr uint32_t kTmemColumns = 512u;
constexpr uint32_t kTmemSfa = 256u, kTmemSfb = 288u;       // column offsets behind the 256 accumulator columns
constexpr uint32_t kPanel = 8u;                            // tile columns per panel of the tile walk

__host__ __device__ inline uint64_t align256(uint64_t v) { return (v + 255ull) & ~255ull; }

// Caller scratch of one native linear.
// Calls of at most kSkinnyRows rows (one row tile) may cut K over up to kMaxSplits CTAs per output tile, so that a call
// with few output tiles still uses every SM; the FP32 partial tiles go to the end of the scratch.
constexpr uint32_t kSkinnyRows = 64, kMaxSplits = 8;

struct ActivationLayout {
    uint64_t sfa_offset, global_offset, sfb_offset, partial_offset, bytes;
    uint32_t row_tiles, k_blocks;
    __host__ __device__ ActivationLayout(uint32_t rows, uint32_t k, uint32_t out_features = 0) {
        const uint64_t kp = ((uint64_t)k + 127u) / 128u * 128u;
        row_tiles = (rows + kTileM - 1u) / kTileM;
        k_blocks = (uint32_t)(kp / kBlockK);
        sfa_offset = align256((uint64_t)kTerms * rows * (kp / 2u));
        global_offset = align256(sfa_offset + (uint64_t)row_tiles * k_blocks * kTerms * kAtom);
        sfb_offset = align256(global_offset + 4ull * rows);
        const uint64_t n128 = ((uint64_t)out_features + 255u) / 256u * 2u;
        partial_offset = align256(sfb_offset + n128 * k_blocks * kAtom);
        bytes = rows <= kSkinnyRows && out_features != 0u ? partial_offset + (uint64_t)kMaxSplits * rows * out_features * 4u : partial_offset;
    }
};

__host__ __device__ inline uint32_t atom_byte(uint32_t row_in_tile, uint32_t scale) {
    return (row_in_tile & 31u) * 16u + (row_in_tile >> 5) * 4u + scale;
}

// ---- 1. activation quantizer -----------------------------------------------------------------------------------------
// The arithmetic is the reference's, operation for operation (native/src/nvfp4_native/native.cuh:105-127, pinned bit for
// bit against that kernel compiled for this GPU): global = amax / (6 * 448) (1 for a zero row); per block of 16:
// scale = e4m3_satfinite(amax * (1/6) * (1/global)); codes = e2m1_rn(v * ((1/global) / scale)), saturating; the next term
// quantizes fma(-decoded, scale * global, v). All in FP32 with the hardware conversions.
// The work split is this kernel's own: one warp per row, eight rows per CTA, no shared memory and no CTA barrier. Four
// neighbouring lanes share a K block of 64 values, one 16-value block each; their four scale bytes meet by two shuffles
// and leave as ONE 4-byte store, which is exactly one row's entry of the 512-byte atom tcgen05 reads; their codes leave
// as 32 contiguous bytes per term.
constexpr uint32_t kQuantizeWarps = 8;

// One block of 16 values: its scale code, its 8 code bytes, and v replaced by the residual.
__device__ __forceinline__ uint32_t quantize_block(float (&v)[16], float global, float inverse_global, uint2* codes) {
    float block_max = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) block_max = fmaxf(block_max, fabsf(v[i]));
    const __nv_fp8_storage_t scale = __nv_cvt_float_to_fp8(__fmul_rn(__fmul_rn(block_max, 1.0f / 6.0f), inverse_global), __NV_SATFINITE, __NV_E4M3);
    const float decoded = __half2float(__half(__nv_cvt_fp8_to_halfraw(scale, __NV_E4M3)));
    const float inverse = decoded > 0.0f ? __fdiv_rn(inverse_global, decoded) : 0.0f;
    const float step = __fmul_rn(decoded, global);
    uint32_t packed[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const __nv_fp4x2_storage_t pair = __nv_cvt_float2_to_fp4x2(
                make_float2(__fmul_rn(v[2 * i], inverse), __fmul_rn(v[2 * i + 1], inverse)), __NV_E2M1, cudaRoundNearest);
        packed[i >> 2] |= (uint32_t)pair << (8 * (i & 3));
        const __half2_raw back = __nv_cvt_fp4x2_to_halfraw2(pair, __NV_E2M1);
        const float2 q = __half22float2(*reinterpret_cast<const __half2*>(&back));
        v[2 * i] = __fmaf_rn(-q.x, step, v[2 * i]);       // the residual in one rounding, as the reference's build contracts it
        v[2 * i + 1] = __fmaf_rn(-q.y, step, v[2 * i + 1]);
    }
    *codes = make_uint2(packed[0], packed[1]);
    return (uint32_t)scale;
}

__global__ void __launch_bounds__(32 * kQuantizeWarps, 5) quantize_rows(const __nv_bfloat16* __restrict__ input, uint8_t* __restrict__ scratch,
        uint32_t rows, uint32_t k) {
    const uint32_t lane = threadIdx.x & 31u, row = blockIdx.x * kQuantizeWarps + (threadIdx.x >> 5);
    const ActivationLayout layout(rows, k);
    eb::pdl_launch_dependents();
    eb::pdl_wait();
    if (row >= rows) return;
    const uint4* x = reinterpret_cast<const uint4*>(input + (uint64_t)row * k);   // 8 values per element
    const uint32_t vectors = k / 8u, blocks64 = k / kBlockK;
    float amax = 0.0f;
#pragma unroll 4   // four loads in flight per lane: the pass is bound by load latency
    for (uint32_t i = lane; i < vectors; i += 32u) {
        const uint4 w = x[i];
        const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
            amax = fmaxf(amax, fmaxf(fabsf(eb::bf16_bits_to_float(words[j] & 0xFFFFu)), fabsf(__uint_as_float(words[j] & 0xFFFF0000u))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float global = amax > 0.0f ? __fdiv_rn(amax, 6.0f * 448.0f) : 1.0f;
    const float inverse_global = __fdiv_rn(1.0f, global);
    uint8_t* sfa = scratch + layout.sfa_offset + (uint64_t)(row / kTileM) * layout.k_blocks * kTerms * kAtom + atom_byte(row % kTileM, 0);
    const uint64_t plane = (uint64_t)rows * (k / 2u);
    uint8_t* codes_row = scratch + (uint64_t)row * (k / 2u);
    // Four neighbouring lanes share a K block of 64 values, one 16-value block each; a warp covers eight K blocks per turn.
    const uint32_t sub = lane & 3u;
    for (uint32_t first = 0; first < blocks64; first += 8u) {   // the row was just read: these loads hit L1 / L2
        const uint32_t b = first + (lane >> 2);
        const bool live = b < blocks64;
        uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
        if (live) {
            lo = x[2u * (4u * b + sub)];
            hi = x[2u * (4u * b + sub) + 1u];
        }
        const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float v[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[2 * i] = eb::bf16_bits_to_float(words[i] & 0xFFFFu);
            v[2 * i + 1] = __uint_as_float(words[i] & 0xFFFF0000u);
        }
#pragma unroll
        for (uint32_t t = 0; t < kTerms; ++t) {
            uint2 codes;
            uint32_t scales = quantize_block(v, global, inverse_global, &codes) << (8u * sub);
            scales |= __shfl_xor_sync(0xffffffffu, scales, 1);   // the K block's four scale bytes, in every one of the four lanes
            scales |= __shfl_xor_sync(0xffffffffu, scales, 2);
            if (live) {
                *reinterpret_cast<uint2*>(codes_row + t * plane + 32u * b + 8u * sub) = codes;
                if (sub == 0u) *reinterpret_cast<uint32_t*>(sfa + ((uint64_t)b * kTerms + t) * kAtom) = scales;
            }
        }
    }
    if (lane == 0) reinterpret_cast<float*>(scratch + layout.global_offset)[row] = global;
}

// ---- 2. weight scale repack ---------------------------------------------------------------------------------------------
// scales[n][K/16] (row-major E4M3 bytes) -> atoms [n / 128][K / 64][512]. One thread per (row, K block): 4 bytes.
// table != nullptr (layout row-split-k128-sd4-v1): `scales` holds 4-bit indices, two per byte with the even block in the
// low nibble, into the tensor's 16 E4M3 codes at `table`; the atoms get the codes, so the GEMM is the same for both layouts.
__global__ void __launch_bounds__(256) repack_weight_scales(const uint8_t* __restrict__ scales, const uint8_t* __restrict__ table,
        uint8_t* __restrict__ atoms, uint32_t n, uint32_t k_blocks, uint32_t n_padded) {
    const uint64_t index = (uint64_t)blockIdx.x * 256u + threadIdx.x;
    eb::pdl_launch_dependents();
    eb::pdl_wait();   // the GEMM of the call before this one may still be reading these atoms
    const uint32_t row = (uint32_t)(index / k_blocks), j = (uint32_t)(index % k_blocks);
    if (row >= n_padded) return;
    uint32_t word = 0u;
    if (row < n && table == nullptr) {
        word = *reinterpret_cast<const uint32_t*>(scales + (uint64_t)row * k_blocks * 4u + 4u * j);
    } else if (row < n) {
        const uint32_t pairs = *reinterpret_cast<const uint16_t*>(scales + (uint64_t)row * k_blocks * 2u + 2u * j);   // four indices
#pragma unroll
        for (uint32_t i = 0; i < 4u; ++i) word |= (uint32_t)table[(pairs >> (4u * i)) & 15u] << (8u * i);
    }
    *reinterpret_cast<uint32_t*>(atoms + ((uint64_t)(row >> 7) * k_blocks + j) * kAtom + atom_byte(row & 127u, 0)) = word;
}

// ---- 3. the GEMM ----------------------------------------------------------------------------------------------------------

using eb::tma_load_2d;
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
                         eb::smem_u32(dst)),
            "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(eb::smem_u32(bar))
            : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows under the 128-byte swizzle: 8-row groups are
// 1024 bytes apart, descriptor version 1 (sm_100), layout type 2.
__device__ __forceinline__ uint64_t tile_descriptor(const void* smem_tile) {
    uint64_t d = 0;
    d |= (uint64_t)((eb::smem_u32(smem_tile) & 0x3FFFFu) >> 4);
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Descriptor of a 512-byte scale atom for tcgen05.cp: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t atom_descriptor(const void* smem_atom) {
    uint64_t d = 0;
    d |= (uint64_t)((eb::smem_u32(smem_atom) & 0x3FFFFu) >> 4);
    d |= (uint64_t)(128u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
// kind::mxf4nvf4 instruction descriptor: E2M1 x E2M1, UE4M3 scales, both operands K-major, M 128, N 256.
constexpr uint32_t kInstruction = (1u << 7) | (1u << 10) | ((kTileN >> 3) << 17) | (0u << 23) | ((kTileM >> 4) << 24);

__device__ __forceinline__ void tmem_copy_atom(uint32_t tmem_address, uint64_t descriptor) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_address), "l"(descriptor) : "memory");
}
__device__ __forceinline__ void mma_block_scaled(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t sfa_tmem, uint32_t sfb_tmem,
        uint32_t accumulate) {
    asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
            "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%4], [%5], p;\n}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(kInstruction), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
            : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(eb::smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive accumulator columns of the calling warp's 32 lanes (one row per thread) into registers.
__device__ __forceinline__ void tmem_load_32(uint32_t (&r)[32], uint32_t address) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
            "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
              "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
              "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
              "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(address));
}

// A thread's row of an epilogue block, scaled, rounded to BF16 and stored 16 bytes at a time from column col0.
// plain: r holds 4 x 32 consecutive columns. paired (the gate/up region): r[0], r[1] are 64 gate columns, r[2], r[3] the 64
// up columns that match them; out[row][col] = bf16(silu(gate) * up) with gate and up rounded to BF16 first (the reference's
// region, native/src/nvfp4_native/native.cuh:390-413: the same expression, expf and division).
__device__ __forceinline__ void store_block(const uint32_t (&r)[4][32], uint16_t* __restrict__ out, uint32_t row, uint32_t rows, uint32_t n,
        uint32_t col0, float scale, bool paired) {
    if (row >= rows) return;
#pragma unroll
    for (uint32_t cb = 0; cb < 4u; ++cb) {
        if (paired && cb >= 2u) break;
        const uint32_t col = col0 + cb * 32u;
        if (col >= n) continue;
        uint16_t* dst = out + (uint64_t)row * n + col;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            uint32_t packed[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float value[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = 8 * v + 2 * i + e;
                    const float first = __fmul_rn(__uint_as_float(r[cb][c]), scale);
                    if (paired) {
                        const float gate = eb::bf16_bits_to_float(eb::float_to_bf16_bits(first));
                        const float up = eb::bf16_bits_to_float(eb::float_to_bf16_bits(__fmul_rn(__uint_as_float(r[(cb + 2u) & 3u][c]), scale)));
                        value[e] = __fmul_rn(__fdiv_rn(gate, __fadd_rn(1.0f, expf(-gate))), up);
                    } else {
                        value[e] = first;
                    }
                }
                packed[i] = (uint32_t)eb::float_to_bf16_bits(value[0]) | (uint32_t)eb::float_to_bf16_bits(value[1]) << 16;
            }
            if (col + 8u * v < n) *reinterpret_cast<uint4*>(dst + 8 * v) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
    }
}

struct TileWalk {
    uint32_t tiles_m, tiles_n, total;
    __device__ TileWalk(uint32_t rows, uint32_t n, uint32_t tile_columns) : tiles_m((rows + kTileM - 1u) / kTileM), tiles_n((n + tile_columns - 1u) / tile_columns) {
        total = tiles_m * tiles_n;
    }
    // Panels of kPanel tile columns; inside a panel the row index runs fastest across the panel's columns.
    __device__ void at(uint32_t tile, uint32_t* tm, uint32_t* tn) const {
        const uint32_t per_panel = tiles_m * kPanel;
        const uint32_t panel = tile / per_panel, rest = tile - panel * per_panel;
        const uint32_t width = min(kPanel, tiles_n - panel * kPanel);
        *tm = rest / width;
        *tn = panel * kPanel + rest % width;
    }
};

__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
        const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, const float* __restrict__ row_globals,
        const float* __restrict__ tensor_global, uint16_t* __restrict__ out, float* __restrict__ partials, uint32_t splits, uint32_t rows,
        uint32_t n, uint32_t k, uint32_t pair_tiles, uint32_t* __restrict__ error) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;
    uint64_t* acc_empty = acc_full + 1;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 1);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    // pair_tiles != 0: the gate/up region. `n` is the output width (half of the weight rows); an output tile of 128 columns
    // takes the 128 gate rows at its own place and the 128 up rows pair_tiles * 128 further down as the halves of its B tile.
    const bool paired = pair_tiles != 0u;
    const TileWalk walk(rows, n, paired ? 128u : kTileN);
    const uint32_t k_steps = k / kStepK, k_blocks = k / kBlockK;
    // A work item is an output tile and one of `splits` ranges of its K steps (one range unless the call is skinny).
    const uint32_t items = walk.total * splits;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            eb::mbar_init(&full[s], 1);
            eb::mbar_init(&empty[s], 1);
        }
        eb::mbar_init(acc_full, 1);
        eb::mbar_init(acc_empty, 8);
        eb::mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(eb::smem_u32(tmem_holder)), "r"(kTmemColumns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = *tmem_holder;
    eb::pdl_launch_dependents();
    eb::pdl_wait();   // the scratch comes from the two launches before this one

    if (warp == 0) {
        if (lane == 0) {
            uint32_t step = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
                uint32_t tm, tn;
                walk.at(item / splits, &tm, &tn);
                const uint32_t split = item % splits, ks_end = (split + 1u) * k_steps / splits;
                for (uint32_t ks = split * k_steps / splits; ks < ks_end; ++ks, ++step) {
                    const uint32_t s = step % kStages, round = step / kStages;
                    if (round > 0 && !eb::mbar_wait(&empty[s], (round - 1u) & 1u)) {
                        atomicOr(error, 8u);
                        ok = false;
                        break;
                    }
                    uint8_t* stage = smem + s * kStageBytes;
                    eb::mbar_arrive_expect_tx(&full[s], kStageBytes);
                    tma_load_3d(stage, &map_a, (int)(ks * 128u), (int)(tm * kTileM), 0, &full[s]);
                    tma_load_3d(stage + kATile, &map_a, (int)(ks * 128u), (int)(tm * kTileM), 1, &full[s]);
                    // the B tile's two halves of 128 weight rows, as 128-row tiles of the weight matrix
                    const uint32_t low = paired ? tn : 2u * tn, high = paired ? pair_tiles + tn : 2u * tn + 1u;
                    tma_load_2d(stage + kTerms * kATile, &map_b, (int)(ks * 128u), (int)(low * 128u), &full[s]);
                    tma_load_2d(stage + kTerms * kATile + kBTile / 2u, &map_b, (int)(ks * 128u), (int)(high * 128u), &full[s]);
                    uint8_t* sf = stage + kTerms * kATile + kBTile;
                    eb::bulk_g2s(sf, sfa + ((uint64_t)tm * k_blocks + ks * 4u) * kTerms * kAtom, kSfaStage, &full[s]);
                    eb::bulk_g2s(sf + kSfaStage, sfb + ((uint64_t)low * k_blocks + ks * 4u) * kAtom, 4u * kAtom, &full[s]);
                    eb::bulk_g2s(sf + kSfaStage + 4u * kAtom, sfb + ((uint64_t)high * k_blocks + ks * 4u) * kAtom, 4u * kAtom, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t step = 0, local = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x, ++local) {
                if (local > 0 && !eb::mbar_wait(acc_empty, (local - 1u) & 1u)) {
                    atomicOr(error, 8u);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t split = item % splits, ks_begin = split * k_steps / splits, ks_end = (split + 1u) * k_steps / splits;
                for (uint32_t ks = ks_begin; ks < ks_end; ++ks, ++step) {
                    const uint32_t s = step % kStages, round = step / kStages;
                    if (!eb::mbar_wait(&full[s], round & 1u)) {
                        atomicOr(error, 8u);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint8_t* stage = smem + s * kStageBytes;
                    const uint8_t* sf = stage + kTerms * kATile + kBTile;
                    const uint64_t a0 = tile_descriptor(stage), a1 = tile_descriptor(stage + kATile), b = tile_descriptor(stage + kTerms * kATile);
                    auto cp_a = [&](uint32_t j, uint32_t t) { tmem_copy_atom(tmem + kTmemSfa + (j * 2u + t) * 4u, atom_descriptor(sf + (j * 2u + t) * kAtom)); };
                    auto cp_b = [&](uint32_t j, uint32_t h) { tmem_copy_atom(tmem + kTmemSfb + j * 8u + h * 4u, atom_descriptor(sf + kSfaStage + (h * 4u + j) * kAtom)); };
                    auto mma = [&](uint32_t j, uint32_t t) {
                        mma_block_scaled(tmem, (t ? a1 : a0) + 2u * j, b + 2u * j, tmem + kTmemSfa + (j * 2u + t) * 4u, tmem + kTmemSfb + j * 8u,
                                t ? 1u : (uint32_t)(((ks - ks_begin) | j) != 0u));
                    };
                    // K block by K block: its scale atoms, then its two MMAs (6 % faster than all sixteen copies of the stage first)
#pragma unroll
                    for (uint32_t j = 0; j < 4u; ++j) {
                        cp_a(j, 0);
                        cp_b(j, 0);
                        cp_b(j, 1);
                        mma(j, 0);
                        cp_a(j, 1);
                        mma(j, 1);
                    }
                    mma_commit(&empty[s]);
                }
                if (ok) mma_commit(acc_full);
            }
        }
    } else {
        // Epilogue: warp w may read the 32 accumulator rows of lane quarter w % 4 only; warps 2..5 take columns 0..127 of
        // their quarter, warps 6..9 columns 128..255. A warp first drains its 32 x 128 block into registers and hands the
        // accumulator back (the MMA warp starts the next tile while this one is scaled, rounded and stored).
        const uint32_t quarter = warp & 3u, half = (warp - 2u) >> 2;
        const float scale_w = *tensor_global;
        uint32_t local = 0;
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, ++local) {
            uint32_t tm, tn;
            walk.at(item / splits, &tm, &tn);
            if (!eb::mbar_wait(acc_full, local & 1u)) {
                if (lane == 0) atomicOr(error, 8u);
                break;
            }
            tcgen05_fence_after();
            uint32_t r[4][32];
            // plain: 128 consecutive columns; paired: 64 gate columns (r[0], r[1]) and the 64 up columns that match them (r[2], r[3])
            const uint32_t from = tmem + ((quarter * 32u) << 16) + (paired ? half * 64u : half * 128u);
            const uint32_t other = paired ? from + 128u : from + 64u;
            tmem_load_32(r[0], from);
            tmem_load_32(r[1], from + 32u);
            tmem_load_32(r[2], other);
            tmem_load_32(r[3], other + 32u);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) eb::mbar_arrive(acc_empty);
            const uint32_t row = tm * kTileM + quarter * 32u + lane;
            const float scale = row < rows ? __fmul_rn(row_globals[row], scale_w) : 0.0f;
            if (splits > 1u) {
                // the raw FP32 sums of this K range: partials[split][row][n]; finish_splits adds the ranges in order
#pragma unroll
                for (uint32_t cb = 0; cb < 4u; ++cb) {
                    const uint32_t col = tn * kTileN + half * 128u + cb * 32u;
                    if (row < rows && col < n) {
                        float4* dst = reinterpret_cast<float4*>(partials + ((uint64_t)(item % splits) * rows + row) * n + col);
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            if (col + 4u * v < n)
                                dst[v] = make_float4(__uint_as_float(r[cb][4 * v]), __uint_as_float(r[cb][4 * v + 1]), __uint_as_float(r[cb][4 * v + 2]),
                                        __uint_as_float(r[cb][4 * v + 3]));
                    }
                }
            } else {
                store_block(r, out, row, rows, n, paired ? tn * 128u + half * 64u : tn * kTileN + half * 128u, scale, paired);
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns) : "memory");
    }
}

// ---- the same GEMM on CTA pairs -----------------------------------------------------------------------------------------
// Two CTAs of a cluster share an output tile of 256 rows x 256 columns: each holds its own 128 activation rows (both
// terms) and HALF of the weight tile (128 weight rows), and one thread of the even CTA issues tcgen05.mma.cta_group::2
// (M 256, N 256, K 64), which reads both CTAs' shared memory and accumulates each CTA's 128 rows in its own tensor
// memory. A stage is 56 KB per CTA instead of 72 KB for the same FLOP, so four stages fit and the ring carries 22 % fewer
// bytes per MMA. Measured on B200 it is 6-9 % SLOWER than gemm_kernel (4.1 against 4.5 PFLOP/s issued on the gate shape,
// three stages or four alike), so it runs only when the caller selects it. Every CTA issues its own plain TMA loads into its own shared memory (no load names another CTA); the odd
// CTA's MMA warp only relays "my stage has landed" to a barrier of the even CTA; tcgen05.commit signals the ring's and the
// accumulator's barriers of both CTAs. Weight scale atoms (all 256 columns) are loaded by both.
constexpr uint32_t kPairStages = 4;
constexpr uint32_t kPairBTile = 128u * 128u;
constexpr uint32_t kPairStageBytes = kTerms * kATile + kPairBTile + kSfaStage + kSfbStage;
constexpr uint32_t kPairShared = kPairStages * kPairStageBytes + 256u + 1024u;
constexpr uint32_t kPairInstruction = (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | (0u << 23) | ((256u >> 4) << 24);

__device__ __forceinline__ void pair_copy_atom(uint32_t tmem_address, uint64_t descriptor) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_address), "l"(descriptor) : "memory");
}
__device__ __forceinline__ void pair_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
            "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%4], [%5], p;\n}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(kPairInstruction), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
            : "memory");
}
// Arrives (once the MMAs issued so far are done) on the barrier at this shared address in both CTAs of the pair.
__device__ __forceinline__ void pair_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(eb::smem_u32(bar)),
            "h"((uint16_t)3)
            : "memory");
}
__device__ __forceinline__ void arrive_at_rank(uint64_t* bar, uint32_t rank) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(eb::map_to_rank(eb::smem_u32(bar), rank)) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1) gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a,
        const __grid_constant__ CUtensorMap map_b, const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb,
        const float* __restrict__ row_globals, const float* __restrict__ tensor_global, uint16_t* __restrict__ out, uint32_t rows, uint32_t n,
        uint32_t k, uint32_t pair_tiles, uint32_t* __restrict__ error) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~(uintptr_t)1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
    uint64_t* empty = full + kPairStages;
    uint64_t* peer_full = empty + kPairStages;   // even CTA: the odd CTA's stage has landed
    uint64_t* acc_full = peer_full + kPairStages;
    uint64_t* acc_empty = acc_full + 1;          // even CTA: both CTAs' epilogue warps have drained the accumulator
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 1);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = eb::cluster_rank(), pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    // pair_tiles != 0: the gate/up region; the even CTA's half of the weight tile is the gate rows, the odd CTA's the up rows.
    const bool paired = pair_tiles != 0u;
    const uint32_t tiles_m = (rows + 255u) / 256u, tiles_n = paired ? pair_tiles : (n + 255u) / 256u, items = tiles_m * tiles_n;
    const uint32_t row_tiles = (rows + kTileM - 1u) / kTileM;
    const uint32_t k_steps = k / kStepK, k_blocks = k / kBlockK;
    // Panels of kPanel tile columns; inside a panel the row index runs fastest across the panel's columns.
    auto place = [&](uint32_t item, uint32_t* tm, uint32_t* tn) {
        const uint32_t per_panel = tiles_m * kPanel, panel = item / per_panel, rest = item - panel * per_panel;
        const uint32_t width = min(kPanel, tiles_n - panel * kPanel);
        *tm = rest / width;
        *tn = panel * kPanel + rest % width;
    };

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kPairStages; ++s) {
            eb::mbar_init(&full[s], 1);
            eb::mbar_init(&empty[s], 1);
            eb::mbar_init(&peer_full[s], 1);
        }
        eb::mbar_init(acc_full, 1);
        eb::mbar_init(acc_empty, 16);
        eb::mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(eb::smem_u32(tmem_holder)), "r"(kTmemColumns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    eb::cluster_sync();   // both CTAs' barriers exist before anything arrives on them from the other CTA
    tcgen05_fence_after();
    const uint32_t tmem = *tmem_holder;
    eb::pdl_launch_dependents();
    eb::pdl_wait();   // the scratch comes from the two launches before this one

    if (warp == 0) {
        if (lane == 0) {
            uint32_t step = 0;
            bool ok = true;
            for (uint32_t item = pair; item < items && ok; item += pairs) {
                uint32_t tm, tn;
                place(item, &tm, &tn);
                const uint32_t row_tile = 2u * tm + rank;                      // this CTA's 128 rows
                const uint32_t weight_tile = paired ? (rank == 0u ? tn : pair_tiles + tn) : 2u * tn + rank;   // its 128 weight rows
                const uint32_t low = paired ? tn : 2u * tn, high = paired ? pair_tiles + tn : 2u * tn + 1u;
                const uint32_t scale_tile = min(row_tile, row_tiles - 1u);     // a CTA without rows multiplies zeros by some tile's scales
                for (uint32_t ks = 0; ks < k_steps; ++ks, ++step) {
                    const uint32_t s = step % kPairStages, round = step / kPairStages;
                    if (round > 0 && !eb::mbar_wait(&empty[s], (round - 1u) & 1u)) {
                        atomicOr(error, 8u);
                        ok = false;
                        break;
                    }
                    uint8_t* stage = smem + s * kPairStageBytes;
                    eb::mbar_arrive_expect_tx(&full[s], kPairStageBytes);
                    tma_load_3d(stage, &map_a, (int)(ks * 128u), (int)(row_tile * kTileM), 0, &full[s]);
                    tma_load_3d(stage + kATile, &map_a, (int)(ks * 128u), (int)(row_tile * kTileM), 1, &full[s]);
                    tma_load_2d(stage + kTerms * kATile, &map_b, (int)(ks * 128u), (int)(weight_tile * 128u), &full[s]);
                    uint8_t* sf = stage + kTerms * kATile + kPairBTile;
                    eb::bulk_g2s(sf, sfa + ((uint64_t)scale_tile * k_blocks + ks * 4u) * kTerms * kAtom, kSfaStage, &full[s]);
                    eb::bulk_g2s(sf + kSfaStage, sfb + ((uint64_t)low * k_blocks + ks * 4u) * kAtom, 4u * kAtom, &full[s]);
                    eb::bulk_g2s(sf + kSfaStage + 4u * kAtom, sfb + ((uint64_t)high * k_blocks + ks * 4u) * kAtom, 4u * kAtom, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank != 0u) {
            // the odd CTA: tell the even one about every stage that has landed here
            uint32_t step = 0;
            bool ok = true;
            for (uint32_t item = pair; item < items && ok; item += pairs)
                for (uint32_t ks = 0; ks < k_steps; ++ks, ++step) {
                    const uint32_t s = step % kPairStages, round = step / kPairStages;
                    if (!eb::mbar_wait(&full[s], round & 1u)) {
                        atomicOr(error, 8u);
                        ok = false;
                        break;
                    }
                    arrive_at_rank(&peer_full[s], 0u);
                }
        } else if (lane == 0) {
            uint32_t step = 0, local = 0;
            bool ok = true;
            for (uint32_t item = pair; item < items && ok; item += pairs, ++local) {
                if (local > 0 && !eb::mbar_wait(acc_empty, (local - 1u) & 1u)) {
                    atomicOr(error, 8u);
                    break;
                }
                tcgen05_fence_after();
                for (uint32_t ks = 0; ks < k_steps; ++ks, ++step) {
                    const uint32_t s = step % kPairStages, round = step / kPairStages;
                    if (!eb::mbar_wait(&full[s], round & 1u) || !eb::mbar_wait(&peer_full[s], round & 1u)) {
                        atomicOr(error, 8u);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint8_t* stage = smem + s * kPairStageBytes;
                    const uint8_t* sf = stage + kTerms * kATile + kPairBTile;
                    const uint64_t a0 = tile_descriptor(stage), a1 = tile_descriptor(stage + kATile), b = tile_descriptor(stage + kTerms * kATile);
#pragma unroll
                    for (uint32_t j = 0; j < 4u; ++j) {
                        pair_copy_atom(tmem + kTmemSfa + (j * 2u) * 4u, atom_descriptor(sf + (j * 2u) * kAtom));
                        pair_copy_atom(tmem + kTmemSfb + j * 8u, atom_descriptor(sf + kSfaStage + j * kAtom));
                        pair_copy_atom(tmem + kTmemSfb + j * 8u + 4u, atom_descriptor(sf + kSfaStage + (4u + j) * kAtom));
                        pair_mma(tmem, a0 + 2u * j, b + 2u * j, tmem + kTmemSfa + (j * 2u) * 4u, tmem + kTmemSfb + j * 8u, (ks | j) != 0u);
                        pair_copy_atom(tmem + kTmemSfa + (j * 2u + 1u) * 4u, atom_descriptor(sf + (j * 2u + 1u) * kAtom));
                        pair_mma(tmem, a1 + 2u * j, b + 2u * j, tmem + kTmemSfa + (j * 2u + 1u) * 4u, tmem + kTmemSfb + j * 8u, 1u);
                    }
                    pair_commit(&empty[s]);
                }
                if (ok) pair_commit(acc_full);
            }
        }
    } else {
        // Epilogue, in both CTAs, each over its own 128 rows: as in gemm_kernel.
        const uint32_t quarter = warp & 3u, half = (warp - 2u) >> 2;
        const float scale_w = *tensor_global;
        uint32_t local = 0;
        for (uint32_t item = pair; item < items; item += pairs, ++local) {
            uint32_t tm, tn;
            place(item, &tm, &tn);
            if (!eb::mbar_wait(acc_full, local & 1u)) {
                if (lane == 0) atomicOr(error, 8u);
                break;
            }
            tcgen05_fence_after();
            uint32_t r[4][32];
            const uint32_t from = tmem + ((quarter * 32u) << 16) + (paired ? half * 64u : half * 128u);
            const uint32_t other = paired ? from + 128u : from + 64u;
            tmem_load_32(r[0], from);
            tmem_load_32(r[1], from + 32u);
            tmem_load_32(r[2], other);
            tmem_load_32(r[3], other + 32u);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) arrive_at_rank(acc_empty, 0u);
            const uint32_t row = (2u * tm + rank) * kTileM + quarter * 32u + lane;
            const float scale = row < rows ? __fmul_rn(row_globals[row], scale_w) : 0.0f;
            store_block(r, out, row, rows, n, paired ? tn * 128u + half * 64u : tn * kTileN + half * 128u, scale, paired);
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    eb::cluster_sync();   // neither CTA leaves while the other may still read its shared memory or arrive on its barriers
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns) : "memory");
    }
}

// Skinny calls: out[row][col] = bf16((sum over the K ranges in order) * row scale * tensor scale). One thread per 4 columns.
__global__ void __launch_bounds__(256) finish_splits(const float* __restrict__ partials, const float* __restrict__ row_globals,
        const float* __restrict__ tensor_global, uint16_t* __restrict__ out, uint32_t splits, uint32_t rows, uint32_t n) {
    const uint64_t index = (uint64_t)blockIdx.x * 256u + threadIdx.x;
    eb::pdl_launch_dependents();
    eb::pdl_wait();
    const uint32_t quads = n / 4u;
    if (index >= (uint64_t)rows * quads) return;
    const uint32_t row = (uint32_t)(index / quads), col = (uint32_t)(index % quads) * 4u;
    float4 sum = *reinterpret_cast<const float4*>(partials + (uint64_t)row * n + col);
    for (uint32_t s = 1; s < splits; ++s) {
        const float4 part = *reinterpret_cast<const float4*>(partials + ((uint64_t)s * rows + row) * n + col);
        sum.x = __fadd_rn(sum.x, part.x);
        sum.y = __fadd_rn(sum.y, part.y);
        sum.z = __fadd_rn(sum.z, part.z);
        sum.w = __fadd_rn(sum.w, part.w);
    }
    const float scale = __fmul_rn(row_globals[row], *tensor_global);
    const uint32_t lo = (uint32_t)eb::float_to_bf16_bits(__fmul_rn(sum.x, scale)) | (uint32_t)eb::float_to_bf16_bits(__fmul_rn(sum.y, scale)) << 16;
    const uint32_t hi = (uint32_t)eb::float_to_bf16_bits(__fmul_rn(sum.z, scale)) | (uint32_t)eb::float_to_bf16_bits(__fmul_rn(sum.w, scale)) << 16;
    *reinterpret_cast<uint2*>(out + (uint64_t)row * n + col) = make_uint2(lo, hi);
}

// ---- host side ------------------------------------------------------------------------------------------------------------

using eb::EncodeTiled;
using eb::encoder;

inline cudaError_t initialize() {
    const cudaError_t e = cudaFuncSetAttribute(gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSharedBytes);
    return e != cudaSuccess ? e : cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPairShared);
}

constexpr uint32_t kPairRows = 512;   // fewer rows than this always run on single CTAs

template <typename... Params, typename... Args>
inline cudaError_t launch_on(cudaStream_t stream, bool pdl, void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = pdl ? 1u : 0u;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// The three launches of a native linear. Shapes are pre-checked by the caller: k % 256 == 0, out_features % 128 == 0,
// scratch aligned to 16 bytes and at least ActivationLayout(rows, k, out_features).bytes long.
// quantize: BF16 rows -> the activation part of the scratch (code planes, scale atoms, row scales).
inline cudaError_t quantize(const void* input, void* scratch, uint32_t rows, uint32_t k, cudaStream_t stream, bool pdl) {
    return launch_on(stream, pdl, quantize_rows, dim3((rows + kQuantizeWarps - 1u) / kQuantizeWarps), dim3(32u * kQuantizeWarps), 0,
            static_cast<const __nv_bfloat16*>(input), static_cast<uint8_t*>(scratch), rows, k);
}

// multiply: the weight scale plane -> scale atoms in the scratch, then the GEMM over the quantized activations found there.
// paired: the weights are a gate/up object (gate rows first); the output is [rows][out_features / 2] SwiGLU values.
// pairs: calls of kPairRows rows and more run on CTA pairs (gemm_pair_kernel).
inline cudaError_t multiply(const void* weights, void* output, void* scratch, uint32_t rows, uint32_t k, uint32_t out_features, int sms,
        cudaStream_t stream, bool pdl, uint32_t* error, bool paired = false, bool pairs = false, bool table_scales = false) {
    const EncodeTiled encode = encoder();
    if (encode == nullptr) return cudaErrorNotSupported;
    const ActivationLayout layout(rows, k, out_features);
    uint8_t* base = static_cast<uint8_t*>(scratch);
    const uint8_t* w = static_cast<const uint8_t*>(weights);
    const uint64_t row_bytes = k / 2u;
    // plain: scale bytes, then the FP32 tensor scale; table-indexed: index bytes, then 16 table codes and the tensor scale
    const uint64_t scale_offset = align256((uint64_t)out_features * row_bytes);
    const uint64_t table_offset = align256(scale_offset + (uint64_t)out_features * (k / (table_scales ? 32u : 16u)));
    const uint64_t global_offset = table_scales ? table_offset + 16u : table_offset;
    CUtensorMap map_a, map_b;
    const cuuint32_t ones[3] = {1u, 1u, 1u};
    const cuuint64_t a_dims[3] = {row_bytes, rows, kTerms}, a_strides[2] = {row_bytes, row_bytes * rows};
    const cuuint32_t a_box[3] = {128u, kTileM, 1u};
    const cuuint64_t b_dims[2] = {row_bytes, out_features}, b_strides[1] = {row_bytes};
    const cuuint32_t b_box[2] = {128u, 128u};   // half a B tile: the kernel places the two halves itself
    CUresult r = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base, a_dims, a_strides, a_box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS)
        r = encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(w), b_dims, b_strides, b_box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    const uint32_t n_padded = (out_features + 255u) / 256u * 256u;
    const uint64_t items = (uint64_t)n_padded * layout.k_blocks;
    cudaError_t e = launch_on(stream, pdl, repack_weight_scales, dim3((unsigned)((items + 255u) / 256u)), dim3(256), 0, w + scale_offset,
            table_scales ? w + table_offset : static_cast<const uint8_t*>(nullptr), base + layout.sfb_offset, out_features, layout.k_blocks, n_padded);
    if (e != cudaSuccess) return e;
    const uint32_t pair_tiles = paired ? out_features / 256u : 0u, width = paired ? out_features / 2u : out_features;
    const uint32_t tiles = ((rows + kTileM - 1u) / kTileM) * (paired ? pair_tiles : (out_features + kTileN - 1u) / kTileN);
    // The skinny route (the reference's 9..64-row kernel, native/src/nvfp4_native/native.cuh:435-585, cuts K the same way):
    // few rows make few output tiles; K is cut so that about every SM gets a work item.
    uint32_t splits = 1;
    if (!paired && rows <= kSkinnyRows && tiles * 2u <= (uint32_t)sms) splits = std::max(1u, std::min(std::min(kMaxSplits, k / kStepK), (uint32_t)sms / tiles));
    const uint32_t work = tiles * splits, grid = work < (uint32_t)sms ? work : (uint32_t)sms;
    float* partials = reinterpret_cast<float*>(base + layout.partial_offset);
    const float* row_globals = reinterpret_cast<const float*>(base + layout.global_offset);
    const float* tensor_global = reinterpret_cast<const float*>(w + global_offset);
    if (pairs && rows >= kPairRows) {
        const uint32_t pair_items = ((rows + 255u) / 256u) * (paired ? pair_tiles : (out_features + 255u) / 256u);
        const uint32_t ctas = 2u * std::max(1u, std::min((uint32_t)sms / 2u, pair_items));
        return launch_on(stream, pdl, gemm_pair_kernel, dim3(ctas), dim3(kThreads), kPairShared, map_a, map_b, base + layout.sfa_offset,
                base + layout.sfb_offset, row_globals, tensor_global, static_cast<uint16_t*>(output), rows, width, k, pair_tiles, error);
    }
    e = launch_on(stream, pdl, gemm_kernel, dim3(grid), dim3(kThreads), kSharedBytes, map_a, map_b, base + layout.sfa_offset,
            base + layout.sfb_offset, row_globals, tensor_global, static_cast<uint16_t*>(output), partials, splits, rows, width, k, pair_tiles, error);
    if (e != cudaSuccess || splits == 1u) return e;
    const uint64_t quads = (uint64_t)rows * (out_features / 4u);
    return launch_on(stream, pdl, finish_splits, dim3((unsigned)((quads + 255u) / 256u)), dim3(256), 0, partials, row_globals, tensor_global,
            static_cast<uint16_t*>(output), splits, rows, out_features);
}

inline cudaError_t run(const void* input, const void* weights, void* output, void* scratch, uint32_t rows, uint32_t k, uint32_t out_features,
        int sms, cudaStream_t stream, bool pdl, uint32_t* error, bool paired = false, bool pairs = false, bool table_scales = false) {
    const cudaError_t e = quantize(input, scratch, rows, k, stream, pdl);
    return e != cudaSuccess ? e : multiply(weights, output, scratch, rows, k, out_features, sms, stream, pdl, error, paired, pairs, table_scales);
}

}  // namespace nvfp4n
