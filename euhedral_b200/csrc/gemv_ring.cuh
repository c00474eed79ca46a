// The decode GEMV skeleton shared by the NVFP4 and Q3 formats on sm_100a: y[M, N] = x[M, K] . W^T for 1 to 8 BF16
// activation rows, with the format (byte geometry, activation staging, register decode) supplied as a policy class.
//
//   * A CTA owns a run of 16-row tiles of the weight and one K slice; the S CTAs of a thread-block cluster own the S
//     slices of the same rows. Tile i's S partial sums go through distributed shared memory to rank i % S, which adds
//     them in rank order. S depends on K only, so a row's summation order is a function of K alone: N-sharded copies
//     of a tensor give bitwise the unsharded result.
//   * The grid is either one tile per warp, when all of it is resident at once, or as many clusters as the GPU holds
//     at two CTAs per SM, each with an even share of the tiles: no second wave of CTAs, the activation slice is staged
//     once per CTA, and every SM gets the same work.
//   * Warp w of RT takes tiles w, w + RT, .. of its CTA and runs its own pipeline over them, one after the other
//     without draining: a private ring of 2 or 3 shared-memory slots, each slot two boxes of 16 rows x two 128-value
//     chunks of code bytes, each box fetched by a single tiled TMA copy through a tensor map of the code plane (one
//     instruction per box, completion of both on the slot's mbarrier). The copy engine moves the code bytes past L1
//     and the load/store unit; the warp decodes slot i while slots i+1.. are in flight, and no CTA-wide barrier is
//     taken after the activations are staged, so the warps of an SM drift apart instead of loading and computing in
//     lock-step.
//   * The block scales are too small and too misaligned for TMA (a slice may start at any multiple of 4 bytes): a warp
//     brings the scales of a whole tile (16 rows x the slice) into a private double buffer with 4- or 8-byte cp.async
//     copies, one tile ahead of the tile it is decoding.
//   * Weights do not depend on the previous kernel, so the whole ring is requested before griddepcontrol.wait: under
//     programmatic dependent launch the weight stream of call i+1 overlaps the tail of call i.
//   * mma.sync.m16n8k16 (BF16, FP32 accumulate) with weights as the 16-row operand and the activation rows as the 8
//     columns: each activation row is computed independently of the others (row exactness). Lanes whose column is
//     beyond the last activation row read the last row again; their sums are never stored.
//
// A policy F provides:
//   Geometry(n, k)                  byte geometry of the tensor: row_bytes, scale_row_bytes, scale_offset
//   kCodeBytes, kScaleBytes         bytes per row and chunk of codes / of scales
//   kErrorBit                       bit of the device error word for a wait that gave up
//   extra_bytes(chunks)             extra shared bytes next to the activation slice
//   stage(...)                      CTA-wide staging of the activation slice in the decode's pairing
//   lane_scale_offset(q)            byte offset of lane q's scales within a chunk's scale bytes
//   State                           accumulators: chunk<I>(...) consumes chunk I of a slot given the shared addresses of
//                                   the slot's codes (row g of box 0; row g+8 is 8 ring rows further, box 1 sixteen),
//                                   of the two rows' scales and of the lane's activations, and the slot's first
//                                   chunk index; result(out) yields the lane's four sums; reset()
//   Finish(w, geo)                  apply(sum) = the value to round to BF16
#pragma once

#include "common.cuh"

namespace gemv {

// Diagnostic build only (-DEB_X_TRACE): thread 0 of every CTA records the global timer at six points of the kernel and
// its SM, read back through euhedral_b200_debug_trace. The regular build compiles none of it.
#ifdef EB_X_TRACE
__device__ unsigned long long g_trace[4 * 2048 * 8];
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define EB_TRACE(slot) if (tid == 0 && blockIdx.x < 2048) g_trace[((trace_generation & 3u) * 2048 + blockIdx.x) * 8 + (slot)] = now_ns()
#define EB_TRACE_SM() if (tid == 0 && blockIdx.x < 2048) { unsigned sm; asm volatile("mov.u32 %0, %%smid;" : "=r"(sm)); g_trace[((trace_generation & 3u) * 2048 + blockIdx.x) * 8 + 7] = sm; }
#else
#define EB_TRACE(slot)
#define EB_TRACE_SM()
#endif

constexpr uint32_t kChunk = 128;   // K values per chunk
constexpr uint32_t kBox = 2;       // chunks per TMA box (16 rows x kBox chunks)
constexpr uint32_t kMaxPair = 2;   // boxes per ring slot, 1 or 2 (chosen by the launcher): one mbarrier wait covers up to four chunks
constexpr uint32_t kMaxRows = 8;   // activation rows per launch
constexpr uint32_t kMaxSplit = 8;  // portable cluster size
constexpr uint32_t kMaxSlots = 3;  // ring slots per warp: 2 or 3, chosen by the launcher

// K slices per row (cluster size): a function of K alone.
__host__ __device__ inline uint32_t split_of(uint32_t k) {
    const uint32_t chunks = k / kChunk;
    return chunks <= 12u ? 1u : chunks <= 24u ? 2u : chunks <= 48u ? 4u : 8u;
}

// Shared memory of one CTA.
template <class F>
struct Layout {
    uint32_t stride_x, stride_scales, off_extra, off_gather, off_scales, off_ring, off_bars, bytes;
    // span: the most 16-row tiles a CTA owns; slots: ring slots per warp; pair: boxes per slot.
    __host__ __device__ Layout(uint32_t rt, uint32_t span, uint32_t slots, uint32_t pair, uint32_t chunks_max, uint32_t rows, uint32_t split) {
        stride_x = chunks_max * 256u + 64u;   // 64 modulo 128: the rows a quarter-warp reads fall in distinct banks
        stride_scales = (chunks_max + 1u) * F::kScaleBytes;   // an odd number of pieces: rows fall in distinct banks
        off_extra = rows * stride_x;
        off_gather = off_extra + F::extra_bytes(chunks_max);
        off_scales = (off_gather + (split > 1u ? (span + split - 1u) / split * split * 16u * rows * 4u : 0u) + 15u) & ~15u;
        off_ring = (off_scales + rt * 2u * 16u * stride_scales + 127u) & ~127u;
        off_bars = off_ring + rt * slots * pair * 16u * kBox * F::kCodeBytes;
        bytes = off_bars + rt * slots * 8u;
    }
};

// The tensor map of a code plane: bytes [n rows][row_bytes], boxes of 16 rows x kBox chunks, no swizzle.
template <class F>
inline bool encode_codes(CUtensorMap* map, const void* weights, uint32_t n, uint32_t k) {
    const eb::EncodeTiled encode = eb::encoder();
    if (encode == nullptr) return false;
    const typename F::Geometry geo(n, k);
    const cuuint64_t dims[2] = {geo.row_bytes, n}, strides[1] = {geo.row_bytes};
    const cuuint32_t box[2] = {kBox * F::kCodeBytes, 16u}, ones[2] = {1u, 1u};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(weights), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
            == CUDA_SUCCESS;
}

// WARPS_PER_SM bounds the registers: 24 for the all-resident grid (three CTAs of eight warps per SM), 16 for the
// persistent grid (two per SM, more registers: nothing is recomputed inside the box loop).
template <class F, int RT, int WARPS_PER_SM>
__global__ void __launch_bounds__(32 * RT, WARPS_PER_SM / RT) kernel(const __grid_constant__ CUtensorMap codes, const uint16_t* __restrict__ x,
        const uint8_t* __restrict__ w, uint16_t* __restrict__ y, uint32_t rows, uint32_t k, uint32_t n, uint32_t split, uint32_t span,
        uint32_t slots, uint32_t pair, uint32_t* __restrict__ error
#ifdef EB_X_TRACE
        , uint32_t trace_generation
#endif
        ) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t kRb = 16u * RT, kThreads = 32u * RT, kRowBytes = kBox * F::kCodeBytes, kBoxBytes = 16u * kRowBytes;
    const uint32_t slot_bytes = pair * kBoxBytes, slot_chunks = pair * kBox;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, q = lane & 3u;
    const uint32_t rank = split > 1u ? eb::cluster_rank() : 0u;
    // The clusters share the tensor's 16-row tiles evenly: cluster i of G owns tiles [i T / G, (i + 1) T / G), at most `span`.
    const uint32_t groups = gridDim.x / split, group = blockIdx.x / split, all_tiles = n / 16u;
    const uint32_t tile_begin = (uint32_t)((uint64_t)group * all_tiles / groups), tile_end = (uint32_t)((uint64_t)(group + 1u) * all_tiles / groups);
    const uint32_t cta_tiles = tile_end - tile_begin, row0 = tile_begin * 16u;
    const uint32_t chunks = k / kChunk;
    const uint32_t c_begin = (uint32_t)((uint64_t)rank * chunks / split), c_end = (uint32_t)((uint64_t)(rank + 1u) * chunks / split);
    const uint32_t nc = c_end - c_begin, nc_max = (chunks + split - 1u) / split;
    const uint32_t boxes = (nc + slot_chunks - 1u) / slot_chunks;   // ring slots (box pairs) per tile
    const Layout<F> layout(RT, span, slots, pair, nc_max, rows, split);
    const typename F::Geometry geo(n, k);
    const uint32_t smem_a = eb::smem_u32(smem);
    const uint32_t ring_a = smem_a + layout.off_ring + warp * slots * slot_bytes;
    const uint32_t bars_a = smem_a + layout.off_bars + warp * slots * 8u;
    const uint32_t scale_bytes = 16u * layout.stride_scales, scales_a = smem_a + layout.off_scales + warp * 2u * scale_bytes;
    float* gather = reinterpret_cast<float*>(smem + layout.off_gather);
    EB_TRACE(0);
    EB_TRACE_SM();

    // The warp's tiles: warp, warp + RT, warp + 2 RT .. of the CTA's tiles. The boxes of all its tiles form one
    // sequence, so the ring keeps streaming across tiles. Lane (g, q) decodes rows g and g+8 of a tile.
    const uint32_t first_row = row0 + warp * 16u;
    const uint32_t tiles = warp < cta_tiles ? (cta_tiles - warp + RT - 1u) / RT : 0u;
    const uint32_t total = tiles * boxes;

    if (lane == 0) {
        for (uint32_t s = 0; s < slots; ++s) eb::mbar_init(reinterpret_cast<uint64_t*>(smem + layout.off_bars) + warp * slots + s, 1);
        eb::mbar_fence_init();
    }
    __syncwarp();

    // The scales of the warp's tile `t` into scale buffer t % 2: lane l copies row l % 16, every other piece.
    auto fetch_scales = [&](uint32_t t) {
        if (t < tiles) {
            const uint8_t* from = w + geo.scale_offset + (uint64_t)(first_row + t * kRb + (lane & 15u)) * geo.scale_row_bytes
                    + (uint64_t)c_begin * F::kScaleBytes;
            const uint32_t to = scales_a + (t & 1u) * scale_bytes + (lane & 15u) * layout.stride_scales;
            for (uint32_t piece = lane >> 4; piece < nc; piece += 2u) {
                if (F::kScaleBytes == 8u) eb::cp_async_8_to(to + piece * 8u, from + piece * 8u);
                else eb::cp_async_4_to(to + piece * 4u, from + piece * 4u);
            }
        }
        eb::cp_async_commit();
    };
    // Requests the next box pair of the sequence into slot `slot`; the slot's previous contents have been consumed by
    // every lane. The second box is skipped when the slice ends before it; a box that reaches past the slice or the row
    // brings bytes that are never decoded (zeros past the row).
    uint32_t ask_box = 0, ask_row = first_row, unasked = total;
    auto request = [&](uint32_t slot) {
        if (lane == 0) {
            const uint32_t first = ask_box * slot_chunks;
            const bool both = pair == 2u && first + kBox < nc;
            const uint32_t bar = bars_a + slot * 8u, to = ring_a + slot * slot_bytes;
            eb::tma_load_2d_expect(to, &codes, (int)((c_begin + first) * F::kCodeBytes), (int)ask_row, bar, both ? slot_bytes : kBoxBytes);
            if (both) eb::tma_load_2d_at(to + kBoxBytes, &codes, (int)((c_begin + first + kBox) * F::kCodeBytes), (int)ask_row, bar);
        }
        --unasked;
        if (++ask_box == boxes) {
            ask_box = 0;
            ask_row += kRb;
        }
    };
    for (uint32_t s = 0; s < slots; ++s) {
        if (s < total) request(s);
    }
    fetch_scales(0);
    fetch_scales(1);
    const typename F::Finish finish(w, geo);

    // The activations may come from the kernel before this one.
    eb::pdl_launch_dependents();
    EB_TRACE(1);
    eb::pdl_wait();
    EB_TRACE(2);
    F::stage(smem, smem + layout.off_extra, x, rows, k, c_begin, nc, layout.stride_x, tid, kThreads);
    __syncthreads();
    EB_TRACE(3);

    const uint32_t x_a = eb::pinned(smem_a + (g < rows ? g : rows - 1u) * layout.stride_x + q * 16u);
    const uint32_t ring_lane = eb::pinned(ring_a + g * kRowBytes), scale_lane = eb::pinned(g * layout.stride_scales + F::lane_scale_offset(q));
    const uint32_t t0 = 2u * q;
    typename F::State state(smem_a + layout.off_extra, q);
    static_assert(kBox == 2 && kMaxPair == 2, "the slot loop below decodes up to four chunks per slot");
    bool complete = true;
    uint32_t slot = 0, parity = 0, row_g = first_row + g;
    for (uint32_t t = 0; t < tiles; ++t) {
        eb::cp_async_wait_group<1>();
        __syncwarp();
        state.reset();
        const uint32_t scale_g = scales_a + (t & 1u) * scale_bytes + scale_lane;
        for (uint32_t box = 0; box < boxes; ++box) {
            complete = eb::mbar_wait_at(bars_a + slot * 8u, parity) && complete;
            // Everything a slot needs hangs off four shared addresses; the offsets inside are compile-time constants.
            const uint32_t code_slot = ring_lane + slot * slot_bytes;
            const uint32_t first = box * slot_chunks, left = min(slot_chunks, nc - first);
            const uint32_t scale_slot = scale_g + first * F::kScaleBytes, x_slot = x_a + first * 256u;
            const uint32_t scale_slot_h = scale_slot + 8u * layout.stride_scales;
            state.template chunk<0>(code_slot, scale_slot, scale_slot_h, x_slot, first);
            if (left > 1u) state.template chunk<1>(code_slot, scale_slot, scale_slot_h, x_slot, first);
            if (left > 2u) state.template chunk<2>(code_slot, scale_slot, scale_slot_h, x_slot, first);
            if (left > 3u) state.template chunk<3>(code_slot, scale_slot, scale_slot_h, x_slot, first);
            __syncwarp();
            if (unasked != 0u) request(slot);
            if (++slot == slots) {
                slot = 0;
                parity ^= 1u;
            }
        }
        // The tile is done: lane (g, q) holds rows g and g+8 for activation rows 2q and 2q+1.
        float acc[4];
        state.result(acc);
        if (split == 1u) {
            if (t0 < rows) {
                y[(uint64_t)t0 * n + row_g] = eb::float_to_bf16_bits(finish.apply(acc[0]));
                y[(uint64_t)t0 * n + row_g + 8u] = eb::float_to_bf16_bits(finish.apply(acc[2]));
            }
            if (t0 + 1u < rows) {
                y[(uint64_t)(t0 + 1u) * n + row_g] = eb::float_to_bf16_bits(finish.apply(acc[1]));
                y[(uint64_t)(t0 + 1u) * n + row_g + 8u] = eb::float_to_bf16_bits(finish.apply(acc[3]));
            }
        } else {
            // Tile i of the CTA is summed by rank i % S: its gather buffer is [i / S][source rank][row of the tile][activation row].
            const uint32_t tile = warp + t * RT, owner = tile % split;
            const uint32_t at = eb::map_to_rank(smem_a + layout.off_gather, owner) + ((((tile / split) * split + rank) * 16u + g) * rows + t0) * 4u;
            if (t0 < rows) {
                eb::st_cluster_f32(at, acc[0]);
                eb::st_cluster_f32(at + 8u * rows * 4u, acc[2]);
            }
            if (t0 + 1u < rows) {
                eb::st_cluster_f32(at + 4u, acc[1]);
                eb::st_cluster_f32(at + 8u * rows * 4u + 4u, acc[3]);
            }
        }
        row_g += kRb;
        __syncwarp();
        fetch_scales(t + 2u);
    }
    eb::cp_async_wait_all();
    if (!complete && lane == 0) atomicOr(error, F::kErrorBit);
    EB_TRACE(4);
    if (split == 1u) {
        EB_TRACE(6);
        return;
    }
    // Every rank adds the slices' sums of the tiles it owns, in rank order.
    eb::cluster_sync();
    EB_TRACE(5);
    const uint32_t owned = cta_tiles > rank ? (cta_tiles - rank + split - 1u) / split : 0u;
    for (uint32_t i = tid; i < owned * 16u * rows; i += kThreads) {
        const uint32_t local = i / (16u * rows), rest = i - local * (16u * rows), t = rest >> 4, r = rest & 15u;
        const float* from = gather + (local * split * 16u + r) * rows + t;
        float sum = from[0];
        for (uint32_t s = 1; s < split; ++s) sum += from[s * 16u * rows];
        y[(uint64_t)t * n + row0 + (local * split + rank) * 16u + r] = eb::float_to_bf16_bits(finish.apply(sum));
    }
    EB_TRACE(6);
}

}  // namespace gemv
