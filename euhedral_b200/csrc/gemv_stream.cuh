// The decode GEMV skeleton shared by the NVFP4 and Q3 formats on sm_100a: y[M, N] = x[M, K] . W^T for 1 to 8 BF16
// activation rows, for ONE weight tensor or for a GROUP of tensors that share K and the row count (the q, k, v
// projections of a layer, or gate and up), all in one persistent launch. The format (byte geometry, activation staging,
// register decode) is a policy class.
//
// Summation order (a function of the format and K only, so that every row of a multi-row call, every N-shard of a
// tensor and every member of a group gives bitwise the result of its own one-row, whole-tensor, single call):
//   * K is cut into S slices (S = 1 up to K = 6144, then 2, 4, 8) and a slice into T pieces of P or P - 1 chunks of 128
//     values (T a power of two up to 16). A piece's 16 x pc x 128 products are summed by the tensor core in chunk order.
//   * The T piece sums of a slice are added in piece order, the S slice sums in slice order.
//
// Execution:
//   * One CTA per SM (a cluster of S CTAs when S > 1, rank r staging and streaming slice r only). The 16-row tiles of
//     all tensors of the group form one list, cut evenly over the CTAs (clusters): a CTA walks a contiguous run of it.
//   * A CTA's warps form teams of T; team member j owns piece j of every tile its team takes. A warp streams its pieces
//     through a private ring of 2 or 3 shared-memory slots. A slot is filled by two tiled TMA copies signalled on one
//     mbarrier: the piece's code bytes through a tensor map of the code plane - always a box of 16 rows x P chunks, so a
//     piece of P - 1 chunks brings one chunk it does not decode (the next piece's first, or zeros past the row): rows
//     of P chunks keep the shared-memory loads of a warp free of bank conflicts for both piece widths - and the piece's
//     block scales through a tensor map of the scale plane whose box is widened to start on a 16-byte boundary (the
//     lane indexes from the remainder). The ring runs ahead across tiles and across the tensors of the group. Scale
//     planes whose row pitch is not a multiple of 16 bytes cannot be described to TMA; their scales come by cp.async.
//   * Weights do not depend on the kernel before this one: the rings are requested before griddepcontrol.wait.
//   * A piece is decoded straight-line (every shared-memory offset an immediate) into mma.sync.m16n8k16 (BF16, FP32
//     accumulate), weights as the 16-row operand and the activation rows as the 8 columns, so that each activation row
//     is computed independently of the others. Lanes whose column is beyond the last activation row read the last row
//     again; those sums are never used.
//   * The T piece sums of a tile meet in shared memory and are added in piece order, then rounded and stored as BF16
//     (S = 1) or handed to the tile's owner rank through distributed shared memory; owners add the S slice sums in
//     rank order after a cluster barrier at the end of each tensor. Who adds is the policy's choice (kAddingWarp):
//     the team itself after a named barrier per tile (teams of 8: the barrier costs less than the hand-over), or one
//     extra warp of the CTA that the teams signal through mbarriers, so that no decoding warp ever waits for another
//     (teams of 16, where the barrier would stop the whole CTA once per tile).
//
// A policy F provides:
//   Geometry(n, k)                  byte geometry of the tensor: row_bytes, scale_row_bytes, scale_offset
//   kCodeBytes, kScaleBytes         bytes per row and chunk of codes / of scales
//   kScaleBox                       bytes per row of a slot's scale box (a multiple of 16, >= kMaxPiece * kScaleBytes + 12,
//                                   an odd multiple of 16 so that the rows of a quarter-warp fall in distinct banks)
//   kPieceChunks, kMaxPiece         preferred and largest chunks per piece
//   kErrorBit                       bit of the device error word for a wait that gave up
//   kAddingWarp                     whether an extra warp adds the piece sums (else the team does, behind a barrier)
//   extra_bytes(chunks)             extra shared bytes next to the activation slice
//   stage(...)                      CTA-wide staging of the activation slice in the decode's pairing
//   lane_scale_offset(q)            byte offset of lane q's scales within a chunk's scale bytes
//   State                           accumulators: tensor(w, geo) at the start of every tensor; chunk<I, W>(codes, scales, x) consumes chunk I of a piece whose box rows
//                                   are W chunks wide, given the lane's shared addresses; result(out); reset()
//   Finish(w, geo)                  apply(sum) = the value to round to BF16
#pragma once

#include "common.cuh"

namespace gemv {

constexpr uint32_t kChunk = 128;    // K values per chunk
constexpr uint32_t kMaxRows = 8;    // activation rows per launch
constexpr uint32_t kMaxWarps = 16;  // one CTA per SM
constexpr uint32_t kMaxGroup = 8;   // tensors per launch
constexpr uint32_t kPartial = 512;  // bytes of one piece's sums: 16 rows x 8 columns of FP32

// How K is cut: fixes the summation order.
struct Order {
    uint32_t chunks, split, team, piece;   // chunks of 128, slices, pieces per slice, chunks of the widest piece
    bool ok;
};

template <class F>
__host__ __device__ inline Order order_of(uint32_t k) {
    Order o;
    o.chunks = k / kChunk;
    o.split = o.chunks <= 48u ? 1u : o.chunks <= 96u ? 2u : o.chunks <= 192u ? 4u : 8u;
    const uint32_t widest = (o.chunks + o.split - 1u) / o.split, narrowest = o.chunks / o.split;
    o.team = 1u;
    while (o.team < kMaxWarps && (widest + o.team - 1u) / o.team > F::kPieceChunks && o.team * 2u <= narrowest) o.team *= 2u;
    o.piece = (widest + o.team - 1u) / o.team;
    o.ok = k != 0u && k % kChunk == 0u && o.piece <= F::kMaxPiece;
    return o;
}

// One tensor of a group.
struct alignas(64) Tensor {
    CUtensorMap codes;         // box: 16 rows x `piece` chunks
    CUtensorMap scales;        // box: 16 rows x F::kScaleBox bytes
    const uint16_t* x;
    const uint8_t* w;
    uint16_t* y;
    uint32_t n;
    uint32_t tile_end;         // end of this tensor's tiles in the group's list
};

struct alignas(64) Group {
    Tensor tensor[kMaxGroup];
    uint32_t count, rows, k, tiles;   // tensors, activation rows, K, 16-row tiles of all tensors together
    uint32_t depth, span;             // ring slots per warp; the most tiles of one tensor a cluster takes (S > 1)
};

// Shared memory of one CTA.
template <class F>
struct Layout {
    uint32_t stride_x, off_extra, off_partials, off_gather, off_slots, off_bars, off_sum_bars, slot_bytes, code_bytes, bytes;
    __host__ __device__ Layout(const Order& o, uint32_t rows, uint32_t warps, uint32_t depth, uint32_t span) {
        const uint32_t widest = (o.chunks + o.split - 1u) / o.split;
        stride_x = widest * 256u + 64u;   // 64 modulo 128: the rows a quarter-warp reads fall in distinct banks
        off_extra = rows * stride_x;
        off_partials = (off_extra + F::extra_bytes(widest) + 127u) & ~127u;
        off_gather = off_partials + warps * 2u * kPartial;
        const uint32_t owned = o.split > 1u ? (span + o.split - 1u) / o.split + 1u : 0u;
        off_slots = (off_gather + owned * o.split * kPartial + 127u) & ~127u;
        code_bytes = 16u * o.piece * F::kCodeBytes;
        slot_bytes = code_bytes + 16u * F::kScaleBox;
        off_bars = off_slots + warps * depth * slot_bytes;
        off_sum_bars = off_bars + warps * depth * 8u;   // per team and sum buffer: a full and an empty barrier
        bytes = off_sum_bars + (F::kAddingWarp ? (warps / o.team) * 2u * 16u : 0u);
    }
};

// The tensor maps of one weight tensor. Codes: 32-bit elements [n rows][row_bytes / 4], boxes of 16 rows x `piece` chunks.
// Scales: bytes [n rows][scale_row_bytes], boxes of 16 rows x kScaleBox bytes (only when the pitch is a multiple of 16).
template <class F>
inline bool encode_tensor(Tensor* t, const void* weights, uint32_t n, uint32_t k, const Order& o, bool tma_scales) {
    const eb::EncodeTiled encode = eb::encoder();
    if (encode == nullptr) return false;
    const typename F::Geometry geo(n, k);
    const cuuint32_t ones[2] = {1u, 1u};
    const cuuint64_t dims[2] = {geo.row_bytes / 4u, n}, strides[1] = {geo.row_bytes};
    const cuuint32_t box[2] = {o.piece * F::kCodeBytes / 4u, 16u};
    if (encode(&t->codes, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(weights), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
            != CUDA_SUCCESS)
        return false;
    if (!tma_scales) {
        t->scales = t->codes;
        return true;
    }
    const cuuint64_t sdims[2] = {geo.scale_row_bytes, n}, sstrides[1] = {geo.scale_row_bytes};
    const cuuint32_t sbox[2] = {F::kScaleBox, 16u};
    return encode(&t->scales, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(static_cast<const uint8_t*>(weights) + geo.scale_offset),
                   sdims, sstrides, sbox, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
            == CUDA_SUCCESS;
}

__device__ __forceinline__ void team_sync(uint32_t team, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(team + 1u), "r"(threads) : "memory");
}
__device__ __forceinline__ void st_shared_f2(uint32_t address, float a, float b) {
    asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(address), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ float ld_shared_f(uint32_t address) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(address) : "memory");
    return v;
}

// Decodes one piece of PC chunks from a filled slot into the lane's four sums.
template <class F, int P, int PC>
__device__ __forceinline__ void decode_piece(typename F::template State<P>& state, uint32_t codes, uint32_t scales, uint32_t x, float (&acc)[4]) {
    state.reset();
    eb::static_for<PC>([&](auto index) {
        constexpr int I = decltype(index)::value;
        state.template chunk<I, P>(codes, scales, x);   // the box rows are always P chunks wide
    });
    state.result(acc);
}

template <class F, int P, bool kTmaScales>
__global__ void __launch_bounds__(32 * (kMaxWarps + (F::kAddingWarp ? 1 : 0)), 1) kernel(const __grid_constant__ Group group, uint32_t* __restrict__ error) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, q = lane & 3u;
    constexpr bool kAdder = F::kAddingWarp;   // piece sums are added by a warp of their own (the CTA's last) or by the team itself
    const uint32_t warps = (blockDim.x >> 5) - (kAdder ? 1u : 0u), threads = blockDim.x;   // decoding warps
    const uint32_t rows = group.rows, depth = group.depth;
    const Order order = order_of<F>(group.k);
    const uint32_t split = order.split, team_size = order.team;
    const uint32_t teams = warps / team_size;
    const uint32_t rank = split > 1u ? eb::cluster_rank() : 0u;
    const uint32_t clusters = gridDim.x / split, cluster = blockIdx.x / split;
    // This cluster's run of the group's tile list.
    const uint32_t run_begin = (uint32_t)((uint64_t)cluster * group.tiles / clusters), run_end = (uint32_t)((uint64_t)(cluster + 1u) * group.tiles / clusters);
    const uint32_t slice_begin = (uint32_t)((uint64_t)rank * order.chunks / split), slice_end = (uint32_t)((uint64_t)(rank + 1u) * order.chunks / split);
    const uint32_t slice = slice_end - slice_begin;
    const Layout<F> layout(order, rows, warps, depth, group.span);
    const uint32_t smem_a = eb::smem_u32(smem);
    // Piece sums travel from a team's warps to the adding warp through two buffers per team, each guarded by a `full`
    // barrier (one arrival per team member) and an `empty` barrier (one arrival by the adding warp).
    const uint32_t sums_a = smem_a + layout.off_sum_bars;   // [team][buffer][full, empty]

    if (warp < warps) {
        if (lane == 0) {
            for (uint32_t s = 0; s < depth; ++s) eb::mbar_init(reinterpret_cast<uint64_t*>(smem + layout.off_bars) + warp * depth + s, 1);
        }
    } else if (kAdder && lane == 0) {
        for (uint32_t i = 0; i < teams * 2u; ++i) {
            eb::mbar_init(reinterpret_cast<uint64_t*>(smem + layout.off_sum_bars) + 2u * i, team_size);
            eb::mbar_init(reinterpret_cast<uint64_t*>(smem + layout.off_sum_bars) + 2u * i + 1u, 1);
        }
    }
    if (lane == 0) eb::mbar_fence_init();
    __syncwarp();
    if (split > 1u) eb::cluster_arrive();   // every CTA of the cluster has started before its shared memory is written to

    bool complete = true;
    const uint16_t* staged = nullptr;
    // Stages a tensor's activations when they are not the ones in shared memory already. Taken by every warp of the CTA
    // at the same points of the tensor loop.
    auto stage = [&](const Tensor& t) {
        if (t.x != staged) {
            __syncthreads();   // every warp is done with the activations staged before
            F::stage(smem, smem + layout.off_extra, t.x, rows, group.k, slice_begin, slice, layout.stride_x, tid, threads);
            staged = t.x;
            __syncthreads();
        }
    };
    // With K slices: every rank adds the slice sums of the tiles it owns, in rank order. Taken by every thread of the cluster.
    auto join_slices = [&](const Tensor& t, uint32_t first_tile, uint32_t segment_begin, uint32_t segment_end) {
        const typename F::Finish finish(t.w, typename F::Geometry(t.n, group.k));
        eb::cluster_sync();
        const uint32_t count = segment_end - segment_begin;
        const uint32_t owned = count > rank ? (count - rank + split - 1u) / split : 0u;
        for (uint32_t e = tid; e < owned * 128u; e += threads) {
            const uint32_t local = e >> 7, rest = e & 127u, column = rest & 7u, row = rest >> 3;
            if (column < rows) {
                const uint32_t from = smem_a + layout.off_gather + local * split * kPartial + rest * 4u;
                float sum = ld_shared_f(from);
                for (uint32_t s = 1; s < split; ++s) sum = __fadd_rn(sum, ld_shared_f(from + s * kPartial));
                t.y[(uint64_t)column * t.n + (segment_begin - first_tile + local * split + rank) * 16u + row] = eb::float_to_bf16_bits(finish.apply(sum));
            }
        }
        eb::cluster_sync();   // the gather buffers are free for the next tensor
    };

    // Adds the T piece sums of a tile in piece order and rounds to BF16 (one slice) or hands the slice sum to the tile's
    // owner rank. The tile's 16 x rows outputs are dealt to the calling threads: `e` from `begin` in steps of `step`.
    auto add_pieces = [&](const Tensor& t, const typename F::Finish& finish, uint32_t pieces, uint32_t row0, uint32_t local, uint32_t begin, uint32_t step) {
        for (uint32_t e = begin; e < 16u * rows; e += step) {
            const uint32_t column = e >> 4, row = e & 15u, at = (row * 8u + column) * 4u;
            float sum = ld_shared_f(pieces + at);
            for (uint32_t j = 1; j < team_size; ++j) sum = __fadd_rn(sum, ld_shared_f(pieces + j * kPartial + at));
            if (split == 1u) {
                t.y[(uint64_t)column * t.n + row0 + row] = eb::float_to_bf16_bits(finish.apply(sum));
            } else {
                // Tile i of the segment is summed by rank i % S: its gather buffer is [i / S][source rank][row][column].
                const uint32_t owner = local % split;
                eb::st_cluster_f32(eb::map_to_rank(smem_a + layout.off_gather, owner) + ((local / split) * split + rank) * kPartial + at, sum);
            }
        }
    };

    if (kAdder && warp == warps) {
        // ---- the adding warp: the T piece sums of a tile in piece order, then BF16 (one slice) or the tile's owner rank ----
        eb::pdl_launch_dependents();
        eb::pdl_wait();
        if (split > 1u) eb::cluster_wait();
        uint32_t first_tile = 0;
        for (uint32_t ti = 0; ti < group.count; ++ti) {
            const Tensor& t = group.tensor[ti];
            const uint32_t segment_begin = max(run_begin, first_tile), segment_end = min(run_end, t.tile_end);
            if (segment_begin < segment_end) {
                stage(t);
                const typename F::Finish finish(t.w, typename F::Geometry(t.n, group.k));
                for (uint32_t tile = segment_begin; tile < segment_end; ++tile) {
                    // Tile run_begin + i belongs to team i % teams and is that team's tile number i / teams.
                    const uint32_t index = tile - run_begin, team = index % teams, turn = index / teams, buffer = turn & 1u;
                    const uint32_t bars = sums_a + (team * 2u + buffer) * 16u;
                    if (complete) complete = eb::mbar_wait_at<400>(bars, (turn >> 1) & 1u);   // a team needs microseconds per tile: poll rarely
                    const uint32_t pieces = smem_a + layout.off_partials + (team * 2u + buffer) * team_size * kPartial;
                    add_pieces(t, finish, pieces, (tile - first_tile) * 16u, tile - segment_begin, lane, 32u);
                    __syncwarp();
                    if (lane == 0) eb::mbar_arrive(reinterpret_cast<uint64_t*>(smem + layout.off_sum_bars) + (team * 2u + buffer) * 2u + 1u);
                }
                if (split > 1u) join_slices(t, first_tile, segment_begin, segment_end);
            }
            first_tile = t.tile_end;
        }
        if (!complete && lane == 0) atomicOr(error, F::kErrorBit);
        return;
    }

    // ---- a decoding warp: member j of its team owns piece j of the slice for every tile the team takes ----
    const uint32_t team = warp / team_size, member = warp % team_size;
    const uint32_t piece_begin = slice_begin + member * slice / team_size, piece_end = slice_begin + (member + 1u) * slice / team_size;
    const bool wide = piece_end - piece_begin == (uint32_t)P;
    const uint32_t slots_a = smem_a + layout.off_slots + warp * depth * layout.slot_bytes;
    const uint32_t bars_a = smem_a + layout.off_bars + warp * depth * 8u;
    // Where a piece's bytes sit in the planes: the code box starts at the piece; the scale box starts on the 16-byte
    // boundary at or before the piece's scales.
    const uint32_t code_x = piece_begin * (F::kCodeBytes / 4u);
    const uint32_t scale_byte = piece_begin * F::kScaleBytes, scale_x = scale_byte & ~15u;
    const uint32_t scale_rem = kTmaScales ? scale_byte - scale_x : 0u;
    const uint32_t fill_bytes = 16u * (uint32_t)P * F::kCodeBytes + (kTmaScales ? 16u * F::kScaleBox : 0u);

    // The team's tiles: run_begin + team, + teams, ... Two cursors walk them: `ask` requests, `use` decodes.
    uint32_t ask_tile = run_begin + team, ask_slot = 0, ask_tensor = 0, ask_first = 0, ask_end = group.tensor[0].tile_end;
    auto request = [&]() {
        if (ask_tile < run_end) {
            while (ask_tile >= ask_end) {   // the next tensor of the group
                ask_first = ask_end;
                ask_end = group.tensor[++ask_tensor].tile_end;
            }
            const Tensor& t = group.tensor[ask_tensor];
            const uint32_t row = (ask_tile - ask_first) * 16u;
            const uint32_t to = slots_a + ask_slot * layout.slot_bytes, bar = bars_a + ask_slot * 8u;
            if (lane == 0) {
                eb::tma_load_2d_expect(to, &t.codes, (int)code_x, (int)row, bar, fill_bytes);
                if (kTmaScales) eb::tma_load_2d_at(to + layout.code_bytes, &t.scales, (int)scale_x, (int)row, bar);
            }
            if (!kTmaScales) {
                // lane l copies row l % 16, every other chunk's scales
                const typename F::Geometry geo(t.n, group.k);
                const uint8_t* from = t.w + geo.scale_offset + (uint64_t)(row + (lane & 15u)) * geo.scale_row_bytes + (uint64_t)piece_begin * F::kScaleBytes;
                const uint32_t into = to + layout.code_bytes + (lane & 15u) * F::kScaleBox;
                for (uint32_t c = lane >> 4; c < piece_end - piece_begin; c += 2u) {
                    if (F::kScaleBytes == 8u) eb::cp_async_8_to(into + c * 8u, from + c * 8u);
                    else eb::cp_async_4_to(into + c * 4u, from + c * 4u);
                }
            }
            ask_tile += teams;
            if (++ask_slot == depth) ask_slot = 0;
        }
        if (!kTmaScales) eb::cp_async_commit();
    };
    for (uint32_t s = 0; s < depth; ++s) request();

    // The activations may come from the kernel before this one.
    eb::pdl_launch_dependents();
    eb::pdl_wait();
    if (split > 1u) eb::cluster_wait();

    // Lane constants. Lane (g, q) decodes rows g and g + 8 of a tile; its activations are those of row min(g, rows - 1).
    const uint32_t x_lane = eb::pinned(smem_a + (g < rows ? g : rows - 1u) * layout.stride_x + q * 16u + (piece_begin - slice_begin) * 256u);
    const uint32_t code_lane = eb::pinned(g * (uint32_t)P * F::kCodeBytes);
    const uint32_t scale_lane = eb::pinned(layout.code_bytes + g * F::kScaleBox + scale_rem + F::lane_scale_offset(q));
    const uint32_t extra_lane = smem_a + layout.off_extra + (piece_begin - slice_begin) * (F::extra_bytes(2) - F::extra_bytes(1));
    // This lane's place in its team's two sum buffers: [buffer][member][row of the tile][activation row]; lane (g, q) holds
    // rows g, g + 8 for columns 2q, 2q + 1.
    const uint32_t sum_lane = smem_a + layout.off_partials + (team * 2u * team_size + member) * kPartial + (g * 8u + 2u * q) * 4u;
    const uint32_t sum_bars = sums_a + team * 32u;
    typename F::template State<P> state(extra_lane, q);

    uint32_t use_tile = run_begin + team, use_slot = 0, parity = 0, turn = 0, first_tile = 0;
    for (uint32_t ti = 0; ti < group.count; ++ti) {
        const Tensor& t = group.tensor[ti];
        const uint32_t segment_begin = max(run_begin, first_tile), segment_end = min(run_end, t.tile_end);
        if (segment_begin < segment_end) {   // uniform over the cluster
            stage(t);
            const typename F::Finish finish(t.w, typename F::Geometry(t.n, group.k));
            state.tensor(t.w, typename F::Geometry(t.n, group.k));   // what the decode keeps per tensor (a scale table, if the format has one)
            for (; use_tile < segment_end; use_tile += teams, ++turn) {
                if (!kTmaScales) {
                    if (depth == 2u) eb::cp_async_wait_group<1>();
                    else eb::cp_async_wait_group<2>();
                    __syncwarp();
                }
                if (complete) complete = eb::mbar_wait_at(bars_a + use_slot * 8u, parity);   // after one wait gave up, no further wait is taken
                const uint32_t slot = slots_a + use_slot * layout.slot_bytes;
                float acc[4];
                if (P == 1 || wide) decode_piece<F, P, P>(state, slot + code_lane, slot + scale_lane, x_lane, acc);
                else decode_piece<F, P, (P > 1 ? P - 1 : 1)>(state, slot + code_lane, slot + scale_lane, x_lane, acc);
                const uint32_t buffer = turn & 1u;
                // With an adding warp: the sum buffer of this turn was read two turns ago (the first two turns find it free).
                if (kAdder && complete) complete = eb::mbar_wait_at(sum_bars + buffer * 16u + 8u, ((turn >> 1) & 1u) ^ 1u);
                const uint32_t mine = sum_lane + buffer * team_size * kPartial;
                st_shared_f2(mine, acc[0], acc[1]);
                st_shared_f2(mine + 256u, acc[2], acc[3]);
                __syncwarp();   // every lane is done with the slot and has written its sums
                if (kAdder && lane == 0) eb::mbar_arrive_at(sum_bars + buffer * 16u);
                request();
                if (++use_slot == depth) {
                    use_slot = 0;
                    parity ^= 1u;
                }
                if (!kAdder) {
                    // The team meets on its named barrier; its threads share the tile's outputs. Two buffers: a warp that runs
                    // ahead writes the other one, and passes the next barrier only after every teammate has finished here.
                    if (team_size > 1u) team_sync(team, team_size * 32u);
                    add_pieces(t, finish, smem_a + layout.off_partials + (team * 2u + buffer) * team_size * kPartial, (use_tile - first_tile) * 16u,
                            use_tile - segment_begin, tid - team * team_size * 32u, team_size * 32u);
                }
            }
            if (split > 1u) join_slices(t, first_tile, segment_begin, segment_end);
        }
        first_tile = t.tile_end;
    }
    if (!kTmaScales) eb::cp_async_wait_all();
    if (!complete && lane == 0) atomicOr(error, F::kErrorBit);
}

}  // namespace gemv
