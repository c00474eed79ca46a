// Trellis tile encoder on sm_100a: quantizes 256-weight tiles to the tail-biting ring of 16-bit states that
// trellis.cuh decodes (the converter's side of the trellis-tile16-v1 format; the reference's encoder is
// quantization/src/main/resources/cuda/trellis.cu:34-399, from exllamav3's Viterbi kernels).
//
// The search is fixed by the format's golden tiles, so its arithmetic is the contract: position i brings
// d(i) = ka + [i odd][half-step rate] new bits; a node is the top 16 - d bits of a state; the cost of reaching node v at
// a position is the least, over the 2^d states that end in v, of fp16 fma(e, e, cost of the state's predecessor node)
// with e = fp16(value(state) - w) (first position: fp16(e * e)), the lowest predecessor on equal costs. Two passes: from
// an open start at position 128 all round, the best end node (ties by a bit-reversed rank of the node) traced back to
// the node that enters position 0; then from position 0 pinned to that node, traced back in full.
//
// How it runs here: one CTA per SM, 1024 threads, persistent over the tile list. The CTA first writes the codebook value of
// every one of the 65,536 states to shared memory (128 KB of FP16) - a state's neighbours sit side by side there. The
// threads then work as two groups of 512 that encode tiles independently of each other (a named barrier per group; at
// 2 and 2.5 bits the cost rows are too large for two groups and one group of 1024 runs): a group keeps its two cost rows
// in shared memory as FP16; a thread takes runs of 2, 4 or 8 neighbouring nodes, which share their predecessors, reads
// their values with one load per predecessor and updates their costs with packed FP16 arithmetic and bit selects. The
// history - one byte per position and node: which of the 2^d states won - goes to a slab of the group in global memory
// (up to 4 MB per pass) and one thread of the group walks it back; while it does, the other group has the SM's issue
// slots. No waits on other CTAs.
#pragma once

#include "common.cuh"
#include "trellis_codebook.cuh"

namespace trellis_encode {

constexpr int kThreads = 1024;
constexpr uint32_t kInfinity = 0x7C00u;
constexpr uint32_t kTableBytes = 65536u * 2u;

__host__ __device__ constexpr int position_bits(int position, int ka, bool half_step) { return ka + ((half_step && (position & 1)) ? 1 : 0); }

// Bytes of history one group needs: 256 positions x the most nodes of a position.
__host__ __device__ constexpr uint64_t history_bytes(int ka) { return 256ull * (65536ull >> ka); }

// Groups of a CTA that encode side by side: two where their cost rows fit beside the value table.
__host__ __device__ constexpr int groups_of(int ka) { return ka >= 3 ? 2 : 1; }

// Dynamic shared memory of a CTA: the value table, then per group two cost rows and the tile's 256 weights.
__host__ __device__ constexpr uint32_t shared_bytes(int ka) { return kTableBytes + (uint32_t)groups_of(ka) * (4u * (65536u >> ka) + 512u); }

__device__ __forceinline__ uint32_t reverse5(uint32_t v) { return __brev(v) >> 27; }

template <int GROUP_THREADS>
__device__ __forceinline__ void group_sync(int group) {
    if (GROUP_THREADS == kThreads) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(GROUP_THREADS) : "memory");
}

// Nodes a thread takes at a time: they must share their predecessors (2^KIN neighbours do) and there should be at least
// as many runs as threads.
template <int KIN, int KOUT, int GROUP_THREADS>
struct Run {
    static constexpr int kNodes = 65536 >> KOUT;
    static constexpr int kShared = 1 << KIN;
    static constexpr int kWanted = kNodes / GROUP_THREADS >= 8 ? 8 : kNodes / GROUP_THREADS >= 4 ? 4 : 2;
    static constexpr int value = kWanted < kShared ? kWanted : (kShared < 8 ? kShared : 8);
};

// One step of a pass: costs of the nodes after a position from the costs before it. `table`: FP16 value of every state.
template <int KIN, int KOUT, int GROUP_THREADS, bool kFirst>
__device__ __forceinline__ void step(const __half* __restrict__ table, const __half* __restrict__ before, __half* __restrict__ after,
        uint8_t* __restrict__ history_row, __half w, int pinned, bool write, int tid) {
    constexpr int kShift = 16 - KOUT, kNodes = 65536 >> KOUT, kStates = 1 << KOUT;
    constexpr int G = Run<KIN, KOUT, GROUP_THREADS>::value, H = G / 2;
    const __half2 w2 = __half2half2(w);
    const uint32_t infinity = kInfinity | kInfinity << 16;
    for (int run = tid; run < kNodes / G; run += GROUP_THREADS) {
        const int node = run * G, from_low = node >> KIN;   // the G nodes of the run have the same predecessors
        uint32_t best[H], winner[H];
#pragma unroll
        for (int s = 0; s < kStates; ++s) {
            const uint32_t state = ((uint32_t)s << kShift) | (uint32_t)node;
            const int from = (s << (kShift - KIN)) | from_low;
            uint32_t values[H];
            if constexpr (G == 8) {
                const uint4 v = *reinterpret_cast<const uint4*>(table + state);
                values[0] = v.x, values[1] = v.y, values[2] = v.z, values[3] = v.w;
            } else if constexpr (G == 4) {
                const uint2 v = *reinterpret_cast<const uint2*>(table + state);
                values[0] = v.x, values[1] = v.y;
            } else {
                values[0] = *reinterpret_cast<const uint32_t*>(table + state);
            }
            __half2 previous;
            if (!kFirst) previous = __half2half2(before[from]);
#pragma unroll
            for (int j = 0; j < H; ++j) {
                const __half2 e = __hsub2(*reinterpret_cast<const __half2*>(&values[j]), w2);
                uint32_t cost;
                if (kFirst) {
                    const __half2 square = __hmul2(e, e);
                    cost = pinned >= 0 && from != pinned ? infinity : *reinterpret_cast<const uint32_t*>(&square);
                } else {
                    const __half2 sum = __hfma2(e, e, previous);
                    cost = *reinterpret_cast<const uint32_t*>(&sum);
                }
                if (s == 0) {
                    best[j] = cost;
                    winner[j] = 0;
                } else {
                    // strictly less, half by half: the lowest state keeps a tie
                    const uint32_t less = __hlt2_mask(*reinterpret_cast<const __half2*>(&cost), *reinterpret_cast<const __half2*>(&best[j]));
                    best[j] = (cost & less) | (best[j] & ~less);
                    winner[j] = (((uint32_t)s * 0x00010001u) & less) | (winner[j] & ~less);
                }
            }
        }
        if constexpr (G == 8) {
            *reinterpret_cast<uint4*>(after + node) = make_uint4(best[0], best[1], best[2], best[3]);
            if (write) *reinterpret_cast<uint2*>(history_row + node) = make_uint2(__byte_perm(winner[0], winner[1], 0x6420), __byte_perm(winner[2], winner[3], 0x6420));
        } else if constexpr (G == 4) {
            *reinterpret_cast<uint2*>(after + node) = make_uint2(best[0], best[1]);
            if (write) *reinterpret_cast<uint32_t*>(history_row + node) = __byte_perm(winner[0], winner[1], 0x6420);
        } else {
            *reinterpret_cast<uint32_t*>(after + node) = best[0];
            if (write) *reinterpret_cast<uint16_t*>(history_row + node) = (uint16_t)__byte_perm(winner[0], 0, 0x4420);
        }
    }
}

// tiles f32 [count][256] -> states u16 [count][256] (and, when asked for, their codebook values as f32). history:
// history_bytes(KA) bytes per CTA and group.
//   grid: any (group g of CTA b takes tiles b G + g, + gridDim.x G, ...), block kThreads, dynamic shared shared_bytes(KA).
template <int KA, bool kHalfStep>
__global__ void __launch_bounds__(kThreads, 1) viterbi_kernel(const float* __restrict__ tiles, uint32_t count, uint16_t* __restrict__ states,
        float* __restrict__ decoded, uint8_t* __restrict__ history) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int kMost = 65536 >> KA;   // nodes of a position that brings KA bits
    constexpr int KB = kHalfStep ? KA + 1 : KA;
    constexpr int kGroups = groups_of(KA), T = kThreads / kGroups;
    __shared__ uint32_t warp_best[kGroups][T / 32];
    __shared__ int node_shared[kGroups];
    const int group = kGroups == 1 ? 0 : threadIdx.x / T, tid = threadIdx.x - group * T;
    __half* table = reinterpret_cast<__half*>(smem);
    __half* row_a = reinterpret_cast<__half*>(smem + kTableBytes + (uint32_t)group * (4u * kMost + 512u));
    __half* row_b = row_a + kMost;
    __half* weights = row_b + kMost;
    uint8_t* slab = history + ((uint64_t)blockIdx.x * kGroups + (uint32_t)group) * history_bytes(KA);

    for (uint32_t state = threadIdx.x; state < 65536u; state += kThreads) table[state] = __ushort_as_half(trellis::value_bits(state));
    __syncthreads();

    for (uint32_t tile = blockIdx.x * kGroups + group; tile < count; tile += gridDim.x * kGroups) {
        group_sync<T>(group);   // the tile before is done with the group's rows
        if (tid < 256) weights[tid] = __float2half_rn(tiles[(uint64_t)tile * 256u + (uint32_t)tid]);
        group_sync<T>(group);
        __half *before = row_a, *after = row_b;
        int pinned = -1;
        for (int pass = 0; pass < 2; ++pass) {
            const int roll = pass == 0 ? 128 : 0;
            for (int i = 0; i < 256; ++i) {
                const int ri = (i + roll) & 255;
                __half* swap = before;
                before = after;
                after = swap;
                const bool write = pass == 1 || ri < 128;
                uint8_t* row = slab + (uint64_t)ri * kMost;
                const __half w = weights[ri];
                // a position brings KA bits, or KA + 1 at odd positions of a half-step rate; the next one likewise
                if (i == 0) {
                    if (!kHalfStep) step<KA, KA, T, true>(table, before, after, row, w, pinned, write, tid);
                    else step<KA, KB, T, true>(table, before, after, row, w, pinned, write, tid);   // both passes start at an even position
                } else if (!kHalfStep) {
                    step<KA, KA, T, false>(table, before, after, row, w, pinned, write, tid);
                } else if ((ri & 1) == 0) {
                    step<KA, KB, T, false>(table, before, after, row, w, pinned, write, tid);
                } else {
                    step<KB, KA, T, false>(table, before, after, row, w, pinned, write, tid);
                }
                group_sync<T>(group);
            }
            if (pass == 0) {
                // the best node after position 127 (the open pass's last), ties by the rank of the node
                constexpr int kLast = 65536 >> KA;   // position 128 is even: KA bits
                uint32_t best = (kInfinity << 16) | 0xFFFFu;
                for (int e = tid; e < kLast; e += T) {
                    const uint32_t v = (uint32_t)e & 1023u;
                    const uint32_t rank = (reverse5(v >> 5) << 10) | (reverse5(v & 31u) << 5) | ((uint32_t)e >> 10);
                    best = min(best, ((uint32_t)__half_as_ushort(after[e]) << 16) | rank);
                }
                best = __reduce_min_sync(0xFFFFFFFFu, best);
                if ((tid & 31) == 0) warp_best[group][tid >> 5] = best;
                group_sync<T>(group);
                if (tid == 0) {
                    for (int i = 1; i < T / 32; ++i) best = min(best, warp_best[group][i]);
                    int node = 0;
                    if (best < (kInfinity << 16)) {
                        const uint32_t rank = best & 65535u;
                        node = (int)(((rank & 31u) << 10) | (reverse5(rank >> 10) << 5) | reverse5((rank >> 5) & 31u));
                    }
                    // back through positions 127 .. 0 to the node that enters position 0
                    for (int ri = 127; ri >= 0; --ri) {
                        const int kin = position_bits(ri, KA, kHalfStep), kout = position_bits(ri + 1, KA, kHalfStep);
                        const int s = slab[(uint64_t)ri * kMost + (uint32_t)node];
                        node = (s << (16 - kout - kin)) | (node >> kin);
                    }
                    node_shared[group] = node;
                }
                group_sync<T>(group);
                pinned = node_shared[group];
            } else if (tid == 0) {
                int node = pinned;
                for (int ri = 255; ri >= 0; --ri) {
                    const int kin = position_bits(ri, KA, kHalfStep), kout = position_bits(ri + 1, KA, kHalfStep);
                    const int s = slab[(uint64_t)ri * kMost + (uint32_t)node];
                    const int from = (s << (16 - kout - kin)) | (node >> kin);
                    const uint32_t state = (((uint32_t)from << kin) | (uint32_t)node) & 0xFFFFu;
                    states[(uint64_t)tile * 256u + (uint32_t)ri] = (uint16_t)state;
                    if (decoded != nullptr) decoded[(uint64_t)tile * 256u + (uint32_t)ri] = __half2float(table[state]);
                    node = from;
                }
            }
        }
    }
}

// states u16 [count][256] -> payload words [count][w] (16-bit words; w = 16 ka + 8 at a half-step rate): the low d(i) bits of
// state i, most significant bit first, in 32-bit little-endian words - the ring trellis.cuh reads. A thread per 32-bit word.
__global__ void __launch_bounds__(256) pack_kernel(const uint16_t* __restrict__ states, uint32_t count, int ka, int half_step,
        uint32_t* __restrict__ words) {
    const uint32_t per_tile = (uint32_t)(8 * ka + (half_step ? 4 : 0));   // 32-bit words of a tile
    const uint64_t index = (uint64_t)blockIdx.x * 256u + threadIdx.x;
    if (index >= (uint64_t)count * per_tile) return;
    const uint32_t tile = (uint32_t)(index / per_tile), word = (uint32_t)(index % per_tile);
    const int first_bit = (int)word * 32;
    // position i starts at bit i ka + i / 2 (half-step: one more bit before every odd position's successor)
    uint32_t value = 0;
    for (int i = 0; i < 256; ++i) {
        const int start = i * ka + (half_step ? i / 2 : 0), bits = position_bits(i, ka, half_step != 0);
        if (start + bits <= first_bit) continue;
        if (start >= first_bit + 32) break;
        const uint32_t field = (uint32_t)states[(uint64_t)tile * 256u + (uint32_t)i] & ((1u << bits) - 1u);
        // the field occupies stream bits [start, start + bits); stream bit b of this word is word bit 31 - (b - first_bit)
        const int shift = first_bit + 32 - (start + bits);
        value |= shift >= 0 ? field << shift : field >> -shift;
    }
    words[index] = value;
}

}  // namespace trellis_encode
