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
// How it runs here: one CTA per tile at a time (persistent over the tile list), 512 threads. The two cost rows live in
// shared memory as FP16; a thread takes pairs of neighbouring nodes (they share their predecessors) and evaluates both
// with packed FP16 arithmetic, recomputing the codebook value of a state from its hash instead of keeping tables. The
// history - one byte per position and node: which of the 2^d states won - goes to a scratch slab of the CTA in global
// memory (up to 4 MB per pass) and is read back by one thread for the trace. No waits on other CTAs.
#pragma once

#include "common.cuh"
#include "trellis_codebook.cuh"

namespace trellis_encode {

constexpr int kThreads = 512;
constexpr uint32_t kInfinity = 0x7C00u;

__host__ __device__ constexpr int position_bits(int position, int ka, bool half_step) { return ka + ((half_step && (position & 1)) ? 1 : 0); }

// Bytes of history one CTA needs: 256 positions x the most nodes of a position.
__host__ __device__ constexpr uint64_t history_bytes(int ka) { return 256ull * (65536ull >> ka); }

__device__ __forceinline__ uint32_t reverse5(uint32_t v) { return __brev(v) >> 27; }

// One step of a pass at ring position `ri`: costs of the nodes after the position from the costs before it.
template <int KIN, int KOUT>
__device__ __forceinline__ void step(const __half* __restrict__ before, __half* __restrict__ after, uint8_t* __restrict__ history_row, __half w,
        bool first, int pinned, bool write) {
    constexpr int kShift = 16 - KOUT, kNodes = 65536 >> KOUT, kStates = 1 << KOUT;
    const __half2 w2 = __half2half2(w), infinity = __half2half2(__ushort_as_half((unsigned short)kInfinity));
    for (int pair = threadIdx.x; pair < kNodes / 2; pair += kThreads) {
        const int node = 2 * pair, from_low = node >> KIN;   // both nodes of the pair have the same predecessors
        __half2 best = infinity;
        uint32_t winner0 = 0, winner1 = 0;
#pragma unroll
        for (int s = 0; s < kStates; ++s) {
            const uint32_t state = ((uint32_t)s << kShift) | (uint32_t)node;
            const int from = (s << (kShift - KIN)) | from_low;
            const uint32_t values = trellis::value_pair(state, state + 1u);
            const __half2 e = __hsub2(*reinterpret_cast<const __half2*>(&values), w2);
            __half2 cost;
            if (first) {
                cost = pinned >= 0 && from != pinned ? infinity : __hmul2(e, e);
            } else {
                cost = __hfma2(e, e, __half2half2(before[from]));
            }
            if (s == 0 || __hlt(__low2half(cost), __low2half(best))) {
                best = __halves2half2(__low2half(cost), __high2half(best));
                winner0 = (uint32_t)s;
            }
            if (s == 0 || __hlt(__high2half(cost), __high2half(best))) {
                best = __halves2half2(__low2half(best), __high2half(cost));
                winner1 = (uint32_t)s;
            }
        }
        reinterpret_cast<__half2*>(after)[pair] = best;
        if (write) reinterpret_cast<uint16_t*>(history_row)[pair] = (uint16_t)(winner0 | winner1 << 8);
    }
}

// tiles f32 [count][256] -> states u16 [count][256] (and, when asked for, their codebook values as f32). history:
// history_bytes(KA) bytes per CTA.
//   grid: any (CTAs take tiles blockIdx.x, + gridDim.x, ...), block kThreads, dynamic shared 4 * (65536 >> KA) + 512 bytes.
template <int KA, bool kHalfStep>
__global__ void __launch_bounds__(kThreads, 1) viterbi_kernel(const float* __restrict__ tiles, uint32_t count, uint16_t* __restrict__ states,
        float* __restrict__ decoded, uint8_t* __restrict__ history) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int kMost = 65536 >> KA;   // nodes of a position that brings KA bits
    constexpr int KB = kHalfStep ? KA + 1 : KA;
    __half* row_a = reinterpret_cast<__half*>(smem);
    __half* row_b = row_a + kMost;
    __half* weights = row_b + kMost;
    __shared__ uint32_t warp_best[kThreads / 32];
    __shared__ int node_shared;
    uint8_t* slab = history + (uint64_t)blockIdx.x * history_bytes(KA);
    const int tid = threadIdx.x;

    for (uint32_t tile = blockIdx.x; tile < count; tile += gridDim.x) {
        __syncthreads();   // the tile before is done with the shared rows
        if (tid < 256) weights[tid] = __float2half_rn(tiles[(uint64_t)tile * 256u + (uint32_t)tid]);
        __syncthreads();
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
                // a position brings KA bits, or KA + 1 at odd positions of a half-step rate; the next one likewise
                if (!kHalfStep || (ri & 1) == 0) {
                    if (!kHalfStep) step<KA, KA>(before, after, row, weights[ri], i == 0, pinned, write);
                    else step<KA, KB>(before, after, row, weights[ri], i == 0, pinned, write);
                } else {
                    step<KB, KA>(before, after, row, weights[ri], i == 0, pinned, write);
                }
                __syncthreads();
            }
            if (pass == 0) {
                // the best node after position 127 (the open pass's last), ties by the rank of the node
                constexpr int kLast = 65536 >> KA;   // position 128 is even: KA bits
                uint32_t best = (kInfinity << 16) | 0xFFFFu;
                for (int e = tid; e < kLast; e += kThreads) {
                    const uint32_t v = (uint32_t)e & 1023u;
                    const uint32_t rank = (reverse5(v >> 5) << 10) | (reverse5(v & 31u) << 5) | ((uint32_t)e >> 10);
                    best = min(best, ((uint32_t)__half_as_ushort(after[e]) << 16) | rank);
                }
                best = __reduce_min_sync(0xFFFFFFFFu, best);
                if ((tid & 31) == 0) warp_best[tid >> 5] = best;
                __syncthreads();
                if (tid == 0) {
                    for (int i = 1; i < kThreads / 32; ++i) best = min(best, warp_best[i]);
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
                    node_shared = node;
                }
                __syncthreads();
                pinned = node_shared;
            } else if (tid == 0) {
                __threadfence_block();
                int node = pinned;
                for (int ri = 255; ri >= 0; --ri) {
                    const int kin = position_bits(ri, KA, kHalfStep), kout = position_bits(ri + 1, KA, kHalfStep);
                    const int s = slab[(uint64_t)ri * kMost + (uint32_t)node];
                    const int from = (s << (16 - kout - kin)) | (node >> kin);
                    const uint32_t state = (((uint32_t)from << kin) | (uint32_t)node) & 0xFFFFu;
                    states[(uint64_t)tile * 256u + (uint32_t)ri] = (uint16_t)state;
                    if (decoded != nullptr) decoded[(uint64_t)tile * 256u + (uint32_t)ri] = __half2float(__ushort_as_half(trellis::value_bits(state)));
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
