// Device-side building blocks shared by the sm_100a kernels: BF16 rounding, mbarriers, bulk asynchronous copies,
// programmatic dependent launch, thread-block clusters and warp-level BF16 MMA.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace eb {

// Every wait in these kernels gives up after this many polls (each poll itself blocks for a bounded time), raises the
// kernel's error word and lets the CTA run to its end, so a wedged copy can never hang the device.
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// BF16 round-to-nearest-even by integer arithmetic: the reference's output rounding (native/src/q3/numeric.cuh:17-21).
__device__ __forceinline__ uint16_t float_to_bf16_bits(float value) {
    uint32_t bits = __float_as_uint(value);
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}
__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits) { return __uint_as_float(bits << 16); }

// ---- programmatic dependent launch -----------------------------------------------------------------------------
// No-ops unless the launch carries the programmatic-stream-serialization attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- mbarrier -------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_at(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
    return done != 0;
}
// One poll that lets the hardware park the thread until the phase completes or about `kParkNs` have passed, so that a
// warp waiting for its copy does not spend issue slots on polling.
constexpr uint32_t kParkNs = 20000;
constexpr uint32_t kParkLimit = 1u << 15;   // polls before a parked wait gives up (well under a second)
__device__ __forceinline__ bool mbar_try_wait_at(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
            "selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(bar), "r"(parity), "r"(kParkNs)
            : "memory");
    return done != 0;
}
// Bounded wait on a barrier given by its 32-bit shared address. A poll that fails is followed by a sleep of kNap
// nanoseconds: the hardware returns from a parked poll long before its time hint, and a warp that polls back to back
// takes issue slots from the warps whose work it is waiting for.
template <uint32_t kNap = 64>
__device__ __forceinline__ bool mbar_wait_at(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kParkLimit; ++spin) {
        if (mbar_try_wait_at(bar, parity)) return true;
        asm volatile("nanosleep.u32 %0;" ::"n"(kNap));
    }
    return false;
}
// Bounded wait: false when the phase did not complete within kSpinLimit polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// ---- bulk asynchronous copy global -> shared (TMA engine, no tensor map) ----------------------------------------
// Source, destination and size are multiples of 16 bytes. Completion is signalled on `bar` (complete_tx).
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
            "l"(src), "r"(bytes), "r"(smem_u32(bar))
            : "memory");
}

// ---- tiled asynchronous copy global -> shared through a tensor map (TMA) -----------------------------------------
// c0 is the innermost coordinate: c0 times the element size must be a multiple of 16 bytes. The whole box is written
// (out-of-range elements as zeros) and signalled on `bar`.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                         smem_u32(dst)),
            "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
            : "memory");
}

// The same with destination and barrier given as 32-bit shared addresses, preceded by the barrier's expect_tx.
__device__ __forceinline__ void tma_load_2d_expect(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
            "l"(map), "r"(c0), "r"(c1), "r"(bar)
            : "memory");
}

__device__ __forceinline__ void tma_load_2d_at(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
            "l"(map), "r"(c0), "r"(c1), "r"(bar)
            : "memory");
}

// ---- cp.async (LDGSTS) for pieces too small or too misaligned for a bulk copy ------------------------------------
__device__ __forceinline__ void cp_async_4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_8(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's most recent groups are still in flight.
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// cp.async with the destination given as a 32-bit shared address.
__device__ __forceinline__ void cp_async_4_to(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_8_to(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}

// ---- shared-memory loads by 32-bit shared address plus a compile-time byte offset (folded into the instruction) -------
template <int OFFSET>
__device__ __forceinline__ uint32_t lds_u32(uint32_t address) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(address), "n"(OFFSET));
    return v;
}
template <int OFFSET>
__device__ __forceinline__ uint32_t lds_u16(uint32_t address) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(address), "n"(OFFSET));
    return v;
}
template <int OFFSET>
__device__ __forceinline__ uint4 lds_v4(uint32_t address) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address), "n"(OFFSET));
    return v;
}
template <int OFFSET>
__device__ __forceinline__ float4 lds_f4(uint32_t address) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(address), "n"(OFFSET));
    return v;
}
template <int OFFSET>
__device__ __forceinline__ float2 lds_f2(uint32_t address) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2+%3];" : "=f"(v.x), "=f"(v.y) : "r"(address), "n"(OFFSET));
    return v;
}

// ---- thread-block clusters ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync() {
    cluster_arrive();
    cluster_wait();
}
// Address of `local` (a shared-memory address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
// Global loads of weight bytes. Streamed bytes are read once and bypass L1; small pieces that neighbouring chunks share
// (scales, overlapping code words) keep the default L1 policy.
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_u16(const void* p) {
    uint16_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ void st_cluster_f32(uint32_t address, float value) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(address), "f"(value) : "memory");
}

// ---- warp-level tensor-core MMA ---------------------------------------------------------------------------------
// D[16x8] += A[16x16] * B[16x8], BF16 operands, FP32 accumulation. Fragment ownership for lane (g = lane / 4, q = lane % 4):
//   a0: row g, k 2q..2q+1   a1: row g+8, k 2q..2q+1   a2: row g, k 2q+8..2q+9   a3: row g+8, k 2q+8..2q+9
//   b0: k 2q..2q+1, col g   b1: k 2q+8..2q+9, col g
//   d0, d1: row g, cols 2q, 2q+1   d2, d3: row g+8, cols 2q, 2q+1
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
        uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D = A * B + C with C in registers of its own (a group's starting value that must survive, or a constant).
__device__ __forceinline__ void mma_bf16_16816_from(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
        uint32_t b1, const float4& c) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c.x), "f"(c.y), "f"(c.z), "f"(c.w));
}
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
        uint32_t b1) {
    asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D[16x8] = A[16x32] * B[32x8] + C, unsigned bytes in, 32-bit integers out. Lane (g = lane / 4, q = lane % 4) owns
//   a0: row g, k 4q..4q+3   a1: row g+8, k 4q..4q+3   a2: row g, k 16+4q..   a3: row g+8, k 16+4q..
//   b0: k 4q..4q+3, col g   b1: k 16+4q.., col g        d0, d1: row g, cols 2q, 2q+1   d2, d3: row g+8, cols 2q, 2q+1
__device__ __forceinline__ void mma_u8_16832_from(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
        uint32_t b1, uint32_t c) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}

// One LOP3: the bitwise function of (a, b, c) whose truth table is LUT (bit i of LUT = f for a, b, c = bits 2, 1, 0 of i).
// Spelled out because the optimiser does not always merge a mask and a combine into one instruction.
template <int LUT>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(d) : "r"(a), "r"(b), "r"(c), "n"(LUT));
    return d;
}
// A value the compiler must treat as unknown and keep in a register: lane constants (addresses, shift counts, masks)
// that it would otherwise recompute from the thread index inside the inner loop to save a register.
__device__ __forceinline__ uint32_t pinned(uint32_t v) {
    asm volatile("mov.b32 %0, %0;" : "+r"(v));
    return v;
}
// The same with the third operand as an immediate (the instruction takes one).
template <int LUT, uint32_t C>
__device__ __forceinline__ uint32_t lop3_imm(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(d) : "r"(a), "r"(b), "n"(C), "n"(LUT));
    return d;
}
// f(integral_constant<int, 0>), .., f(integral_constant<int, N - 1>): a loop whose index is a compile-time constant in
// every turn (shared-memory offsets become immediates).
template <int N, int I = 0, class Body>
__device__ __forceinline__ void static_for(Body&& body) {
    if constexpr (I < N) {
        body(std::integral_constant<int, I>{});
        static_for<N, I + 1>(body);
    }
}
constexpr int kLutAndXor = 0x6A;     // (a & b) ^ c
constexpr int kLutAndOr = 0xEA;      // (a & b) | c
constexpr int kLutSelect = 0xE4;     // (a & c) | (b & ~c)

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// ---- host side: the driver's tensor-map encoder, looked up through the runtime (no link against libcuda) -----------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
        const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled encoder() {
    static EncodeTiled cached = [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &query) != cudaSuccess || query != cudaDriverEntryPointSuccess)
            entry = nullptr;
        return reinterpret_cast<EncodeTiled>(entry);
    }();
    return cached;
}

}  // namespace eb
