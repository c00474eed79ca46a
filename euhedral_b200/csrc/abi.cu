// Host side of libeuhedral_cuda.so: the C entry points declared in include/euhedral_cuda.h, their argument
// validation and routing (as native/src/host/{nvfp4_linear,q3_linear_bf16,linear_kernels,kernel_table,reference}.c of
// the reference do it), and the launches of the sm_100a kernels. No entry point allocates device memory or
// synchronizes when a stream is selected, so every call can be recorded into a CUDA graph.
#include "../../include/euhedral_cuda.h"

#include <atomic>
#include <cstring>
#include <algorithm>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "exact_kernels.cuh"
#include "nvfp4_gemv.cuh"
#include "nvfp4_native.cuh"
#include "q3_gemv.cuh"
#include "trellis.cuh"

namespace {

// ---- per-thread and per-process selections (native/src/host/euhedral_cuda.c:30-38, cuda_kernel_loader.c:259-300) ---
thread_local cudaStream_t t_stream = nullptr;
thread_local int t_pdl = 0;
thread_local int t_row_exact = 0;
std::atomic<int> g_exact{0};

__device__ uint32_t g_error_word;

// Scratch of euhedral_b200_linear_trellis_bf16_static: lives in the library's own device image, so that entry point
// needs no allocation by anybody. Every device that loads the library holds these bytes until the process exits.
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
struct DeviceState {
    std::once_flag once;
    int status = cudaSuccess;
    int sms = 0;
    int major = 0;
    uint32_t* error_word = nullptr;
    unsigned char* static_scratch = nullptr;   // device address of g_static_scratch on this device
};
DeviceState g_devices[kMaxDevices];

int finish(cudaError_t status) {
    if (status != cudaSuccess) return (int)status;
    if (t_stream != nullptr) return EUHEDRAL_CUDA_SUCCESS;
    const cudaError_t sync = cudaDeviceSynchronize();
    return sync == cudaSuccess ? EUHEDRAL_CUDA_SUCCESS : (int)sync;
}

constexpr int kBigSmem = 200 * 1024;

template <typename K>
cudaError_t allow_big_smem(K kernel) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBigSmem);
}

template <int W>
cudaError_t allow_trellis_width() {
    cudaError_t e = allow_big_smem(trellis::mma_kernel<W, 1>);
    if (e == cudaSuccess) e = allow_big_smem(trellis::mma_kernel<W, 4>);
    return e;
}

template <class F>
cudaError_t allow_gemv() {
    cudaError_t e = cudaSuccess;
#define EB_ALLOW_GEMV(RT)                                                               \
    if (e == cudaSuccess) e = allow_big_smem(gemv::kernel<F, RT, 24>);                  \
    if (e == cudaSuccess) e = allow_big_smem(gemv::kernel<F, RT, 16>);
    EB_ALLOW_GEMV(1)
    EB_ALLOW_GEMV(2)
    EB_ALLOW_GEMV(4)
    EB_ALLOW_GEMV(8)
#undef EB_ALLOW_GEMV
    return e;
}

void initialize_device(int device, DeviceState* state) {
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e == cudaSuccess) {
        state->sms = prop.multiProcessorCount;
        state->major = prop.major;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&state->error_word), g_error_word);
    }
    // In host code the array's name is only a handle; the kernels need its device address on this device.
    if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&state->static_scratch), g_static_scratch);
    if (e == cudaSuccess) e = allow_gemv<nvfp4::Format>();
    if (e == cudaSuccess) e = allow_gemv<q3::Format>();
    if (e == cudaSuccess) e = allow_big_smem(exact::trellis_linear);
#define EB_ALLOW(W) if (e == cudaSuccess) e = allow_trellis_width<W>();
    EB_TRELLIS_WIDTHS(EB_ALLOW)
#undef EB_ALLOW
    if (e == cudaSuccess) e = nvfp4n::initialize();
    state->status = (int)e;
}

// Binds the call to the thread's current device and makes sure that device's kernels are configured.
int bind(DeviceState** out) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= kMaxDevices) return EUHEDRAL_CUDA_KERNEL_UNAVAILABLE;
    DeviceState* state = &g_devices[device];
    std::call_once(state->once, initialize_device, device, state);
    if (state->status != cudaSuccess) return state->status;
    if (state->major != 10) return EUHEDRAL_CUDA_KERNEL_UNAVAILABLE;   // sm_100a code only
    *out = state;
    return EUHEDRAL_CUDA_SUCCESS;
}

// One launch on the selected stream, with the cluster dimension and the programmatic-dependent-launch attribute when asked.
template <typename... Params, typename... Args>
cudaError_t launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared, unsigned cluster, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared;
    config.stream = t_stream;
    cudaLaunchAttribute attributes[2];
    unsigned count = 0;
    if (cluster > 1) {
        attributes[count].id = cudaLaunchAttributeClusterDimension;
        attributes[count].val.clusterDim.x = cluster;
        attributes[count].val.clusterDim.y = 1;
        attributes[count].val.clusterDim.z = 1;
        ++count;
    }
    if (t_pdl) {
        attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    config.attrs = attributes;
    config.numAttrs = count;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// ---- decode GEMV planning ---------------------------------------------------------------------------------------------
// K slices per row depend on K only (gemv::split_of). A CTA has one warp per 16-row tile in flight (8, 4, 2 or 1 warps).
// If a grid of one tile per warp is resident at once (the ring shrinks to make room), that grid is launched. Otherwise
// the grid is the number of clusters the device holds at two CTAs per SM and every cluster takes an even share of the
// tiles (`span` at most), its warps several tiles each in turn.
constexpr uint32_t kSpanCap = 32;

struct DecodePlan {
    uint32_t rt, warps_per_sm, span, slots, pair, split, ctas, shared;
};

template <class F, int RT, int WARPS_PER_SM>
int query_clusters(uint32_t shared, uint32_t split) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(split * 4096u);
    config.blockDim = dim3(32u * RT);
    config.dynamicSmemBytes = shared;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = split;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemv::kernel<F, RT, WARPS_PER_SM>, &config) != cudaSuccess) {
        (void)cudaGetLastError();
        return -1;   // no answer
    }
    return clusters;   // 0: this CTA shape cannot be launched as a cluster on this device
}

// Clusters of `split` CTAs of this kernel that the current device holds at once (0: none fit); cached per (device,
// kernel, shape of the CTA).
// Without a device: three CTAs of eight warps per SM, as far as shared memory allows.
template <class F>
uint32_t resident_clusters(uint32_t rt, uint32_t warps_per_sm, uint32_t shared, uint32_t split, int sms) {
    struct Entry {
        int device;
        uint32_t error_bit, rt, warps, shared, split, clusters;
    };
    static std::mutex mutex;
    static std::vector<Entry> cache;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess) {
        (void)cudaGetLastError();
        device = -1;
    }
    if (device >= 0) {
        std::lock_guard<std::mutex> lock(mutex);
        for (const Entry& e : cache)
            if (e.device == device && e.error_bit == F::kErrorBit && e.rt == rt && e.warps == warps_per_sm && e.shared == shared && e.split == split)
                return e.clusters;
        int found = -1;
        if (warps_per_sm == 24u)
            found = rt == 8 ? query_clusters<F, 8, 24>(shared, split) : rt == 4 ? query_clusters<F, 4, 24>(shared, split)
                    : rt == 2 ? query_clusters<F, 2, 24>(shared, split) : query_clusters<F, 1, 24>(shared, split);
        else
            found = rt == 8 ? query_clusters<F, 8, 16>(shared, split) : rt == 4 ? query_clusters<F, 4, 16>(shared, split)
                    : rt == 2 ? query_clusters<F, 2, 16>(shared, split) : query_clusters<F, 1, 16>(shared, split);
        if (found >= 0) {
            cache.push_back({device, F::kErrorBit, rt, warps_per_sm, shared, split, (uint32_t)found});
            return (uint32_t)found;
        }
    }
    const uint32_t per_sm = std::min<uint32_t>(warps_per_sm / rt, (227u * 1024u) / (shared + 1024u));
    return std::max<uint32_t>(1u, (uint32_t)sms * per_sm / split);
}

template <class F>
bool plan_decode_uncached(uint32_t rows, uint32_t k, uint32_t n, int sms, DecodePlan* plan) {
    if (k == 0 || k % 128u != 0 || n == 0 || n % 16u != 0 || rows == 0 || rows > gemv::kMaxRows) return false;
    const uint32_t chunks = k / 128u, split = gemv::split_of(k);
    const uint32_t chunks_max = (chunks + split - 1u) / split;
    const uint32_t tiles = n / 16u;
    plan->split = split;
    // Ring shapes from deepest to shallowest: (slots, boxes per slot).
    const uint32_t shapes[4][2] = {{3u, 2u}, {2u, 2u}, {3u, 1u}, {2u, 1u}};
    // First choice: one tile per warp with the whole grid resident at once. Widths (warps per CTA) are tried in the order
    // of a cost estimate: the fullest SM gets ceil(CTAs / SMs) CTAs, each worth its warps plus about 1.5 warps for
    // staging its activation slice (fitted to measurements: 5120 x 5120 runs best as 320 CTAs of 4 warps, 5120 x 17408 as
    // 640 of 4, 1024 x 5120 as 128 of 2). Of equal estimates the wider goes first. The shared-memory request is raised so
    // that no SM takes more than its even share of the CTAs, rounded up: the hardware fills the SMs that free up first,
    // and without the cap some end up with twice the work of others.
    uint32_t order[4] = {8u, 4u, 2u, 1u}, cost[4];
    for (int i = 0; i < 4; ++i) {
        const uint64_t ctas = (uint64_t)((tiles + order[i] - 1u) / order[i]) * split;
        const uint64_t fullest = (ctas + (uint64_t)sms - 1u) / (uint64_t)sms;
        cost[i] = (uint32_t)std::min<uint64_t>(fullest * (2u * order[i] + 3u), 1u << 30);
    }
    for (int i = 1; i < 4; ++i)   // stable insertion sort, cheapest first
        for (int j = i; j > 0 && cost[j] < cost[j - 1]; --j) {
            std::swap(cost[j], cost[j - 1]);
            std::swap(order[j], order[j - 1]);
        }
    // A tensor with fewer than four warps of work per SM (the shards of an 8-GPU job) is bound by latency, not by any
    // SM's throughput: there the narrowest CTAs that still give two per SM - most often one warp each - spread the
    // loads over the most SMs (8 GPUs: 143 us per step against 161 us with the estimate above).
    if ((uint64_t)tiles * split < 4ull * (uint64_t)sms) {
        uint32_t narrow = 8;
        while (narrow > 1u && (uint64_t)((tiles + narrow - 1u) / narrow) * split < 2ull * (uint64_t)sms) narrow >>= 1;
        uint32_t at = 0;
        while (order[at] != narrow) ++at;
        for (; at > 0; --at) std::swap(order[at], order[at - 1]);
    }
    for (uint32_t rt : order) {
        const uint32_t groups = (tiles + rt - 1u) / rt;
        const uint32_t even_share = (groups * split + (uint32_t)sms - 1u) / (uint32_t)sms;
        const uint32_t capped = (227u * 1024u) / (even_share + 1u) + 1u;
        for (const auto& shape : shapes) {
            const uint32_t needed = gemv::Layout<F>(rt, rt, shape[0], shape[1], chunks_max, rows, split).bytes;
            const uint32_t shared = std::min<uint32_t>(std::max(needed, capped), (uint32_t)kBigSmem);
            if (needed <= (uint32_t)kBigSmem && groups <= resident_clusters<F>(rt, 24u, shared, split, sms)) {
                plan->rt = rt;
                plan->warps_per_sm = 24;
                plan->span = rt;
                plan->slots = shape[0];
                plan->pair = shape[1];
                plan->ctas = groups * split;
                plan->shared = shared;
                return true;
            }
        }
    }
    // Otherwise a persistent grid of the widest CTAs that still give two CTAs per SM.
    uint32_t rt = 8;
    while (rt > 1u && (uint64_t)((tiles + rt - 1u) / rt) * split < 2ull * (uint64_t)sms) rt >>= 1;
    plan->rt = rt;
    const uint32_t groups = (tiles + rt - 1u) / rt;
    // Even shares over the resident clusters, two CTAs per SM (measured: three CTAs of eight warps, or one of sixteen, are
    // slower - more CTAs pay more staging, wider CTAs wait longer on their slowest warp). The shared-memory request is
    // raised to more than a third of an SM so that the hardware cannot stack three CTAs on one SM and leave another with
    // one. The ring is the deepest that fits. A larger share needs a larger gather buffer, which can lower the resident
    // count once.
    const uint32_t two_per_sm = (227u * 1024u) / 3u + 1024u;
    for (const auto& shape : shapes) {
        const uint32_t slots = shape[0], pair = shape[1];
        uint32_t span = rt, shared = std::max(two_per_sm / (8u / rt), gemv::Layout<F>(rt, span, slots, pair, chunks_max, rows, split).bytes);
        if (shared > (uint32_t)kBigSmem) continue;
        // Every warp takes the same number of tiles, `turns`: the fewest that fit the resident clusters. That usually
        // leaves a few clusters of slack, which a straggler of the previous launch can hold without delaying this one.
        // A share is at most kSpanCap tiles (the gather buffer grows with it): very tall tensors run several waves.
        const uint32_t most_turns = std::max(1u, kSpanCap / rt);
        uint32_t resident = std::min(groups, resident_clusters<F>(rt, 16u, shared, split, sms));
        bool fits = resident != 0u;
        for (int round = 0; fits && round < 3; ++round) {
            const uint32_t turns = std::min(most_turns, (tiles + rt * resident - 1u) / (rt * resident));
            span = rt * turns;
            shared = std::max(two_per_sm / (8u / rt), gemv::Layout<F>(rt, span, slots, pair, chunks_max, rows, split).bytes);
            if (shared > (uint32_t)kBigSmem) {
                fits = false;
                break;
            }
            const uint32_t again = std::min(groups, resident_clusters<F>(rt, 16u, shared, split, sms));
            if (again >= resident) break;
            resident = again;
            fits = resident != 0u;
        }
        if (!fits) continue;
        if ((uint64_t)resident * split * rt < 16ull * (uint64_t)sms * 9u / 10u && !(slots == 2u && pair == 1u)) continue;   // too few warps per SM
        plan->warps_per_sm = 16;
        plan->span = span;
        plan->slots = slots;
        plan->pair = pair;
        plan->ctas = (tiles + span - 1u) / span * split;
        plan->shared = shared;
        return true;
    }
    return false;
}

// The calling thread remembers the last plans it made (a plan costs several occupancy look-ups).
template <class F>
bool plan_decode(uint32_t rows, uint32_t k, uint32_t n, int sms, DecodePlan* plan) {
    struct Cached {
        int device;
        uint32_t rows, k, n;
        bool ok;
        DecodePlan plan;
    };
    constexpr int kCached = 32;
    thread_local Cached cache[kCached] = {};
    thread_local int next = 0;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess) {
        (void)cudaGetLastError();
        device = -1;
    }
    for (int i = 0; i < kCached; ++i) {
        const Cached& c = cache[i];
        if (c.k == k && c.n == n && c.rows == rows && c.device == device && c.k != 0) {
            *plan = c.plan;
            return c.ok;
        }
    }
    Cached& slot = cache[next];
    next = (next + 1) % kCached;
    slot.device = device;
    slot.rows = rows;
    slot.k = k;
    slot.n = n;
    slot.ok = plan_decode_uncached<F>(rows, k, n, sms, &slot.plan);
    if (k == 0) return slot.ok;   // never cached: k == 0 marks an empty slot
    *plan = slot.plan;
    return slot.ok;
}

template <class F>
cudaError_t launch_gemv(const DecodePlan& p, const void* x, const void* w, void* y, uint32_t rows, uint32_t k, uint32_t n,
        uint32_t* error) {
    const dim3 grid(p.ctas), block(32u * p.rt);
    // Encoding a tensor map costs about a microsecond of host time: the calling thread keeps the last few it made. A map
    // holds only the address and the shape, so a stale entry for a reused address is still the right map.
    struct Cached {
        const void* weights;
        uint32_t n, k, format;
        CUtensorMap map;
    };
    constexpr int kCached = 32;
    thread_local Cached cache[kCached] = {};
    thread_local int next = 0;
    const CUtensorMap* found = nullptr;
    for (int i = 0; i < kCached; ++i)
        if (cache[i].weights == w && cache[i].n == n && cache[i].k == k && cache[i].format == F::kErrorBit) found = &cache[i].map;
    if (found == nullptr) {
        Cached& slot = cache[next];
        if (!gemv::encode_codes<F>(&slot.map, w, n, k)) return cudaErrorNotSupported;
        slot.weights = w;
        slot.n = n;
        slot.k = k;
        slot.format = F::kErrorBit;
        found = &slot.map;
        next = (next + 1) % kCached;
    }
    const CUtensorMap& map = *found;
    auto xs = static_cast<const uint16_t*>(x);
    auto ws = static_cast<const uint8_t*>(w);
    auto ys = static_cast<uint16_t*>(y);
#ifdef EB_X_TRACE
    static std::atomic<uint32_t> generation{0};
    const uint32_t trace_generation = generation.fetch_add(1);
#define EB_LAUNCH_GEMV(RT, WARPS) \
    launch(gemv::kernel<F, RT, WARPS>, grid, block, p.shared, p.split, map, xs, ws, ys, rows, k, n, p.split, p.span, p.slots, p.pair, error, trace_generation)
#else
#define EB_LAUNCH_GEMV(RT, WARPS) \
    launch(gemv::kernel<F, RT, WARPS>, grid, block, p.shared, p.split, map, xs, ws, ys, rows, k, n, p.split, p.span, p.slots, p.pair, error)
#endif
    if (p.warps_per_sm == 24u) {
        switch (p.rt) {
            case 8: return EB_LAUNCH_GEMV(8, 24);
            case 4: return EB_LAUNCH_GEMV(4, 24);
            case 2: return EB_LAUNCH_GEMV(2, 24);
            default: return EB_LAUNCH_GEMV(1, 24);
        }
    }
    switch (p.rt) {
        case 8: return EB_LAUNCH_GEMV(8, 16);
        case 4: return EB_LAUNCH_GEMV(4, 16);
        case 2: return EB_LAUNCH_GEMV(2, 16);
        default: return EB_LAUNCH_GEMV(1, 16);
    }
#undef EB_LAUNCH_GEMV
}

uint32_t capped_grid(uint64_t count) { return count > 2147483647ull ? 2147483647u : (uint32_t)count; }

// NVFP4 tensor byte size: 0 plain, 1 SD4 (table-indexed scales), -1 neither (native/src/host/nvfp4_linear.c:79-91).
int nvfp4_layout(uint32_t rows, uint32_t k, uint64_t bytes) {
    if (bytes == nvfp4::Geometry(rows, k).size) return 0;
    const uint64_t kp = ((uint64_t)k + 127u) / 128u * 128u;
    const uint64_t index_offset = nvfp4::align256((uint64_t)rows * kp / 2u);
    if (bytes == nvfp4::align256(index_offset + (uint64_t)rows * kp / 32u) + 20u) return 1;
    return -1;
}

// ---- trellis table ------------------------------------------------------------------------------------------------------
struct TableEntry {
    const char* name;
    int available;
    int count;
    uint8_t sizes[12];
};
// Order is the ABI (native/src/host/linear_kernels.c:7-24). Entries whose kernels this build does not carry stay in
// the table, unavailable: the whole-K prefill kernels and their epilogue, the FP8 kernels, the embedding lookup.
const TableEntry kTable[] = {
        {"euhedral_trellis_prepass", 1, 7, {8, 8, 8, 4, 4, 4, 4}},
        {"euhedral_trellis_mma", 1, 12, {8, 8, 8, 8, 8, 8, 4, 4, 4, 4, 4, 4}},
        {"euhedral_trellis_mma_rows", 0, 11, {8, 8, 8, 8, 8, 4, 4, 4, 4, 4, 4}},
        {"euhedral_trellis_mma_rows64", 0, 11, {8, 8, 8, 8, 8, 4, 4, 4, 4, 4, 4}},
        {"euhedral_trellis_epilogue", 1, 6, {8, 4, 8, 8, 4, 4}},
        {"euhedral_trellis_decode_bf16", 1, 5, {8, 8, 4, 4, 4}},
        {"euhedral_trellis_epilogue_bf16", 0, 7, {8, 8, 4, 8, 8, 4, 4}},
        {"euhedral_trellis_reference", 1, 11, {8, 8, 8, 8, 8, 4, 8, 4, 4, 4, 4}},
        {"euhedral_trellis_mma_rows_fp8", 0, 11, {8, 8, 8, 8, 8, 4, 4, 4, 4, 4, 4}},
        {"euhedral_trellis_mma_rows64_fp8", 0, 11, {8, 8, 8, 8, 8, 4, 4, 4, 4, 4, 4}},
        {"euhedral_nvfp4_embedding", 0, 0, {0}},
};
constexpr int kTableCount = (int)(sizeof(kTable) / sizeof(kTable[0]));

bool trellis_width_valid(int w) { return w >= 16 && w <= 128 && w % 8 == 0; }

template <int W>
cudaError_t launch_trellis_mma(const uint64_t* a, uint32_t* error) {
    const int rows = (int)a[6], k = (int)a[7], n = (int)a[8], splits = (int)a[10], s = (int)a[11];
    const dim3 grid((unsigned)(n / 128), (unsigned)splits), block(256);
    const size_t shared = (size_t)trellis::kStages * trellis::kStageTiles * 8u * W * 2u;
    auto act = reinterpret_cast<const uint16_t*>(a[0]);
    auto words = reinterpret_cast<const uint16_t*>(a[1]);
    auto ends = reinterpret_cast<const int*>(a[2]);
    auto svh = reinterpret_cast<const uint16_t*>(a[3]);
    auto partials = reinterpret_cast<float*>(a[4]);
    auto out = reinterpret_cast<uint16_t*>(a[5]);
    // The payload as [k / 16][n / 16 * W / 4] 8-byte elements; a box is one ring stage of one 128-column block. The calling
    // thread keeps the last few maps (encoding costs about a microsecond).
    struct Cached {
        const void* words;
        int k, n, w;
        CUtensorMap map;
    };
    constexpr int kCached = 16;
    thread_local Cached cache[kCached] = {};
    thread_local int next = 0;
    const CUtensorMap* map = nullptr;
    for (int i = 0; i < kCached; ++i)
        if (cache[i].words == words && cache[i].k == k && cache[i].n == n && cache[i].w == W) map = &cache[i].map;
    if (map == nullptr) {
        const eb::EncodeTiled encode = eb::encoder();
        if (encode == nullptr) return cudaErrorNotSupported;
        Cached& slot = cache[next];
        const cuuint64_t dims[2] = {(cuuint64_t)(n / 16) * (W / 4), (cuuint64_t)(k / 16)}, strides[1] = {(cuuint64_t)(n / 16) * W * 2u};
        const cuuint32_t box[2] = {2u * W, (cuuint32_t)trellis::kStageTiles}, ones[2] = {1u, 1u};
        if (encode(&slot.map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint16_t*>(words), dims, strides, box, ones,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
        slot.words = words;
        slot.k = k;
        slot.n = n;
        slot.w = W;
        map = &slot.map;
        next = (next + 1) % kCached;
    }
    if (rows <= 8)
        return launch(trellis::mma_kernel<W, 1>, grid, block, shared, 1u, *map, act, words, ends, svh, partials, out, rows, k, n, splits, s, error);
    return launch(trellis::mma_kernel<W, 4>, grid, block, shared, 1u, *map, act, words, ends, svh, partials, out, rows, k, n, splits, s, error);
}

cudaError_t launch_trellis_prepass(const void* x, const void* suh, void* act, int rows, int k, int s, int layout) {
    return launch(trellis::prepass_kernel, dim3((unsigned)((k + 511) / 512), (unsigned)rows, (unsigned)s), dim3(128), 0, 1u,
            static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(suh), static_cast<uint16_t*>(act), rows, k, s, layout);
}

cudaError_t launch_trellis_epilogue(const void* partials, int splits, const void* svh, void* out, int rows, int n) {
    return launch(trellis::epilogue_kernel, dim3((unsigned)((n + 511) / 512), (unsigned)rows), dim3(128), 0, 1u,
            static_cast<const float*>(partials), splits, static_cast<const uint16_t*>(svh), static_cast<uint16_t*>(out), rows, n);
}

cudaError_t launch_trellis_mma_width(int w, const uint64_t* a, uint32_t* error) {
    switch (w) {
#define EB_CASE(W) case W: return launch_trellis_mma<W>(a, error);
        EB_TRELLIS_WIDTHS(EB_CASE)
#undef EB_CASE
    }
    return cudaErrorInvalidValue;
}

}  // namespace

extern "C" {

void* euhedral_cuda_submission_stream(void) { return t_stream; }

int euhedral_cuda_set_include_directory(const char* path) {
    if (path == nullptr || path[0] == '\0' || std::strlen(path) >= 4096) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    return EUHEDRAL_CUDA_SUCCESS;
}

void* euhedral_cuda_malloc(uint64_t byte_size) {
    if (byte_size == 0) return nullptr;
    void* address = nullptr;
    return cudaMalloc(&address, (size_t)byte_size) == cudaSuccess ? address : nullptr;
}

int euhedral_cuda_free(void* address) {
    if (address == nullptr) return EUHEDRAL_CUDA_SUCCESS;
    const cudaError_t e = cudaFree(address);
    return e == cudaSuccess ? EUHEDRAL_CUDA_SUCCESS : (int)e;
}

void* euhedral_cuda_host_malloc(uint64_t byte_size) {
    if (byte_size == 0) return nullptr;
    void* address = nullptr;
    return cudaMallocHost(&address, (size_t)byte_size) == cudaSuccess ? address : nullptr;
}

int euhedral_cuda_host_free(void* address) {
    if (address == nullptr) return EUHEDRAL_CUDA_SUCCESS;
    const cudaError_t e = cudaFreeHost(address);
    return e == cudaSuccess ? EUHEDRAL_CUDA_SUCCESS : (int)e;
}

int euhedral_cuda_multiprocessor_count(int32_t* count) {
    if (count == nullptr) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    int device = 0, value = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return (int)e;
    *count = value;
    return EUHEDRAL_CUDA_SUCCESS;
}

int euhedral_cuda_compute_capability(int32_t* major, int32_t* minor) {
    if (major == nullptr || minor == nullptr) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    int device = 0, high = 0, low = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&high, cudaDevAttrComputeCapabilityMajor, device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&low, cudaDevAttrComputeCapabilityMinor, device);
    if (e != cudaSuccess) return (int)e;
    *major = high;
    *minor = low;
    return EUHEDRAL_CUDA_SUCCESS;
}

int euhedral_cuda_copy_host_to_device(void* device_address, const void* host_address, uint64_t byte_size) {
    if (byte_size == 0) return EUHEDRAL_CUDA_SUCCESS;
    if (device_address == nullptr || host_address == nullptr) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    cudaError_t e = t_stream == nullptr ? cudaMemcpy(device_address, host_address, (size_t)byte_size, cudaMemcpyHostToDevice)
                                        : cudaMemcpyAsync(device_address, host_address, (size_t)byte_size, cudaMemcpyHostToDevice, t_stream);
    if (e == cudaSuccess && t_stream != nullptr) e = cudaStreamSynchronize(t_stream);
    return e == cudaSuccess ? EUHEDRAL_CUDA_SUCCESS : (int)e;
}

int euhedral_cuda_copy_upload_to_device(void* device_address, const void* host_address, uint64_t byte_size) {
    if (device_address == nullptr || host_address == nullptr || byte_size == 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    const cudaError_t e = t_stream == nullptr ? cudaMemcpy(device_address, host_address, (size_t)byte_size, cudaMemcpyHostToDevice)
                                              : cudaMemcpyAsync(device_address, host_address, (size_t)byte_size, cudaMemcpyHostToDevice, t_stream);
    return e == cudaSuccess ? EUHEDRAL_CUDA_SUCCESS : (int)e;
}

int euhedral_cuda_copy_device_to_host(void* host_address, const void* device_address, uint64_t byte_size) {
    if (byte_size == 0) return EUHEDRAL_CUDA_SUCCESS;
    if (host_address == nullptr || device_address == nullptr) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    cudaError_t e = t_stream == nullptr ? cudaMemcpy(host_address, device_address, (size_t)byte_size, cudaMemcpyDeviceToHost)
                                        : cudaMemcpyAsync(host_address, device_address, (size_t)byte_size, cudaMemcpyDeviceToHost, t_stream);
    if (e == cudaSuccess && t_stream != nullptr) e = cudaStreamSynchronize(t_stream);
    return e == cudaSuccess ? EUHEDRAL_CUDA_SUCCESS : (int)e;
}

int euhedral_cuda_copy_device_to_readback(void* host_address, const void* device_address, uint64_t byte_size) {
    if (host_address == nullptr || device_address == nullptr || byte_size == 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    const cudaError_t e = t_stream == nullptr ? cudaMemcpy(host_address, device_address, (size_t)byte_size, cudaMemcpyDeviceToHost)
                                              : cudaMemcpyAsync(host_address, device_address, (size_t)byte_size, cudaMemcpyDeviceToHost, t_stream);
    return e == cudaSuccess ? EUHEDRAL_CUDA_SUCCESS : (int)e;
}

int euhedral_cuda_synchronize(void) {
    const cudaError_t e = cudaDeviceSynchronize();
    return e == cudaSuccess ? EUHEDRAL_CUDA_SUCCESS : (int)e;
}

uint64_t euhedral_cuda_stream_create(void) {
    cudaStream_t stream = nullptr;
    if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) return 0;
    return (uint64_t)(uintptr_t)stream;
}

int euhedral_cuda_stream_destroy(uint64_t stream) {
    if (stream == 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    const cudaError_t e = cudaStreamDestroy((cudaStream_t)(uintptr_t)stream);
    return e == cudaSuccess ? EUHEDRAL_CUDA_SUCCESS : (int)e;
}

int euhedral_cuda_stream_synchronize(uint64_t stream) {
    if (stream == 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    const cudaError_t e = cudaStreamSynchronize((cudaStream_t)(uintptr_t)stream);
    return e == cudaSuccess ? EUHEDRAL_CUDA_SUCCESS : (int)e;
}

int euhedral_cuda_stream_select(uint64_t stream) {
    if (stream == 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    t_stream = (cudaStream_t)(uintptr_t)stream;
    return EUHEDRAL_CUDA_SUCCESS;
}

void euhedral_cuda_stream_clear(void) { t_stream = nullptr; }
void euhedral_cuda_pdl_select(int enabled) { t_pdl = enabled != 0; }
void euhedral_cuda_row_exact_select(int enabled) { t_row_exact = enabled != 0; }
int euhedral_cuda_select_exact_numerics(int exact) { return g_exact.exchange(exact != 0 ? 1 : 0); }

// ---- Q3 -------------------------------------------------------------------------------------------------------------

static int q3_reference(DeviceState* state, const void* input, const void* weights, void* output, uint32_t rows,
        uint32_t in_features, uint32_t out_features) {
    (void)state;
    const uint64_t count = (uint64_t)rows * out_features;
    if (count > 2147483647ull) return EUHEDRAL_CUDA_SIZE_OVERFLOW;
    const q3::Geometry geo(out_features, in_features);
    return finish(launch(exact::q3_linear, dim3((unsigned)count), dim3(128), 0, 1u, static_cast<const uint16_t*>(input),
            static_cast<const uint8_t*>(weights), static_cast<uint16_t*>(output), rows, in_features, out_features,
            (uint64_t)geo.scale_offset));
}

static int q3_validate(const void* input, const void* weights, void* output, uint32_t rows, uint32_t in_features,
        uint32_t out_features, uint64_t bytes) {
    if (input == nullptr || weights == nullptr || output == nullptr || rows == 0 || in_features == 0 || out_features == 0 || bytes == 0)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    if (q3::Geometry(out_features, in_features).size != bytes) return EUHEDRAL_CUDA_FORMAT_MISMATCH;
    return EUHEDRAL_CUDA_SUCCESS;
}

int euhedral_cuda_linear_q3_bf16(const void* input, const void* weights, void* output, uint32_t rows, uint32_t in_features,
        uint32_t out_features, uint64_t weights_byte_size) {
    int status = q3_validate(input, weights, output, rows, in_features, out_features, weights_byte_size);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    DeviceState* state = nullptr;
    status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    DecodePlan plan;
    const bool qualified = rows <= 32u && ((uintptr_t)input & 15u) == 0 && ((uintptr_t)weights & 15u) == 0
            && plan_decode<q3::Format>(rows < 8u ? rows : 8u, in_features, out_features, state->sms, &plan);
    if (g_exact.load() || !qualified) return q3_reference(state, input, weights, output, rows, in_features, out_features);
    for (uint32_t first = 0; first < rows; first += 8u) {
        const uint32_t group = rows - first < 8u ? rows - first : 8u;
        plan_decode<q3::Format>(group, in_features, out_features, state->sms, &plan);
        const cudaError_t e = launch_gemv<q3::Format>(plan, static_cast<const uint16_t*>(input) + (uint64_t)first * in_features, weights,
                static_cast<uint16_t*>(output) + (uint64_t)first * out_features, group, in_features, out_features, state->error_word);
        if (e != cudaSuccess) return (int)e;
    }
    return finish(cudaSuccess);
}

int euhedral_cuda_linear_q3_reference_bf16(const void* input, const void* weights, void* output, uint32_t rows,
        uint32_t in_features, uint32_t out_features, uint64_t weights_byte_size) {
    int status = q3_validate(input, weights, output, rows, in_features, out_features, weights_byte_size);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    DeviceState* state = nullptr;
    status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    return q3_reference(state, input, weights, output, rows, in_features, out_features);
}

// ---- NVFP4 ------------------------------------------------------------------------------------------------------------

int euhedral_cuda_linear_nvfp4_bf16(const void* input, const void* weights, void* output, uint32_t rows, uint32_t in_features,
        uint32_t out_features, uint64_t weights_byte_size) {
    if (input == nullptr || weights == nullptr || output == nullptr || rows == 0 || in_features == 0 || out_features == 0)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    const int layout = nvfp4_layout(out_features, in_features, weights_byte_size);
    if (layout < 0) return EUHEDRAL_CUDA_FORMAT_MISMATCH;
    if (in_features % 32u != 0 || ((uintptr_t)input & 15u) != 0 || ((uintptr_t)weights & 15u) != 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    if (layout == 1) return EUHEDRAL_CUDA_KERNEL_UNAVAILABLE;   // table-indexed scales (SD4): no kernel in this build
    DeviceState* state = nullptr;
    const int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    DecodePlan plan;
    const bool qualified = rows <= 32u && plan_decode<nvfp4::Format>(rows < 8u ? rows : 8u, in_features, out_features, state->sms, &plan);
    if (g_exact.load() || !qualified) {
        return finish(launch(exact::nvfp4_linear, dim3(capped_grid((uint64_t)rows * out_features)), dim3(128), 0, 1u,
                static_cast<const uint16_t*>(input), static_cast<const uint8_t*>(weights), static_cast<uint16_t*>(output), rows,
                in_features, out_features));
    }
    for (uint32_t first = 0; first < rows; first += 8u) {
        const uint32_t group = rows - first < 8u ? rows - first : 8u;
        plan_decode<nvfp4::Format>(group, in_features, out_features, state->sms, &plan);
        const cudaError_t e = launch_gemv<nvfp4::Format>(plan, static_cast<const uint16_t*>(input) + (uint64_t)first * in_features, weights,
                static_cast<uint16_t*>(output) + (uint64_t)first * out_features, group, in_features, out_features, state->error_word);
        if (e != cudaSuccess) return (int)e;
    }
    return finish(cudaSuccess);
}

int euhedral_cuda_nvfp4_native_available(void) {
    DeviceState* state = nullptr;
    return bind(&state) == EUHEDRAL_CUDA_SUCCESS ? 1 : 0;
}

uint64_t euhedral_cuda_nvfp4_native_scratch_bytes(uint32_t rows, uint32_t in_features, uint32_t out_features) {
    return nvfp4n::ActivationLayout(rows, in_features, out_features).bytes;
}

int euhedral_cuda_linear_nvfp4_native_bf16(const void* input, const void* weights, void* output, void* scratch, uint32_t rows,
        uint32_t in_features, uint32_t out_features, uint64_t weights_byte_size, uint64_t scratch_byte_size) {
    DeviceState* state = nullptr;
    int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    if (in_features % 128u != 0 || g_exact.load()) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    if (input == nullptr || weights == nullptr || output == nullptr || rows == 0 || in_features == 0 || out_features == 0)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    const int layout = nvfp4_layout(out_features, in_features, weights_byte_size);
    if (layout < 0) return EUHEDRAL_CUDA_FORMAT_MISMATCH;
    if (((uintptr_t)input & 15u) != 0 || ((uintptr_t)weights & 15u) != 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    if (layout == 1 || in_features % 256u != 0 || out_features % 128u != 0 || ((uintptr_t)scratch & 127u) != 0)
        return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    if (scratch == nullptr || scratch_byte_size < nvfp4n::ActivationLayout(rows, in_features, out_features).bytes)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    if (((uint64_t)rows + 127u) / 128u * (out_features / 128u) > 2147483647ull) return EUHEDRAL_CUDA_SIZE_OVERFLOW;
    return finish(nvfp4n::run(input, weights, output, scratch, rows, in_features, out_features, state->sms, t_stream, t_pdl != 0,
            state->error_word));
}

// ---- kernel table -------------------------------------------------------------------------------------------------------

int euhedral_cuda_linear_kernel_count(void) { return kTableCount; }

const char* euhedral_cuda_linear_kernel_name(int index) { return index >= 0 && index < kTableCount ? kTable[index].name : nullptr; }

int euhedral_cuda_linear_kernel_available(int32_t kernel) {
    if (kernel < 0 || kernel >= kTableCount) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    DeviceState* state = nullptr;
    const int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    return kTable[kernel].available;
}

int euhedral_cuda_linear_launch(int32_t kernel, uint32_t grid_x, uint32_t grid_y, uint32_t grid_z, uint32_t block_x,
        uint32_t block_y, uint32_t block_z, uint32_t shared_bytes, const uint64_t* words, const uint8_t* sizes, int32_t count) {
    (void)shared_bytes;
    if (kernel < 0 || kernel >= kTableCount || words == nullptr || sizes == nullptr || count < 0 || count > 32 || grid_x == 0
            || grid_y == 0 || grid_z == 0 || block_x == 0 || block_y == 0 || block_z == 0)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    DeviceState* state = nullptr;
    const int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    const TableEntry& entry = kTable[kernel];
    if (!entry.available) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    if (count != entry.count) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    uint64_t a[12];
    for (int i = 0; i < count; ++i) {
        if (sizes[i] != entry.sizes[i]) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
        a[i] = sizes[i] == 8 ? words[i] : (uint64_t)(uint32_t)words[i];
    }
    switch (kernel) {
        case 0: {   // prepass(x, suh, out, rows, k, s, layout)
            const int rows = (int)a[3], k = (int)a[4], s = (int)a[5], layout = (int)a[6];
            if (rows <= 0 || k <= 0 || k % 128 != 0 || s <= 0 || rows > 65535 || s > 65535) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
            if (layout != 0 && layout != 1) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;   // 2 = block FP8: no kernel here
            return finish(launch_trellis_prepass(reinterpret_cast<const void*>(a[0]), reinterpret_cast<const void*>(a[1]),
                    reinterpret_cast<void*>(a[2]), rows, k, s, layout));
        }
        case 1: {   // mma(act, words, ends, svh, partials, out, rows, k, n, w, splits, s)
            const int rows = (int)a[6], k = (int)a[7], n = (int)a[8], w = (int)a[9], splits = (int)a[10], s = (int)a[11];
            if (rows <= 0 || k <= 0 || k % 128 != 0 || n <= 0 || n % 128 != 0 || !trellis_width_valid(w) || splits <= 0
                    || splits > k / 16 || splits > 65535 || s <= 0 || (a[1] & 15u) != 0)
                return EUHEDRAL_CUDA_INVALID_ARGUMENT;
            return finish(launch_trellis_mma_width(w, a, state->error_word));
        }
        case 4: {   // epilogue(partials, splits, svh, out, rows, n)
            const int splits = (int)a[1], rows = (int)a[4], n = (int)a[5];
            if (splits <= 0 || rows <= 0 || rows > 65535 || n <= 0 || n % 128 != 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
            return finish(launch_trellis_epilogue(reinterpret_cast<const void*>(a[0]), splits, reinterpret_cast<const void*>(a[2]),
                    reinterpret_cast<void*>(a[3]), rows, n));
        }
        case 5: {   // decode_bf16(words, out, k, n, w)
            const int k = (int)a[2], n = (int)a[3], w = (int)a[4];
            if (k <= 0 || k % 16 != 0 || n <= 0 || n % 16 != 0 || !trellis_width_valid(w)) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
            const uint64_t tiles = (uint64_t)(k / 16) * (uint64_t)(n / 16);
            if (tiles > 2147483647ull) return EUHEDRAL_CUDA_SIZE_OVERFLOW;
            return finish(launch(trellis::decode_bf16_kernel, dim3((unsigned)tiles), dim3(256), 0, 1u,
                    reinterpret_cast<const uint16_t*>(a[0]), reinterpret_cast<uint16_t*>(a[1]), k, n, w));
        }
        case 7: {   // reference(x, words, suh, svh, ends, s, out, rows, k, n, w)
            const int s = (int)a[5], rows = (int)a[7], k = (int)a[8], n = (int)a[9], w = (int)a[10];
            if (s <= 0 || rows <= 0 || k <= 0 || k % 128 != 0 || n <= 0 || n % 128 != 0 || !trellis_width_valid(w)) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
            const uint64_t grid = (uint64_t)rows * (uint64_t)n;
            if (grid > 2147483647ull) return EUHEDRAL_CUDA_SIZE_OVERFLOW;
            if ((size_t)k * 4u > (size_t)kBigSmem) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
            return finish(launch(exact::trellis_linear, dim3((unsigned)grid), dim3(128), (size_t)k * 4u, 1u,
                    reinterpret_cast<const uint16_t*>(a[0]), reinterpret_cast<const uint16_t*>(a[1]), reinterpret_cast<const uint16_t*>(a[2]),
                    reinterpret_cast<const uint16_t*>(a[3]), reinterpret_cast<const int*>(a[4]), s, reinterpret_cast<uint16_t*>(a[6]), rows, k, n, w));
        }
        default: return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    }
}

// ---- additions -----------------------------------------------------------------------------------------------------------

int euhedral_b200_take_device_error(uint32_t* word) {
    if (word == nullptr) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    DeviceState* state = nullptr;
    const int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(word, state->error_word, 4, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemset(state->error_word, 0, 4);
    return e == cudaSuccess ? EUHEDRAL_CUDA_SUCCESS : (int)e;
}

uint64_t euhedral_b200_static_scratch_bytes(void) { return kStaticScratchBytes; }

// A whole trellis linear (prepass, tensor-core GEMM, epilogue when the K range is split) whose scratch is the library's
// own static device array instead of caller memory. Nothing is allocated or freed here, by CUDA or by any library.
int euhedral_b200_linear_trellis_bf16_static(const void* input, const void* words, const void* suh, const void* svh,
        const void* segment_ends, void* output, uint32_t rows, uint32_t in_features, uint32_t out_features, uint32_t tile_words,
        uint32_t segments, uint32_t splits) {
    if (input == nullptr || words == nullptr || suh == nullptr || svh == nullptr || segment_ends == nullptr || output == nullptr
            || rows == 0 || in_features == 0 || in_features % 128u != 0 || out_features == 0 || out_features % 128u != 0
            || !trellis_width_valid((int)tile_words) || segments == 0 || splits == 0 || splits > in_features / 16u
            || ((uintptr_t)words & 15u) != 0)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    // Activations (FP16, every segment) on a 256-byte boundary, then the FP32 partials of every split.
    const uint64_t activations = ((uint64_t)segments * rows * in_features * 2u + 255u) & ~255ull;
    const uint64_t partials = splits > 1u ? (uint64_t)splits * rows * out_features * 4u : 0u;
    if (rows > 65535u || segments > 65535u || splits > 65535u || activations + partials > kStaticScratchBytes)
        return EUHEDRAL_CUDA_SIZE_OVERFLOW;   // beyond the static scratch: use the table launches with caller scratch
    DeviceState* state = nullptr;
    const int status = bind(&state);   // first call on a device: resolves the scratch's device address
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    unsigned char* scratch = state->static_scratch;
    cudaError_t e = launch_trellis_prepass(input, suh, scratch, (int)rows, (int)in_features, (int)segments, 0);
    if (e != cudaSuccess) return (int)e;
    const uint64_t a[12] = {(uint64_t)(uintptr_t)scratch, (uint64_t)(uintptr_t)words, (uint64_t)(uintptr_t)segment_ends,
            (uint64_t)(uintptr_t)svh, (uint64_t)(uintptr_t)(scratch + activations), (uint64_t)(uintptr_t)output, rows, in_features,
            out_features, tile_words, splits, segments};
    e = launch_trellis_mma_width((int)tile_words, a, state->error_word);
    if (e != cudaSuccess) return (int)e;
    if (splits > 1u) e = launch_trellis_epilogue(scratch + activations, (int)splits, svh, output, (int)rows, (int)out_features);
    return finish(e);
}

int euhedral_b200_decode_plan(int format, uint32_t rows, uint32_t in_features, uint32_t out_features, uint32_t* row_tiles,
        uint32_t* k_slices, uint32_t* ctas, uint32_t* shared_bytes) {
    if (row_tiles == nullptr || k_slices == nullptr || ctas == nullptr || shared_bytes == nullptr) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    int sms = 148;
    DeviceState* state = nullptr;
    if (bind(&state) == EUHEDRAL_CUDA_SUCCESS) sms = state->sms;
    DecodePlan plan;
    const bool ok = format == 0 ? plan_decode<nvfp4::Format>(rows, in_features, out_features, sms, &plan)
                                : plan_decode<q3::Format>(rows, in_features, out_features, sms, &plan);
    if (!ok) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    *row_tiles = plan.span;
    *k_slices = plan.split;
    *ctas = plan.ctas;
    *shared_bytes = plan.shared;
    return EUHEDRAL_CUDA_SUCCESS;
}

}  // extern "C"

#ifdef EB_X_TRACE
extern "C" EUHEDRAL_CUDA_EXPORT int euhedral_b200_debug_trace(void* host, uint64_t bytes) {
    cudaDeviceSynchronize();
    return (int)cudaMemcpyFromSymbol(host, gemv::g_trace, bytes);
}

// Launch-period probe: a kernel that idles for `ns` nanoseconds, launched `launches` times on the selected stream with
// the thread's programmatic-dependent-launch flag.
__global__ void debug_idle_kernel(unsigned ns, int wait_first, unsigned long long* sink) {
    if (wait_first) eb::pdl_wait();
    eb::pdl_launch_dependents();
    if (!wait_first) eb::pdl_wait();
    const unsigned long long t0 = gemv::now_ns();
    unsigned long long t = t0;
    while (t - t0 < ns) t = gemv::now_ns();
    if (threadIdx.x == 0 && blockIdx.x == 0) sink[0] = t;
}

extern "C" EUHEDRAL_CUDA_EXPORT int euhedral_b200_debug_idle(uint32_t ctas, uint32_t threads, uint32_t cluster, uint32_t shared,
        uint32_t ns, int32_t wait_first, uint32_t launches) {
    DeviceState* state = nullptr;
    int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    cudaError_t e = allow_big_smem(debug_idle_kernel);
    for (uint32_t i = 0; i < launches && e == cudaSuccess; ++i)
        e = launch(debug_idle_kernel, dim3(ctas), dim3(threads), shared, cluster, ns, (int)wait_first,
                reinterpret_cast<unsigned long long*>(state->static_scratch));
    return (int)e;
}
#endif
