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
#include "bf16_gemm.cuh"
#include "q3_gemv.cuh"
#include "trellis.cuh"
#include "trellis_encode.cuh"

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

constexpr int kBigSmem = 200 * 1024;    // kernels that also hold static shared memory
constexpr int kGemvSmem = 227 * 1024;   // the most dynamic shared memory of a CTA on sm_100 (the decode GEMV holds no static bytes)

template <typename K>
cudaError_t allow_big_smem(K kernel) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBigSmem);
}

template <int W>
cudaError_t allow_trellis_width() {
    cudaError_t e = allow_big_smem(trellis::linear_kernel<W, 1>);
    if (e == cudaSuccess) e = allow_big_smem(trellis::linear_kernel<W, 4>);
    return e;
}

template <class F>
cudaError_t allow_gemv();

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
    if (e == cudaSuccess) e = allow_gemv<nvfp4::FormatSd4>();
    if (e == cudaSuccess) e = allow_gemv<q3::Format>();
    if (e == cudaSuccess) e = allow_big_smem(exact::trellis_linear);
#define EB_ALLOW_ENCODER(KA, HALF) if (e == cudaSuccess) e = allow_big_smem(trellis_encode::viterbi_kernel<KA, HALF>);
    EB_ALLOW_ENCODER(2, false) EB_ALLOW_ENCODER(2, true) EB_ALLOW_ENCODER(3, false) EB_ALLOW_ENCODER(3, true)
    EB_ALLOW_ENCODER(4, false) EB_ALLOW_ENCODER(5, false) EB_ALLOW_ENCODER(6, false)
#undef EB_ALLOW_ENCODER
#define EB_ALLOW(W) if (e == cudaSuccess) e = allow_trellis_width<W>();
    EB_TRELLIS_WIDTHS(EB_ALLOW)
#undef EB_ALLOW
    if (e == cudaSuccess) e = nvfp4n::initialize();
    if (e == cudaSuccess) e = bf16n::initialize();
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

// One launch on the selected stream, with the cluster dimension when asked. The programmatic-dependent-launch
// attribute goes only to kernels that execute griddepcontrol.wait before their first dependent read (`overlappable`),
// and only when a stream is selected: a kernel without the wait that carried the attribute could start before the
// launch in front of it has written its input (the reference registers such kernels one by one,
// native/src/host/cuda_kernel_loader.c:302-325).
enum Overlap { kOrdered = 0, kOverlappable = 1 };

template <typename... Params, typename... Args>
cudaError_t launch(Overlap overlap, void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared, unsigned cluster, Args... args) {
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
    if (t_pdl && overlap == kOverlappable && t_stream != nullptr) {
        attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    config.attrs = attributes;
    config.numAttrs = count;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// ---- decode GEMV planning ---------------------------------------------------------------------------------------------
// How K is cut (slices, pieces: gemv::order_of) depends on the format and K only and fixes the summation order. What is
// chosen here changes no bit of the result: decoding warps per CTA (a multiple of the team size), ring depth, CTAs (one per SM,
// clusters of `split`), and the shared-memory request.
struct DecodePlan {
    gemv::Order order;
    uint32_t warps, depth, ctas, span, shared;
    bool tma_scales;
};

template <class F>
using GemvKernel = void (*)(const gemv::Group, uint32_t*);

template <class F, int P>
GemvKernel<F> gemv_kernel_from(uint32_t piece, bool tma_scales) {
    if constexpr (P > (int)F::kMaxPiece) {
        return nullptr;
    } else {
        if (piece == (uint32_t)P) return tma_scales ? gemv::kernel<F, P, true> : gemv::kernel<F, P, false>;
        return gemv_kernel_from<F, P + 1>(piece, tma_scales);
    }
}
template <class F>
GemvKernel<F> gemv_kernel(uint32_t piece, bool tma_scales) { return gemv_kernel_from<F, 1>(piece, tma_scales); }

template <class F>
cudaError_t allow_gemv() {
    cudaError_t e = cudaSuccess;
    for (uint32_t piece = 1; piece <= F::kMaxPiece && e == cudaSuccess; ++piece)
        for (int tma = 0; tma < 2 && e == cudaSuccess; ++tma) e = cudaFuncSetAttribute(gemv_kernel<F>(piece, tma != 0), cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmem);
    return e;
}

// Clusters of `split` CTAs of this kernel that the current device holds at once (0: none fit), cached per (device, kernel,
// shape of the CTA). Without a device: one CTA per SM.
template <class F>
uint32_t resident_clusters(GemvKernel<F> kernel, uint32_t warps, uint32_t shared, uint32_t split, int sms) {
    struct Entry {
        int device;
        const void* kernel;
        uint32_t warps, shared, split, clusters;
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
            if (e.device == device && e.kernel == (const void*)kernel && e.warps == warps && e.shared == shared && e.split == split) return e.clusters;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(split * 1024u);
        config.blockDim = dim3(32u * (warps + (F::kAddingWarp ? 1u : 0u)));   // the decoding warps and the adding warp
        config.dynamicSmemBytes = shared;
        cudaLaunchAttribute attribute;
        attribute.id = cudaLaunchAttributeClusterDimension;
        attribute.val.clusterDim.x = split;
        attribute.val.clusterDim.y = 1;
        attribute.val.clusterDim.z = 1;
        config.attrs = &attribute;
        config.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) == cudaSuccess) {
            cache.push_back({device, (const void*)kernel, warps, shared, split, (uint32_t)clusters});
            return (uint32_t)clusters;
        }
        (void)cudaGetLastError();
    }
    return (uint32_t)sms / split;
}

// tiles: 16-row tiles of all tensors of the launch; widest: of the tallest tensor.
template <class F>
bool plan_decode(uint32_t rows, uint32_t k, uint32_t tiles, uint32_t widest, int sms, DecodePlan* plan) {
    if (rows == 0 || rows > gemv::kMaxRows || tiles == 0) return false;
    const gemv::Order order = gemv::order_of<F>(k);
    if (!order.ok) return false;
    plan->order = order;
    plan->tma_scales = typename F::Geometry(16, k).scale_row_bytes % 16u == 0;
    const GemvKernel<F> kernel = gemv_kernel<F>(order.piece, plan->tma_scales);
    if (kernel == nullptr) return false;
    for (uint32_t warps = gemv::kMaxWarps; warps >= order.team; warps >>= 1) {
        for (uint32_t depth = 3; depth >= 2; --depth) {
            // The gather buffer grows with a cluster's share of the tallest tensor, which depends on the cluster count,
            // which can depend on the shared-memory request: settle in two rounds.
            uint32_t clusters = std::min<uint32_t>(std::max(1u, (uint32_t)sms / order.split), tiles);
            uint32_t span = 0, shared = 0;
            bool fits = true;
            for (int round = 0; round < 2 && fits; ++round) {
                span = std::min(widest, (tiles + clusters - 1u) / clusters + 1u);
                shared = gemv::Layout<F>(order, rows, warps, depth, span).bytes;
                if (shared > (uint32_t)kGemvSmem) {
                    fits = false;
                    break;
                }
                if (order.split == 1u) break;
                const uint32_t resident = resident_clusters<F>(kernel, warps, shared, order.split, sms);
                if (resident == 0u) fits = false;
                const uint32_t now = std::min(resident, tiles);
                if (now >= clusters) break;
                clusters = now;
            }
            if (!fits) continue;
            plan->warps = warps;
            plan->depth = depth;
            plan->ctas = clusters * order.split;
            plan->span = span;
            plan->shared = shared;
            return true;
        }
        if (warps == 1u) break;
    }
    return false;
}

// The tensor maps of the weight tensors the calling thread used last (encoding three maps costs a few microseconds of
// host time), with whether the weights are plain device memory: tensor maps address device memory only, so anything else
// (host-mapped, managed) is kept off this path, as the reference keeps such weights off its TMA kernels
// (core/.../gpu/ExecutionGpu.java:398-402). A map holds only the address and the shape, so a stale entry for a reused
// address is still the right map.
template <class F>
const gemv::Tensor* cached_tensor(const void* w, uint32_t n, uint32_t k, const DecodePlan& plan, bool* device_memory) {
    struct Cached {
        const void* weights;
        uint32_t n, k, format, piece;
        int device;
        bool tma_scales, device_memory;
        gemv::Tensor tensor;
    };
    constexpr uint32_t kCached = 512;
    thread_local std::vector<Cached> cache(kCached);
    int device = 0;
    (void)cudaGetDevice(&device);
    Cached& slot = cache[(uint32_t)(((uintptr_t)w >> 8) * 0x9E3779B1u >> 16) % kCached];
    if (slot.weights != w || slot.n != n || slot.k != k || slot.format != F::kErrorBit || slot.piece != plan.order.piece
            || slot.tma_scales != plan.tma_scales || slot.device != device) {
        cudaPointerAttributes attributes;
        bool plain = cudaPointerGetAttributes(&attributes, w) == cudaSuccess && attributes.type == cudaMemoryTypeDevice;
        (void)cudaGetLastError();
        slot.weights = nullptr;
        if (plain && !gemv::encode_tensor<F>(&slot.tensor, w, n, k, plan.order, plan.tma_scales)) return nullptr;
        slot.weights = w;
        slot.n = n;
        slot.k = k;
        slot.format = F::kErrorBit;
        slot.piece = plan.order.piece;
        slot.tma_scales = plan.tma_scales;
        slot.device = device;
        slot.device_memory = plain;
    }
    *device_memory = slot.device_memory;
    return &slot.tensor;
}

struct DecodeItem {
    const void* x;
    const void* w;
    void* y;
    uint32_t n;
};

// One launch over `count` tensors (at most gemv::kMaxGroup) that share K and the row count. cudaErrorNotSupported when a
// tensor's weights are not plain device memory (the caller takes the scalar kernel).
template <class F>
cudaError_t launch_gemv(const DecodeItem* items, uint32_t count, uint32_t rows, uint32_t k, int sms, uint32_t* error) {
    uint32_t tiles = 0, widest = 0;
    for (uint32_t i = 0; i < count; ++i) {
        tiles += items[i].n / 16u;
        widest = std::max(widest, items[i].n / 16u);
    }
    DecodePlan plan;
    if (!plan_decode<F>(rows, k, tiles, widest, sms, &plan)) return cudaErrorInvalidConfiguration;
    gemv::Group group = {};
    uint32_t end = 0;
    for (uint32_t i = 0; i < count; ++i) {
        bool device_memory = false;
        const gemv::Tensor* maps = cached_tensor<F>(items[i].w, items[i].n, k, plan, &device_memory);
        if (maps == nullptr) return cudaErrorInvalidValue;
        if (!device_memory) return cudaErrorNotSupported;
        gemv::Tensor& t = group.tensor[i];
        t = *maps;
        t.x = static_cast<const uint16_t*>(items[i].x);
        t.w = static_cast<const uint8_t*>(items[i].w);
        t.y = static_cast<uint16_t*>(items[i].y);
        t.n = items[i].n;
        end += items[i].n / 16u;
        t.tile_end = end;
    }
    group.count = count;
    group.rows = rows;
    group.k = k;
    group.tiles = tiles;
    group.depth = plan.depth;
    group.span = plan.span;
    return launch(kOverlappable, gemv_kernel<F>(plan.order.piece, plan.tma_scales), dim3(plan.ctas), dim3(32u * (plan.warps + (F::kAddingWarp ? 1u : 0u))), plan.shared,
            plan.order.split, group, error);
}

// A decode call of up to 32 rows over `count` tensors: groups of at most 8 rows (every row is independent of the others),
// halved again while the activations of a group do not fit beside the rings. False: no decode kernel takes the shape.
template <class F>
bool decode_takes(uint32_t k, uint32_t n) {
    return n != 0 && n % 16u == 0 && k != 0 && k % 128u == 0 && gemv::order_of<F>(k).ok;
}

template <class F>
cudaError_t run_decode(DecodeItem* items, uint32_t count, uint32_t rows, uint32_t k, int sms, uint32_t* error) {
    uint32_t tiles = 0, widest = 0;
    for (uint32_t i = 0; i < count; ++i) {
        tiles += items[i].n / 16u;
        widest = std::max(widest, items[i].n / 16u);
    }
    uint32_t group = std::min<uint32_t>(rows, gemv::kMaxRows);
    DecodePlan plan;
    while (group > 1u && !plan_decode<F>(group, k, tiles, widest, sms, &plan)) group = (group + 1u) / 2u;
    for (uint32_t first = 0; first < rows; first += group) {
        const uint32_t now = std::min(group, rows - first);
        DecodeItem shifted[gemv::kMaxGroup];
        for (uint32_t i = 0; i < count; ++i) {
            shifted[i] = items[i];
            shifted[i].x = static_cast<const uint16_t*>(items[i].x) + (uint64_t)first * k;
            shifted[i].y = static_cast<uint16_t*>(items[i].y) + (uint64_t)first * items[i].n;
        }
        const cudaError_t e = launch_gemv<F>(shifted, count, now, k, sms, error);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
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
// the table, unavailable: the whole-K prefill kernels, the FP8 kernels, the embedding lookup.
const TableEntry kTable[] = {
        {"euhedral_trellis_prepass", 1, 7, {8, 8, 8, 4, 4, 4, 4}},
        {"euhedral_trellis_mma", 1, 12, {8, 8, 8, 8, 8, 8, 4, 4, 4, 4, 4, 4}},
        {"euhedral_trellis_mma_rows", 0, 11, {8, 8, 8, 8, 8, 4, 4, 4, 4, 4, 4}},
        {"euhedral_trellis_mma_rows64", 0, 11, {8, 8, 8, 8, 8, 4, 4, 4, 4, 4, 4}},
        {"euhedral_trellis_epilogue", 1, 6, {8, 4, 8, 8, 4, 4}},
        {"euhedral_trellis_decode_bf16", 1, 5, {8, 8, 4, 4, 4}},
        {"euhedral_trellis_epilogue_bf16", 1, 7, {8, 8, 4, 8, 8, 4, 4}},
        {"euhedral_trellis_reference", 1, 11, {8, 8, 8, 8, 8, 4, 8, 4, 4, 4, 4}},
        {"euhedral_trellis_mma_rows_fp8", 0, 11, {8, 8, 8, 8, 8, 4, 4, 4, 4, 4, 4}},
        {"euhedral_trellis_mma_rows64_fp8", 0, 11, {8, 8, 8, 8, 8, 4, 4, 4, 4, 4, 4}},
        {"euhedral_nvfp4_embedding", 0, 0, {0}},
};
constexpr int kTableCount = (int)(sizeof(kTable) / sizeof(kTable[0]));

bool trellis_width_valid(int w) { return w >= 16 && w <= 128 && w % 8 == 0; }

// The payload as [k / 16][n / 16 * W / 4] 8-byte elements; a box is one streaming stage of one 128-column block. The
// calling thread keeps the maps of the last 512 objects per width (encoding costs about a microsecond).
template <int W>
const CUtensorMap* trellis_payload_map(const uint16_t* words, int k, int n) {
    struct Cached {
        const void* words;
        int k, n, w;
        CUtensorMap map;
    };
    constexpr uint32_t kCached = 512;   // direct-mapped by the payload address: every trellis object of a model, per width
    thread_local std::vector<Cached> cache(kCached);
    Cached& slot = cache[(uint32_t)(((uintptr_t)words >> 8) * 0x9E3779B1u >> 16) % kCached];
    if (slot.words == words && slot.k == k && slot.n == n && slot.w == W) return &slot.map;
    const eb::EncodeTiled encode = eb::encoder();
    if (encode == nullptr) return nullptr;
    const cuuint64_t dims[2] = {(cuuint64_t)(n / 16) * (W / 4), (cuuint64_t)(k / 16)}, strides[1] = {(cuuint64_t)(n / 16) * W * 2u};
    const cuuint32_t box[2] = {2u * W, (cuuint32_t)trellis::kStageTiles}, ones[2] = {1u, 1u};
    slot.words = nullptr;
    if (encode(&slot.map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint16_t*>(words), dims, strides, box, ones,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
            != CUDA_SUCCESS)
        return nullptr;
    slot.words = words;
    slot.k = k;
    slot.n = n;
    slot.w = W;
    return &slot.map;
}

template <int W>
cudaError_t launch_trellis_linear(const uint16_t* words, const trellis::Job& job, uint32_t* error) {
    const CUtensorMap* map = trellis_payload_map<W>(words, job.k, job.n);
    if (map == nullptr) return cudaErrorNotSupported;
    const dim3 grid((unsigned)(job.n / 128), (unsigned)job.splits), block(trellis::kThreads);
    const size_t stages = (size_t)trellis::kStages * trellis::kStageTiles * 16u * W;
    if (job.rows <= 8)
        return launch(kOverlappable, trellis::linear_kernel<W, 1>, grid, block, stages + trellis::act_bytes(1), 1u, *map, job, error);
    return launch(kOverlappable, trellis::linear_kernel<W, 4>, grid, block, stages + trellis::act_bytes(4), 1u, *map, job, error);
}

cudaError_t launch_trellis_linear_width(int w, const uint16_t* words, const trellis::Job& job, uint32_t* error) {
    switch (w) {
#define EB_CASE(W) case W: return launch_trellis_linear<W>(words, job, error);
        EB_TRELLIS_WIDTHS(EB_CASE)
#undef EB_CASE
    }
    return cudaErrorInvalidValue;
}

// Table entry 1: the activations come from the scratch a rotate launch filled; a split K leaves its partials there.
cudaError_t launch_trellis_mma(const uint64_t* a, uint32_t* error) {
    trellis::Job job = {};
    job.activations = reinterpret_cast<const uint16_t*>(a[0]);
    job.ends = reinterpret_cast<const int*>(a[2]);
    job.svh = reinterpret_cast<const uint16_t*>(a[3]);
    job.partials = reinterpret_cast<float*>(a[4]);
    job.out = reinterpret_cast<uint16_t*>(a[5]);
    job.rows = (int)a[6];
    job.k = (int)a[7];
    job.n = (int)a[8];
    job.splits = (int)a[10];
    job.s = (int)a[11];
    return launch_trellis_linear_width((int)a[9], reinterpret_cast<const uint16_t*>(a[1]), job, error);
}

cudaError_t launch_trellis_rotate(const void* x, const void* suh, void* act, int rows, int k, int s, int layout) {
    const long long tasks = (long long)s * rows * (k / 128);
    if (tasks > 2147483647ll) return cudaErrorInvalidValue;   // the kernels count tasks in 32 bits
    if (layout == 1 && rows >= 64 && s <= 65535 && (((uintptr_t)x | (uintptr_t)suh | (uintptr_t)act) & 15u) == 0) {
        // many rows in the BF16 column layout (the prefill plan): blocks through shared memory, a thread per block
        const long long per_segment = (long long)rows * (k / 128);
        return launch(kOverlappable, trellis::rotate_rows_kernel, dim3((unsigned)((per_segment + 127) / 128), (unsigned)s),
                dim3(trellis::kRotateRowsThreads), 0, 1u, static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(suh),
                static_cast<uint16_t*>(act), (uint32_t)rows, (uint32_t)k);
    }
    return launch(kOverlappable, trellis::rotate_kernel, dim3((unsigned)((tasks + 7) / 8)), dim3(256), 0, 1u,
            static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(suh), static_cast<uint16_t*>(act), rows, k, s, layout);
}

cudaError_t launch_trellis_decode_bf16(const void* words, void* out, int k, int n, int w) {
    const uint64_t tiles = (uint64_t)(k / 16) * (uint64_t)(n / 16);
    switch (w) {
#define EB_CASE(W) \
        case W: \
            return launch(kOrdered, trellis::decode_bf16_kernel<W>, dim3((unsigned)((tiles + 8 * trellis::kBatch - 1) / (8 * trellis::kBatch))), dim3(256), 0, 1u, \
                    static_cast<const uint16_t*>(words), static_cast<uint16_t*>(out), k, n);
        EB_TRELLIS_WIDTHS(EB_CASE)
#undef EB_CASE
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_trellis_finish_bf16(const void* rotated, const void* ends, int s, const void* svh, void* out, int rows, int n) {
    const long long tasks = (long long)rows * (n / 128);
    return launch(kOverlappable, trellis::finish_bf16_kernel, dim3((unsigned)((tasks + 7) / 8)), dim3(256), 0, 1u,
            static_cast<const uint16_t*>(rotated), static_cast<const int*>(ends), s, static_cast<const uint16_t*>(svh), static_cast<uint16_t*>(out), rows, n);
}

cudaError_t launch_trellis_finish(const void* partials, int splits, const void* svh, void* out, int rows, int n) {
    const long long tasks = (long long)rows * (n / 128);
    return launch(kOverlappable, trellis::finish_kernel, dim3((unsigned)((tasks + 7) / 8)), dim3(256), 0, 1u,
            static_cast<const float*>(partials), splits, static_cast<const uint16_t*>(svh), static_cast<uint16_t*>(out), rows, n);
}

// Several decode linears that share K and the row count (the q, k and v projections of a layer, or gate and up) as ONE
// launch per 8 tensors. Every output is bit for bit what the single-tensor entry point gives.
template <class F>
int linear_group(uint32_t count, const void* const* inputs, const void* const* weights, void* const* outputs, uint32_t rows,
        uint32_t in_features, const uint32_t* out_features, const uint64_t* weights_byte_sizes) {
    if (count == 0 || inputs == nullptr || weights == nullptr || outputs == nullptr || out_features == nullptr || weights_byte_sizes == nullptr
            || rows == 0 || in_features == 0)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    for (uint32_t i = 0; i < count; ++i) {
        if (inputs[i] == nullptr || weights[i] == nullptr || outputs[i] == nullptr || out_features[i] == 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
        if (typename F::Geometry(out_features[i], in_features).size != weights_byte_sizes[i]) return EUHEDRAL_CUDA_FORMAT_MISMATCH;
        if (((uintptr_t)inputs[i] & 15u) != 0 || ((uintptr_t)weights[i] & 15u) != 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
        if (!decode_takes<F>(in_features, out_features[i])) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    }
    if (rows > 32u || g_exact.load()) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    DeviceState* state = nullptr;
    const int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    for (uint32_t first = 0; first < count; first += gemv::kMaxGroup) {
        const uint32_t now = std::min<uint32_t>(gemv::kMaxGroup, count - first);
        DecodeItem items[gemv::kMaxGroup];
        for (uint32_t i = 0; i < now; ++i) items[i] = {inputs[first + i], weights[first + i], outputs[first + i], out_features[first + i]};
        const cudaError_t e = run_decode<F>(items, now, rows, in_features, state->sms, state->error_word);
        if (e == cudaErrorNotSupported || e == cudaErrorInvalidConfiguration) return first == 0 ? EUHEDRAL_CUDA_ROUTE_UNAVAILABLE : EUHEDRAL_CUDA_KERNEL_UNAVAILABLE;
        if (e != cudaSuccess) return (int)e;
    }
    return finish(cudaSuccess);
}

// The decode kernel of the layout (plain or table-indexed scales) when it takes the shape, else the scalar kernel.
template <class F, bool kTable>
int nvfp4_decode(DeviceState* state, const void* input, const void* weights, void* output, uint32_t rows, uint32_t in_features,
        uint32_t out_features) {
    if (!g_exact.load() && rows <= 32u && decode_takes<F>(in_features, out_features)) {
        DecodeItem item = {input, weights, output, out_features};
        const cudaError_t e = run_decode<F>(&item, 1, rows, in_features, state->sms, state->error_word);
        if (e != cudaErrorNotSupported && e != cudaErrorInvalidConfiguration) return finish(e);
    }
    return finish(launch(kOrdered, exact::nvfp4_linear<kTable>, dim3(capped_grid((uint64_t)rows * out_features)), dim3(128), 0, 1u,
            static_cast<const uint16_t*>(input), static_cast<const uint8_t*>(weights), static_cast<uint16_t*>(output), rows,
            in_features, out_features));
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
    return finish(launch(kOrdered, exact::q3_linear, dim3((unsigned)count), dim3(128), 0, 1u, static_cast<const uint16_t*>(input),
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
    const bool qualified = rows <= 32u && ((uintptr_t)input & 15u) == 0 && ((uintptr_t)weights & 15u) == 0
            && decode_takes<q3::Format>(in_features, out_features);
    if (!g_exact.load() && qualified) {
        DecodeItem item = {input, weights, output, out_features};
        const cudaError_t e = run_decode<q3::Format>(&item, 1, rows, in_features, state->sms, state->error_word);
        if (e != cudaErrorNotSupported && e != cudaErrorInvalidConfiguration) return finish(e);
    }
    return q3_reference(state, input, weights, output, rows, in_features, out_features);
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

// ---- Q3 prefill --------------------------------------------------------------------------------------------------------------
// The reference's entry points for Q3 linears of 9 rows and more (native/include/euhedral_cuda.h:173-197; its kernels run
// block-scaled FP8 MMAs of sm_12x on two-term E4M3 activations). Here the operands are exact the other way round: every
// weight code * f32(scale) is written to the scratch as two BF16 terms whose sum is the weight exactly
// (bf16n::q3_terms_kernel), and one tcgen05 BF16 GEMM over K' = 2 K multiplies both planes with the unchanged BF16
// activations, FP32 sums in tensor memory: sums of exact products, rounded once to BF16, as the reference's route gives.
constexpr uint32_t kQ3PrefillMinRows = 33;

int euhedral_cuda_q3_mx_available(void) {
    DeviceState* state = nullptr;
    return bind(&state) == EUHEDRAL_CUDA_SUCCESS ? 1 : 0;
}

uint64_t euhedral_cuda_q3_mx_scratch_bytes(uint32_t rows, uint32_t width, uint32_t weight_rows) {
    (void)rows;   // the activations are read where they are
    return ((uint64_t)weight_rows * width * 4u + 255u) & ~(uint64_t)255u;
}

// No K split on this route: the summation order is the K order whatever the tensor's rows.
void euhedral_cuda_q3_mx_select_split_rows(uint32_t weight_rows) { (void)weight_rows; }

static int q3_prefill(const void* input, const void* weights, void* output, void* scratch, uint32_t rows, uint32_t in_features,
        uint32_t weight_rows, uint64_t weights_byte_size, uint64_t scratch_byte_size, bool paired) {
    int status = q3_validate(input, weights, output, rows, in_features, weight_rows, weights_byte_size);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    if (scratch == nullptr) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    // the reference declines the route under exact numerics and row-exact execution (the bits are not the decode kernels');
    // here it also declines up to 32 rows, which the decode kernels take as groups of 8 several times faster than the
    // expansion of the whole tensor costs (gate at 32 rows: 90 us against 160)
    if (rows <= kQ3PrefillMinRows - 1u || in_features % 128u != 0 || weight_rows % (paired ? 256u : 128u) != 0 || g_exact.load() || t_row_exact
            || (((uintptr_t)input | (uintptr_t)weights | (uintptr_t)output) & 15u) != 0 || ((uintptr_t)scratch & 255u) != 0)
        return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    if (euhedral_cuda_q3_mx_scratch_bytes(rows, in_features, weight_rows) > scratch_byte_size) return EUHEDRAL_CUDA_SIZE_OVERFLOW;
    DeviceState* state = nullptr;
    status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    const q3::Geometry geo(weight_rows, in_features);
    const uint64_t groups = (uint64_t)weight_rows * (in_features / 64u);
    cudaError_t e = launch(kOrdered, bf16n::q3_terms_kernel, dim3((unsigned)((groups * 8u + 255u) / 256u)), dim3(256), 0, 1u,
            static_cast<const uint8_t*>(weights), geo.scale_offset, static_cast<uint16_t*>(scratch), weight_rows, in_features);
    if (e == cudaSuccess)
        e = bf16n::linear(input, scratch, output, nullptr, 0, rows, 2u * in_features, weight_rows, state->sms, t_stream, false, state->error_word,
                in_features, paired);
    return finish(e);
}

int euhedral_cuda_linear_q3_mx_bf16(const void* input, const void* weights, void* output, void* scratch, uint32_t rows, uint32_t in_features,
        uint32_t out_features, uint64_t weights_byte_size, uint64_t scratch_byte_size) {
    return q3_prefill(input, weights, output, scratch, rows, in_features, out_features, weights_byte_size, scratch_byte_size, false);
}

// The paired gate/up region: `outputs` weight rows (gate first), outputs / 2 SwiGLU values per row; gate and up rounded to
// BF16 before the SwiGLU (the reference's paired kernel, docs/kernels/PREFILL_MX.md). An output tile is 128 columns wide.
int euhedral_cuda_q3_mx_gate_up_swiglu_bf16(const void* input, const void* weights, void* output, void* scratch, uint32_t rows, uint32_t width,
        uint32_t outputs, uint64_t weight_bytes, uint64_t scratch_byte_size) {
    if (outputs % 2u != 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    return q3_prefill(input, weights, output, scratch, rows, width, outputs, weight_bytes, scratch_byte_size, true);
}

// ---- NVFP4 ------------------------------------------------------------------------------------------------------------

int euhedral_cuda_linear_nvfp4_bf16(const void* input, const void* weights, void* output, uint32_t rows, uint32_t in_features,
        uint32_t out_features, uint64_t weights_byte_size) {
    if (input == nullptr || weights == nullptr || output == nullptr || rows == 0 || in_features == 0 || out_features == 0)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    const int layout = nvfp4_layout(out_features, in_features, weights_byte_size);
    if (layout < 0) return EUHEDRAL_CUDA_FORMAT_MISMATCH;
    if (in_features % 32u != 0 || ((uintptr_t)input & 15u) != 0 || ((uintptr_t)weights & 15u) != 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    DeviceState* state = nullptr;
    const int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    return layout == 1 ? nvfp4_decode<nvfp4::FormatSd4, true>(state, input, weights, output, rows, in_features, out_features)
                       : nvfp4_decode<nvfp4::Format, false>(state, input, weights, output, rows, in_features, out_features);
}

// Process-wide: native calls of 512 rows and more run on CTA pairs (tcgen05 cta_group::2). Off unless selected.
static std::atomic<bool> g_native_pairs{false};

void euhedral_b200_select_native_pairs(int enabled) { g_native_pairs.store(enabled != 0); }

int euhedral_cuda_nvfp4_native_available(void) {
    DeviceState* state = nullptr;
    return bind(&state) == EUHEDRAL_CUDA_SUCCESS ? 1 : 0;
}

uint64_t euhedral_cuda_nvfp4_native_scratch_bytes(uint32_t rows, uint32_t in_features, uint32_t out_features) {
    return nvfp4n::ActivationLayout(rows, in_features, out_features).bytes;
}

// Validation shared by the native entry points; `input` is null for the call that finds the activations quantized already.
static int native_validate(bool has_input, const void* input, const void* weights, const void* output, const void* scratch, uint32_t rows,
        uint32_t in_features, uint32_t out_features, uint64_t weights_byte_size, uint64_t scratch_byte_size, bool* table_scales) {
    if (in_features % 128u != 0 || g_exact.load()) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    if ((has_input && input == nullptr) || weights == nullptr || output == nullptr || rows == 0 || in_features == 0 || out_features == 0)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    const int layout = nvfp4_layout(out_features, in_features, weights_byte_size);
    if (layout < 0) return EUHEDRAL_CUDA_FORMAT_MISMATCH;
    // 16-byte vector loads of the input and 16-byte stores of the output; the scratch is cut at multiples of 256 bytes from
    // its base, so a 16-byte-aligned base (what the reference asks for, native/src/host/nvfp4_linear.c:310) is enough for
    // every tensor map and bulk copy into it.
    if (((uintptr_t)input & 15u) != 0 || ((uintptr_t)weights & 15u) != 0 || ((uintptr_t)output & 15u) != 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    *table_scales = layout == 1;   // SD4: the scale repack looks the indices up in the tensor's table
    if (in_features % 256u != 0 || out_features % 128u != 0 || ((uintptr_t)scratch & 15u) != 0) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    if (scratch == nullptr || scratch_byte_size < nvfp4n::ActivationLayout(rows, in_features, out_features).bytes)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    if (((uint64_t)rows + 127u) / 128u * (out_features / 128u) > 2147483647ull) return EUHEDRAL_CUDA_SIZE_OVERFLOW;
    return EUHEDRAL_CUDA_SUCCESS;
}

int euhedral_cuda_linear_nvfp4_native_bf16(const void* input, const void* weights, void* output, void* scratch, uint32_t rows,
        uint32_t in_features, uint32_t out_features, uint64_t weights_byte_size, uint64_t scratch_byte_size) {
    DeviceState* state = nullptr;
    int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    bool table_scales = false;
    status = native_validate(true, input, weights, output, scratch, rows, in_features, out_features, weights_byte_size, scratch_byte_size, &table_scales);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    return finish(nvfp4n::run(input, weights, output, scratch, rows, in_features, out_features, state->sms, t_stream, t_pdl != 0 && t_stream != nullptr,
            state->error_word, false, g_native_pairs.load(), table_scales));
}

// The paired gate/up region (native/src/host/nvfp4_linear.c:288-295): `weights` is a gate/up object of `outputs` rows, gate
// rows first; the output is [rows][outputs / 2], bf16(silu(gate) * up) with gate and up rounded to BF16 first. An output
// tile here is 128 columns wide (the reference's: 64), so outputs / 2 must be a multiple of 128, else ROUTE_UNAVAILABLE.
int euhedral_cuda_nvfp4_native_gate_up_swiglu_bf16(const void* input, const void* weights, void* output, void* scratch, uint32_t rows,
        uint32_t width, uint32_t outputs, uint64_t weight_bytes, uint64_t scratch_byte_size) {
    DeviceState* state = nullptr;
    int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    if (outputs % 2u != 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    bool table_scales = false;
    status = native_validate(true, input, weights, output, scratch, rows, width, outputs, weight_bytes, scratch_byte_size, &table_scales);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    if (outputs % 256u != 0) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    return finish(nvfp4n::run(input, weights, output, scratch, rows, width, outputs, state->sms, t_stream, t_pdl != 0 && t_stream != nullptr,
            state->error_word, true, g_native_pairs.load(), table_scales));
}

int euhedral_b200_nvfp4_native_quantize(const void* input, void* scratch, uint32_t rows, uint32_t in_features, uint64_t scratch_byte_size) {
    DeviceState* state = nullptr;
    const int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    if (in_features == 0 || in_features % 256u != 0 || g_exact.load() || ((uintptr_t)scratch & 15u) != 0) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    if (input == nullptr || scratch == nullptr || rows == 0 || ((uintptr_t)input & 15u) != 0
            || scratch_byte_size < nvfp4n::ActivationLayout(rows, in_features, 0).bytes)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    return finish(nvfp4n::quantize(input, scratch, rows, in_features, t_stream, t_pdl != 0 && t_stream != nullptr));
}

int euhedral_b200_linear_nvfp4_native_prequantized_bf16(const void* weights, void* output, void* scratch, uint32_t rows, uint32_t in_features,
        uint32_t out_features, uint64_t weights_byte_size, uint64_t scratch_byte_size) {
    DeviceState* state = nullptr;
    int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    bool table_scales = false;
    status = native_validate(false, nullptr, weights, output, scratch, rows, in_features, out_features, weights_byte_size, scratch_byte_size,
            &table_scales);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    return finish(nvfp4n::multiply(weights, output, scratch, rows, in_features, out_features, state->sms, t_stream, t_pdl != 0 && t_stream != nullptr,
            state->error_word, false, g_native_pairs.load(), table_scales));
}

// ---- kernel table -------------------------------------------------------------------------------------------------------

int euhedral_cuda_linear_kernel_count(void) { return kTableCount; }

const char* euhedral_cuda_linear_kernel_name(int index) { return index >= 0 && index < kTableCount ? kTable[index].name : nullptr; }

int euhedral_cuda_linear_kernel_available(int32_t kernel) {
    if (kernel < 0 || kernel >= kTableCount) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    DeviceState* state = nullptr;
    const int status = bind(&state);
    // 1 available, 0 not carried by this build, negative status otherwise (reference header :449-451): a CUDA error
    // (no device, a failed initialization) reads as "no kernel".
    if (status != EUHEDRAL_CUDA_SUCCESS) return status > 0 ? EUHEDRAL_CUDA_KERNEL_UNAVAILABLE : status;
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
            if (rows <= 0 || k <= 0 || k % 128 != 0 || s <= 0 || rows > 65535 || s > 65535 || ((a[0] | a[1] | a[2]) & 7u) != 0)
                return EUHEDRAL_CUDA_INVALID_ARGUMENT;   // 8-byte vector loads and stores
            if (layout != 0 && layout != 1) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;   // 2 = block FP8: no kernel here
            return finish(launch_trellis_rotate(reinterpret_cast<const void*>(a[0]), reinterpret_cast<const void*>(a[1]),
                    reinterpret_cast<void*>(a[2]), rows, k, s, layout));
        }
        case 1: {   // mma(act, words, ends, svh, partials, out, rows, k, n, w, splits, s)
            const int rows = (int)a[6], k = (int)a[7], n = (int)a[8], w = (int)a[9], splits = (int)a[10], s = (int)a[11];
            if (rows <= 0 || k <= 0 || k % 128 != 0 || n <= 0 || n % 128 != 0 || !trellis_width_valid(w) || splits <= 0
                    || splits > k / 16 || splits > 65535 || s <= 0 || (a[1] & 15u) != 0 || ((a[0] | a[3] | a[5]) & 7u) != 0 || (a[4] & 3u) != 0)
                return EUHEDRAL_CUDA_INVALID_ARGUMENT;   // activations, svh and output move as 8-byte vectors
            return finish(launch_trellis_mma(a, state->error_word));
        }
        case 4: {   // epilogue(partials, splits, svh, out, rows, n)
            const int splits = (int)a[1], rows = (int)a[4], n = (int)a[5];
            if (splits <= 0 || rows <= 0 || rows > 65535 || n <= 0 || n % 128 != 0 || (a[0] & 15u) != 0 || ((a[2] | a[3]) & 7u) != 0)
                return EUHEDRAL_CUDA_INVALID_ARGUMENT;   // 16-byte loads of the partial sums, 8-byte vectors of svh and output
            return finish(launch_trellis_finish(reinterpret_cast<const void*>(a[0]), splits, reinterpret_cast<const void*>(a[2]),
                    reinterpret_cast<void*>(a[3]), rows, n));
        }
        case 5: {   // decode_bf16(words, out, k, n, w)
            const int k = (int)a[2], n = (int)a[3], w = (int)a[4];
            if (k <= 0 || k % 16 != 0 || n <= 0 || n % 16 != 0 || !trellis_width_valid(w) || (a[0] & 3u) != 0 || (a[1] & 15u) != 0)
                return EUHEDRAL_CUDA_INVALID_ARGUMENT;   // 4-byte loads of the ring words, 16-byte stores of eight values
            const uint64_t tiles = (uint64_t)(k / 16) * (uint64_t)(n / 16);
            if (tiles > 2147483647ull) return EUHEDRAL_CUDA_SIZE_OVERFLOW;
            return finish(launch_trellis_decode_bf16(reinterpret_cast<const void*>(a[0]), reinterpret_cast<void*>(a[1]), k, n, w));
        }
        case 6: {   // epilogue_bf16(rotated, ends, s, svh, out, rows, n)
            const int s = (int)a[2], rows = (int)a[5], n = (int)a[6];
            if (s <= 0 || rows <= 0 || rows > 65535 || n <= 0 || n % 128 != 0 || ((a[0] | a[3] | a[4]) & 7u) != 0 || (a[1] & 3u) != 0)
                return EUHEDRAL_CUDA_INVALID_ARGUMENT;   // 8-byte vectors of the products, svh and the output
            return finish(launch_trellis_finish_bf16(reinterpret_cast<const void*>(a[0]), reinterpret_cast<const void*>(a[1]), s,
                    reinterpret_cast<const void*>(a[3]), reinterpret_cast<void*>(a[4]), rows, n));
        }
        case 7: {   // reference(x, words, suh, svh, ends, s, out, rows, k, n, w)
            const int s = (int)a[5], rows = (int)a[7], k = (int)a[8], n = (int)a[9], w = (int)a[10];
            if (s <= 0 || rows <= 0 || k <= 0 || k % 128 != 0 || n <= 0 || n % 128 != 0 || !trellis_width_valid(w)) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
            const uint64_t grid = (uint64_t)rows * (uint64_t)n;
            if (grid > 2147483647ull) return EUHEDRAL_CUDA_SIZE_OVERFLOW;
            if ((size_t)k * 4u > (size_t)kBigSmem) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
            return finish(launch(kOrdered, exact::trellis_linear, dim3((unsigned)grid), dim3(128), (size_t)k * 4u, 1u,
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

// A whole trellis linear as ONE launch. The scratch holds what the K splits exchange: a flag per (column block, split),
// then the FP32 partials of every split; nothing of it needs clearing (a call's flags carry a tag of its own) and nothing
// is allocated or freed. With one split the scratch is not touched.
static std::atomic<unsigned long long> g_trellis_tag{0x9E3779B97F4A7C15ull ^ (unsigned long long)(uintptr_t)&g_trellis_tag};

// The split count of a one-launch trellis linear when the caller leaves it open: the one that needs the fewest tile rows
// per SM slot in sequence - waves of resident CTAs times the tile rows of a split, plus a few tile rows' worth of rotate,
// flag exchange and in-order sum for every split - among splits of 20 tile rows or more.
static uint32_t trellis_default_splits(uint32_t rows, uint32_t in_features, uint32_t out_features, uint32_t tile_words, int sms) {
    const uint32_t groups = rows <= 8u ? 1u : 4u;
    const uint32_t shared = (uint32_t)trellis::kStages * trellis::kStageTiles * 16u * tile_words + trellis::act_bytes((int)groups) + 1024u + 128u;
    const uint32_t per_sm = std::max(1u, std::min(groups == 1u ? (uint32_t)trellis::kResident : 2u, (uint32_t)kGemvSmem / shared));
    const uint32_t resident = per_sm * (uint32_t)sms, blocks = out_features / 128u, tiles = in_features / 16u;
    uint32_t best = 1u, best_cost = 0xFFFFFFFFu;
    for (uint32_t splits = 1u; splits <= std::max(1u, tiles / 20u); ++splits) {
        const uint32_t waves = (blocks * splits + resident - 1u) / resident;
        const uint32_t cost = waves * ((tiles + splits - 1u) / splits + (splits > 1u ? 6u : 0u));
        if (cost < best_cost) {
            best_cost = cost;
            best = splits;
        }
    }
    return best;
}

static uint64_t trellis_flag_bytes(uint32_t out_features, uint32_t splits) {
    return splits > 1u ? ((uint64_t)(out_features / 128u) * splits * 8u + 255u) & ~255ull : 0u;
}

static int trellis_linear(unsigned char* scratch, uint64_t scratch_bytes, const void* input, const void* words, const void* suh, const void* svh,
        const void* segment_ends, void* output, uint32_t rows, uint32_t in_features, uint32_t out_features, uint32_t tile_words, uint32_t segments,
        uint32_t splits) {
    if (input == nullptr || words == nullptr || suh == nullptr || svh == nullptr || segment_ends == nullptr || output == nullptr
            || rows == 0 || in_features == 0 || in_features % 128u != 0 || out_features == 0 || out_features % 128u != 0
            || !trellis_width_valid((int)tile_words) || segments == 0 || splits > in_features / 16u
            || ((uintptr_t)words & 15u) != 0 || (((uintptr_t)input | (uintptr_t)suh | (uintptr_t)svh | (uintptr_t)output) & 7u) != 0)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    DeviceState* state = nullptr;
    const int status = bind(&state);   // first call on a device: resolves the static scratch's device address
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    if (scratch == nullptr) {
        scratch = state->static_scratch;
        scratch_bytes = kStaticScratchBytes;
    }
    // splits == 0: the count that keeps the SMs' resident CTA slots busiest (trellis_default_splits). (The reference's host
    // aims at 8 blocks per SM, core/.../artifact/format/TrellisFormat.java:369-376; a caller that wants that count passes it.)
    if (splits == 0u) splits = trellis_default_splits(rows, in_features, out_features, tile_words, state->sms);
    const uint64_t flags = trellis_flag_bytes(out_features, splits);
    const uint64_t partials = splits > 1u ? (uint64_t)splits * rows * out_features * 4u : 0u;
    if (rows > 65535u || segments > 65535u || splits > 65535u || flags + partials > scratch_bytes || ((uintptr_t)scratch & 15u) != 0)
        return EUHEDRAL_CUDA_SIZE_OVERFLOW;
    trellis::Job job = {};
    job.x = static_cast<const uint16_t*>(input);
    job.suh = static_cast<const uint16_t*>(suh);
    job.ends = static_cast<const int*>(segment_ends);
    job.svh = static_cast<const uint16_t*>(svh);
    job.out = static_cast<uint16_t*>(output);
    if (splits > 1u) {
        job.flags = reinterpret_cast<unsigned long long*>(scratch);
        job.partials = reinterpret_cast<float*>(scratch + flags);
        job.tag = g_trellis_tag.fetch_add(0x9E3779B97F4A7C15ull, std::memory_order_relaxed);
    }
    job.rows = (int)rows;
    job.k = (int)in_features;
    job.n = (int)out_features;
    job.splits = (int)splits;
    job.s = (int)segments;
    return finish(launch_trellis_linear_width((int)tile_words, static_cast<const uint16_t*>(words), job, state->error_word));
}

// The scratch is the library's own static device array instead of caller memory.
int euhedral_b200_linear_trellis_bf16_static(const void* input, const void* words, const void* suh, const void* svh,
        const void* segment_ends, void* output, uint32_t rows, uint32_t in_features, uint32_t out_features, uint32_t tile_words,
        uint32_t segments, uint32_t splits) {
    if (splits == 0u) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    return trellis_linear(nullptr, 0, input, words, suh, svh, segment_ends, output, rows, in_features, out_features, tile_words, segments, splits);
}

uint64_t euhedral_b200_linear_trellis_scratch_bytes(uint32_t rows, uint32_t in_features, uint32_t out_features, uint32_t segments, uint32_t splits) {
    (void)segments;
    const uint32_t most = splits != 0u ? splits : std::max(1u, in_features / 256u);
    return most > 1u ? trellis_flag_bytes(out_features, most) + (uint64_t)most * rows * out_features * 4u : 0u;
}

int euhedral_b200_linear_trellis_bf16(const void* input, const void* words, const void* suh, const void* svh, const void* segment_ends,
        void* output, void* scratch, uint64_t scratch_bytes, uint32_t rows, uint32_t in_features, uint32_t out_features, uint32_t tile_words,
        uint32_t segments, uint32_t splits) {
    if (scratch == nullptr && splits != 1u) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    alignas(16) static unsigned char unused[16];   // one split: the scratch is never dereferenced
    return trellis_linear(scratch != nullptr ? static_cast<unsigned char*>(scratch) : unused, scratch_bytes, input, words, suh, svh,
            segment_ends, output, rows, in_features, out_features, tile_words, segments, splits);
}

// ---- trellis prefill: rotate, decode to BF16, tcgen05 BF16 GEMM per segment with the rotate-back in its epilogue ----------------
// The reference host's prefill plan (core/.../artifact/format/TrellisFormat.java:560-625) as one call: its prepass in the
// column-order BF16 layout, its decode of the payload to a BF16 matrix, and a BF16 linear per segment on the segment's
// rotated activations whose epilogue does what the plan's BF16 epilogue launch does (round the sums to BF16, rotate each
// 128-column block, scale by svh), so the products never travel through memory. Scratch: activations [s][rows][k] and the
// decoded weight [n][k], each rounded up to 256 bytes.
static uint64_t align_scratch(uint64_t bytes) { return (bytes + 255u) & ~(uint64_t)255u; }

uint64_t euhedral_b200_prefill_trellis_scratch_bytes(uint32_t rows, uint32_t in_features, uint32_t out_features, uint32_t segments) {
    return align_scratch((uint64_t)segments * rows * in_features * 2u) + align_scratch((uint64_t)out_features * in_features * 2u);
}

// out[r][j] = bf16(sum_k input[r][k] * weights[j][k]): the BF16 linear of the prefill plan on its own (the reference's
// RowExactBf16.linear, core/.../artifact/format/RowExactBf16.java:52-84, takes the same operands).
int euhedral_b200_linear_bf16(const void* input, const void* weights, void* output, uint32_t rows, uint32_t in_features, uint32_t out_features) {
    if (input == nullptr || weights == nullptr || output == nullptr || rows == 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    if (in_features == 0 || in_features % 64u != 0 || out_features == 0 || out_features % 128u != 0) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    if ((((uintptr_t)input | (uintptr_t)weights | (uintptr_t)output) & 15u) != 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    DeviceState* state = nullptr;
    const int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    return finish(bf16n::linear(input, weights, output, nullptr, out_features, rows, in_features, out_features, state->sms, t_stream,
            t_pdl != 0 && t_stream != nullptr, state->error_word));
}

// Process-wide: whether BF16 linears of 512 rows and more (the trellis and Q3 prefill) run on CTA pairs. Same bits either
// way; on by default.
void euhedral_b200_select_bf16_pairs(int enabled) { bf16n::g_pairs.store(enabled != 0); }

int euhedral_b200_prefill_trellis_bf16(const void* input, const void* words, const void* suh, const void* svh, const void* segment_ends,
        const int32_t* host_segment_ends, void* output, void* scratch, uint64_t scratch_bytes, uint32_t rows, uint32_t in_features,
        uint32_t out_features, uint32_t tile_words, uint32_t segments) {
    const uint32_t k = in_features, n = out_features;
    (void)segment_ends;   // the device copy of the ends: the fused epilogue needs the host copy only
    if (input == nullptr || words == nullptr || suh == nullptr || svh == nullptr || host_segment_ends == nullptr || output == nullptr
            || scratch == nullptr || rows == 0 || rows > 0x7FFFFFFFu / 256u || segments == 0 || segments > 64u)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    if (k == 0 || k % 128u != 0 || n == 0 || n % 128u != 0 || !trellis_width_valid((int)tile_words)) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    if ((((uintptr_t)input | (uintptr_t)suh) & 7u) != 0 || (((uintptr_t)words | (uintptr_t)svh | (uintptr_t)output) & 15u) != 0
            || ((uintptr_t)scratch & 255u) != 0)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    int32_t start = 0;
    for (uint32_t g = 0; g < segments; ++g) {   // ascending multiples of 128, the last one n (TrellisLayout.validateSegments)
        const int32_t end = host_segment_ends[g];
        if (end <= start || end % 128 != 0 || (uint32_t)end > n) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
        start = end;
    }
    if ((uint32_t)start != n) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    if (euhedral_b200_prefill_trellis_scratch_bytes(rows, k, n, segments) > scratch_bytes) return EUHEDRAL_CUDA_SIZE_OVERFLOW;
    if ((uint64_t)(k / 16u) * (n / 16u) > 2147483647ull) return EUHEDRAL_CUDA_SIZE_OVERFLOW;
    DeviceState* state = nullptr;
    const int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    uint8_t* activations = static_cast<uint8_t*>(scratch);
    uint8_t* decoded = activations + align_scratch((uint64_t)segments * rows * k * 2u);
    cudaError_t e = launch_trellis_rotate(input, suh, activations, (int)rows, (int)k, (int)segments, 1);
    if (e == cudaSuccess) e = launch_trellis_decode_bf16(words, decoded, (int)k, (int)n, (int)tile_words);
    start = 0;
    for (uint32_t g = 0; g < segments && e == cudaSuccess; ++g) {
        const uint32_t width = (uint32_t)(host_segment_ends[g] - start);
        e = bf16n::linear(activations + (uint64_t)g * rows * k * 2u, decoded + (uint64_t)start * k * 2u, static_cast<uint16_t*>(output) + start,
                static_cast<const uint16_t*>(svh) + start, n, rows, k, width, state->sms, t_stream, false, state->error_word);
        start = host_segment_ends[g];
    }
    return finish(e);
}

// The converter's tile encoder: 256-weight tiles (FP32, kernel element order) -> the 16-bit state of every position, for
// the rates the format stores tiles at (tile_words = 16 x bits per weight: 32, 40, 48, 56, 64, 80, 96). The scratch holds
// one history slab per group of a resident CTA (one CTA per SM, one or two groups that encode side by side).
static uint32_t encoder_ctas(uint32_t count, uint32_t ka, int sms) {
    const uint32_t groups = (uint32_t)trellis_encode::groups_of((int)ka);
    return std::max(1u, std::min((count + groups - 1u) / groups, (uint32_t)sms));
}
static uint64_t encoder_scratch(uint32_t count, uint32_t ka, int sms) {
    return (uint64_t)encoder_ctas(count, ka, sms) * (uint64_t)trellis_encode::groups_of((int)ka) * trellis_encode::history_bytes((int)ka);
}

uint64_t euhedral_b200_trellis_encode_scratch_bytes(uint32_t count, uint32_t tile_words) {
    if (tile_words < 32u || tile_words > 96u || tile_words % 8u != 0) return 0;
    int sms = 148;
    DeviceState* state = nullptr;
    if (bind(&state) == EUHEDRAL_CUDA_SUCCESS) sms = state->sms;
    return encoder_scratch(count, tile_words / 16u, sms);
}

int euhedral_b200_trellis_encode_tiles(const void* tiles, uint32_t count, uint32_t tile_words, void* states, void* decoded, void* words,
        void* scratch, uint64_t scratch_bytes) {
    if (tiles == nullptr || states == nullptr || scratch == nullptr || count == 0 || ((uintptr_t)tiles & 3u) != 0 || ((uintptr_t)states & 1u) != 0
            || ((uintptr_t)decoded & 3u) != 0 || ((uintptr_t)words & 3u) != 0)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    const uint32_t ka = tile_words / 16u;
    const bool half_step = tile_words % 16u == 8u;
    if (tile_words % 8u != 0 || ka < 2u || ka > 6u || (half_step && ka > 3u)) return EUHEDRAL_CUDA_ROUTE_UNAVAILABLE;
    DeviceState* state = nullptr;
    const int status = bind(&state);
    if (status != EUHEDRAL_CUDA_SUCCESS) return status;
    const uint32_t ctas = encoder_ctas(count, ka, state->sms);
    if (encoder_scratch(count, ka, state->sms) > scratch_bytes) return EUHEDRAL_CUDA_SIZE_OVERFLOW;
    const size_t shared = trellis_encode::shared_bytes((int)ka);
    auto run = [&](auto kernel) {
        return launch(kOrdered, kernel, dim3(ctas), dim3(trellis_encode::kThreads), shared, 1u, static_cast<const float*>(tiles), count,
                static_cast<uint16_t*>(states), static_cast<float*>(decoded), static_cast<uint8_t*>(scratch));
    };
    cudaError_t e = cudaErrorInvalidValue;
    switch (tile_words) {
        case 32: e = run(trellis_encode::viterbi_kernel<2, false>); break;
        case 40: e = run(trellis_encode::viterbi_kernel<2, true>); break;
        case 48: e = run(trellis_encode::viterbi_kernel<3, false>); break;
        case 56: e = run(trellis_encode::viterbi_kernel<3, true>); break;
        case 64: e = run(trellis_encode::viterbi_kernel<4, false>); break;
        case 80: e = run(trellis_encode::viterbi_kernel<5, false>); break;
        case 96: e = run(trellis_encode::viterbi_kernel<6, false>); break;
    }
    if (e == cudaSuccess && words != nullptr) {
        const uint64_t total = (uint64_t)count * (tile_words / 2u);
        e = launch(kOrdered, trellis_encode::pack_kernel, dim3((unsigned)((total + 255u) / 256u)), dim3(256), 0, 1u,
                static_cast<const uint16_t*>(states), count, (int)ka, half_step ? 1 : 0, static_cast<uint32_t*>(words));
    }
    return finish(e);
}

int euhedral_b200_decode_plan(int format, uint32_t rows, uint32_t in_features, uint32_t out_features, uint32_t* k_slices,
        uint32_t* pieces, uint32_t* piece_chunks, uint32_t* ctas, uint32_t* shared_bytes) {
    if (k_slices == nullptr || pieces == nullptr || piece_chunks == nullptr || ctas == nullptr || shared_bytes == nullptr)
        return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    int sms = 148;
    DeviceState* state = nullptr;
    if (bind(&state) == EUHEDRAL_CUDA_SUCCESS) sms = state->sms;
    if (out_features == 0 || out_features % 16u != 0 || in_features % 128u != 0) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    DecodePlan plan;
    const uint32_t tiles = out_features / 16u;
    const bool ok = format == 0 ? plan_decode<nvfp4::Format>(rows, in_features, tiles, tiles, sms, &plan)
                                : plan_decode<q3::Format>(rows, in_features, tiles, tiles, sms, &plan);
    if (!ok) return EUHEDRAL_CUDA_INVALID_ARGUMENT;
    *k_slices = plan.order.split;
    *pieces = plan.order.team;
    *piece_chunks = plan.order.piece;
    *ctas = plan.ctas;
    *shared_bytes = plan.shared;
    return EUHEDRAL_CUDA_SUCCESS;
}

int euhedral_b200_linear_group_q3_bf16(uint32_t count, const void* const* inputs, const void* const* weights, void* const* outputs,
        uint32_t rows, uint32_t in_features, const uint32_t* out_features, const uint64_t* weights_byte_sizes) {
    return linear_group<q3::Format>(count, inputs, weights, outputs, rows, in_features, out_features, weights_byte_sizes);
}

int euhedral_b200_linear_group_nvfp4_bf16(uint32_t count, const void* const* inputs, const void* const* weights, void* const* outputs,
        uint32_t rows, uint32_t in_features, const uint32_t* out_features, const uint64_t* weights_byte_sizes) {
    // plain or table-indexed scales, told apart by the first tensor's byte size; a group holds one layout
    if (count != 0 && out_features != nullptr && weights_byte_sizes != nullptr && out_features[0] != 0
            && nvfp4_layout(out_features[0], in_features, weights_byte_sizes[0]) == 1)
        return linear_group<nvfp4::FormatSd4>(count, inputs, weights, outputs, rows, in_features, out_features, weights_byte_sizes);
    return linear_group<nvfp4::Format>(count, inputs, weights, outputs, rows, in_features, out_features, weights_byte_sizes);
}

}  // extern "C"
