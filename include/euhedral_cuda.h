/* C ABI of libeuhedral_cuda.so (sm_100a build): the quantized-linear subset of the reference's native library, with
 * the same names, argument meaning, status codes and threading rules, so that a host that binds these symbols (the
 * reference's Java FFM downcalls, its Rust loader, or ctypes) can load this library in place of the reference's for
 * the linear path. Each declaration cites the reference declaration it replaces (native/include/euhedral_cuda.h of
 * the reference project unless another file is named).
 *
 * Status codes: 0 success; negative = the library's own codes below; positive = a raw cudaError_t.
 * All pointers named device_* / input / weights / output / scratch are device addresses owned by the caller.
 * Thread-local state: selected stream, programmatic-dependent-launch flag, row-exact flag. Process-wide: exact numerics.
 * With a stream selected a call only enqueues work; with none it runs on the default stream and synchronizes the
 * device before returning. */
#ifndef EUHEDRAL_B200_CUDA_H
#define EUHEDRAL_B200_CUDA_H

#include <stdint.h>

#define EUHEDRAL_CUDA_EXPORT __attribute__((visibility("default")))

/* reference :15-21 */
#define EUHEDRAL_CUDA_SUCCESS 0
#define EUHEDRAL_CUDA_INVALID_ARGUMENT (-1)
#define EUHEDRAL_CUDA_SIZE_OVERFLOW (-2)
#define EUHEDRAL_CUDA_FORMAT_MISMATCH (-3)
#define EUHEDRAL_CUDA_KERNEL_UNAVAILABLE (-4)
#define EUHEDRAL_CUDA_ROUTE_UNAVAILABLE (-5)

#ifdef __cplusplus
extern "C" {
#endif

/* ---- supporting symbols needed to drive the linear path ---------------------------------------------------------- */

/* reference :7 - the calling thread's selected stream, NULL when none. */
EUHEDRAL_CUDA_EXPORT void* euhedral_cuda_submission_stream(void);
/* reference :30 - kernels here are prebuilt for sm_100a; accepted and ignored (same argument validation). */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_set_include_directory(const char* path);
/* reference :31-32 */
EUHEDRAL_CUDA_EXPORT void* euhedral_cuda_malloc(uint64_t byte_size);
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_free(void* address);
/* reference :35-36 - pinned host memory. */
EUHEDRAL_CUDA_EXPORT void* euhedral_cuda_host_malloc(uint64_t byte_size);
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_host_free(void* address);
/* reference :46-49 */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_multiprocessor_count(int32_t* count);
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_compute_capability(int32_t* major, int32_t* minor);
/* reference :51-60 - a copy that completes before returning; and a copy queued on the selected stream from pinned memory. */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_copy_host_to_device(void* device_address, const void* host_address, uint64_t byte_size);
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_copy_upload_to_device(void* device_address, const void* host_address, uint64_t byte_size);
/* reference :62-65 - completes before returning (the selected stream is synchronized). */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_copy_device_to_host(void* host_address, const void* device_address, uint64_t byte_size);
/* reference :67-72 - pinned destination, queued on the selected stream without synchronizing. */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_copy_device_to_readback(void* host_address, const void* device_address, uint64_t byte_size);
/* reference :392-397 */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_synchronize(void);
EUHEDRAL_CUDA_EXPORT uint64_t euhedral_cuda_stream_create(void);
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_stream_destroy(uint64_t stream);
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_stream_synchronize(uint64_t stream);
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_stream_select(uint64_t stream);
EUHEDRAL_CUDA_EXPORT void euhedral_cuda_stream_clear(void);
/* reference :399-402 */
EUHEDRAL_CUDA_EXPORT void euhedral_cuda_pdl_select(int enabled);
EUHEDRAL_CUDA_EXPORT void euhedral_cuda_row_exact_select(int enabled);
/* reference :147 - nonzero routes every quantized linear to its scalar FP32 kernel; returns the previous selection. */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_select_exact_numerics(int exact);

/* ---- quantized linears ------------------------------------------------------------------------------------------- */

/* reference :127-134 - Q3G64_F16S weights, BF16 rows in and out. 1..8 rows on the decode kernel, 9..32 as groups of 8
 * (every row bit for bit the one-row result); exact numerics, other row counts, shapes (in_features % 128,
 * out_features % 16) or alignments (input, weights 16 bytes) on the scalar kernel. */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_linear_q3_bf16(const void* device_input, const void* device_weights,
        void* device_output, uint32_t rows, uint32_t in_features, uint32_t out_features, uint64_t weights_byte_size);
/* reference :136-143 - the scalar Q3 kernel, always. */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_linear_q3_reference_bf16(const void* device_input, const void* device_weights,
        void* device_output, uint32_t rows, uint32_t in_features, uint32_t out_features, uint64_t weights_byte_size);
/* reference :152-154 - NVFP4 weights, BF16 rows in and out, same routing as Q3. The layout is read off the byte size:
 * row-split-k128-v1 (one E4M3 scale per block) or row-split-k128-sd4-v1 (a 4-bit index per block into the tensor's table
 * of 16 E4M3 codes); a size that is neither: FORMAT_MISMATCH. */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_linear_nvfp4_bf16(const void* input, const void* weights, void* output,
        uint32_t rows, uint32_t in_features, uint32_t out_features, uint64_t weights_byte_size);
/* reference :159-167 - the native FP4 route: activations quantized to two NVFP4 terms in `scratch`, block-scaled FP4
 * tensor-core GEMM (tcgen05 kind::mxf4nvf4 here). ROUTE_UNAVAILABLE under exact numerics or unsupported shapes. */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_nvfp4_native_available(void);
EUHEDRAL_CUDA_EXPORT uint64_t euhedral_cuda_nvfp4_native_scratch_bytes(uint32_t rows, uint32_t in_features, uint32_t out_features);
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_linear_nvfp4_native_bf16(const void* input, const void* weights, void* output,
        void* scratch, uint32_t rows, uint32_t in_features, uint32_t out_features, uint64_t weights_byte_size,
        uint64_t scratch_byte_size);
/* The paired gate/up region on the native route (reference native/include/euhedral_cuda.h:168-172): `weights` is a
 * gate/up object of `outputs` weight rows, gate rows first; output BF16 [rows][outputs / 2] = silu(gate) * up with gate and
 * up rounded to BF16 before the SwiGLU. Scratch as for a linear of `outputs` columns. -1 for odd `outputs`; -5 unless
 * outputs / 2 is a multiple of 128 (an output tile here is 128 columns wide). */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_nvfp4_native_gate_up_swiglu_bf16(const void* input, const void* weights, void* output,
        void* scratch, uint32_t rows, uint32_t width, uint32_t outputs, uint64_t weight_bytes, uint64_t scratch_byte_size);

/* ---- the shared linear kernel table (trellis launches) ------------------------------------------------------------ */

/* reference :446-453; table order native/src/host/linear_kernels.c:7-24. `words` holds the arguments, each 8 bytes wide
 * in the array and sizes[i] (4 or 8) bytes wide in the kernel's signature; count and widths are checked. The launch
 * geometry is re-derived from the arguments; the grid and block passed must be nonzero. */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_linear_kernel_count(void);
EUHEDRAL_CUDA_EXPORT const char* euhedral_cuda_linear_kernel_name(int index);
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_linear_kernel_available(int32_t kernel);
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_linear_launch(int32_t kernel, uint32_t grid_x, uint32_t grid_y, uint32_t grid_z,
        uint32_t block_x, uint32_t block_y, uint32_t block_z, uint32_t shared_bytes, const uint64_t* words,
        const uint8_t* sizes, int32_t count);

/* ---- additions without a counterpart in the reference -------------------------------------------------------------- */

/* Reads and clears the current device's kernel error word: nonzero when a bounded wait inside a kernel gave up
 * (bit 0 NVFP4 GEMV, bit 1 Q3 GEMV, bit 2 trellis GEMM, bit 3 NVFP4 prefill GEMM, bit 4 the BF16 GEMM of the Q3 and trellis
 * prefill). Synchronizes the device. */
EUHEDRAL_CUDA_EXPORT int euhedral_b200_take_device_error(uint32_t* word);
/* How a decode GEMV of this shape runs. k_slices (cluster size), pieces (warps that share a 16-row tile's slice) and
 * piece_chunks (128-value chunks of the widest piece) depend on the format and in_features only and fix the summation
 * order; ctas and shared_bytes are the launch for `rows` activation rows. format: 0 NVFP4, 1 Q3. Returns 0, or -1 for a
 * shape the decode kernels do not take. */
EUHEDRAL_CUDA_EXPORT int euhedral_b200_decode_plan(int format, uint32_t rows, uint32_t in_features, uint32_t out_features,
        uint32_t* k_slices, uint32_t* pieces, uint32_t* piece_chunks, uint32_t* ctas, uint32_t* shared_bytes);

/* No counterpart in the reference (its host calls one linear per launch). `count` decode linears that share in_features
 * and the row count - the q, k and v projections of a layer, or gate and up - as one launch per 8 tensors: the 16-row
 * tiles of all tensors form one work list over one persistent grid. inputs[i] BF16 [rows][in_features] (the same address
 * may repeat), weights[i] a whole tensor of out_features[i] rows and weights_byte_sizes[i] bytes, outputs[i] BF16
 * [rows][out_features[i]]. Every output is bit for bit what the single-tensor entry point writes. 1..32 rows.
 * Status codes as the single-tensor entry points; ROUTE_UNAVAILABLE (nothing ran) when a shape or exact numerics
 * needs the scalar kernel or a tensor is not in device memory: call the single-tensor entry point per tensor then. */
EUHEDRAL_CUDA_EXPORT int euhedral_b200_linear_group_q3_bf16(uint32_t count, const void* const* inputs,
        const void* const* weights, void* const* outputs, uint32_t rows, uint32_t in_features,
        const uint32_t* out_features, const uint64_t* weights_byte_sizes);
EUHEDRAL_CUDA_EXPORT int euhedral_b200_linear_group_nvfp4_bf16(uint32_t count, const void* const* inputs,
        const void* const* weights, void* const* outputs, uint32_t rows, uint32_t in_features,
        const uint32_t* out_features, const uint64_t* weights_byte_sizes);

/* No counterpart in the reference. A whole trellis linear for callers that cannot provide scratch because they cannot
 * allocate device memory at the point of the call: a host that only holds the weight and activation addresses it was
 * given, a plugin running inside somebody else's memory plan, or a step that runs after the process's allocator has
 * been frozen. The scratch (a flag per column block and K split, then the FP32 partial sums of the splits) lives in a static
 * device array inside the library, euhedral_b200_static_scratch_bytes() bytes (8 MiB) on every device that loads the
 * library, held until the process exits. The call allocates and frees nothing.
 *   input BF16 [rows][in_features]; words the payload [in/16][out/16][tile_words]; suh FP16 [segments][in]; svh FP16 [out];
 *   segment_ends int32 [segments]; output BF16 [rows][out]; splits = the K splits (1: nothing is exchanged).
 * Needs splits > 1 ? align256(out/128*splits*8) + splits*rows*out*4 : 0 <= the static size, else SIZE_OVERFLOW
 * (use euhedral_b200_linear_trellis_bf16 with caller scratch). Same results, bit for bit, as the three table launches.
 * The first call on a device looks the array's device address up; make that call before any stream capture.
 * Every call uses the same array and leaves its last contents there: calls that overlap on the GPU (two streams, or
 * two threads) race on it. Nothing in it needs clearing between calls - a flag counts only when it holds the call's own tag. */
EUHEDRAL_CUDA_EXPORT uint64_t euhedral_b200_static_scratch_bytes(void);
EUHEDRAL_CUDA_EXPORT int euhedral_b200_linear_trellis_bf16_static(const void* input, const void* words, const void* suh,
        const void* svh, const void* segment_ends, void* output, uint32_t rows, uint32_t in_features, uint32_t out_features,
        uint32_t tile_words, uint32_t segments, uint32_t splits);

/* No counterpart in the reference (its native route quantizes inside every call). The two halves of the native route
 * for linears that share their input - the q, k and v projections, or gate and up: quantize the BF16 rows into the
 * scratch once, then run each linear on the quantized activations found there. The scratch is sized for the widest of
 * those linears by euhedral_cuda_nvfp4_native_scratch_bytes; the activation part does not depend on out_features.
 * quantize + prequantized gives bit for bit what euhedral_cuda_linear_nvfp4_native_bf16 gives. Same status codes. */
EUHEDRAL_CUDA_EXPORT int euhedral_b200_nvfp4_native_quantize(const void* input, void* scratch, uint32_t rows,
        uint32_t in_features, uint64_t scratch_byte_size);
EUHEDRAL_CUDA_EXPORT int euhedral_b200_linear_nvfp4_native_prequantized_bf16(const void* weights, void* output,
        void* scratch, uint32_t rows, uint32_t in_features, uint32_t out_features, uint64_t weights_byte_size,
        uint64_t scratch_byte_size);

/* No counterpart in the reference. Process-wide switch of the native route: when enabled, calls of 512 rows and more run
 * the GEMM on CTA pairs (tcgen05 cta_group::2: an output tile of 256 x 256 per pair, half of the weight tile per CTA);
 * the results are bit for bit those of the single-CTA kernel. Off by default: on B200 the pairs measured 4-7 % slower. */
EUHEDRAL_CUDA_EXPORT void euhedral_b200_select_native_pairs(int enabled);

/* No counterpart in the reference, whose Java host plans a trellis linear as three launches through the kernel table
 * (core/.../artifact/format/TrellisFormat.java:484-567). Here the whole linear is ONE launch: the activations are rotated
 * inside the kernel, and the CTA that finishes a column block last adds the K splits in split order, rotates, scales and
 * writes BF16. Caller scratch of at least euhedral_b200_linear_trellis_scratch_bytes(...) bytes (16-byte aligned, contents
 * arbitrary, 0 bytes with one split): a 64-bit flag per column block and split, then the FP32 partial sums of the splits.
 * splits = 0 takes this device's one-wave split count; with the reference host's count (TrellisFormat.java:369-376) the
 * result is bit for bit that of the three table launches; an N-shard passes the split count of the whole tensor so that
 * it reproduces the whole tensor's bits. Arguments otherwise as euhedral_b200_linear_trellis_bf16_static. */
EUHEDRAL_CUDA_EXPORT uint64_t euhedral_b200_linear_trellis_scratch_bytes(uint32_t rows, uint32_t in_features,
        uint32_t out_features, uint32_t segments, uint32_t splits);
EUHEDRAL_CUDA_EXPORT int euhedral_b200_linear_trellis_bf16(const void* input, const void* words, const void* suh,
        const void* svh, const void* segment_ends, void* output, void* scratch, uint64_t scratch_bytes, uint32_t rows,
        uint32_t in_features, uint32_t out_features, uint32_t tile_words, uint32_t segments, uint32_t splits);

/* Q3 linears of 9 rows and more (reference: native/include/euhedral_cuda.h:173-197, the MXFP8 route of sm_12x). Same
 * names, arguments and statuses; what runs is this build's own: the weights code * f32(scale) are written to `scratch`
 * as two BF16 terms whose sum is the weight exactly, and one tcgen05 BF16 GEMM multiplies both planes with the unchanged
 * BF16 activations (FP32 sums of exact products, rounded once). scratch: 256-byte aligned,
 * euhedral_cuda_q3_mx_scratch_bytes(rows, width, weight_rows) bytes = 4 bytes per weight (larger than the reference's,
 * which holds activation planes). -5 (nothing ran) for 32 rows and fewer (the decode entry point runs them as groups of 8,
 * several times faster than expanding the tensor), when in_features or the weight rows are not multiples of 128 (256 for
 * the paired region), under exact numerics or row-exact execution, or for operands not aligned to 16 bytes (scratch:
 * 256); -3 when weights_byte_size is not the Q3G64_F16S size of the shape; -2 for too little scratch.
 * euhedral_cuda_q3_mx_select_split_rows is accepted and has no effect: K is never split, so a chunk of a tensor's output
 * rows gives the whole tensor's bits anyway. */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_q3_mx_available(void);
EUHEDRAL_CUDA_EXPORT uint64_t euhedral_cuda_q3_mx_scratch_bytes(uint32_t rows, uint32_t width, uint32_t weight_rows);
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_linear_q3_mx_bf16(const void* input, const void* weights, void* output, void* scratch,
        uint32_t rows, uint32_t in_features, uint32_t out_features, uint64_t weights_byte_size, uint64_t scratch_byte_size);
EUHEDRAL_CUDA_EXPORT void euhedral_cuda_q3_mx_select_split_rows(uint32_t weight_rows);
/* The paired gate/up region: `outputs` weight rows (gate first), outputs / 2 SwiGLU values per row, gate and up rounded
 * to BF16 before the SwiGLU. outputs / 2 a multiple of 128, else -5; odd outputs: -1. */
EUHEDRAL_CUDA_EXPORT int euhedral_cuda_q3_mx_gate_up_swiglu_bf16(const void* input, const void* weights, void* output, void* scratch,
        uint32_t rows, uint32_t width, uint32_t outputs, uint64_t weight_bytes, uint64_t scratch_byte_size);

/* Process-wide: whether the BF16 linear behind the trellis and Q3 prefill runs calls of 512 rows and more on CTA pairs
 * (tcgen05 cta_group::2: a 256 x 256 tile over two SMs). Same bits either way. On by default. */
EUHEDRAL_CUDA_EXPORT void euhedral_b200_select_bf16_pairs(int enabled);
/* The reference host's trellis prefill plan (core/.../artifact/format/TrellisFormat.java:560-625: prepass in the
 * column-order BF16 layout, euhedral_trellis_decode_bf16, its row-exact BF16 linear per segment (RowExactBf16.java:52-84),
 * euhedral_trellis_epilogue_bf16) as ONE call: the BF16 linear runs on tcgen05 and its epilogue does the plan's last
 * launch (sums rounded to BF16, each 128-column block rotated, times svh), so the products are never stored. Arguments as
 * euhedral_b200_linear_trellis_bf16, plus host_segment_ends: the same `segments` exclusive ends in HOST memory (the
 * reference's prefill takes them too: they size the per-segment launches; segment_ends, the device copy, is not read).
 * scratch: 256-byte aligned device memory of at least euhedral_b200_prefill_trellis_scratch_bytes(rows, in_features,
 * out_features, segments) bytes (rotated activations [segments][rows][in], the decoded BF16 weight [out][in]). Any row
 * count; every row's bits are independent of the rows beside it. -5 for shapes the trellis format does not have
 * (in/out features not multiples of 128, tile_words), -1 for misaligned pointers (words, svh, output 16 bytes; input, suh
 * 8) or segment ends that are not ascending multiples of 128 ending at out_features, -2 for too little scratch. */
EUHEDRAL_CUDA_EXPORT uint64_t euhedral_b200_prefill_trellis_scratch_bytes(uint32_t rows, uint32_t in_features, uint32_t out_features,
        uint32_t segments);
EUHEDRAL_CUDA_EXPORT int euhedral_b200_prefill_trellis_bf16(const void* input, const void* words, const void* suh, const void* svh,
        const void* segment_ends, const int32_t* host_segment_ends, void* output, void* scratch, uint64_t scratch_bytes, uint32_t rows,
        uint32_t in_features, uint32_t out_features, uint32_t tile_words, uint32_t segments);
/* The BF16 linear of that plan on its own: output[r][j] = bf16(sum over k of input[r][k] * weights[j][k]) for BF16 weights
 * [out_features][in_features] (the operands of the reference's RowExactBf16.linear). Every output is one FP32 sum over K in K
 * order on the tensor cores, whatever the row count. in_features % 64 == 0, out_features % 128 == 0 (else -5); pointers
 * 16-byte aligned (else -1). */
EUHEDRAL_CUDA_EXPORT int euhedral_b200_linear_bf16(const void* input, const void* weights, void* output, uint32_t rows,
        uint32_t in_features, uint32_t out_features);

/* No counterpart in the reference's C ABI (its trellis encoder lives in the quantization module's own CUDA image,
 * quantization/src/main/resources/cuda/trellis.cu:34-399). The converter's tile encoder: `count` tiles of 256 FP32 weights
 * in kernel element order -> the 16-bit trellis state of every position (uint16 [count][256]), by the format's tail-biting
 * Viterbi search; bit for bit the reference encoder's states on its golden tiles. tile_words = 16 x bits per weight, one
 * of 32, 40, 48, 56, 64, 80, 96 (else -5). decoded (may be null): the states' codebook values, float [count][256]. words
 * (may be null): the packed payload, int16 [count][tile_words], as the linears read it. scratch: at least
 * euhedral_b200_trellis_encode_scratch_bytes(count, tile_words) bytes of device memory (-2 if smaller). */
EUHEDRAL_CUDA_EXPORT uint64_t euhedral_b200_trellis_encode_scratch_bytes(uint32_t count, uint32_t tile_words);
EUHEDRAL_CUDA_EXPORT int euhedral_b200_trellis_encode_tiles(const void* tiles, uint32_t count, uint32_t tile_words, void* states,
        void* decoded, void* words, void* scratch, uint64_t scratch_bytes);

#ifdef __cplusplus
}
#endif

#endif
