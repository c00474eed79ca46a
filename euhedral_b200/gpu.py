"""The operator surface of the GPU binding, mirroring the reference's `CudaGpuMemory` / `ExecutionGpu` for the
quantized-linear path (core/.../gpu/CudaGpuMemory.java:1695-1728,2300-2317,2426-2493,3089-3124;
core/.../gpu/ExecutionGpu.java:356-420,710-722): same method names (snake case), same routing by row count, same error
behaviour (a nonzero status raises GpuMemoryException carrying the operation and the status).

Addresses are plain integers (device pointers), exactly as the Java side passes `MemorySegment.ofAddress(long)`.
"""

from __future__ import annotations

import contextlib
import ctypes as C

from euhedral_b200 import library

NVFP4_NATIVE_MIN_ROWS = 9      # CudaGpuMemory.java:2108-2110
Q3_DECODE_MAX_ROWS = 8
LINEAR_KERNELS = (             # core/.../artifact/format/LinearKernel.java:8-34 (table order is the ABI)
    "TRELLIS_PREPASS", "TRELLIS_MMA", "TRELLIS_MMA_ROWS", "TRELLIS_MMA_ROWS64", "TRELLIS_EPILOGUE", "TRELLIS_DECODE_BF16",
    "TRELLIS_EPILOGUE_BF16", "TRELLIS_REFERENCE", "TRELLIS_MMA_ROWS_FP8", "TRELLIS_MMA_ROWS64_FP8", "NVFP4_EMBEDDING",
)
LINEAR_KERNEL_INDEX = {name: index for index, name in enumerate(LINEAR_KERNELS)}


class GpuMemoryException(RuntimeError):
    def __init__(self, operation: str, status: int):
        super().__init__(f"{operation} failed with status {status}")
        self.operation = operation
        self.status = status


class KernelArguments:
    """Argument words of a table launch: 8 bytes each in the array, 4 or 8 wide in the kernel's signature
    (core/.../gpu/KernelArguments.java)."""

    def __init__(self):
        self.words: list[int] = []
        self.sizes: list[int] = []

    def pointer(self, address: int) -> "KernelArguments":
        self.words.append(int(address) & 0xFFFFFFFFFFFFFFFF)
        self.sizes.append(8)
        return self

    def int32(self, value: int) -> "KernelArguments":
        self.words.append(int(value) & 0xFFFFFFFF)
        self.sizes.append(4)
        return self


class CudaGpuMemory:
    """One per process and device. Thread-local selections (stream, PDL, row exactness) live in the library."""

    def __init__(self):
        self.lib = library.load()
        self._native_scratch = 0
        self._native_scratch_bytes = 0

    # ---- memory and streams ------------------------------------------------------------------------------------------
    def allocate(self, byte_size: int) -> int:
        address = self.lib.euhedral_cuda_malloc(byte_size)
        if not address:
            raise GpuMemoryException("device allocation", -1)
        return address

    def free(self, address: int) -> None:
        self._check("device free", self.lib.euhedral_cuda_free(address))

    def copy_host_to_device(self, device_address: int, host_address: int, byte_size: int) -> None:
        self._check("host to device copy", self.lib.euhedral_cuda_copy_host_to_device(device_address, host_address, byte_size))

    def copy_upload_to_device(self, device_address: int, host_address: int, byte_size: int) -> None:
        self._check("upload", self.lib.euhedral_cuda_copy_upload_to_device(device_address, host_address, byte_size))

    def copy_device_to_host(self, host_address: int, device_address: int, byte_size: int) -> None:
        self._check("device to host copy", self.lib.euhedral_cuda_copy_device_to_host(host_address, device_address, byte_size))

    def copy_device_to_readback(self, host_address: int, device_address: int, byte_size: int) -> None:
        self._check("readback", self.lib.euhedral_cuda_copy_device_to_readback(host_address, device_address, byte_size))

    def synchronize(self) -> None:
        self._check("synchronize", self.lib.euhedral_cuda_synchronize())

    def multiprocessor_count(self) -> int:
        count = C.c_int32()
        self._check("multiprocessor count", self.lib.euhedral_cuda_multiprocessor_count(C.byref(count)))
        return count.value

    @contextlib.contextmanager
    def submit(self, stream: int, pdl: bool = False, row_exact: bool = False):
        """Runs the body with `stream` selected on this thread (GpuStream.submit, CudaGpuMemory.java:769-796)."""
        self._check("stream select", self.lib.euhedral_cuda_stream_select(stream))
        self.lib.euhedral_cuda_pdl_select(1 if pdl else 0)
        self.lib.euhedral_cuda_row_exact_select(1 if row_exact else 0)
        self._row_exact = row_exact
        try:
            yield self
        finally:
            self.lib.euhedral_cuda_pdl_select(0)
            self.lib.euhedral_cuda_row_exact_select(0)
            self._row_exact = False
            self.lib.euhedral_cuda_stream_clear()

    _row_exact = False
    _exact = False

    def select_exact_numerics(self, exact: bool) -> bool:
        previous = self.lib.euhedral_cuda_select_exact_numerics(1 if exact else 0) != 0
        self._exact = exact
        return previous

    def exact_numerics(self) -> bool:
        return self._exact

    def take_device_error(self) -> int:
        word = C.c_uint32()
        self._check("device error word", self.lib.euhedral_b200_take_device_error(C.byref(word)))
        return word.value

    # ---- linears --------------------------------------------------------------------------------------------------------
    def linear_q3_bf16(self, input: int, weights: int, output: int, rows: int, in_features: int, out_features: int,
                       weight_bytes: int) -> None:
        """CudaGpuMemory.linearQ3Bf16 (java:1695-1728): more than 8 rows try the prefill route (`invokeQ3Mx`); when it
        declines - up to 32 rows, row-exact execution, exact numerics, a shape that is not a multiple of 128 - the decode
        entry runs the rows as groups of 8."""
        if rows > Q3_DECODE_MAX_ROWS and self.linear_q3_mx_bf16(input, weights, output, rows, in_features, out_features, weight_bytes):
            return
        self._check("Q3 linear", self.lib.euhedral_cuda_linear_q3_bf16(input, weights, output, rows, in_features,
                                                                       out_features, weight_bytes))

    def linear_q3_mx_bf16(self, input, weights, output, rows, in_features, out_features, weight_bytes) -> bool:
        """CudaGpuMemory.invokeQ3Mx: the Q3 prefill entry over the shared scratch. False when the route declined."""
        if self._row_exact or self._exact or self.lib.euhedral_cuda_q3_mx_available() != 1:
            return False
        scratch = self.native_scratch(self.lib.euhedral_cuda_q3_mx_scratch_bytes(rows, in_features, out_features))
        status = self.lib.euhedral_cuda_linear_q3_mx_bf16(input, weights, output, scratch, rows, in_features, out_features, weight_bytes,
                                                          self._native_scratch_bytes)
        if status == library.ROUTE_UNAVAILABLE:
            return False
        self._check("Q3 prefill linear", status)
        return True

    def q3_mx_gate_up_swiglu_bf16(self, input, weights, output, rows, width, outputs, weight_bytes) -> bool:
        """The paired gate/up region of the Q3 prefill (CudaGpuMemory.q3MxGateUpSwigluBf16): `weights` holds `outputs` rows,
        gate rows first; `output` gets [rows][outputs / 2] SwiGLU values. False when the route declined."""
        if self._row_exact or self._exact:
            return False
        scratch = self.native_scratch(self.lib.euhedral_cuda_q3_mx_scratch_bytes(rows, width, outputs))
        status = self.lib.euhedral_cuda_q3_mx_gate_up_swiglu_bf16(input, weights, output, scratch, rows, width, outputs, weight_bytes,
                                                                  self._native_scratch_bytes)
        if status == library.ROUTE_UNAVAILABLE:
            return False
        self._check("Q3 prefill gate/up SwiGLU", status)
        return True

    def linear_q3_reference_bf16(self, input, weights, output, rows, in_features, out_features, weight_bytes) -> None:
        self._check("Q3 reference linear", self.lib.euhedral_cuda_linear_q3_reference_bf16(
            input, weights, output, rows, in_features, out_features, weight_bytes))

    def linear_group_bf16(self, fmt: str, inputs, weights, outputs, rows: int, in_features: int, out_features, weight_bytes) -> bool:
        """Several decode linears that share in_features and the row count (q, k, v of a layer; gate and up) as one
        launch per 8 tensors; `fmt` is 'q3' or 'nvfp4'. No counterpart in the reference, whose host queues one linear
        per launch. False when the route declined (nothing ran): queue the linears one by one then."""
        count = len(weights)
        entry = self.lib.euhedral_b200_linear_group_q3_bf16 if fmt == "q3" else self.lib.euhedral_b200_linear_group_nvfp4_bf16
        status = entry(count, (C.c_void_p * count)(*inputs), (C.c_void_p * count)(*weights), (C.c_void_p * count)(*outputs), rows,
                       in_features, (C.c_uint32 * count)(*out_features), (C.c_uint64 * count)(*weight_bytes))
        if status == library.ROUTE_UNAVAILABLE:
            return False
        self._check(f"{fmt} linear group", status)
        return True

    def nvfp4_native_available(self) -> bool:
        return self.lib.euhedral_cuda_nvfp4_native_available() == 1

    def native_scratch(self, byte_size: int) -> int:
        """The shared scratch of the native route, grown on demand (the reference keeps one event-ordered scratch per
        GPU, CudaGpuMemory.java:2426-2466). Growing allocates: size it before recording a graph."""
        if byte_size > self._native_scratch_bytes:
            if self._native_scratch:
                self.synchronize()
                self.free(self._native_scratch)
            self._native_scratch = self.allocate(byte_size)
            self._native_scratch_bytes = byte_size
        return self._native_scratch

    def linear_nvfp4_bf16(self, input: int, weights: int, output: int, rows: int, in_features: int, out_features: int,
                          weight_bytes: int) -> None:
        """CudaGpuMemory.linearNvfp4Bf16 (java:2300-2317): 9 rows or more, not row-exact, not exact numerics and K a
        multiple of 128 try the native FP4 route; ROUTE_UNAVAILABLE falls through to the decode entry."""
        route = rows >= NVFP4_NATIVE_MIN_ROWS and not self._row_exact and not self._exact
        if route and in_features % 128 == 0 and self.nvfp4_native_available():
            if self.linear_nvfp4_native_bf16(input, weights, output, rows, in_features, out_features, weight_bytes):
                return
        self._check("NVFP4 linear", self.lib.euhedral_cuda_linear_nvfp4_bf16(input, weights, output, rows, in_features,
                                                                             out_features, weight_bytes))

    def linear_nvfp4_native_bf16(self, input, weights, output, rows, in_features, out_features, weight_bytes) -> bool:
        """False when the route declined (java:2458-2459 treats ROUTE_UNAVAILABLE as "did not run")."""
        need = self.lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, in_features, out_features)
        scratch = self.native_scratch(need)
        status = self.lib.euhedral_cuda_linear_nvfp4_native_bf16(input, weights, output, scratch, rows, in_features,
                                                                 out_features, weight_bytes, self._native_scratch_bytes)
        if status == library.ROUTE_UNAVAILABLE:
            return False
        self._check("native NVFP4 linear", status)
        return True

    def nvfp4_native_gate_up_swiglu_bf16(self, input, weights, output, rows, width, outputs, weight_bytes) -> bool:
        """The paired gate/up region (CudaGpuMemory.nvfp4NativeGateUpSwigluBf16): `weights` holds `outputs` rows, gate rows
        first; `output` gets [rows][outputs / 2] SwiGLU values. False when the route declined."""
        need = self.lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, width, outputs)
        scratch = self.native_scratch(need)
        status = self.lib.euhedral_cuda_nvfp4_native_gate_up_swiglu_bf16(input, weights, output, scratch, rows, width, outputs, weight_bytes,
                                                                         self._native_scratch_bytes)
        if status == library.ROUTE_UNAVAILABLE:
            return False
        self._check("native NVFP4 gate/up SwiGLU", status)
        return True

    def nvfp4_native_quantize(self, input: int, rows: int, in_features: int, out_features: int) -> bool:
        """First half of the native route for linears that share their input: quantizes the rows into the shared scratch
        (sized for the widest linear, `out_features`). No counterpart in the reference. False when the route declined."""
        need = self.lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, in_features, out_features)
        scratch = self.native_scratch(need)
        status = self.lib.euhedral_b200_nvfp4_native_quantize(input, scratch, rows, in_features, self._native_scratch_bytes)
        if status == library.ROUTE_UNAVAILABLE:
            return False
        self._check("native NVFP4 quantize", status)
        return True

    def linear_nvfp4_native_prequantized_bf16(self, weights, output, rows, in_features, out_features, weight_bytes) -> bool:
        """Second half: one linear over the activations quantized into the shared scratch by nvfp4_native_quantize."""
        status = self.lib.euhedral_b200_linear_nvfp4_native_prequantized_bf16(weights, output, self._native_scratch, rows, in_features,
                                                                              out_features, weight_bytes, self._native_scratch_bytes)
        if status == library.ROUTE_UNAVAILABLE:
            return False
        self._check("native NVFP4 linear (prequantized)", status)
        return True

    def linear_trellis_bf16(self, input: int, words: int, suh: int, svh: int, ends: int, output: int, scratch: int, scratch_bytes: int,
                            rows: int, in_features: int, out_features: int, tile_words: int, segments: int, splits: int = 0) -> None:
        """A whole trellis linear as one launch (activations rotated and K splits joined inside the kernel). No counterpart
        in the reference, whose host queues three table launches; same bits for the same split count. splits = 0: the
        device's one-wave default."""
        self._check("trellis linear", self.lib.euhedral_b200_linear_trellis_bf16(
            input, words, suh, svh, ends, output, scratch, scratch_bytes, rows, in_features, out_features, tile_words, segments, splits))

    def prefill_trellis_bf16(self, input: int, words: int, suh: int, svh: int, ends: int, host_ends, output: int, scratch: int,
                             scratch_bytes: int, rows: int, in_features: int, out_features: int, tile_words: int) -> None:
        """The reference host's trellis prefill plan (TrellisFormat.prefill) as one call; `host_ends` the segment ends as a
        Python sequence (the plan's `bounds`)."""
        bounds = (C.c_int32 * len(host_ends))(*host_ends)
        self._check("trellis prefill", self.lib.euhedral_b200_prefill_trellis_bf16(
            input, words, suh, svh, ends, C.cast(bounds, C.c_void_p), output, scratch, scratch_bytes, rows, in_features, out_features, tile_words,
            len(host_ends)))

    # ---- the linear kernel table -------------------------------------------------------------------------------------------
    def table_kernel_available(self, kernel: str | int) -> bool:
        index = LINEAR_KERNEL_INDEX[kernel] if isinstance(kernel, str) else kernel
        return self.lib.euhedral_cuda_linear_kernel_available(index) == 1

    def launch_table_kernel(self, kernel: str | int, grid_x: int, grid_y: int, grid_z: int, block_x: int, block_y: int,
                            block_z: int, shared_bytes: int, arguments: KernelArguments) -> None:
        index = LINEAR_KERNEL_INDEX[kernel] if isinstance(kernel, str) else kernel
        count = len(arguments.words)
        words = (C.c_uint64 * max(count, 1))(*arguments.words)
        sizes = (C.c_uint8 * max(count, 1))(*arguments.sizes)
        self._check(f"linear kernel {index}", self.lib.euhedral_cuda_linear_launch(
            index, grid_x, grid_y, grid_z, block_x, block_y, block_z, shared_bytes, words, sizes, count))

    @staticmethod
    def _check(operation: str, status: int) -> None:
        if status != 0:
            raise GpuMemoryException(operation, status)
