"""ctypes binding of libeuhedral_cuda.so: the part the reference's Java host plays with FFM downcalls
(core/.../gpu/CudaGpuMemory.java:227-651 binds the same symbols with Linker.downcallHandle; descriptors
core/.../gpu/ExecutionGpu.java:157-165,287-292). Loading fails loudly when the library has not been built: there is
no fallback implementation."""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
LIBRARY_PATH = PACKAGE / "lib" / "libeuhedral_cuda.so"

SUCCESS = 0
INVALID_ARGUMENT = -1
SIZE_OVERFLOW = -2
FORMAT_MISMATCH = -3
KERNEL_UNAVAILABLE = -4
ROUTE_UNAVAILABLE = -5

_u32, _u64, _i32, _ptr = C.c_uint32, C.c_uint64, C.c_int32, C.c_void_p
_LINEAR7 = [_ptr, _ptr, _ptr, _u32, _u32, _u32, _u64]

# name -> (restype, argtypes): every symbol include/euhedral_cuda.h declares.
SIGNATURES = {
    "euhedral_cuda_submission_stream": (_ptr, []),
    "euhedral_cuda_set_include_directory": (C.c_int, [C.c_char_p]),
    "euhedral_cuda_malloc": (_ptr, [_u64]),
    "euhedral_cuda_free": (C.c_int, [_ptr]),
    "euhedral_cuda_host_malloc": (_ptr, [_u64]),
    "euhedral_cuda_host_free": (C.c_int, [_ptr]),
    "euhedral_cuda_multiprocessor_count": (C.c_int, [C.POINTER(_i32)]),
    "euhedral_cuda_compute_capability": (C.c_int, [C.POINTER(_i32), C.POINTER(_i32)]),
    "euhedral_cuda_copy_host_to_device": (C.c_int, [_ptr, _ptr, _u64]),
    "euhedral_cuda_copy_upload_to_device": (C.c_int, [_ptr, _ptr, _u64]),
    "euhedral_cuda_copy_device_to_host": (C.c_int, [_ptr, _ptr, _u64]),
    "euhedral_cuda_copy_device_to_readback": (C.c_int, [_ptr, _ptr, _u64]),
    "euhedral_cuda_synchronize": (C.c_int, []),
    "euhedral_cuda_stream_create": (_u64, []),
    "euhedral_cuda_stream_destroy": (C.c_int, [_u64]),
    "euhedral_cuda_stream_synchronize": (C.c_int, [_u64]),
    "euhedral_cuda_stream_select": (C.c_int, [_u64]),
    "euhedral_cuda_stream_clear": (None, []),
    "euhedral_cuda_pdl_select": (None, [C.c_int]),
    "euhedral_cuda_row_exact_select": (None, [C.c_int]),
    "euhedral_cuda_select_exact_numerics": (C.c_int, [C.c_int]),
    "euhedral_cuda_linear_q3_bf16": (C.c_int, _LINEAR7),
    "euhedral_cuda_linear_q3_reference_bf16": (C.c_int, _LINEAR7),
    "euhedral_cuda_linear_nvfp4_bf16": (C.c_int, _LINEAR7),
    "euhedral_cuda_nvfp4_native_available": (C.c_int, []),
    "euhedral_cuda_nvfp4_native_scratch_bytes": (_u64, [_u32, _u32, _u32]),
    "euhedral_cuda_linear_nvfp4_native_bf16": (C.c_int, [_ptr, _ptr, _ptr, _ptr, _u32, _u32, _u32, _u64, _u64]),
    "euhedral_cuda_nvfp4_native_gate_up_swiglu_bf16": (C.c_int, [_ptr, _ptr, _ptr, _ptr, _u32, _u32, _u32, _u64, _u64]),
    "euhedral_cuda_linear_kernel_count": (C.c_int, []),
    "euhedral_cuda_linear_kernel_name": (C.c_char_p, [C.c_int]),
    "euhedral_cuda_linear_kernel_available": (C.c_int, [_i32]),
    "euhedral_cuda_linear_launch": (C.c_int, [_i32, _u32, _u32, _u32, _u32, _u32, _u32, _u32, C.POINTER(_u64),
                                              C.POINTER(C.c_uint8), _i32]),
    "euhedral_b200_take_device_error": (C.c_int, [C.POINTER(_u32)]),
    "euhedral_b200_static_scratch_bytes": (_u64, []),
    "euhedral_b200_linear_trellis_bf16_static": (C.c_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _u32, _u32, _u32, _u32, _u32, _u32]),
    "euhedral_b200_nvfp4_native_quantize": (C.c_int, [_ptr, _ptr, _u32, _u32, _u64]),
    "euhedral_b200_linear_nvfp4_native_prequantized_bf16": (C.c_int, [_ptr, _ptr, _ptr, _u32, _u32, _u32, _u64, _u64]),
    "euhedral_b200_select_native_pairs": (None, [C.c_int]),
    "euhedral_b200_trellis_encode_scratch_bytes": (_u64, [_u32, _u32]),
    "euhedral_cuda_q3_mx_available": (C.c_int, []),
    "euhedral_cuda_q3_mx_scratch_bytes": (_u64, [_u32, _u32, _u32]),
    "euhedral_cuda_linear_q3_mx_bf16": (C.c_int, [_ptr, _ptr, _ptr, _ptr, _u32, _u32, _u32, _u64, _u64]),
    "euhedral_cuda_q3_mx_select_split_rows": (None, [_u32]),
    "euhedral_cuda_q3_mx_gate_up_swiglu_bf16": (C.c_int, [_ptr, _ptr, _ptr, _ptr, _u32, _u32, _u32, _u64, _u64]),
    "euhedral_b200_select_bf16_pairs": (None, [C.c_int]),
    "euhedral_b200_linear_bf16": (C.c_int, [_ptr, _ptr, _ptr, _u32, _u32, _u32]),
    "euhedral_b200_prefill_trellis_scratch_bytes": (_u64, [_u32, _u32, _u32, _u32]),
    "euhedral_b200_prefill_trellis_bf16": (C.c_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _u64, _u32, _u32, _u32, _u32, _u32]),
    "euhedral_b200_trellis_encode_tiles": (C.c_int, [_ptr, _u32, _u32, _ptr, _ptr, _ptr, _ptr, _u64]),
    "euhedral_b200_linear_trellis_scratch_bytes": (_u64, [_u32, _u32, _u32, _u32, _u32]),
    "euhedral_b200_linear_trellis_bf16": (C.c_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _u64, _u32, _u32, _u32, _u32, _u32, _u32]),
    "euhedral_b200_decode_plan": (C.c_int, [C.c_int, _u32, _u32, _u32, C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32),
                                            C.POINTER(_u32), C.POINTER(_u32)]),
    "euhedral_b200_linear_group_q3_bf16": (C.c_int, [_u32, C.POINTER(_ptr), C.POINTER(_ptr), C.POINTER(_ptr), _u32, _u32,
                                                     C.POINTER(_u32), C.POINTER(_u64)]),
    "euhedral_b200_linear_group_nvfp4_bf16": (C.c_int, [_u32, C.POINTER(_ptr), C.POINTER(_ptr), C.POINTER(_ptr), _u32, _u32,
                                                        C.POINTER(_u32), C.POINTER(_u64)]),
}

_LIB = None


class LibraryMissing(RuntimeError):
    pass


def load(path: Path | None = None) -> C.CDLL:
    """The bound library. Raises LibraryMissing when it has not been built (python -m euhedral_b200.build)."""
    global _LIB
    if _LIB is not None and path is None:
        return _LIB
    # EUHEDRAL_CUDA_LIBRARY names another build of the same library (e.g. one compiled with bounds checks).
    target = Path(path) if path else Path(os.environ.get("EUHEDRAL_CUDA_LIBRARY", LIBRARY_PATH))
    if not target.exists():
        raise LibraryMissing(f"{target} is missing: build it with `python -m euhedral_b200.build`; there is no CPU fallback")
    lib = C.CDLL(str(target))
    for name, (restype, argtypes) in SIGNATURES.items():
        function = getattr(lib, name)   # AttributeError when a declared symbol is not exported
        function.restype = restype
        function.argtypes = argtypes
    if path is None:
        _LIB = lib
    return lib


def decode_plan(fmt: str, rows: int, k: int, n: int) -> dict:
    """How a decode GEMV of this shape runs (format 'nvfp4' or 'q3'); host arithmetic only, works without a GPU.
    k_slices, pieces and piece_chunks fix the summation order and depend on the format and k alone."""
    out = [_u32() for _ in range(5)]
    status = load().euhedral_b200_decode_plan(0 if fmt == "nvfp4" else 1, rows, k, n, *[C.byref(v) for v in out])
    if status != 0:
        raise ValueError(f"no decode kernel takes rows={rows} k={k} n={n}")
    return {"k_slices": out[0].value, "pieces": out[1].value, "piece_chunks": out[2].value, "ctas": out[3].value,
            "shared_bytes": out[4].value}
