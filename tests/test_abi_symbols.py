"""The C ABI library loads without a GPU, exports every symbol include/euhedral_cuda.h declares, and its pure
host-side entry points (no device work) behave: table names, decode plans, scratch sizes, argument validation."""

import ctypes as C
import re
from pathlib import Path

import pytest

from euhedral_b200 import layouts, library

HEADER = Path(__file__).resolve().parents[1] / "include" / "euhedral_cuda.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return re.findall(r"EUHEDRAL_CUDA_EXPORT\s+[\w\s\*]+?\b(euhedral_\w+)\s*\(", text)


def test_every_declared_symbol_is_exported_and_bound():
    lib = library.load()
    names = declared_symbols()
    assert len(names) >= 35
    for name in names:
        assert hasattr(lib, name), name
    assert set(names) == set(library.SIGNATURES), set(names) ^ set(library.SIGNATURES)


def test_kernel_table_order_is_the_reference_abi():
    lib = library.load()
    # native/src/host/linear_kernels.c:7-24; Java mirror core/.../artifact/format/LinearKernel.java:8-34
    expect = ["euhedral_trellis_prepass", "euhedral_trellis_mma", "euhedral_trellis_mma_rows", "euhedral_trellis_mma_rows64",
              "euhedral_trellis_epilogue", "euhedral_trellis_decode_bf16", "euhedral_trellis_epilogue_bf16", "euhedral_trellis_reference",
              "euhedral_trellis_mma_rows_fp8", "euhedral_trellis_mma_rows64_fp8", "euhedral_nvfp4_embedding"]
    assert lib.euhedral_cuda_linear_kernel_count() == len(expect)
    assert [lib.euhedral_cuda_linear_kernel_name(i).decode() for i in range(len(expect))] == expect
    assert lib.euhedral_cuda_linear_kernel_name(99) is None


def test_argument_validation_needs_no_device():
    lib = library.load()
    assert lib.euhedral_cuda_linear_nvfp4_bf16(None, None, None, 1, 128, 16, 0) == library.INVALID_ARGUMENT
    assert lib.euhedral_cuda_linear_nvfp4_bf16(16, 16, 16, 1, 128, 16, 12345) == library.FORMAT_MISMATCH
    assert lib.euhedral_cuda_linear_q3_bf16(16, 16, 16, 1, 128, 16, 12345) == library.FORMAT_MISMATCH
    assert lib.euhedral_cuda_linear_q3_bf16(16, 16, 16, 0, 128, 16, 12345) == library.INVALID_ARGUMENT
    assert lib.euhedral_cuda_stream_select(0) == library.INVALID_ARGUMENT
    assert lib.euhedral_cuda_set_include_directory(None) == library.INVALID_ARGUMENT
    assert lib.euhedral_cuda_set_include_directory(b"/usr/include") == 0
    words, sizes = (C.c_uint64 * 1)(), (C.c_uint8 * 1)()
    assert lib.euhedral_cuda_linear_launch(99, 1, 1, 1, 1, 1, 1, 0, words, sizes, 0) == library.INVALID_ARGUMENT
    assert lib.euhedral_cuda_linear_launch(1, 0, 1, 1, 1, 1, 1, 0, words, sizes, 0) == library.INVALID_ARGUMENT
    assert lib.euhedral_cuda_select_exact_numerics(1) == 0 and lib.euhedral_cuda_select_exact_numerics(0) == 1
    assert lib.euhedral_b200_static_scratch_bytes() == 8 << 20


def test_decode_plans_depend_on_k_only_for_the_summation_order():
    plans = {}
    for n in (128, 640, 1024, 5120, 17408):
        for rows in (1, 5, 8):
            for fmt in ("nvfp4", "q3"):
                if (fmt, rows) == ("nvfp4", 8):
                    continue   # 8 rows of K = 5120 do not fit beside the NVFP4 rings: such a call runs as two groups of 4
                plan = library.decode_plan(fmt, rows, 5120, n)
                plans.setdefault(fmt, set()).add((plan["k_slices"], plan["pieces"], plan["piece_chunks"]))
                assert plan["ctas"] % plan["k_slices"] == 0 and 1 <= plan["ctas"] <= 148
                assert plan["shared_bytes"] <= 227 * 1024
    assert all(len(v) == 1 for v in plans.values())      # a row's K order is the same whatever the shard's N and the row count
    assert library.decode_plan("nvfp4", 1, 17408, 5120)["k_slices"] == 4
    assert library.decode_plan("q3", 3, 5120, 17408)["k_slices"] == 1
    with pytest.raises(ValueError):
        library.decode_plan("nvfp4", 1, 100, 16)
    with pytest.raises(ValueError):
        library.decode_plan("q3", 9, 1024, 16)


def test_native_scratch_covers_every_region():
    lib = library.load()
    for rows, k, n in ((16, 256, 128), (4096, 5120, 17408), (300, 5120, 1024)):
        need = lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, k, n)
        codes = layouts.align_up(2 * rows * k // 2, 256)
        atoms_a = -(-rows // 128) * (k // 64) * 2 * 512
        atoms_b = -(-n // 256) * 2 * (k // 64) * 512
        fixed = layouts.align_up(layouts.align_up(layouts.align_up(codes + atoms_a, 256) + 4 * rows, 256) + atoms_b, 256)
        # calls of at most 64 rows may cut K over up to 8 CTAs per output tile: FP32 partial tiles follow
        assert need == fixed + (8 * rows * n * 4 if rows <= 64 else 0)


def test_decode_plans_stay_launchable_and_cut_k_by_k_alone():
    """Host arithmetic only: whatever the shape, a CTA count is a whole number of clusters, the cut of K depends on the
    format and K alone, every piece fits the instantiated kernels and the shared-memory request stays launchable."""
    rng = __import__("numpy").random.default_rng(7)
    cuts = {}
    shapes = [(16, 128), (48, 4352), (1024, 5120), (5120, 5120), (17408, 5120), (5120, 17408), (151936, 5120), (248320, 2048),
              (2000, 1536), (9232, 8192), (640, 14336)]
    shapes += [(16 * int(rng.integers(1, 3000)), 128 * int(rng.integers(1, 200))) for _ in range(40)]
    for n, k in shapes:
        for fmt in ("nvfp4", "q3"):
            for rows in (1, 3, 8):
                try:
                    plan = library.decode_plan(fmt, rows, k, n)
                except ValueError:
                    continue   # the caller halves the row group, or the scalar kernel takes the shape
                clusters, rest = divmod(plan["ctas"], plan["k_slices"])
                assert rest == 0 and clusters >= 1
                assert plan["k_slices"] in (1, 2, 4, 8) and plan["pieces"] in (1, 2, 4, 8, 16)
                chunks = k // 128
                assert plan["pieces"] * plan["piece_chunks"] * plan["k_slices"] >= chunks
                assert plan["piece_chunks"] <= (4 if fmt == "nvfp4" else 5)
                assert plan["shared_bytes"] <= 227 * 1024
                cut = (plan["k_slices"], plan["pieces"], plan["piece_chunks"])
                assert cuts.setdefault((fmt, k), cut) == cut


def test_prefill_entry_points_validate_without_a_device():
    lib = library.load()
    # sizes are pure arithmetic
    assert lib.euhedral_cuda_q3_mx_scratch_bytes(4096, 5120, 17408) == 17408 * 5120 * 4
    assert lib.euhedral_b200_prefill_trellis_scratch_bytes(100, 256, 384, 2) == 2 * 100 * 256 * 2 + 384 * 256 * 2
    assert lib.euhedral_b200_prefill_trellis_scratch_bytes(3, 128, 128, 1) == 768 + 32768      # each region rounded up to 256 bytes
    # argument checks come before any device work
    assert lib.euhedral_cuda_linear_q3_mx_bf16(None, 16, 16, 256, 40, 128, 128, 1, 1 << 20) == library.INVALID_ARGUMENT
    assert lib.euhedral_cuda_linear_q3_mx_bf16(16, 16, 16, 256, 40, 128, 128, 12345, 1 << 20) == library.FORMAT_MISMATCH
    size = layouts.q3_byte_size(128, 128)
    assert lib.euhedral_cuda_linear_q3_mx_bf16(16, 16, 16, 256, 40, 128, 128, size, 16) == library.SIZE_OVERFLOW
    assert lib.euhedral_cuda_linear_q3_mx_bf16(16, 16, 16, 256, 32, 128, 128, size, 1 << 20) == library.ROUTE_UNAVAILABLE   # few rows: the decode kernels
    assert lib.euhedral_cuda_linear_q3_mx_bf16(16, 16, 16, 128, 40, 128, 128, size, 1 << 20) == library.ROUTE_UNAVAILABLE   # scratch not 256-aligned
    assert lib.euhedral_cuda_q3_mx_gate_up_swiglu_bf16(16, 16, 16, 256, 40, 128, 129, size, 1 << 20) == library.INVALID_ARGUMENT
    ends = (C.c_int32 * 1)(256)
    host = C.cast(ends, C.c_void_p)
    assert lib.euhedral_b200_prefill_trellis_bf16(256, 256, 256, 256, 256, host, 256, 256, 1 << 30, 4, 256, 200, 48, 1) == library.ROUTE_UNAVAILABLE
    assert lib.euhedral_b200_prefill_trellis_bf16(256, 256, 256, 256, 256, host, 256, 256, 1 << 30, 4, 256, 384, 48, 1) == library.INVALID_ARGUMENT
    assert lib.euhedral_b200_prefill_trellis_bf16(256, 256, 256, 256, 256, host, 256, 256, 16, 4, 256, 256, 48, 1) == library.SIZE_OVERFLOW
    assert lib.euhedral_b200_linear_bf16(16, 16, 16, 4, 96, 128) == library.ROUTE_UNAVAILABLE
    assert lib.euhedral_b200_linear_bf16(16, 16, 18, 4, 64, 128) == library.INVALID_ARGUMENT
    assert lib.euhedral_b200_trellis_encode_tiles(None, 1, 48, 16, None, None, 16, 1 << 20) == library.INVALID_ARGUMENT
    assert lib.euhedral_b200_trellis_encode_tiles(16, 1, 72, 16, None, None, 16, 1 << 20) == library.ROUTE_UNAVAILABLE
    lib.euhedral_cuda_q3_mx_select_split_rows(17408)      # accepted, no effect
    lib.euhedral_cuda_q3_mx_select_split_rows(0)


def test_operators_route_by_row_count(monkeypatch):
    """CudaGpuMemory.linear_q3_bf16 and TrellisFormat.linear pick the prefill entries by row count (the reference's
    linearQ3Bf16 and TrellisFormat.linear), shown with a library that only records what was called."""
    from euhedral_b200 import gpu as G
    from euhedral_b200.formats import LinearLaunch, TensorHandle, TrellisFormat, TrellisSettings
    calls = []

    class Recorder:
        def __getattr__(self, name):
            def call(*args):
                calls.append((name, args))
                if name == "euhedral_cuda_q3_mx_available":
                    return 1
                if name.endswith("scratch_bytes"):
                    return 4096
                if name == "euhedral_cuda_malloc":
                    args[1]._obj.value = 0x10000
                    return 0
                return 0
            return call

    memory = G.CudaGpuMemory.__new__(G.CudaGpuMemory)
    memory.lib, memory._native_scratch, memory._native_scratch_bytes = Recorder(), 0x10000, 1 << 20
    memory.linear_q3_bf16(16, 32, 48, 8, 256, 256, 99)
    assert [name for name, _ in calls] == ["euhedral_cuda_linear_q3_bf16"]          # 8 rows: the decode entry
    calls.clear()
    memory.linear_q3_bf16(16, 32, 48, 9, 256, 256, 99)
    assert "euhedral_cuda_linear_q3_mx_bf16" in [name for name, _ in calls] and "euhedral_cuda_linear_q3_bf16" not in [name for name, _ in calls]
    calls.clear()
    memory._row_exact = True
    memory.linear_q3_bf16(16, 32, 48, 9, 256, 256, 99)
    assert [name for name, _ in calls] == ["euhedral_cuda_linear_q3_bf16"]          # row-exact launches stay on the decode kernels
    memory._row_exact = False
    calls.clear()
    fmt = TrellisFormat(TrellisSettings(target_ctas=148))
    handles = [TensorHandle("p", (16, 16, 48), 0x1000, 16 * 16 * 96), TensorHandle("suh", (1, 256), 0x2000, 512),
               TensorHandle("svh", (256,), 0x3000, 512), TensorHandle("ends", (1,), 0x4000, 4)]
    fmt.linear(memory, LinearLaunch(0x5000, 0x6000, handles, 600, 256, 256, scratch=0x7000, scratch_bytes=1 << 20, segment_ends=[256]))
    assert [name for name, _ in calls][-1] == "euhedral_b200_prefill_trellis_bf16"
    calls.clear()
    fmt.linear(memory, LinearLaunch(0x5000, 0x6000, handles, 64, 256, 256, scratch=0x7000, scratch_bytes=1 << 20))   # one segment: ends = [n]
    assert [name for name, _ in calls][-1] == "euhedral_b200_prefill_trellis_bf16"
    calls.clear()
    fmt.linear(memory, LinearLaunch(0x5000, 0x6000, handles, 63, 256, 256, scratch=0x7000, scratch_bytes=1 << 20))
    assert "euhedral_b200_prefill_trellis_bf16" not in [name for name, _ in calls]
    assert [name for name, _ in calls].count("euhedral_cuda_linear_launch") >= 2                                      # prepass + mma
