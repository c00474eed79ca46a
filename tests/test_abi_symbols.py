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
