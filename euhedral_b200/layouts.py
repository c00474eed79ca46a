"""Byte geometry of the weight formats on the quantized-linear path (pure integer host logic).

NVFP4 `row-split-k128-v1`: core/.../artifact/Nvfp4Layout.java:32-66 and tools/euhedral_artifacts/nvfp4.py:49-57.
Q3G64_F16S `row-split-k128-v1`: tools/euhedral_artifacts/grouped.py:24-36 (core/.../artifact/CompactTensorLayout.java).
Trellis `trellis-tile16-v1`: core/.../artifact/TrellisLayout.java:12-52, core/.../artifact/format/TrellisFormat.java:98-115.
Native activation buffer: native/src/host/nvfp4_linear.c:252-265.
"""

from __future__ import annotations

NVFP4_BLOCK = 16
Q3_GROUP = 64
Q3_GROUP_BYTES = 24
TRELLIS_TILE = 16
TRELLIS_BLOCK = 128          # output columns per Hadamard block
SCRATCH_ALIGNMENT = 256


def align_up(value: int, unit: int) -> int:
    return (value + unit - 1) // unit * unit


def padded_k(k: int) -> int:
    return align_up(k, 128)


# ---- NVFP4 ---------------------------------------------------------------------------------------------------------

def nvfp4_scale_offset(n: int, k: int) -> int:
    return align_up(n * padded_k(k) // 2, 256)


def nvfp4_trailer_offset(n: int, k: int) -> int:
    return align_up(nvfp4_scale_offset(n, k) + n * padded_k(k) // NVFP4_BLOCK, 256)


def nvfp4_byte_size(n: int, k: int) -> int:
    return nvfp4_trailer_offset(n, k) + 4


def nvfp4_sd4_table_offset(n: int, k: int) -> int:
    """Table-indexed variant (row-split-k128-sd4-v1): the index plane (4 bits per block) starts where the scale plane
    would; the 16 E4M3 codes of the table and then the FP32 tensor scale follow it (nvfp4_linear.c:79-91)."""
    return align_up(nvfp4_scale_offset(n, k) + n * padded_k(k) // 32, 256)


def nvfp4_sd4_byte_size(n: int, k: int) -> int:
    return nvfp4_sd4_table_offset(n, k) + 20


def nvfp4_algorithmic_bytes(n: int, k: int) -> int:
    """Planes only, no alignment padding: 0.5625 B per weight + the FP32 scale."""
    return n * padded_k(k) // 2 + n * padded_k(k) // 16 + 4


# ---- Q3G64_F16S ----------------------------------------------------------------------------------------------------

def q3_groups(k: int) -> int:
    return padded_k(k) // Q3_GROUP


def q3_scale_offset(n: int, k: int) -> int:
    return align_up(n * q3_groups(k) * Q3_GROUP_BYTES, 256)


def q3_byte_size(n: int, k: int) -> int:
    return q3_scale_offset(n, k) + n * q3_groups(k) * 2


def q3_algorithmic_bytes(n: int, k: int) -> int:
    return n * q3_groups(k) * (Q3_GROUP_BYTES + 2)


# ---- trellis -------------------------------------------------------------------------------------------------------

def trellis_words_valid(w: int) -> bool:
    return 16 <= w <= 128 and w % 8 == 0


def trellis_payload_shape(n: int, k: int, w: int) -> tuple[int, int, int]:
    if n % TRELLIS_BLOCK or k % TRELLIS_BLOCK or not trellis_words_valid(w):
        raise ValueError(f"not a trellis object: n={n} k={k} w={w}")
    return k // TRELLIS_TILE, n // TRELLIS_TILE, w


def trellis_byte_size(n: int, k: int, w: int) -> int:
    kt, nt, w = trellis_payload_shape(n, k, w)
    return kt * nt * w * 2


def trellis_algorithmic_bytes(n: int, k: int, w: int, segments: int) -> int:
    """Payload + suh + svh + segment ends."""
    return trellis_byte_size(n, k, w) + 2 * segments * k + 2 * n + 4 * segments


def trellis_validate_segments(ends, n: int) -> None:
    """Segment ends: ascending multiples of 128, the last one n, at most 8 (TrellisFormatTest.java:116-141)."""
    ends = list(ends)
    if not ends or len(ends) > 8 or ends[-1] != n:
        raise ValueError(f"segment ends {ends} do not cover {n} columns")
    previous = 0
    for end in ends:
        if end <= previous or end % TRELLIS_BLOCK:
            raise ValueError(f"segment ends {ends} are not ascending multiples of {TRELLIS_BLOCK}")
        previous = end


# ---- native activation buffer ---------------------------------------------------------------------------------------

def activation_bytes(rows: int, k: int, terms: int = 2) -> int:
    kp = padded_k(k)
    pad = align_up(rows, 128)
    scale_offset = align_up(rows * terms * kp // 2, 256)
    global_offset = align_up(scale_offset + kp // 128 * terms * pad * 8, 256)
    return global_offset + 4 * rows
