"""CPU restatement (NumPy) of the reference's quantized-linear arithmetic. TEST INFRASTRUCTURE ONLY.

This module is the parity checker for the CUDA kernels. Nothing on the product path imports it: only the
test-suite, the smoke check and the CPU-baseline leg of the benchmark do. Every function names the reference
source it restates (paths are relative to the reference project root).

Pinned against: the reference's Python converter and NumPy trellis decoder run on seeded inputs (fixtures under
tests/golden, produced by tests/golden/make_golden.py) and the reference's own golden files (GPTQ decode fixtures,
trellis tile fixtures). The prefill activation quantizer (`quantize_activations`) restates CUDA conversion
intrinsics for which the reference holds no vector; it is pinned on the GPU instead, bit for bit, against the
reference's own quantize_rows kernel compiled for sm_100a (oracle/make_ref_quantize.py, tests/test_ref_quantize_gpu.py).
"""

from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------------------------------------------
# Small-float helpers
# --------------------------------------------------------------------------------------------------------------

E2M1_MAGNITUDES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def e4m3_value(codes) -> np.ndarray:
    """Unsigned E4M3 (bias 7, subnormals, bit 7 ignored) -> float32. tools/euhedral_artifacts/nvfp4.py:25-28
    tabulates the same 127 values; native/src/nvfp4/nvfp4.cuh:60-62 decodes them the same way on the device."""
    c = np.asarray(codes).astype(np.int64) & 0x7F
    exponent, mantissa = c >> 3, c & 7
    normal = np.ldexp(1.0 + mantissa / 8.0, exponent - 7)
    subnormal = np.ldexp(mantissa / 8.0, -6)
    return np.where(exponent == 0, subnormal, normal).astype(np.float32)


def e4m3_encode(values) -> np.ndarray:
    """Nearest unsigned E4M3 code (0..126) of non-negative float32 values, ties to the even code, saturating at
    448. Same result as the table search of tools/euhedral_artifacts/nvfp4.py:72-82 over its 127-entry table, here
    computed arithmetically."""
    v = np.asarray(values, dtype=np.float64)
    out = np.zeros(v.shape, dtype=np.int64)
    tiny = v < 2.0 ** -6
    # Subnormal range: steps of 2^-9; rint is ties-to-even and code parity equals mantissa parity.
    out[tiny] = np.rint(v[tiny] * 512.0).astype(np.int64)
    big = ~tiny
    mant, exp2 = np.frexp(v[big])  # v = mant * 2^exp2, mant in [0.5, 1)
    e = exp2.astype(np.int64) - 1
    q = np.rint(np.ldexp(v[big], 3 - e)).astype(np.int64)  # 8..16
    carry = q == 16
    e = e + carry
    q = np.where(carry, 8, q)
    out[big] = (e + 7) * 8 + (q - 8)
    return np.clip(out, 0, 126).astype(np.uint8)


def e2m1_encode_magnitude(values) -> np.ndarray:
    """Index (0..7) of the nearest E2M1 magnitude of non-negative values, ties to the even index, saturating at 6.
    Same result as tools/euhedral_artifacts/nvfp4.py:72-82 over E2M1_VALUES."""
    v = np.asarray(values, dtype=np.float32)
    index = np.zeros(v.shape, dtype=np.uint8)
    # (midpoint between index i and i + 1, True when the tie goes up, i.e. i + 1 is even)
    for i, (mid, tie_up) in enumerate([(0.25, False), (0.75, True), (1.25, False), (1.75, True),
                                       (2.5, False), (3.5, True), (5.0, False)]):
        above = (v >= np.float32(mid)) if tie_up else (v > np.float32(mid))
        index[above] = i + 1
    return index


def bf16_bits(values) -> np.ndarray:
    """float32 -> BF16 bit patterns, round to nearest even by integer arithmetic (native/src/q3/numeric.cuh:17-21)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_to_f32(bits) -> np.ndarray:
    return (np.asarray(bits).astype(np.uint32) << 16).view(np.float32)


def round_bf16(values) -> np.ndarray:
    return bf16_to_f32(bf16_bits(values))


def align_up(value: int, unit: int) -> int:
    return (value + unit - 1) // unit * unit


# --------------------------------------------------------------------------------------------------------------
# NVFP4 (layout row-split-k128-v1)
# --------------------------------------------------------------------------------------------------------------

def nvfp4_offsets(n: int, k: int) -> tuple[int, int, int]:
    """(scale plane offset, global scale offset, byte size). tools/euhedral_artifacts/nvfp4.py:49-57,
    core/.../artifact/Nvfp4Layout.java:32-66, native/src/host/nvfp4_linear.c:79-91."""
    kp = align_up(k, 128)
    scale_off = align_up(n * kp // 2, 256)
    global_off = align_up(scale_off + n * kp // 16, 256)
    return scale_off, global_off, global_off + 4


def nvfp4_global_scale(amax: float) -> np.float32:
    """tools/euhedral_artifacts/nvfp4.py:85-86 (Java twin: quantization/.../mtp/Nvfp4Rounding.java divides by 2688f)."""
    return np.float32(np.float32(amax) / np.float32(2688.0))


def nvfp4_quantize_rows(values: np.ndarray, global_scale: np.float32):
    """float32 [rows, K] (K % 16 == 0) -> (packed codes u8 [rows, K/2], E4M3 scales u8 [rows, K/16]).
    tools/euhedral_artifacts/nvfp4.py:89-105: block scale = fp32(fp32(amax / 6) / global), nearest E4M3; code =
    nearest E2M1 of |v| / fp32(e4m3 * global); sign bit only on a nonzero magnitude; even K in the low nibble."""
    values = np.ascontiguousarray(values, dtype=np.float32)
    rows, k = values.shape
    blocks = values.reshape(rows, k // 16, 16)
    g = np.float32(global_scale)
    if g > 0:
        amax = np.abs(blocks).max(axis=2)
        ratio = ((amax / np.float32(6.0)).astype(np.float32) / g).astype(np.float32)
    else:
        ratio = np.zeros(blocks.shape[:2], dtype=np.float32)
    scales = e4m3_encode(ratio)
    step = (e4m3_value(scales) * g).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        scaled = np.where(step[..., None] > 0, np.abs(blocks) / step[..., None], np.float32(0)).astype(np.float32)
    mag = e2m1_encode_magnitude(scaled)
    code = (mag | (((blocks < 0) & (mag > 0)).astype(np.uint8) << 3)).reshape(rows, k)
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).astype(np.uint8)
    return packed, scales


def nvfp4_pack(weights: np.ndarray) -> bytes:
    """A whole NVFP4 tensor as the converter writes it (tools/euhedral_artifacts/nvfp4.py:226-266, no calibration):
    K padded with zeros to 128, global = amax / 2688."""
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    n, k = weights.shape
    kp = align_up(k, 128)
    if kp != k:
        padded = np.zeros((n, kp), dtype=np.float32)
        padded[:, :k] = weights
        weights = padded
    g = nvfp4_global_scale(float(np.abs(weights).max()))
    packed, scales = nvfp4_quantize_rows(weights, g)
    scale_off, global_off, size = nvfp4_offsets(n, k)
    blob = bytearray(size)
    blob[:packed.size] = packed.tobytes()
    blob[scale_off:scale_off + scales.size] = scales.tobytes()
    blob[global_off:global_off + 4] = np.float32(g).astype("<f4").tobytes()
    return bytes(blob)


def nvfp4_unpack(blob: bytes, n: int, k: int):
    """(codes u8 [n, Kp] one E2M1 code per entry, scales u8 [n, Kp/16], global float32) of a tensor's bytes."""
    kp = align_up(k, 128)
    scale_off, global_off, size = nvfp4_offsets(n, k)
    assert len(blob) == size, (len(blob), size)
    raw = np.frombuffer(blob, dtype=np.uint8)
    packed = raw[:n * kp // 2].reshape(n, kp // 2)
    codes = np.empty((n, kp), dtype=np.uint8)
    codes[:, 0::2] = packed & 15
    codes[:, 1::2] = packed >> 4
    scales = raw[scale_off:scale_off + n * kp // 16].reshape(n, kp // 16)
    g = np.frombuffer(blob[global_off:global_off + 4], dtype="<f4")[0]
    return codes, scales, np.float32(g)


def nvfp4_dequantize(codes: np.ndarray, scales: np.ndarray, global_scale: np.float32) -> np.ndarray:
    """Dense float32 weights: fp32(e2m1 * sign) * fp32(e4m3 * global) (tools/euhedral_artifacts/nvfp4.py:108-115).
    This product order defines "dequantised weights bit-exact"."""
    signed = E2M1_MAGNITUDES[codes & 7] * np.where(codes & 8, np.float32(-1), np.float32(1))
    block = np.repeat((e4m3_value(scales) * np.float32(global_scale)).astype(np.float32), 16, axis=1)
    return (signed * block).astype(np.float32)


def nvfp4_dense(blob: bytes, n: int, k: int) -> np.ndarray:
    codes, scales, g = nvfp4_unpack(blob, n, k)
    return nvfp4_dequantize(codes, scales, g)[:, :k]


# NVFP4 with table-indexed block scales (layout row-split-k128-sd4-v1): the scale plane holds 4-bit indices, two per byte
# with the even block in the low nibble, into 16 E4M3 codes that follow the index plane; then the FP32 tensor scale.

def nvfp4_sd4_offsets(n: int, k: int) -> tuple[int, int, int]:
    """(index plane offset, table offset, byte size). tools/euhedral_artifacts/nvfp4.py:60-69,
    native/src/host/nvfp4_linear.c:79-91."""
    kp = align_up(k, 128)
    index_off = align_up(n * kp // 2, 256)
    table_off = align_up(index_off + n * kp // 32, 256)
    return index_off, table_off, table_off + 16 + 4


def nvfp4_sd4_to_plain(blob: bytes, n: int, k: int) -> bytes:
    """The same tensor in the plain layout (every block's table entry written out as its E4M3 scale byte,
    tools/euhedral_artifacts/nvfp4.py:217-223), so that every function above applies to it. The values are the same bit
    for bit: a block's scale IS its table entry."""
    kp = align_up(k, 128)
    index_off, table_off, size = nvfp4_sd4_offsets(n, k)
    assert len(blob) == size, (len(blob), size)
    raw = np.frombuffer(bytes(blob), dtype=np.uint8)
    packed = raw[index_off:index_off + n * kp // 32].reshape(n, kp // 32)
    indices = np.empty((n, kp // 16), dtype=np.uint8)
    indices[:, 0::2] = packed & 15
    indices[:, 1::2] = packed >> 4
    scales = raw[table_off:table_off + 16][indices]
    scale_off, global_off, plain_size = nvfp4_offsets(n, k)
    plain = bytearray(plain_size)
    plain[:n * kp // 2] = raw[:n * kp // 2].tobytes()
    plain[scale_off:scale_off + scales.size] = scales.tobytes()
    plain[global_off:global_off + 4] = raw[table_off + 16:table_off + 20].tobytes()
    return bytes(plain)


def nvfp4_sd4_dense(blob: bytes, n: int, k: int) -> np.ndarray:
    return nvfp4_dense(nvfp4_sd4_to_plain(blob, n, k), n, k)


def nvfp4_sd4_from_plain(blob: bytes, n: int, k: int, rng) -> bytes:
    """A valid table-indexed tensor for kernel tests, made from a plain one without the converter's table search: sixteen of
    the scale codes the tensor uses become the table (the smallest, the largest and random ones between), every block takes
    the nearest table entry; the E2M1 codes stay. Not what the converter would choose - the kernels only decode."""
    kp = align_up(k, 128)
    scale_off, global_off, _ = nvfp4_offsets(n, k)
    raw = np.frombuffer(bytes(blob), dtype=np.uint8)
    scales = raw[scale_off:scale_off + n * kp // 16].reshape(n, kp // 16)
    used = np.unique(scales)
    if len(used) > 16:
        inner = rng.choice(used[1:-1], size=14, replace=False)
        table = np.sort(np.concatenate([[used[0], used[-1]], inner])).astype(np.uint8)
    else:
        table = np.sort(np.concatenate([used, np.setdiff1d(np.arange(127, dtype=np.uint8), used)[:16 - len(used)]])).astype(np.uint8)
    values = e4m3_value(table)
    nearest = np.abs(e4m3_value(scales)[..., None] - values[None, None, :]).argmin(axis=2).astype(np.uint8)
    index_off, table_off, size = nvfp4_sd4_offsets(n, k)
    out = bytearray(size)
    out[:n * kp // 2] = raw[:n * kp // 2].tobytes()
    out[index_off:index_off + n * kp // 32] = (nearest[:, 0::2] | (nearest[:, 1::2] << 4)).astype(np.uint8).tobytes()
    out[table_off:table_off + 16] = table.tobytes()
    out[table_off + 16:table_off + 20] = raw[global_off:global_off + 4].tobytes()
    return bytes(out)


def nvfp4_unscaled(blob: bytes, n: int, k: int):
    """(e2m1 * e4m3 per weight as float32 [n, k] - exact -, global): what the kernels sum before applying the global
    scale to the sum (native/src/nvfp4/nvfp4.cuh:97-198, native/src/reference/kernels.cu:125-149)."""
    codes, scales, g = nvfp4_unpack(blob, n, k)
    signed = E2M1_MAGNITUDES[codes & 7] * np.where(codes & 8, np.float32(-1), np.float32(1))
    return (signed * np.repeat(e4m3_value(scales), 16, axis=1))[:, :k].astype(np.float32), g


# --------------------------------------------------------------------------------------------------------------
# Q3G64_F16S (layout row-split-k128-v1)
# --------------------------------------------------------------------------------------------------------------

def q3_offsets(n: int, k: int) -> tuple[int, int]:
    """(scale plane offset, byte size). tools/euhedral_artifacts/grouped.py:24-36; native/src/host/q3_linear_bf16.c:82-84."""
    groups = align_up(k, 128) // 64
    scale_off = align_up(n * groups * 24, 256)
    return scale_off, scale_off + n * groups * 2


def q3_quantize(weights: np.ndarray):
    """float32 [n, K] -> (codes int8 [n, Kp] in -4..3, scales float16 [n, Kp/64]). Round-to-nearest path of
    tools/euhedral_artifacts/grouped.py:39-51,129-135: scale = f16(f32(f64(max|v|) / 3)), 2^-24 if that underflows on
    a nonzero group; code = clip(rint(v * f32(1 / f64(scale))), -4, 3)."""
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    n, k = weights.shape
    kp = align_up(k, 128)
    if kp != k:
        padded = np.zeros((n, kp), dtype=np.float32)
        padded[:, :k] = weights
        weights = padded
    grouped = weights.reshape(n, kp // 64, 64)
    amax = np.abs(grouped).max(axis=2)
    scales = (amax.astype(np.float64) / 3.0).astype(np.float32).astype(np.float16)
    scales = np.where((scales == 0) & (amax > 0), np.float16(2.0 ** -24), scales)
    inverse = np.zeros(amax.shape, dtype=np.float32)
    positive = scales > 0
    inverse[positive] = (1.0 / scales[positive].astype(np.float64)).astype(np.float32)
    codes = np.clip(np.rint(grouped * inverse[..., None]), -4, 3).astype(np.int8)
    return codes.reshape(n, kp), scales


def q3_pack_codes(codes: np.ndarray) -> np.ndarray:
    """int8 [n, Kp] -> u8 [n, Kp/64*24]: code i of a group at bits [3i, 3i+3) of its 24-byte little-endian stream
    (tools/euhedral_artifacts/grouped.py:54-66)."""
    n, kp = codes.shape
    fields = (codes.astype(np.int16) & 7).astype(np.uint8).reshape(n, kp // 64, 64)
    bits = np.zeros((n, kp // 64, 64, 3), dtype=np.uint8)
    for b in range(3):
        bits[..., b] = (fields >> b) & 1
    # LSB-first bit stream -> bytes
    return np.packbits(bits.reshape(n, kp // 64, 192), axis=2, bitorder="little").reshape(n, kp // 64 * 24)


def q3_pack(weights: np.ndarray) -> bytes:
    n, k = weights.shape
    codes, scales = q3_quantize(weights)
    return q3_assemble(codes, scales, n, k)


def q3_assemble(codes: np.ndarray, scales: np.ndarray, n: int, k: int) -> bytes:
    scale_off, size = q3_offsets(n, k)
    blob = bytearray(size)
    packed = q3_pack_codes(codes)
    blob[:packed.size] = packed.tobytes()
    blob[scale_off:] = np.ascontiguousarray(scales.astype("<f2")).tobytes()
    return bytes(blob)


def q3_unpack(blob: bytes, n: int, k: int):
    """(codes int8 [n, Kp], scales float16 [n, Kp/64])."""
    kp = align_up(k, 128)
    groups = kp // 64
    scale_off, size = q3_offsets(n, k)
    assert len(blob) == size, (len(blob), size)
    raw = np.frombuffer(blob, dtype=np.uint8)
    stream = np.unpackbits(raw[:n * groups * 24].reshape(n, groups, 24), axis=2, bitorder="little")
    fields = stream.reshape(n, groups, 64, 3)
    unsigned = fields[..., 0] | (fields[..., 1] << 1) | (fields[..., 2] << 2)
    codes = unsigned.astype(np.int8) - ((unsigned >= 4).astype(np.int8) << 3)
    scales = np.frombuffer(blob[scale_off:scale_off + n * groups * 2], dtype="<f2").reshape(n, groups)
    return codes.reshape(n, kp), scales


def q3_dense(blob: bytes, n: int, k: int) -> np.ndarray:
    """Dense float32 weights code * f32(scale); exact (native/src/reference/kernels.cu:27-41)."""
    codes, scales = q3_unpack(blob, n, k)
    return (codes.astype(np.float32) * np.repeat(scales.astype(np.float32), 64, axis=1))[:, :k]


# --------------------------------------------------------------------------------------------------------------
# Linear references
# --------------------------------------------------------------------------------------------------------------

def linear_f64(x_bits: np.ndarray, dense: np.ndarray) -> np.ndarray:
    """y = x . W^T in float64 from BF16 activations (bit patterns [rows, K]) and dense float32 weights [N, K]."""
    return bf16_to_f32(x_bits).astype(np.float64) @ dense.astype(np.float64).T


def linear_f32(x_bits: np.ndarray, dense: np.ndarray) -> np.ndarray:
    """FP32-accumulated reference (float32 GEMM)."""
    return bf16_to_f32(x_bits) @ np.ascontiguousarray(dense, dtype=np.float32).T


def nvfp4_linear_scalar_kernel(x_bits: np.ndarray, blob: bytes, n: int, k: int) -> np.ndarray:
    """BF16 bits of the scalar device oracle's output, in its own summation order: 128 partial sums (element k goes
    to partial k % 128, fused multiply-add), a 7-step pairwise tree, times the global scale, BF16
    (native/src/reference/kernels.cu:81-91,125-149). Vectorised over outputs; float64 emulation of fmaf is exact here
    because x * w has at most 14 significant bits."""
    w, g = nvfp4_unscaled(blob, n, k)
    x = bf16_to_f32(x_bits)
    rows = x.shape[0]
    out = np.zeros((rows, n), dtype=np.uint16)
    for r in range(rows):
        partial = np.zeros((n, 128), dtype=np.float32)
        for k0 in range(0, k, 128):
            width = min(128, k - k0)
            prod = (w[:, k0:k0 + width].astype(np.float64) * x[r, k0:k0 + width].astype(np.float64))
            partial[:, :width] = (partial[:, :width].astype(np.float64) + prod).astype(np.float32)
        stride = 64
        while stride:
            partial[:, :stride] = partial[:, :stride] + partial[:, stride:2 * stride]
            stride >>= 1
        out[r] = bf16_bits(partial[:, 0] * g)
    return out


def q3_linear_scalar_kernel(x_bits: np.ndarray, blob: bytes, n: int, k: int) -> np.ndarray:
    """BF16 bits of the scalar Q3 device oracle: sum += (x * code) * scale without fusing, strided by 128 threads,
    pairwise tree (native/src/reference/kernels.cu:17-48)."""
    codes, scales = q3_unpack(blob, n, k)
    scale = np.repeat(scales.astype(np.float32), 64, axis=1)
    x = bf16_to_f32(x_bits)
    rows = x.shape[0]
    out = np.zeros((rows, n), dtype=np.uint16)
    for r in range(rows):
        partial = np.zeros((n, 128), dtype=np.float32)
        for k0 in range(0, k, 128):
            width = min(128, k - k0)
            term = (x[r, k0:k0 + width][None, :] * codes[:, k0:k0 + width].astype(np.float32)).astype(np.float32)
            term = (term * scale[:, k0:k0 + width]).astype(np.float32)
            partial[:, :width] = partial[:, :width] + term
        stride = 64
        while stride:
            partial[:, :stride] = partial[:, :stride] + partial[:, stride:2 * stride]
            stride >>= 1
        out[r] = bf16_bits(partial[:, 0])
    return out


# --------------------------------------------------------------------------------------------------------------
# Trellis (layout trellis-tile16-v1): payload int16 [K/16, N/16, w]
# --------------------------------------------------------------------------------------------------------------

INV_SQRT_128 = np.float32(0.08838834764831845)


def trellis_window_ends(w: int) -> np.ndarray:
    """Ring bit at which the 16-bit window of each of the 256 positions of a tile ends:
    S(p) = (p >> 4) * w + sum_{j <= p & 15} (w // 16 + halfstep(j)), halfstep(j) = 1 on odd j when w % 16 == 8
    (native/src/trellis/codebook.cuh:40-49)."""
    p = np.arange(256)
    m = p & 15
    whole = w // 16
    odd_bits = (m + 1) // 2 if w % 16 == 8 else 0  # odd j in 0..m
    return (p >> 4) * w + whole * (m + 1) + odd_bits


def trellis_decode_tiles(words: np.ndarray, w: int) -> np.ndarray:
    """int16 words [tiles, w] -> float16 [tiles, 256] in tensor-core position order. The ring is read MSB first from
    uint32 words formed of little-endian int16 pairs; the value is one FP16 fma of (0x6400 + byte sum of
    state * 0x83DCD12D) with constants 0x1EEE, 0xC931 (native/src/trellis/codebook.cuh:18-37,51-61; NumPy twin
    native/tests/trellis_reference.py:20-33). Implemented over an explicit bit array."""
    words = np.ascontiguousarray(words, dtype="<i2").reshape(-1, w)
    tiles = words.shape[0]
    u32 = words.view("<u4")  # [tiles, w/2]
    # MSB-first bits of each uint32, words in order.
    bits = np.unpackbits(u32.astype(">u4").view(np.uint8).reshape(tiles, -1), axis=1)  # [tiles, 16w]
    ring = 16 * w
    start = (trellis_window_ends(w) - 16) % ring
    index = (start[:, None] + np.arange(16)[None, :]) % ring  # [256, 16]
    weights16 = (1 << np.arange(15, -1, -1)).astype(np.uint32)
    state = (bits[:, index].astype(np.uint32) * weights16).sum(axis=2).astype(np.uint64)  # [tiles, 256]
    product = (state * np.uint64(0x83DCD12D)) & np.uint64(0xFFFFFFFF)
    total = np.uint64(0x6400) + (product & np.uint64(255)) + ((product >> np.uint64(8)) & np.uint64(255)) \
        + ((product >> np.uint64(16)) & np.uint64(255)) + (product >> np.uint64(24))
    a = total.astype(np.uint16).view(np.float16).astype(np.float64)
    b = np.float64(np.array(0x1EEE, dtype=np.uint16).view(np.float16))
    c = np.float64(np.array(0xC931, dtype=np.uint16).view(np.float16))
    return (a * b + c).astype(np.float16)


def trellis_position_rc(pos):
    """(row = k within the tile, col = n within the tile) of tensor-core position `pos`
    (native/src/trellis/codebook.cuh:65-71)."""
    pos = np.asarray(pos)
    t, j = pos >> 3, pos & 7
    row = (t & 3) * 2 + ((j >> 1) & 1) * 8 + (j & 1)
    col = (t >> 2) + (j >> 2) * 8
    return row, col


def trellis_rotated_weight(payload: np.ndarray) -> np.ndarray:
    """Q [K, N] float16 of a payload [K/16, N/16, w] (native/tests/trellis_reference.py:43-52)."""
    kt, nt, w = payload.shape
    row, col = trellis_position_rc(np.arange(256))
    values = trellis_decode_tiles(payload.reshape(kt * nt, w), w).reshape(kt, nt, 256)
    q = np.zeros((kt, 16, nt, 16), dtype=np.float16)
    q[:, row, :, col] = np.transpose(values, (2, 0, 1))
    return q.reshape(kt * 16, nt * 16)


def hadamard128(x, dtype=np.float32) -> np.ndarray:
    """Sylvester butterfly over blocks of 128 of the last axis, stages h = 1..64, then * 1/sqrt(128); in `dtype`
    (float32 = the engine's arithmetic: native/src/trellis/codebook.cuh:76-113)."""
    x = np.array(x, dtype=dtype)
    shape = x.shape
    x = x.reshape(-1, 128)
    h = 1
    while h < 128:
        y = x.reshape(-1, 128 // (2 * h), 2, h)
        a, b = y[:, :, 0, :].copy(), y[:, :, 1, :].copy()
        y[:, :, 0, :] = a + b
        y[:, :, 1, :] = a - b
        x = y.reshape(-1, 128)
        h *= 2
    if dtype == np.float32:
        x = x * INV_SQRT_128
    else:
        x = x / np.sqrt(dtype(128.0))
    return x.reshape(shape)


def trellis_prepass(x_bits: np.ndarray, suh: np.ndarray) -> np.ndarray:
    """FP16 rotated activations [s, rows, K] in column order: fp16_rn(H128_f32(f32(bf16 x) * f32(fp16 suh)))
    (native/src/trellis/prepass.cuh:27-33,70-79)."""
    x = bf16_to_f32(x_bits)
    suh = np.asarray(suh, dtype=np.float16).reshape(-1, x.shape[1]).astype(np.float32)
    return hadamard128((x[None, :, :] * suh[:, None, :]).astype(np.float32)).astype(np.float16)


def trellis_segment_of_block(ends, n: int) -> np.ndarray:
    """Segment index of every 128-column block: first g with c0 < ends[g] (native/src/trellis/mma.cuh:440-443)."""
    c0 = np.arange(0, n, 128)
    return np.searchsorted(np.asarray(ends), c0, side="right")


def trellis_linear_f64(x_bits, payload, suh, svh, ends) -> np.ndarray:
    """y = svh * H_n(H_k(x * suh[seg]) . Q) in float64 (native/tests/trellis_reference.py:88-106)."""
    x = bf16_to_f32(x_bits).astype(np.float64)
    kt, nt, w = payload.shape
    k, n = kt * 16, nt * 16
    suh = np.asarray(suh, dtype=np.float64).reshape(len(ends), k)
    q = trellis_rotated_weight(payload).astype(np.float64)
    z = np.zeros((x.shape[0], n))
    start = 0
    for g, end in enumerate(ends):
        u = hadamard128(x * suh[g], np.float64)
        z[:, start:end] = u @ q[:, start:end]
        start = end
    return np.asarray(svh, dtype=np.float64) * hadamard128(z, np.float64)


def trellis_linear_kernel_model(x_bits, payload, suh, svh, ends) -> np.ndarray:
    """float32 model of the production route: FP16 prepass, FP16 x FP16 products summed in float64 (stands in for the
    tensor core's FP32 accumulation), float32 output Hadamard, * f32(svh). Not bit-exact with any kernel; used with
    the reference's tolerance (native/tests/test_trellis.py:157-165)."""
    kt, nt, w = payload.shape
    n = nt * 16
    act = trellis_prepass(x_bits, suh).astype(np.float64)  # [s, rows, k]
    q = trellis_rotated_weight(payload).astype(np.float64)
    seg = np.repeat(trellis_segment_of_block(ends, n), 128)
    z = np.zeros((act.shape[1], n), dtype=np.float32)
    for g in range(len(ends)):
        cols = seg == g
        z[:, cols] = (act[g] @ q[:, cols]).astype(np.float32)
    return hadamard128(z) * np.asarray(svh, dtype=np.float16).astype(np.float32)


def trellis_prefill_model(x_bits, payload, suh, svh, ends) -> np.ndarray:
    """Model of the reference's trellis prefill plan (core/.../artifact/format/TrellisFormat.java:560-625): BF16 column-order
    prepass, the payload decoded to BF16 (native/src/trellis/decode.cuh), a BF16 linear per segment rounded to BF16 (the
    sum over K in float64 stands in for the tensor core's FP32 accumulation), then bf16(f32(svh) * H128_f32(.))
    (native/src/trellis/epilogue.cuh:46-61). float32 [rows, n] of the BF16 results."""
    x = bf16_to_f32(x_bits)
    kt, nt, w = payload.shape
    k, n = kt * 16, nt * 16
    scales = np.asarray(suh, dtype=np.float16).reshape(len(ends), k).astype(np.float32)
    act = round_bf16(hadamard128((x[None, :, :] * scales[:, None, :]).astype(np.float32))).astype(np.float64)   # [s, rows, k]
    q = round_bf16(trellis_rotated_weight(payload).astype(np.float32)).astype(np.float64)                        # [k, n]
    seg = np.repeat(trellis_segment_of_block(ends, n), 128)
    z = np.zeros((x.shape[0], n), dtype=np.float32)
    for g in range(len(ends)):
        cols = seg == g
        z[:, cols] = round_bf16((act[g] @ q[:, cols]).astype(np.float32))
    return round_bf16(hadamard128(z) * np.asarray(svh, dtype=np.float16).astype(np.float32))


def trellis_fragment_order(values) -> np.ndarray:
    """The reference prepass's FP16 layout: in each group of 16, elements 2q, 2q+1, 2q+8, 2q+9 contiguous at 4q
    (native/src/trellis/prepass.cuh:70-79; native/tests/trellis_reference.py:115-122)."""
    e = np.arange(16)
    position = 4 * ((e & 7) >> 1) + 2 * (e >> 3) + (e & 1)
    groups = np.asarray(values).reshape(*np.shape(values)[:-1], -1, 16)
    out = np.empty_like(groups)
    out[..., position] = groups
    return out.reshape(np.shape(values))


def trellis_splits(k: int, n: int, target_ctas: int) -> int:
    """core/.../artifact/format/TrellisFormat.java:299-303."""
    blocks = n // 128
    return max(1, min(-(-target_ctas // blocks), k // 256))


def trellis_payload_bytes(k: int, n: int, w: int) -> int:
    return (k // 16) * (n // 16) * w * 2


# --------------------------------------------------------------------------------------------------------------
# Prefill: two-term NVFP4 activation quantizer (parity UNPINNED at bit level, see module docstring)
# --------------------------------------------------------------------------------------------------------------

def e4m3_encode_satfinite(values) -> np.ndarray:
    """cvt.rn.satfinite.e4m3 of non-negative float32: nearest even, saturating to 448 (code 0x7E)."""
    return e4m3_encode(np.minimum(np.asarray(values, dtype=np.float32), np.float32(448.0)))


def activation_layout(rows: int, k: int, terms: int = 2):
    """(scale offset, global offset, bytes, pad) of the native activation buffer
    (native/src/nvfp4_native/native.cuh:66-82; native/src/host/nvfp4_linear.c:252-257)."""
    kp = align_up(k, 128)
    pad = align_up(rows, 128)
    scale_off = align_up(rows * terms * kp // 2, 256)
    global_off = align_up(scale_off + kp // 128 * terms * pad * 8, 256)
    return scale_off, global_off, global_off + 4 * rows, pad


def quantize_activations(x_bits: np.ndarray, terms: int = 2):
    """BF16 rows -> (codes u8 [terms, rows, K] one E2M1 code per entry, scales u8 [terms, rows, K/16], globals f32
    [rows]). native/src/nvfp4_native/native.cuh:105-168: global = amax / 2688 (1 when the row is zero); per block of
    16: scale = e4m3_satfinite(amax * (1/6) * (1/global)); code = e2m1_rn_sat(v * ((1/global) / decoded)); the next
    term quantizes fma(-q, decoded * global, v). All in float32."""
    x = bf16_to_f32(x_bits)
    rows, k = x.shape
    amax = np.abs(x).max(axis=1)
    g = np.where(amax > 0, (amax / np.float32(2688.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    inv_g = (np.float32(1.0) / g).astype(np.float32)
    v = x.reshape(rows, k // 16, 16).copy()
    codes = np.zeros((terms, rows, k), dtype=np.uint8)
    scales = np.zeros((terms, rows, k // 16), dtype=np.uint8)
    sixth = np.float32(1.0) / np.float32(6.0)
    for t in range(terms):
        bmax = np.abs(v).max(axis=2)
        want = ((bmax * sixth).astype(np.float32) * inv_g[:, None]).astype(np.float32)
        sc = e4m3_encode_satfinite(want)
        decoded = e4m3_value(sc)
        with np.errstate(divide="ignore", invalid="ignore"):
            inverse = np.where(decoded > 0, (inv_g[:, None] / decoded).astype(np.float32), np.float32(0))
        step = (decoded * g[:, None]).astype(np.float32)
        scaled = (v * inverse[..., None]).astype(np.float32)
        mag = e2m1_encode_magnitude(np.abs(scaled))
        sign = (np.signbit(scaled)).astype(np.uint8) << 3  # the hardware conversion keeps the sign of zero
        q = E2M1_MAGNITUDES[mag] * np.where(sign > 0, np.float32(-1), np.float32(1))
        # v - q * step in one rounding (the reference's build contracts the statement into a fused multiply-add); in
        # float64 the product (3 x 24 bits) and the sum of two values a few binades apart are exact, so rounding the
        # float64 result to float32 is that single rounding
        v = (v.astype(np.float64) - q.astype(np.float64) * step[..., None].astype(np.float64)).astype(np.float32)
        codes[t] = (mag | sign).reshape(rows, k)
        scales[t] = sc
    return codes, scales, g


def activations_dense(codes, scales, g) -> np.ndarray:
    """float64 [rows, K]: sum over terms of e2m1 * e4m3 * global (the operand the prefill GEMM really multiplies)."""
    value = E2M1_MAGNITUDES[codes & 7].astype(np.float64) * np.where(codes & 8, -1.0, 1.0)
    value = value * np.repeat(e4m3_value(scales).astype(np.float64), 16, axis=2)
    return value.sum(axis=0) * np.asarray(g, dtype=np.float64)[:, None]


def trellis_pack_states(states: np.ndarray, ka: int, mask: int = 0) -> np.ndarray:
    """uint16 [count, 256] states -> int16 [count, w] payload words: the low d(i) bits of state i, most significant bit
    first, into 32-bit little-endian words (pack.cu / frac.cu as restated in quantization/src/main/resources/cuda/
    trellis.cu:401-462); w = 16 ka + popcount(mask)."""
    states = np.asarray(states, dtype=np.uint16)
    count = states.shape[0]
    bits_per = np.array([ka + ((mask >> (i & 15)) & 1) for i in range(256)])
    total = int(bits_per.sum())
    stream = np.zeros((count, total), dtype=np.uint8)
    at = 0
    for i in range(256):
        d = int(bits_per[i])
        for b in range(d - 1, -1, -1):
            stream[:, at] = (states[:, i] >> b) & 1
            at += 1
    words = np.packbits(stream.reshape(count, total // 32, 32), axis=2, bitorder="big").reshape(count, total // 32, 4)
    big = (words[..., 0].astype(np.uint32) << 24) | (words[..., 1].astype(np.uint32) << 16) | (words[..., 2].astype(np.uint32) << 8) | words[..., 3]
    return big.astype("<u4").view("<i2").reshape(count, total // 16)
