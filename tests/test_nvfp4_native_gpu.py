"""NVFP4 prefill route (activation quantizer + tcgen05 block-scaled GEMM) through the C ABI, modelled on the
reference's native/tests/test_nvfp4_native.py: the output is checked against float64 over the operands the kernel
really multiplied (the quantized activations read back from the scratch), the quantizer against the CPU restatement."""

import numpy as np
import pytest

from euhedral_b200 import layouts, library
from oracle import oracle_c as OC
from oracle import oracle_np as O
from tests.gpu_util import Device, random_x

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    device = Device()
    yield device
    assert device.gpu.take_device_error() == 0
    device.release()


def run(dev, x_bits, blob, n, k):
    rows = x_bits.shape[0]
    lib = dev.gpu.lib
    need = lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, k, n)
    d_x, d_w, d_y, d_s = dev.put(x_bits), dev.put(blob), dev.empty(rows * n * 2), dev.empty(need + 256, fill=0)
    scratch = (d_s.data_ptr() + 255) & ~255
    with dev.submit(pdl=True):
        status = lib.euhedral_cuda_linear_nvfp4_native_bf16(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), scratch, rows, k, n,
                                                            blob.size, need)
    assert status == 0, status
    y = dev.get(d_y, np.uint16, (rows, n))
    raw = dev.get(d_s, np.uint8, (need + 256,))[scratch - d_s.data_ptr():]
    return y, raw


def unpack_scratch(raw, rows, k):
    """(codes [2, rows, k], scales [2, rows, k/16], globals [rows]) from the kernel's scratch layout."""
    half = k // 2
    planes = raw[:2 * rows * half].reshape(2, rows, half)
    codes = np.empty((2, rows, k), dtype=np.uint8)
    codes[:, :, 0::2] = planes & 15
    codes[:, :, 1::2] = planes >> 4
    sfa_offset = layouts.align_up(2 * rows * half, 256)
    row_tiles, k_blocks = -(-rows // 128), k // 64
    atoms = raw[sfa_offset:sfa_offset + row_tiles * k_blocks * 2 * 512].reshape(row_tiles, k_blocks, 2, 512)
    scales = np.zeros((2, rows, k // 16), dtype=np.uint8)
    for row in range(rows):
        in_tile = row % 128
        for t in range(2):
            for s4 in range(4):
                scales[t, row, s4::4] = atoms[row // 128, :, t, (in_tile % 32) * 16 + (in_tile // 32) * 4 + s4]
    global_offset = layouts.align_up(sfa_offset + row_tiles * k_blocks * 2 * 512, 256)
    g = raw[global_offset:global_offset + 4 * rows].view(np.float32)
    return codes, scales, g


# The last three are skinny calls (9 to 64 rows: the K steps of an output tile are cut over 8, 7 and 2 CTAs and the ranges'
# FP32 sums added in order by a second launch).
@pytest.mark.parametrize("rows,k,n", [(16, 256, 128), (128, 512, 256), (200, 1024, 384), (300, 5120, 1024), (9, 5120, 1024), (33, 17408, 5120),
                                      (64, 5120, 17408)])
def test_native_matches_float64_over_quantized_operands(dev, rows, k, n):
    rng = np.random.default_rng(rows + k + n)
    weights = (rng.standard_normal((n, k)) * rng.uniform(0.01, 1.0, (n, 1))).astype(np.float32)
    blob = OC.nvfp4_quantize(weights)
    dense = OC.nvfp4_dense(blob, n, k).astype(np.float64)
    x = random_x(rng, rows, k)
    y, raw = run(dev, x, blob, n, k)
    codes, scales, g = unpack_scratch(raw, rows, k)
    # the quantizer against its CPU restatement (bit level) and against the activations (reconstruction error)
    ref_codes, ref_scales, ref_g = O.quantize_activations(x, 2)
    assert np.array_equal(g, ref_g)
    assert np.array_equal(scales, ref_scales)
    assert np.array_equal(codes & 7, ref_codes & 7) and np.array_equal(codes[(codes & 7) > 0], ref_codes[(codes & 7) > 0])
    quantized = O.activations_dense(codes, scales, g)
    xf = O.bf16_to_f32(x).astype(np.float64)
    assert np.linalg.norm(quantized - xf) / np.linalg.norm(xf) < 0.012
    expect = quantized @ dense.T
    got = O.bf16_to_f32(y).astype(np.float64)
    assert np.max(np.abs(got - expect)) <= 2.0 ** -7 * np.max(np.abs(expect))
    # and against the BF16-activation result: the two-term approximation costs about 1% (reported, loosely bounded)
    exact = xf @ dense.T
    assert np.linalg.norm(got - exact) / np.linalg.norm(exact) < 0.03


def unpack_rows(raw, rows, k, sample):
    """unpack_scratch for the rows in `sample` only: (codes [2, len, k], scales [2, len, k/16], globals [len])."""
    half = k // 2
    planes = raw[:2 * rows * half].reshape(2, rows, half)[:, sample]
    codes = np.empty((2, len(sample), k), dtype=np.uint8)
    codes[:, :, 0::2] = planes & 15
    codes[:, :, 1::2] = planes >> 4
    sfa_offset = layouts.align_up(2 * rows * half, 256)
    row_tiles, k_blocks = -(-rows // 128), k // 64
    atoms = raw[sfa_offset:sfa_offset + row_tiles * k_blocks * 2 * 512].reshape(row_tiles, k_blocks, 2, 512)
    scales = np.zeros((2, len(sample), k // 16), dtype=np.uint8)
    for i, row in enumerate(sample):
        in_tile = row % 128
        for t in range(2):
            for s4 in range(4):
                scales[t, i, s4::4] = atoms[row // 128, :, t, (in_tile % 32) * 16 + (in_tile // 32) * 4 + s4]
    global_offset = layouts.align_up(sfa_offset + row_tiles * k_blocks * 2 * 512, 256)
    g = raw[global_offset:global_offset + 4 * rows].view(np.float32)[sample]
    return codes, scales, g


# Shapes where every persistent CTA walks many output tiles (the accumulator hand-over between tiles, the stage ring
# running on across tiles, several panels of the tile walk): the layer's gate and down shapes at 4096 tokens, its q shape
# at 32768 tokens, a token count that is not a multiple of 128, more tiles than SMs with a narrow last panel, and an
# output width that is an odd multiple of 128.
@pytest.mark.parametrize("rows,k,n", [(1024, 512, 4352), (256, 512, 1408), (4096, 5120, 17408), (4096, 17408, 5120), (4100, 5120, 5120),
                                      (32768, 5120, 5120)])
def test_native_at_model_shapes(dev, rows, k, n):
    rng = np.random.default_rng(rows + k + n)
    weights = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    blob = OC.nvfp4_quantize(weights)
    del weights
    x = O.bf16_bits(rng.standard_normal((rows, k), dtype=np.float32))
    y, raw = run(dev, x, blob, n, k)
    # 64 token rows spread over the whole range (first and last included), every output column
    sample = np.unique(np.concatenate([[0, rows - 1, rows // 2], rng.integers(0, rows, 61)]))
    codes, scales, g = unpack_rows(raw, rows, k, sample)
    ref_codes, ref_scales, ref_g = O.quantize_activations(x[sample], 2)
    assert np.array_equal(g, ref_g) and np.array_equal(scales, ref_scales)
    assert np.array_equal(codes & 7, ref_codes & 7) and np.array_equal(codes[(codes & 7) > 0], ref_codes[(codes & 7) > 0])
    quantized = O.activations_dense(codes, scales, g)
    got = O.bf16_to_f32(y[sample]).astype(np.float64)
    expect = np.empty((len(sample), n), dtype=np.float64)
    dense = OC.nvfp4_dense(blob, n, k)
    for first in range(0, n, 2048):
        expect[:, first:first + 2048] = quantized @ dense[first:first + 2048].astype(np.float64).T
    del dense
    top = np.max(np.abs(expect))
    assert np.max(np.abs(got - expect)) <= (2e-3 + 2.0 ** -8) * top
    assert np.all(np.abs(got - expect) <= np.abs(expect) * 2.0 ** -7 + top * 1e-3)
    # untouched rows around the sample were written too: no row of the output kept the fill pattern
    assert not np.any(np.all(y == 0xA5A5, axis=1))


def test_quantize_once_for_linears_that_share_their_input(dev):
    """quantize + prequantized linears give bit for bit what the whole native call gives."""
    rng = np.random.default_rng(91)
    rows, k = 200, 1024
    x = random_x(rng, rows, k)
    shapes = (384, 128)
    blobs = [OC.nvfp4_quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32)) for n in shapes]
    whole = [run(dev, x, blob, n, k)[0] for blob, n in zip(blobs, shapes)]
    lib = dev.gpu.lib
    need = lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, k, max(shapes))
    d_x, d_s = dev.put(x), dev.empty(need, fill=0)
    d_w = [dev.put(blob) for blob in blobs]
    d_y = [dev.empty(rows * n * 2) for n in shapes]
    with dev.submit(pdl=True):
        assert lib.euhedral_b200_nvfp4_native_quantize(d_x.data_ptr(), d_s.data_ptr(), rows, k, need) == 0
        for w, y, blob, n in zip(d_w, d_y, blobs, shapes):
            assert lib.euhedral_b200_linear_nvfp4_native_prequantized_bf16(w.data_ptr(), y.data_ptr(), d_s.data_ptr(), rows, k, n, blob.size, need) == 0
    for y, n, expect in zip(d_y, shapes, whole):
        assert np.array_equal(dev.get(y, np.uint16, (rows, n)), expect)
    assert lib.euhedral_b200_nvfp4_native_quantize(d_x.data_ptr(), d_s.data_ptr(), rows, 384, need) == library.ROUTE_UNAVAILABLE
    assert lib.euhedral_b200_nvfp4_native_quantize(d_x.data_ptr(), d_s.data_ptr(), rows, k, 16) == library.INVALID_ARGUMENT


def test_native_route_declines(dev):
    lib = dev.gpu.lib
    rows, k, n = 16, 384, 128      # k % 256 != 0
    blob = OC.nvfp4_quantize(np.ones((n, k), dtype=np.float32))
    d = dev.empty(1 << 20)
    assert lib.euhedral_cuda_linear_nvfp4_native_bf16(d.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(), rows, k, n, blob.size, 1 << 20) == library.ROUTE_UNAVAILABLE
    dev.gpu.select_exact_numerics(True)
    try:
        assert lib.euhedral_cuda_linear_nvfp4_native_bf16(d.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(), 16, 256, 128, 1, 1) == library.ROUTE_UNAVAILABLE
    finally:
        dev.gpu.select_exact_numerics(False)
    assert lib.euhedral_cuda_nvfp4_native_available() == 1


# The paired gate/up region (the reference's euhedral_cuda_nvfp4_native_gate_up_swiglu_bf16, native/src/nvfp4_native/
# native.cuh:390-413): gate and up are the BF16 values the plain native linear gives for the same fused tensor, bit for
# bit (same accumulators, same scaling and rounding); the SwiGLU on top is FP32 with expf and a division, so the BF16
# result is compared with a float32 NumPy evaluation: equal almost everywhere, one unit in the last place at most.
@pytest.mark.parametrize("rows,k,outputs", [(200, 1024, 768), (9, 1024, 512), (300, 5120, 34816), (700, 5120, 34816), (1000, 1024, 768)])
def test_gate_up_swiglu_region(dev, rows, k, outputs):
    rng = np.random.default_rng(rows + outputs)
    blob = OC.nvfp4_quantize((rng.standard_normal((outputs, k)) * 0.05).astype(np.float32))
    x = random_x(rng, rows, k)
    full, _ = run(dev, x, blob, outputs, k)
    half = outputs // 2
    lib = dev.gpu.lib
    need = lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, k, outputs)
    d_x, d_w, d_y, d_s = dev.put(x), dev.put(blob), dev.empty(rows * half * 2), dev.empty(need)
    with dev.submit(pdl=True):
        assert lib.euhedral_cuda_nvfp4_native_gate_up_swiglu_bf16(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), d_s.data_ptr(), rows, k,
                                                                  outputs, blob.size, need) == 0
        assert lib.euhedral_cuda_nvfp4_native_gate_up_swiglu_bf16(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), d_s.data_ptr(), rows, k,
                                                                  outputs - 1, blob.size, need) == library.INVALID_ARGUMENT
    got = dev.get(d_y, np.uint16, (rows, half))
    gate, up = O.bf16_to_f32(full[:, :half]), O.bf16_to_f32(full[:, half:])
    one = np.float32(1.0)
    value = (gate / (one + np.exp(-gate, dtype=np.float32))).astype(np.float32) * up
    expect = O.bf16_bits(value.astype(np.float32))
    distance = np.abs(got.astype(np.int32) - expect.astype(np.int32))
    assert distance.max() <= 1, int(distance.max())
    assert np.mean(distance == 0) >= 0.995, float(np.mean(distance == 0))
    assert got.any()


def test_gate_up_swiglu_needs_whole_tiles(dev):
    rng = np.random.default_rng(5)
    k, outputs, rows = 1024, 384, 16          # 192 outputs: not a multiple of the 128-column tile
    blob = OC.nvfp4_quantize((rng.standard_normal((outputs, k)) * 0.05).astype(np.float32))
    lib = dev.gpu.lib
    need = lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, k, outputs)
    d_x, d_w, d_y, d_s = dev.put(random_x(rng, rows, k)), dev.put(blob), dev.empty(rows * outputs), dev.empty(need)
    with dev.submit():
        assert lib.euhedral_cuda_nvfp4_native_gate_up_swiglu_bf16(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), d_s.data_ptr(), rows, k,
                                                                  outputs, blob.size, need) == library.ROUTE_UNAVAILABLE


def test_cta_pairs_give_the_single_cta_bits(dev):
    """With euhedral_b200_select_native_pairs(1), calls of 512 rows and more run on CTA pairs (tcgen05 cta_group::2): the
    plain linear at shapes with many tiles per pair, a last pair whose odd CTA has no rows, K = 17408, and the gate/up
    SwiGLU region give bit for bit what the single-CTA kernel gives."""
    rng = np.random.default_rng(17)
    lib = dev.gpu.lib
    for rows, k, n in ((1100, 1024, 1280), (4096, 5120, 17408), (600, 17408, 5120)):
        blob = OC.nvfp4_quantize((rng.standard_normal((n, k)) * 0.03).astype(np.float32))
        x = random_x(rng, rows, k)
        single, _ = run(dev, x, blob, n, k)
        lib.euhedral_b200_select_native_pairs(1)
        try:
            pairs, _ = run(dev, x, blob, n, k)
        finally:
            lib.euhedral_b200_select_native_pairs(0)
        assert np.array_equal(pairs, single), (rows, k, n)
    rows, k, outputs = 700, 1024, 1536
    blob = OC.nvfp4_quantize((rng.standard_normal((outputs, k)) * 0.05).astype(np.float32))
    need = lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, k, outputs)
    d_x, d_w, d_s = dev.put(random_x(rng, rows, k)), dev.put(blob), dev.empty(need)
    results = []
    for enabled in (0, 1):
        d_y = dev.empty(rows * outputs)
        lib.euhedral_b200_select_native_pairs(enabled)
        try:
            with dev.submit(pdl=True):
                assert lib.euhedral_cuda_nvfp4_native_gate_up_swiglu_bf16(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), d_s.data_ptr(), rows, k,
                                                                          outputs, blob.size, need) == 0
        finally:
            lib.euhedral_b200_select_native_pairs(0)
        results.append(dev.get(d_y, np.uint16, (rows, outputs // 2)))
    assert np.array_equal(results[0], results[1]) and results[0].any()
