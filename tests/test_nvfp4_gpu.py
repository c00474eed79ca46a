"""NVFP4 decode GEMV through the C ABI against the oracle (modelled on the reference's native/tests/test_nvfp4.py)."""

import numpy as np
import pytest

from euhedral_b200 import library
from oracle import oracle_c as OC
from oracle import oracle_np as O
from tests.gpu_util import Device, elementwise_bound, max_relative_error, random_x

pytestmark = pytest.mark.gpu

SHAPES = [(640, 32), (1024, 64), (5120, 96), (17408, 32), (5120, 1024), (128, 16), (2560, 192)]  # (K, N)


@pytest.fixture(scope="module")
def dev():
    device = Device()
    yield device
    assert device.gpu.take_device_error() == 0
    device.release()


def tensor(rng, n, k, spread=True):
    scale = rng.uniform(0.01, 1.0, (n, 1)) if spread else 0.02
    weights = (rng.standard_normal((n, k)) * scale).astype(np.float32)
    blob = OC.nvfp4_quantize(weights)
    return blob, OC.nvfp4_dense(blob, n, k)


def run(dev, x_bits, blob, n, k, **select):
    rows = x_bits.shape[0]
    d_x, d_w, d_y = dev.put(x_bits), dev.put(blob), dev.empty(rows * n * 2)
    with dev.submit(**select) as gpu:
        gpu.linear_nvfp4_bf16(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), rows, k, n, blob.size)
    return dev.get(d_y, np.uint16, (rows, n))


@pytest.mark.parametrize("k,n", SHAPES)
def test_decode_matches_float64(dev, k, n):
    rng = np.random.default_rng(k * 31 + n)
    blob, dense = tensor(rng, n, k)
    for rows in (1, 2, 3, 4, 5, 8):
        x = random_x(rng, rows, k)
        got = O.bf16_to_f32(run(dev, x, blob, n, k, row_exact=True)).astype(np.float64)
        expect = O.linear_f64(x, dense)
        assert np.all(np.abs(got - expect) <= elementwise_bound(expect)), (rows, k, n)
        assert max_relative_error(got, expect) <= 2e-3 + 2.0 ** -8   # 2e-3 plus the BF16 rounding of the output


@pytest.mark.parametrize("k,n", SHAPES)
def test_rows_are_bitwise_the_one_row_call(dev, k, n):
    rng = np.random.default_rng(k + n)
    blob, _ = tensor(rng, n, k)
    x = random_x(rng, 8, k)
    single = np.concatenate([run(dev, x[r:r + 1], blob, n, k, row_exact=True) for r in range(8)])
    for rows in (2, 4, 5, 8):
        assert np.array_equal(run(dev, x[:rows], blob, n, k, row_exact=True), single[:rows])
    many = random_x(rng, 27, k)
    grouped = run(dev, many, blob, n, k, row_exact=True)
    for r in (0, 8, 9, 26):
        assert np.array_equal(grouped[r], run(dev, many[r:r + 1], blob, n, k, row_exact=True)[0])


def test_deterministic_and_with_dependent_launch(dev):
    rng = np.random.default_rng(5)
    k, n = 5120, 512
    blob, _ = tensor(rng, n, k)
    x = random_x(rng, 4, k)
    first = run(dev, x, blob, n, k)
    for _ in range(3):
        assert np.array_equal(run(dev, x, blob, n, k), first)
    assert np.array_equal(run(dev, x, blob, n, k, pdl=True), first)


def test_exact_numerics_is_the_scalar_kernel(dev):
    rng = np.random.default_rng(6)
    k, n = 640, 48
    blob, dense = tensor(rng, n, k)
    x = random_x(rng, 3, k)
    dev.gpu.select_exact_numerics(True)
    try:
        got = run(dev, x, blob, n, k)
    finally:
        dev.gpu.select_exact_numerics(False)
    assert np.array_equal(got, O.nvfp4_linear_scalar_kernel(x, blob.tobytes(), n, k))
    # a shape no decode kernel takes (K % 128 != 0) runs the same scalar kernel
    k2, n2 = 96, 24
    blob2, _ = tensor(rng, n2, k2)
    x2 = random_x(rng, 2, k2)
    assert np.array_equal(run(dev, x2, blob2, n2, k2), O.nvfp4_linear_scalar_kernel(x2, blob2.tobytes(), n2, k2))


def crafted(n, k, code_byte, scale_byte, global_scale):
    scale_off, global_off, size = O.nvfp4_offsets(n, k)
    blob = np.zeros(size, dtype=np.uint8)
    blob[:n * k // 2] = code_byte
    blob[scale_off:scale_off + n * k // 16] = scale_byte
    blob[global_off:global_off + 4] = np.frombuffer(np.float32(global_scale).tobytes(), dtype=np.uint8)
    return blob


def test_edge_tensors(dev):
    """The smallest code (0.5), subnormal and largest E4M3 scales, negative zero codes: exact small sums."""
    k, n = 256, 16
    ones = O.bf16_bits(np.ones((1, k), dtype=np.float32))
    # every weight 0.5 * 1.0: the code whose BF16 image is subnormal before scaling
    assert np.array_equal(O.bf16_to_f32(run(dev, ones, crafted(n, k, 0x11, 0x38, 1.0), n, k)), np.full((1, n), 128.0, np.float32))
    # every weight -1.0 * 2^-9 (smallest subnormal scale), tensor scale 4
    assert np.array_equal(O.bf16_to_f32(run(dev, ones, crafted(n, k, 0xAA, 0x01, 4.0), n, k)), np.full((1, n), -2.0, np.float32))
    # every weight 6 * 448 (largest code and scale)
    assert np.array_equal(O.bf16_to_f32(run(dev, ones, crafted(n, k, 0x77, 0x7E, 2.0 ** -10), n, k)), np.full((1, n), 672.0, np.float32))
    # negative zero codes and zero scales contribute nothing
    assert not O.bf16_to_f32(run(dev, ones, crafted(n, k, 0x88, 0x38, 1.0), n, k)).any()
    assert not O.bf16_to_f32(run(dev, ones, crafted(n, k, 0x77, 0x00, 1.0), n, k)).any()
    # a quantized tensor with zero blocks, tiny blocks and an outlier, against float64
    weights = np.zeros((n, k), dtype=np.float32)
    weights[1, 5] = 3.0
    weights[2, :] = 1e-6
    weights[3, :] = np.linspace(-1, 1, k, dtype=np.float32) * 1e-4
    weights[4, 16:32] = 6.0
    weights[6, :] = np.random.default_rng(1).standard_normal(k).astype(np.float32) * 1e-3
    blob = OC.nvfp4_quantize(weights)
    codes, scales, g = O.nvfp4_unpack(blob.tobytes(), n, k)
    assert (scales < 8).any() and (scales > 100).any()   # subnormal and large scale codes are both present
    x = random_x(np.random.default_rng(9), 2, k)
    got = O.bf16_to_f32(run(dev, x, blob, n, k)).astype(np.float64)
    expect = O.linear_f64(x, O.nvfp4_dense(blob.tobytes(), n, k))
    assert np.all(np.abs(got - expect) <= np.abs(expect) * 2.0 ** -8 + 1e-12)


def test_status_codes(dev):
    lib = library.load()
    k, n = 256, 16
    blob, _ = tensor(np.random.default_rng(2), n, k)
    d_x, d_w, d_y = dev.put(random_x(np.random.default_rng(3), 1, k)), dev.put(blob), dev.empty(n * 2)
    call = lib.euhedral_cuda_linear_nvfp4_bf16
    assert call(None, d_w.data_ptr(), d_y.data_ptr(), 1, k, n, blob.size) == library.INVALID_ARGUMENT
    assert call(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), 0, k, n, blob.size) == library.INVALID_ARGUMENT
    assert call(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), 1, k, n, blob.size - 4) == library.FORMAT_MISMATCH
    assert call(d_x.data_ptr() + 2, d_w.data_ptr(), d_y.data_ptr(), 1, k, n, blob.size) == library.INVALID_ARGUMENT
    assert call(d_x.data_ptr(), d_w.data_ptr(), d_y.data_ptr(), 1, k, n, blob.size) == library.SUCCESS  # no stream: synchronous


def test_row_shards_equal_the_whole(dev):
    """N-sharded copies of a tensor give bitwise the unsharded result (the K order depends on K only)."""
    from euhedral_b200 import sharding
    rng = np.random.default_rng(8)
    k, n = 5120, 1024
    blob, _ = tensor(rng, n, k)
    x = random_x(rng, 5, k)
    whole = run(dev, x, blob, n, k)
    for shards in (2, 8):
        parts = [run(dev, x, sharding.nvfp4_rows(blob, n, k, s * n // shards, n // shards), n // shards, k) for s in range(shards)]
        assert np.array_equal(np.concatenate(parts, axis=1), whole)


# The last two are the fused objects the reference's converter emits and its host calls as one tensor: query_key_value
# (5120 + 1024 + 1024 rows) and gate_up (2 x 17408 rows), tools/euhedral_artifacts/trellis.py:128-146.
@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408), (1024, 5120), (5120, 5120), (7168, 5120), (34816, 5120)])
def test_model_shapes(dev, n, k):
    rng = np.random.default_rng(0xE0)
    weights = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    blob = OC.nvfp4_quantize(weights)
    for rows in (1, 3, 4, 5):
        x = random_x(np.random.default_rng(0xA0 + rows), rows, k)
        got = O.bf16_to_f32(run(dev, x, blob, n, k)).astype(np.float64)
        expect = OC.nvfp4_linear(x, blob, n, k).astype(np.float64)   # FP32-accumulated reference
        assert max_relative_error(got, expect) <= 2e-3 + 2.0 ** -8


# Shapes that take every launch geometry of the decode kernel: tall tensors on the persistent grid (several tiles per warp
# in turn, a last cluster with a short share, an odd tile count), one K slice (no cluster) on the persistent grid, two K
# slices, an odd number of chunks per slice, few rows of tiles.
GRID_SHAPES = [(17424, 5120), (40000, 1024), (3088, 2048), (2000, 1536), (5120, 17408), (48, 4352), (9232, 8192)]  # (N, K)


@pytest.mark.parametrize("n,k", GRID_SHAPES)
def test_launch_geometries(dev, n, k):
    plan = library.decode_plan("nvfp4", 5, k, n)
    assert plan["ctas"] % plan["k_slices"] == 0
    rng = np.random.default_rng(n * 31 + k)
    weights = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    blob = OC.nvfp4_quantize(weights)
    for rows in (1, 2, 5, 8):
        x = random_x(np.random.default_rng(0xB0 + rows), rows, k)
        got_bits = run(dev, x, blob, n, k)
        got = O.bf16_to_f32(got_bits).astype(np.float64)
        expect = OC.nvfp4_linear(x, blob, n, k).astype(np.float64)
        assert max_relative_error(got, expect) <= 2e-3 + 2.0 ** -8, (rows, n, k)
        if rows == 5:   # every row of the call is the one-row call, bit for bit
            for r in (0, 4):
                assert np.array_equal(run(dev, x[r:r + 1], blob, n, k)[0], got_bits[r])

